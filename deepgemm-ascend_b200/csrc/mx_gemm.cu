// Instantiation and launch of the block-scaled GEMM kernel, plus the split-K finalisation kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "host_common.h"
#include "launch.h"
#include "mx_gemm.cuh"

namespace dg {

// Device status word: 0, or the code of the first bounded wait that gave up.
__device__ int32_t g_device_status;

// Split-K finalisation: D = cast(workspace (+ bias)) or D += workspace, and the workspace is zeroed
// again so that the next launch can reduce into it without a memset.
__global__ void splitk_finalize_kernel(float* __restrict__ ws, uint64_t ws_stride, void* __restrict__ d,
                                       uint64_t d_stride, uint32_t m, uint32_t n, uint32_t d_is_fp32,
                                       uint32_t accumulate, const void* __restrict__ bias) {
    const uint32_t n4 = (n + 3) / 4;
    const uint64_t total = (uint64_t)m * n4;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / n4), c = (uint32_t)(i % n4) * 4;
        float4* wp = reinterpret_cast<float4*>(ws + (uint64_t)r * ws_stride + c);
        const float4 v4 = *wp;
        *wp = make_float4(0.f, 0.f, 0.f, 0.f);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
        #pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            if (c + j >= n) break;
            float f = v[j];
            if (d_is_fp32) {
                float* dp = reinterpret_cast<float*>(d) + (uint64_t)r * d_stride + c + j;
                if (bias) f += reinterpret_cast<const float*>(bias)[c + j];
                *dp = accumulate ? *dp + f : f;
            } else {
                __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(d) + (uint64_t)r * d_stride + c + j;
                if (bias) f += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[c + j]);
                *dp = accumulate ? __float2bfloat16_rn(__bfloat162float(*dp) + f) : __float2bfloat16_rn(f);
            }
        }
    }
}

// K-grouped layout: a group whose K range is empty contributes no tile, so its D[g] is cleared here
// (the reference does this on its vector cores, deep_gemm/include/deep_gemm/epilogue.hpp:108-141).
__global__ void zero_empty_k_groups_kernel(uint8_t* __restrict__ d, const int32_t* __restrict__ psum, uint32_t num_groups,
                                           uint32_t rows, uint64_t row_bytes, uint64_t row_pitch, uint64_t group_pitch) {
    for (uint32_t g = 0; g < num_groups; ++g) {
        const uint32_t begin = g == 0 ? 0u : ((uint32_t)psum[g - 1] + 255u) / 256u * 256u;
        if ((uint32_t)psum[g] > begin) continue;
        const uint64_t total = (uint64_t)rows * row_bytes;
        for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x)
            d[g * group_pitch + (i / row_bytes) * row_pitch + i % row_bytes] = 0;
    }
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const CUtensorMap, const CUtensorMap, const GemmKernelArgs);

static KernelFn pick_kernel(int cta_group, int major_a, int major_b, bool decode_b, bool lean, bool fp4_pair, bool bf16_pair,
                            bool wide_epi, bool simple_epi, bool wide_tile) {
    if (wide_tile && fp4_pair) return mx_gemm_kernel<2, 0, 0, false, false, true, false, false, false, true>;
    if (wide_tile && bf16_pair) return mx_gemm_kernel<2, 0, 0, false, false, false, true, false, false, true>;
    if (wide_tile)          // E4M3 x E4M3, K-major operands, CTA pair, block_n > 256
        return simple_epi ? mx_gemm_kernel<2, 0, 0, false, false, false, false, false, true, true>
                          : mx_gemm_kernel<2, 0, 0, false, false, false, false, false, false, true>;
    if (simple_epi) {       // E4M3 x E4M3, K-major operands, plain BF16 output through TMA stores
        if (wide_epi)
            return cta_group == 2 ? mx_gemm_kernel<2, 0, 0, false, false, false, false, true, true>
                                  : mx_gemm_kernel<1, 0, 0, false, false, false, false, true, true>;
        return cta_group == 2 ? mx_gemm_kernel<2, 0, 0, false, false, false, false, false, true>
                              : mx_gemm_kernel<1, 0, 0, false, false, false, false, false, true>;
    }
    if (wide_epi)
        return cta_group == 2 ? mx_gemm_kernel<2, 0, 0, false, false, false, false, true>
                              : mx_gemm_kernel<1, 0, 0, false, false, false, false, true>;
    if (bf16_pair) {
        static const KernelFn bf16_table[2][2][2] = {
            {{mx_gemm_kernel<1, 0, 0, false, false, false, true>, mx_gemm_kernel<1, 0, 1, false, false, false, true>},
             {mx_gemm_kernel<1, 1, 0, false, false, false, true>, mx_gemm_kernel<1, 1, 1, false, false, false, true>}},
            {{mx_gemm_kernel<2, 0, 0, false, false, false, true>, mx_gemm_kernel<2, 0, 1, false, false, false, true>},
             {mx_gemm_kernel<2, 1, 0, false, false, false, true>, mx_gemm_kernel<2, 1, 1, false, false, false, true>}},
        };
        return bf16_table[cta_group - 1][major_a][major_b];
    }
    if (fp4_pair)
        return cta_group == 2 ? mx_gemm_kernel<2, 0, 0, false, false, true> : mx_gemm_kernel<1, 0, 0, false, false, true>;
    if (lean) {
        static const KernelFn lean_table[2][2] = {
            {mx_gemm_kernel<1, 0, 0, false, true>, mx_gemm_kernel<1, 0, 1, false, true>},
            {mx_gemm_kernel<1, 1, 0, false, true>, mx_gemm_kernel<1, 1, 1, false, true>},
        };
        return lean_table[major_a][major_b];
    }
    static const KernelFn table[2][2][2][2] = {
        {{{mx_gemm_kernel<1, 0, 0, false>, mx_gemm_kernel<1, 0, 0, true>}, {mx_gemm_kernel<1, 0, 1, false>, mx_gemm_kernel<1, 0, 1, true>}},
         {{mx_gemm_kernel<1, 1, 0, false>, mx_gemm_kernel<1, 1, 0, true>}, {mx_gemm_kernel<1, 1, 1, false>, mx_gemm_kernel<1, 1, 1, true>}}},
        {{{mx_gemm_kernel<2, 0, 0, false>, mx_gemm_kernel<2, 0, 0, true>}, {mx_gemm_kernel<2, 0, 1, false>, mx_gemm_kernel<2, 0, 1, true>}},
         {{mx_gemm_kernel<2, 1, 0, false>, mx_gemm_kernel<2, 1, 0, true>}, {mx_gemm_kernel<2, 1, 1, false>, mx_gemm_kernel<2, 1, 1, true>}}},
    };
    return table[cta_group - 1][major_a][major_b][decode_b ? 1 : 0];
}

int get_status_pointer(int32_t** out) {
    static std::mutex mu;
    static int32_t* ptrs[64] = {};
    int dev = 0;
    DG_CHECK_CUDA(cudaGetDevice(&dev));
    DG_CHECK_ARG(dev >= 0 && dev < 64, "device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        DG_CHECK_CUDA(cudaGetSymbolAddress(&p, g_device_status));
        DG_CHECK_CUDA(cudaMemset(p, 0, sizeof(int32_t)));
        ptrs[dev] = static_cast<int32_t*>(p);
    }
    *out = ptrs[dev];
    return DG_OK;
}

int launch_gemm_kernel(const LaunchPlan& plan, cudaStream_t stream) {
    KernelFn fn = pick_kernel(plan.cta_group, plan.major_a, plan.major_b, plan.decode_b, plan.lean, plan.fp4_pair, plan.bf16_pair, plan.wide_epi, plan.simple_epi, plan.wide_tile);
    // The attribute is per device and per function; setting it is cheap, so do it on every launch.
    DG_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));

    GemmKernelArgs args = plan.args;
    DG_CHECK_ARG(get_status_pointer(&args.status) == DG_OK, "%s", dg_last_error());

    // DG_TRACE=1 (debugging only): the launch becomes synchronous and prints where each CTA spent its time.
    static const bool trace_enabled = [] { const char* e = getenv("DG_TRACE"); return e && atoi(e) != 0; }();
    static unsigned long long* trace_buf = nullptr;
    if (trace_enabled) {
        if (trace_buf == nullptr) DG_CHECK_CUDA(cudaMalloc(&trace_buf, 2048 * 16 * sizeof(unsigned long long)));
        DG_CHECK_CUDA(cudaMemsetAsync(trace_buf, 0, 2048 * 16 * sizeof(unsigned long long), stream));
        args.trace = trace_buf;
    }

    if (plan.zero_empty_groups) {
        zero_empty_k_groups_kernel<<<148, 256, 0, stream>>>(static_cast<uint8_t*>(plan.zero_d), plan.args.grouped_layout,
                                                            plan.args.num_groups, plan.args.m, plan.zero_row_bytes,
                                                            plan.zero_row_pitch, plan.zero_group_pitch);
        DG_CHECK_CUDA(cudaGetLastError());
        count_kernel_launch();
    }

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.num_ctas, 1, 1);
    cfg.blockDim = dim3((plan.decode_b || plan.wide_epi) ? kNumThreadsDecode : kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = plan.cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // A persistent grid must be fully co-resident: a CTA (pair) that only starts after another one has finished its
    // whole tile sequence doubles the run time. Not every SM pair can host a 2-CTA cluster, so ask the runtime.
    uint32_t grid = plan.num_ctas;
    if (plan.cta_group > 1) {
        struct Key { const void* fn; uint32_t smem; int dev; int clusters; };
        static std::mutex mu;
        static Key cache[32];
        static int cached = 0;
        int dev = 0;
        DG_CHECK_CUDA(cudaGetDevice(&dev));
        int clusters = -1;
        {
            std::lock_guard<std::mutex> lock(mu);
            for (int i = 0; i < cached; ++i)
                if (cache[i].fn == (const void*)fn && cache[i].smem == plan.smem_bytes && cache[i].dev == dev) clusters = cache[i].clusters;
        }
        if (clusters < 0) {
            cudaLaunchConfig_t probe = cfg;
            probe.gridDim = dim3(148 * 2, 1, 1);
            DG_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&clusters, fn, &probe));
            std::lock_guard<std::mutex> lock(mu);
            if (cached < 32) cache[cached++] = Key{(const void*)fn, plan.smem_bytes, dev, clusters};
        }
        DG_CHECK_ARG(clusters > 0, "no CTA pair of this kernel fits on the device");
        if (grid > (uint32_t)clusters * plan.cta_group) grid = (uint32_t)clusters * plan.cta_group;
        cfg.gridDim = dim3(grid, 1, 1);
    }
    DG_CHECK_CUDA(cudaLaunchKernelEx(&cfg, fn, plan.tm_a, plan.tm_b, plan.tm_sfa, plan.tm_sfb, plan.tm_d, plan.tm_d_tail, args));
    count_kernel_launch();
    if (trace_enabled) {
        DG_CHECK_CUDA(cudaStreamSynchronize(stream));
        static unsigned long long host[1024 * 16];
        const uint32_t n = grid < 1024 ? grid : 1024;
        DG_CHECK_CUDA(cudaMemcpy(host, trace_buf, n * 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        unsigned long long t0 = ~0ull, t1 = 0;
        double sum[16] = {0}, mx[16] = {0};
        for (uint32_t i = 0; i < n; ++i) {
            if (host[i * 16] < t0) t0 = host[i * 16];
            if (host[i * 16] > t1) t1 = host[i * 16];
            for (int j = 2; j < 16; ++j) {
                const double d = host[i * 16 + j] ? (double)(host[i * 16 + j] - host[i * 16 + 1]) : 0.0;
                sum[j] += d; if (d > mx[j]) mx[j] = d;
            }
        }
        fprintf(stderr, "[dg_trace] producer: role-start %.0f sched %.0f wait %.0f ab-issued %.0f stage0-issued %.0f | epilogue: sent %.0f reduce-ready %.0f chunks-done %.0f\n",
                sum[8] / n, sum[9] / n, sum[10] / n, sum[11] / n, sum[12] / n, sum[13] / n, sum[14] / n, sum[15] / n);
        fprintf(stderr, "[dg_trace] m=%u n=%u k=%u bn=%u cg=%d split=%u ctas=%u start-skew=%.2f us | cycles since entry avg/max: "
                "setup %.0f/%.0f  first-tma %.0f/%.0f  first-data %.0f/%.0f  last-mma %.0f/%.0f  first-acc %.0f/%.0f  epi-done %.0f/%.0f\n",
                args.m, args.n, args.k, args.block_n, plan.cta_group, args.split_k, grid, (t1 - t0) / 1e3,
                sum[2] / n, mx[2], sum[3] / n, mx[3], sum[4] / n, mx[4], sum[5] / n, mx[5], sum[6] / n, mx[6], sum[7] / n, mx[7]);
    }

#ifdef DG_EPI_PROF
    if (trace_enabled) {
        static unsigned long long h2[1024 * 16];
        const uint32_t n = grid < 1024 ? grid : 1024;
        DG_CHECK_CUDA(cudaMemcpy(h2, trace_buf + 1024 * 16, n * 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        double s[16] = {0};
        for (uint32_t i = 0; i < n; ++i) for (int j = 0; j < 16; ++j) s[j] += (double)h2[i * 16 + j];
        const double ch = s[8] > 0 ? s[8] : 1, tl = s[12] > 0 ? s[12] : 1;
        fprintf(stderr, "[dg_epi] tiles/cta %.1f chunks/tile %.1f | per chunk: ldissue %.0f ldwait %.0f pre %.0f cvt %.0f math %.0f storewait %.0f stsmem %.0f | per box-ish (per chunk avg): fence %.0f issue %.0f | per tile: accwait %.0f epilogue %.0f\n",
                tl / n, ch / tl, s[10] / ch, s[0] / ch, s[11] / ch, s[9] / ch, s[1] / ch, s[2] / ch, s[3] / ch, s[4] / ch, s[5] / ch, s[6] / tl, s[7] / tl);
        const double tiles_lead = tl / plan.cta_group;
        fprintf(stderr, "[dg_mma] per tile: accumulator-free wait %.0f  data wait %.0f (first K block %.0f)\n",
                s[13] / tiles_lead, s[14] / tiles_lead, s[15] / tiles_lead);
    }
#endif
    if (plan.finalize) {
        const uint64_t total = (uint64_t)plan.args.m * ((plan.args.n + 3) / 4);
        const uint32_t grid = (uint32_t)((total + 255) / 256 < 148ull * 8 ? (total + 255) / 256 : 148ull * 8);
        splitk_finalize_kernel<<<grid, 256, 0, stream>>>(plan.ws, plan.ws_stride, plan.final_d, plan.final_d_stride,
                                                         plan.args.m, plan.args.n, plan.final_d_is_fp32,
                                                         plan.final_accumulate, plan.final_bias);
        DG_CHECK_CUDA(cudaGetLastError());
        count_kernel_launch();
    }
    return DG_OK;
}

}  // namespace dg

extern "C" int dg_device_status(int32_t* out_status) {
    DG_CHECK_ARG(out_status != nullptr, "dg_device_status: null output");
    int32_t* p = nullptr;
    if (int rc = dg::get_status_pointer(&p)) return rc;
    DG_CHECK_CUDA(cudaDeviceSynchronize());
    DG_CHECK_CUDA(cudaMemcpy(out_status, p, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (*out_status != 0) DG_CHECK_CUDA(cudaMemset(p, 0, sizeof(int32_t)));
    return DG_OK;
}
