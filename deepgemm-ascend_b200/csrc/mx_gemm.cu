// Instantiation and launch of the block-scaled GEMM kernel, plus the split-K finalisation kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <mutex>

#include "host_common.h"
#include "launch.h"
#include "mx_gemm.cuh"

namespace dg {

// Device status word: 0, or the code of the first bounded wait that gave up (zero from module load on: nothing has
// to be cleared, and so nothing synchronises, before the first launch on a device).
__device__ int32_t g_device_status = 0;

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

int query_resident_clusters(uint32_t cluster_size, int* out) {
    KernelFn fn = mx_gemm_kernel<1, 0, 0, false, true>;          // the lean kernel, which is what splits K over a cluster
    constexpr int kSmem = 200 * 1024;                             // one CTA per SM, as every tiling of that kernel has
    DG_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(cluster_size * 148, 1, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DG_CHECK_CUDA(cudaOccupancyMaxActiveClusters(out, fn, &cfg));
    return DG_OK;
}

// Caller-owned trace buffers, one per device (see dg_debug_set_trace_buffer).
static std::mutex g_trace_mu;
static unsigned long long* g_trace_buf[64] = {};
static size_t g_trace_bytes[64] = {};

// 1: GEMM kernels are launched with programmatic stream serialisation (default; DG_OVERLAP_LAUNCHES=0 or
// dg_set_overlap_launches(0) turns it off).
static std::atomic<int> g_overlap_launches{-1};
bool overlap_launches_enabled() {
    int v = g_overlap_launches.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("DG_OVERLAP_LAUNCHES");
        v = (e == nullptr || atoi(e) != 0) ? 1 : 0;
        g_overlap_launches.store(v, std::memory_order_relaxed);
    }
    return v != 0;
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
        ptrs[dev] = static_cast<int32_t*>(p);
    }
    *out = ptrs[dev];
    return DG_OK;
}

int launch_gemm_kernel(const LaunchPlan& plan, cudaStream_t stream) {
    KernelFn fn = pick_kernel(plan.cta_group, plan.major_a, plan.major_b, plan.decode_b, plan.lean, plan.fp4_pair, plan.bf16_pair, plan.wide_epi, plan.simple_epi, plan.wide_tile);
    int dev = 0;
    DG_CHECK_CUDA(cudaGetDevice(&dev));
    DG_CHECK_ARG(dev >= 0 && dev < 64, "device index out of range");
    // The dynamic shared-memory limit is an attribute per device and per function: raise it when a launch needs more
    // than any earlier launch of that function on that device did.
    {
        struct Raised { const void* fn; int dev; uint32_t bytes; };
        static std::mutex mu;
        static Raised raised[128];
        static int count = 0;
        std::lock_guard<std::mutex> lock(mu);
        int slot = -1;
        for (int i = 0; i < count; ++i)
            if (raised[i].fn == (const void*)fn && raised[i].dev == dev) { slot = i; break; }
        if (slot < 0 || raised[slot].bytes < plan.smem_bytes) {
            DG_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));
            if (slot < 0 && count < 128) slot = count++;
            if (slot >= 0) raised[slot] = Raised{(const void*)fn, dev, plan.smem_bytes};
        }
    }

    GemmKernelArgs args = plan.args;
    if (int rc = get_status_pointer(&args.status)) return rc;

    // Debugging aid: per-CTA timestamps go to a buffer the caller handed over (dg_debug_set_trace_buffer), if any.
    {
        std::lock_guard<std::mutex> lock(g_trace_mu);
        args.trace = (dev >= 0 && dev < 64 && g_trace_bytes[dev] >= (size_t)plan.num_ctas * kTraceSlots * sizeof(unsigned long long))
                         ? g_trace_buf[dev] : nullptr;
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
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = plan.cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Programmatic dependent launch: the kernel may be scheduled while the kernel in front of it in the stream is
    // still draining; it waits for that kernel (griddepcontrol.wait) before it reads or writes any global data.
    if (overlap_launches_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    // A persistent grid must be fully co-resident: a CTA (pair) that only starts after another one has finished its
    // whole tile sequence doubles the run time. Not every SM pair can host a 2-CTA cluster, so ask the runtime.
    uint32_t grid = plan.num_ctas;
    if (plan.cta_group > 1) {
        struct Key { const void* fn; uint32_t smem; int dev; int clusters; };
        static std::mutex mu;
        static Key cache[32];
        static int cached = 0;
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

namespace dg {
// One thread per pair of packed bytes: four codes in, four E4M3 bytes out (two 2-byte stores).
__global__ void expand_fp4_kernel(const uint8_t* __restrict__ src, uint64_t src_pitch, uint8_t* __restrict__ dst, uint64_t dst_pitch,
                                  uint64_t rows, uint64_t packed_bytes) {
    const uint64_t pairs = (packed_bytes + 1) / 2, total = rows * pairs;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / pairs, c = (i - r * pairs) * 2;
        const uint8_t* s = src + r * src_pitch + c;
        const bool two = c + 1 < packed_bytes;
        const uint32_t codes = (uint32_t)s[0] | (two ? (uint32_t)s[1] << 8 : 0u);
        const uint32_t out = e2m1x4_to_e4m3x4(codes);
        uint16_t* d = reinterpret_cast<uint16_t*>(dst + r * dst_pitch + 2 * c);
        d[0] = (uint16_t)(out & 0xFFFFu);
        if (two) d[1] = (uint16_t)(out >> 16);
    }
}
}  // namespace dg

extern "C" int dg_expand_fp4_launch(const void* src, uint64_t src_pitch_bytes, void* dst, uint64_t dst_pitch_bytes,
                                    uint64_t rows, uint64_t packed_bytes, void* stream) {
    DG_CHECK_ARG(src != nullptr && dst != nullptr, "expand_fp4: null pointer");
    DG_CHECK_ARG(dst_pitch_bytes >= 2 * packed_bytes && dst_pitch_bytes % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) & 1) == 0,
                 "expand_fp4: destination rows must hold two bytes per packed byte and be 2-byte aligned");
    if (rows == 0 || packed_bytes == 0) return DG_OK;
    const uint64_t total = rows * ((packed_bytes + 1) / 2);
    const uint32_t grid = (uint32_t)((total + 255) / 256 < 148ull * 16 ? (total + 255) / 256 : 148ull * 16);
    dg::expand_fp4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(src), src_pitch_bytes, static_cast<uint8_t*>(dst), dst_pitch_bytes, rows, packed_bytes);
    DG_CHECK_CUDA(cudaGetLastError());
    dg::count_kernel_launch();
    return DG_OK;
}

extern "C" int dg_set_overlap_launches(int enabled) {
    dg::g_overlap_launches.store(enabled ? 1 : 0, std::memory_order_relaxed);
    return DG_OK;
}
extern "C" int dg_get_overlap_launches(void) { return dg::overlap_launches_enabled() ? 1 : 0; }

extern "C" int dg_debug_set_trace_buffer(void* device_buffer, size_t bytes) {
    int dev = 0;
    DG_CHECK_CUDA(cudaGetDevice(&dev));
    DG_CHECK_ARG(dev >= 0 && dev < 64, "device index out of range");
    DG_CHECK_ARG((reinterpret_cast<uintptr_t>(device_buffer) & 7) == 0, "the trace buffer must be 8-byte aligned");
    std::lock_guard<std::mutex> lock(dg::g_trace_mu);
    dg::g_trace_buf[dev] = static_cast<unsigned long long*>(device_buffer);
    dg::g_trace_bytes[dev] = device_buffer ? bytes : 0;
    return DG_OK;
}

extern "C" int dg_device_status(int32_t* out_status) {
    DG_CHECK_ARG(out_status != nullptr, "dg_device_status: null output");
    int32_t* p = nullptr;
    if (int rc = dg::get_status_pointer(&p)) return rc;
    DG_CHECK_CUDA(cudaDeviceSynchronize());
    DG_CHECK_CUDA(cudaMemcpy(out_status, p, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (*out_status != 0) DG_CHECK_CUDA(cudaMemset(p, 0, sizeof(int32_t)));
    return DG_OK;
}
