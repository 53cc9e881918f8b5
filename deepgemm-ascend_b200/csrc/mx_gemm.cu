// Instantiation and launch of the block-scaled GEMM kernel, plus the split-K finalisation kernel.
#include <cuda.h>
#include <cuda_runtime.h>
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

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const CUtensorMap, const GemmKernelArgs);

static KernelFn pick_kernel(int cta_group, int major_a, int major_b) {
    static const KernelFn table[2][2][2] = {
        {{mx_gemm_kernel<1, 0, 0>, mx_gemm_kernel<1, 0, 1>}, {mx_gemm_kernel<1, 1, 0>, mx_gemm_kernel<1, 1, 1>}},
        {{mx_gemm_kernel<2, 0, 0>, mx_gemm_kernel<2, 0, 1>}, {mx_gemm_kernel<2, 1, 0>, mx_gemm_kernel<2, 1, 1>}},
    };
    return table[cta_group - 1][major_a][major_b];
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
    KernelFn fn = pick_kernel(plan.cta_group, plan.major_a, plan.major_b);
    // The attribute is per device and per function; setting it is cheap, so do it on every launch.
    DG_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem_bytes));

    GemmKernelArgs args = plan.args;
    DG_CHECK_ARG(get_status_pointer(&args.status) == DG_OK, "%s", dg_last_error());

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.num_ctas, 1, 1);
    cfg.blockDim = dim3(kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = plan.cta_group;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DG_CHECK_CUDA(cudaLaunchKernelEx(&cfg, fn, plan.tm_a, plan.tm_b, plan.tm_sfa, plan.tm_sfb, plan.tm_d, args));

    if (plan.finalize) {
        const uint64_t total = (uint64_t)plan.args.m * ((plan.args.n + 3) / 4);
        const uint32_t grid = (uint32_t)((total + 255) / 256 < 148ull * 8 ? (total + 255) / 256 : 148ull * 8);
        splitk_finalize_kernel<<<grid, 256, 0, stream>>>(plan.ws, plan.ws_stride, plan.final_d, plan.final_d_stride,
                                                         plan.args.m, plan.args.n, plan.final_d_is_fp32,
                                                         plan.final_accumulate, plan.final_bias);
        DG_CHECK_CUDA(cudaGetLastError());
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
