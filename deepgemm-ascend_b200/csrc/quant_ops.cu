// The step in front of a block-scaled GEMM: BF16 activations -> E4M3 with one UE8M0 scale per 32 channels, the scales
// written straight into the layout the GEMM reads (int16 [tokens, ceil(H/64)], token-major columns), so that no
// scale-factor relayout runs between the producer and the GEMM. Optionally with SwiGLU in front
// (out = silu(x[:, :H]) * x[:, H:] * weight), which is the operator between the two expert GEMMs of an MoE layer.
//
// Follows third-party/tilelang_ops/swiglu_apply_weight_to_fp8.py of the reference: clamp (:156-161), SiLU = x / (1 + e^-x)
// (:162-165; here with the fast exponential and the hardware reciprocal, each within 2 ulp of the exact operation: a value
// on a rounding boundary of E4M3 may land on the neighbouring code, and the exact division cost a third of the run time), scale = 2^ceil(log2(max(amax, 1e-4) / 448)) from the bit pattern (:80-90), values times the
// inverse scale rounded to E4M3 (:250-252), packed scales transposed per group of 32 tokens (:104-125), tokens in
// the padding of a psum layout skipped (:263-268).
//
// HBM-bound: 4 H bytes read and H + H/32 bytes written per token (2 H + H + H/32 without SwiGLU).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dg_b200.h"
#include "host_common.h"

namespace dg {

constexpr uint32_t kTokenGroup = 32;         // tokens per CTA: one 64-byte run of every scale column
constexpr uint32_t kQuantThreads = 256;      // 8 warps, 4 tokens each

struct QuantArgs {
    const __nv_bfloat16* x; uint64_t x_stride;          // [tokens, (swiglu ? 2 : 1) * hidden], elements
    uint8_t* out; uint64_t out_stride;                  // [tokens, hidden] E4M3
    uint8_t* out_sf; uint64_t sf_col_stride;            // int16 [ceil(hidden/64)][sf_col_stride] seen as bytes, 2 per token
    const float* weights;                               // [tokens] or nullptr
    const int32_t* psum; uint32_t num_experts, alignment;
    uint32_t tokens, hidden;
    float clamp; uint32_t has_clamp, swiglu;
};

// Expert whose aligned row range holds `token`, or num_experts.
__device__ __forceinline__ uint32_t expert_of(const QuantArgs& a, uint32_t token) {
    uint32_t lo = 0, hi = a.num_experts;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) / 2;
        const uint32_t end = ((uint32_t)__ldg(a.psum + mid) + a.alignment - 1) / a.alignment * a.alignment;
        if (end > token) hi = mid; else lo = mid + 1;
    }
    return lo;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__global__ void __launch_bounds__(kQuantThreads) quant_fp8_kernel(const QuantArgs a) {
    extern __shared__ uint8_t sf_smem[];                 // [kTokenGroup][groups_pad] scale bytes, groups_pad even
    const uint32_t groups = a.hidden / 32, groups_pad = (groups + 1) & ~1u;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t num_token_groups = (a.tokens + kTokenGroup - 1) / kTokenGroup;

    for (uint32_t tg = blockIdx.x; tg < num_token_groups; tg += gridDim.x) {
        const uint32_t token_base = tg * kTokenGroup;
        uint32_t valid_end = min(a.tokens, token_base + kTokenGroup);
        if (a.psum != nullptr) {
            const uint32_t e = expert_of(a, token_base);
            valid_end = e < a.num_experts ? min(valid_end, (uint32_t)max(__ldg(a.psum + e), 0)) : token_base;
        }
        if (valid_end <= token_base) continue;            // the whole group is padding (uniform over the CTA)

        for (uint32_t tl = warp; tl < kTokenGroup; tl += kQuantThreads / 32) {
            const uint32_t token = token_base + tl;
            if (token >= valid_end) break;
            const float weight = a.weights ? __ldg(a.weights + token) : 1.0f;
            const __nv_bfloat16* row = a.x + (uint64_t)token * a.x_stride;
            // one pass = 256 channels: lane l holds channels [8 l, 8 l + 8), four lanes make one 32-channel block;
            // the loads of kUnroll passes are issued before any of them is used
            constexpr uint32_t kUnroll = 4;
            for (uint32_t c0 = 0; c0 < a.hidden; c0 += 256 * kUnroll) {
                uint4 left[kUnroll], right[kUnroll];
                #pragma unroll
                for (uint32_t u = 0; u < kUnroll; ++u) {
                    const uint32_t c = c0 + u * 256 + lane * 8;
                    left[u] = right[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (c < a.hidden) {
                        left[u] = __ldg(reinterpret_cast<const uint4*>(row + c));
                        if (a.swiglu) right[u] = __ldg(reinterpret_cast<const uint4*>(row + a.hidden + c));
                    }
                }
                #pragma unroll
                for (uint32_t u = 0; u < kUnroll; ++u) {
                    const uint32_t c = c0 + u * 256 + lane * 8;
                    if (c0 + u * 256 >= a.hidden) break;          // uniform over the warp
                    const uint32_t lw[4] = {left[u].x, left[u].y, left[u].z, left[u].w};
                    const uint32_t rw[4] = {right[u].x, right[u].y, right[u].z, right[u].w};
                    float v[8];
                    if (a.swiglu) {
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float xl[2] = {bf16_lo(lw[i]), bf16_hi(lw[i])}, xr[2] = {bf16_lo(rw[i]), bf16_hi(rw[i])};
                            #pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                if (a.has_clamp) {
                                    xl[k] = fminf(xl[k], a.clamp);
                                    xr[k] = fmaxf(fminf(xr[k], a.clamp), -a.clamp);
                                }
                                const float silu = __fdividef(xl[k], 1.0f + __expf(-xl[k]));
                                float y = silu * xr[k];
                                if (a.weights) y *= weight;
                                v[i * 2 + k] = y;
                            }
                        }
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) { v[i * 2] = bf16_lo(lw[i]); v[i * 2 + 1] = bf16_hi(lw[i]); }
                    }
                    float amax = 0.f;
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    // scale = max(amax, 1e-4) * (1/448) rounded up to a power of two; exponent byte from the bit pattern
                    const uint32_t bits = __float_as_uint(fmaxf(amax, 1e-4f) * (1.0f / 448.0f));
                    const uint32_t e = ((bits - 1u) >> 23) + 1u;
                    const float inv = __uint_as_float((254u - e) << 23);
                    if (c < a.hidden) {
                        uint32_t q[2];
                        #pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(v[h * 4] * inv, v[h * 4 + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                            const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(v[h * 4 + 2] * inv, v[h * 4 + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                            q[h] = (uint32_t)p0 | ((uint32_t)p1 << 16);
                        }
                        *reinterpret_cast<uint2*>(a.out + (uint64_t)token * a.out_stride + c) = make_uint2(q[0], q[1]);
                        if ((lane & 3u) == 0) sf_smem[tl * groups_pad + c / 32] = (uint8_t)e;
                    }
                }
            }
            if (lane == 0 && groups_pad != groups) sf_smem[tl * groups_pad + groups] = 0;
        }
        __syncthreads();
        // scale column j (int16 = channels [64 j, 64 j + 64)) of the valid tokens: one contiguous run of 2-byte elements
        const uint32_t valid = valid_end - token_base, cols = groups_pad / 2;
        for (uint32_t i = threadIdx.x; i < cols * kTokenGroup; i += kQuantThreads) {
            const uint32_t col = i / kTokenGroup, tl = i % kTokenGroup;
            if (tl < valid) {
                const uint16_t pair = *reinterpret_cast<const uint16_t*>(sf_smem + tl * groups_pad + col * 2);
                *reinterpret_cast<uint16_t*>(a.out_sf + ((uint64_t)col * a.sf_col_stride + token_base + tl) * 2) = pair;
            }
        }
        __syncthreads();
    }
}

}  // namespace dg

using namespace dg;

extern "C" int dg_quant_fp8_launch(const void* x, uint64_t x_stride, uint32_t tokens, uint32_t hidden, int swiglu,
                                   const float* topk_weights, const int32_t* psum, uint32_t num_experts, uint32_t alignment,
                                   int has_clamp, float clamp_value, void* out, uint64_t out_stride,
                                   int16_t* out_sf, uint64_t sf_col_stride, void* stream) {
    DG_CHECK_ARG(x != nullptr && out != nullptr && out_sf != nullptr, "quant_fp8: null pointer");
    DG_CHECK_ARG(hidden > 0 && hidden % 32 == 0, "quant_fp8: hidden must be a multiple of 32");
    DG_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15) == 0 && x_stride % 8 == 0,
                 "quant_fp8: input rows must start on 16-byte boundaries");
    DG_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 7) == 0 && out_stride % 8 == 0,
                 "quant_fp8: output rows must start on 8-byte boundaries");
    DG_CHECK_ARG(!swiglu || hidden % 8 == 0, "quant_fp8: hidden must be a multiple of 8");
    DG_CHECK_ARG(sf_col_stride >= tokens, "quant_fp8: scale column stride smaller than the token count");
    DG_CHECK_ARG(psum == nullptr || (num_experts > 0 && alignment > 0 && alignment % kTokenGroup == 0),
                 "quant_fp8: a psum layout needs experts and an alignment that is a multiple of 32");
    if (tokens == 0) return DG_OK;
    QuantArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(x); a.x_stride = x_stride;
    a.out = static_cast<uint8_t*>(out); a.out_stride = out_stride;
    a.out_sf = reinterpret_cast<uint8_t*>(out_sf); a.sf_col_stride = sf_col_stride;
    a.weights = topk_weights; a.psum = psum; a.num_experts = psum ? num_experts : 0; a.alignment = alignment;
    a.tokens = tokens; a.hidden = hidden;
    a.clamp = clamp_value; a.has_clamp = has_clamp ? 1u : 0u; a.swiglu = swiglu ? 1u : 0u;
    const uint32_t groups_pad = (hidden / 32 + 1) & ~1u;
    const size_t smem = (size_t)kTokenGroup * groups_pad;
    DG_CHECK_ARG(smem <= 48 * 1024, "quant_fp8: hidden too large");
    const uint32_t token_groups = (tokens + kTokenGroup - 1) / kTokenGroup;
    const uint32_t grid = token_groups < 148u * 8 ? token_groups : 148u * 8;
    quant_fp8_kernel<<<grid, kQuantThreads, smem, static_cast<cudaStream_t>(stream)>>>(a);
    DG_CHECK_CUDA(cudaGetLastError());
    count_kernel_launch();
    return DG_OK;
}
