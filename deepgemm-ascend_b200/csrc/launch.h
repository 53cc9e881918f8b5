// The launch plan: everything the host derives from (descriptor, configuration) before enqueueing.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "mx_gemm.cuh"

namespace dg {

struct LaunchPlan {
    GemmKernelArgs args;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb, tm_d, tm_d_tail;
    int cta_group, major_a, major_b;
    bool decode_b;               // B is packed E2M1 and is decoded to E4M3 in shared memory
    uint32_t num_ctas, smem_bytes;
    bool wide_epi;                    // eight epilogue warps (384 threads)
    bool wide_tile;                   // block_n > 256: two column halves per K step
    bool simple_epi;                  // the instantiation whose epilogue only casts to BF16 and issues TMA stores
    bool bf16_pair;                   // both operands BF16 (kind::f16, no scale factors)
    bool fp4_pair;                    // both operands packed E2M1 (kind::mxf4)
    bool lean;                        // the instantiation without the staged-store / alpha / stochastic / FP8 epilogues
    uint32_t cluster_x;               // cluster size: the CTA pair, or the K splits that reduce through shared memory
    // k-grouped layout without accumulation: zero D[g] of the groups that own no K
    bool zero_empty_groups;
    void* zero_d;
    uint64_t zero_row_bytes, zero_row_pitch, zero_group_pitch;
    // split-K finalisation (workspace -> D)
    bool finalize;
    float* ws;
    uint64_t ws_stride;
    void* final_d;
    uint64_t final_d_stride;
    uint32_t final_d_is_fp32, final_accumulate;
    const void* final_bias;
};

int launch_gemm_kernel(const LaunchPlan& plan, cudaStream_t stream);
int get_status_pointer(int32_t** out);
// How many thread-block clusters of `cluster_size` single-CTA-per-SM GEMM CTAs the current device keeps resident at once
// (a cluster must fit into one GPC). Loads the kernel: call it only where a launch is about to happen anyway.
int query_resident_clusters(uint32_t cluster_size, int* out);

}  // namespace dg
