/*
 * dg_b200.h — C ABI of libdg_b200.so: block-scaled FP8 / FP8xFP4 GEMM for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a DeepGEMM-Ascend host layer binds instead of its bisheng JIT: every entry
 * point replaces one `jit->compile(...)` + `jit->launch(...)` pair of the reference, or one host
 * helper directly in front of it. Plain C: pointers, sizes and enums only; no torch types.
 *
 * Conventions
 *   - every function returns 0 on success and a negative DG_ERR_* code otherwise; the message of the
 *     last failure on the calling thread is returned by dg_last_error();
 *   - nothing here synchronises the device or allocates device memory; all work is enqueued on the
 *     `stream` argument (a cudaStream_t passed as void*; NULL is the legacy default stream);
 *   - device pointers must belong to the device that is current on the calling thread;
 *   - functions are thread-safe (the reference pre-compiles from a thread pool).
 */
#ifndef DG_B200_H_
#define DG_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DG_B200_ABI_VERSION 3

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

enum {
    DG_OK = 0,
    DG_ERR_INVALID = -1,      /* argument rejected by validation (message says which) */
    DG_ERR_UNSUPPORTED = -2,  /* legal in the reference's API but not built here */
    DG_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed */
    DG_ERR_WORKSPACE = -4     /* workspace missing or too small */
};

/* deep_gemm/include/deep_gemm/common.hpp:82 (Major) */
typedef enum { DG_MAJOR_K = 0, DG_MAJOR_MN = 1 } dg_major_t;

/* deep_gemm/include/deep_gemm/common.hpp:87-92 (GemmType); MASKED is the entry point the reference
 * only names (csrc/apis/gemm.hpp:606,630). */
typedef enum {
    DG_GEMM_NORMAL = 0,
    DG_GEMM_M_GROUPED_PSUM = 1,
    DG_GEMM_K_GROUPED_PSUM = 2, /* A [M,K_total], B [N,K_total] (both MN-major), D [G,M,N]; csrc/apis/gemm.hpp:351-384 */
    DG_GEMM_BATCHED = 3,        /* A [B,M,K], B [B,N,K], D [B,M,N]; csrc/apis/einsum.hpp:37-71 */
    DG_GEMM_M_GROUPED_MASKED = 4
} dg_gemm_type_t;

/* csrc/utils/dtype.hpp:9 (packed FP4 is stored as int8, two E2M1 codes per byte, low nibble first) */
typedef enum { DG_E4M3 = 0, DG_E2M1X2 = 1, DG_BF16 = 2, DG_F32 = 3 } dg_dtype_t;

/* csrc/jit_kernels/epilogue_class.hpp:29-66 (Identity / ScaleByAlpha / AddBias) */
/* STOCHASTIC_BF16: csrc/jit_kernels/epilogue_class.hpp:68-78, operators.hpp:224-343 (BF16 output, no C) */
typedef enum {
    DG_EPILOGUE_IDENTITY = 0,
    DG_EPILOGUE_ALPHA = 1,
    DG_EPILOGUE_BIAS = 2,
    DG_EPILOGUE_STOCHASTIC_BF16 = 3,
    DG_EPILOGUE_FP8_QUANT = 4   /* E4M3 output + UE8M0 scales per 1x32, epilogue_class.hpp:80-108, operators.hpp:345-447 */
} dg_epilogue_t;

/*
 * Problem descriptor. Mirrors GemmDesc, csrc/jit_kernels/gemm_config.hpp:39-95, plus the
 * epilogue::Args of deep_gemm/include/deep_gemm/common.hpp:96-102.
 *
 *   Normal            A [M,K]          B [N,K]        D [M,N]
 *   M-grouped psum    A [M_total,K]    B [G,N,K]      D [M_total,N]     grouped_layout = psum int32[G]
 *   M-grouped masked  A [G,max_m,K]    B [G,N,K]      D [G,max_m,N]     grouped_layout = masked_m int32[G], m = max_m
 *   Batched           A [G,M,K]        B [G,N,K]      D [G,M,N]         num_groups = G, no layout array
 *   K-grouped psum    A [M,K_total]    B [N,K_total]  D [G,M,N]         grouped_layout = psum int32[G] along K; empty
 *                                                                       groups give D[g] = 0 (or leave it when accumulating)
 *
 * "[MN,K]" is the logical shape; `major_*` says which axis is contiguous in memory and
 * `outer_stride_*` is the stride of the other axis in ELEMENTS (bytes for packed FP4 operands:
 * the stride counts int8 storage elements). sfa / sfb are in the required layout
 * (int16 [MN, ceil(K/64)], MN-major, csrc/apis/layout.hpp:19-36); `sf*_stride` is the distance in
 * int16 elements between consecutive K64 columns (== MN for a dense tensor) and must be a multiple
 * of 8; sf*_group_stride is the distance between groups of scales in int16 elements.
 *
 * Operand dtype pairs (csrc/apis/gemm.hpp:22-33): E4M3 x E4M3; E4M3 x E2M1X2 (B read by the tensor cores as E2M1,
 * either major; decoded to E4M3 on the fly when TMA cannot unpack it); E2M1X2 x E2M1X2: tcgen05 kind::mxf4 at twice
 * the FP8 rate when A and B are K-major, kind::mxf8f6f4 with both operands read as E2M1 when one of them is MN-major
 * or the layout is the K-grouped one (a packed A must then satisfy dg_fp4_expansion_needed). Per-32 scales.
 * E2M1X2 x E4M3 is rejected as in the reference.
 * BF16 x BF16 (csrc/apis/gemm.hpp:412-514, launch_bf16_gemm): a_dtype = b_dtype = DG_BF16, sfa = sfb = NULL, strides in
 * BF16 elements, rows 16-byte aligned; every layout, both majors.
 */
typedef struct {
    const void* a;
    const void* b;
    void* d;
    const int16_t* sfa;
    const int16_t* sfb;
    int32_t a_dtype, b_dtype, d_dtype;        /* dg_dtype_t */
    uint32_t m, n, k;
    int32_t major_a, major_b;                 /* dg_major_t */
    uint64_t outer_stride_a, outer_stride_b, outer_stride_d;
    uint64_t group_stride_a, group_stride_b, group_stride_d; /* elements between groups (B always; A, D: masked) */
    uint64_t sfa_stride, sfb_stride;
    uint64_t sfa_group_stride, sfb_group_stride;             /* int16 elements between groups of scales */
    int32_t accumulate;                       /* D += A B^T (csrc/apis/gemm.hpp:106-112,180) */
    int32_t gemm_type;                        /* dg_gemm_type_t */
    const int32_t* grouped_layout;            /* device pointer, read on device only */
    uint32_t num_groups;
    uint32_t expected_m;                      /* heuristic hint (gemm_config.hpp:59) */
    int32_t epilogue;                         /* dg_epilogue_t */
    float alpha;
    const void* bias;                         /* [1,N], D's dtype */
    uint32_t num_sms;                         /* cap of the persistent grid; 0 = all SMs */
    /* DG_EPILOGUE_FP8_QUANT only (d_dtype = DG_E4M3): int16 scale output [M, groups * N / 64], two UE8M0 bytes per
     * element, element (row, col) at sfd[col * sfd_stride + row]; batch g owns columns [g*N/64, (g+1)*N/64) */
    int16_t* sfd;
    uint64_t sfd_stride;
    /* use_deterministic_algorithms, csrc/apis/runtime.hpp:56-62: non-zero keeps the heuristic away from every tiling
     * whose result depends on timing (split-K through the FP32 workspace, which adds partial sums in arrival order)
     * and makes an explicit config that asks for one an error. Everything else is bit-reproducible as it is. */
    int32_t deterministic;
    int32_t reserved0;                        /* must be 0 */
} dg_gemm_desc_t;

/* Tiling chosen for a problem. Replaces GemmConfig, csrc/jit_kernels/gemm_config.hpp:98-121. */
typedef struct {
    uint32_t block_m, block_n, block_k;   /* block_m = 128 x cta_group, block_k = 128 bytes of K; block_n a multiple of 32 up to 256,
                                           * or 320 / 384 / 448 (CTA pairs, E4M3 x E4M3, E2M1 x E2M1 or BF16 x BF16 (also 512), K-major operands): a wide
                                           * tile computed as two column halves per K step that share the A tile */
    uint32_t num_stages;
    uint32_t cta_group;       /* 1, or 2 = two CTAs of a cluster share one 256-row UMMA */
    uint32_t split_k;         /* >1: partial sums reduced in FP32 through the workspace */
    uint32_t num_ctas;        /* persistent grid size */
    uint32_t tmem_cols;
    uint32_t smem_bytes;
    uint32_t epilogue_mode;   /* 0 TMA store, 1 TMA reduce-add, 2 plain stores, 3 plain atomics */
    uint32_t reserved[6];     /* [0] TMEM accumulators (1 or 2, derived); [1] epilogue staging boxes per warp (0 = auto:
                               *     one when that buys a pipeline stage, else two; 1..4);
                               * [2] K stagger: tile column j starts its K loop at block (j * value) % blocks (0 = off);
                               * [3] split_k > 1 only: 0 = partial sums go to the FP32 workspace and a second kernel casts
                               *     them, 1 = the splits of a tile run as one thread-block cluster (cta_group 1,
                               *     split_k <= 8, B not packed) and reduce through shared memory: no workspace;
                               * [4] dense GEMM: row blocks per rasterisation group (tiles are handed out row block fastest
                               *     inside groups of this many row blocks, so that CTAs running together share their
                               *     B panels in L2); 0 = 8;
                               * [5] epilogue warps: 0 = auto, 1 = four, 2 = eight (two warps per TMEM lane quarter, each
                               *     taking alternate 32-column chunks; E4M3 x E4M3 with K-major operands only) */
} dg_gemm_config_t;

/* The B200 tiling heuristic. Replaces select_gemm_config, csrc/jit_kernels/heuristics.hpp:592-755. */
int dg_select_config(const dg_gemm_desc_t* desc, dg_gemm_config_t* out);

/* Bytes of zero-initialised device scratch dg_gemm_launch needs for (desc, config); 0 when none.
 * The library keeps the scratch zero between calls once the caller has zeroed it once. */
size_t dg_gemm_workspace_bytes(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config);

/* Enqueue the GEMM. Replaces launch_fp8_gemm / launch_fp4_gemm / launch_fp8_dequant_gemm,
 * csrc/jit_kernels/fp8_gemm.hpp:11-79,83-151 and csrc/jit_kernels/fp8_dequant_gemm.hpp:24-95.
 * `config` may be NULL (the heuristic is used). The first launch of a kernel variant on a device loads it, looks up
 * the status word's address and raises the variant's shared-memory limit: make one launch of every problem a stream
 * capture will contain before the capture begins (a warm-up pass does). */
int dg_gemm_launch(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config,
                   void* workspace, size_t workspace_bytes, void* stream);

/* dg_gemm_launch memoises what it derives on the host (validation, tiling, encoded tensor maps, kernel arguments) on
 * the bytes of (desc, config, workspace, device, SM limit): a call that repeats an earlier one only enqueues. The
 * reference re-runs its search per call (csrc/jit_kernels/heuristics.hpp:593). Counters for tests and benchmarks. */
void dg_plan_cache_stats(uint64_t* hits, uint64_t* misses);

/*
 * Split-K GEMM for callers that cannot allocate device memory. No counterpart in the reference.
 *
 * Some hosts of this library may not call cudaMalloc (or torch's allocator) around a GEMM: a runtime that has
 * handed all device memory to its own pool, code running inside a region where allocation is forbidden, a plugin
 * that only receives pointers. dg_gemm_launch asks exactly those callers for a zeroed workspace whenever the tiling
 * splits K. This entry point is the same GEMM with the FP32 partial-sum scratch taken from a fixed array inside the
 * library instead: DG_STATIC_SCRATCH_BYTES of device memory that every GPU which loads the library holds until the
 * process exits. The caller passes only inputs and outputs.
 *
 *   - it allocates nothing and calls no allocating routine;
 *   - problems whose scratch (m * round_up(n, 4) * 4 bytes, needed only when the tiling uses split_k > 1) exceeds
 *     DG_STATIC_SCRATCH_BYTES are rejected with DG_ERR_WORKSPACE and a message that states both sizes; pass a
 *     config with split_k = 1 or use dg_gemm_launch for those;
 *   - the first call on each device looks up the array's device address (with that device current); make that first
 *     call before any stream capture begins;
 *   - all calls share the one array, which keeps whatever the previous call left: the part a call needs is cleared
 *     on `stream` before the GEMM, and two calls whose GPU work overlaps (different streams, different threads) race
 *     on it — order them on one stream.
 */
#define DG_STATIC_SCRATCH_BYTES (4u << 20)
int dg_gemm_launch_static_scratch(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config, void* stream);

/* Validate (desc, config) and build the launch plan without touching the device: the counterpart
 * of the reference's dry-run compile, csrc/jit_kernels/fp8_gemm.hpp:67-70. */
int dg_gemm_dry_run(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config);

/*
 * Scale-factor relayout into the required layout. Replaces launch_transform_sf,
 * csrc/jit_kernels/transform_sf.hpp:15-105, and the device kernel
 * deep_gemm/include/deep_gemm/transform_sf.hpp:447-639.
 *
 *   src            fp32 [B, src_rows, src_cols] (src_is_fp32) or int16 with two UE8M0 bytes per element
 *   src_row_stride / src_col_stride / src_batch_stride   in source elements (either major is fine)
 *   dst            int16, element (b, mn, c) at dst[b*dst_batch_stride + c*dst_col_stride + mn]
 *   dst_mn         rows of the result; row mn reads source row mn / gran_mn
 *   k32_blocks     number of 32-wide K blocks of the operand, ceil(K/32)
 *   k_repeat       1 (gran_k = 32) or 4 (gran_k = 128: each source scale covers four blocks)
 *   psum           NULL, or int32[num_groups] psum layout: rows in a group's padding get scale byte 0
 *   k_psum         NULL, or int32[num_k_groups] psum layout along K (K-grouped operands,
 *                  csrc/apis/layout.hpp:94-111): scales of the K units inside a group's padding become 0
 *   invalid_flag   NULL, or a device int32 set to 1 when an fp32 scale is negative or has mantissa bits
 *                  (the reference asserts on device, transform_sf.hpp:13-21; this library never traps)
 */
int dg_transform_sf_launch(const void* src, int src_is_fp32,
                           uint64_t src_row_stride, uint64_t src_col_stride, uint64_t src_batch_stride,
                           uint32_t src_rows, uint32_t src_cols,
                           int16_t* dst, uint64_t dst_col_stride, uint64_t dst_batch_stride,
                           uint32_t dst_mn, uint32_t k32_blocks, uint32_t gran_mn, uint32_t k_repeat,
                           uint32_t num_batches, const int32_t* psum, uint32_t num_groups,
                           uint32_t alignment, int32_t* invalid_flag,
                           const int32_t* k_psum, uint32_t num_k_groups, void* stream);

/* BF16 activations -> E4M3 plus UE8M0 scales per 1x32, the scales written directly in the layout the GEMM reads
 * (int16 [tokens, ceil(hidden/64)], consecutive tokens contiguous, `sf_col_stride` int16 elements between columns), so
 * no dg_transform_sf_launch runs between this producer and the GEMM. With `swiglu` the input row is [2 * hidden] and
 * the quantised value is silu(x[:hidden]) * x[hidden:] (* topk_weights[token]), optionally clamped: the reference's
 * third-party/tilelang_ops/swiglu_apply_weight_to_fp8.py:411-449 (the operator between the two expert GEMMs of an MoE
 * layer). Without `swiglu` it is the plain cast of x[tokens, hidden] (no reference counterpart: the reference has no
 * stand-alone quantiser). `psum` / `num_experts` / `alignment`: tokens in the padding of a psum layout are skipped, the
 * alignment must be a multiple of 32. hidden % 32 == 0; x rows 16-byte aligned, out rows 8-byte aligned. */
int dg_quant_fp8_launch(const void* x, uint64_t x_stride, uint32_t tokens, uint32_t hidden, int swiglu,
                        const float* topk_weights, const int32_t* psum, uint32_t num_experts, uint32_t alignment,
                        int has_clamp, float clamp_value, void* out, uint64_t out_stride,
                        int16_t* out_sf, uint64_t sf_col_stride, void* stream);

/* Copy a 2-D byte matrix into a buffer whose row pitch satisfies the 16-byte rule of TMA, zero
 * filling the tail of each row. Used for operands whose contiguous extent is not a multiple of 16
 * bytes (the unaligned-K / unaligned-MN cases of tests/generators.py:491-541). */
int dg_pad_rows_launch(const void* src, uint64_t src_pitch_bytes, void* dst, uint64_t dst_pitch_bytes,
                       uint64_t rows, uint64_t row_bytes, void* stream);

/* Expand a 2-D matrix of packed E2M1 codes (two per byte along the row, low nibble first) into E4M3 bytes, exactly
 * (every E2M1 value is an E4M3 value; the byte map of deep_gemm/include/deep_gemm/fp8_dequant_gemm.hpp:24-38). For packed
 * operands that the GEMM cannot take as they are: a packed A (or a k-grouped packed B) whose base, strides or extent
 * break the rules of TMA's 4-bit unpacking. dst row r holds 2 * packed_bytes bytes; dst 2-byte aligned, pitch even. */
int dg_expand_fp4_launch(const void* src, uint64_t src_pitch_bytes, void* dst, uint64_t dst_pitch_bytes,
                         uint64_t rows, uint64_t packed_bytes, void* stream);

/* Which packed-FP4 operands of `desc` the GEMM cannot take as they are and the caller has to expand to E4M3 first
 * (dg_expand_fp4_launch): a packed A outside the K-major x K-major FP4 kernel, or a packed B of the k-grouped layout,
 * whose base or strides are not multiples of 32 bytes or whose contiguous extent is not a multiple of 128 elements.
 * No reference counterpart: its kernels load packed operands in either major themselves. */
int dg_fp4_expansion_needed(const dg_gemm_desc_t* desc, int* expand_a, int* expand_b);

/* Thread-block clusters of `cluster_size` (1..8) CTAs, one CTA per SM, that the tiling heuristic assumes are resident at
 * once when it splits K over a cluster: figures measured on B200 until the first dg_gemm_launch of the process has asked
 * the runtime (cudaOccupancyMaxActiveClusters) for the device's own. No reference counterpart. */
uint32_t dg_resident_clusters(uint32_t cluster_size);

/* Writes a buffer larger than L2 so that the next kernel starts cold (deep_gemm/testing/bench.py:263-268). */
int dg_l2_flush_launch(void* buffer, size_t bytes, void* stream);

/* Device-side status word of the most recent kernels on this device: 0, or a code recorded by a
 * bounded wait that gave up. Reading it synchronises the device. */
int dg_device_status(int32_t* out_status);

/* Number of kernels this library has enqueued in this process (all devices, all threads). Benchmarks
 * read it before and after a timed region to report how many of the library's kernels ran. */
uint64_t dg_kernel_launch_count(void);

/* Busy-wait marker kernel, one block per SM for `sleep_cycles` SM clock cycles (at most 4e9, about two seconds):
 * replaces npu_sleep, csrc/apis/runtime.hpp:64-79 + deep_gemm/include/deep_gemm/sleep.hpp:5-15. `marker` only selects
 * the kernel's name (sleep_kernel<0>, <1>, <2>; any other value shares <3>) so that a profiler can find begin / end
 * marks; `num_blocks` is the grid size (the reference launches one block per core). */
int dg_sleep_launch(int64_t sleep_cycles, uint32_t marker, int num_blocks, void* stream);

/* GEMM kernels are launched with programmatic stream serialisation by default: a GEMM may be scheduled while the
 * kernel in front of it in the stream is still draining, runs its set-up (barriers, TMEM allocation, descriptor
 * prefetch) and then waits for that kernel before it touches operands or outputs, so results are unchanged. 0 turns
 * it off (also: environment DG_OVERLAP_LAUNCHES=0). No counterpart in the reference. */
int dg_set_overlap_launches(int enabled);
int dg_get_overlap_launches(void);

/* Debugging aid, no counterpart in the reference: hand the library a device buffer of at least 256 bytes per CTA and
 * every GEMM kernel launched on the current device afterwards records per-CTA timestamps in it (32 slots of 8 bytes
 * per CTA: kernel entry, set-up done, first operands landed, last MMA, epilogue done, kernel end, ...); NULL stops it. The
 * library neither allocates, reads nor synchronises for this. */
int dg_debug_set_trace_buffer(void* device_buffer, size_t bytes);

/* Runtime knobs, csrc/apis/runtime.hpp:12-62 / csrc/jit/jit.hpp:18-76. */
int dg_get_num_sms(void);
int dg_set_num_sms(int num_sms);
int dg_get_mk_alignment_for_contiguous_layout(void); /* fixed at 256, csrc/jit/jit.hpp:59-73 */

const char* dg_last_error(void);
int dg_abi_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* DG_B200_H_ */
