// C ABI of libdg_b200.so: validation, the B200 tiling heuristic, TMA descriptor construction, launch.
//
// Host-side counterpart of the reference's launchers (csrc/jit_kernels/fp8_gemm.hpp:11-151,
// fp8_dequant_gemm.hpp:24-95), of its tiling search (csrc/jit_kernels/heuristics.hpp:592-755) and of the
// runtime knobs (csrc/jit/jit.hpp:18-76). Nothing here allocates device memory or synchronises.
#include <string>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "host_common.h"
#include "launch.h"

namespace dg {

// ------------------------------------------------------------------------------------------------
// Errors
// ------------------------------------------------------------------------------------------------
static thread_local char tls_error[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
    va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};
void count_kernel_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ------------------------------------------------------------------------------------------------
// Runtime knobs
// ------------------------------------------------------------------------------------------------
static std::atomic<int> g_num_sms{0};   // 0 = not set: use the device's SM count

static int device_sm_count() {
    static std::atomic<int> cached{0};
    int v = cached.load();
    if (v > 0) return v;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
        cached.store(sms);
        return sms;
    }
    (void)cudaGetLastError();
    return 148;    // B200; used when planning without a device (dry run)
}

// Thread-block clusters of a given size that are resident at once with one CTA per SM. A cluster lives inside one GPC,
// so this is less than SMs / size. The table holds what cudaOccupancyMaxActiveClusters reports on a B200 (and what the
// timings show: 33 clusters of 4 run as one wave and 34 take two; 24 of 5 run as one and 27 do not; 18 of 6 do and 24 do
// not); the first real launch replaces it with the figures of the device at hand.
static std::atomic<uint32_t> g_cluster_capacity[9] = {{0}, {148}, {74}, {45}, {33}, {26}, {22}, {15}, {15}};
static void refresh_cluster_capacity() {
    static std::once_flag once;
    std::call_once(once, [] {
        for (uint32_t size = 2; size <= 8; ++size) {
            int n = 0;
            if (query_resident_clusters(size, &n) == DG_OK && n > 0) g_cluster_capacity[size].store((uint32_t)n);
        }
        (void)cudaGetLastError();
    });
}

static uint32_t effective_num_sms(const dg_gemm_desc_t& d) {
    int n = d.num_sms ? (int)d.num_sms : (g_num_sms.load() > 0 ? g_num_sms.load() : device_sm_count());
    return (uint32_t)(n < 1 ? 1 : n);
}

// ------------------------------------------------------------------------------------------------
// Small helpers
// ------------------------------------------------------------------------------------------------
static inline uint32_t ceil_div_u32(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
static inline uint64_t align_u64(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline uint32_t elem_size(int dtype) { return dtype == DG_F32 ? 4u : dtype == DG_BF16 ? 2u : 1u; }

static bool is_grouped(int t) {
    return t == DG_GEMM_M_GROUPED_PSUM || t == DG_GEMM_M_GROUPED_MASKED || t == DG_GEMM_BATCHED || t == DG_GEMM_K_GROUPED_PSUM;
}
// A, SFA and D carry a group / batch dimension of their own (the psum layout keeps them flat)
static bool has_row_groups(int t) { return t == DG_GEMM_M_GROUPED_MASKED || t == DG_GEMM_BATCHED; }

// Can D (or the split-K workspace) be written through TMA?
static bool tma_store_ok(const dg_gemm_desc_t& d) {
    const uint32_t es = elem_size(d.d_dtype);
    return aligned16(d.d) && (d.outer_stride_d * es) % 16 == 0 &&
           ((!has_row_groups(d.gemm_type) && d.gemm_type != DG_GEMM_K_GROUPED_PSUM) || (d.group_stride_d * es) % 16 == 0);
}

// Both operands packed E2M1 and K-major: the kind::mxf4 path (which reads K-major operands only). The kernel then
// counts K in bytes (two elements each). Packed E2M1 operands in any other arrangement (an MN-major one among them,
// the k-grouped layout, an E4M3 A) go through kind::mxf8f6f4, see native_fp4_a / native_fp4_b.
static bool is_fp4_pair(const dg_gemm_desc_t& d) {
    return d.a_dtype == DG_E2M1X2 && d.b_dtype == DG_E2M1X2 && d.major_a == DG_MAJOR_K && d.major_b == DG_MAJOR_K &&
           d.gemm_type != DG_GEMM_K_GROUPED_PSUM;
}
// Both operands BF16: kind::f16, no scale factors; strides are in BF16 elements.
static bool is_bf16_pair(const dg_gemm_desc_t& d) { return d.a_dtype == DG_BF16 && d.b_dtype == DG_BF16; }
static uint32_t ab_elem_bytes(const dg_gemm_desc_t& d) { return is_bf16_pair(d) ? 2u : 1u; }
static uint32_t k_bytes(const dg_gemm_desc_t& d) { return is_fp4_pair(d) ? d.k / 2 : d.k * ab_elem_bytes(d); }
static uint32_t sf_atoms(const dg_gemm_desc_t& d) { return is_bf16_pair(d) ? 0u : is_fp4_pair(d) ? 2u : 1u; }
// K elements in one 128-byte stage row
static uint32_t stage_k(const dg_gemm_desc_t& d) { return is_fp4_pair(d) ? 256u : kBlockK / ab_elem_bytes(d); }
// packed E2M1 B next to an E4M3 A is decoded to E4M3 in shared memory
static bool feature_disabled(const char* name);
// Packed E2M1 B next to an E4M3 A. tcgen05.mma kind::mxf8f6f4 reads E2M1 operands itself when shared memory holds
// them as groups of sixteen 4-bit values in 16-byte containers (8 bytes of codes, 8 bytes of padding), and TMA
// expands the packed global bytes into exactly that form (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B): no decoding in
// the kernel, and B crosses HBM and the SM's port at half a byte per element. That tensor-map type wants a 32-byte
// aligned base, strides that are multiples of 32 bytes and a contiguous extent that is a multiple of 128 elements;
// anything else takes the decoder warps (the packed bytes are expanded to E4M3 in shared memory).
static bool tma_can_expand_fp4(const void* base, uint64_t outer_stride, uint64_t group_stride, uint32_t inner_elems) {
    return (reinterpret_cast<uintptr_t>(base) & 31) == 0 && outer_stride % 32 == 0 && group_stride % 32 == 0 && inner_elems % 128 == 0;
}
static bool native_fp4_b(const dg_gemm_desc_t& d) {
    if (d.b_dtype != DG_E2M1X2 || is_fp4_pair(d)) return false;
    if (d.a_dtype == DG_E4M3 && feature_disabled("native_fp4")) return false;      // (an E2M1 A has no decoder to fall back to)
    return tma_can_expand_fp4(d.b, d.outer_stride_b, d.group_stride_b, d.major_b == DG_MAJOR_K ? d.k : d.n);
}
static bool decodes_b(const dg_gemm_desc_t& d) { return d.b_dtype == DG_E2M1X2 && !is_fp4_pair(d) && !native_fp4_b(d); }
// A packed E2M1 A outside the kind::mxf4 path is always expanded by TMA; operands that break the rules of that
// tensor-map type are refused (the caller expands them to E4M3 first: dg_expand_fp4_launch).
static bool unpacks_fp4_a(const dg_gemm_desc_t& d) { return d.a_dtype == DG_E2M1X2 && !is_fp4_pair(d); }

static int validate(const dg_gemm_desc_t& d) {
    DG_CHECK_ARG(d.gemm_type == DG_GEMM_NORMAL || is_grouped(d.gemm_type) ||
                 d.gemm_type == DG_GEMM_K_GROUPED_PSUM || d.gemm_type == DG_GEMM_BATCHED, "Unknown gemm type %d", d.gemm_type);
    if (!is_bf16_pair(d)) {
        DG_CHECK_ARG(d.a_dtype == DG_E4M3 || d.a_dtype == DG_E2M1X2, "Unsupported operand dtypes");
        DG_CHECK_ARG(d.b_dtype == DG_E4M3 || d.b_dtype == DG_E2M1X2, "Unsupported operand dtypes");
        DG_CHECK_ARG(!(d.a_dtype == DG_E2M1X2 && d.b_dtype == DG_E4M3), "Unsupported operand dtypes");
    } else {
        DG_CHECK_ARG(d.epilogue != DG_EPILOGUE_FP8_QUANT, "BF16 matmul has no FP8 output");
    }
    if (d.b_dtype == DG_E2M1X2) {
        DG_CHECK_ARG(d.k % 2 == 0, "packed FP4 needs an even K");
        DG_CHECK_ARG(d.major_b == DG_MAJOR_K || d.n % 2 == 0, "MN-major packed FP4 needs an even N");
    }
    if (d.a_dtype == DG_E2M1X2)
        DG_CHECK_ARG(d.major_a == DG_MAJOR_K || d.m % 2 == 0, "MN-major packed FP4 needs an even M");
    if (unpacks_fp4_a(d)) {
        DG_UNSUPPORTED(!tma_can_expand_fp4(d.a, d.outer_stride_a, d.group_stride_a, d.major_a == DG_MAJOR_K ? d.k : d.m),
                       "A (packed FP4 with an MN-major or k-grouped operand): base and strides must be multiples of 32 bytes and the "
                       "contiguous extent a multiple of 128 elements (expand A to E4M3 otherwise)");
        DG_UNSUPPORTED(decodes_b(d) && d.gemm_type == DG_GEMM_K_GROUPED_PSUM,
                       "B (packed FP4, k-grouped): base and strides must be multiples of 32 bytes and N a multiple of 128 "
                       "(expand B to E4M3 otherwise)");
    }
    if (d.epilogue == DG_EPILOGUE_FP8_QUANT) {
        DG_CHECK_ARG(d.d_dtype == DG_E4M3 && !d.accumulate, "FP8 quantization requires a direct E4M3 output");
        DG_CHECK_ARG(d.n % 128 == 0, "FP8 output requires N to be a multiple of 128");
        DG_CHECK_ARG(d.sfd != nullptr && d.sfd_stride >= d.m, "FP8 quantization needs the scale output tensor");
        DG_CHECK_ARG(aligned16(d.d) && d.outer_stride_d % 16 == 0 && d.group_stride_d % 16 == 0,
                     "FP8 output: base and strides must be multiples of 16 bytes");
    } else {
        DG_CHECK_ARG(d.d_dtype == DG_BF16 || d.d_dtype == DG_F32, "D must be bf16 or fp32");
    }
    DG_CHECK_ARG(d.major_a == DG_MAJOR_K || d.major_a == DG_MAJOR_MN, "bad major_a");
    DG_CHECK_ARG(d.major_b == DG_MAJOR_K || d.major_b == DG_MAJOR_MN, "bad major_b");
    DG_CHECK_ARG(d.m > 0 && d.n > 0 && d.k > 0, "empty problems are handled by the caller (m, n, k must be > 0)");
    DG_CHECK_ARG(d.a && d.b && d.d && (is_bf16_pair(d) || (d.sfa && d.sfb)), "null operand pointer");
    DG_CHECK_ARG(d.epilogue == DG_EPILOGUE_IDENTITY || d.epilogue == DG_EPILOGUE_ALPHA || d.epilogue == DG_EPILOGUE_BIAS ||
                 d.epilogue == DG_EPILOGUE_STOCHASTIC_BF16 || d.epilogue == DG_EPILOGUE_FP8_QUANT, "unknown epilogue");
    DG_CHECK_ARG(d.epilogue != DG_EPILOGUE_STOCHASTIC_BF16 || (d.d_dtype == DG_BF16 && !d.accumulate),
                 "Stochastic rounding requires a direct BF16 output");
    DG_CHECK_ARG(!(d.epilogue == DG_EPILOGUE_BIAS && d.bias == nullptr), "bias epilogue without a bias pointer");
    DG_CHECK_ARG(!(d.epilogue == DG_EPILOGUE_BIAS && d.accumulate), "bias and accumulation cannot be used together");
    if (d.gemm_type == DG_GEMM_K_GROUPED_PSUM) {
        DG_CHECK_ARG(d.grouped_layout != nullptr && d.num_groups > 0, "grouped GEMM needs grouped_layout and num_groups");
        DG_CHECK_ARG(d.major_a == DG_MAJOR_MN && d.major_b == DG_MAJOR_MN, "A and B must be MN-major for the k-grouped layout");
        DG_CHECK_ARG(d.epilogue == DG_EPILOGUE_IDENTITY || d.epilogue == DG_EPILOGUE_STOCHASTIC_BF16,
                     "k-grouped matmul takes no epilogue besides accumulation and stochastic BF16 rounding");
        DG_CHECK_ARG(d.k % 256 == 0, "k-grouped psum layout: total K must be a multiple of the 256 alignment");
        DG_UNSUPPORTED(decodes_b(d), "B (packed FP4, k-grouped): base and strides must be multiples of 32 bytes and N a multiple "
                                     "of 128 (expand B to E4M3 otherwise)");
    } else if (d.gemm_type == DG_GEMM_BATCHED) {
        DG_CHECK_ARG(d.num_groups > 0, "batched GEMM needs num_groups (the batch count)");
        DG_CHECK_ARG(d.epilogue != DG_EPILOGUE_BIAS, "batched matmul doesn't support bias");
    } else if (is_grouped(d.gemm_type)) {
        DG_CHECK_ARG(d.grouped_layout != nullptr && d.num_groups > 0, "grouped GEMM needs grouped_layout and num_groups");
        DG_CHECK_ARG(d.major_a == DG_MAJOR_K, "A must be K-major for m-grouped GEMM");
        DG_CHECK_ARG(!d.accumulate, "grouped matmul doesn't support accumulation");
        DG_CHECK_ARG(d.epilogue != DG_EPILOGUE_BIAS, "grouped matmul doesn't support bias");
    }
    if (d.gemm_type == DG_GEMM_M_GROUPED_PSUM)
        DG_CHECK_ARG(d.m % 256 == 0, "m-grouped psum layout: total rows must be a multiple of the 256-row alignment");

    // What TMA needs from the operands. The caller repacks (dg_pad_rows_launch) when these fail.
    const uint32_t eb = ab_elem_bytes(d);
    DG_UNSUPPORTED(!aligned16(d.a) || (d.outer_stride_a * eb) % 16 != 0 || (d.group_stride_a * eb) % 16 != 0,
                   "A: base and strides must be multiples of 16 bytes");
    DG_UNSUPPORTED(!aligned16(d.b) || (d.outer_stride_b * eb) % 16 != 0 || (d.group_stride_b * eb) % 16 != 0,
                   "B: base and strides must be multiples of 16 bytes");
    if (!is_bf16_pair(d)) {
        DG_UNSUPPORTED(!aligned16(d.sfa) || d.sfa_stride % 8 != 0 || d.sfa_group_stride % 8 != 0,
                       "SFA: base and strides must be multiples of 16 bytes");
        DG_UNSUPPORTED(!aligned16(d.sfb) || d.sfb_stride % 8 != 0 || d.sfb_group_stride % 8 != 0,
                       "SFB: base and strides must be multiples of 16 bytes");
    }
    return DG_OK;
}

// ------------------------------------------------------------------------------------------------
// Heuristic
// ------------------------------------------------------------------------------------------------
// TMEM columns of the scale factors: four per 128 rows of A / of the B tile, per 32-bit word of scales
static uint32_t sf_tmem_cols(uint32_t block_n, uint32_t atoms) { return atoms * (4 + 4 * (sfb_rows(block_n) / 128)); }

static uint32_t tmem_cols_for(uint32_t block_n, uint32_t accum_stages, uint32_t atoms) {
    const uint32_t need = accum_stages * block_n + sf_tmem_cols(block_n, atoms);
    uint32_t cols = 32;
    while (cols < need) cols *= 2;
    return cols;
}

static uint32_t max_stages_for(uint32_t block_n, uint32_t cta_group, bool decode_b, uint32_t store_bufs, uint32_t cluster_split,
                               uint32_t atoms = 1, uint32_t epi_warps = kNumEpilogueWarps) {
    constexpr uint32_t kSmemCap = 227 * 1024;
    uint32_t best = 0;
    for (uint32_t s = 1; s <= kMaxStages; ++s)
        if (make_smem_layout(block_n, s, cta_group, decode_b, store_bufs, cluster_split, atoms, epi_warps).total <= kSmemCap) best = s;
    return best;
}
// Eight epilogue warps (reserved[5] == 2) exist for the FP8 x FP8 kernels with K-major operands
static bool wide_epilogue(const dg_gemm_config_t& c) { return c.reserved[5] == 2; }

// Two ways to split K: partial sums reduced into an FP32 workspace that a second kernel casts (reserved[3] == 0), or
// the splits of one tile form a thread-block cluster and reduce through shared memory (reserved[3] == 1).
// DG_DISABLE=lean,cluster,wide,simple,straight,wide_tile,half_tiles,tma_store,native_fp4 (debugging aid for A/B timing): keeps the
// heuristic away from cluster split-K, from eight epilogue warps, from wide tiles or from half tiles in their last wave,
// from TMA stores (plain stores instead), and / or the launch away from the lean and the cast-and-store-only kernel
// instantiations or from the short chunk loop. Every alternative computes the same values.
static bool feature_disabled(const char* name) {
    static const std::string list = [] { const char* e = getenv("DG_DISABLE"); return std::string(e ? e : ""); }();
    return list.find(name) != std::string::npos;
}
// Wide tiles (block_n in (256, 448]: two accumulators of block_n / 2 columns fed by one A tile per K step) exist for the
// FP8 x FP8, FP4 x FP4 and BF16 kernels with K-major operands; 2 * 224 accumulator columns + 20 (40) scale columns is
// what fits in TMEM (BF16 has no scale columns and goes to 2 * 256).
constexpr uint32_t kMaxWideBlockN = 448;
static uint32_t max_wide_block_n(const dg_gemm_desc_t& d) { return d.a_dtype == DG_BF16 ? 512u : kMaxWideBlockN; }
static bool wide_tile_possible(const dg_gemm_desc_t& d) {
    return ((d.a_dtype == DG_E4M3 && d.b_dtype == DG_E4M3) || (d.a_dtype == DG_E2M1X2 && d.b_dtype == DG_E2M1X2) ||
            (d.a_dtype == DG_BF16 && d.b_dtype == DG_BF16)) &&
           d.major_a == DG_MAJOR_K && d.major_b == DG_MAJOR_K;
}
static bool splits_in_cluster(const dg_gemm_config_t& c) { return c.split_k > 1 && c.reserved[3] != 0; }
static bool splits_in_workspace(const dg_gemm_config_t& c) { return c.split_k > 1 && c.reserved[3] == 0; }
constexpr uint32_t kMaxClusterSplit = 8;        // portable cluster size

// Fill the derived fields of a configuration whose block_n / cta_group / split_k are set.
static int complete_config(const dg_gemm_desc_t& d, dg_gemm_config_t& c) {
    const uint32_t num_sms = effective_num_sms(d);
    c.block_m = kBlockM * c.cta_group;
    c.block_k = kBlockK;
    if (c.split_k > 1) {
        // every split must own at least one K block: settle the split count before anything is derived from it (the
        // reduce buffers of a cluster split grow when the count drops, e.g. 4 -> 3 splits of a 128-column tile)
        const uint32_t nkb_all = ceil_div_u32(k_bytes(d), kBlockK);
        DG_CHECK_ARG(c.split_k <= nkb_all, "split_k larger than the number of K blocks");
        c.split_k = ceil_div_u32(nkb_all, ceil_div_u32(nkb_all, c.split_k));
    }
    if (c.split_k <= 1) c.reserved[3] = 0;
    const bool split = splits_in_workspace(c);
    const bool in_cluster = splits_in_cluster(c);
    const bool tma_ok = split || tma_store_ok(d);
    if (d.epilogue == DG_EPILOGUE_FP8_QUANT) c.epilogue_mode = kEpiFp8Quant;
    else if (split) c.epilogue_mode = kEpiTmaReduce;
    // (a BF16 D that is accumulated into is read, added in FP32 and rounded once: no reduce-add in memory)
    else if (d.accumulate) c.epilogue_mode = d.d_dtype == DG_BF16 ? kEpiPlainStore : (tma_ok ? kEpiTmaReduce : kEpiPlainAtomic);
    else c.epilogue_mode = tma_ok ? kEpiTmaStore : kEpiPlainStore;

    const uint32_t gran = 32u;
    DG_CHECK_ARG(c.cta_group == 1 || c.cta_group == 2, "cta_group must be 1 or 2");
    if (c.block_n > 256) {
        // wide tile: two column halves per K step that share the A operand
        DG_CHECK_ARG(wide_tile_possible(d) && c.cta_group == 2 && !wide_epilogue(c),
                     "block_n > 256 needs E4M3 x E4M3, E2M1 x E2M1 or BF16 x BF16 with K-major operands, cta_group 2 and four epilogue warps");
        DG_CHECK_ARG(c.block_n <= max_wide_block_n(d) && c.block_n % 64 == 0, "a wide block_n must be a multiple of 64 in (256, %u]", max_wide_block_n(d));
        // (the wide-tile walk hands out half tiles by tile index and knows nothing of K splits)
        DG_CHECK_ARG(c.split_k <= 1, "block_n > 256 cannot be combined with split_k > 1");
    } else {
        DG_CHECK_ARG(c.block_n >= gran && c.block_n % gran == 0, "block_n must be a multiple of %u in [%u, 256]", gran, gran);
        DG_CHECK_ARG(c.block_n % (16 * c.cta_group) == 0, "block_n not valid for this cta_group");
    }
    if (d.major_b == DG_MAJOR_MN)      // MN-major B comes in 128-byte atoms along N
        DG_CHECK_ARG((c.block_n / c.cta_group) % (128 / ab_elem_bytes(d)) == 0,
                     "MN-major B needs block_n / cta_group to be a multiple of %u", 128 / ab_elem_bytes(d));
    DG_CHECK_ARG(c.cta_group == 1 || d.gemm_type != DG_GEMM_M_GROUPED_MASKED, "masked grouped GEMM uses cta_group 1");
    DG_CHECK_ARG(!split || d.epilogue != DG_EPILOGUE_FP8_QUANT, "FP8 quantization cannot be combined with split-K");
    DG_CHECK_ARG(c.split_k <= 1 || d.gemm_type == DG_GEMM_NORMAL, "split-K is only available for the dense GEMM");
    DG_CHECK_ARG(!split || d.epilogue != DG_EPILOGUE_STOCHASTIC_BF16, "stochastic rounding cannot be combined with split-K");
    // The workspace reduction adds the partial sums of a tile in arrival order; the cluster reduction adds them in rank order.
    DG_CHECK_ARG(!split || !d.deterministic, "deterministic algorithms: split-K through the workspace adds in arrival order; "
                 "use the cluster reduction (reserved[3] = 1) or split_k = 1");
    DG_CHECK_ARG(!in_cluster || (c.cta_group == 1 && c.split_k <= kMaxClusterSplit && !decodes_b(d)),
                 "cluster split-K needs cta_group 1, unpacked B and at most %u splits", kMaxClusterSplit);
    const uint32_t cluster_split = in_cluster ? c.split_k : 1u;

    const uint32_t atoms = sf_atoms(d);
    // reserved[5]: epilogue warps, 0 = choose, 1 = four, 2 = eight
    const bool wide_possible = d.a_dtype == DG_E4M3 && d.b_dtype == DG_E4M3 && d.major_a == DG_MAJOR_K && d.major_b == DG_MAJOR_K &&
                               !in_cluster;
    DG_CHECK_ARG(c.reserved[5] <= 2 && (c.reserved[5] != 2 || wide_possible),
                 "eight epilogue warps need FP8 x FP8, K-major operands and no cluster split-K");
    const uint32_t nkb_tile = ceil_div_u32(ceil_div_u32(k_bytes(d), kBlockK), c.split_k > 1 ? c.split_k : 1);
    if (c.reserved[5] == 0) {
        // Short K and several tiles per CTA: the epilogue, not the main loop, bounds a tile (4096x32768x512: 124 -> 93 us
        // with eight warps); with longer K the lost pipeline stage costs more than the faster drain gains.
        const uint64_t dense_tiles = (uint64_t)ceil_div_u32(d.m, kBlockM * c.cta_group) * ceil_div_u32(d.n, c.block_n);
        const bool several_tiles = d.gemm_type != DG_GEMM_NORMAL || dense_tiles > num_sms / c.cta_group;
        // A plain BF16 output runs the cast-and-store-only instantiation, whose four warps drain an accumulator as fast
        // as eight do (4096x32768x512: 78 us with four warps, 81 us with eight).
        const bool cast_and_store_only = d.d_dtype == DG_BF16 && !split && d.epilogue == DG_EPILOGUE_IDENTITY &&
                                         c.epilogue_mode <= kEpiTmaReduce && !feature_disabled("simple");
        // (measured on wide tiles too: eight warps gain nothing there and their staging costs a pipeline stage)
        const bool short_k = several_tiles && d.gemm_type != DG_GEMM_K_GROUPED_PSUM && nkb_tile <= 8 && !cast_and_store_only;
        c.reserved[5] = (wide_possible && short_k && c.block_n <= 256 && !feature_disabled("wide")) ? 2u : 1u;
    }
    const uint32_t epi_warps = wide_epilogue(c) ? 2 * kNumEpilogueWarps : kNumEpilogueWarps;
    const uint32_t accum_stages = (2 * c.block_n + sf_tmem_cols(c.block_n, atoms) <= 512) ? 2u : 1u;
    c.tmem_cols = tmem_cols_for(c.block_n, accum_stages, atoms);
    c.reserved[0] = accum_stages;
    const bool decode_b = decodes_b(d);
    const uint32_t nkb = ceil_div_u32(k_bytes(d), kBlockK);
    // Staging boxes per epilogue warp. Measured: more than two never helped (the stores then compete with the operand
    // loads), and the shared memory is worth more as pipeline stages: the main loop is bound by the bytes in flight
    // (4096x7168x16384: 5 -> 6 stages = +9 %), so one box per warp is taken when that buys a stage.
    if (c.reserved[1] == 0) {
        const uint32_t cs = in_cluster ? c.split_k : 1u;
        c.reserved[1] = max_stages_for(c.block_n, c.cta_group, d.b_dtype == DG_E2M1X2 && !is_fp4_pair(d), 1, cs, sf_atoms(d), epi_warps) >
                        max_stages_for(c.block_n, c.cta_group, d.b_dtype == DG_E2M1X2 && !is_fp4_pair(d), 2, cs, sf_atoms(d), epi_warps) ? 1u : 2u;
    }
    DG_CHECK_ARG(c.reserved[1] >= 1 && c.reserved[1] <= kMaxStoreBufs, "store buffers per warp must be 1..4");
    DG_CHECK_ARG(c.reserved[4] <= 64, "raster group must be at most 64 row blocks");
    const uint32_t store_bufs = c.reserved[1];
    uint32_t max_stages = max_stages_for(c.block_n, c.cta_group, decode_b, store_bufs, cluster_split, atoms, epi_warps);
    if (c.num_stages == 0 || c.num_stages > max_stages) c.num_stages = max_stages;
    DG_CHECK_ARG(c.num_stages >= 1, "tile does not fit in shared memory");
    if (c.num_stages > nkb * 4 && c.num_stages > 2) c.num_stages = nkb * 4 > 2 ? nkb * 4 : 2;
    if (c.num_stages > max_stages) c.num_stages = max_stages;
    // cluster split-K stages its outgoing partial sums (16 KB per 32 columns) and its output boxes in the operand ring
    if (in_cluster) {
        const uint32_t ring = c.num_stages * (kBlockM * kBlockK + c.block_n * kBlockK);
        // (outgoing partial sums, the staging boxes of the epilogue warps, and one more box each for the second set of warps
        //  a lean kernel uses)
        const uint32_t need = (c.block_n / 32) * kReduceSlabBytes + kNumEpilogueWarps * (store_bufs + 1) * kStoreBufBytes;
        DG_CHECK_ARG(ring >= need, "cluster split-K needs a pipeline of at least %u bytes, %u stages give %u", need, c.num_stages, ring);
    }
    // one CTA per SM: keep the dynamic shared memory above half of the SM's capacity
    const uint32_t need = make_smem_layout(c.block_n, c.num_stages, c.cta_group, decode_b, store_bufs,
                                           splits_in_cluster(c) ? c.split_k : 1u, atoms, epi_warps).total;
    c.smem_bytes = need < 120u * 1024 ? 120u * 1024 : need;

    uint32_t grid_units;
    const uint32_t max_units = num_sms / c.cta_group;
    if (d.gemm_type == DG_GEMM_NORMAL) {
        const uint64_t tiles = (uint64_t)ceil_div_u32(d.m, c.block_m) * ceil_div_u32(d.n, c.block_n) * c.split_k;
        grid_units = (uint32_t)(tiles < max_units ? tiles : max_units);
        // cluster split-K is not persistent: one tile per CTA, the splits of a tile adjacent in the grid
        if (splits_in_cluster(c)) {
            DG_CHECK_ARG(tiles <= 0x7fffffffull, "too many tiles");
            grid_units = (uint32_t)tiles;
        }
    } else {
        uint64_t bound;   // an upper bound on the tile count; the real count is only known on device
        if (d.gemm_type == DG_GEMM_M_GROUPED_PSUM) bound = (uint64_t)ceil_div_u32(d.m, c.block_m) * ceil_div_u32(d.n, c.block_n);
        else bound = (uint64_t)d.num_groups * ceil_div_u32(d.m, c.block_m) * ceil_div_u32(d.n, c.block_n);   // masked, batched, k-grouped
        grid_units = (uint32_t)(bound < max_units ? bound : max_units);
    }
    if (grid_units == 0) grid_units = 1;
    c.num_ctas = grid_units * c.cta_group;
    if (c.epilogue_mode == kEpiTmaStore && feature_disabled("tma_store")) c.epilogue_mode = kEpiPlainStore;
    // A CTA with a single tile cannot hide its epilogue behind a next tile, and there the TMA store (staging, proxy
    // fence, descriptor fetch) costs more latency than plain 16-byte stores straight from the registers.
    if (c.epilogue_mode == kEpiTmaStore && d.gemm_type == DG_GEMM_NORMAL && c.cta_group == 1 &&
        (uint64_t)ceil_div_u32(d.m, c.block_m) * ceil_div_u32(d.n, c.block_n) * c.split_k <= grid_units)
        c.epilogue_mode = kEpiPlainStore;
    return DG_OK;
}

// Modelled cycles one CTA (or CTA pair) spends on one 128-wide K block of a tile. The tensor pipe needs
// 2 * block_n cycles for 128 x block_n x 128 (16384 FP8 flop per cycle per SM). Operand bytes enter an SM at about
// 50 bytes per cycle (measured: 43-56 B/clk/SM across tilings, the L2-to-SM path), which is what bounds every tiling
// that does not share operands across SMs; a CTA pair halves the B bytes per SM.
static double k_block_cycles(uint32_t cta_group, uint32_t bn, bool packed_b = false, bool decoded = true) {
    const double mma = 2.0 * bn;
    const double ingest = (128.0 + (double)bn / cta_group / (packed_b ? 2 : 1)) * 128.0 / 50.0;
    const double decode = (packed_b && decoded) ? 2.5 * bn / cta_group : 0.0;       // four decoder warps, ~40 instructions per 16 codes
    double t = mma > ingest ? mma : ingest;
    return t > decode ? t : decode;
}

// Modelled cycles of the main loop of one whole tile for problems with many rows (the tensor-bound regime), from
// in-kernel clock reads: everything that crosses the SM's port to L2 (operands, scales, and the tile of D going out)
// moves at about 58 bytes per cycle whatever the tiling, and the tensor pipe needs 2 * block_n cycles per K block.
static double tile_main_cycles(uint32_t cta_group, uint32_t bn, uint32_t k_blocks, uint32_t atoms, uint32_t d_elem_bytes, bool packed_b,
                               bool decoded = true) {
    const double mma = (atoms == 2 ? 1.0 : 2.0) * bn * k_blocks;      // (kind::mxf4 runs a 128-byte K block in half the cycles)
    const double per_kb = (128.0 + (double)bn / cta_group / (packed_b ? 2 : 1)) * 128.0 + (128.0 + sfb_rows(bn)) * 4.0 * atoms;
    // (a wide tile keeps four or five 40-46 KB stages in flight instead of six 32 KB ones and measures nearer 55)
    const double ingest = (per_kb * k_blocks + 128.0 * bn * d_elem_bytes) / (bn > 256 ? 55.0 : 58.0);
    const double decode = (packed_b && decoded) ? 2.5 * bn / cta_group * k_blocks : 0.0;
    double t = mma > ingest ? mma : ingest;
    return t > decode ? t : decode;
}

static int select_config(const dg_gemm_desc_t& d, dg_gemm_config_t& c) {
    memset(&c, 0, sizeof(c));
    const uint32_t num_sms = effective_num_sms(d);
    const bool d_fp32 = d.d_dtype == DG_F32;
    // K blocks one tile runs through (the k-grouped layout splits K over the groups)
    const uint32_t nkb = d.gemm_type == DG_GEMM_K_GROUPED_PSUM ? ceil_div_u32(ceil_div_u32(d.k, d.num_groups), kBlockK)
                                                               : ceil_div_u32(k_bytes(d), kBlockK);
    const uint32_t atoms = sf_atoms(d);
    const bool grouped = is_grouped(d.gemm_type) && d.gemm_type != DG_GEMM_K_GROUPED_PSUM;

    // Rows the problem has (an estimate for the masked layout, whose row counts live on the device).
    uint64_t rows;
    if (d.gemm_type == DG_GEMM_M_GROUPED_MASKED) {
        const uint32_t per_group = d.expected_m ? (d.expected_m < d.m ? d.expected_m : d.m) : d.m;
        rows = (uint64_t)d.num_groups * per_group;
    } else if (d.gemm_type == DG_GEMM_BATCHED || d.gemm_type == DG_GEMM_K_GROUPED_PSUM) {
        rows = (uint64_t)d.num_groups * d.m;
    } else {
        rows = d.m;
    }
    const double hbm_bytes = (double)(d.gemm_type == DG_GEMM_K_GROUPED_PSUM ? d.m : rows) * k_bytes(d) +
                             (double)d.n * k_bytes(d) * (grouped ? d.num_groups : 1) +
                             (double)rows * d.n * elem_size(d.d_dtype);
    const double t_hbm = hbm_bytes / 6400.0;       // ns at 6.4 TB/s

    double best_cost = 1e30;
    uint32_t best_bn = 0, best_split = 1, best_cg = 1;
    for (uint32_t cg = 1; cg <= 2; ++cg) {
        if (cg == 2 && (d.gemm_type == DG_GEMM_M_GROUPED_MASKED || rows <= kBlockM || num_sms < 2 ||
                        ((d.gemm_type == DG_GEMM_BATCHED || d.gemm_type == DG_GEMM_K_GROUPED_PSUM) && d.m <= kBlockM))) continue;
        const uint32_t units = num_sms / cg;
        const uint32_t tile_m = kBlockM * cg;
        uint64_t m_tiles;
        if (has_row_groups(d.gemm_type) || d.gemm_type == DG_GEMM_K_GROUPED_PSUM)
            m_tiles = (uint64_t)d.num_groups * ceil_div_u32((uint32_t)(rows / d.num_groups), tile_m);
        else
            m_tiles = (rows + tile_m - 1) / tile_m;
        for (uint32_t split = 1; split <= 16; ++split) {
            if (split > 1 && (d.gemm_type != DG_GEMM_NORMAL || nkb / split < 2 || cg == 2 || d.deterministic ||
                              d.epilogue == DG_EPILOGUE_STOCHASTIC_BF16 || d.epilogue == DG_EPILOGUE_FP8_QUANT)) break;
            const bool out_fp32 = d_fp32 || split > 1;
            const uint32_t step = d.major_b == DG_MAJOR_MN ? (128u / ab_elem_bytes(d)) * cg : 32u;   // MN-major B comes in 128-byte atoms
            // (single CTAs gain little from a wide tile: A + 2 x B per stage leaves them two or three stages)
            const uint32_t bn_max = (split == 1 && cg == 2 && wide_tile_possible(d) && !feature_disabled("wide_tile")) ? max_wide_block_n(d) : 256u;
            for (uint32_t bn = step; bn <= bn_max; bn += (bn >= 256 ? 64u : step)) {
                if (bn > step && bn - step >= d.n) continue;                 // a narrower legal tile already covers N
                if (bn % (16 * cg) != 0) continue;
                // (packed E2M1 pairs copy twice the scale atoms per K block: only full 224-column halves pay off.
                //  Measured, 4096x4096x7168: 320 columns 71.7 us against 65.6 us with 256; 4096x7168x16384: 448 columns
                //  191 us against 205 us with 224)
                if (bn > 256 && atoms == 2 && bn != kMaxWideBlockN) continue;
                // (BF16: the narrow tiling already runs at 95 % of the cuBLAS figure; measured, a wide tile gains 4 % at
                //  K = 7168 and loses 5 % at K = 2048, where its exposed epilogue weighs more)
                if (bn > 256 && atoms == 0 && nkb < 48) continue;
                const uint32_t n_tiles = ceil_div_u32(d.n, bn);
                const uint64_t tiles = m_tiles * n_tiles * split;
                const uint64_t waves = (tiles + units - 1) / units;
                const uint32_t kb_per = ceil_div_u32(nkb, split);
                const bool single_accum = 2 * bn + sf_tmem_cols(bn, atoms) > 512;
                // (a wide tile has one accumulator: ~290 cycles per 32-column chunk are not hidden behind the next tile)
                const double t_epi = bn > 256 ? bn * 12.0 : bn * (out_fp32 ? 8.0 : 6.0);
                const bool packed_b = d.b_dtype == DG_E2M1X2 && !is_fp4_pair(d);
                double main_loop = rows > kBlockM ? tile_main_cycles(cg, bn, kb_per, atoms, out_fp32 ? 4 : elem_size(d.d_dtype), packed_b, decodes_b(d))
                                                  : kb_per * k_block_cycles(cg, bn, packed_b, decodes_b(d));
                // One tile per CTA and that is all (a few hundred rows): the steady-state figures above do not hold, a K
                // block was never measured under about 520 cycles (256 x 2112 x 7168 as 66 pairs of 32 columns: 18.4 us,
                // as 66 single CTAs of 64 columns: 18.8 us; both modelled at 11-12 us without this floor, so the K splits
                // in a cluster that take 12.2 us lost to them)
                if (rows > kBlockM && waves == 1 && d.gemm_type == DG_GEMM_NORMAL) main_loop = std::max(main_loop, 520.0 * kb_per);
                const double cycles = main_loop + ((single_accum || waves == 1) ? t_epi : 0.0) + 700.0;
                double cost = (double)waves * cycles / 1.8;                   // ns at ~1.8 GHz
                if (cost < t_hbm) cost = t_hbm + 1e-3 * cost;     // HBM-bound: the cheaper schedule still wins ties
                // second kernel (launch gap, FP32 read + zero + write) and the FP32 reduce traffic of the partials
                if (split > 1) cost += 6000.0 + 0.004 * (double)d.m * d.n * split;
                if (cost < best_cost * (1.0 - 1e-9) || (cost <= best_cost * (1.0 + 1e-9) && bn > best_bn)) {
                    best_cost = cost; best_bn = bn; best_split = split; best_cg = cg;
                }
            }
        }
    }
    // Cluster split-K (dense GEMM, single CTAs, unpacked B): the K splits of one tile run as one thread-block cluster
    // and reduce through shared memory, so no second kernel and no FP32 round trip through L2. Modelled cost: the
    // main loop of one split, the exchange (staging, bulk copies, waiting for the slowest rank, summation: measured
    // 5000-7000 cycles, growing with the chunks sent and the cluster size), and a cluster launch that starts ~2.5 us
    // later than a plain one.
    bool best_in_cluster = false;
    if (d.gemm_type == DG_GEMM_NORMAL && !decodes_b(d) && d.major_b == DG_MAJOR_K && !feature_disabled("cluster")) {
        const uint64_t m_tiles = (rows + kBlockM - 1) / kBlockM;
        for (uint32_t split = 2; split <= kMaxClusterSplit && nkb / split >= 2; ++split) {
            for (uint32_t bn = 32; bn <= 256; bn += 32) {
                if (bn > 32 && bn - 32 >= d.n) continue;
                if (max_stages_for(bn, 1, false, 2, split, atoms) < 4) continue;
                // (fewer clusters than SMs / split are resident at once: g_cluster_capacity)
                const uint64_t clusters = m_tiles * ceil_div_u32(d.n, bn);
                const uint64_t resident = std::max<uint64_t>(1, (uint64_t)g_cluster_capacity[split].load() * num_sms / 148);
                const uint64_t waves = (clusters + resident - 1) / resident;
                const uint32_t kb_per = ceil_div_u32(nkb, split);
                // exchange: staging and sending the chunks a rank does not own, the cluster barrier, the summation
                const uint32_t chunks = bn / 32, sent = chunks - chunks / split;
                const double exchange = 3000.0 + 900.0 * sent + 150.0 * split;
                const double cycles = kb_per * k_block_cycles(1, bn) + bn * (d_fp32 ? 8.0 : 6.0) + 700.0 + exchange;
                double cost = (double)waves * cycles / 1.8 + 2500.0;
                if (cost < t_hbm) cost = t_hbm + 1e-3 * cost;
                if (cost < best_cost * (1.0 - 1e-9)) {
                    best_cost = cost; best_bn = bn; best_split = split; best_cg = 1; best_in_cluster = true;
                }
            }
        }
    }
    DG_CHECK_ARG(best_bn != 0, "no legal tiling for this problem");
    c.block_n = best_bn;
    c.split_k = best_split;
    c.cta_group = best_cg;
    c.reserved[3] = best_in_cluster ? 1u : 0u;
    return complete_config(d, c);
}

// ------------------------------------------------------------------------------------------------
// Tensor maps
// ------------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static std::atomic<void*> cached{nullptr};
    void* fn = cached.load();
    if (fn == nullptr) {
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        cached.store(fn);
    }
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

// dims / box innermost first; strides_bytes has rank-1 entries (innermost is contiguous).
static int encode_map(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle, const char* what) {
    auto fn = get_encode_fn();
    if (fn == nullptr) { set_last_error("cuTensorMapEncodeTiled is not available from this driver"); return DG_ERR_CUDA; }
    cuuint64_t gdim[5]; cuuint64_t gstr[4]; cuuint32_t bdim[5]; cuuint32_t estr[5];
    for (uint32_t i = 0; i < rank; ++i) { gdim[i] = dims[i]; bdim[i] = box[i]; estr[i] = 1; }
    for (uint32_t i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    CUresult r = fn(out, dtype, rank, const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed for %s with code %d (dims %llu x %llu x %llu, strides %llu, %llu, box %u x %u x %u)",
                       what, (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)(rank > 2 ? dims[2] : 1),
                       (unsigned long long)strides_bytes[0], (unsigned long long)(rank > 2 ? strides_bytes[1] : 0), box[0], box[1], rank > 2 ? box[2] : 1);
        return DG_ERR_CUDA;
    }
    return DG_OK;
}

static uint64_t nonzero_stride(uint64_t s, uint64_t fallback) { return s ? s : fallback; }

static int build_plan(const dg_gemm_desc_t& d, const dg_gemm_config_t& c, void* workspace, size_t workspace_bytes,
                      bool encode, LaunchPlan& plan) {
    memset(&plan, 0, sizeof(plan));
    GemmKernelArgs& a = plan.args;
    const bool masked = has_row_groups(d.gemm_type);       // A, SFA and D have a group / batch dimension
    const bool grouped = is_grouped(d.gemm_type);
    const bool split = splits_in_workspace(c);
    const uint32_t accum_stages = c.reserved[0];
    const bool k_grouped = d.gemm_type == DG_GEMM_K_GROUPED_PSUM;
    const uint32_t groups = (grouped && !k_grouped) ? d.num_groups : 1;     // group dimension of B / SFB (and A / SFA when `masked`)
    const uint32_t d_groups = (masked || k_grouped) ? d.num_groups : 1;     // group dimension of D

    a.m = d.m; a.n = d.n; a.k = d.k;
    a.block_n = c.block_n;
    a.num_stages = c.num_stages;
    a.num_k_blocks = ceil_div_u32(k_bytes(d), kBlockK);
    a.stage_k = stage_k(d);
    a.num_m_blocks = ceil_div_u32(d.m, c.block_m);
    a.num_n_blocks = ceil_div_u32(d.n, c.block_n);
    a.gemm_type = (uint32_t)d.gemm_type;
    a.num_groups = grouped ? d.num_groups : 1;
    a.grouped_layout = d.grouped_layout;
    a.split_k = c.split_k;
    a.k_blocks_per_split = ceil_div_u32(a.num_k_blocks, c.split_k);
    a.raster_group = c.reserved[4] ? c.reserved[4] : 8;
    while (a.raster_group > 1 && (uint64_t)a.raster_group * a.num_n_blocks >= (1u << 16)) a.raster_group /= 2;
    {
        // the kernel divides tile indices by multiplying with these (fast_div): indices below 2^24, index x divisor below 2^40
        const uint64_t repeats = (grouped && d.gemm_type != DG_GEMM_M_GROUPED_PSUM) ? d.num_groups : 1;
        const uint64_t tile_bound = repeats * (a.num_m_blocks + (grouped ? d.num_groups : 0)) * a.num_n_blocks * c.split_k + c.num_ctas;
        DG_CHECK_ARG(tile_bound < (1u << 24) && (uint64_t)a.raster_group * a.num_n_blocks < (1u << 16),
                     "the problem has too many tiles (%llu)", (unsigned long long)tile_bound);
        const uint32_t last_rows = a.num_m_blocks % a.raster_group;
        a.magic_per_group = fast_div_magic(a.raster_group * a.num_n_blocks);
        a.magic_rows_full = fast_div_magic(a.raster_group);
        a.magic_rows_last = fast_div_magic(last_rows ? last_rows : a.raster_group);
        a.magic_n_blocks = fast_div_magic(a.num_n_blocks);
    }
    a.epilogue_mode = c.epilogue_mode;
    a.d_is_fp32 = (split || d.d_dtype == DG_F32) ? 1u : 0u;
    a.has_alpha = d.epilogue == DG_EPILOGUE_ALPHA ? 1u : 0u;
    a.stochastic = d.epilogue == DG_EPILOGUE_STOCHASTIC_BF16 ? 1u : 0u;
    a.sfd = reinterpret_cast<uint8_t*>(d.sfd);
    a.sfd_stride = d.sfd_stride;
    a.alpha = d.alpha;
    a.has_bias = (d.epilogue == DG_EPILOGUE_BIAS && !split) ? 1u : 0u;
    a.bias = d.bias;
    a.d = d.d;
    a.d_stride = d.outer_stride_d;
    a.d_group_stride = d.group_stride_d;
    a.tmem_cols = c.tmem_cols;
    a.accum_stages = accum_stages;
    a.store_bufs = c.reserved[1];
    a.k_stagger = c.reserved[2];
    a.cluster_split = splits_in_cluster(c) ? c.split_k : 1u;
    plan.cluster_x = c.cta_group > 1 ? c.cta_group : a.cluster_split;
    // Instruction descriptor (block-scaled, kind::mxf8f6f4): E4M3 x E4M3, UE8M0 scales, FP32 accumulate.
    a.idesc = ((uint32_t)d.major_a << 15) | ((uint32_t)d.major_b << 16) | (((c.block_n / tile_halves(c.block_n)) >> 3) << 17) | (1u << 23) |
              (((kBlockM * c.cta_group) >> 4) << 24);
    if (is_fp4_pair(d)) a.idesc |= (1u << 7) | (1u << 10);       // kind::mxf4: both operand formats E2M1
    if (native_fp4_b(d)) a.idesc |= (5u << 10);                  // kind::mxf8f6f4: B format E2M1
    if (unpacks_fp4_a(d)) a.idesc |= (5u << 7);                  // kind::mxf8f6f4: A format E2M1
    a.b_tx_shift = native_fp4_b(d) ? 1u : 0u;
    a.a_tx_shift = unpacks_fp4_a(d) ? 1u : 0u;
    a.add_c_bf16 = (d.accumulate && d.d_dtype == DG_BF16 && !split) ? 1u : 0u;
    if (is_bf16_pair(d))                                         // kind::f16: FP32 accumulator, BF16 operands, no scale fields
        a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)d.major_a << 15) | ((uint32_t)d.major_b << 16) |
                  (((c.block_n / tile_halves(c.block_n)) >> 3) << 17) | (((kBlockM * c.cta_group) >> 4) << 24);

    plan.cta_group = (int)c.cta_group;
    plan.major_a = d.major_a;
    plan.major_b = d.major_b;
    plan.decode_b = decodes_b(d);
    plan.fp4_pair = is_fp4_pair(d);
    plan.bf16_pair = is_bf16_pair(d);
    plan.wide_epi = wide_epilogue(c);
    // (the lean kernel is built for CTAs that have one tile each: once that tile is multiplied its producer, MMA and packer
    //  warps turn into epilogue warps. Plain stores are also what a D that TMA cannot write gets, with any number of tiles)
    const bool one_tile_each = (uint64_t)a.num_m_blocks * a.num_n_blocks * c.split_k <= c.num_ctas;
    plan.lean = d.gemm_type == DG_GEMM_NORMAL && c.cta_group == 1 && !plan.decode_b && c.epilogue_mode == kEpiPlainStore && one_tile_each &&
                (d.epilogue == DG_EPILOGUE_IDENTITY || d.epilogue == DG_EPILOGUE_BIAS) && !plan.fp4_pair && !plan.bf16_pair && !plan.wide_epi &&
                !a.add_c_bf16 && !feature_disabled("lean");
    a.epi_simple = (d.epilogue == DG_EPILOGUE_IDENTITY && !a.has_alpha && !a.has_bias && !a.stochastic &&
                    c.epilogue_mode <= kEpiTmaReduce && !splits_in_cluster(c) && !feature_disabled("straight")) ? 1u : 0u;
    plan.wide_tile = c.block_n > 256;
    {
        // Wide tiles, dense: when the last wave of tiles fills at most half of the CTA pairs, its tiles are handed out
        // as single column halves (two work items per tile), which makes that wave half as long.
        const uint32_t tiles = a.num_m_blocks * a.num_n_blocks, units = c.num_ctas / c.cta_group;
        const uint32_t rem = tiles % units;
        a.half_from = (plan.wide_tile && d.gemm_type == DG_GEMM_NORMAL && c.split_k == 1 && tiles > units && rem > 0 && 2 * rem <= units &&
                       !feature_disabled("half_tiles")) ? tiles - rem : tiles;
    }
    plan.simple_epi = !plan.lean && !plan.decode_b && !plan.fp4_pair && !plan.bf16_pair && d.major_a == DG_MAJOR_K && d.major_b == DG_MAJOR_K &&
                      !a.d_is_fp32 && d.epilogue == DG_EPILOGUE_IDENTITY && !a.has_alpha && !a.has_bias && !a.stochastic &&
                      c.epilogue_mode <= kEpiTmaReduce && !splits_in_cluster(c) && !feature_disabled("simple");
    // k-grouped, no accumulation: D of groups whose K range is empty must read as zero
    plan.zero_empty_groups = k_grouped && !d.accumulate;
    plan.zero_d = d.d;
    plan.zero_row_bytes = (uint64_t)d.n * elem_size(d.d_dtype);
    plan.zero_row_pitch = d.outer_stride_d * elem_size(d.d_dtype);
    plan.zero_group_pitch = nonzero_stride(d.group_stride_d, (uint64_t)d.m * d.outer_stride_d) * elem_size(d.d_dtype);
    plan.num_ctas = c.num_ctas;
    plan.smem_bytes = c.smem_bytes;

    const uint32_t ws_stride = (uint32_t)align_u64(d.n, 4);
    if (split) {
        const size_t need = (size_t)d.m * ws_stride * sizeof(float);
        if (encode && (workspace == nullptr || workspace_bytes < need || !aligned16(workspace))) {
            set_last_error("split-K needs %zu bytes of zeroed, 16-byte aligned workspace", need);
            return DG_ERR_WORKSPACE;
        }
        plan.finalize = true;
        plan.ws = static_cast<float*>(workspace);
        plan.ws_stride = ws_stride;
        plan.final_d = d.d;
        plan.final_d_stride = d.outer_stride_d;
        plan.final_d_is_fp32 = d.d_dtype == DG_F32;
        plan.final_accumulate = d.accumulate ? 1u : 0u;
        plan.final_bias = d.epilogue == DG_EPILOGUE_BIAS ? d.bias : nullptr;
    }
    if (!encode) return DG_OK;

    const uint32_t load_n = c.block_n / tile_halves(c.block_n) / c.cta_group;      // rows of one B box
    const uint64_t k64 = (d.k + 63) / 64;
    const uint64_t rows_a = d.m;      // rows per group for masked, all rows otherwise
    // ---- A
    // Operand maps count in TMA elements: bytes for the 8-bit and packed 4-bit kinds, BF16 elements for BF16. A stage is
    // 128 bytes of K per row; an MN-major tile is fetched as one box per 128-byte atom along MN.
    const uint32_t eb = ab_elem_bytes(d);
    const CUtensorMapDataType ab_type = is_bf16_pair(d) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const uint64_t k_elems = k_bytes(d) / eb;
    const uint32_t box_k = kBlockK / eb, atom_mn = 128 / eb;
    if (unpacks_fp4_a(d)) {
        // packed E2M1 expanded by TMA into 16-byte containers of sixteen codes: dimensions count 4-bit elements, strides bytes
        if (d.major_a == DG_MAJOR_K) {
            const uint64_t gs = nonzero_stride(d.group_stride_a, rows_a * d.outer_stride_a);
            const uint64_t dims[3] = {d.k, rows_a, masked ? groups : 1};
            const uint64_t str[2] = {d.outer_stride_a, gs};
            const uint32_t box[3] = {kBlockK, kBlockM, 1};
            if (int rc = encode_map(&plan.tm_a, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, d.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "A (E2M1)")) return rc;
        } else {
            const uint64_t dims[3] = {rows_a, d.k, masked ? groups : 1};
            const uint64_t str[2] = {d.outer_stride_a, masked ? nonzero_stride(d.group_stride_a, (uint64_t)d.k * d.outer_stride_a)
                                                               : align_u64((uint64_t)d.k * d.outer_stride_a, 32)};
            const uint32_t box[3] = {128, kBlockK, 1};
            if (int rc = encode_map(&plan.tm_a, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, d.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "A (E2M1)")) return rc;
        }
    } else {
        const uint64_t gs = nonzero_stride(d.group_stride_a, rows_a * d.outer_stride_a);
        if (d.major_a == DG_MAJOR_K) {
            const uint64_t dims[3] = {k_elems, rows_a, masked ? groups : 1};
            const uint64_t str[2] = {d.outer_stride_a * eb, gs * eb};
            const uint32_t box[3] = {box_k, kBlockM, 1};
            if (int rc = encode_map(&plan.tm_a, ab_type, 3, d.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "A")) return rc;
        } else {
            const uint64_t dims[3] = {rows_a, k_elems, masked ? groups : 1};
            const uint64_t str[2] = {d.outer_stride_a * eb, masked ? nonzero_stride(d.group_stride_a, (uint64_t)d.k * d.outer_stride_a) * eb
                                                                    : align_u64((uint64_t)d.k * d.outer_stride_a * eb, 16)};
            const uint32_t box[3] = {atom_mn, box_k, 1};
            if (int rc = encode_map(&plan.tm_a, ab_type, 3, d.a, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "A")) return rc;
        }
    }
    // ---- B
    if (plan.decode_b) {
        // packed E2M1, fetched as plain bytes (no swizzle) and decoded in shared memory
        if (d.major_b == DG_MAJOR_K) {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.n * d.outer_stride_b);
            const uint64_t dims[3] = {d.k / 2, d.n, groups};
            const uint64_t str[2] = {d.outer_stride_b, gs};
            const uint32_t box[3] = {kBlockK / 2, load_n, 1};
            if (int rc = encode_map(&plan.tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE, "B (packed FP4)")) return rc;
        } else {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.k * d.outer_stride_b);
            const uint64_t dims[3] = {d.n / 2, d.k, groups};
            const uint64_t str[2] = {d.outer_stride_b, gs};
            const uint32_t box[3] = {load_n / 2, kBlockK, 1};
            if (int rc = encode_map(&plan.tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE, "B (packed FP4)")) return rc;
        }
    } else if (native_fp4_b(d)) {
        // packed E2M1 expanded by TMA into 16-byte containers of sixteen codes: dimensions count 4-bit elements, strides bytes
        if (d.major_b == DG_MAJOR_K) {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.n * d.outer_stride_b);
            const uint64_t dims[3] = {d.k, d.n, groups};
            const uint64_t str[2] = {d.outer_stride_b, gs};
            const uint32_t box[3] = {kBlockK, load_n, 1};
            if (int rc = encode_map(&plan.tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "B (E2M1)")) return rc;
        } else {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.k * d.outer_stride_b);
            const uint64_t dims[3] = {d.n, d.k, groups};
            const uint64_t str[2] = {d.outer_stride_b, gs};
            const uint32_t box[3] = {128, kBlockK, 1};
            if (int rc = encode_map(&plan.tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "B (E2M1)")) return rc;
        }
    } else {
        if (d.major_b == DG_MAJOR_K) {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.n * d.outer_stride_b);
            const uint64_t dims[3] = {k_elems, d.n, groups};
            const uint64_t str[2] = {d.outer_stride_b * eb, gs * eb};
            const uint32_t box[3] = {box_k, load_n, 1};
            if (int rc = encode_map(&plan.tm_b, ab_type, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "B")) return rc;
        } else {
            const uint64_t gs = nonzero_stride(d.group_stride_b, (uint64_t)d.k * d.outer_stride_b);
            const uint64_t dims[3] = {d.n, k_elems, groups};
            const uint64_t str[2] = {d.outer_stride_b * eb, gs * eb};
            const uint32_t box[3] = {atom_mn, box_k, 1};
            if (int rc = encode_map(&plan.tm_b, ab_type, 3, d.b, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "B")) return rc;
        }
    }
    // ---- scale factors: int16 [rows (contiguous), K64, groups]
    if (is_bf16_pair(d)) {
        plan.tm_sfa = plan.tm_a;      // never used by the BF16 kernel, but the parameters must be valid descriptors
        plan.tm_sfb = plan.tm_b;
    } else {
        const uint64_t gs = nonzero_stride(d.sfa_group_stride, k64 * d.sfa_stride);
        const uint64_t dims[3] = {rows_a, k64, masked ? groups : 1};
        const uint64_t str[2] = {d.sfa_stride * 2, gs * 2};
        const uint32_t box[3] = {128, 2 * sf_atoms(d), 1};
        if (int rc = encode_map(&plan.tm_sfa, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.sfa, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE, "SFA")) return rc;
    }
    if (!is_bf16_pair(d)) {
        const uint64_t gs = nonzero_stride(d.sfb_group_stride, k64 * d.sfb_stride);
        const uint64_t dims[3] = {d.n, k64, groups};
        const uint64_t str[2] = {d.sfb_stride * 2, gs * 2};
        const uint32_t box[3] = {sfb_rows(c.block_n) / tile_halves(c.block_n), 2 * sf_atoms(d), 1};
        if (int rc = encode_map(&plan.tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, d.sfb, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE, "SFB")) return rc;
    }
    // ---- D (or the split-K workspace)
    if (c.epilogue_mode <= kEpiTmaReduce) {
        if (split) {
            const uint64_t dims[3] = {d.n, d.m, 1};
            const uint64_t str[2] = {(uint64_t)ws_stride * 4, align_u64((uint64_t)d.m * ws_stride * 4, 16)};
            const uint32_t box[3] = {32, kStoreBoxRows, 1};
            if (int rc = encode_map(&plan.tm_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, workspace, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "workspace")) return rc;
        } else {
            const uint32_t es = elem_size(d.d_dtype);
            const uint64_t gs = nonzero_stride(d.group_stride_d, (uint64_t)d.m * d.outer_stride_d);
            const uint64_t dims[3] = {d.n, d.m, d_groups};
            const uint64_t str[2] = {d.outer_stride_d * es, align_u64(gs * es, 16)};
            const uint32_t box[3] = {es == 4 ? 32u : 64u, kStoreBoxRows, 1};
            if (int rc = encode_map(&plan.tm_d, es == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                                    d.d, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, "D")) return rc;
            plan.tm_d_tail = plan.tm_d;
            if (es == 2) {
                // half-width box for the last 32 columns of a tile whose block_n is an odd multiple of 32
                const uint32_t tail_box[3] = {32u, kStoreBoxRows, 1};
                if (int rc = encode_map(&plan.tm_d_tail, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d.d, dims, str, tail_box,
                                        CU_TENSOR_MAP_SWIZZLE_64B, "D tail")) return rc;
            }
        }
        if (split) plan.tm_d_tail = plan.tm_d;
    } else {
        plan.tm_d = plan.tm_a;    // unused by the plain-store epilogue, but must be a valid descriptor
        plan.tm_d_tail = plan.tm_a;
    }
    return DG_OK;
}

static void maybe_print_config(const dg_gemm_desc_t& d, const dg_gemm_config_t& c) {
    // One line per launch when DG_PRINT_CONFIGS is set (csrc/jit_kernels/heuristics.hpp:749-753).
    static const bool enabled = [] { const char* e = getenv("DG_PRINT_CONFIGS"); return e && atoi(e) != 0; }();
    if (!enabled) return;
    fprintf(stderr, "[dg_b200] type=%d m=%u n=%u k=%u majors=%d%d d=%s acc=%d groups=%u -> block=%ux%ux%u stages=%u cta_group=%u "
            "split_k=%u%s ctas=%u tmem=%u smem=%u epilogue=%u\n",
            d.gemm_type, d.m, d.n, d.k, d.major_a, d.major_b, d.d_dtype == DG_F32 ? "f32" : "bf16", d.accumulate, d.num_groups,
            c.block_m, c.block_n, c.block_k, c.num_stages, c.cta_group, c.split_k, splits_in_cluster(c) ? " (cluster)" : "", c.num_ctas, c.tmem_cols, c.smem_bytes, c.epilogue_mode);
}

static int resolve_config(const dg_gemm_desc_t& d, const dg_gemm_config_t* in, dg_gemm_config_t& out) {
    if (in == nullptr) return select_config(d, out);
    out = *in;
    if (out.cta_group == 0) out.cta_group = 1;
    if (out.split_k == 0) out.split_k = 1;
    return complete_config(d, out);
}

// ------------------------------------------------------------------------------------------------
// Launch-plan cache
// ------------------------------------------------------------------------------------------------
// The reference re-runs its tiling search on every call and notes that as a gap (csrc/jit_kernels/heuristics.hpp:593).
// Here everything the host derives from a call (validated problem, tiling, the six encoded tensor maps, kernel
// arguments) is a pure function of the descriptor, the optional configuration, the workspace, the device and the
// SM limit, so a repeated call (a decode loop over the same buffers) finds its plan by comparing those bytes.
struct PlanKey {
    dg_gemm_desc_t d;
    dg_gemm_config_t c;
    const void* workspace;
    size_t workspace_bytes;
    int32_t has_config, device, num_sms, pad;
};
struct PlanSlot {
    bool used = false;
    uint64_t hash = 0;
    PlanKey key;
    LaunchPlan plan;
    dg_gemm_config_t cfg;
};
constexpr uint32_t kPlanSlots = 256;
static std::mutex g_plan_mu;
static PlanSlot* g_plan_slots = nullptr;       // allocated on first use, lives until process exit
static std::atomic<unsigned long long> g_plan_hits{0}, g_plan_misses{0};

static uint64_t hash_bytes(const void* p, size_t n) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}

static void make_plan_key(PlanKey& key, const dg_gemm_desc_t& d, const dg_gemm_config_t* c, const void* ws, size_t ws_bytes, int dev) {
    memset(&key, 0, sizeof(key));
    key.d = d;
    if (c != nullptr) { key.c = *c; key.has_config = 1; }
    key.workspace = ws;
    key.workspace_bytes = ws_bytes;
    key.device = dev;
    key.num_sms = g_num_sms.load();
}

static bool plan_cache_find(const PlanKey& key, uint64_t hash, LaunchPlan& plan, dg_gemm_config_t& cfg) {
    std::lock_guard<std::mutex> lock(g_plan_mu);
    if (g_plan_slots == nullptr) return false;
    const PlanSlot& slot = g_plan_slots[hash % kPlanSlots];
    if (!slot.used || slot.hash != hash || memcmp(&slot.key, &key, sizeof(key)) != 0) return false;
    plan = slot.plan;
    cfg = slot.cfg;
    return true;
}

static void plan_cache_store(const PlanKey& key, uint64_t hash, const LaunchPlan& plan, const dg_gemm_config_t& cfg) {
    std::lock_guard<std::mutex> lock(g_plan_mu);
    if (g_plan_slots == nullptr) g_plan_slots = new PlanSlot[kPlanSlots];
    PlanSlot& slot = g_plan_slots[hash % kPlanSlots];
    slot.used = true;
    slot.hash = hash;
    slot.key = key;
    slot.plan = plan;
    slot.cfg = cfg;
}

// ------------------------------------------------------------------------------------------------
// Fixed split-K scratch for callers that cannot allocate (dg_gemm_launch_static_scratch)
// ------------------------------------------------------------------------------------------------
// Lives in every GPU's memory from module load to process exit. In host code the name below is only a handle for
// cudaGetSymbolAddress: it is not a device address and must never be handed to a kernel or a memset directly.
static __device__ __align__(256) float g_static_scratch[DG_STATIC_SCRATCH_BYTES / sizeof(float)];

// Device address of the array on the current device, looked up once per device.
static int static_scratch_address(float** out) {
    static std::mutex mu;
    static float* addresses[64] = {};
    int dev = 0;
    DG_CHECK_CUDA(cudaGetDevice(&dev));
    DG_CHECK_ARG(dev >= 0 && dev < 64, "device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (addresses[dev] == nullptr) {
        float* ptr = nullptr;
        DG_CHECK_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        DG_CHECK_ARG(ptr != nullptr, "cudaGetSymbolAddress returned a null scratch address");
        addresses[dev] = ptr;
    }
    *out = addresses[dev];
    return DG_OK;
}

}  // namespace dg

using namespace dg;

extern "C" {

int dg_gemm_launch_static_scratch(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config, void* stream) {
    DG_CHECK_ARG(desc != nullptr, "dg_gemm_launch_static_scratch: null descriptor");
    if (int rc = validate(*desc)) return rc;
    dg_gemm_config_t c;
    if (int rc = resolve_config(*desc, config, c)) return rc;
    float* scratch = nullptr;
    size_t need = 0;
    if (splits_in_workspace(c)) {
        need = (size_t)desc->m * align_u64(desc->n, 4) * sizeof(float);
        if (need > DG_STATIC_SCRATCH_BYTES) {
            set_last_error("split-K scratch of %zu bytes (m=%u, n=%u) exceeds the built-in %u bytes: pass a config with "
                           "split_k = 1 or call dg_gemm_launch with a workspace", need, desc->m, desc->n,
                           (unsigned)DG_STATIC_SCRATCH_BYTES);
            return DG_ERR_WORKSPACE;
        }
        if (int rc = static_scratch_address(&scratch)) return rc;
        // The array keeps the previous call's contents; the reduction must start from zero.
        DG_CHECK_CUDA(cudaMemsetAsync(scratch, 0, need, static_cast<cudaStream_t>(stream)));
    }
    LaunchPlan plan;
    if (int rc = build_plan(*desc, c, scratch, need, /*encode=*/true, plan)) return rc;
    maybe_print_config(*desc, c);
    return launch_gemm_kernel(plan, static_cast<cudaStream_t>(stream));
}

const char* dg_last_error(void) { return tls_error; }
int dg_abi_version(void) { return DG_B200_ABI_VERSION; }
uint64_t dg_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int dg_get_num_sms(void) { return g_num_sms.load() > 0 ? g_num_sms.load() : device_sm_count(); }
int dg_set_num_sms(int num_sms) {
    DG_CHECK_ARG(num_sms >= 0 && num_sms <= 1024, "num_sms out of range");
    g_num_sms.store(num_sms);
    return DG_OK;
}
int dg_get_mk_alignment_for_contiguous_layout(void) { return 256; }

int dg_select_config(const dg_gemm_desc_t* desc, dg_gemm_config_t* out) {
    DG_CHECK_ARG(desc != nullptr && out != nullptr, "dg_select_config: null argument");
    if (int rc = validate(*desc)) return rc;
    return select_config(*desc, *out);
}

size_t dg_gemm_workspace_bytes(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config) {
    if (desc == nullptr) return 0;
    dg_gemm_config_t c;
    if (validate(*desc) != DG_OK || resolve_config(*desc, config, c) != DG_OK) return 0;
    if (!splits_in_workspace(c)) return 0;
    return (size_t)desc->m * align_u64(desc->n, 4) * sizeof(float);
}

int dg_gemm_dry_run(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config) {
    DG_CHECK_ARG(desc != nullptr, "dg_gemm_dry_run: null descriptor");
    if (int rc = validate(*desc)) return rc;
    dg_gemm_config_t c;
    if (int rc = resolve_config(*desc, config, c)) return rc;
    LaunchPlan plan;
    if (int rc = build_plan(*desc, c, nullptr, 0, /*encode=*/false, plan)) return rc;
    maybe_print_config(*desc, c);
    return DG_OK;
}

int dg_gemm_launch(const dg_gemm_desc_t* desc, const dg_gemm_config_t* config,
                   void* workspace, size_t workspace_bytes, void* stream) {
    DG_CHECK_ARG(desc != nullptr, "dg_gemm_launch: null descriptor");
    int dev = 0;
    DG_CHECK_CUDA(cudaGetDevice(&dev));
    PlanKey key;
    make_plan_key(key, *desc, config, workspace, workspace_bytes, dev);
    const uint64_t hash = hash_bytes(&key, sizeof(key));
    LaunchPlan plan;
    dg_gemm_config_t c;
    if (plan_cache_find(key, hash, plan, c)) {
        g_plan_hits.fetch_add(1, std::memory_order_relaxed);
    } else {
        g_plan_misses.fetch_add(1, std::memory_order_relaxed);
        refresh_cluster_capacity();
        if (int rc = validate(*desc)) return rc;
        if (int rc = resolve_config(*desc, config, c)) return rc;
        if (int rc = build_plan(*desc, c, workspace, workspace_bytes, /*encode=*/true, plan)) return rc;
        plan_cache_store(key, hash, plan, c);
    }
    maybe_print_config(*desc, c);
    return launch_gemm_kernel(plan, static_cast<cudaStream_t>(stream));
}

int dg_fp4_expansion_needed(const dg_gemm_desc_t* desc, int* expand_a, int* expand_b) {
    DG_CHECK_ARG(desc != nullptr && expand_a != nullptr && expand_b != nullptr, "dg_fp4_expansion_needed: null argument");
    const dg_gemm_desc_t& d = *desc;
    *expand_b = (decodes_b(d) && d.gemm_type == DG_GEMM_K_GROUPED_PSUM) ? 1 : 0;
    // (an expanded B is E4M3, and a packed A next to an E4M3 B is not a supported pair: A follows)
    *expand_a = (unpacks_fp4_a(d) && (*expand_b || !tma_can_expand_fp4(d.a, d.outer_stride_a, d.group_stride_a,
                                                                        d.major_a == DG_MAJOR_K ? d.k : d.m))) ? 1 : 0;
    return DG_OK;
}

uint32_t dg_resident_clusters(uint32_t cluster_size) {
    return cluster_size >= 1 && cluster_size <= 8 ? g_cluster_capacity[cluster_size].load() : 0u;
}

void dg_plan_cache_stats(uint64_t* hits, uint64_t* misses) {
    if (hits) *hits = g_plan_hits.load(std::memory_order_relaxed);
    if (misses) *misses = g_plan_misses.load(std::memory_order_relaxed);
}

}  // extern "C"
