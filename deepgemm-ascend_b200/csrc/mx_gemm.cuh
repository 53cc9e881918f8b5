// Block-scaled FP8 / FP8xFP4 GEMM for sm_100a: D = A * B^T with one UE8M0 scale per row per 32 K.
//
// Replaces the device kernels of the reference, deep_gemm/include/deep_gemm/fp8_gemm.hpp:36-287
// (fp8_gemm_impl) and fp8_dequant_gemm.hpp:113-443 (fp8_dequant_gemm_impl), the tile scheduler
// scheduler.hpp:42-249 and the epilogue epilogue.hpp:15-142 + epilogue/operators.hpp:119-221.
//
// One persistent CTA per SM (or one CTA pair per two SMs), 256 threads, warp-specialised:
//   warp 0      TMA producer: A, B tiles (128B-swizzled) and the two scale-factor slabs per K block
//   warp 1      MMA issuer: tcgen05.cp of the scales into TMEM, then 4 x tcgen05.mma (K = 32 each)
//   warp 2      scale-factor packer: int16-pair columns -> the 32x16B atom tcgen05.cp expects;
//               also owns TMEM allocation
//   warp 3      FP4 -> E4M3 decoder helper (mixed FP8xFP4 with MN-major packed B), idle otherwise
//   warps 4..7  epilogue: tcgen05.ld, alpha / bias, cast, swizzled smem staging, TMA store or
//               TMA reduce-add (accumulate, split-K), or bounds-checked plain stores / atomics
// The accumulator is double-buffered in TMEM so that the epilogue of tile i overlaps the main loop
// of tile i+1. Every wait is bounded: a wait that gives up records a code in the device status word,
// raises the CTA's abort flag and lets all roles drain and free TMEM.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>
#include <type_traits>

#include "ptx.cuh"

namespace dg {

constexpr uint32_t kBlockM = 128;        // rows of A per CTA
constexpr uint32_t kBlockK = 128;        // K elements (bytes of FP8) per pipeline stage
constexpr uint32_t kUmmaK = 32;          // K per tcgen05.mma for 8-bit operands
constexpr uint32_t kNumThreads = 256;
constexpr uint32_t kNumDecodeWarps = 4;                    // extra warps 8..11 when B is packed FP4
constexpr uint32_t kNumThreadsDecode = kNumThreads + kNumDecodeWarps * 32;
constexpr uint32_t kNumEpilogueWarps = 4;
constexpr uint32_t kStoreBoxRows = 32;   // each epilogue warp stores its own 32 rows
constexpr uint32_t kStoreBufBytes = kStoreBoxRows * 128;  // one 128B-swizzled box
constexpr uint32_t kMaxStoreBufs = 4;    // staging boxes per epilogue warp (2..4, chosen per problem)
constexpr uint32_t kMaxStages = 12;
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;  // 2 s

enum GemmTypeDev : uint32_t { kNormal = 0, kMGroupedPsum = 1, kKGroupedPsum = 2, kBatched = 3, kMGroupedMasked = 4 };
enum EpilogueMode : uint32_t { kEpiTmaStore = 0, kEpiTmaReduce = 1, kEpiPlainStore = 2, kEpiPlainAtomic = 3, kEpiFp8Quant = 4 };
enum StatusCode : int32_t {
    kStatusOk = 0,
    kStatusTimeoutProducer = 101, kStatusTimeoutPacker = 102, kStatusTimeoutMma = 103,
    kStatusTimeoutEpilogue = 104, kStatusTimeoutDrain = 105, kStatusTimeoutDecoder = 106, kStatusTimeoutReduce = 107,
};

struct GemmKernelArgs {
    uint32_t m, n, k;                 // m: rows of D (normal), total rows (psum), max_m (masked)
    uint32_t block_n;                 // multiple of 32, <= 256
    uint32_t num_stages;
    uint32_t num_k_blocks;            // K blocks of 128 bytes per row
    uint32_t stage_k;                 // K elements in one block: 128 (FP8), 256 (packed FP4 pair), 64 (BF16)
    uint32_t num_m_blocks, num_n_blocks;
    uint32_t gemm_type;
    uint32_t num_groups;
    const int32_t* grouped_layout;    // psum[G] or masked_m[G]
    uint32_t split_k, k_blocks_per_split;
    uint32_t raster_group;            // m-blocks per rasterisation group (L2 reuse of B)
    // floor(2^40 / d) + 1 for the three divisors of the tile walk (see fast_div): m-blocks x n-blocks of a raster
    // group, m-blocks of a full and of the last raster group, n-blocks
    uint64_t magic_per_group, magic_rows_full, magic_rows_last, magic_n_blocks;
    uint32_t epilogue_mode;
    uint32_t d_is_fp32;
    uint32_t half_from;   // wide tiles, dense: tiles from this index on (the last, partial wave) run as two half tiles
    uint32_t epi_simple;  // nothing but cast (or FP32) + staged TMA store / reduce: the epilogue takes its short loop
    uint32_t has_bias, has_alpha;
    uint32_t stochastic;              // BF16 output is rounded stochastically instead of to nearest
    uint8_t* sfd;                     // FP8-quantised output: UE8M0 scale bytes, two per int16 element
    uint64_t sfd_stride;              // int16 elements between consecutive 64-column groups
    float alpha;
    const void* bias;
    void* d;                          // plain-store modes only
    uint64_t d_stride, d_group_stride;  // elements
    uint32_t idesc;                   // tcgen05 instruction descriptor without the scale ids
    uint32_t tmem_cols, accum_stages;
    uint32_t store_bufs;              // staging boxes per epilogue warp
    uint32_t cluster_split;           // 1, or the K splits of one tile run as one cluster and reduce through shared memory
    uint32_t k_stagger;               // dense GEMM: tile with column index nb starts its K loop at block (nb * k_stagger) % len
    uint32_t b_tx_shift;              // 1 when TMA expands packed E2M1 rows of B into 16-byte containers: the barrier then
                                      // counts the packed bytes it read (half of what lands in shared memory), else 0
    uint32_t a_tx_shift;              // the same for a packed E2M1 A
    uint32_t add_c_bf16;              // BF16 D accumulated into: the epilogue reads D, adds in FP32 and rounds once
    int32_t* status;
    unsigned long long* trace;        // debugging aid: per-CTA timestamps (8 slots each), or nullptr
};

// ------------------------------------------------------------------------------------------------
// Bounded waits
// ------------------------------------------------------------------------------------------------
struct AbortFlag {
    volatile uint32_t* flag;   // shared memory
    int32_t* status;           // global memory
    __device__ __forceinline__ bool raised() const { return *flag != 0; }
    __device__ __forceinline__ void raise(int32_t code) const {
        *flag = 1;
        atomicCAS(status, 0, code);
    }
};

// Returns false when the wait gave up or the CTA is aborting.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, const AbortFlag& ab, int32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xff) == 0) {
            if (ab.raised()) return false;
            if (global_timer_ns() - t0 > kWaitTimeoutNs) { ab.raise(code); return false; }
        }
    }
    return true;
}
__device__ __forceinline__ bool wait_barrier_cluster(uint32_t bar, uint32_t parity, const AbortFlag& ab, int32_t code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 0xff) == 0) {
            if (ab.raised()) return false;
            if (global_timer_ns() - t0 > kWaitTimeoutNs) { ab.raise(code); return false; }
        }
    }
    return true;
}

// Slot meanings: 0 kernel entry (globaltimer ns), 1..7 clock64 at: entry, set-up done, first stage about to be
// requested, first operands landed (MMA side), last MMA committed, first accumulator ready (epilogue side), epilogue
// done; 8..12 producer: role entered, first tile known, first stage free, A and B requested, first stage requested;
// 13..15 epilogue: partial sums sent (cluster split-K), partial sums received, all chunks of the first tile written.
// 16, 17: globaltimer ns when the wait for the preceding kernel returned and at the end of the kernel; 18: clock64 at the end.
constexpr uint32_t kTraceSlots = 32;         // 8-byte slots per CTA
__device__ __forceinline__ void trace_mark(const GemmKernelArgs& p, uint32_t slot) {
    if (p.trace != nullptr)
        p.trace[blockIdx.x * kTraceSlots + slot] = (slot == 0 || slot == 16 || slot == 17) ? global_timer_ns() : (unsigned long long)clock64();
}

// ------------------------------------------------------------------------------------------------
// Tile scheduler (every role runs its own copy; the sequence is a pure function of the arguments)
// ------------------------------------------------------------------------------------------------
struct Tile {
    uint32_t row0;        // first row of this CTA in A / SFA / D (within the group for masked)
    uint32_t row_z;       // third TMA coordinate of A / SFA (group for masked / batched, else 0)
    uint32_t d_z;         // third TMA coordinate of D (as row_z, but the group for the K-grouped layout)
    uint32_t halves;      // wide tiles: bit h set = column half h of the tile is computed (3 = the whole tile)
    uint32_t n0;          // first column of D == first row of B
    uint32_t b_z;         // third TMA coordinate of B / SFB (group)
    uint32_t kb_begin, kb_end;
    uint32_t kb_rot;      // the loads walk the K blocks rotated by this much (CTAs that share A then read different lines)
};

// Every role walks the tile sequence on its own, once per tile, and that walk sits on the critical path between two
// tiles (the MMA thread between the last MMA of a tile and the first of the next, the epilogue warps between two
// accumulators), so the divisions by run-time constants are multiplications by host-made reciprocals:
// n / d == (n * (floor(2^40 / d) + 1)) >> 40, exact for n < 2^24 and n * d < 2^40 (checked on the host).
__host__ __device__ __forceinline__ uint64_t fast_div_magic(uint32_t d) { return (1ull << 40) / d + 1; }
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint64_t magic) { return (uint32_t)(((uint64_t)n * magic) >> 40); }

// kLean: dense GEMM only (the other layouts are compiled out).
template <int kCtaGroup, bool kLean = false, bool kWideTile = false>
struct Scheduler {
    const GemmKernelArgs& p;
    uint32_t tile, stride;
    uint32_t cur_group = 0, cur_first = 0, cur_blocks = 0, cur_row0 = 0;
    bool group_loaded = false;

    __device__ Scheduler(const GemmKernelArgs& args) : p(args) {
        tile = blockIdx.x / kCtaGroup;
        stride = gridDim.x / kCtaGroup;
    }

    // m-blocks are counted in units of (128 * kCtaGroup) rows.
    uint32_t cur_kb_begin = 0, cur_kb_end = 0;

    __device__ __forceinline__ void load_group() {
        if (p.gemm_type == kKGroupedPsum) {
            // scheduler.hpp:163-180: group g owns the K range [align(psum[g-1],256), psum[g]); every group spans the
            // whole M x N grid, an empty group has no tiles (its D is zeroed by a separate kernel).
            const uint32_t start = cur_group == 0 ? 0u : ((uint32_t)__ldg(p.grouped_layout + cur_group - 1) + 255u) / 256u * 256u;
            const uint32_t end = (uint32_t)__ldg(p.grouped_layout + cur_group);
            cur_row0 = 0;
            cur_kb_begin = start / p.stage_k;
            cur_kb_end = end > start ? (end + p.stage_k - 1) / p.stage_k : cur_kb_begin;
            cur_blocks = end > start ? p.num_m_blocks : 0u;
        } else if (p.gemm_type == kMGroupedPsum) {
            // scheduler.hpp:147-162: group g owns rows [align(psum[g-1],256), psum[g]) and the
            // kernel computes whole 256-row blocks of it.
            const uint32_t start = cur_group == 0 ? 0u : ((uint32_t)__ldg(p.grouped_layout + cur_group - 1) + 255u) / 256u * 256u;
            const uint32_t end = (uint32_t)__ldg(p.grouped_layout + cur_group);
            const uint32_t rows = end > start ? end - start : 0u;
            cur_row0 = start;
            cur_blocks = (rows + 255u) / 256u * (256u / (kBlockM * kCtaGroup));
        } else {
            // masked: the group's valid row count comes from the device array; batched: every row is valid
            const uint32_t rows = p.gemm_type == kBatched ? p.m : min((uint32_t)max(__ldg(p.grouped_layout + cur_group), 0), p.m);
            cur_row0 = 0;
            cur_blocks = (rows + kBlockM * kCtaGroup - 1) / (kBlockM * kCtaGroup);
        }
        group_loaded = true;
    }

    __device__ bool next(Tile& t) {
        const uint32_t rank = kCtaGroup == 2 ? (blockIdx.x & 1u) : 0u;
        if constexpr (kWideTile) t.halves = 3u;
        if (kLean || p.gemm_type == kNormal) {
            const uint32_t total = p.num_m_blocks * p.num_n_blocks * p.split_k;
            uint32_t ks = 0, mn = tile;
            if constexpr (kWideTile) {
                // The tiles of the last, partial wave are handed out as single column halves, two indices per tile, so
                // that twice as many CTA pairs share that wave and it takes half as long.
                if (tile >= total + (total - p.half_from)) return false;
                if (tile >= p.half_from) {
                    t.halves = 1u << ((tile - p.half_from) & 1u);
                    mn = p.half_from + ((tile - p.half_from) >> 1);
                }
            } else {
                if (tile >= total) return false;
            }
            if (p.split_k > 1) { mn = tile / p.split_k; ks = tile - mn * p.split_k; }
            const uint32_t per_group = p.raster_group * p.num_n_blocks;
            const uint32_t gi = fast_div(mn, p.magic_per_group), in_group = mn - gi * per_group;
            const uint32_t first_m = gi * p.raster_group;
            const bool full = first_m + p.raster_group <= p.num_m_blocks;
            const uint32_t rows = full ? p.raster_group : p.num_m_blocks - first_m;
            const uint32_t nb = fast_div(in_group, full ? p.magic_rows_full : p.magic_rows_last);
            const uint32_t mb = first_m + in_group - nb * rows;
            t.row0 = (mb * kCtaGroup + rank) * kBlockM;
            t.row_z = 0;
            t.d_z = 0;
            t.n0 = nb * p.block_n;
            t.b_z = 0;
            t.kb_begin = ks * p.k_blocks_per_split;
            t.kb_end = min(t.kb_begin + p.k_blocks_per_split, p.num_k_blocks);
            t.kb_rot = p.k_stagger ? (nb * p.k_stagger) % (t.kb_end - t.kb_begin) : 0u;
        } else if constexpr (!kLean) {
            const uint32_t mb_lin = fast_div(tile, p.magic_n_blocks), nb = tile - mb_lin * p.num_n_blocks;
            while (true) {
                if (cur_group >= p.num_groups) return false;
                if (!group_loaded) load_group();
                if (mb_lin < cur_first + cur_blocks) break;
                cur_first += cur_blocks;
                cur_group += 1;
                group_loaded = false;
            }
            const uint32_t mb = mb_lin - cur_first;
            t.row0 = cur_row0 + (mb * kCtaGroup + rank) * kBlockM;
            const bool flat_rows = p.gemm_type == kMGroupedPsum || p.gemm_type == kKGroupedPsum;
            t.row_z = flat_rows ? 0u : cur_group;
            t.d_z = p.gemm_type == kMGroupedPsum ? 0u : cur_group;
            t.n0 = nb * p.block_n;
            t.b_z = p.gemm_type == kKGroupedPsum ? 0u : cur_group;
            t.kb_begin = p.gemm_type == kKGroupedPsum ? cur_kb_begin : 0u;
            t.kb_end = p.gemm_type == kKGroupedPsum ? cur_kb_end : p.num_k_blocks;
            t.kb_rot = 0;
        }
        tile += stride;
        return true;
    }
};

// ------------------------------------------------------------------------------------------------
// Descriptors
// ------------------------------------------------------------------------------------------------
// K-major operand tile, 128-byte rows, 128B swizzle: 8-row groups are 1024 B apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;                    // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
    d |= (uint64_t)1 << 46;                    // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}
// MN-major operand tile: [mn atoms of 128 B][block_k rows][128 B], 128B swizzle over 8 K rows.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t atom_stride_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)((atom_stride_bytes >> 4) & 0x3fff) << 16;   // leading: next 128-B atom along MN
    d |= (uint64_t)(1024 >> 4) << 32;                           // stride: next 8 rows along K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 B, no swizzle, 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// A tile wider than 256 columns is computed as two halves of block_n / 2 columns (two MMAs per K step that share the
// A operand): each half has its own rows of B and its own scale-factor slabs.
__host__ __device__ __forceinline__ uint32_t tile_halves(uint32_t block_n) { return block_n > 256u ? 2u : 1u; }
__host__ __device__ __forceinline__ uint32_t sfb_rows(uint32_t block_n) {
    const uint32_t h = tile_halves(block_n);
    return (block_n / h + 127u) / 128u * 128u * h;
}

// Shared-memory carve-up, computed identically on host and device.
struct SmemLayout {
    uint32_t store_bufs, a, b, b_raw, sf_raw_a, sf_raw_b, sf_pack_a, sf_pack_b, reduce, barriers, total;
    uint32_t a_stage, b_stage, b_raw_stage, sfa_stage, sfb_stage;
};
// Cluster split-K: 32-column chunk c of the tile is finalised by cluster rank c % S, which receives the other ranks'
// partial sums of that chunk as [128 rows][32 floats] slabs: slab index (c / S) * (S - 1) + sender.
constexpr uint32_t kReduceSlabBytes = kBlockM * 32 * 4;
__host__ __device__ __forceinline__ uint32_t cluster_reduce_bytes(uint32_t block_n, uint32_t cluster_split) {
    if (cluster_split <= 1) return 0;
    const uint32_t chunks = block_n / 32;
    return (chunks + cluster_split - 1) / cluster_split * (cluster_split - 1) * kReduceSlabBytes;
}
// sf_atoms: 32-bit words of scales per row and stage: 1 for 8-bit operands (128 K-elements per stage, one scale per
// 32), 2 when both operands are packed E2M1 (256 K-elements per stage).
__host__ __device__ inline SmemLayout make_smem_layout(uint32_t block_n, uint32_t num_stages, uint32_t cta_group,
                                                       bool decode_b, uint32_t store_bufs, uint32_t cluster_split = 1,
                                                       uint32_t sf_atoms = 1, uint32_t epilogue_warps = kNumEpilogueWarps) {
    SmemLayout L;
    L.a_stage = kBlockM * kBlockK;
    L.b_stage = (block_n / cta_group) * kBlockK;
    L.b_raw_stage = decode_b ? (block_n / cta_group) * (kBlockK / 2) : 0;    // packed FP4: two codes per byte
    L.sfa_stage = 128 * 4 * sf_atoms;
    L.sfb_stage = sfb_rows(block_n) * 4 * sf_atoms;
    uint32_t off = 0;
    if (cluster_split > 1) {
        // One tile per CTA: when the epilogue runs the operand ring is free, so the outgoing partial sums (one 16 KB
        // slab per 32 columns) and the store staging behind them live there and the ring keeps the memory.
        L.store_bufs = (block_n / 32) * kReduceSlabBytes;
    } else {
        L.store_bufs = off; off += epilogue_warps * store_bufs * kStoreBufBytes;
    }
    L.a = off; off += num_stages * L.a_stage;
    L.b = off; off += num_stages * L.b_stage;
    off = (off + 1023u) & ~1023u;
    L.b_raw = off; off += num_stages * L.b_raw_stage;
    off = (off + 1023u) & ~1023u;
    // the scale factors are packed in place: what TMA delivered is read into registers and the atoms written over it
    L.sf_raw_a = off; L.sf_pack_a = off; off += num_stages * L.sfa_stage;
    L.sf_raw_b = off; L.sf_pack_b = off; off += num_stages * L.sfb_stage;
    off = (off + 127u) & ~127u;
    L.reduce = off; off += cluster_reduce_bytes(block_n, cluster_split);
    L.barriers = off; off += (4 * kMaxStages + 4) * 8 + 16;
    L.total = off + 1024;    // slack for the manual 1024-B alignment of the dynamic base
    return L;
}

// ------------------------------------------------------------------------------------------------
// Packed E2M1 -> E4M3 (exact: every E2M1 value is an E4M3 value). Same byte map as the reference's vector-core
// decoder, deep_gemm/include/deep_gemm/fp8_dequant_gemm.hpp:24-38: magnitude 0 -> 0x00, 1 -> 0x30,
// m >= 2 -> 0x30 + 4m, sign bit 3 -> bit 7. Four codes (the low 16 bits of `codes`) become four bytes.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
    return d;
}
__device__ __forceinline__ uint32_t e2m1x4_to_e4m3x4(uint32_t codes) {
    // byte permute as an 8-entry table look-up: selector nibble i picks the byte for code i
    const uint32_t mag = prmt_b32(0x3C383000u, 0x4C484440u, codes & 0x7777u);
    // prmt.b32 with bit 3 of a selector nibble set replicates the MSB of the selected byte over the result byte:
    // 0x80 becomes 0xFF for a negative code and stays 0x80 otherwise, so bit 0 of each byte is the sign
    const uint32_t sgn = prmt_b32(0x80808080u, 0x80808080u, codes & 0xFFFFu);
    return mag | ((sgn << 7) & 0x80808080u);
}
// Eight bytes (16 codes, low nibble first) -> 16 E4M3 bytes.
__device__ __forceinline__ uint4 e2m1x16_to_e4m3x16(uint2 packed) {
    return make_uint4(e2m1x4_to_e4m3x4(packed.x), e2m1x4_to_e4m3x4(packed.x >> 16),
                      e2m1x4_to_e4m3x4(packed.y), e2m1x4_to_e4m3x4(packed.y >> 16));
}

// ------------------------------------------------------------------------------------------------
// FP32 -> BF16 with stochastic rounding, bit-compatible with the reference's StochasticRoundToBF16
// (deep_gemm/include/deep_gemm/epilogue/operators.hpp:224-343; model in tests/utils.py:70-92): the four FP32 bit
// patterns of an aligned column quartet and the quartet's index within the row seed a hash; each value's discarded
// 16 bits are compared against its 16 random bits. NaN becomes 0x7fc0. `v` are raw bits, columns past N count as 0.
// Returns the four BF16 patterns packed as two 32-bit words.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint2 stochastic_round_quartet(uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3, uint32_t quartet) {
    uint32_t h = v0 * 0x5671d42bu + v1 * 0x9995e499u + v2 * 0xace1b8a5u + v3 * 0xe153538du + quartet;
    h = (h ^ (h >> 23)) * 0x7feb352du;
    h ^= h >> 16;
    uint32_t h1 = h * 0x846ca68bu, h2 = h * 0xd35a2d97u;
    h1 ^= h1 >> 11;
    h2 ^= h2 >> 11;
    auto round_one = [](uint32_t v, uint32_t random16) -> uint32_t {
        if ((v & 0x7fffffffu) > 0x7f800000u) return 0x7fc0u;
        return ((v >> 16) + ((v & 0xffffu) > (0xffffu - random16) ? 1u : 0u)) & 0xffffu;
    };
    return make_uint2(round_one(v0, h1 & 0xffffu) | (round_one(v1, h1 >> 16) << 16),
                      round_one(v2, h2 & 0xffffu) | (round_one(v3, h2 >> 16) << 16));
}

// ------------------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------------------
// kMajorA / kMajorB: 0 = K-major, 1 = MN-major operand in global memory.
// kDecodeB: B is packed E2M1 in global memory; warps 8..11 decode each stage into the E4M3 tile the MMA reads.
// kLean: dense GEMM whose CTAs have one tile each and write BF16 / FP32 with plain stores (optional bias). Such a
// kernel runs its set-up and its epilogue exactly once, straight from a cold instruction cache, and the generic
// epilogue (staged TMA stores, alpha, stochastic rounding, FP8 quantisation) costs it several microseconds of
// instruction fetch for code it never needs; the lean instantiation leaves all of that out.
// kFp4: both operands are packed E2M1, K-major: a stage is still 128 bytes of K per row (256 elements), the MMA is
// kind::mxf4 with two scales per row per instruction, and a stage carries eight scale bytes per row instead of four.
// kBf16: BF16 operands, no scale factors (kind::f16): a stage is 128 bytes = 64 K-elements per row; the packer
// warp idles and the MMA thread waits for the operands directly.
// kWideEpi: eight epilogue warps instead of four (warps 8..11 take every other 64-column group of the tile). One warp
// retires about one instruction every five to six cycles on the dependent chains of the epilogue (164 instructions per
// 32x32 chunk), so for short K, where the epilogue and not the main loop bounds a tile, a second warp per scheduler
// doubles the rate at which accumulators are drained.
// kWideTile: block_n in (256, 448]: the tile is two column halves of block_n / 2, each with its own rows of B, scale
// slabs and MMAs, that share the A tile of every stage (28 % fewer bytes per flop into the SM than two narrow tiles);
// one accumulator of block_n columns. A template parameter because the stage loop of every role is a latency chain
// the ring's throughput depends on: the narrow kernels must not carry the extra loops.
// kSimpleEpi: the output is BF16 written (or reduce-added) through staged TMA stores with no alpha, bias, stochastic
// rounding, FP8 quantisation or cluster exchange. The generic epilogue decides all of that per chunk at run time, and
// although every decision is a uniform branch, the code that is jumped over spreads the few instructions a chunk
// really needs across kilobytes: the same sixteen conversions take three times as long as in a straight-line loop
// (in-kernel clock reads), all of it instruction fetch. This instantiation keeps only the straight line.
template <int kCtaGroup, int kMajorA, int kMajorB, bool kDecodeB, bool kLean = false, bool kFp4 = false, bool kBf16 = false,
          bool kWideEpi = false, bool kSimpleEpi = false, bool kWideTile = false>
__global__ void __launch_bounds__((kDecodeB || kWideEpi) ? kNumThreadsDecode : kNumThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
               const __grid_constant__ CUtensorMap tm_d, const __grid_constant__ CUtensorMap tm_d_tail,
               const GemmKernelArgs p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    static_assert(!(kLean && kSimpleEpi), "lean kernels store plainly, simple ones through TMA");
    const uint32_t cluster_split = (kCtaGroup == 1 && !kDecodeB && !kWideEpi && !kSimpleEpi) ? p.cluster_split : 1u;
    constexpr uint32_t kSfAtoms = kBf16 ? 0u : kFp4 ? 2u : 1u;
    constexpr uint32_t kElemBytes = kBf16 ? 2u : 1u;              // bytes per operand element as TMA counts them
    constexpr uint32_t kStageK = kBlockK / kElemBytes;            // TMA elements of K per stage (= K rows of an MN-major tile)
    constexpr uint32_t kAtomMn = 128 / kElemBytes;                // MN elements in one 128-byte swizzle atom
    static_assert(!(kDecodeB && kWideEpi), "warps 8..11 are either decoders or epilogue warps");
    constexpr uint32_t kEpiWarps = kWideEpi ? 2 * kNumEpilogueWarps : kNumEpilogueWarps;
    const SmemLayout L = make_smem_layout(p.block_n, p.num_stages, kCtaGroup, kDecodeB, p.store_bufs, cluster_split, kSfAtoms, kEpiWarps);

    const uint32_t warp = threadIdx.x / 32, lane = lane_id();
    const uint32_t cta_rank = kCtaGroup == 2 ? cluster_ctarank() : 0u;
    const bool is_leader = cta_rank == 0;

    // Barrier block: full[s], sf_full[s], empty[s], sf_tma[s], tmem_full[2], tmem_empty[2], tmem ptr, abort flag
    const uint32_t bar_base = smem_base + L.barriers;
    auto full_bar = [&](uint32_t s) { return bar_base + s * 8; };
    auto sf_full_bar = [&](uint32_t s) { return bar_base + (kMaxStages + s) * 8; };
    auto empty_bar = [&](uint32_t s) { return bar_base + (2 * kMaxStages + s) * 8; };
    auto sf_tma_bar = [&](uint32_t s) { return bar_base + (3 * kMaxStages + s) * 8; };   // the scale columns of a stage have landed
    auto tmem_full_bar = [&](uint32_t e) { return bar_base + (4 * kMaxStages + e) * 8; };
    auto tmem_empty_bar = [&](uint32_t e) { return bar_base + (4 * kMaxStages + 2 + e) * 8; };
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + L.barriers + (4 * kMaxStages + 4) * 8);
    const AbortFlag ab{tmem_ptr_smem + 1, p.status};
    const uint32_t reduce_bar = bar_base + (4 * kMaxStages + 5) * 8;     // cluster split-K: partial sums have arrived

    const uint32_t num_stages = p.num_stages;
    const uint32_t load_n = p.block_n / kCtaGroup;            // rows of B this CTA fetches
    const uint32_t sfb_slabs = sfb_rows(p.block_n) / 128;
    // wide tiles (block_n > 256, K-major 8-bit operands only): two column halves per K step
    static_assert(!kWideTile || (kCtaGroup == 2 && kMajorA == 0 && kMajorB == 0 && !kDecodeB && !kLean && !kWideEpi),
                  "wide tiles: CTA pairs with K-major operands");
    constexpr uint32_t n_halves = kWideTile ? 2u : 1u;
    const uint32_t half_n = p.block_n / n_halves, load_half = load_n / n_halves, slabs_half = sfb_slabs / n_halves;

    if (threadIdx.x == 0) {
        trace_mark(p, 0); trace_mark(p, 1);
        tmem_ptr_smem[1] = 0;
        for (uint32_t s = 0; s < num_stages; ++s) {
            mbar_init(full_bar(s), 1);
            // one arrival per warp that prepares the stage for the MMA: the packer, and the decoders if any
            mbar_init(sf_full_bar(s), kCtaGroup * (1 + (kDecodeB ? kNumDecodeWarps : 0)));
            mbar_init(empty_bar(s), 1);
            mbar_init(sf_tma_bar(s), 1);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            mbar_init(tmem_full_bar(e), 1);
            mbar_init(tmem_empty_bar(e), kEpiWarps * kCtaGroup);   // one arrival per epilogue warp
        }
        if (cluster_split > 1) {
            // the chunks this rank finalises arrive as bulk copies from the other ranks, counted in bytes; how many bytes
            // depends on how many of the tile's rows exist, so the epilogue posts the expected count
            mbar_init(reduce_bar, 1);
        }
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_b);
        tma_prefetch_desc(&tm_sfa); tma_prefetch_desc(&tm_sfb);
        if (!kLean) { tma_prefetch_desc(&tm_d); tma_prefetch_desc(&tm_d_tail); }
    }
    __syncwarp();
    if (warp == 2) {
        tmem_alloc<kCtaGroup>(smem_u32((const void*)tmem_ptr_smem), p.tmem_cols);
        tmem_relinquish<kCtaGroup>();
    }
    tc_fence_before_sync();
    // Warp 0 (whose first lane initialised the barriers and is the TMA producer) only checks in: its loads fill this
    // CTA's own ring and need nothing from the other warps or CTAs, so they start while TMEM is still being allocated.
    const bool in_cluster = kCtaGroup == 2 || cluster_split > 1;
    const uint32_t num_threads = (kDecodeB || kWideEpi) ? kNumThreadsDecode : kNumThreads;
    if (in_cluster) {
        cluster_arrive();
        if (warp != 0) cluster_wait();
    } else {
        if (warp == 0) named_bar_arrive(1, num_threads); else named_bar_sync(1, num_threads);
    }
    tc_fence_after_sync();
    // Programmatic dependent launch: everything above (barriers, TMEM, descriptor prefetch) touches no global data and
    // may run while the preceding kernel of the stream is still finishing; everything below reads operands or writes
    // D and waits for that kernel. The kernel behind this one may start its own set-up as soon as SMs free up.
    griddep_wait();
    griddep_launch_dependents();
    if (threadIdx.x == 0) trace_mark(p, 16);
    const uint32_t tmem_base = tmem_ptr_smem[0];      // (possibly not yet written when warp 0 gets here: see the epilogue)
    if (threadIdx.x == 0) trace_mark(p, 2);
    // TMEM columns: accumulators first, then the scale factors of A and of B.
    const uint32_t tmem_sfa = tmem_base + p.accum_stages * p.block_n;
    const uint32_t tmem_sfb = tmem_sfa + 4 * kSfAtoms;

    if (warp == 0) {
        // ======================================================================== TMA producer
        if (lane == 0) {        // the thread that initialised the barriers
            trace_mark(p, 8);
            Scheduler<kCtaGroup, kLean, kWideTile> sched(p);
            Tile t;
            uint32_t stage = 0, phase = 0;
            bool ok = true, first_issue = true, ring_used = false;
            while (ok && sched.next(t)) {
                if (first_issue) trace_mark(p, 9);
                const uint32_t kb_len = t.kb_end - t.kb_begin;
                for (uint32_t i = 0; i < kb_len; ++i) {
                    const uint32_t kb = t.kb_begin + (i + t.kb_rot >= kb_len ? i + t.kb_rot - kb_len : i + t.kb_rot);
                    // (on the first pass over the ring every stage is free by construction)
                    if (ring_used && !(ok = wait_barrier(empty_bar(stage), phase ^ 1, ab, kStatusTimeoutProducer))) break;
                    if (first_issue) trace_mark(p, 10);
                    const uint32_t bar = full_bar(stage);
                    // The operands and the (much smaller) scale columns complete on barriers of their own, so that the
                    // scales are usually packed by the time the last operand byte lands.
                    // (half tiles of a wide-tile launch fetch one half's rows of B and scale columns only)
                    const uint32_t act_halves = kWideTile ? (t.halves == 3u ? 2u : 1u) : 1u;
                    const uint32_t bytes = (L.a_stage >> p.a_tx_shift) + (kDecodeB ? L.b_raw_stage : kWideTile ? act_halves * load_half * kBlockK
                                                                                           : (load_n * kBlockK) >> p.b_tx_shift);
                    static_assert(!kBf16 || !kDecodeB, "BF16 operands are never decoded");
                    mbar_arrive_expect_tx(bar, bytes);
                    const uint32_t sf_bar = sf_tma_bar(stage);
                    if constexpr (!kBf16) mbar_arrive_expect_tx(sf_bar, L.sfa_stage + (kWideTile ? act_halves * (L.sfb_stage / 2) : L.sfb_stage));
                    if (first_issue) { trace_mark(p, 3); first_issue = false; }
                    const uint32_t sa = smem_base + L.a + stage * L.a_stage;
                    const uint32_t sb = smem_base + L.b + stage * L.b_stage;
                    const int32_t k0 = (int32_t)(kb * kStageK);
                    if constexpr (kMajorA == 0) {
                        tma_load_3d(sa, &tm_a, bar, k0, (int32_t)t.row0, (int32_t)t.row_z);
                    } else {
                        // one box per 128-byte atom along M: [atom][K rows of the stage][128 B]
                        #pragma unroll
                        for (uint32_t a0 = 0; a0 < kBlockM; a0 += kAtomMn)
                            tma_load_3d(sa + (a0 / kAtomMn) * kStageK * 128, &tm_a, bar, (int32_t)(t.row0 + a0), k0, (int32_t)t.row_z);
                    }
                    const uint32_t bn0 = t.n0 + cta_rank * load_n;
                    if constexpr (kDecodeB) {
                        // packed bytes, unswizzled: [load_n rows][64 B of K] or [128 K rows][load_n / 2 B of N]
                        const uint32_t sraw = smem_base + L.b_raw + stage * L.b_raw_stage;
                        if constexpr (kMajorB == 0) tma_load_3d(sraw, &tm_b, bar, k0 / 2, (int32_t)bn0, (int32_t)t.b_z);
                        else tma_load_3d(sraw, &tm_b, bar, (int32_t)(bn0 / 2), k0, (int32_t)t.b_z);
                    } else if constexpr (kMajorB == 0) {
                        // (in a CTA pair every half is split between the two CTAs, as its MMA expects)
                        for (uint32_t h = 0; h < n_halves; ++h)
                            if (!kWideTile || ((t.halves >> h) & 1u))
                                tma_load_3d(sb + h * load_half * kBlockK, &tm_b, bar, k0,
                                            (int32_t)(t.n0 + h * half_n + cta_rank * load_half), (int32_t)t.b_z);
                    } else {
                        // one box per 128-byte atom along N: [atom][K rows of the stage][128 B]
                        for (uint32_t a0 = 0; a0 < load_n; a0 += kAtomMn)
                            tma_load_3d(sb + (a0 / kAtomMn) * kStageK * 128, &tm_b, bar, (int32_t)(bn0 + a0), k0, (int32_t)t.b_z);
                    }
                    if (i == 0) trace_mark(p, 11);
                    if constexpr (!kBf16) {
                        tma_load_3d(smem_base + L.sf_raw_a + stage * L.sfa_stage, &tm_sfa, sf_bar,
                                    (int32_t)t.row0, (int32_t)(kb * 2 * kSfAtoms), (int32_t)t.row_z);
                        for (uint32_t h = 0; h < n_halves; ++h)
                            if (!kWideTile || ((t.halves >> h) & 1u))
                                tma_load_3d(smem_base + L.sf_raw_b + stage * L.sfb_stage + h * (L.sfb_stage / n_halves), &tm_sfb, sf_bar,
                                            (int32_t)(t.n0 + h * half_n), (int32_t)(kb * 2 * kSfAtoms), (int32_t)t.b_z);
                    }
                    if (i == 0) trace_mark(p, 12);
                    if (++stage == num_stages) { stage = 0; phase ^= 1; ring_used = true; }
                }
            }
            // Before leaving, make sure nothing this thread issued is still writing into shared memory:
            // the consumers release a stage only after its bytes have landed, so draining the ring is enough.
            for (uint32_t i = 0; i < num_stages && !ab.raised(); ++i) {
                if (!wait_barrier(empty_bar(stage), phase ^ 1, ab, kStatusTimeoutDrain)) break;
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
        __syncwarp();
        if (in_cluster) cluster_wait();       // second half of the set-up barrier
    } else if (warp == 1) {
        // ======================================================================== MMA issuer
        if (is_leader && elect_one()) {
            Scheduler<kCtaGroup, kLean, kWideTile> sched(p);
            Tile t;
            uint32_t stage = 0, phase = 0, tile_iter = 0;
            bool ok = true;
            while (ok && sched.next(t)) {
                const uint32_t e = p.accum_stages == 2 ? (tile_iter & 1u) : 0u;
                const uint32_t e_phase = p.accum_stages == 2 ? ((tile_iter >> 1) & 1u) : (tile_iter & 1u);
                // the epilogue(s) must have drained this accumulator
                if (kCtaGroup == 2) ok = wait_barrier_cluster(tmem_empty_bar(e), e_phase ^ 1, ab, kStatusTimeoutMma);
                else ok = wait_barrier(tmem_empty_bar(e), e_phase ^ 1, ab, kStatusTimeoutMma);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + e * p.block_n;
                for (uint32_t kb = t.kb_begin; kb < t.kb_end; ++kb) {
                    // (BF16: the packer only forwards the arrival of the operands, which in a CTA pair is how the
                    // leader learns that the peer's half has landed too)
                    if (kCtaGroup == 2) ok = wait_barrier_cluster(sf_full_bar(stage), phase, ab, kStatusTimeoutMma);
                    else ok = wait_barrier(sf_full_bar(stage), phase, ab, kStatusTimeoutMma);
                    if (!ok) break;
                    if (tile_iter == 0 && kb == t.kb_begin) trace_mark(p, 4);
                    tc_fence_after_sync();
                    // scales: smem -> TMEM (A: 128 rows = one slab; B: one slab per 128 columns)
                    // (packed E2M1: word g of a row holds the scales of K-elements [128 g, 128 g + 128) of the stage)
                    #pragma unroll
                    for (uint32_t g = 0; g + 1 <= kSfAtoms; ++g) {
                        utccp_32x128b_warpx4<kCtaGroup>(tmem_sfa + g * 4,
                                                        make_sf_desc(smem_base + L.sf_pack_a + stage * L.sfa_stage + g * 512));
                        for (uint32_t i = 0; i < sfb_slabs; ++i)
                            utccp_32x128b_warpx4<kCtaGroup>(tmem_sfb + (g * sfb_slabs + i) * 4,
                                                            make_sf_desc(smem_base + L.sf_pack_b + stage * L.sfb_stage + (g * sfb_slabs + i) * 512));
                    }
                    const uint32_t sa = smem_base + L.a + stage * L.a_stage;
                    const uint32_t sb = smem_base + L.b + stage * L.b_stage;
                    const bool first_half = !kWideTile || (t.halves & 1u), second_half = kWideTile && (t.halves & 2u);   // (half tiles of the last wave)
                    #pragma unroll
                    for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k) {
                        // every instruction consumes 32 bytes of K per row: 32 FP8, 64 FP4 or 16 BF16 elements
                        constexpr uint32_t kMmaKRows = kUmmaK / kElemBytes;
                        uint64_t da, db;
                        if constexpr (kMajorA == 0) da = make_kmajor_sw128_desc(sa + k * kUmmaK);
                        else da = make_mnmajor_sw128_desc(sa + k * kMmaKRows * 128, kStageK * 128);
                        if constexpr (kMajorB == 0) db = make_kmajor_sw128_desc(sb + k * kUmmaK);
                        else db = make_mnmajor_sw128_desc(sb + k * kMmaKRows * 128, kStageK * 128);
                        if constexpr (kBf16) {
                            if (first_half) umma_f16<kCtaGroup>(tmem_d, da, db, p.idesc, (kb > t.kb_begin || k > 0) ? 1u : 0u);
                            if (second_half)              // second column half: its own rows of B
                                umma_f16<kCtaGroup>(tmem_d + half_n, da, make_kmajor_sw128_desc(sb + load_half * kBlockK + k * kUmmaK),
                                                    p.idesc, (kb > t.kb_begin || k > 0) ? 1u : 0u);
                        } else if constexpr (kFp4) {
                            // instruction k reads 64 K-elements: scale bytes 2(k&1), 2(k&1)+1 of word k/2
                            const uint32_t id = (k & 1u) * 2u, g = k >> 1;
                            if (first_half)
                                umma_mxf4<kCtaGroup>(tmem_d, da, db, p.idesc | (id << 4) | (id << 29), tmem_sfa + g * 4,
                                                     tmem_sfb + g * sfb_slabs * 4, (kb > t.kb_begin || k > 0) ? 1u : 0u);
                            if (second_half)              // second column half: its own rows of B and scale slabs
                                umma_mxf4<kCtaGroup>(tmem_d + half_n, da, make_kmajor_sw128_desc(sb + load_half * kBlockK + k * kUmmaK),
                                                     p.idesc | (id << 4) | (id << 29), tmem_sfa + g * 4,
                                                     tmem_sfb + (g * sfb_slabs + slabs_half) * 4, (kb > t.kb_begin || k > 0) ? 1u : 0u);
                        } else {
                            const uint32_t idesc = p.idesc | (k << 4) | (k << 29);   // scale ids of B and of A
                            if (first_half)
                                umma_mxf8f6f4<kCtaGroup>(tmem_d, da, db, idesc, tmem_sfa, tmem_sfb,
                                                         (kb > t.kb_begin || k > 0) ? 1u : 0u);
                            if (second_half) {
                                // second column half of a wide tile: its own rows of B, scale slabs and accumulator columns
                                umma_mxf8f6f4<kCtaGroup>(tmem_d + half_n, da, make_kmajor_sw128_desc(sb + load_half * kBlockK + k * kUmmaK),
                                                             idesc, tmem_sfa, tmem_sfb + slabs_half * 4,
                                                             (kb > t.kb_begin || k > 0) ? 1u : 0u);
                            }
                        }
                    }
                    // release the stage once these MMAs have read it
                    if constexpr (kCtaGroup == 2) umma_commit_2cta(empty_bar(stage), 3);
                    else umma_commit_1cta(empty_bar(stage));
                    if (++stage == num_stages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if constexpr (kCtaGroup == 2) umma_commit_2cta(tmem_full_bar(e), 3);
                else umma_commit_1cta(tmem_full_bar(e));
                trace_mark(p, 5);
                ++tile_iter;
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ======================================================================== scale-factor packer
        // raw slab (TMA): [2 K64 columns][rows] int16  ->  packed: [32][4] uint32, entry [l][j] = the four
        // UE8M0 bytes (K blocks 0..3 of this stage) of row j*32+l.
        Scheduler<kCtaGroup, kLean, kWideTile> sched(p);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        const uint32_t leader_sf_full0 = kCtaGroup == 2 ? mapa_shared(sf_full_bar(0), 0) : sf_full_bar(0);
        while (ok && sched.next(t)) {
            for (uint32_t kb = t.kb_begin; kb < t.kb_end; ++kb) {
                if constexpr (!kBf16) {
                    if (!(ok = wait_barrier(sf_tma_bar(stage), phase, ab, kStatusTimeoutPacker))) break;
                }
                const uint16_t* raw_a = reinterpret_cast<const uint16_t*>(smem_gen + L.sf_raw_a + stage * L.sfa_stage);
                uint4* pack_a = reinterpret_cast<uint4*>(smem_gen + L.sf_pack_a + stage * L.sfa_stage);
                const uint32_t rows_b = slabs_half * 128;        // rows of one half's raw columns
                const uint16_t* raw_b = reinterpret_cast<const uint16_t*>(smem_gen + L.sf_raw_b + stage * L.sfb_stage);
                uint4* pack_b = reinterpret_cast<uint4*>(smem_gen + L.sf_pack_b + stage * L.sfb_stage);
                // In place: everything is read into registers first, then the atoms overwrite the raw columns.
                constexpr uint32_t kMaxSlabs = kWideTile ? 4 : 2;           // block_n <= 256, or two halves
                uint4 va[kSfAtoms ? kSfAtoms : 1], vb[kSfAtoms ? kSfAtoms : 1][kMaxSlabs];
                #pragma unroll
                for (uint32_t g = 0; g + 1 <= kSfAtoms; ++g) {   // word g of a row = int16 columns 2g and 2g + 1
                    uint32_t v[4];
                    #pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        v[j] = (uint32_t)raw_a[(2 * g) * 128 + j * 32 + lane] | ((uint32_t)raw_a[(2 * g + 1) * 128 + j * 32 + lane] << 16);
                    va[g] = make_uint4(v[0], v[1], v[2], v[3]);
                    #pragma unroll
                    for (uint32_t i = 0; i < kMaxSlabs; ++i) {
                        if (i < sfb_slabs) {
                            // slab i belongs to half i / slabs_half, whose raw columns are an array of their own
                            const uint32_t hh = (kWideTile && i >= slabs_half) ? 1u : 0u;
                            const uint16_t* raw_h = raw_b + hh * (2 * kSfAtoms * rows_b);
                            #pragma unroll
                            for (uint32_t j = 0; j < 4; ++j) {
                                const uint32_t r = (i - hh * slabs_half) * 128 + j * 32 + lane;
                                v[j] = (uint32_t)raw_h[(2 * g) * rows_b + r] | ((uint32_t)raw_h[(2 * g + 1) * rows_b + r] << 16);
                            }
                            vb[g][i] = make_uint4(v[0], v[1], v[2], v[3]);
                        }
                    }
                }
                __syncwarp();
                #pragma unroll
                for (uint32_t g = 0; g + 1 <= kSfAtoms; ++g) {
                    pack_a[g * 32 + lane] = va[g];
                    #pragma unroll
                    for (uint32_t i = 0; i < kMaxSlabs; ++i)
                        if (i < sfb_slabs) pack_b[(g * sfb_slabs + i) * 32 + lane] = vb[g][i];
                }
                fence_proxy_async_smem();
                // the arrival below also tells the MMA thread (in a CTA pair: the leader's) that this CTA's operands are in
                if (!(ok = wait_barrier(full_bar(stage), phase, ab, kStatusTimeoutPacker))) break;
                __syncwarp();
                // one (possibly remote) arrival per warp: remote arrivals are slow enough to matter per K block
                if (lane == 0) {
                    if constexpr (kCtaGroup == 2) mbar_arrive_cluster(leader_sf_full0 + stage * 8);
                    else mbar_arrive(sf_full_bar(stage));
                }
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (kDecodeB && warp >= 8) {
        // ======================================================================== FP4 decoders
        // One work item = 8 packed bytes (16 codes) -> one 16-byte chunk of the swizzled E4M3 tile.
        Scheduler<kCtaGroup, kLean, kWideTile> sched(p);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        const uint32_t tid = threadIdx.x - 256;                         // 0..127
        const uint32_t leader_sf_full0 = kCtaGroup == 2 ? mapa_shared(sf_full_bar(0), 0) : sf_full_bar(0);
        while (ok && sched.next(t)) {
            for (uint32_t kb = t.kb_begin; kb < t.kb_end; ++kb) {
                if (!(ok = wait_barrier(full_bar(stage), phase, ab, kStatusTimeoutDecoder))) break;
                const uint8_t* raw = smem_gen + L.b_raw + stage * L.b_raw_stage;
                uint8_t* tile = smem_gen + L.b + stage * L.b_stage;
                const uint32_t items = load_n * (kBlockK / 16);
                if constexpr (kMajorB == 0) {
                    // raw [n][64 B]; tile row n = 128 B, chunk c at position c ^ (n & 7)
                    for (uint32_t i = tid; i < items; i += kNumDecodeWarps * 32) {
                        const uint32_t n = i >> 3, c = i & 7u;
                        const uint2 v = *reinterpret_cast<const uint2*>(raw + n * 64 + c * 8);
                        *reinterpret_cast<uint4*>(tile + n * 128 + ((c ^ (n & 7u)) * 16)) = e2m1x16_to_e4m3x16(v);
                    }
                } else {
                    // raw [k][load_n / 2 B]; tile [atom of 128 n][k][128 B], chunk c at position c ^ (k & 7)
                    const uint32_t raw_pitch = load_n / 2;
                    for (uint32_t i = tid; i < items; i += kNumDecodeWarps * 32) {
                        const uint32_t c = i & 7u, k = (i >> 3) & (kBlockK - 1), atom = i >> 10;
                        const uint2 v = *reinterpret_cast<const uint2*>(raw + k * raw_pitch + atom * 64 + c * 8);
                        *reinterpret_cast<uint4*>(tile + atom * (kBlockK * 128) + k * 128 + ((c ^ (k & 7u)) * 16)) =
                            e2m1x16_to_e4m3x16(v);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (kCtaGroup == 2) mbar_arrive_cluster(leader_sf_full0 + stage * 8);
                    else mbar_arrive(sf_full_bar(stage));
                }
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
    }
    // A lean kernel has one tile per CTA: when that tile has been multiplied, warps 0..3 have nothing left to do, and one
    // warp alone retires the ~160 dependent instructions of a 32-column chunk in about 900 cycles. So they join as a second
    // set of epilogue warps (warp w reads the same TMEM lane quarter as warp w + 4) and the two sets take alternate chunks.
    if ((warp >= 4 && warp < 4 + kEpiWarps) || (kLean && warp < 4)) {
        // ======================================================================== epilogue
        const uint32_t q = warp % 4;                         // TMEM lane quadrant == warp index % 4
        const uint32_t eset = (kLean && warp < 4) ? 1u : 0u; // lean kernels: the second set of epilogue warps
        const uint32_t col_half = kLean ? 0u : (warp - 4) / 4;   // wide epilogue: which 64-column groups this warp takes
        constexpr uint32_t kColStep = kWideEpi ? 128u : 64u;
        Scheduler<kCtaGroup, kLean, kWideTile> sched(p);
        Tile t;
        uint32_t tile_iter = 0, buf = 0;
        bool ok = true;
        // Staging boxes: one set per warp of the first set in the region laid out for them; the second set of a lean kernel
        // takes boxes in the operand ring, which is free once the only tile has been multiplied (behind the outgoing partial
        // sums and the first set's boxes when the K splits reduce through the cluster).
        const uint32_t box_off = eset == 0 ? L.store_bufs + (warp - 4) * p.store_bufs * kStoreBufBytes
                                           : (cluster_split > 1 ? L.store_bufs + (4 * p.store_bufs + warp) * kStoreBufBytes
                                                                : L.a + warp * kStoreBufBytes);
        const uint32_t store_base = smem_base + box_off;
        uint8_t* store_gen = smem_gen + box_off;
        auto out_is_fp32 = [&]() -> bool { return !kSimpleEpi && p.d_is_fp32 != 0; };   // a kernel-argument read, not a register
        const uint32_t leader_tmem_empty0 = kCtaGroup == 2 ? mapa_shared(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
        while (ok && sched.next(t)) {
            const uint32_t e = p.accum_stages == 2 ? (tile_iter & 1u) : 0u;
            const uint32_t e_phase = p.accum_stages == 2 ? ((tile_iter >> 1) & 1u) : (tile_iter & 1u);
            if (!(ok = wait_barrier(tmem_full_bar(e), e_phase, ab, kStatusTimeoutEpilogue))) break;
            if (tile_iter == 0 && threadIdx.x == 128) trace_mark(p, 6);
            tc_fence_after_sync();
            const uint32_t row = t.row0 + q * 32 + lane;       // row of D held by this thread
            // Warp 0 read tmem_base right after checking in at the set-up barrier, possibly before the allocation had
            // written it; the accumulator barrier it has just passed orders this read behind the allocation.
            const uint32_t taddr = (eset != 0 ? tmem_ptr_smem[0] : tmem_base) + ((q * 32u) << 16) + e * p.block_n;
            // columns of the tile this launch of the epilogue covers (a half tile of a wide-tile launch: one half)
            const uint32_t col_begin = (kWideTile && t.halves == 2u) ? half_n : 0u;
            const uint32_t col_end = (kWideTile && t.halves == 1u) ? half_n : p.block_n;

            // Lean kernels write D with plain stores. A thread holds one row of the tile, so storing straight from the
            // registers makes every store instruction touch 32 rows (32 separate sectors): measured, about 900 cycles per
            // 32-column chunk per CTA, all of it transaction issue. Instead a warp stages its 32 rows x 64 (or 32) columns
            // in its staging box, then every store instruction writes whole 128-byte (64-byte) row segments.
            uint32_t col_stop = col_end;            // the chunk loop of the plain-store path ends at the last column of D
            const bool lean_vec_ok = kLean && (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0 &&
                                     ((p.d_stride * (p.d_is_fp32 ? 4u : 2u)) & 15u) == 0;

            // One 32-column chunk of this thread's row: alpha / bias, cast, stage, store.
            // `single`: the chunk goes out on its own (BF16 boxes normally pair two chunks).
            // `simple_tag`: std::true_type leaves only cast + staged TMA store (the caller has checked that nothing else
            // is asked for), so that the loop over the chunks of such a tile is a short straight line of code.
            auto process_chunk = [&](auto simple_tag, uint32_t (&v)[32], uint32_t c0, bool single) {
                constexpr bool kSimple = kSimpleEpi || decltype(simple_tag)::value;
                const uint32_t col0 = t.n0 + c0;
                if (!kLean && !kSimple && p.has_alpha) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * p.alpha);
                }
                if (!kSimple && p.has_bias) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float bv = 0.f;
                        if (col0 + i < p.n)
                            bv = out_is_fp32() ? __ldg(reinterpret_cast<const float*>(p.bias) + col0 + i)
                                             : __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0 + i));
                        v[i] = __float_as_uint(__uint_as_float(v[i]) + bv);
                    }
                }
                if (!kLean && !kSimple && p.add_c_bf16) {
                    // D = bf16(A B + D): a reduce-add in memory would round the product to BF16 before adding, which costs
                    // up to an ulp of the larger addend when the two nearly cancel; here the old D joins the FP32 sum.
                    if (row < p.m) {
                        const __nv_bfloat16* old_d = reinterpret_cast<const __nv_bfloat16*>(p.d) + (uint64_t)t.d_z * p.d_group_stride +
                                                     (uint64_t)row * p.d_stride + col0;
                        if (col0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(old_d) & 15u) == 0) {
                            #pragma unroll
                            for (uint32_t c = 0; c < 4; ++c) {
                                const uint4 x = reinterpret_cast<const uint4*>(old_d)[c];
                                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
                                #pragma unroll
                                for (uint32_t j = 0; j < 4; ++j) {
                                    v[c * 8 + 2 * j] = __float_as_uint(__uint_as_float(v[c * 8 + 2 * j]) + __uint_as_float(w[j] << 16));
                                    v[c * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(v[c * 8 + 2 * j + 1]) + __uint_as_float(w[j] & 0xffff0000u));
                                }
                            }
                        } else {
                            #pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (col0 + i < p.n) v[i] = __float_as_uint(__uint_as_float(v[i]) + __bfloat162float(old_d[i]));
                        }
                    }
                }
                if (!kLean && !kSimple && p.epilogue_mode == kEpiFp8Quant) {
                    // E4M3 output with one UE8M0 scale per row per 32 columns (exactly this thread's chunk). As the
                    // reference does (operators.hpp:368-411, tests/test_einsum.py:74-84): round to BF16 first, scale =
                    // 2^ceil(log2(max(amax, 1e-4) / 448)), divide, round to nearest E4M3.
                    float y[32], amax = 0.f;
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        y[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i])));
                        amax = fmaxf(amax, fabsf(y[i]));
                    }
                    const uint32_t xbits = __float_as_uint(__fdiv_rn(fmaxf(amax, 1e-4f), 448.0f));
                    uint32_t e = ((xbits >> 23) & 0xffu) + ((xbits & 0x7fffffu) != 0u ? 1u : 0u);
                    e = min(max(e, 1u), 254u);
                    const float inv = __uint_as_float((254u - e) << 23);           // 2^(127 - e), exact for e <= 253
                    uint32_t q[8];
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint32_t word = 0;
                        #pragma unroll
                        for (int j = 0; j < 4; ++j)
                            word |= (uint32_t)__nv_cvt_float_to_fp8(y[i * 4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
                        q[i] = word;
                    }
                    if (row < p.m && col0 + 32 <= p.n) {
                        uint8_t* dst = reinterpret_cast<uint8_t*>(p.d) + (uint64_t)t.d_z * p.d_group_stride + (uint64_t)row * p.d_stride + col0;
                        reinterpret_cast<uint4*>(dst)[0] = make_uint4(q[0], q[1], q[2], q[3]);
                        reinterpret_cast<uint4*>(dst)[1] = make_uint4(q[4], q[5], q[6], q[7]);
                        const uint64_t sf_col = ((uint64_t)t.d_z * p.n + col0) >> 6;
                        p.sfd[(sf_col * p.sfd_stride + row) * 2 + ((col0 >> 5) & 1u)] = (uint8_t)e;
                    }
                    return;
                }
                // BF16 output: sixteen packed pairs, rounded to nearest or stochastically
                uint32_t w16[16];
                if (!out_is_fp32()) {
                    if (!kLean && !kSimple && p.stochastic) {
                        #pragma unroll
                        for (uint32_t g = 0; g < 8; ++g) {
                            uint32_t x[4];
                            #pragma unroll
                            for (uint32_t i = 0; i < 4; ++i) x[i] = (col0 + g * 4 + i < p.n) ? v[g * 4 + i] : 0u;
                            const uint2 r = stochastic_round_quartet(x[0], x[1], x[2], x[3], (col0 >> 2) + g);
                            w16[g * 2] = r.x;
                            w16[g * 2 + 1] = r.y;
                        }
                    } else {
                        #pragma unroll
                        for (uint32_t i = 0; i < 16; ++i) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[i * 2]), __uint_as_float(v[i * 2 + 1]));
                            w16[i] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                }
                asm volatile("" :: "r"(w16[0]), "r"(w16[5]), "r"(w16[10]), "r"(w16[15]) : "memory");
                if (kSimple || (!kLean && p.epilogue_mode <= kEpiTmaReduce)) {
                    // Stage a [32 rows x 128 B] box, 16-byte chunk c of row r at chunk (c ^ (r & 7)). A BF16 box holds two
                    // 32-column groups; when block_n is an odd multiple of 32 the last group goes out alone as a
                    // [32 rows x 64 B] box (64B swizzle: chunk c of row r at c ^ ((r >> 1) & 3)) through tm_d_tail.
                    const uint32_t half = (out_is_fp32() || single) ? 0u : ((c0 / 32) & 1u);
                    const bool tail = !out_is_fp32() && half == 0 && (single || c0 + 32 >= col_end);
                    if (half == 0) {
                        // the buffer may still be read by the store issued `store_bufs` boxes ago
                        if (p.store_bufs == 1) tma_store_wait_read<0>();
                        else if (p.store_bufs == 2) tma_store_wait_read<1>();
                        else if (p.store_bufs == 3) tma_store_wait_read<2>();
                        else tma_store_wait_read<3>();
                        __syncwarp();
                    }
                    uint8_t* bufp = store_gen + buf * kStoreBufBytes;
                    if (out_is_fp32()) {
                        uint8_t* rowp = bufp + lane * 128;
                        #pragma unroll
                        for (uint32_t c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(rowp + ((c ^ (lane & 7u)) * 16)) =
                                make_uint4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                    } else {
                        #pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            uint8_t* dst = tail ? bufp + lane * 64 + ((c ^ ((lane >> 1) & 3u)) * 16)
                                                : bufp + lane * 128 + (((half * 4 + c) ^ (lane & 7u)) * 16);
                            *reinterpret_cast<uint4*>(dst) = make_uint4(w16[c * 4], w16[c * 4 + 1], w16[c * 4 + 2], w16[c * 4 + 3]);
                        }
                    }
                    const bool box_done = out_is_fp32() || half == 1 || tail;
                    if (box_done) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int32_t x = (int32_t)(t.n0 + (tail ? c0 : (out_is_fp32() ? c0 : (c0 & ~63u))));
                            const int32_t y = (int32_t)(t.row0 + q * 32);
                            const CUtensorMap* map = tail ? &tm_d_tail : &tm_d;
                            if (p.epilogue_mode == kEpiTmaStore)
                                tma_store_3d(map, store_base + buf * kStoreBufBytes, x, y, (int32_t)t.d_z);
                            else
                                tma_reduce_add_3d(map, store_base + buf * kStoreBufBytes, x, y, (int32_t)t.d_z);
                            tma_store_commit();
                        }
                        if (++buf == p.store_bufs) buf = 0;
                    }
                } else {
                    // plain path: bounds-checked element stores / atomics, any N and any stride; a whole chunk that lies
                    // inside D on a 16-byte boundary goes out as 16-byte stores
                    if constexpr (kLean) {
                        if (lean_vec_ok && col0 + 32 <= p.n) {
                            const uint32_t es = out_is_fp32() ? 4u : 2u;
                            // BF16: two chunks share a box of 128-byte rows when both lie inside D, else the chunk goes alone
                            const uint32_t pair_c0 = c0 & ~63u;
                            const bool pair = !out_is_fp32() && !single && t.n0 + pair_c0 + 64 <= p.n && pair_c0 + 64 <= col_stop;
                            const uint32_t half = pair ? ((c0 >> 5) & 1u) : 0u;
                            uint8_t* bufp = store_gen;
                            if (out_is_fp32()) {
                                #pragma unroll
                                for (uint32_t c = 0; c < 8; ++c)
                                    *reinterpret_cast<uint4*>(bufp + lane * 128 + ((c ^ (lane & 7u)) * 16)) =
                                        make_uint4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                            } else {
                                #pragma unroll
                                for (uint32_t c = 0; c < 4; ++c) {
                                    uint8_t* dst = pair ? bufp + lane * 128 + (((half * 4 + c) ^ (lane & 7u)) * 16)
                                                        : bufp + lane * 64 + ((c ^ ((lane >> 1) & 3u)) * 16);
                                    *reinterpret_cast<uint4*>(dst) = make_uint4(w16[c * 4], w16[c * 4 + 1], w16[c * 4 + 2], w16[c * 4 + 3]);
                                }
                            }
                            if (pair && half == 0) return;              // the box is written out with its second half
                            __syncwarp();
                            uint8_t* out = reinterpret_cast<uint8_t*>(p.d) +
                                           ((uint64_t)t.d_z * p.d_group_stride + t.n0 + (pair ? pair_c0 : c0)) * es;
                            const uint32_t row_base = t.row0 + q * 32;
                            if (out_is_fp32() || pair) {
                                #pragma unroll
                                for (uint32_t it = 0; it < 8; ++it) {          // four rows of 128 bytes per instruction
                                    const uint32_t r = it * 4 + (lane >> 3), c = lane & 7u;
                                    const uint4 x = *reinterpret_cast<const uint4*>(bufp + r * 128 + ((c ^ (r & 7u)) * 16));
                                    if (row_base + r < p.m)
                                        *reinterpret_cast<uint4*>(out + (uint64_t)(row_base + r) * p.d_stride * es + c * 16) = x;
                                }
                            } else {
                                #pragma unroll
                                for (uint32_t it = 0; it < 4; ++it) {          // eight rows of 64 bytes per instruction
                                    const uint32_t r = it * 8 + (lane >> 2), c = lane & 3u;
                                    const uint4 x = *reinterpret_cast<const uint4*>(bufp + r * 64 + ((c ^ ((r >> 1) & 3u)) * 16));
                                    if (row_base + r < p.m)
                                        *reinterpret_cast<uint4*>(out + (uint64_t)(row_base + r) * p.d_stride * es + c * 16) = x;
                                }
                            }
                            __syncwarp();                                   // the box is free again
                            return;
                        }
                    }
                    const bool row_ok = row < p.m;
                    const uint64_t base = (uint64_t)t.d_z * p.d_group_stride + (uint64_t)row * p.d_stride;
                    if ((kLean || p.epilogue_mode == kEpiPlainStore) && col0 + 32 <= p.n) {
                        uint8_t* dst = reinterpret_cast<uint8_t*>(p.d) + (base + col0) * (out_is_fp32() ? 4u : 2u);
                        if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                            if (row_ok) {
                                if (out_is_fp32()) {
                                    #pragma unroll
                                    for (uint32_t c = 0; c < 8; ++c)
                                        reinterpret_cast<uint4*>(dst)[c] = make_uint4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                                } else {
                                    #pragma unroll
                                    for (uint32_t c = 0; c < 4; ++c)
                                        reinterpret_cast<uint4*>(dst)[c] = make_uint4(w16[c * 4], w16[c * 4 + 1], w16[c * 4 + 2], w16[c * 4 + 3]);
                                }
                            }
                            return;
                        }
                    }
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (row_ok && col0 + i < p.n) {
                            const float f = __uint_as_float(v[i]);
                            if (out_is_fp32()) {
                                float* dst = reinterpret_cast<float*>(p.d) + base + col0 + i;
                                if (!kLean && p.epilogue_mode == kEpiPlainAtomic) atomicAdd(dst, f); else *dst = f;
                            } else {
                                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.d) + base + col0 + i;
                                if (!kLean && p.epilogue_mode == kEpiPlainAtomic) atomicAdd(dst, __float2bfloat16_rn(f));
                                else *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(w16[i >> 1] >> ((i & 1) * 16));
                            }
                        }
                    }
                }
            };

            uint32_t va[32], vb[32];
            if (cluster_split > 1) {
                // Cluster split-K: this CTA holds the partial sums of its K range. Chunk c is finalised by rank
                // c % S: everybody else pushes its partial chunk into that rank's shared memory, the owner adds
                // the partials in rank order (so the result does not depend on timing) and runs the usual epilogue.
                const uint32_t S = cluster_split, r = cluster_ctarank();
                const uint32_t chunks = p.block_n / 32;
                const uint32_t row_off = (q * 32 + lane) * 128, sw = lane & 7u;
                // Only the 32-row quarters of the tile that hold rows of D take part (M = 64: two of four).
                const uint32_t rows_here = p.m > t.row0 ? p.m - t.row0 : 0u;
                const uint32_t live_quarters = min(4u, (rows_here + 31u) / 32u);
                const bool live = q < live_quarters;
                if (threadIdx.x == 128) {
                    const uint32_t owned = r < chunks ? (chunks - r + S - 1) / S : 0u;
                    if (owned) mbar_arrive_expect_tx(reduce_bar, owned * (S - 1) * live_quarters * 4096u);
                }
                // Outgoing chunks are staged in the operand ring (this CTA's only tile has been multiplied, so the
                // ring is free) and leave as one 4 KB bulk copy per warp; the staging must stay untouched until the
                // copy has been read, which the cluster barrier at the end of the kernel guarantees.
                // (the two sets of epilogue warps of a lean kernel take alternate outgoing chunks)
                uint32_t sent = 0;
                for (uint32_t c = 0; live && c < chunks; ++c) {
                    const uint32_t owner = c % S;
                    if (owner == r) continue;
                    if (!kLean || (sent & 1u) == eset) {
                        tmem_ld_32x32b_x32(taddr + c * 32, va);
                        tmem_ld_wait();
                        uint8_t* out = smem_gen + L.a + sent * kReduceSlabBytes + row_off;
                        #pragma unroll
                        for (uint32_t u = 0; u < 8; ++u)
                            *reinterpret_cast<uint4*>(out + ((u ^ sw) * 16)) = make_uint4(va[u * 4], va[u * 4 + 1], va[u * 4 + 2], va[u * 4 + 3]);
                    }
                    ++sent;
                }
                if (kLean && threadIdx.x == 128) trace_mark(p, 21);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && live) {
                    sent = 0;
                    for (uint32_t c = 0; c < chunks; ++c) {
                        const uint32_t owner = c % S;
                        if (owner == r) continue;
                        const uint32_t slab = (c / S) * (S - 1) + (r < owner ? r : r - 1);
                        if (!kLean || (sent & 1u) == eset)
                            bulk_copy_to_cluster(mapa_shared(smem_base + L.reduce + slab * kReduceSlabBytes + q * 4096, owner),
                                                 smem_base + L.a + sent * kReduceSlabBytes + q * 4096, 4096,
                                                 mapa_shared(reduce_bar, owner));
                        ++sent;
                    }
                }
                if (threadIdx.x == 128) trace_mark(p, 13);
                if (r < chunks && live) {
                    if (!(ok = wait_barrier(reduce_bar, tile_iter & 1u, ab, kStatusTimeoutReduce))) break;
                    if (threadIdx.x == 128) trace_mark(p, 14);
                    for (uint32_t slot = 0, c = r; c < chunks; ++slot, c += S) {
                        if (t.n0 + c * 32 >= p.n && (kLean || p.epilogue_mode >= kEpiPlainStore)) break;   // beyond N
                        if (kLean && (slot & 1u) != eset) continue;                                       // the other set's chunk
                        tmem_ld_32x32b_x32(taddr + c * 32, va);
                        tmem_ld_wait();
                        if (kLean && slot == 0 && threadIdx.x == 128) trace_mark(p, 22);
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) vb[i] = 0u;        // +0.0f
                        for (uint32_t s = 0; s < S; ++s) {
                            if (s == r) {
                                #pragma unroll
                                for (int i = 0; i < 32; ++i) vb[i] = __float_as_uint(__uint_as_float(vb[i]) + __uint_as_float(va[i]));
                            } else {
                                const uint8_t* slab = smem_gen + L.reduce + (slot * (S - 1) + (s < r ? s : s - 1)) * kReduceSlabBytes + row_off;
                                #pragma unroll
                                for (uint32_t u = 0; u < 8; ++u) {
                                    const uint4 x = *reinterpret_cast<const uint4*>(slab + ((u ^ sw) * 16));
                                    vb[u * 4] = __float_as_uint(__uint_as_float(vb[u * 4]) + __uint_as_float(x.x));
                                    vb[u * 4 + 1] = __float_as_uint(__uint_as_float(vb[u * 4 + 1]) + __uint_as_float(x.y));
                                    vb[u * 4 + 2] = __float_as_uint(__uint_as_float(vb[u * 4 + 2]) + __uint_as_float(x.z));
                                    vb[u * 4 + 3] = __float_as_uint(__uint_as_float(vb[u * 4 + 3]) + __uint_as_float(x.w));
                                }
                            }
                        }
                        if (kLean && slot == 0 && threadIdx.x == 128) trace_mark(p, 23);
                        process_chunk(std::false_type{}, vb, c * 32, true);
                        if (kLean && slot == 0 && threadIdx.x == 128) trace_mark(p, 24);
                    }
                }
            } else {
            // Two register sets: the TMEM load of the next chunk is in flight while this one is converted and staged.
            // With plain stores the columns of the tile that lie beyond N are not even read (the staged TMA boxes are
            // clipped by the hardware instead).
            const bool plain = !kSimpleEpi && (kLean || p.epilogue_mode == kEpiPlainStore || p.epilogue_mode == kEpiPlainAtomic);
            const uint32_t cols = plain ? min(col_end, (p.n - t.n0 + 31u) & ~31u) : col_end;
            col_stop = cols;
            auto run_chunks = [&](auto simple_tag) {
                uint32_t c_first = kWideTile ? col_begin : col_half * 64;
                if (kWideTile && (c_first & 32u) && c_first < cols) {
                    // a second half that starts on an odd 32-column chunk: that chunk goes out on its own, the rest in pairs
                    tmem_ld_32x32b_x32(taddr + c_first, va);
                    tmem_ld_wait();
                    process_chunk(simple_tag, va, c_first, true);
                    c_first += 32;
                }
                if (c_first < cols) tmem_ld_32x32b_x32(taddr + c_first, va);
                for (uint32_t c0 = c_first; c0 < cols; c0 += kColStep) {
                    tmem_ld_wait();
                    if (c0 + 32 < cols) tmem_ld_32x32b_x32(taddr + c0 + 32, vb);
                    process_chunk(simple_tag, va, c0, false);
                    if (c0 + 32 < cols) {
                        tmem_ld_wait();
                        if (c0 + kColStep < cols) tmem_ld_32x32b_x32(taddr + c0 + kColStep, va);
                        process_chunk(simple_tag, vb, c0 + 32, false);
                    }
                }
            };
            // (the 384-thread instantiations have 168 registers per thread: two copies of the loop make them spill)
            constexpr bool kTwoLoops = !kSimpleEpi && !kLean && !kDecodeB && !kWideEpi;
            if constexpr (kLean) {
                // one tile, two sets of warps: chunk c goes to set c % 2, every chunk as a box of its own
                (void)run_chunks;
                uint32_t c0 = eset * 32;
                if (c0 < cols) tmem_ld_32x32b_x32(taddr + c0, va);
                for (; c0 < cols; c0 += 128) {
                    tmem_ld_wait();
                    if (c0 == 0 && threadIdx.x == 128) trace_mark(p, 19);
                    if (c0 + 64 < cols) tmem_ld_32x32b_x32(taddr + c0 + 64, vb);
                    process_chunk(std::false_type{}, va, c0, true);
                    if (c0 == 0 && threadIdx.x == 128) trace_mark(p, 20);
                    if (c0 + 64 < cols) {
                        tmem_ld_wait();
                        if (c0 + 128 < cols) tmem_ld_32x32b_x32(taddr + c0 + 128, va);
                        process_chunk(std::false_type{}, vb, c0 + 64, true);
                    }
                }
            } else if (kSimpleEpi || (kTwoLoops && p.epi_simple)) run_chunks(std::true_type{});
            else if constexpr (!kSimpleEpi) run_chunks(std::false_type{});
            }
            if (tile_iter == 0 && threadIdx.x == 128) trace_mark(p, 15);
            // this accumulator may be overwritten by the next-but-one tile
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0 && eset == 0) {
                if constexpr (kCtaGroup == 2) mbar_arrive_cluster(leader_tmem_empty0 + e * 8);
                else mbar_arrive(tmem_empty_bar(e));
            }
            ++tile_iter;
        }
        // shared memory must outlive the bulk stores that read it; their global writes complete with the grid
        tma_store_wait_read<0>();
        if (threadIdx.x == 128) trace_mark(p, 7);
    }

    // ============================================================================ teardown
    tc_fence_before_sync();
    if (kCtaGroup == 2 || cluster_split > 1) { cluster_arrive(); cluster_wait(); } else { __syncthreads(); }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc<kCtaGroup>(tmem_base, p.tmem_cols);
    }
    if (threadIdx.x == 0) { trace_mark(p, 17); trace_mark(p, 18); }
}

}  // namespace dg
