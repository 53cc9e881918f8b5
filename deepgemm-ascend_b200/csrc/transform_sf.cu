// Scale-factor relayout into the layout the GEMM kernel reads: int16 [MN, ceil(K/64)], MN-major,
// two UE8M0 bytes per element (low byte = even 32-wide K block).
//
// Replaces the reference's transform_sf kernel, deep_gemm/include/deep_gemm/transform_sf.hpp:447-639:
// exponent extraction and validation (:13-21), pair packing (:276-279), K-major -> MN-major transpose,
// replication over gran_mn rows (:616-619) and zeroing of the rows in a group's padding (:374-445).
// Added here: k_repeat = 4 expands a per-128-K scale over the four 32-wide blocks it covers.
//
// HBM-bound streaming kernel. Each CTA produces a [128 rows x 32 int16 columns] output tile: the
// source region it needs (at most 128 rows x 64 scales) is read coalesced along whichever source
// axis is contiguous, reduced to bytes in shared memory, and written back coalesced along MN.
#include <algorithm>
#include <cstdlib>
#include <cuda_runtime.h>
#include <cstdint>

#include "host_common.h"

namespace dg {

constexpr uint32_t kTileRows = 128;      // output rows per CTA
constexpr uint32_t kTileCols = 32;       // output int16 columns per CTA (= 64 K blocks)
constexpr uint32_t kTsfThreads = 256;

struct TransformSfArgs {
    const void* src;
    int16_t* dst;
    uint64_t src_row_stride, src_col_stride, src_batch_stride;
    uint64_t dst_col_stride, dst_batch_stride;
    uint32_t src_rows, src_cols;
    uint32_t src_scales;                   // scale bytes per source row (src_cols, or twice that for a packed source)
    uint32_t dst_mn, dst_cols, k32_blocks;
    uint32_t gran_mn, k_repeat;
    uint32_t gran_shift, k_repeat_shift;   // log2 of the two (both are powers of two): the per-element loops shift instead of dividing
    uint32_t src_is_fp32;
    const int32_t* psum;
    uint32_t num_groups, alignment;
    int32_t* invalid_flag;
    uint32_t tiles_m, tiles_c;
    const int32_t* k_psum;            // K-grouped operands: psum layout along K, scales inside a group's padding become 0
    uint32_t num_k_groups;
};

// Is K unit `idx` (a 32-wide block when div = 32, an int16 column when div = 64) inside the padding of a K group?
// Group g pads the units [ceil(psum[g]/div), align(psum[g], alignment)/div)  (tests/test_layout.py:95-97).
__device__ __forceinline__ bool k_unit_in_group_padding(const TransformSfArgs& a, uint32_t idx, uint32_t div) {
    uint32_t lo = 0, hi = a.num_k_groups;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) / 2;
        const uint32_t p = (uint32_t)__ldg(a.k_psum + mid);
        const uint32_t end = (p + a.alignment - 1) / a.alignment * a.alignment / div;
        if (end > idx) hi = mid; else lo = mid + 1;
    }
    if (lo >= a.num_k_groups) return true;
    const uint32_t p = (uint32_t)__ldg(a.k_psum + lo);
    return idx >= (p + div - 1) / div;
}

// Is source row r (in units of gran_mn rows) inside the padding of some group?  Group g pads the
// source rows [ceil(psum[g]/gran), align(psum[g], alignment)/gran).
__device__ __forceinline__ bool row_in_group_padding(const TransformSfArgs& a, uint32_t r) {
    uint32_t lo = 0, hi = a.num_groups;          // first g with align(psum[g])/gran > r
    while (lo < hi) {
        const uint32_t mid = (lo + hi) / 2;
        const uint32_t p = (uint32_t)__ldg(a.psum + mid);
        const uint32_t end = (p + a.alignment - 1) / a.alignment * a.alignment / a.gran_mn;
        if (end > r) hi = mid; else lo = mid + 1;
    }
    if (lo >= a.num_groups) return true;         // beyond the last group: nothing valid lives there
    const uint32_t p = (uint32_t)__ldg(a.psum + lo);
    return r >= (p + a.gran_mn - 1) / a.gran_mn;
}

__global__ void __launch_bounds__(kTsfThreads) transform_sf_kernel(const TransformSfArgs a) {
    __shared__ uint8_t bytes[kTileRows][64 + 4];    // [source row][source scale], as UE8M0 bytes
    __shared__ uint8_t padded[kTileRows];

    const uint32_t tiles_per_batch = a.tiles_m * a.tiles_c;
    for (uint32_t tile = blockIdx.x; tile < tiles_per_batch; tile += gridDim.x) {
        const uint32_t batch = blockIdx.y;
        const uint32_t tm = tile % a.tiles_m, tc = tile / a.tiles_m;
        const uint32_t mn0 = tm * kTileRows, c0 = tc * kTileCols;
        const uint32_t r0 = mn0 >> a.gran_shift;
        const uint32_t rows = min((kTileRows + a.gran_mn - 1) >> a.gran_shift, a.src_rows > r0 ? a.src_rows - r0 : 0u);
        // source scales covering K blocks [2*c0, 2*c0 + 64)
        const uint32_t s0 = (2 * c0) >> a.k_repeat_shift;
        const uint32_t scales = 64u >> a.k_repeat_shift;
        const uint32_t scales_shift = 6u - a.k_repeat_shift;

        __syncthreads();                       // previous tile's readers are done with shared memory
        if (threadIdx.x < kTileRows)
            padded[threadIdx.x] = (a.psum != nullptr && threadIdx.x < rows) ? row_in_group_padding(a, r0 + threadIdx.x) : 0;
        __syncthreads();

        const uint8_t* src_base = reinterpret_cast<const uint8_t*>(a.src);
        if (a.src_is_fp32) {
            const uint32_t total = rows * scales;
            const bool row_fast = a.src_row_stride == 1 && a.src_col_stride != 1;
            bool bad = false;
            for (uint32_t i = threadIdx.x; i < total; i += kTsfThreads) {
                const uint32_t r = row_fast ? i % rows : i >> scales_shift;
                const uint32_t s = row_fast ? i / rows : i & (scales - 1);
                uint8_t e = 0;
                if (s0 + s < a.src_cols && !padded[r]) {
                    const uint64_t off = batch * a.src_batch_stride + (uint64_t)(r0 + r) * a.src_row_stride + (uint64_t)(s0 + s) * a.src_col_stride;
                    const uint32_t bits = __ldg(reinterpret_cast<const uint32_t*>(src_base) + off);
                    e = (uint8_t)((bits >> 23) & 0xff);
                    // negative, or not a power of two (scales inside a K group's padding are garbage by contract)
                    if ((bits & 0x807fffffu) != 0 && !(a.k_psum != nullptr && k_unit_in_group_padding(a, s0 + s, 32))) bad = true;
                }
                bytes[r][s] = e;
            }
            if (bad && a.invalid_flag != nullptr) atomicExch(a.invalid_flag, 1);
        } else {
            // int16 source: each element already holds two bytes (two consecutive source scales)
            const uint32_t words = scales / 2 > 0 ? scales / 2 : 1;
            const uint32_t w0 = s0 / 2;
            const uint32_t total = rows * words;
            const bool row_fast = a.src_row_stride == 1 && a.src_col_stride != 1;
            for (uint32_t i = threadIdx.x; i < total; i += kTsfThreads) {
                const uint32_t r = row_fast ? i % rows : i / words;
                const uint32_t w = row_fast ? i / rows : i % words;
                uint16_t v = 0;
                if (w0 + w < a.src_cols && !padded[r]) {
                    const uint64_t off = batch * a.src_batch_stride + (uint64_t)(r0 + r) * a.src_row_stride + (uint64_t)(w0 + w) * a.src_col_stride;
                    v = __ldg(reinterpret_cast<const uint16_t*>(src_base) + off);
                }
                bytes[r][2 * w] = (uint8_t)(v & 0xff);
                bytes[r][2 * w + 1] = (uint8_t)(v >> 8);
            }
        }
        __syncthreads();

        // Packed int16 input at gran_k = 32 passes its bytes through untouched, including the high
        // byte of a last odd block (tests/test_layout.py:39-50); every other input leaves K blocks
        // that do not exist at 0.
        const bool passthrough = !a.src_is_fp32 && a.k_repeat == 1;
        for (uint32_t i = threadIdx.x; i < kTileRows * kTileCols; i += kTsfThreads) {
            const uint32_t ml = i % kTileRows, c = i / kTileRows;
            const uint32_t mn = mn0 + ml, col = c0 + c;
            if (mn >= a.dst_mn || col >= a.dst_cols) continue;
            const uint32_t r = ml >> a.gran_shift;
            uint32_t lo = 0, hi = 0;
            if (r < rows) {
                const uint32_t kb = 2 * col;
                // when k_repeat = 4 and s0 was rounded down, index relative to the K blocks of s0
                const uint32_t rel0 = (kb >> a.k_repeat_shift) - s0, rel1 = ((kb + 1) >> a.k_repeat_shift) - s0;
                if (passthrough || kb < a.k32_blocks) lo = bytes[r][rel0];
                if (passthrough || kb + 1 < a.k32_blocks) hi = bytes[r][rel1];
                if (a.k_psum != nullptr) {
                    if (passthrough) {
                        if (k_unit_in_group_padding(a, col, 64)) lo = hi = 0;
                    } else {
                        if (k_unit_in_group_padding(a, kb, 32)) lo = 0;
                        if (k_unit_in_group_padding(a, kb + 1, 32)) hi = 0;
                    }
                }
            }
            a.dst[batch * a.dst_batch_stride + (uint64_t)col * a.dst_col_stride + mn] = (int16_t)(lo | (hi << 8));
        }
    }
}

// Streaming form of the kernel above for the common case: a K-major source (scales of a row contiguous) whose rows
// are 16-byte aligned, and a destination whose columns are 16-byte aligned; no K-group padding. Same tiles and the
// same staging in shared memory, but every thread moves 16 bytes at a time: four FP32 scales (or eight packed scale
// bytes) in, eight int16 results of eight consecutive rows out, so the instruction count per byte drops by about six
// and the kernel follows HBM instead of the issue rate.
// kPerRow (gran_mn = 1, the scales of activations and of per-row quantised weights): the staging area is kept
// transposed, one array of int16 results per output column, so that the eight consecutive rows a thread writes are two
// 8-byte shared-memory loads instead of sixteen byte gathers.
constexpr uint32_t kColPitch = kTileRows + 4;      // int16 elements per staged column (8-byte aligned, spreads the banks)
template <bool kFp32, bool kPerRow>
__global__ void __launch_bounds__(kTsfThreads, 4) transform_sf_stream_kernel(const TransformSfArgs a) {
    __shared__ __align__(16) uint8_t bytes[kPerRow ? 1 : kTileRows][64 + 4];
    __shared__ __align__(16) uint16_t cols[kPerRow ? kTileCols : 1][kColPitch];
    __shared__ uint8_t padded[kTileRows];

    const uint32_t tiles_per_batch = a.tiles_m * a.tiles_c;
    const uint32_t batch = blockIdx.y;
    bool bad = false;
    for (uint32_t tile = blockIdx.x; tile < tiles_per_batch; tile += gridDim.x) {
        const uint32_t tm = tile % a.tiles_m, tc = tile / a.tiles_m;
        const uint32_t mn0 = tm * kTileRows, c0 = tc * kTileCols;
        const uint32_t r0 = mn0 >> a.gran_shift;
        const uint32_t rows = min((kTileRows + a.gran_mn - 1) >> a.gran_shift, a.src_rows > r0 ? a.src_rows - r0 : 0u);
        const uint32_t s0 = (2 * c0) >> a.k_repeat_shift;             // first source scale of the tile
        const uint32_t scales_shift = 6u - a.k_repeat_shift;          // log2(source scales per tile row)

        __syncthreads();
        if (threadIdx.x < kTileRows)
            padded[threadIdx.x] = (a.psum != nullptr && threadIdx.x < rows) ? row_in_group_padding(a, r0 + threadIdx.x) : 0;
        __syncthreads();

        // ---- in: units of four scale bytes
        // (a tile has at most 128 rows x 16 units = 8 per thread: all loads are issued before the first is used)
        const uint32_t unit_shift = scales_shift - 2u, units = rows << unit_shift;
        constexpr uint32_t kUnitsPerThread = kTileRows * 16 / kTsfThreads;
        uint4 in[kUnitsPerThread];
        #pragma unroll
        for (uint32_t it = 0; it < kUnitsPerThread; ++it) {
            const uint32_t i = threadIdx.x + it * kTsfThreads;
            in[it] = make_uint4(0u, 0u, 0u, 0u);
            if (i >= units) continue;
            const uint32_t r = i >> unit_shift, u = i & ((1u << unit_shift) - 1u);
            const uint32_t s = s0 + 4u * u;
            if (padded[r] || s >= a.src_scales) continue;
            const uint64_t row_off = batch * a.src_batch_stride + (uint64_t)(r0 + r) * a.src_row_stride;
            if constexpr (kFp32) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(a.src) + row_off + s;
                if (s + 4u <= a.src_scales) {
                    in[it] = __ldg(reinterpret_cast<const uint4*>(src));
                } else {
                    in[it].x = __ldg(src);
                    if (s + 1u < a.src_scales) in[it].y = __ldg(src + 1);
                    if (s + 2u < a.src_scales) in[it].z = __ldg(src + 2);
                }
            } else {
                // packed source: int16 element w holds scale bytes 2w and 2w + 1
                const uint16_t* src = reinterpret_cast<const uint16_t*>(a.src) + row_off + s / 2u;
                if (s + 4u <= a.src_scales) in[it].x = __ldg(reinterpret_cast<const uint32_t*>(src));
                else in[it].x = __ldg(src);                                // (an odd tail of one int16)
            }
        }
        #pragma unroll
        for (uint32_t it = 0; it < kUnitsPerThread; ++it) {
            const uint32_t i = threadIdx.x + it * kTsfThreads;
            if (i >= (kPerRow ? (kTileRows << unit_shift) : units)) continue;      // (transposed staging: rows without a source get zeros)
            const uint32_t r = i >> unit_shift, u = i & ((1u << unit_shift) - 1u);
            uint32_t word = in[it].x;
            if constexpr (kFp32) {
                const uint32_t v[4] = {in[it].x, in[it].y, in[it].z, in[it].w};
                word = 0;
                #pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    word |= ((v[j] >> 23) & 0xffu) << (8u * j);
                    if ((v[j] & 0x807fffffu) != 0u) bad = true;       // negative or not a power of two
                }
            }
            if constexpr (kPerRow) {
                if (a.k_repeat_shift == 0) {          // bytes 0..3 = K blocks 4u..4u+3 -> int16 columns 2u, 2u + 1
                    cols[2u * u][r] = (uint16_t)(word & 0xffffu);
                    cols[2u * u + 1u][r] = (uint16_t)(word >> 16);
                } else {                               // each byte covers four K blocks -> two equal int16 columns
                    #pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint16_t both = (uint16_t)(((word >> (8u * j)) & 0xffu) * 0x0101u);
                        cols[8u * u + 2u * j][r] = both;
                        cols[8u * u + 2u * j + 1u][r] = both;
                    }
                }
            } else {
                *reinterpret_cast<uint32_t*>(&bytes[r][4u * u]) = word;
            }
        }
        __syncthreads();

        // ---- out: eight consecutive rows of one int16 column per thread
        const bool passthrough = !kFp32 && a.k_repeat == 1;
        for (uint32_t v = threadIdx.x; v < (kTileRows / 8) * kTileCols; v += kTsfThreads) {
            const uint32_t g8 = v % (kTileRows / 8), c = v / (kTileRows / 8);
            const uint32_t ml0 = g8 * 8u, mn = mn0 + ml0, col = c0 + c;
            if (mn >= a.dst_mn || col >= a.dst_cols) continue;
            const uint32_t kb = 2u * col;
            const uint32_t keep = ((passthrough || kb < a.k32_blocks) ? 0x00ffu : 0u) | ((passthrough || kb + 1u < a.k32_blocks) ? 0xff00u : 0u);
            uint4 packed;
            if constexpr (kPerRow) {
                const uint2 lo = *reinterpret_cast<const uint2*>(&cols[c][ml0]);
                const uint2 hi = *reinterpret_cast<const uint2*>(&cols[c][ml0 + 4u]);
                const uint32_t keep2 = keep | (keep << 16);
                packed = make_uint4(lo.x & keep2, lo.y & keep2, hi.x & keep2, hi.y & keep2);
            } else {
                const uint32_t rel0 = (kb >> a.k_repeat_shift) - s0, rel1 = ((kb + 1u) >> a.k_repeat_shift) - s0;
                if (a.gran_shift >= 3u) {
                    // the eight rows share one source row: one look-up, replicated
                    const uint32_t r = ml0 >> a.gran_shift;
                    const uint32_t one = r < rows ? (((uint32_t)bytes[r][rel0] | ((uint32_t)bytes[r][rel1] << 8)) & keep) : 0u;
                    const uint32_t two = one | (one << 16);
                    packed = make_uint4(two, two, two, two);
                } else {
                    uint32_t out[8];
                    #pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        const uint32_t r = (ml0 + j) >> a.gran_shift;
                        out[j] = r < rows ? (((uint32_t)bytes[r][rel0] | ((uint32_t)bytes[r][rel1] << 8)) & keep) : 0u;
                    }
                    packed = make_uint4(out[0] | (out[1] << 16), out[2] | (out[3] << 16), out[4] | (out[5] << 16), out[6] | (out[7] << 16));
                }
            }
            int16_t* dst = a.dst + batch * a.dst_batch_stride + (uint64_t)col * a.dst_col_stride + mn;
            if (mn + 8u <= a.dst_mn) {
                *reinterpret_cast<uint4*>(dst) = packed;
            } else {
                const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
                for (uint32_t j = 0; mn + j < a.dst_mn; ++j) dst[j] = (int16_t)(w[j >> 1] >> (16u * (j & 1u)));
            }
        }
    }
    if (kFp32 && bad && a.invalid_flag != nullptr) atomicExch(a.invalid_flag, 1);
}

// An MN-major source with one scale row per operand row (gran_mn = 1) already has the destination's orientation: output
// column c of eight consecutive rows is two runs of eight source scales (K blocks 2c and 2c + 1), so every thread moves
// 64 (FP32) or 16 (packed) contiguous bytes in and 16 contiguous bytes out, with no staging at all. Rows in the padding
// of a psum layout are written as zero. Needs 16-byte aligned source columns and destination columns.
template <bool kFp32>
__global__ void __launch_bounds__(kTsfThreads) transform_sf_mn_major_kernel(const TransformSfArgs a) {
    const uint32_t chunks = (a.dst_mn + 7u) / 8u;
    const uint64_t total = (uint64_t)chunks * a.dst_cols;
    const uint32_t batch = blockIdx.y;
    bool bad = false;
    for (uint64_t i = blockIdx.x * (uint64_t)kTsfThreads + threadIdx.x; i < total; i += (uint64_t)gridDim.x * kTsfThreads) {
        const uint32_t col = (uint32_t)(i / chunks), mn = (uint32_t)(i - (uint64_t)col * chunks) * 8u;
        const uint32_t live = min(8u, a.dst_mn - mn);
        // rows of this chunk that hold data: all of them, or those below the end of the psum group the chunk lies in
        // (groups start on multiples of the alignment, which is a multiple of 8: a chunk never straddles two groups)
        uint32_t valid = live;
        if (a.psum != nullptr) {
            uint32_t lo = 0, hi = a.num_groups;
            while (lo < hi) {
                const uint32_t mid = (lo + hi) / 2;
                const uint32_t end = ((uint32_t)__ldg(a.psum + mid) + a.alignment - 1) / a.alignment * a.alignment;
                if (end > mn) hi = mid; else lo = mid + 1;
            }
            const uint32_t end = lo < a.num_groups ? (uint32_t)__ldg(a.psum + lo) : 0u;
            valid = end > mn ? min(live, end - mn) : 0u;
        }
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        if (valid != 0u) {
            if constexpr (kFp32) {
                #pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t kb = 2u * col + h;
                    if (kb >= a.k32_blocks) continue;
                    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.src) + batch * a.src_batch_stride +
                                          (uint64_t)(kb >> a.k_repeat_shift) * a.src_col_stride + mn;
                    uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    if (live == 8u) {
                        const uint4 x = __ldg(reinterpret_cast<const uint4*>(src)), y = __ldg(reinterpret_cast<const uint4*>(src) + 1);
                        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
                    } else {
                        for (uint32_t j = 0; j < live; ++j) v[j] = __ldg(src + j);
                    }
                    #pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        if (j >= valid) continue;
                        if ((v[j] & 0x807fffffu) != 0u) bad = true;            // negative or not a power of two
                        out[j >> 1] |= ((v[j] >> 23) & 0xffu) << (16u * (j & 1u) + 8u * h);
                    }
                }
            } else {
                const uint16_t* src = reinterpret_cast<const uint16_t*>(a.src) + batch * a.src_batch_stride + (uint64_t)col * a.src_col_stride + mn;
                if (live == 8u) {
                    const uint4 x = __ldg(reinterpret_cast<const uint4*>(src));
                    out[0] = x.x; out[1] = x.y; out[2] = x.z; out[3] = x.w;
                } else {
                    for (uint32_t j = 0; j < live; ++j) out[j >> 1] |= (uint32_t)__ldg(src + j) << (16u * (j & 1u));
                }
                #pragma unroll
                for (uint32_t j = 0; j < 8; ++j)
                    if (j >= valid) out[j >> 1] &= ~(0xffffu << (16u * (j & 1u)));
            }
        }
        int16_t* dst = a.dst + batch * a.dst_batch_stride + (uint64_t)col * a.dst_col_stride + mn;
        if (live == 8u) *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
        else for (uint32_t j = 0; j < live; ++j) dst[j] = (int16_t)(out[j >> 1] >> (16u * (j & 1u)));
    }
    if (kFp32 && bad && a.invalid_flag != nullptr) atomicExch(a.invalid_flag, 1);
}

__global__ void pad_rows_kernel(const uint8_t* __restrict__ src, uint64_t src_pitch, uint8_t* __restrict__ dst,
                                uint64_t dst_pitch, uint64_t rows, uint64_t row_bytes) {
    const uint64_t total = rows * dst_pitch;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / dst_pitch, c = i - r * dst_pitch;
        dst[i] = c < row_bytes ? src[r * src_pitch + c] : 0;
    }
}

__global__ void l2_flush_kernel(uint4* __restrict__ buf, size_t n16) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        buf[i] = make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace dg

using namespace dg;

extern "C" int dg_transform_sf_launch(const void* src, int src_is_fp32,
                                      uint64_t src_row_stride, uint64_t src_col_stride, uint64_t src_batch_stride,
                                      uint32_t src_rows, uint32_t src_cols,
                                      int16_t* dst, uint64_t dst_col_stride, uint64_t dst_batch_stride,
                                      uint32_t dst_mn, uint32_t k32_blocks, uint32_t gran_mn, uint32_t k_repeat,
                                      uint32_t num_batches, const int32_t* psum, uint32_t num_groups,
                                      uint32_t alignment, int32_t* invalid_flag,
                                      const int32_t* k_psum, uint32_t num_k_groups, void* stream) {
    DG_CHECK_ARG(src != nullptr && dst != nullptr, "transform_sf: null pointer");
    DG_CHECK_ARG(gran_mn >= 1 && gran_mn <= 128 && (gran_mn & (gran_mn - 1)) == 0,
                 "gran_mn only support a power of two in [1, 128]");
    DG_CHECK_ARG(k_repeat == 1 || k_repeat == 4, "transform_sf: gran_k must be 32 or 128");
    DG_CHECK_ARG(psum == nullptr || (num_groups > 0 && num_batches == 1),
                 "Grouped transform SF requires one logical batch and grouped_layout");
    DG_CHECK_ARG(alignment > 0 && alignment % gran_mn == 0, "transform_sf: alignment must be a multiple of gran_mn");
    DG_CHECK_ARG(num_batches >= 1 && num_batches <= 65535, "transform_sf: num_batches out of range");
    DG_CHECK_ARG(k_psum == nullptr || (num_k_groups > 0 && num_batches == 1 && k_repeat == 1 && psum == nullptr),
                 "K-grouped transform SF requires one logical batch, gran_k = 32 and a non-empty psum layout");
    if (dst_mn == 0 || k32_blocks == 0) return DG_OK;

    TransformSfArgs a{};
    a.src = src; a.dst = dst;
    a.src_row_stride = src_row_stride; a.src_col_stride = src_col_stride; a.src_batch_stride = src_batch_stride;
    a.dst_col_stride = dst_col_stride; a.dst_batch_stride = dst_batch_stride;
    a.src_rows = src_rows; a.src_cols = src_cols;
    a.dst_mn = dst_mn; a.k32_blocks = k32_blocks;
    a.dst_cols = (k32_blocks + 1) / 2;
    if (!src_is_fp32 && k_repeat == 1) a.dst_cols = src_cols;    // pass-through keeps the source's column count
    a.gran_mn = gran_mn; a.k_repeat = k_repeat; a.src_is_fp32 = src_is_fp32 ? 1 : 0;
    for (a.gran_shift = 0; (1u << a.gran_shift) < gran_mn; ++a.gran_shift) {}
    a.k_repeat_shift = k_repeat == 4 ? 2u : 0u;
    a.psum = psum; a.num_groups = num_groups; a.alignment = alignment;
    a.invalid_flag = invalid_flag;
    a.k_psum = k_psum; a.num_k_groups = num_k_groups;
    a.tiles_m = (dst_mn + kTileRows - 1) / kTileRows;
    a.tiles_c = (a.dst_cols + kTileCols - 1) / kTileCols;
    const uint64_t tiles = (uint64_t)a.tiles_m * a.tiles_c;
    const uint32_t grid_x = (uint32_t)(tiles < 148ull * 16 ? tiles : 148ull * 16);
    a.src_scales = src_is_fp32 ? src_cols : 2 * src_cols;
    // the streaming form: K-major source with 16-byte aligned rows, 16-byte aligned destination columns, no K groups
    const uint64_t src_elem = src_is_fp32 ? 4 : 2;
    const bool stream_ok = k_psum == nullptr && (src_col_stride == 1 || src_cols == 1) &&
                           (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (src_row_stride * src_elem) % 16 == 0 &&
                           (src_batch_stride * src_elem) % 16 == 0 &&
                           (reinterpret_cast<uintptr_t>(dst) & 15) == 0 && dst_col_stride % 8 == 0 && dst_batch_stride % 8 == 0 &&
                           getenv("DG_TRANSFORM_GENERIC") == nullptr;
    auto s = static_cast<cudaStream_t>(stream);
    const bool per_row = gran_mn == 1;
    // an MN-major per-row source (FP32 with either K granularity, or packed with per-32 scales)
    const bool mn_major_ok = per_row && k_psum == nullptr && src_row_stride == 1 && src_cols > 1 && (src_is_fp32 || k_repeat == 1) &&
                             (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (src_col_stride * src_elem) % 16 == 0 &&
                             (src_batch_stride * src_elem) % 16 == 0 &&
                             (reinterpret_cast<uintptr_t>(dst) & 15) == 0 && dst_col_stride % 8 == 0 && dst_batch_stride % 8 == 0 &&
                             alignment % 8 == 0 && getenv("DG_TRANSFORM_GENERIC") == nullptr;
    if (mn_major_ok) {
        const uint64_t items = (uint64_t)((dst_mn + 7) / 8) * a.dst_cols;
        const uint32_t grid = (uint32_t)std::min<uint64_t>((items + kTsfThreads - 1) / kTsfThreads, 148ull * 32);
        if (src_is_fp32) transform_sf_mn_major_kernel<true><<<dim3(grid, num_batches), kTsfThreads, 0, s>>>(a);
        else transform_sf_mn_major_kernel<false><<<dim3(grid, num_batches), kTsfThreads, 0, s>>>(a);
        DG_CHECK_CUDA(cudaGetLastError());
        count_kernel_launch();
        return DG_OK;
    }
    if (stream_ok && src_is_fp32 && per_row) transform_sf_stream_kernel<true, true><<<dim3(grid_x, num_batches), kTsfThreads, 0, s>>>(a);
    else if (stream_ok && src_is_fp32) transform_sf_stream_kernel<true, false><<<dim3(grid_x, num_batches), kTsfThreads, 0, s>>>(a);
    else if (stream_ok && per_row) transform_sf_stream_kernel<false, true><<<dim3(grid_x, num_batches), kTsfThreads, 0, s>>>(a);
    else if (stream_ok) transform_sf_stream_kernel<false, false><<<dim3(grid_x, num_batches), kTsfThreads, 0, s>>>(a);
    else transform_sf_kernel<<<dim3(grid_x, num_batches), kTsfThreads, 0, s>>>(a);
    DG_CHECK_CUDA(cudaGetLastError());
    count_kernel_launch();
    return DG_OK;
}

extern "C" int dg_pad_rows_launch(const void* src, uint64_t src_pitch_bytes, void* dst, uint64_t dst_pitch_bytes,
                                  uint64_t rows, uint64_t row_bytes, void* stream) {
    DG_CHECK_ARG(src != nullptr && dst != nullptr, "pad_rows: null pointer");
    DG_CHECK_ARG(dst_pitch_bytes >= row_bytes, "pad_rows: destination pitch smaller than a row");
    if (rows == 0 || dst_pitch_bytes == 0) return DG_OK;
    const uint64_t total = rows * dst_pitch_bytes;
    const uint32_t grid = (uint32_t)((total + 255) / 256 < 148ull * 32 ? (total + 255) / 256 : 148ull * 32);
    pad_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(src), src_pitch_bytes, static_cast<uint8_t*>(dst), dst_pitch_bytes, rows, row_bytes);
    DG_CHECK_CUDA(cudaGetLastError());
    count_kernel_launch();
    return DG_OK;
}

extern "C" int dg_l2_flush_launch(void* buffer, size_t bytes, void* stream) {
    DG_CHECK_ARG(buffer != nullptr && (reinterpret_cast<uintptr_t>(buffer) & 15) == 0, "l2_flush: buffer must be 16-byte aligned");
    const size_t n16 = bytes / 16;
    if (n16 == 0) return DG_OK;
    l2_flush_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(buffer), n16);
    DG_CHECK_CUDA(cudaGetLastError());
    return DG_OK;
}
