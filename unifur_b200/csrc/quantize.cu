// Blockwise-absmax NF4 quantize / dequantize / double-quantize kernels (sm_100a).
//
// All four are HBM-bound streaming kernels: 4.5625 algorithmic bytes per value
// (4 B of f32 on one side, 0.5 B of nibbles + 4/64 B of absmax on the other).
// Layout: values and outputs are flat arrays; a thread owns 8 consecutive values
// (one 32-byte sector of f32, one 32-bit word of nibbles), 8 lanes own one
// 64-value block, a warp owns 4 blocks, and warps stride over the array.
#include <cuda_bf16.h>

#include "nf4_common.cuh"

namespace nf4 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;

__device__ __forceinline__ float group8_max(float m) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    return m;
}

// Full 64-blocks only: `nfull` blocks starting at values[0].  PACKED selects nibble
// packing (two codes per byte) versus one code per byte.
template <bool PACKED>
__global__ void __launch_bounds__(kThreads, 8)
quantize_full_kernel(const float4 *__restrict__ values, uint64_t nfull,
                     uint8_t *__restrict__ codes, float *__restrict__ absmax) {
    __shared__ uint32_t s_cells[32];
    if (threadIdx.x < 32) s_cells[threadIdx.x] = c_cell_table[threadIdx.x];
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const uint64_t nwarps = (uint64_t)gridDim.x * kWarpsPerCta;
    const uint64_t nchunks = (nfull + 3) / 4;  // one warp-chunk = 4 blocks
    for (uint64_t chunk = warp; chunk < nchunks; chunk += nwarps) {
        const uint64_t blk = chunk * 4 + (lane >> 3);
        const bool live = blk < nfull;
        const uint64_t g = chunk * 32 + lane;  // group of 8 values
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (live) {
            a = __ldcs(values + 2 * g);
            b = __ldcs(values + 2 * g + 1);
        }
        float m = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                        fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
        // fold from 0.0 with maxNum: NaNs drop out exactly as f32::max does
        m = fmaxf(0.0f, m);
        m = group8_max(m);
        if (!live) continue;
        // one exact reciprocal per thread; each value is then decided from x * rcp, and the
        // whole group is redone exactly if any of its values lands next to a decision threshold
        bool unsure = !(m >= 1e-30f && m <= 1e30f);
        const float rcp = __fdiv_rn(1.0f, m);
        uint32_t c0 = code_of_fast(a.x, rcp, s_cells, unsure),
                 c1 = code_of_fast(a.y, rcp, s_cells, unsure),
                 c2 = code_of_fast(a.z, rcp, s_cells, unsure),
                 c3 = code_of_fast(a.w, rcp, s_cells, unsure),
                 c4 = code_of_fast(b.x, rcp, s_cells, unsure),
                 c5 = code_of_fast(b.y, rcp, s_cells, unsure),
                 c6 = code_of_fast(b.z, rcp, s_cells, unsure),
                 c7 = code_of_fast(b.w, rcp, s_cells, unsure);
        if (unsure) {
            c0 = code_of_exact(a.x, m); c1 = code_of_exact(a.y, m);
            c2 = code_of_exact(a.z, m); c3 = code_of_exact(a.w, m);
            c4 = code_of_exact(b.x, m); c5 = code_of_exact(b.y, m);
            c6 = code_of_exact(b.z, m); c7 = code_of_exact(b.w, m);
        }
        if (PACKED) {
            const uint32_t word = c0 | (c1 << 4) | (c2 << 8) | (c3 << 12) | (c4 << 16) |
                                  (c5 << 20) | (c6 << 24) | (c7 << 28);
            reinterpret_cast<uint32_t *>(codes)[g] = word;
        } else {
            uint2 w;
            w.x = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
            w.y = c4 | (c5 << 8) | (c6 << 16) | (c7 << 24);
            reinterpret_cast<uint2 *>(codes)[g] = w;
        }
        if ((lane & 7u) == 0) absmax[blk] = m;
    }
}

// Generic path: any alignment, any length.  One warp per block, two values per lane.
// Used for the ragged last block and for buffers that are not 16-byte aligned.
template <bool PACKED>
__global__ void __launch_bounds__(kThreads)
quantize_generic_kernel(const float *__restrict__ values, uint64_t len, uint64_t first_block,
                        uint64_t nblocks, uint8_t *__restrict__ codes,
                        float *__restrict__ absmax) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const uint64_t nwarps = (uint64_t)gridDim.x * kWarpsPerCta;
    for (uint64_t i = warp; i < nblocks; i += nwarps) {
        const uint64_t blk = first_block + i;
        const uint64_t e0 = blk * kBlock + 2 * lane;
        const bool h0 = e0 < len, h1 = e0 + 1 < len;
        const float x0 = h0 ? values[e0] : 0.0f;
        const float x1 = h1 ? values[e0 + 1] : 0.0f;
        float m = fmaxf(0.0f, fmaxf(h0 ? fabsf(x0) : 0.0f, h1 ? fabsf(x1) : 0.0f));
        #pragma unroll
        for (int s = 1; s < 32; s <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
        const uint32_t c0 = h0 ? code_of(x0, m) : 0u;
        const uint32_t c1 = h1 ? code_of(x1, m) : 0u;  // a missing partner leaves the nibble 0
        if (PACKED) {
            if (h0) codes[e0 >> 1] = (uint8_t)(c0 | (c1 << 4));
        } else {
            if (h0) codes[e0] = (uint8_t)c0;
            if (h1) codes[e0 + 1] = (uint8_t)c1;
        }
        if (lane == 0) absmax[blk] = m;
    }
}

// ---- dequantize -------------------------------------------------------------

__device__ __forceinline__ float block_scale(const float *__restrict__ absmax,
                                             const uint8_t *__restrict__ scale_codes, float sos,
                                             uint64_t blk) {
    return absmax ? __ldg(absmax + blk) : dq_scale(__ldg(scale_codes + blk), sos);
}

// Full 64-blocks, 16-byte aligned buffers.  A lane reads the codes of eight consecutive values;
// neighbouring lanes then swap halves so that the pair's two 128-bit stores each fill whole
// 32-byte sectors (lane 2j writes values 16j..16j+3 and 16j+8..16j+11, lane 2j+1 the other two
// quads).  Four such groups are in flight per thread to cover the load latency.
template <bool PACKED>
__global__ void __launch_bounds__(kThreads, 8)
dequantize_full_kernel(const uint8_t *__restrict__ codes, uint64_t nfull,
                       const float *__restrict__ absmax, const uint8_t *__restrict__ scale_codes,
                       const float *__restrict__ scale_of_scales, float4 *__restrict__ out) {
    constexpr int kInFlight = 4;
    __shared__ float s_levels[16];
    if (threadIdx.x < 16) s_levels[threadIdx.x] = __uint_as_float(c_level_bits[threadIdx.x]);
    __syncthreads();
    const float sos = scale_of_scales ? __ldg(scale_of_scales) : 0.0f;
    const uint64_t ngroups = nfull * 8;  // 8 values per group; a multiple of 8, so lane pairs stay whole
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    const uint32_t lane = threadIdx.x & 31u;
    const bool odd = lane & 1u;
    const uint64_t first = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
    for (uint64_t g0 = first; g0 - lane < ngroups; g0 += stride * kInFlight) {
        uint32_t lo[kInFlight], hi[kInFlight];  // codes of the first / second quad this lane stores
        float s[kInFlight];
        #pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint64_t g = g0 + u * stride;
            const bool live = g < ngroups;
            uint32_t a = 0, b = 0;  // codes of values 0..3 and 4..7 of the group
            if (PACKED) {
                const uint32_t w = live ? __ldcs(reinterpret_cast<const uint32_t *>(codes) + g) : 0u;
                a = w & 0xffffu;
                b = w >> 16;
            } else {
                const uint2 w = live ? __ldcs(reinterpret_cast<const uint2 *>(codes) + g)
                                     : make_uint2(0u, 0u);
                a = w.x;
                b = w.y;
            }
            s[u] = live ? block_scale(absmax, scale_codes, sos, g >> 3) : 0.0f;
            const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
            lo[u] = odd ? got : a;  // even: own first quad;   odd: partner's second quad
            hi[u] = odd ? b : got;  // even: partner's first quad; odd: own second quad
        }
        #pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint64_t g = g0 + u * stride;
            if (g >= ngroups) continue;
            constexpr int kBits = PACKED ? 4 : 8;
            float4 q0, q1;
            q0.x = __fmul_rn(s_levels[(lo[u] >> (0 * kBits)) & 15u], s[u]);
            q0.y = __fmul_rn(s_levels[(lo[u] >> (1 * kBits)) & 15u], s[u]);
            q0.z = __fmul_rn(s_levels[(lo[u] >> (2 * kBits)) & 15u], s[u]);
            q0.w = __fmul_rn(s_levels[(lo[u] >> (3 * kBits)) & 15u], s[u]);
            q1.x = __fmul_rn(s_levels[(hi[u] >> (0 * kBits)) & 15u], s[u]);
            q1.y = __fmul_rn(s_levels[(hi[u] >> (1 * kBits)) & 15u], s[u]);
            q1.z = __fmul_rn(s_levels[(hi[u] >> (2 * kBits)) & 15u], s[u]);
            q1.w = __fmul_rn(s_levels[(hi[u] >> (3 * kBits)) & 15u], s[u]);
            // pair base = float4 index 2 * (g & ~1); even lane stores quads 0 and 2, odd 1 and 3
            float4 *dst = out + 2 * (g & ~(uint64_t)1) + (odd ? 1 : 0);
            __stcs(dst, q0);
            __stcs(dst + 2, q1);
        }
    }
}

template <bool PACKED>
__global__ void __launch_bounds__(kThreads)
dequantize_generic_kernel(const uint8_t *__restrict__ codes, uint64_t len, uint64_t first,
                          const float *__restrict__ absmax,
                          const uint8_t *__restrict__ scale_codes,
                          const float *__restrict__ scale_of_scales, float *__restrict__ out) {
    const float sos = scale_of_scales ? __ldg(scale_of_scales) : 0.0f;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = first + (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < len; i += stride) {
        uint32_t c;
        if (PACKED) {
            const uint32_t byte = codes[i >> 1];
            c = (i & 1u) ? (byte >> 4) : (byte & 15u);
        } else {
            c = codes[i] & 15u;
        }
        const float s = block_scale(absmax, scale_codes, sos, i / kBlock);
        out[i] = __fmul_rn(__uint_as_float(c_level_bits[c]), s);
    }
}

// ---- load path: quantize the transpose of a checkpoint matrix without materialising it ----
// src is [rows, cols] row-major (a PyTorch linear weight [out, in], bf16 or f32); the result is
// the packed NF4 of its transpose [cols, rows] flattened row-major, i.e. element (c, r) at flat
// index c * rows + r.  With rows % 64 == 0 a 64-block of the result is 64 consecutive r for one
// c: a column segment of src.  One CTA takes a 64 x 64 tile of src through shared memory
// (coalesced reads along c, conflict-free reads along r) and its eight warps quantize the tile's
// 64 blocks with the same arithmetic as quantize_full_kernel.
constexpr int kTTile = 64;
constexpr int kTStride = kTTile + 1;  // floats between the tile's transposed rows (odd: spreads the banks)

template <bool SRC_BF16>
__global__ void __launch_bounds__(kThreads)
quantize_transposed_kernel(const void *__restrict__ src, uint64_t rows, uint64_t cols,
                           uint8_t *__restrict__ codes, float *__restrict__ absmax) {
    __shared__ float s_t[kTTile * kTStride];  // s_t[c][r]
    __shared__ uint32_t s_cells[32];
    if (threadIdx.x < 32) s_cells[threadIdx.x] = c_cell_table[threadIdx.x];
    const uint64_t tiles_c = (cols + kTTile - 1) / kTTile;
    const uint64_t r0 = (blockIdx.x / tiles_c) * kTTile, c0 = (blockIdx.x % tiles_c) * kTTile;
    // 256 threads: thread t reads row (t >> 4) + 16 i, columns 4 (t & 15) .. + 3
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint64_t r = r0 + (threadIdx.x >> 4) + 16 * i;
        const uint64_t c = c0 + 4 * (threadIdx.x & 15u);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (c + 3 < cols) {
            if (SRC_BF16) {
                const uint2 w = __ldcs(reinterpret_cast<const uint2 *>(
                    static_cast<const __nv_bfloat16 *>(src) + r * cols + c));
                v[0] = __uint_as_float(w.x << 16);
                v[1] = __uint_as_float(w.x & 0xffff0000u);
                v[2] = __uint_as_float(w.y << 16);
                v[3] = __uint_as_float(w.y & 0xffff0000u);
            } else {
                const float4 w = __ldcs(reinterpret_cast<const float4 *>(
                    static_cast<const float *>(src) + r * cols + c));
                v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
            }
        } else {
            for (int k = 0; k < 4; ++k)
                if (c + k < cols)
                    v[k] = SRC_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16 *>(src)[r * cols + c + k])
                                    : static_cast<const float *>(src)[r * cols + c + k];
        }
        const uint32_t rl = (threadIdx.x >> 4) + 16 * i, cl = 4 * (threadIdx.x & 15u);
        #pragma unroll
        for (int k = 0; k < 4; ++k) s_t[(cl + k) * kTStride + rl] = v[k];
    }
    __syncthreads();
    // warp w quantizes the blocks of columns c0 + 8 w .. + 7, four at a time: lane l owns values
    // 8 (l & 7) .. + 7 of block (l >> 3)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    #pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t cl = 8 * warp + 4 * half + (lane >> 3);
        const uint64_t c = c0 + cl;
        const float *sp = &s_t[cl * kTStride + 8 * (lane & 7u)];
        const float4 a = make_float4(sp[0], sp[1], sp[2], sp[3]);
        const float4 b = make_float4(sp[4], sp[5], sp[6], sp[7]);
        float m = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                        fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
        m = group8_max(fmaxf(0.0f, m));
        if (c >= cols) continue;
        bool unsure = !(m >= 1e-30f && m <= 1e30f);
        const float rcp = __fdiv_rn(1.0f, m);
        uint32_t q0 = code_of_fast(a.x, rcp, s_cells, unsure), q1 = code_of_fast(a.y, rcp, s_cells, unsure),
                 q2 = code_of_fast(a.z, rcp, s_cells, unsure), q3 = code_of_fast(a.w, rcp, s_cells, unsure),
                 q4 = code_of_fast(b.x, rcp, s_cells, unsure), q5 = code_of_fast(b.y, rcp, s_cells, unsure),
                 q6 = code_of_fast(b.z, rcp, s_cells, unsure), q7 = code_of_fast(b.w, rcp, s_cells, unsure);
        if (unsure) {
            q0 = code_of_exact(a.x, m); q1 = code_of_exact(a.y, m); q2 = code_of_exact(a.z, m);
            q3 = code_of_exact(a.w, m); q4 = code_of_exact(b.x, m); q5 = code_of_exact(b.y, m);
            q6 = code_of_exact(b.z, m); q7 = code_of_exact(b.w, m);
        }
        const uint64_t e = c * rows + r0 + 8 * (lane & 7u);  // flat index of this lane's first value
        reinterpret_cast<uint32_t *>(codes)[e / 8] = q0 | (q1 << 4) | (q2 << 8) | (q3 << 12) | (q4 << 16) |
                                                     (q5 << 20) | (q6 << 24) | (q7 << 28);
        if ((lane & 7u) == 0) absmax[e / kBlock] = m;
    }
}

// Any shape: the transpose written out as f32 (then quantized by the flat kernels).
template <bool SRC_BF16>
__global__ void __launch_bounds__(kThreads)
transpose_to_f32_kernel(const void *__restrict__ src, uint64_t rows, uint64_t cols,
                        float *__restrict__ out) {
    __shared__ float s_t[32][33];
    const uint64_t tiles_c = (cols + 31) / 32;
    const uint64_t r0 = (blockIdx.x / tiles_c) * 32, c0 = (blockIdx.x % tiles_c) * 32;
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // 32 x 8
    for (uint32_t i = ty; i < 32; i += 8) {
        const uint64_t r = r0 + i, c = c0 + tx;
        float v = 0.0f;
        if (r < rows && c < cols)
            v = SRC_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16 *>(src)[r * cols + c])
                         : static_cast<const float *>(src)[r * cols + c];
        s_t[i][tx] = v;
    }
    __syncthreads();
    for (uint32_t i = ty; i < 32; i += 8) {
        const uint64_t c = c0 + i, r = r0 + tx;
        if (r < rows && c < cols) out[c * rows + r] = s_t[tx][i];
    }
}

// ---- embedding: gather rows of a packed table and dequantize them ---------------------
// out[t][j] = level[code(ids[t] * d_model + j)] * scale(block of that element): the rows a batch
// of token ids selects, without materialising the table.  Blocks run over the flat table, so
// with d_model % 8 == 0 a group of eight consecutive elements of a row shares one 32-bit code
// word and one block scale; other widths take the element-wise path.  An id outside
// [0, n_embedding) yields a row of NaNs (the reference's gather would panic; a device kernel
// must not trap).
template <bool BF16>
__global__ void __launch_bounds__(kThreads)
embedding_gather_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ absmax,
                        const uint8_t *__restrict__ scale_codes,
                        const float *__restrict__ scale_of_scales, uint64_t n_embedding,
                        uint64_t d_model, const int64_t *__restrict__ ids, uint64_t n_ids,
                        void *__restrict__ out) {
    __shared__ float s_levels[16];
    if (threadIdx.x < 16) s_levels[threadIdx.x] = __uint_as_float(c_level_bits[threadIdx.x]);
    __syncthreads();
    const float sos = scale_of_scales ? __ldg(scale_of_scales) : 0.0f;
    const float nan = __uint_as_float(0x7fc00000u);
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    const uint64_t first = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
    if ((d_model & 7u) == 0) {
        const uint64_t groups_per_row = d_model / 8, total = n_ids * groups_per_row;
        for (uint64_t i = first; i < total; i += stride) {
            const uint64_t t = i / groups_per_row, gi = i - t * groups_per_row;
            const int64_t id = __ldg(ids + t);
            float v[8];
            if (id < 0 || (uint64_t)id >= n_embedding) {
                #pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = nan;
            } else {
                const uint64_t e = (uint64_t)id * d_model + gi * 8;  // a multiple of 8
                const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(codes) + e / 8);
                const float sc = block_scale(absmax, scale_codes, sos, e / kBlock);
                #pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = __fmul_rn(s_levels[(w >> (4 * k)) & 15u], sc);
            }
            if (BF16) {
                uint32_t o[4];
                #pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
                    o[k] = *reinterpret_cast<const uint32_t *>(&h);
                }
                reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
                float4 *dst = reinterpret_cast<float4 *>(out) + 2 * i;
                __stcs(dst, make_float4(v[0], v[1], v[2], v[3]));
                __stcs(dst + 1, make_float4(v[4], v[5], v[6], v[7]));
            }
        }
    } else {
        const uint64_t total = n_ids * d_model;
        for (uint64_t i = first; i < total; i += stride) {
            const uint64_t t = i / d_model, j = i - t * d_model;
            const int64_t id = __ldg(ids + t);
            float v = nan;
            if (id >= 0 && (uint64_t)id < n_embedding) {
                const uint64_t e = (uint64_t)id * d_model + j;
                const uint32_t byte = __ldg(codes + (e >> 1));
                const uint32_t c = (e & 1u) ? (byte >> 4) : (byte & 15u);
                v = __fmul_rn(__uint_as_float(c_level_bits[c]), block_scale(absmax, scale_codes, sos, e / kBlock));
            }
            if (BF16) reinterpret_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(out)[i] = v;
        }
    }
}

// ---- double quantization ------------------------------------------------------

// Pass 1: max over the (non-negative, never-NaN) block scales.  Their f32 bit patterns
// order like unsigned integers, so one atomicMax on the bits per warp is exact.
__global__ void __launch_bounds__(kThreads)
scale_max_kernel(const float *__restrict__ absmax, uint64_t nblocks, uint32_t *max_bits) {
    float m = 0.0f;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < nblocks; i += stride)
        m = fmaxf(m, __ldg(absmax + i));
    #pragma unroll
    for (int s = 1; s < 32; s <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    if ((threadIdx.x & 31u) == 0) atomicMax(max_bits, __float_as_uint(m));
}

// Pass 2: c = round_half_away(s / max * 255) clamped to [0, 255]; 0 when max == 0
// (src/quantize.rs:294-301).  A NaN quotient (inf / inf) casts to 0 as Rust's `as u8`.
__global__ void __launch_bounds__(kThreads)
scale_encode_kernel(const float *__restrict__ absmax, uint64_t nblocks,
                    const float *__restrict__ max_scale_ptr, uint8_t *__restrict__ scale_codes) {
    const float max_scale = *max_scale_ptr;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < nblocks; i += stride) {
        uint32_t c = 0;
        if (max_scale != 0.0f) {
            float q = roundf(__fmul_rn(__fdiv_rn(__ldg(absmax + i), max_scale), 255.0f));
            q = fminf(fmaxf(q, 0.0f), 255.0f);  // NaN -> 0 through fmaxf
            c = (uint32_t)q;
        }
        scale_codes[i] = (uint8_t)c;
    }
}

int grid_for(uint64_t work_items, int per_cta, int max_waves) {
    uint64_t ctas = (work_items + per_cta - 1) / per_cta;
    uint64_t cap = (uint64_t)kNumSMs * max_waves;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return (int)ctas;
}

template <bool PACKED>
int32_t quantize_impl(const float *values, uint64_t len, uint8_t *codes, float *absmax,
                      cudaStream_t stream) {
    if (len == 0) return NF4_OK;
    if (!values || !codes || !absmax) return fail(NF4_ERR_INVALID_ARG, "nf4_quantize: null pointer");
    const uint64_t nblocks = (len + kBlock - 1) / kBlock;
    const bool fast = aligned16(values) && aligned16(codes) && ((uintptr_t)absmax % 4 == 0);
    uint64_t nfull = fast ? len / kBlock : 0;
    if (nfull) {
        const int grid = grid_for((nfull + 3) / 4, kWarpsPerCta, 8);
        quantize_full_kernel<PACKED><<<grid, kThreads, 0, stream>>>(
            reinterpret_cast<const float4 *>(values), nfull, codes, absmax);
        count_launch();
    }
    if (nfull < nblocks) {
        const uint64_t rest = nblocks - nfull;
        const int grid = grid_for(rest, kWarpsPerCta, 8);
        quantize_generic_kernel<PACKED><<<grid, kThreads, 0, stream>>>(values, len, nfull, rest,
                                                                      codes, absmax);
        count_launch();
    }
    return check_cuda(cudaGetLastError(), "nf4_quantize launch");
}

template <bool PACKED>
int32_t dequantize_impl(const uint8_t *codes, uint64_t len, const float *absmax,
                        const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                        cudaStream_t stream) {
    if (len == 0) return NF4_OK;
    if (!codes || !out) return fail(NF4_ERR_INVALID_ARG, "nf4_dequantize: null pointer");
    if ((absmax != nullptr) == (scale_codes != nullptr))
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_dequantize: give either absmax or scale_codes+scale_of_scales");
    if (scale_codes && !scale_of_scales)
        return fail(NF4_ERR_INVALID_ARG, "nf4_dequantize: scale_codes without scale_of_scales");
    const bool fast = aligned16(codes) && aligned16(out);
    const uint64_t nfull = fast ? len / kBlock : 0;
    if (nfull) {
        const int grid = grid_for(nfull * 8, kThreads, 8);
        dequantize_full_kernel<PACKED><<<grid, kThreads, 0, stream>>>(
            codes, nfull, absmax, scale_codes, scale_of_scales, reinterpret_cast<float4 *>(out));
        count_launch();
    }
    if (nfull * kBlock < len) {
        const uint64_t rest = len - nfull * kBlock;
        const int grid = grid_for(rest, kThreads, 8);
        dequantize_generic_kernel<PACKED><<<grid, kThreads, 0, stream>>>(
            codes, len, nfull * kBlock, absmax, scale_codes, scale_of_scales, out);
        count_launch();
    }
    return check_cuda(cudaGetLastError(), "nf4_dequantize launch");
}

}  // namespace

int32_t quantize_packed(const float *values, uint64_t len, uint8_t *packed, float *absmax,
                        cudaStream_t stream) {
    return quantize_impl<true>(values, len, packed, absmax, stream);
}

int32_t quantize_unpacked(const float *values, uint64_t len, uint8_t *codes, float *absmax,
                          cudaStream_t stream) {
    return quantize_impl<false>(values, len, codes, absmax, stream);
}

int32_t dequantize_packed(const uint8_t *packed, uint64_t len, const float *absmax,
                          const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                          cudaStream_t stream) {
    return dequantize_impl<true>(packed, len, absmax, scale_codes, scale_of_scales, out, stream);
}

int32_t dequantize_unpacked(const uint8_t *codes, uint64_t len, const float *absmax,
                            const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                            cudaStream_t stream) {
    return dequantize_impl<false>(codes, len, absmax, scale_codes, scale_of_scales, out, stream);
}

int32_t quantize_transposed(const void *src, bool src_bf16, uint64_t rows, uint64_t cols,
                            uint8_t *packed, float *absmax, void *workspace, uint64_t workspace_bytes,
                            cudaStream_t stream) {
    if (rows == 0 || cols == 0) return NF4_OK;
    if (!src || !packed || !absmax) return fail(NF4_ERR_INVALID_ARG, "nf4_quantize_transposed: null pointer");
    const bool fused = rows % kTTile == 0 && cols % 4 == 0 && aligned16(src) &&
                       (reinterpret_cast<uintptr_t>(packed) & 3u) == 0;
    if (fused) {
        const uint64_t tiles = (rows / kTTile) * ((cols + kTTile - 1) / kTTile);
        if (tiles >= (1ull << 31)) return fail(NF4_ERR_UNSUPPORTED, "nf4_quantize_transposed: matrix too large");
        if (src_bf16)
            quantize_transposed_kernel<true><<<(unsigned)tiles, kThreads, 0, stream>>>(src, rows, cols, packed, absmax);
        else
            quantize_transposed_kernel<false><<<(unsigned)tiles, kThreads, 0, stream>>>(src, rows, cols, packed, absmax);
        count_launch();
        return check_cuda(cudaGetLastError(), "nf4_quantize_transposed launch");
    }
    // other shapes: transpose into the caller's workspace, then the flat quantizer
    const uint64_t need = rows * cols * sizeof(float);
    if (!workspace || workspace_bytes < need)
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_quantize_transposed: this shape needs a workspace of %llu bytes (rows %% 64 != 0)",
                    (unsigned long long)need);
    const uint64_t tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    if (tiles >= (1ull << 31)) return fail(NF4_ERR_UNSUPPORTED, "nf4_quantize_transposed: matrix too large");
    float *t = static_cast<float *>(workspace);
    if (src_bf16)
        transpose_to_f32_kernel<true><<<(unsigned)tiles, kThreads, 0, stream>>>(src, rows, cols, t);
    else
        transpose_to_f32_kernel<false><<<(unsigned)tiles, kThreads, 0, stream>>>(src, rows, cols, t);
    count_launch();
    NF4_CUDA_TRY(cudaGetLastError());
    return quantize_impl<true>(t, rows * cols, packed, absmax, stream);
}

int32_t embedding_gather(const uint8_t *packed, const float *absmax, const uint8_t *scale_codes,
                         const float *scale_of_scales, uint64_t n_embedding, uint64_t d_model,
                         const int64_t *ids, uint64_t n_ids, void *out, bool out_bf16,
                         cudaStream_t stream) {
    if (n_ids == 0 || d_model == 0) return NF4_OK;
    if (!packed || !ids || !out || (!absmax && !scale_codes))
        return fail(NF4_ERR_INVALID_ARG, "nf4_embedding_gather: null pointer");
    if (scale_codes && !scale_of_scales)
        return fail(NF4_ERR_INVALID_ARG, "nf4_embedding_gather: scale_codes without scale_of_scales");
    if ((d_model & 7u) == 0 && (!aligned16(out) || (reinterpret_cast<uintptr_t>(packed) & 3u)))
        return fail(NF4_ERR_INVALID_ARG, "nf4_embedding_gather: out must be 16-byte and packed 4-byte aligned");
    const uint64_t work = (d_model & 7u) == 0 ? n_ids * (d_model / 8) : n_ids * d_model;
    const int grid = grid_for(work, kThreads, 16);
    if (out_bf16)
        embedding_gather_kernel<true><<<grid, kThreads, 0, stream>>>(
            packed, absmax, scale_codes, scale_of_scales, n_embedding, d_model, ids, n_ids, out);
    else
        embedding_gather_kernel<false><<<grid, kThreads, 0, stream>>>(
            packed, absmax, scale_codes, scale_of_scales, n_embedding, d_model, ids, n_ids, out);
    count_launch();
    return check_cuda(cudaGetLastError(), "nf4_embedding_gather launch");
}

int32_t double_quantize(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                        float *scale_of_scales, cudaStream_t stream) {
    if (!scale_of_scales) return fail(NF4_ERR_INVALID_ARG, "nf4_double_quantize: null scale_of_scales");
    NF4_CUDA_TRY(cudaMemsetAsync(scale_of_scales, 0, sizeof(float), stream));
    if (nblocks == 0) return NF4_OK;
    if (!absmax || !scale_codes)
        return fail(NF4_ERR_INVALID_ARG, "nf4_double_quantize: null pointer");
    const int grid = grid_for(nblocks, kThreads * 4, 4);
    scale_max_kernel<<<grid, kThreads, 0, stream>>>(absmax, nblocks,
                                                    reinterpret_cast<uint32_t *>(scale_of_scales));
    scale_encode_kernel<<<grid_for(nblocks, kThreads, 8), kThreads, 0, stream>>>(
        absmax, nblocks, scale_of_scales, scale_codes);
    count_launch(2);
    return check_cuda(cudaGetLastError(), "nf4_double_quantize launch");
}

// ---- exhaustive self-check of the threshold bisection against the literal scan ----
// Walks `count` consecutive f32 bit patterns from `first_bits` and counts disagreements
// over the bisection's domain: NaNs and every value with |v| <= 65536.
__global__ void __launch_bounds__(kThreads)
selfcheck_codes_kernel(uint64_t first_bits, uint64_t count, unsigned long long *mismatches) {
    unsigned long long bad = 0;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < count; i += stride) {
        const uint32_t bits = (uint32_t)(first_bits + i);
        const uint32_t mag = bits & 0x7fffffffu;
        if (mag > 0x47800000u && mag <= 0x7f800000u) continue;  // 65536 < |v| <= inf
        const float v = __uint_as_float(bits);
        bad += code_of_normalized(v) != code_by_scan(v);
    }
    if (bad) atomicAdd(mismatches, bad);
}

// Same walk for the division-free fast path: every f32 x with |x| <= absmax (and NaNs), one
// given absmax, compared with the exact division + literal scan.
__global__ void __launch_bounds__(kThreads)
selfcheck_fast_kernel(uint64_t first_bits, uint64_t count, float absmax,
                      unsigned long long *mismatches) {
    __shared__ uint32_t s_cells[32];
    if (threadIdx.x < 32) s_cells[threadIdx.x] = c_cell_table[threadIdx.x];
    __syncthreads();
    const bool rcp_ok = absmax >= 1e-30f && absmax <= 1e30f;
    const float rcp = __fdiv_rn(1.0f, absmax);
    unsigned long long bad = 0;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < count; i += stride) {
        const float x = __uint_as_float((uint32_t)(first_bits + i));
        if (fabsf(x) > absmax) continue;  // cannot occur inside a block whose absmax this is
        const uint32_t exact = absmax == 0.0f ? 7u : code_by_scan(__fdiv_rn(x, absmax));
        bool unsure = !rcp_ok;
        uint32_t got = code_of_fast(x, rcp, s_cells, unsure);
        if (unsure) got = code_of_exact(x, absmax);
        bad += got != exact;
    }
    if (bad) atomicAdd(mismatches, bad);
}

int32_t selfcheck_fast(uint64_t first_bits, uint64_t count, float absmax,
                       unsigned long long *mismatches_dev, cudaStream_t stream) {
    selfcheck_fast_kernel<<<kNumSMs * 8, kThreads, 0, stream>>>(first_bits, count, absmax,
                                                               mismatches_dev);
    count_launch();
    return check_cuda(cudaGetLastError(), "selfcheck launch");
}

int32_t selfcheck_codes(uint64_t first_bits, uint64_t count, unsigned long long *mismatches_dev,
                        cudaStream_t stream) {
    selfcheck_codes_kernel<<<kNumSMs * 8, kThreads, 0, stream>>>(first_bits, count, mismatches_dev);
    count_launch();
    return check_cuda(cudaGetLastError(), "selfcheck launch");
}

}  // namespace nf4
