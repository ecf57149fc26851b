// The adapter by itself: LoraAdapter::forward, LoraAdapter::delta_weight and QLoraLinear::merged of
// the reference (src/quantize.rs:620-624, 629-634, 717-726), and the gather step of the
// column-sharded forward.  Small CUDA-core kernels: a rank-r product has r multiply-adds per
// output, so these are bound by the bytes of x, A, B and the output they touch.
//
// Arithmetic follows the reference's order in f32: (x A) first, then (.) B, the scale last;
// delta = (A B) * scale; merged = W + delta with W = level * block scale.
#include <cuda_bf16.h>
#include <dlfcn.h>

#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {
namespace {

template <class T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A(k, j) and B(j, n) in either orientation:
//   OUT_IN: A [r, d_in], B [d_out, r]      IN_OUT (the reference's): A [d_in, r], B [r, d_out]
template <class T>
__device__ __forceinline__ float a_at(const T *a, int32_t layout, uint64_t k, uint64_t j, uint64_t d_in, uint32_t rank) {
    return to_f32<T>(layout == NF4_LAYOUT_OUT_IN ? a[j * d_in + k] : a[k * rank + j]);
}
template <class T>
__device__ __forceinline__ float b_at(const T *b, int32_t layout, uint64_t j, uint64_t n, uint64_t d_out, uint32_t rank) {
    return to_f32<T>(layout == NF4_LAYOUT_OUT_IN ? b[n * rank + j] : b[j * d_out + n]);
}

// T[m][j] = sum_k x[m][k] * A(k, j); one warp per (m, j), lanes stride over k.
template <class T>
__global__ void __launch_bounds__(256)
lora_xa_kernel(const T *__restrict__ x, const T *__restrict__ a, float *__restrict__ t, uint64_t rows,
               uint64_t d_in, uint32_t rank, int32_t layout) {
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (warp >= rows * rank) return;
    const uint64_t m = warp / rank, j = warp % rank;
    float acc = 0.0f;
    for (uint64_t k = lane; k < d_in; k += 32) acc = fmaf(to_f32<T>(x[m * d_in + k]), a_at<T>(a, layout, k, j, d_in, rank), acc);
    #pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) t[m * rank + j] = acc;
}

// y[m][n] = (sum_j T[m][j] * B(j, n)) * scale; one thread per (m, n), n fastest.
template <class T>
__global__ void __launch_bounds__(256)
lora_tb_kernel(const float *__restrict__ t, const T *__restrict__ b, T *__restrict__ y, uint64_t rows,
               uint64_t d_out, uint64_t ldy, uint32_t rank, float scale, int32_t layout) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * d_out) return;
    const uint64_t m = i / d_out, n = i % d_out;
    float acc = 0.0f;
    for (uint32_t j = 0; j < rank; ++j) acc = fmaf(t[m * rank + j], b_at<T>(b, layout, j, n, d_out, rank), acc);
    y[m * ldy + n] = from_f32<T>(__fmul_rn(acc, scale));
}

// out(k, n) = [W(k, n) +] (sum_j A(k, j) * B(j, n)) * scale, stored in the weight's own orientation
// (flat index = k * d_out + n for IN_OUT, n * d_in + k for OUT_IN); one thread per element.
template <class T, bool MERGE>
__global__ void __launch_bounds__(256)
lora_delta_kernel(const T *__restrict__ a, const T *__restrict__ b, const uint8_t *__restrict__ packed,
                  const float *__restrict__ absmax, const uint8_t *__restrict__ scale_codes,
                  const float *__restrict__ scale_of_scales, float *__restrict__ out, uint64_t d_in,
                  uint64_t d_out, uint32_t rank, float scale, int32_t layout) {
    const uint64_t flat = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (flat >= d_in * d_out) return;
    const uint64_t k = layout == NF4_LAYOUT_OUT_IN ? flat % d_in : flat / d_out;
    const uint64_t n = layout == NF4_LAYOUT_OUT_IN ? flat / d_in : flat % d_out;
    float acc = 0.0f;
    for (uint32_t j = 0; j < rank; ++j)
        acc = fmaf(a_at<T>(a, layout, k, j, d_in, rank), b_at<T>(b, layout, j, n, d_out, rank), acc);
    float v = __fmul_rn(acc, scale);
    if (MERGE) {
        const uint32_t byte = __ldg(packed + (flat >> 1));
        const uint32_t code = (flat & 1u) ? (byte >> 4) : (byte & 15u);
        const uint64_t blk = flat / kBlock;
        const float s = absmax ? __ldg(absmax + blk) : dq_scale(__ldg(scale_codes + blk), __ldg(scale_of_scales));
        v = __fadd_rn(__fmul_rn(__uint_as_float(c_level_bits[code]), s), v);
    }
    out[flat] = v;
}

// The same T for a factor stored k-major (A(k, j) = a[k * rank + j]: the reference's A [d_in][r], or
// B [d_out][r] of the other orientation read as the factor of U = grad_y B^T), where the kernel above
// would read 32 sectors per load.  A CTA takes eight rows of x; x passes through shared memory in
// pieces of 256 k; warp w multiplies the k of its 32-wide part of the piece, eight k at a time with
// their factor rows loaded first; lanes own ranks (lane, lane + 32, ...: coalesced rows of the
// factor); the warps' sums meet in warp order.  KJ: ranks per lane and pass.
template <class T, int KJ>
__global__ void __launch_bounds__(256)
lora_xa_kmajor_kernel(const T *__restrict__ x, const T *__restrict__ a, float *__restrict__ t, uint64_t rows,
                      uint64_t d_in, uint32_t rank) {
    constexpr int kRows = 8, kPiece = 256, kStep = 8;
    __shared__ float xs[kRows][kPiece];
    __shared__ float red[8][kRows][32 * KJ + 1];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint64_t m0 = (uint64_t)blockIdx.x * kRows;
    for (uint32_t j0 = 0; j0 < rank; j0 += 32 * KJ) {
        float acc[kRows][KJ];
        #pragma unroll
        for (int m = 0; m < kRows; ++m)
            #pragma unroll
            for (int q = 0; q < KJ; ++q) acc[m][q] = 0.0f;
        for (uint64_t k0 = 0; k0 < d_in; k0 += kPiece) {
            __syncthreads();
            #pragma unroll
            for (int m = 0; m < kRows; ++m) {
                const uint64_t k = k0 + threadIdx.x;
                xs[m][threadIdx.x] = (m0 + m < rows && k < d_in) ? to_f32<T>(x[(m0 + m) * d_in + k]) : 0.0f;
            }
            __syncthreads();
            const uint64_t kw = k0 + warp * 32;
            #pragma unroll 1
            for (uint32_t kk = 0; kk < 32; kk += kStep) {
                float av[kStep][KJ];
                #pragma unroll
                for (int i = 0; i < kStep; ++i)
                    #pragma unroll
                    for (int q = 0; q < KJ; ++q) {
                        const uint32_t j = j0 + lane + 32 * q;
                        av[i][q] = (j < rank && kw + kk + i < d_in) ? to_f32<T>(a[(kw + kk + i) * rank + j]) : 0.0f;
                    }
                #pragma unroll
                for (int i = 0; i < kStep; ++i)
                    #pragma unroll
                    for (int m = 0; m < kRows; ++m) {
                        const float xv = xs[m][warp * 32 + kk + i];
                        #pragma unroll
                        for (int q = 0; q < KJ; ++q) acc[m][q] = fmaf(xv, av[i][q], acc[m][q]);
                    }
            }
        }
        __syncthreads();
        #pragma unroll
        for (int m = 0; m < kRows; ++m)
            #pragma unroll
            for (int q = 0; q < KJ; ++q) red[warp][m][lane + 32 * q] = acc[m][q];
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < kRows * 32 * KJ; i += 256) {
            const uint32_t m = i / (32 * KJ), jj = i % (32 * KJ);
            float v = 0.0f;
            #pragma unroll
            for (int w = 0; w < 8; ++w) v += red[w][m][jj];
            if (m0 + m < rows && j0 + jj < rank) t[(m0 + m) * rank + j0 + jj] = v;
        }
    }
}

// The adapter gradients: out(p, j) = scale * sum_m X[m][p] R[m][j] (X = x or grad_y in the io type,
// R = the f32 intermediate of the other factor).  A CTA takes 32 columns p and up to 64 ranks; X and R
// pass through shared memory in pieces of 128 rows m; the eight warps split the rows of a piece; a
// thread owns one p and all the ranks (64 accumulators), reads X[m][p] and R[m][.] (every lane the
// same address) from shared memory.  The warps' sums meet in warp order.  `p_major`: out is
// [P][rank] (else [rank][P]).
constexpr int kXtrP = 32, kXtrJ = 64, kXtrM = 128;
template <class T>
constexpr size_t xtr_smem_bytes() { return (size_t)kXtrM * kXtrJ * 4 + (size_t)kXtrM * kXtrP * sizeof(T); }

template <class T>
__global__ void __launch_bounds__(256)
lora_xtr_tile_kernel(const T *__restrict__ x, const float *__restrict__ r, T *__restrict__ out, uint64_t rows,
                     uint64_t P, uint32_t rank, float scale, int p_major) {
    constexpr int kP = kXtrP, kJ = kXtrJ, kM = kXtrM;
    extern __shared__ __align__(16) unsigned char xtr_smem[];
    float (*rs)[kJ] = reinterpret_cast<float(*)[kJ]>(xtr_smem);                     // 32 KB; afterwards the sums
    T (*xs)[kP] = reinterpret_cast<T(*)[kP]>(xtr_smem + (size_t)kM * kJ * 4);      // the piece of X
    const uint32_t pl = threadIdx.x & 31u, grp = threadIdx.x >> 5;
    const uint64_t p0 = (uint64_t)blockIdx.x * kP;
    for (uint32_t j0 = 0; j0 < rank; j0 += kJ) {
        float acc[kJ];
        #pragma unroll
        for (int j = 0; j < kJ; ++j) acc[j] = 0.0f;
        for (uint64_t m0 = 0; m0 < rows; m0 += kM) {
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < kM * kJ; i += 256) {
                const uint32_t m = i / kJ, j = i % kJ;
                rs[m][j] = (m0 + m < rows && j0 + j < rank) ? r[(m0 + m) * rank + j0 + j] : 0.0f;
            }
            for (uint32_t i = threadIdx.x; i < kM * kP; i += 256) {
                const uint32_t m = i / kP, q = i % kP;
                xs[m][q] = (m0 + m < rows && p0 + q < P) ? x[(m0 + m) * P + p0 + q] : from_f32<T>(0.0f);
            }
            __syncthreads();
            #pragma unroll 2
            for (uint32_t mm = 0; mm < kM / 8; ++mm) {
                const uint32_t m = grp * (kM / 8) + mm;
                const float xv = to_f32<T>(xs[m][pl]);
                #pragma unroll
                for (int j4 = 0; j4 < kJ / 4; ++j4) {
                    const float4 rv = *reinterpret_cast<const float4 *>(&rs[m][4 * j4]);
                    acc[4 * j4 + 0] = fmaf(xv, rv.x, acc[4 * j4 + 0]);
                    acc[4 * j4 + 1] = fmaf(xv, rv.y, acc[4 * j4 + 1]);
                    acc[4 * j4 + 2] = fmaf(xv, rv.z, acc[4 * j4 + 2]);
                    acc[4 * j4 + 3] = fmaf(xv, rv.w, acc[4 * j4 + 3]);
                }
            }
        }
        // the eight warps add up in turn through shared memory
        float (*sum)[kJ + 1] = reinterpret_cast<float(*)[kJ + 1]>(xtr_smem);
        for (uint32_t turn = 0; turn < 8; ++turn) {
            __syncthreads();
            if (grp == turn) {
                #pragma unroll
                for (int j = 0; j < kJ; ++j) sum[pl][j] = turn ? sum[pl][j] + acc[j] : acc[j];
            }
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < kP * kJ; i += 256) {
            // p fastest for [rank][P] outputs, j fastest for [P][rank]
            const uint32_t q = p_major ? i / kJ : i % kP, j = p_major ? i % kJ : i / kP;
            const uint64_t pp = p0 + q;
            if (pp < P && j0 + j < rank)
                out[p_major ? pp * rank + j0 + j : (uint64_t)(j0 + j) * P + pp] = from_f32<T>(__fmul_rn(sum[q][j], scale));
        }
    }
}

// The same gradients for bf16 tensors on warp MMAs: out(p, j) = scale * sum_m X[m][p] R[m][j] as
// D[p][j] += A[p][m] B[m][j] with m16n8k16.  A CTA takes 64 columns p and up to 64 ranks; pieces of
// 64 rows m pass through shared memory transposed (X as it is; R split into bf16 high and low parts,
// so that its f32 value survives: two MMAs per tile), which makes every fragment one 32-bit load;
// warp w takes the 16 columns (w & 3) and the two k-steps (w >> 2) of a piece; the two halves meet
// in a fixed order.  P must be even (pairs of columns are read as words).
__global__ void __launch_bounds__(256)
lora_xtr_mma_kernel(const __nv_bfloat16 *__restrict__ x, const float *__restrict__ r, __nv_bfloat16 *__restrict__ out,
                    uint64_t rows, uint64_t P, uint32_t rank, float scale, int p_major) {
    constexpr int kP = 64, kJ = 64, kM = 64, kS = 72;  // kS: halves per transposed row (fragment loads hit 32 banks)
    __shared__ __align__(16) uint16_t xs_t[kP][kS];
    __shared__ __align__(16) uint16_t rh[kJ][kS], rl[kJ][kS];
    __shared__ float sum[kP][kJ + 1];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t pt = warp & 3u, h = warp >> 2;
    const uint64_t p0 = (uint64_t)blockIdx.x * kP;
    const uint32_t lo = threadIdx.x & 31u, hi = threadIdx.x >> 5;  // staging: 8 columns x 4 rows per warp and step
    for (uint32_t j0 = 0; j0 < rank; j0 += kJ) {
        float acc[8][4];
        #pragma unroll
        for (int jt = 0; jt < 8; ++jt) acc[jt][0] = acc[jt][1] = acc[jt][2] = acc[jt][3] = 0.0f;
        for (uint64_t m0 = 0; m0 < rows; m0 += kM) {
            __syncthreads();
            #pragma unroll
            for (int it = 0; it < 8; ++it) {   // X: 64 rows x 32 pairs of columns
                const uint32_t hh = hi + 8 * it;  // 0 .. 63
                const uint32_t pair = (lo & 7u) + 8 * (hh & 3u), m = (lo >> 3) + 4 * (hh >> 2);
                uint32_t v = 0;
                if (m0 + m < rows && p0 + 2 * pair < P)
                    v = __ldg(reinterpret_cast<const uint32_t *>(x + (m0 + m) * P + p0 + 2 * pair));
                xs_t[2 * pair][m] = (uint16_t)(v & 0xffffu);
                xs_t[2 * pair + 1][m] = (uint16_t)(v >> 16);
            }
            #pragma unroll
            for (int it = 0; it < 16; ++it) {  // R: 64 rows x 64 ranks
                const uint32_t hh = hi + 8 * it;  // 0 .. 127
                const uint32_t j = (lo & 7u) + 8 * (hh & 7u), m = (lo >> 3) + 4 * (hh >> 3);
                float v = 0.0f;
                if (m0 + m < rows && j0 + j < rank) v = __ldg(r + (m0 + m) * rank + j0 + j);
                const __nv_bfloat16 vh = __float2bfloat16_rn(v);
                const __nv_bfloat16 vl = __float2bfloat16_rn(v - __bfloat162float(vh));
                rh[j][m] = __bfloat16_as_ushort(vh);
                rl[j][m] = __bfloat16_as_ushort(vl);
            }
            __syncthreads();
            #pragma unroll
            for (int ks2 = 0; ks2 < 2; ++ks2) {
                const uint32_t mb = (2 * h + ks2) * 16 + 2 * t;
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(&xs_t[pt * 16 + g][mb]);
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(&xs_t[pt * 16 + g + 8][mb]);
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(&xs_t[pt * 16 + g][mb + 8]);
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(&xs_t[pt * 16 + g + 8][mb + 8]);
                #pragma unroll
                for (int jt = 0; jt < 8; ++jt) {
                    const uint32_t bh0 = *reinterpret_cast<const uint32_t *>(&rh[jt * 8 + g][mb]);
                    const uint32_t bh1 = *reinterpret_cast<const uint32_t *>(&rh[jt * 8 + g][mb + 8]);
                    const uint32_t bl0 = *reinterpret_cast<const uint32_t *>(&rl[jt * 8 + g][mb]);
                    const uint32_t bl1 = *reinterpret_cast<const uint32_t *>(&rl[jt * 8 + g][mb + 8]);
                    ptx::mma_16816_bf16(acc[jt], a0, a1, a2, a3, bh0, bh1);
                    ptx::mma_16816_bf16(acc[jt], a0, a1, a2, a3, bl0, bl1);
                }
            }
        }
        // the two halves of the rows, in order
        for (uint32_t turn = 0; turn < 2; ++turn) {
            __syncthreads();
            if (h == turn) {
                #pragma unroll
                for (int jt = 0; jt < 8; ++jt) {
                    float *s0 = &sum[pt * 16 + g][jt * 8 + 2 * t], *s1 = &sum[pt * 16 + g + 8][jt * 8 + 2 * t];
                    s0[0] = turn ? s0[0] + acc[jt][0] : acc[jt][0];
                    s0[1] = turn ? s0[1] + acc[jt][1] : acc[jt][1];
                    s1[0] = turn ? s1[0] + acc[jt][2] : acc[jt][2];
                    s1[1] = turn ? s1[1] + acc[jt][3] : acc[jt][3];
                }
            }
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < kP * kJ; i += 256) {
            // p fastest for [rank][P] outputs, j fastest for [P][rank]
            const uint32_t q = p_major ? i / kJ : i % kP, j = p_major ? i % kJ : i / kP;
            const uint64_t pp = p0 + q;
            if (pp < P && j0 + j < rank)
                out[p_major ? pp * rank + j0 + j : (uint64_t)(j0 + j) * P + pp] = __float2bfloat16_rn(__fmul_rn(sum[q][j], scale));
        }
    }
}

// y[r][rank * width + c] = gathered[rank][r][c]: the ranks' slabs side by side.  16-byte pieces.
__global__ void __launch_bounds__(256)
place_slabs_kernel(const uint4 *__restrict__ gathered, uint4 *__restrict__ y, uint64_t rows, uint64_t pieces_per_row,
                   uint64_t ldy_pieces, uint32_t world) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t per_rank = rows * pieces_per_row;
    if (i >= per_rank * world) return;
    const uint64_t rk = i / per_rank, rem = i % per_rank, r = rem / pieces_per_row, c = rem % pieces_per_row;
    y[r * ldy_pieces + rk * pieces_per_row + c] = gathered[i];
}

// A rank's columns of its own output, pushed into the same columns of every other rank's output
// over NVLink: 16-byte pieces, plain loads from this GPU's memory and plain stores to the peers'
// (mapped into this process by the host).  A persistent grid walks the pieces; when a CTA is done
// it counts itself out on `done`, and the last one makes the launch's stores visible system-wide
// and, if asked, adds one to every rank's arrival counter (this rank's own included).
struct PushParams {
    const uint4 *src;        // this rank's output at its first column
    uint4 *dest[8];          // the ranks' outputs at the same column (own entry unused)
    uint32_t *arrive[8];
    uint32_t *done;          // a word of scratch, zero at first use, left zero
    uint64_t rows, pieces_per_row, ld_pieces;
    uint32_t world, rank, signal;
};

__global__ void __launch_bounds__(256) push_columns_kernel(const PushParams p) {
    const uint64_t total = p.rows * p.pieces_per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / p.pieces_per_row, c = i - r * p.pieces_per_row;
        const uint64_t at = r * p.ld_pieces + c;
        const uint4 v = __ldcg(p.src + at);
        for (uint32_t d = 0; d < p.world; ++d)
            if (d != p.rank) p.dest[d][at] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
            *p.done = 0;
            if (p.signal) {
                __threadfence_system();
                for (uint32_t d = 0; d < p.world; ++d) atomicAdd_system(p.arrive[d], 1u);
            }
        }
    }
}

// T = X F with the factor F(k, j) in either orientation
template <class T>
void launch_xa(const T *x, const T *f, float *t, uint64_t rows, uint64_t d_in, uint32_t rank, int32_t layout,
               cudaStream_t s) {
    if (layout == NF4_LAYOUT_OUT_IN)
        lora_xa_kernel<T><<<(unsigned)((rows * rank * 32 + 255) / 256), 256, 0, s>>>(x, f, t, rows, d_in, rank, layout);
    else if (rank <= 32)
        lora_xa_kmajor_kernel<T, 1><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(x, f, t, rows, d_in, rank);
    else
        lora_xa_kmajor_kernel<T, 2><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(x, f, t, rows, d_in, rank);
}

template <class T>
int32_t forward_t(const void *x, uint64_t rows, uint64_t d_in, uint64_t d_out, const void *a, const void *b,
                  uint32_t rank, float scale, int32_t layout, void *y, uint64_t ldy, float *t, cudaStream_t s) {
    launch_xa<T>(static_cast<const T *>(x), static_cast<const T *>(a), t, rows, d_in, rank, layout, s);
    lora_tb_kernel<T><<<(unsigned)((rows * d_out + 255) / 256), 256, 0, s>>>(
        t, static_cast<const T *>(b), static_cast<T *>(y), rows, d_out, ldy, rank, scale, layout);
    count_launch(2);
    return check_cuda(cudaGetLastError(), "lora forward launch");
}

template <class T>
int32_t grads_t(const void *x, const void *gy, const void *a, const void *b, uint64_t rows, uint64_t d_in,
                uint64_t d_out, uint32_t rank, float scale, int32_t layout, void *ga, void *gb, float *t,
                float *u, void *scratch, cudaStream_t s) {
    const T *xx = static_cast<const T *>(x), *gg = static_cast<const T *>(gy);
    // T = x A (as in the forward) and U = grad_y B^T (B read as an "A" of the other orientation).
    // bf16: on warp MMAs (products of bf16 values are exact in f32, so the sums differ from the
    // CUDA-core kernels' only in their order); shapes that path declines, and f32, on CUDA cores.
    const int32_t other = layout == NF4_LAYOUT_OUT_IN ? NF4_LAYOUT_IN_OUT : NF4_LAYOUT_OUT_IN;
    bool t_done = false, u_done = false;
    if (sizeof(T) == 2) {
        int32_t rc = adapter_intermediate_bf16(x, a, layout == NF4_LAYOUT_IN_OUT, rows, d_in, rank, t, scratch, s);
        if (rc == NF4_OK) t_done = true;
        else if (rc != NF4_ERR_UNSUPPORTED) return rc;
        rc = adapter_intermediate_bf16(gy, b, other == NF4_LAYOUT_IN_OUT, rows, d_out, rank, u, scratch, s);
        if (rc == NF4_OK) u_done = true;
        else if (rc != NF4_ERR_UNSUPPORTED) return rc;
    }
    if (!t_done) launch_xa<T>(xx, static_cast<const T *>(a), t, rows, d_in, rank, layout, s);
    if (!u_done) launch_xa<T>(gg, static_cast<const T *>(b), u, rows, d_out, rank, other, s);
    // grad_A(k, j) = s sum_m x[m][k] U[m][j];  grad_B(j, n) = s sum_m T[m][j] grad_y[m][n]
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(lora_xtr_tile_kernel<T>), (int)xtr_smem_bytes<T>()));
    auto xtr = [&](const void *X, const float *R, void *out, uint64_t P, int p_major) {
        if (sizeof(T) == 2 && P % 2 == 0 && (reinterpret_cast<uintptr_t>(X) & 3u) == 0)
            lora_xtr_mma_kernel<<<(unsigned)((P + 63) / 64), 256, 0, s>>>(
                static_cast<const __nv_bfloat16 *>(X), R, static_cast<__nv_bfloat16 *>(out), rows, P, rank, scale, p_major);
        else
            lora_xtr_tile_kernel<T><<<(unsigned)((P + kXtrP - 1) / kXtrP), 256, xtr_smem_bytes<T>(), s>>>(
                static_cast<const T *>(X), R, static_cast<T *>(out), rows, P, rank, scale, p_major);
    };
    xtr(x, u, ga, d_in, layout == NF4_LAYOUT_IN_OUT);
    xtr(gy, t, gb, d_out, layout == NF4_LAYOUT_OUT_IN);
    count_launch(4);
    return check_cuda(cudaGetLastError(), "lora gradient launch");
}

// ---- NCCL, looked up at run time: the library is not linked against it, so that hosts
// without NCCL can load everything else ----
typedef int (*AllGatherFn)(const void *, void *, size_t, int, void *, cudaStream_t);
typedef const char *(*ErrStrFn)(int);

AllGatherFn nccl_all_gather(ErrStrFn *err) {
    static AllGatherFn fn = nullptr;
    static ErrStrFn efn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = dlsym(RTLD_DEFAULT, "ncclAllGather");  // already loaded by the host (torch, a Rust binding)
        void *esym = dlsym(RTLD_DEFAULT, "ncclGetErrorString");
        if (!sym) {
            void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (h) {
                sym = dlsym(h, "ncclAllGather");
                esym = dlsym(h, "ncclGetErrorString");
            }
        }
        fn = reinterpret_cast<AllGatherFn>(sym);
        efn = reinterpret_cast<ErrStrFn>(esym);
    });
    *err = efn;
    return fn;
}

}  // namespace

uint64_t lora_workspace_bytes(uint64_t rows, uint32_t rank) { return (rows * rank * 4 + 255) / 256 * 256; }

int32_t lora_forward(const void *x, uint64_t rows, uint64_t d_in, uint64_t d_out, const void *a, const void *b,
                     uint32_t rank, float scale, int32_t layout, int32_t io_dtype, void *y, uint64_t ldy,
                     float *t, cudaStream_t s) {
    if (rows * rank >= (1ull << 40) || rows * d_out >= (1ull << 40))
        return fail(NF4_ERR_UNSUPPORTED, "nf4_lora_forward: shape too large");
    return io_dtype == NF4_DTYPE_F32
               ? forward_t<float>(x, rows, d_in, d_out, a, b, rank, scale, layout, y, ldy, t, s)
               : forward_t<__nv_bfloat16>(x, rows, d_in, d_out, a, b, rank, scale, layout, y, ldy, t, s);
}

// T[m][j] = sum_k x[m][k] A(k, j) alone (f32 out), for callers that finish the adapter term themselves
int32_t lora_intermediate(const void *x, const void *a, float *t, uint64_t rows, uint64_t d_in, uint32_t rank,
                          int32_t layout, int32_t io_dtype, cudaStream_t s) {
    if (io_dtype == NF4_DTYPE_F32)
        launch_xa<float>(static_cast<const float *>(x), static_cast<const float *>(a), t, rows, d_in, rank, layout, s);
    else
        launch_xa<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(a), t, rows,
                                 d_in, rank, layout, s);
    count_launch();
    return check_cuda(cudaGetLastError(), "lora intermediate launch");
}

int32_t lora_delta(const void *a, const void *b, const uint8_t *packed, const float *absmax,
                   const uint8_t *scale_codes, const float *scale_of_scales, uint64_t d_in, uint64_t d_out,
                   uint32_t rank, float scale, int32_t layout, int32_t io_dtype, float *out, cudaStream_t s) {
    const uint64_t n = d_in * d_out;
    if (n >= (1ull << 40)) return fail(NF4_ERR_UNSUPPORTED, "lora delta: shape too large");
    const unsigned grid = (unsigned)((n + 255) / 256);
    const bool merge = packed != nullptr;
    if (io_dtype == NF4_DTYPE_F32) {
        const float *fa = static_cast<const float *>(a), *fb = static_cast<const float *>(b);
        if (merge) lora_delta_kernel<float, true><<<grid, 256, 0, s>>>(fa, fb, packed, absmax, scale_codes, scale_of_scales, out, d_in, d_out, rank, scale, layout);
        else lora_delta_kernel<float, false><<<grid, 256, 0, s>>>(fa, fb, nullptr, nullptr, nullptr, nullptr, out, d_in, d_out, rank, scale, layout);
    } else {
        const __nv_bfloat16 *ha = static_cast<const __nv_bfloat16 *>(a), *hb = static_cast<const __nv_bfloat16 *>(b);
        if (merge) lora_delta_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(ha, hb, packed, absmax, scale_codes, scale_of_scales, out, d_in, d_out, rank, scale, layout);
        else lora_delta_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(ha, hb, nullptr, nullptr, nullptr, nullptr, out, d_in, d_out, rank, scale, layout);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "lora delta launch");
}

// grad_A and grad_B of y = x W + s (x A) B with W frozen; t and u are [rows][rank] f32 scratch,
// `scratch` rank * max(d_in, d_out) * 2 bytes (a factor transposed; used one product at a time).
int32_t lora_grads(const void *x, const void *gy, const void *a, const void *b, uint64_t rows, uint64_t d_in,
                   uint64_t d_out, uint32_t rank, float scale, int32_t layout, int32_t io_dtype, void *ga,
                   void *gb, float *t, float *u, void *scratch, cudaStream_t s) {
    if (rows * rank >= (1ull << 40) || (d_in + d_out) * rank >= (1ull << 40))
        return fail(NF4_ERR_UNSUPPORTED, "lora gradients: shape too large");
    return io_dtype == NF4_DTYPE_F32
               ? grads_t<float>(x, gy, a, b, rows, d_in, d_out, rank, scale, layout, ga, gb, t, u, scratch, s)
               : grads_t<__nv_bfloat16>(x, gy, a, b, rows, d_in, d_out, rank, scale, layout, ga, gb, t, u, scratch, s);
}

// All-gather of the ranks' [rows, width_bytes] slabs into `gathered` ([world][rows][width_bytes]),
// then the slabs side by side into y ([rows][ldy_bytes]).
int32_t gather_slabs(const void *slab, void *gathered, void *y, uint64_t rows, uint64_t width_bytes,
                     uint64_t ldy_bytes, void *comm, int32_t world, cudaStream_t s) {
    if (width_bytes % 16 != 0 || ldy_bytes % 16 != 0 ||
        ((reinterpret_cast<uintptr_t>(gathered) | reinterpret_cast<uintptr_t>(y)) & 15u))
        return fail(NF4_ERR_INVALID_ARG, "sharded forward: slab widths and buffers must be multiples of 16 bytes");
    ErrStrFn estr = nullptr;
    AllGatherFn ag = nccl_all_gather(&estr);
    if (!ag) return fail(NF4_ERR_UNSUPPORTED, "sharded forward: ncclAllGather not found (is NCCL loaded?)");
    const int rc = ag(slab, gathered, (size_t)(rows * width_bytes), /*ncclUint8*/ 1, comm, s);
    if (rc != 0) return fail(NF4_ERR_CUDA, "ncclAllGather failed: %s", estr ? estr(rc) : "unknown NCCL error");
    const uint64_t pieces = rows * (width_bytes / 16) * (uint64_t)world;
    place_slabs_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, s>>>(
        static_cast<const uint4 *>(gathered), static_cast<uint4 *>(y), rows, width_bytes / 16, ldy_bytes / 16,
        (uint32_t)world);
    count_launch();
    return check_cuda(cudaGetLastError(), "slab placement launch");
}

int32_t push_columns(void *const *y_full, uint32_t *const *arrive, uint32_t world, uint32_t rank, uint64_t rows,
                     uint64_t width_bytes, uint64_t ldy_bytes, bool signal, uint32_t *done, cudaStream_t s) {
    if (world == 0 || world > 8 || rank >= world) return fail(NF4_ERR_INVALID_ARG, "push_columns: world 1 ... 8, rank inside it");
    if (width_bytes == 0 || width_bytes % 16 != 0 || ldy_bytes % 16 != 0 || ldy_bytes < width_bytes * world)
        return fail(NF4_ERR_INVALID_ARG, "push_columns: the shard's width and the output's pitch must be multiples of 16 bytes");
    if (!done) return fail(NF4_ERR_INVALID_ARG, "push_columns: needs a word of scratch");
    PushParams p{};
    for (uint32_t d = 0; d < world; ++d) {
        if (!y_full[d] || (signal && !arrive[d]))
            return fail(NF4_ERR_INVALID_ARG, "push_columns: null output or counter of rank %u", d);
        uint8_t *base = static_cast<uint8_t *>(y_full[d]) + (size_t)rank * width_bytes;
        if (reinterpret_cast<uintptr_t>(base) & 15u) return fail(NF4_ERR_INVALID_ARG, "push_columns: outputs must be 16-byte aligned");
        p.dest[d] = reinterpret_cast<uint4 *>(base);
        p.arrive[d] = arrive[d];
    }
    p.src = p.dest[rank];
    p.done = done;
    p.rows = rows;
    p.pieces_per_row = width_bytes / 16;
    p.ld_pieces = ldy_bytes / 16;
    p.world = world;
    p.rank = rank;
    p.signal = signal ? 1u : 0u;
    if (rows == 0) return NF4_OK;
    const uint64_t pieces = rows * p.pieces_per_row;
    uint64_t ctas = (pieces + 255) / 256;
    if (ctas > (uint64_t)kNumSMs * 8) ctas = (uint64_t)kNumSMs * 8;
    push_columns_kernel<<<(unsigned)ctas, 256, 0, s>>>(p);
    count_launch();
    return check_cuda(cudaGetLastError(), "push_columns_kernel launch");
}

}  // namespace nf4
