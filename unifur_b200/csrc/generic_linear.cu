// General-shape NF4 / QLoRA linear forward on CUDA cores.
//
// Covers every combination the tuned kernels do not: both weight orientations
// (including the reference's [d_in, d_out] layout whose 64-blocks run along the flat
// index and may straddle rows), f32 or bf16 activations, double-quantized scales, any
// d_in / d_out / rows / rank.  Weights are dequantized exactly as the reference does
// (one f32 multiply of level and block scale) and accumulated in f32.
#include <cuda_bf16.h>

#include "kernels.cuh"

namespace nf4 {
namespace {

constexpr int kRowsPerPass = 8;

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

struct GenericParams {
    const void *x, *lora_a, *lora_b;
    void *y;
    const uint8_t *packed;
    const float *absmax;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const float *bias;
    float *t;  // [rows][rank]
    uint32_t *counters;  // rows kernel: one byte per column strip (zero at first use, left zero)
    float *partial;      // rows kernel: [k-parts][rows][d_out] f32
    uint32_t k_parts, k_chunk;  // rows kernel: K is cut into k_parts pieces of k_chunk rows of W
    uint64_t rows, d_in, d_out, ldy;
    uint32_t rank;
    float lora_scale;
    int32_t layout;
    int32_t y_f32;
};

__device__ __forceinline__ float weight_at(const GenericParams &p, uint64_t flat, float sos) {
    const uint32_t byte = __ldg(p.packed + (flat >> 1));
    const uint32_t code = (flat & 1u) ? (byte >> 4) : (byte & 15u);
    const uint64_t blk = flat / kBlock;
    const float scale = p.absmax ? __ldg(p.absmax + blk) : dq_scale(__ldg(p.scale_codes + blk), sos);
    return __fmul_rn(__uint_as_float(c_level_bits[code]), scale);
}

// T[m][j] = sum_k x[m][k] * A(k, j); one warp per (m, j).
template <class T>
__global__ void __launch_bounds__(256) generic_lora_t_kernel(const GenericParams p) {
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (warp >= p.rows * p.rank) return;
    const uint64_t m = warp / p.rank, j = warp % p.rank;
    const T *x = static_cast<const T *>(p.x) + m * p.d_in;
    const T *a = static_cast<const T *>(p.lora_a);
    float acc = 0.0f;
    for (uint64_t k = lane; k < p.d_in; k += 32) {
        const float av = to_f32<T>(p.layout == NF4_LAYOUT_OUT_IN ? a[j * p.d_in + k] : a[k * p.rank + j]);
        acc = fmaf(to_f32<T>(x[k]), av, acc);
    }
    #pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) p.t[m * p.rank + j] = acc;
}

// The same with a CTA per (m, j) for the few rows of the strip kernel (a warp per (m, j) leaves
// most SMs idle there and walks all of K in 128 dependent steps): eight warps share K, four loads
// in flight per lane, the warps' sums are added in warp order.
template <class T>
__global__ void __launch_bounds__(256) lora_t_cta_kernel(const GenericParams p) {
    __shared__ float part[8];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint64_t m = blockIdx.x / p.rank, j = blockIdx.x % p.rank;
    const T *x = static_cast<const T *>(p.x) + m * p.d_in;
    const T *a = static_cast<const T *>(p.lora_a);
    const bool out_in = p.layout == NF4_LAYOUT_OUT_IN;
    float acc = 0.0f;
    #pragma unroll 4
    for (uint64_t k = threadIdx.x; k < p.d_in; k += 256)
        acc = fmaf(to_f32<T>(x[k]), to_f32<T>(out_in ? a[j * p.d_in + k] : a[k * p.rank + j]), acc);
    #pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = 0.0f;
        #pragma unroll
        for (int w = 0; w < 8; ++w) v += part[w];
        p.t[m * p.rank + j] = v;
    }
}

template <class T>
__device__ __forceinline__ void finish(const GenericParams &p, uint64_t m, uint64_t n, float acc) {
    if (p.rank) {
        const T *b = static_cast<const T *>(p.lora_b);
        float dot = 0.0f;
        for (uint32_t j = 0; j < p.rank; ++j) {
            const float bv = to_f32<T>(p.layout == NF4_LAYOUT_OUT_IN ? b[n * p.rank + j] : b[(uint64_t)j * p.d_out + n]);
            dot = fmaf(p.t[m * p.rank + j], bv, dot);
        }
        acc = fmaf(dot, p.lora_scale, acc);
    }
    if (p.bias) acc += __ldg(p.bias + n);
    if (p.y_f32) static_cast<float *>(p.y)[m * p.ldy + n] = acc;
    else static_cast<T *>(p.y)[m * p.ldy + n] = from_f32<T>(acc);
}

// W [d_out, d_in]: one warp per output column n, lanes stride over k (coalesced nibbles).
template <class T>
__global__ void __launch_bounds__(256) generic_out_in_kernel(const GenericParams p) {
    const uint64_t n = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (n >= p.d_out) return;
    const float sos = p.scale_of_scales ? __ldg(p.scale_of_scales) : 0.0f;
    const T *x = static_cast<const T *>(p.x);
    for (uint64_t m0 = 0; m0 < p.rows; m0 += kRowsPerPass) {
        float acc[kRowsPerPass];
        #pragma unroll
        for (int i = 0; i < kRowsPerPass; ++i) acc[i] = 0.0f;
        for (uint64_t k = lane; k < p.d_in; k += 32) {
            const float w = weight_at(p, n * p.d_in + k, sos);
            #pragma unroll
            for (int i = 0; i < kRowsPerPass; ++i)
                if (m0 + i < p.rows) acc[i] = fmaf(to_f32<T>(x[(m0 + i) * p.d_in + k]), w, acc[i]);
        }
        #pragma unroll
        for (int i = 0; i < kRowsPerPass; ++i) {
            float v = acc[i];
            #pragma unroll
            for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
            if (lane == 0 && m0 + i < p.rows) finish<T>(p, m0 + i, n, v);
        }
    }
}

// W [d_in, d_out]: one thread per output column n (consecutive lanes read consecutive
// nibbles of one weight row), serial over k.
template <class T>
__global__ void __launch_bounds__(128) generic_in_out_kernel(const GenericParams p) {
    const uint64_t n = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= p.d_out) return;
    const float sos = p.scale_of_scales ? __ldg(p.scale_of_scales) : 0.0f;
    const T *x = static_cast<const T *>(p.x);
    for (uint64_t m0 = (uint64_t)blockIdx.y * kRowsPerPass; m0 < p.rows;
         m0 += (uint64_t)gridDim.y * kRowsPerPass) {
        float acc[kRowsPerPass];
        #pragma unroll
        for (int i = 0; i < kRowsPerPass; ++i) acc[i] = 0.0f;
        for (uint64_t k = 0; k < p.d_in; ++k) {
            const float w = weight_at(p, k * p.d_out + n, sos);
            #pragma unroll
            for (int i = 0; i < kRowsPerPass; ++i)
                if (m0 + i < p.rows) acc[i] = fmaf(to_f32<T>(x[(m0 + i) * p.d_in + k]), w, acc[i]);
        }
        #pragma unroll
        for (int i = 0; i < kRowsPerPass; ++i)
            if (m0 + i < p.rows) finish<T>(p, m0 + i, n, acc[i]);
    }
}

// ---- W [d_in, d_out] with d_out a multiple of 64, up to eight activation rows -----------------
// The reference's own orientation (src/qwennet.rs:230-241: linear(x, W[d_in, d_out]); the 64-blocks
// run along d_out) at decode sizes, on CUDA cores with the reference's arithmetic: every weight is
// level * block scale in f32, products accumulate in f32.
// A CTA owns a strip of 256 columns and a piece of K; its eight warps take the rows of W of that
// piece in turn.  For a row of W a lane reads its eight consecutive codes (one 32-bit load: a warp
// reads 128 contiguous bytes) and the block's scale, looks each byte's two levels up in a per-lane
// copy of a 256-entry table in shared memory (one byte permute forms the address, one 64-bit
// load brings both), and multiplies them with the (up to eight) activations of that k, which sit
// in shared memory.  The warps' sums meet in shared memory in warp order; where K is
// cut into pieces, the pieces meet in global memory and the CTA that arrives last for a strip adds
// them in the order of the pieces (bit-reproducible), then bias, adapter term and the store.
constexpr int kStripCols = 256;
constexpr int kRowsWarps = 8;

template <class T, int MR, bool DQ>
__global__ void __launch_bounds__(256, MR >= 4 ? 2 : 3) in_out_rows_kernel(const GenericParams p) {
    extern __shared__ __align__(16) float dyn[];
    __shared__ uint32_t last_s;
    // [256 byte values][32 lanes] pairs {level of the low nibble, level of the high nibble}
    float2 *lut = reinterpret_cast<float2 *>(dyn);
    float *xs = dyn + 256 * 32 * 2;                   // [k_chunk][MR]
    float *red = xs + (size_t)MR * p.k_chunk;         // [MR][8][32]: column 8 * lane + i at [i][lane]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t strip = blockIdx.x, part = blockIdx.y;
    const uint64_t k_begin = (uint64_t)part * p.k_chunk;
    const uint64_t k_end = k_begin + p.k_chunk < p.d_in ? k_begin + p.k_chunk : p.d_in;
    const uint32_t kc = (uint32_t)(k_end - k_begin);
    const float sos = p.scale_of_scales ? __ldg(p.scale_of_scales) : 0.0f;
    {
        const float2 entry = make_float2(__uint_as_float(c_level_bits[tid & 15u]), __uint_as_float(c_level_bits[tid >> 4]));
        #pragma unroll 8
        for (uint32_t l = 0; l < 32; ++l) lut[tid * 32u + ((l + tid) & 31u)] = entry;  // rotated: the stores spread over the banks
    }
    const T *x = static_cast<const T *>(p.x);
    for (uint32_t i = tid; i < MR * p.k_chunk; i += 256) {
        const uint32_t m = i / p.k_chunk, kk = i - m * p.k_chunk;  // consecutive threads read consecutive k
        xs[kk * MR + m] = (m < p.rows && kk < kc) ? to_f32<T>(x[(uint64_t)m * p.d_in + k_begin + kk]) : 0.0f;
    }
    __syncthreads();

    const uint64_t n = (uint64_t)strip * kStripCols + lane * 8u;
    const bool active = n < p.d_out;
    const uint64_t blocks_per_row = p.d_out / kBlock;
    float acc[MR][8];
    #pragma unroll
    for (int m = 0; m < MR; ++m)
        #pragma unroll
        for (int i = 0; i < 8; ++i) acc[m][i] = 0.0f;
    if (active) {
        // A ring of D rows of W per lane in registers: a row is multiplied, then the load of the
        // row D places on takes its slot.  With one activation row the kernel lives on bytes in
        // flight (24 warps x 12 rows x 144 B per SM).  Rows are walked with running pointers: the
        // warp's rows are eight apart.
        constexpr uint32_t D = MR <= 2 ? 12 : (MR == 4 ? 8 : 4);
        const uint32_t my_rows = kc > warp ? (kc - warp + kRowsWarps - 1) / kRowsWarps : 0u;
        // rows of W are addressed as base + row number * pitch (one wide multiply-add each); the
        // table and the activations through 32-bit shared-memory addresses
        const uint32_t *code_base = reinterpret_cast<const uint32_t *>(p.packed + (n >> 1) + (k_begin + warp) * (p.d_out >> 1));
        const uint32_t code_pitch = (uint32_t)(kRowsWarps * (p.d_out >> 3));         // 32-bit words between this warp's rows
        const uint32_t scale_pitch = (uint32_t)(kRowsWarps * blocks_per_row);
        const float *abs_base = DQ ? nullptr : p.absmax + (k_begin + warp) * blocks_per_row + (n >> 6);
        const uint8_t *sc_base = DQ ? p.scale_codes + (k_begin + warp) * blocks_per_row + (n >> 6) : nullptr;
        uint32_t lut_lane;
        asm("{ .reg .u64 t; cvta.to.shared.u64 t, %1; cvt.u32.u64 %0, t; }" : "=r"(lut_lane) : "l"(lut));
        lut_lane += lane * 8u;
        const float *x_ptr = xs + warp * MR;
        uint32_t codes[D];
        float scale[D];
        uint32_t fetched = 0;  // rows asked for so far
        auto fetch = [&](uint32_t slot) {
            const bool in = fetched < my_rows;
            codes[slot] = in ? __ldg(code_base + (size_t)fetched * code_pitch) : 0u;
            if (DQ) scale[slot] = in ? dq_scale(__ldg(sc_base + (size_t)fetched * scale_pitch), sos) : 0.0f;
            else scale[slot] = in ? __ldg(abs_base + (size_t)fetched * scale_pitch) : 0.0f;
            ++fetched;
        };
        auto multiply = [&](uint32_t slot) {
            float w[8];
            #pragma unroll
            for (int b = 0; b < 4; ++b) {
                // byte b of the codes times 256 plus this lane's place in the entry: the pair's address
                const uint32_t at = __byte_perm(codes[slot], 0u, 0x4404u | ((uint32_t)b << 4)) + lut_lane;
                float lo, hi;
                asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(lo), "=f"(hi) : "r"(at));
                w[2 * b] = __fmul_rn(lo, scale[slot]);
                w[2 * b + 1] = __fmul_rn(hi, scale[slot]);
            }
            #pragma unroll
            for (int m = 0; m < MR; ++m) {
                const float xv = x_ptr[m];
                #pragma unroll
                for (int i = 0; i < 8; ++i) acc[m][i] = fmaf(xv, w[i], acc[m][i]);
            }
            x_ptr += kRowsWarps * MR;
        };
        #pragma unroll
        for (uint32_t d = 0; d < D; ++d) fetch(d);
        uint32_t done = 0;
        #pragma unroll 1
        for (; done + D <= my_rows; done += D) {  // whole turns of the ring: no checks on the rows multiplied
            #pragma unroll
            for (uint32_t d = 0; d < D; ++d) {
                multiply(d);
                fetch(d);
            }
        }
        #pragma unroll
        for (uint32_t d = 0; d < D; ++d)
            if (done + d < my_rows) multiply(d);
    }
    // the warps' sums, in warp order
    for (uint32_t w = 0; w < (uint32_t)kRowsWarps; ++w) {
        if (warp == w) {
            #pragma unroll
            for (int m = 0; m < MR; ++m)
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float *cell = red + (m * 8 + i) * 32 + lane;
                    *cell = w == 0 ? acc[m][i] : *cell + acc[m][i];
                }
        }
        __syncthreads();
    }
    // thread `tid` finishes column strip * 256 + tid
    const uint64_t col = (uint64_t)strip * kStripCols + tid;
    const uint32_t cell = (tid & 7u) * 32u + (tid >> 3);
    if (p.k_parts == 1) {
        if (col < p.d_out)
            for (uint32_t m = 0; m < (uint32_t)MR && m < p.rows; ++m) finish<T>(p, m, col, red[m * 256 + cell]);
        return;
    }
    if (col < p.d_out)
        for (uint32_t m = 0; m < (uint32_t)MR && m < p.rows; ++m)
            p.partial[((uint64_t)part * p.rows + m) * p.d_out + col] = red[m * 256 + cell];
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const uint32_t sh = (strip & 3u) * 8u;
        uint32_t *counter = p.counters + (strip >> 2);
        const uint32_t old = (atomicAdd(counter, 1u << sh) >> sh) & 0xffu;
        if (old == p.k_parts - 1) atomicSub(counter, p.k_parts << sh);
        last_s = old == p.k_parts - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (last_s && col < p.d_out) {
        __threadfence();
        // eight pieces of every row at a time: the loads are in flight together, the additions
        // keep the order of the pieces
        float v[MR];
        #pragma unroll
        for (int m = 0; m < MR; ++m) v[m] = 0.0f;
        for (uint32_t q0 = 0; q0 < p.k_parts; q0 += 8) {
            float part[MR][8];
            #pragma unroll
            for (int m = 0; m < MR; ++m)
                #pragma unroll
                for (int u = 0; u < 8; ++u)
                    part[m][u] = ((uint32_t)m < p.rows && q0 + u < p.k_parts)
                                     ? __ldcg(p.partial + ((uint64_t)(q0 + u) * p.rows + m) * p.d_out + col)
                                     : 0.0f;
            #pragma unroll
            for (int m = 0; m < MR; ++m)
                #pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (q0 + u < p.k_parts) v[m] += part[m][u];
        }
        #pragma unroll
        for (int m = 0; m < MR; ++m)
            if ((uint32_t)m < p.rows) finish<T>(p, m, col, v[m]);
    }
}

// strips and pieces of K for the rows kernel: about four CTAs per SM
struct RowsPlan {
    uint32_t strips, k_parts, k_chunk;
};
bool rows_plan(uint64_t d_in, uint64_t d_out, uint64_t rows, RowsPlan &rp) {
    if (d_out % kBlock != 0 || d_in == 0 || d_in >= (1ull << 31) || d_out >= (1ull << 31)) return false;
    rp.strips = (uint32_t)((d_out + kStripCols - 1) / kStripCols);
    if (rp.strips > 248) return false;  // a byte counter per strip in the workspace's 62 counter words
    // three CTAs per SM (64 KB of table each; two where a launch carries more than two activation
    // rows: their slices of x and the registers of eight rows leave no room for a third), and no
    // more CTAs than fit at once: a second, partly filled round would double the time
    const uint64_t per_sm = rows >= 3 ? 2 : 3;
    uint64_t parts = per_sm * kNumSMs / rp.strips;
    if (parts == 0) parts = 1;
    const uint64_t most = d_in / 64 ? d_in / 64 : 1;  // a piece keeps 64 rows of W at least
    if (parts > most) parts = most;
    if (parts > 255) parts = 255;
    rp.k_chunk = (uint32_t)((d_in + parts - 1) / parts);
    if (rp.k_chunk > 1024) rp.k_chunk = 1024;  // the activations of a piece live in shared memory
    rp.k_parts = (uint32_t)((d_in + rp.k_chunk - 1) / rp.k_chunk);
    return rp.k_parts <= 255;
}

template <class T, int MR, bool DQ>
int32_t launch_rows_as(const GenericParams &p, const RowsPlan &rp, cudaStream_t stream) {
    const size_t smem = (256 * 32 * 2 + (size_t)MR * rp.k_chunk + (size_t)MR * 256) * sizeof(float);
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(in_out_rows_kernel<T, MR, DQ>), (int)smem));
    in_out_rows_kernel<T, MR, DQ><<<dim3(rp.strips, rp.k_parts), 256, smem, stream>>>(p);
    count_launch();
    return check_cuda(cudaGetLastError(), "in_out_rows_kernel launch");
}

template <class T, int MR>
int32_t launch_rows(const GenericParams &p, const RowsPlan &rp, cudaStream_t stream) {
    return p.absmax ? launch_rows_as<T, MR, false>(p, rp, stream) : launch_rows_as<T, MR, true>(p, rp, stream);
}

template <class T>
int32_t run_rows(GenericParams p, const RowsPlan &rp, cudaStream_t stream) {
    if (p.rank) {
        lora_t_cta_kernel<T><<<(unsigned)(p.rows * p.rank), 256, 0, stream>>>(p);
        count_launch();
        NF4_CUDA_TRY(cudaGetLastError());
    }
    p.k_parts = rp.k_parts;
    p.k_chunk = rp.k_chunk;
    // eight activation rows per launch; x, y and T move on with them
    const uint64_t rows = p.rows;
    const size_t esz = sizeof(T);
    for (uint64_t m0 = 0; m0 < rows; m0 += 8) {
        GenericParams q = p;
        q.rows = rows - m0 < 8 ? rows - m0 : 8;
        q.x = static_cast<const uint8_t *>(p.x) + m0 * p.d_in * esz;
        q.y = static_cast<uint8_t *>(p.y) + m0 * p.ldy * (p.y_f32 ? 4 : esz);
        q.t = p.t + m0 * p.rank;
        if (q.rows == 1) NF4_TRY((launch_rows<T, 1>(q, rp, stream)));
        else if (q.rows == 2) NF4_TRY((launch_rows<T, 2>(q, rp, stream)));
        else if (q.rows <= 4) NF4_TRY((launch_rows<T, 4>(q, rp, stream)));
        else NF4_TRY((launch_rows<T, 8>(q, rp, stream)));
    }
    return NF4_OK;
}

template <class T>
int32_t run(const GenericParams &p, cudaStream_t stream) {
    if (p.rank) {
        const uint64_t warps = p.rows * p.rank;
        generic_lora_t_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(p);
        count_launch();
    }
    if (p.layout == NF4_LAYOUT_OUT_IN) {
        generic_out_in_kernel<T><<<(unsigned)((p.d_out * 32 + 255) / 256), 256, 0, stream>>>(p);
    } else {
        uint64_t my = (p.rows + kRowsPerPass - 1) / kRowsPerPass;
        if (my > 65535) my = 65535;
        generic_in_out_kernel<T><<<dim3((unsigned)((p.d_out + 127) / 128), (unsigned)my), 128, 0, stream>>>(p);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "generic linear launch");
}

}  // namespace

namespace {
constexpr uint64_t kCounterBytes = 256;
constexpr uint64_t kRowsKernelMaxRows = 64;
uint64_t t_bytes(uint64_t rows, uint32_t lora_rank) { return (rows * lora_rank * 4 + 255) / 256 * 256; }
}  // namespace

// counters | T | the pieces' sums of the rows kernel (which may serve either orientation's caller)
uint64_t generic_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    uint64_t need = lora_rank ? kCounterBytes + t_bytes(rows, lora_rank) : 0;
    RowsPlan rp;
    if (rows <= kRowsKernelMaxRows && rows_plan(d_in, d_out, rows, rp) && rp.k_parts > 1)
        need = kCounterBytes + t_bytes(rows, lora_rank) + (uint64_t)rp.k_parts * (rows < 8 ? rows : 8) * d_out * 4;
    return need;
}

int32_t generic_forward(const nf4_linear_args &a, cudaStream_t stream) {
    if (a.d_out * 32 / 256 >= (1ull << 31) || a.rows * (a.lora_a ? a.lora_rank : 0) >= (1ull << 40))
        return fail(NF4_ERR_UNSUPPORTED, "generic_forward: shape too large");
    GenericParams p{};
    p.x = a.x;
    p.lora_a = a.lora_a;
    p.lora_b = a.lora_b;
    p.y = a.y;
    p.packed = a.packed;
    p.absmax = a.absmax;
    p.scale_codes = a.scale_codes;
    p.scale_of_scales = a.scale_of_scales;
    p.bias = a.bias;
    p.counters = static_cast<uint32_t *>(a.workspace);
    p.t = reinterpret_cast<float *>(static_cast<uint8_t *>(a.workspace) + kCounterBytes);
    p.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(a.workspace) + kCounterBytes +
                                          t_bytes(a.rows, a.lora_a ? a.lora_rank : 0));
    p.rows = a.rows;
    p.d_in = a.d_in;
    p.d_out = a.d_out;
    p.ldy = a.ldy ? a.ldy : a.d_out;
    p.rank = a.lora_a ? a.lora_rank : 0;
    p.lora_scale = a.lora_scale;
    p.layout = a.layout;
    p.y_f32 = a.y_f32;
    RowsPlan rp;
    if (a.layout == NF4_LAYOUT_IN_OUT && a.rows <= kRowsKernelMaxRows && rows_plan(a.d_in, a.d_out, a.rows, rp) &&
        (reinterpret_cast<uintptr_t>(a.packed) & 3u) == 0 && (rp.k_parts == 1 || a.workspace))
        return a.io_dtype == NF4_DTYPE_F32 ? run_rows<float>(p, rp, stream) : run_rows<__nv_bfloat16>(p, rp, stream);
    return a.io_dtype == NF4_DTYPE_F32 ? run<float>(p, stream) : run<__nv_bfloat16>(p, stream);
}

}  // namespace nf4
