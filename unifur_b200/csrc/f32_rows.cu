// f32 tensors at up to 16 rows with W [d_out, d_in] (the reference's tensor type on the measured
// layout): the decode kernels take bf16 activations, and rounding f32 activations to bf16 would cost
// 1e-3 by itself.  So each row is split into two bf16 rows, x = hi + lo (sixteen bits of mantissa
// between them), the decode kernel multiplies the 2 m rows with f32 outputs, and one more kernel
// adds the two halves, the bias and the adapter term s (x A^T) B^T, which is computed in f32 from
// the f32 factors as the reference does.  At most eight rows per pass (sixteen for the kernel).
#include <cuda_bf16.h>

#include "kernels.cuh"

namespace nf4 {
namespace {

__global__ void __launch_bounds__(256)
split_rows_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ xs, uint32_t m, uint64_t K) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)m * K) return;
    const float v = x[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    float rest = v - __bfloat162float(hi);
    if (!(fabsf(v) < 3.0e38f)) rest = 0.0f;  // infinities and NaNs travel in the high part alone
    xs[i] = hi;
    xs[(uint64_t)m * K + i] = __float2bfloat16_rn(rest);
}

// y[r][n] = yy[r][n] + yy[m + r][n] (+ bias[n]) (+ scale * sum_j t[r][j] * B[n][j])
__global__ void __launch_bounds__(256)
combine_rows_kernel(const float *__restrict__ yy, const float *__restrict__ bias, const float *__restrict__ t,
                    const float *__restrict__ b, float *__restrict__ y, uint32_t m, uint64_t N, uint64_t ldy,
                    uint32_t rank, float scale) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)m * N) return;
    const uint64_t r = i / N, n = i % N;
    float v = yy[i] + yy[(uint64_t)m * N + i];
    if (rank) {
        float acc = 0.0f;
        for (uint32_t j = 0; j < rank; ++j) acc = fmaf(t[r * rank + j], b[n * rank + j], acc);
        v += __fmul_rn(acc, scale);
    }
    if (bias) v += bias[n];
    y[r * ldy + n] = v;
}

inline uint64_t up256(uint64_t v) { return (v + 255) / 256 * 256; }

struct Scratch {
    uint64_t off_xs, off_yy, off_t, bytes;
};
Scratch scratch_layout(uint64_t d_in, uint64_t d_out, uint32_t rank) {
    Scratch s;
    const uint64_t a = decode_workspace_bytes(16, d_in, d_out, 0), b = decode2_workspace_bytes(16, d_in, d_out, 0);
    s.off_xs = up256(a > b ? a : b);
    if (s.off_xs < 256) s.off_xs = 256;
    s.off_yy = s.off_xs + up256(16 * d_in * 2);
    s.off_t = s.off_yy + up256(16 * d_out * 4);
    s.bytes = s.off_t + up256(16ull * rank * 4);
    return s;
}

// the bf16 call one pass makes: 2 m rows, f32 outputs, no bias, no adapter
nf4_linear_args halves_args(const nf4_linear_args &a, uint64_t m, const void *xs, void *yy) {
    nf4_linear_args h = a;
    h.io_dtype = NF4_DTYPE_BF16;
    h.y_f32 = 1;
    h.rows = 2 * m;
    h.x = xs;
    h.y = yy;
    h.ldy = a.d_out;
    h.bias = nullptr;
    h.lora_a = h.lora_b = nullptr;
    h.lora_rank = 0;
    h.lora_scale = 0.0f;
    return h;
}

}  // namespace

uint64_t f32_rows_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    if (rows == 0 || rows > 16) return 0;
    return scratch_layout(d_in, d_out, lora_rank).bytes;
}

bool f32_rows_supported(const nf4_linear_args &a) {
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_F32 || a.rows == 0 || a.rows > 16) return false;
    if (!a.workspace || (reinterpret_cast<uintptr_t>(a.workspace) & 255u)) return false;
    const Scratch sc = scratch_layout(a.d_in, a.d_out, a.lora_a ? a.lora_rank : 0);
    if (a.workspace_bytes < sc.bytes) return false;
    uint8_t *ws = static_cast<uint8_t *>(a.workspace);
    const nf4_linear_args h = halves_args(a, a.rows < 8 ? a.rows : 8, ws + sc.off_xs, ws + sc.off_yy);
    return decode_supported(h) || decode2_supported(h);
}

int32_t f32_rows_forward(const nf4_linear_args &a, cudaStream_t stream) {
    if (!f32_rows_supported(a)) return fail(NF4_ERR_UNSUPPORTED, "f32_rows_forward: unsupported shape");
    const uint32_t rank = a.lora_a ? a.lora_rank : 0;
    const Scratch sc = scratch_layout(a.d_in, a.d_out, rank);
    uint8_t *ws = static_cast<uint8_t *>(a.workspace);
    __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(ws + sc.off_xs);
    float *yy = reinterpret_cast<float *>(ws + sc.off_yy);
    float *t = reinterpret_cast<float *>(ws + sc.off_t);
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;
    const float *x = static_cast<const float *>(a.x);
    float *y = static_cast<float *>(a.y);
    if (rank)  // T = x A^T for all the rows, in f32
        NF4_TRY(lora_intermediate(a.x, a.lora_a, t, a.rows, a.d_in, rank, NF4_LAYOUT_OUT_IN, NF4_DTYPE_F32, stream));
    for (uint64_t r0 = 0; r0 < a.rows; r0 += 8) {
        const uint32_t m = (uint32_t)(a.rows - r0 < 8 ? a.rows - r0 : 8);
        split_rows_kernel<<<(unsigned)((m * a.d_in + 255) / 256), 256, 0, stream>>>(x + r0 * a.d_in, xs, m, a.d_in);
        count_launch();
        NF4_CUDA_TRY(cudaGetLastError());
        nf4_linear_args h = halves_args(a, m, xs, yy);
        h.workspace_bytes = sc.off_xs;
        if (decode_supported(h)) NF4_TRY(decode_forward(h, stream));
        else NF4_TRY(decode2_forward(h, stream));
        combine_rows_kernel<<<(unsigned)((m * a.d_out + 255) / 256), 256, 0, stream>>>(
            yy, a.bias, t + r0 * rank, static_cast<const float *>(a.lora_b), y + r0 * ldy, m, a.d_out, ldy, rank,
            a.lora_scale);
        count_launch();
        NF4_CUDA_TRY(cudaGetLastError());
    }
    return NF4_OK;
}

}  // namespace nf4
