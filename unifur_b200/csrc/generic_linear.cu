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

uint64_t generic_workspace_bytes(uint64_t rows, uint32_t lora_rank) {
    return (rows * lora_rank * 4 + 255) / 256 * 256;
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
    p.t = static_cast<float *>(a.workspace);
    p.rows = a.rows;
    p.d_in = a.d_in;
    p.d_out = a.d_out;
    p.ldy = a.ldy ? a.ldy : a.d_out;
    p.rank = a.lora_a ? a.lora_rank : 0;
    p.lora_scale = a.lora_scale;
    p.layout = a.layout;
    p.y_f32 = a.y_f32;
    return a.io_dtype == NF4_DTYPE_F32 ? run<float>(p, stream) : run<__nv_bfloat16>(p, stream);
}

}  // namespace nf4
