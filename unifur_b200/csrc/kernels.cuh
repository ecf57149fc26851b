// Internal kernel-launcher interface between the C ABI (api.cu) and the kernel files.
#pragma once
#include "nf4_common.cuh"

namespace nf4 {

// Launch `kernel` so that it may start while its predecessor in `stream` is still running
// (programmatic dependent launch); the kernel must call ptx::pdl_wait() before it touches
// anything the predecessor writes.  Falls back to an ordinary launch when `overlap` is false.
template <class... KArgs, class... Args>
int32_t launch_maybe_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, bool overlap, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...), "kernel launch");
}
// api.cu: sets cudaFuncAttributeMaxDynamicSharedMemorySize for `kernel` on the current device,
// once per (kernel, device): the attribute belongs to the device a kernel is loaded on.
int32_t ensure_dynamic_smem(const void *kernel, int bytes);

// lora.cu: the adapter alone, its dense update, the merge, and the gather of column slabs
uint64_t lora_workspace_bytes(uint64_t rows, uint32_t rank);
int32_t lora_forward(const void *x, uint64_t rows, uint64_t d_in, uint64_t d_out, const void *a, const void *b,
                     uint32_t rank, float scale, int32_t layout, int32_t io_dtype, void *y, uint64_t ldy,
                     float *t, cudaStream_t s);
int32_t lora_intermediate(const void *x, const void *a, float *t, uint64_t rows, uint64_t d_in, uint32_t rank,
                          int32_t layout, int32_t io_dtype, cudaStream_t s);
int32_t lora_delta(const void *a, const void *b, const uint8_t *packed, const float *absmax,
                   const uint8_t *scale_codes, const float *scale_of_scales, uint64_t d_in, uint64_t d_out,
                   uint32_t rank, float scale, int32_t layout, int32_t io_dtype, float *out, cudaStream_t s);
int32_t lora_grads(const void *x, const void *gy, const void *a, const void *b, uint64_t rows, uint64_t d_in,
                   uint64_t d_out, uint32_t rank, float scale, int32_t layout, int32_t io_dtype, void *ga,
                   void *gb, float *t, float *u, void *scratch, cudaStream_t s);
int32_t push_columns(void *const *y_full, uint32_t *const *arrive, uint32_t world, uint32_t rank, uint64_t rows,
                     uint64_t width_bytes, uint64_t ldy_bytes, bool signal, uint32_t *done, cudaStream_t s);
int32_t gather_slabs(const void *slab, void *gathered, void *y, uint64_t rows, uint64_t width_bytes,
                     uint64_t ldy_bytes, void *comm, int32_t world, cudaStream_t s);

// quantize.cu
int32_t quantize_packed(const float *values, uint64_t len, uint8_t *packed, float *absmax,
                        cudaStream_t stream);
int32_t quantize_unpacked(const float *values, uint64_t len, uint8_t *codes, float *absmax,
                          cudaStream_t stream);
int32_t dequantize_packed(const uint8_t *packed, uint64_t len, const float *absmax,
                          const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                          cudaStream_t stream);
int32_t dequantize_unpacked(const uint8_t *codes, uint64_t len, const float *absmax,
                            const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                            cudaStream_t stream);
int32_t quantize_transposed(const void *src, bool src_bf16, uint64_t rows, uint64_t cols,
                            uint8_t *packed, float *absmax, void *workspace, uint64_t workspace_bytes,
                            cudaStream_t stream);
int32_t embedding_gather(const uint8_t *packed, const float *absmax, const uint8_t *scale_codes,
                         const float *scale_of_scales, uint64_t n_embedding, uint64_t d_model,
                         const int64_t *ids, uint64_t n_ids, void *out, bool out_bf16,
                         cudaStream_t stream);
int32_t double_quantize(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                        float *scale_of_scales, cudaStream_t stream);
int32_t selfcheck_fast(uint64_t first_bits, uint64_t count, float absmax,
                       unsigned long long *mismatches_dev, cudaStream_t stream);
int32_t selfcheck_codes(uint64_t first_bits, uint64_t count, unsigned long long *mismatches_dev,
                        cudaStream_t stream);

// decode_gemv.cu: rows <= 16, NF4_LAYOUT_OUT_IN, bf16 activations.
bool decode_supported(const nf4_linear_args &a);
uint64_t decode_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank);
// A kernel's failure code goes to its device flag and, where the host has given the kernel's file
// a word of mapped host memory (the host-pointer entry points do, so that they need no copy to
// look at it), to that word as well.
#define NF4_REPORT_FAILURE(flag, host_word, code)                          \
    do {                                                                   \
        atomicExch(&(flag), (code));                                       \
        if (host_word) *reinterpret_cast<volatile int *>(host_word) = (code); \
    } while (0)
int32_t decode_set_host_flag(int *mapped);
int32_t decode2_set_host_flag(int *mapped);
int32_t prefill_set_host_flag(int *mapped);

// api.cu: CTAs a kernel that puts one CTA on every SM may use (the SM count less nf4_reserve_sms)
uint32_t persistent_ctas();
int32_t decode_forward(const nf4_linear_args &a, cudaStream_t stream);
int32_t decode_forward_scatter(const nf4_linear_args &a, void *const *dest, uint32_t *const *arrive, uint32_t world,
                               uint32_t rank, uint64_t ldy, bool signal, uint32_t *wait_on, uint32_t wait_expected,
                               cudaStream_t stream);
int32_t decode_peer_wait(uint32_t *counter, uint32_t expected, uint32_t limit_ns, cudaStream_t stream);
int32_t decode_share_plan(uint32_t rows, uint32_t d_in, uint32_t d_out, uint32_t rank, uint32_t cta, uint32_t *out4);
int32_t decode_forward_grouped(const nf4_linear_args *a, uint32_t count, cudaStream_t stream, bool *taken);

int32_t decode_selftest_wait(uint32_t limit_ns, unsigned long long *waited_ns_dev, cudaStream_t stream);
// device addresses (current device) of the kernels' failure flags
int32_t decode_error_flag_ptr(int **dev_ptr);
int32_t decode2_error_flag_ptr(int **dev_ptr);
int32_t prefill_error_flag_ptr(int **dev_ptr);
uint64_t decode_static_scratch_bytes();
int32_t decode_forward_static_scratch(const nf4_linear_args &a, cudaStream_t stream);

// decode_umma.cu: rows <= 16 through tcgen05 (the fast decode path when its shape rules hold).
bool decode2_supported(const nf4_linear_args &a);
uint64_t decode2_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank);
int32_t decode2_forward(const nf4_linear_args &a, cudaStream_t stream);

// generic_linear.cu: any layout / dtype / shape on CUDA cores (exact f32 weights).
uint64_t generic_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank);
int32_t generic_forward(const nf4_linear_args &a, cudaStream_t stream);

// f32_rows.cu: f32 tensors, NF4_LAYOUT_OUT_IN, rows <= 16: rows split into bf16 halves for the decode kernels
bool f32_rows_supported(const nf4_linear_args &a);
uint64_t f32_rows_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank);
int32_t f32_rows_forward(const nf4_linear_args &a, cudaStream_t stream);

// prefill_gemm.cu: tcgen05 GEMM, NF4_LAYOUT_OUT_IN, bf16 activations.
bool prefill_supported(const nf4_linear_args &a);
// NF4_LAYOUT_IN_OUT at more than 16 rows, bf16 or f32 activations: repacked into the workspace, same GEMM
bool prefill_in_out_supported(const nf4_linear_args &a);
uint64_t prefill_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank);
int32_t prefill_share_plan(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t cta, uint32_t *ctas,
                           uint32_t *segments, uint32_t cap);
int32_t prefill_forward(const nf4_linear_args &a, cudaStream_t stream);
// t32[m][j] = sum_k x[m][k] F(k, j), bf16 operands on warp MMAs; NF4_ERR_UNSUPPORTED (no message) for shapes it declines
int32_t adapter_intermediate_bf16(const void *x, const void *f, bool k_major, uint64_t rows, uint64_t k, uint32_t rank,
                                  float *t32, void *scratch, cudaStream_t stream);

}  // namespace nf4
