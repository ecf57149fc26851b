/*
 * nf4_b200.h -- C ABI of the B200 (sm_100a) NF4 quantized-linear library.
 *
 * The reference crate (Rust, CPU) has no FFI today: its boundary is the Rust API of
 * `src/quantize.rs` and the NF4-resident modules of `src/qwennet.rs`.  Each entry
 * point below names the reference method whose body would call it (file:line within
 * the reference crate).  Plain pointers and sizes only; no exceptions, aborts or
 * device traps cross this boundary.
 *
 * Conventions
 *   - Every function returns an int32 status: 0 = NF4_OK, negative = failure.  The
 *     failing call's message is kept per host thread: nf4_last_error().
 *   - `*_dev` entry points take DEVICE pointers and enqueue on `stream`
 *     (a cudaStream_t passed as void*; NULL = the legacy default stream).  They never
 *     synchronise and never allocate.
 *   - `*_host` entry points take HOST pointers; they copy in, run the same kernels,
 *     copy out and return when the result is in the caller's buffer.
 *   - Device buffers must be 16-byte aligned (anything cudaMalloc returns is).
 *   - Read-only calls on one weight handle may run concurrently from several host
 *     threads (the reference moves modules across its block-executor threads,
 *     src/blockexec.rs:11-17); give each thread its own stream and workspace.
 */
#ifndef NF4_B200_H
#define NF4_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define NF4_API __attribute__((visibility("default")))
#else
#define NF4_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define NF4_BLOCK_SIZE 64 /* src/quantize.rs:37 */

/* status codes */
#define NF4_OK 0
#define NF4_ERR_INVALID_ARG (-1)
#define NF4_ERR_CUDA (-2)
#define NF4_ERR_OOM (-3)
#define NF4_ERR_UNSUPPORTED (-4)
#define NF4_ERR_TIMEOUT (-5)   /* a bounded device-side wait gave up */
#define NF4_ERR_NO_DEVICE (-6)

/* Weight orientation of a linear layer. */
#define NF4_LAYOUT_OUT_IN 0 /* W [d_out, d_in] row-major, quantized along d_in (the measured configs) */
#define NF4_LAYOUT_IN_OUT 1 /* W [d_in, d_out] row-major, flat 64-blocks: Burn's Linear (src/qwennet.rs:2196-2211) */

/* Element type of x, y and the LoRA factors. */
#define NF4_DTYPE_BF16 0
#define NF4_DTYPE_F32 1

/* ---------------------------------------------------------------- misc -- */

/* Library version (major*100 + minor). */
NF4_API int32_t nf4_version(void);

/* Message of the last failing call on this host thread ("" if none). */
NF4_API const char *nf4_last_error(void);

/* Number of kernels this library has launched in this process (all threads). */
NF4_API uint64_t nf4_kernel_launch_count(void);

/* Failure report of the tensor-core kernels.  Every device-side wait in them (on a TMA copy, on
 * another warp) is bounded: when one gives up, the kernel records a code in a per-device flag
 * and returns instead of hanging or trapping, and its output is void.  This call copies the
 * current device's three flags to the host (it synchronises with the device), clears them and
 * returns NF4_OK when all are zero, NF4_ERR_TIMEOUT when a wait gave up, NF4_ERR_CUDA when a
 * launch found its shared memory laid out differently from what it was built for.  The `*_host`
 * entry points make this check themselves before they return; callers of the `*_dev` entry
 * points make it where they synchronise.  Any pointer may be NULL.
 * The reference has no counterpart: its forward cannot fail (src/qwennet.rs:238-241); the
 * Rust shim maps a non-zero status to anyhow::Error (src/lib.rs:16-32). */
NF4_API int32_t nf4_device_status(int32_t *decode, int32_t *decode_split_k, int32_t *prefill);

/* Diagnostic: launches a one-thread kernel that waits on a barrier nobody signals, with the same
 * bounded wait the decode kernel uses and `limit_ns` (at most one second) as its limit.  The kernel
 * returns when the limit has passed and records the failure as the decode kernel would; the call
 * then reports it like any other: NF4_ERR_TIMEOUT, flags cleared.  `waited_ns` (may be NULL) gets
 * the time the wait took.  Nothing hangs, traps or faults; the device stays usable. */
NF4_API int32_t nf4_selftest_bounded_wait(uint64_t limit_ns, uint64_t *waited_ns);

/* Diagnostic: runs the kernels' threshold bisection and the reference's literal
 * sixteen-way scan (src/quantize.rs:208-219) on `count` consecutive f32 bit patterns
 * starting at `first_bits` (only NaNs and |v| <= 65536 are compared: a normalised value
 * never exceeds 1) and returns how many disagree. */
NF4_API int32_t nf4_selfcheck_code_selection(uint64_t first_bits, uint64_t count, uint64_t *mismatches);

/* Diagnostic: for one block scale `absmax`, runs the quantizer's division-free fast path and
 * the exact reference arithmetic (IEEE x / absmax, then the sixteen-way scan) on `count`
 * consecutive f32 bit patterns of x starting at `first_bits` (only |x| <= absmax and NaNs are
 * compared: nothing else can occur in a block with that absmax) and returns how many disagree. */
NF4_API int32_t nf4_selfcheck_quantize_fast_path(uint64_t first_bits, uint64_t count, float absmax,
                                         uint64_t *mismatches);

/* The sixteen NF4 levels, src/quantize.rs:49-66. */
NF4_API void nf4_levels(float out16[16]);

/* Byte accounting, src/quantize.rs:391-399 (PackedNf4Tensor::estimated_resident_bytes). */
NF4_API uint64_t nf4_estimated_resident_bytes(uint64_t len, int32_t double_quantized);
NF4_API uint64_t nf4_num_blocks(uint64_t len);
NF4_API uint64_t nf4_packed_bytes(uint64_t len);

/* ------------------------------------------------- quantize / dequantize -- */

/* Blockwise-absmax NF4 quantization of a flat f32 buffer into packed nibbles (two per
 * byte, low nibble first) and one f32 absmax per 64-block.
 * Replaces PackedNf4Tensor::quantize, src/quantize.rs:262-279 (codes from
 * Nf4Tensor::quantize, :99-124; nearest level, :208-219).
 *   values [len] f32, packed [ceil(len/2)] u8, absmax [ceil(len/64)] f32. */
NF4_API int32_t nf4_quantize_dev(const float *values, uint64_t len, uint8_t *packed, float *absmax,
                         void *stream);
NF4_API int32_t nf4_quantize_host(const float *values, uint64_t len, uint8_t *packed, float *absmax);

/* Same quantization, one code per byte (the simulated form): Nf4Tensor::quantize,
 * src/quantize.rs:99-124.  codes [len] u8. */
NF4_API int32_t nf4_quantize_unpacked_dev(const float *values, uint64_t len, uint8_t *codes,
                                  float *absmax, void *stream);

/* Second-level ("double") quantization of the block scales to 8 bits.
 * Replaces with_double_quantization, src/quantize.rs:129-149 and :284-309.
 *   scale_codes [nblocks] u8, scale_of_scales: one f32 (device memory for _dev). */
NF4_API int32_t nf4_double_quantize_dev(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                                float *scale_of_scales, void *stream);
NF4_API int32_t nf4_double_quantize_host(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                                 float *scale_of_scales);

/* Reconstruct f32 values: out[i] = level[code(i)] * block_scale(i / 64).
 * Replaces PackedNf4Tensor::dequantize, src/quantize.rs:355-366 (block_scale :341-351).
 * Exactly one scale form is given: `absmax` (f32 per block), or `scale_codes` +
 * `scale_of_scales` (double-quantized; `scale_of_scales` points at one f32). */
NF4_API int32_t nf4_dequantize_dev(const uint8_t *packed, uint64_t len, const float *absmax,
                           const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                           void *stream);
NF4_API int32_t nf4_dequantize_host(const uint8_t *packed, uint64_t len, const float *absmax,
                            const uint8_t *scale_codes, const float *scale_of_scales, float *out);

/* One code per byte variant: Nf4Tensor::dequantize, src/quantize.rs:178-185. */
NF4_API int32_t nf4_dequantize_unpacked_dev(const uint8_t *codes, uint64_t len, const float *absmax,
                                    const uint8_t *scale_codes, const float *scale_of_scales,
                                    float *out, void *stream);

/* Load path: packed NF4 of the TRANSPOSE of a checkpoint matrix, without materialising it.
 * `src` is [rows, cols] row-major in device memory (a PyTorch linear weight [out, in]; f32, or
 * bf16 as the reference's importer reads it, src/import.rs:9-12); the outputs are what
 * PackedNf4Tensor::quantize returns for the transposed buffer [cols, rows] flattened row-major --
 * the reference's transpose2d + quantize, src/qwennet.rs:1375-1390 and :1709-1711 -- bit for bit
 * (follow with nf4_double_quantize_dev as the reference does).  rows % 64 == 0 and cols % 4 == 0
 * run fused; other shapes go through `workspace` (nf4_quantize_transposed_workspace_bytes). */
NF4_API uint64_t nf4_quantize_transposed_workspace_bytes(uint64_t rows, uint64_t cols);
NF4_API int32_t nf4_quantize_transposed_dev(const void *src, int32_t src_dtype, uint64_t rows, uint64_t cols,
                                    uint8_t *packed, float *absmax, void *workspace,
                                    uint64_t workspace_bytes, void *stream);

/* Rows of a packed [n_embedding, d_model] table selected by `ids` (int64, device memory),
 * dequantized: out[t][j] = level[code] * block scale of element ids[t] * d_model + j, bit-exact
 * with dequantizing the whole table and gathering.  Replaces the body of Nf4Embedding::forward,
 * src/qwennet.rs:285-291, which rebuilds the whole f32 table on every call.  `out` is
 * [n_ids, d_model] of out_dtype (NF4_DTYPE_F32, or NF4_DTYPE_BF16 = the f32 value rounded once).
 * An id outside [0, n_embedding) gives a row of NaNs. */
NF4_API int32_t nf4_embedding_gather_dev(const uint8_t *packed, const float *absmax,
                                 const uint8_t *scale_codes, const float *scale_of_scales,
                                 uint64_t n_embedding, uint64_t d_model, const int64_t *ids,
                                 uint64_t n_ids, void *out, int32_t out_dtype, void *stream);

/* Quantize then reconstruct in place of a weight: the error a frozen NF4 weight carries.
 * Replaces quantize_dequantize_tensor, src/quantize.rs:404-416 (and the body of
 * Nf4Quantizer::map_float, :469-493).  `workspace` must hold
 * nf4_quantize_dequantize_workspace_bytes(len) bytes of device memory. */
NF4_API uint64_t nf4_quantize_dequantize_workspace_bytes(uint64_t len);
NF4_API int32_t nf4_quantize_dequantize_dev(const float *values, uint64_t len, int32_t double_quantization,
                                    float *out, void *workspace, uint64_t workspace_bytes,
                                    void *stream);
NF4_API int32_t nf4_quantize_dequantize_host(const float *values, uint64_t len,
                                     int32_t double_quantization, float *out);

/* ------------------------------------------------------- QLoRA forward -- */

/* Arguments of one NF4 / QLoRA linear forward
 *     y = x * dequant(W)^T (+ bias) (+ lora_scale * (x * A^T) * B^T).
 * Replaces Nf4Linear::forward, src/qwennet.rs:238-241, and QloraLinear::forward,
 * src/qwennet.rs:325-344 (adapter: LoraAdapter::forward, src/quantize.rs:620-624).
 * All pointers are device pointers.
 *
 * Arithmetic by shape.  NF4_LAYOUT_OUT_IN at any number of rows, and NF4_LAYOUT_IN_OUT at more than
 * 16 rows, with bf16 or f32 tensors (d_in a multiple of 64, for NF4_LAYOUT_IN_OUT d_out too; adapter
 * rank a multiple of 8 for bf16 and of 4 for f32 factors at more than 16 rows), multiply on the tensor
 * cores: f16 operands (activations per row and block scales per weight brought into f16's range by
 * powers of two; f32 activations of up to 16 rows enter as the bf16 high and low part of every row,
 * their adapter term is added in f32), f32 sums: relative L2 error <= 1e-3 against the reference's f32
 * result (measured: 4e-4).  Up to 16 rows of NF4_LAYOUT_IN_OUT (and up to 64 rows of its shapes the
 * tensor-core path does not take) and every other shape multiply exactly dequantized f32 weights
 * with f32 sums as the reference does: <= 1e-5. */
typedef struct nf4_linear_args {
    uint32_t struct_bytes;      /* sizeof(nf4_linear_args), checked */
    int32_t layout;             /* NF4_LAYOUT_* */
    int32_t io_dtype;           /* NF4_DTYPE_*: type of x, y, lora_a, lora_b */
    int32_t y_f32;              /* 0: y has io_dtype; 1: y is f32 whatever io_dtype is */
    uint64_t rows;              /* leading dims of x flattened (src/qwennet.rs:329) */
    uint64_t d_in;
    uint64_t d_out;
    const void *x;              /* [rows, d_in] */
    const uint8_t *packed;      /* ceil(d_in*d_out/2) bytes */
    const float *absmax;        /* f32 scales, or NULL when double-quantized */
    const uint8_t *scale_codes; /* u8 scales (double-quantized), or NULL */
    const float *scale_of_scales; /* one f32 in device memory, or NULL */
    const float *bias;          /* [d_out] f32, or NULL */
    const void *lora_a;         /* OUT_IN: [r, d_in];  IN_OUT: [d_in, r];  NULL = no adapter */
    const void *lora_b;         /* OUT_IN: [d_out, r]; IN_OUT: [r, d_out] */
    uint32_t lora_rank;
    float lora_scale;           /* (alpha / rank) as f32, applied last (src/quantize.rs:623) */
    void *y;                    /* [rows, ldy] */
    uint64_t ldy;               /* row stride of y in elements; 0 means d_out */
    void *workspace;            /* nf4_linear_workspace_bytes() bytes, 256-byte aligned; its first 256
                                   bytes must be zero at the first call that uses it (cudaMemset once
                                   after allocating); every call leaves them zero */
    uint64_t workspace_bytes;
} nf4_linear_args;

/* Scratch the forward needs for these sizes: the LoRA intermediate x*A^T behind 256 bytes of flag
 * words (the CTAs that compute x*A^T and the CTAs that read it meet on them; zero before the first
 * use, zero after every call), and for more than 16 rows the f16 copy of x with its per-row
 * power-of-two scales that the tensor-core kernel reads (plus a 128 x 256 f32 accumulator per SM
 * where it splits tiles between CTAs); for at most 16 rows also the partial sums of the parts of K
 * when d_in exceeds 4096, or, in the reference's weight orientation, of the pieces of K its kernel
 * works in; for more than 16 rows in that orientation the weight's nibbles transposed, its scales
 * as f16 and the adapter factors in the tensor-core kernel's orientation (about d_in * d_out / 2
 * bytes more; the value returned covers either orientation).  One workspace serves one stream: calls
 * that may overlap on the GPU need a workspace each. */
NF4_API uint64_t nf4_linear_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out,
                                    uint32_t lora_rank);

NF4_API int32_t nf4_linear_forward_dev(const nf4_linear_args *args, void *stream);

/* The adapter alone: y = ((x A) B) * lora_scale, the three operations in the reference's order,
 * f32 accumulation.  Replaces LoraAdapter::forward, src/quantize.rs:620-624.  Factor orientation
 * follows `layout` as in nf4_linear_args (NF4_LAYOUT_IN_OUT is the reference's A [d_in, r],
 * B [r, d_out]); x, y and the factors have `io_dtype`.  `workspace` holds
 * nf4_lora_workspace_bytes(rows, lora_rank) bytes (the intermediate x A in f32). */
NF4_API uint64_t nf4_lora_workspace_bytes(uint64_t rows, uint32_t lora_rank);
NF4_API int32_t nf4_lora_forward_dev(const void *x, uint64_t rows, uint64_t d_in, uint64_t d_out,
                                     const void *lora_a, const void *lora_b, uint32_t lora_rank,
                                     float lora_scale, int32_t layout, int32_t io_dtype, void *y, uint64_t ldy,
                                     void *workspace, uint64_t workspace_bytes, void *stream);

/* The dense update dW = (A B) * lora_scale as f32, stored in the weight's orientation
 * ([d_in, d_out] for NF4_LAYOUT_IN_OUT as the reference returns it, [d_out, d_in] for
 * NF4_LAYOUT_OUT_IN).  Replaces LoraAdapter::delta_weight, src/quantize.rs:629-634. */
NF4_API int32_t nf4_lora_delta_weight_dev(const void *lora_a, const void *lora_b, uint64_t d_in, uint64_t d_out,
                                          uint32_t lora_rank, float lora_scale, int32_t layout,
                                          int32_t io_dtype, float *out, void *stream);

/* The adapter folded into the quantized base weight: out = dequant(W) + (A B) * lora_scale, f32, in
 * the weight's orientation.  Replaces QLoraLinear::merged, src/quantize.rs:717-726 (which adds the
 * update to the dequantized base weight it holds).  Scales as in nf4_dequantize_dev. */
NF4_API int32_t nf4_qlora_merge_dev(const uint8_t *packed, const float *absmax, const uint8_t *scale_codes,
                                    const float *scale_of_scales, uint64_t d_in, uint64_t d_out, int32_t layout,
                                    const void *lora_a, const void *lora_b, uint32_t lora_rank,
                                    float lora_scale, int32_t io_dtype, float *out, void *stream);

/* Backward of the QLoRA linear with the base weight frozen, as the reference's autodiff sees the
 * detached NF4 weight (src/qwennet.rs:226-241; used by the training engine, src/qwentrain.rs:421-470).
 * `fwd` is the argument block of the forward being differentiated (x, the packed weight, the
 * adapter; y and bias are not read); `grad_y` is [rows, d_out].  Outputs, all of io_dtype:
 *   grad_x [rows, d_in]  = grad_y W^T + s (grad_y B^T) A^T   (one more NF4 linear over the same packed
 *                          bytes read in the other orientation),
 *   grad_a, grad_b with the shapes of lora_a, lora_b: s x^T (grad_y B^T) and s (x A)^T grad_y.
 * At more than 16 rows grad_x runs on the tensor cores (rel. L2 <= 1e-3 like that forward); with bf16
 * tensors the four rank-r products behind grad_a and grad_b run on warp MMAs with f32 sums (exact
 * products; the outputs are rounded to bf16 once), with f32 tensors on CUDA cores in f32.
 * fwd->workspace must hold nf4_qlora_backward_workspace_bytes() bytes, 256-byte aligned, its first 256
 * bytes zero at the first use like any forward workspace (every call leaves them zero). */
NF4_API uint64_t nf4_qlora_backward_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out,
                                                    uint32_t lora_rank);
NF4_API int32_t nf4_qlora_backward_dev(const nf4_linear_args *fwd, const void *grad_y, void *grad_x,
                                       void *grad_a, void *grad_b, void *stream);

/* One rank's part of a forward whose weight is sharded by output columns over `world` GPUs, and
 * the exchange that completes it.  `shard` describes this rank's slice exactly as for
 * nf4_linear_forward_dev: the rows of the packed weight, of the scales, of the bias and of LoRA B
 * that belong to its columns (every rank the same number of columns, d_out of the shard), x and
 * LoRA A whole, y = the rank's dense slab [rows, d_out].  After the local forward the slabs are
 * all-gathered into `gather_buffer` (nf4_sharded_gather_bytes) with ncclAllGather on `nccl_comm`
 * (an ncclComm_t; NCCL is looked up at run time in the host process, the library does not link it)
 * and placed side by side in y_full [rows, ldy_full] (0 = world * d_out), rank r's columns at
 * r * d_out.  Everything is enqueued on `stream`; every rank of the communicator must make the call.
 * The reference has no multi-GPU path: this is the partition its forward admits without touching
 * the arithmetic (src/qwennet.rs:238-241 computes each output column from one weight column). */
NF4_API uint64_t nf4_sharded_gather_bytes(uint64_t rows, uint64_t d_out_shard, int32_t world, int32_t io_dtype,
                                          int32_t y_f32);
NF4_API int32_t nf4_sharded_linear_forward_dev(const nf4_linear_args *shard, void *nccl_comm, int32_t rank,
                                               int32_t world, void *gather_buffer, uint64_t gather_bytes,
                                               void *y_full, uint64_t ldy_full, void *stream);

/* Several forwards of the same activations in one call: the projections a transformer block
 * applies to one input (q, k, v; gate, up).  The reference calls them one after another
 * (QwenLinear::forward per projection, src/qwennet.rs:372-383); the results are the same, bit for
 * bit, as `count` calls of nf4_linear_forward_dev with args[0] ... args[count - 1].
 * Where the arguments share x, rows, d_in and the form of the scales, rows <= 16 and every
 * forward fits the decode kernel (d_in <= 4096), they run as ONE kernel launch whose CTAs are
 * shared out in proportion to d_out; otherwise as `count` launches.  Every args[i] keeps its own
 * y, weights, adapter and workspace (the workspaces must not overlap).  count <= 4. */
NF4_API int32_t nf4_linear_forward_grouped_dev(const nf4_linear_args *args, uint32_t count, void *stream);

/* How the decode kernel (at most 16 rows) shares a forward out between its CTAs, computed on the
 * host: k0_k1_n0_n1 receives, for CTA `cta`, the range of k it multiplies and the rows of W it owns.
 * Returns the number of CTAs, or a negative status.  For inspection and tests. */
NF4_API int32_t nf4_decode_share_plan(uint32_t rows, uint32_t d_in, uint32_t d_out, uint32_t lora_rank, uint32_t cta,
                                      uint32_t *k0_k1_n0_n1);

/* How the tensor-core kernel (more than 16 rows) shares a forward's 128 x 256 tiles out between its
 * CTAs, computed on the host (no GPU needed): *ctas receives the number of CTAs; segments
 * receives, for CTA `cta`, up to `capacity` triples (tile, first main k-stage, one past the last)
 * in the order the CTA works on them.  Returns the number of the CTA's segments, or a negative
 * status.  Tiles that appear with a partial range of k-stages are split between neighbouring
 * CTAs (the one with the last stages finishes the tile).  For inspection and tests; the
 * reference has no counterpart. */
NF4_API int32_t nf4_prefill_share_plan(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t cta, uint32_t *ctas,
                                       uint32_t *segments, uint32_t capacity);

/* The decode kernel puts one CTA on every SM (it needs a whole SM's shared memory), so a kernel
 * that runs beside it on another stream -- a collective gathering the previous step's outputs --
 * holds back whole CTAs of it.  A host that overlaps such work tells the library to leave `count`
 * SMs free (0 ... 74, default 0; process-wide, takes effect with the next call); the forward's
 * results do not depend on it.  No counterpart in the reference (single device, no streams). */
NF4_API int32_t nf4_reserve_sms(int32_t count);

/* A column-sharded layer at decode sizes without a collective: every rank's kernel stores its
 * columns straight into every rank's output over NVLink (plain peer stores from the epilogue; no
 * gather buffer, no all-gather kernel, no copy).  The host maps each rank's output and arrival
 * counter into every process (CUDA IPC opened with the importing device current, or any other
 * peer mapping) and passes them here:
 *   y_full[r]   rank r's output [rows, ldy_full] (0 = world * d_out) as mapped into THIS process;
 *               this rank's columns start at rank * d_out in each of them,
 *   arrivals[r] rank r's 32-bit arrival counter, likewise (zero at first use).
 * `shard` describes this rank's slice as for nf4_sharded_linear_forward_dev (its y is ignored; its
 * workspace is needed, 256 bytes at least); rows <= 16 and a shape the decode kernel takes, up to
 * eight ranks (NF4_ERR_UNSUPPORTED otherwise).
 *   signal != 0: when the launch's last CTA is done it makes the stores of this launch -- and of
 *               the launches before it in the stream -- visible system-wide and adds ONE to
 *               every rank's counter.  A group of forwards into the same outputs signals with
 *               its last member.
 *   wait_arrivals / wait_expected: if non-NULL, this forward's x is the output of a sharded
 *               layer: before reading x every CTA waits (bounded; NF4_ERR_TIMEOUT shows in
 *               nf4_device_status) until wait_expected arrivals -- one per rank and signal --
 *               are on this rank's own counter, and the launch takes them off it.
 * nf4_peer_arrivals_wait_dev is the wait on its own, for consumers that are not this library's
 * kernels: a one-thread kernel that waits (at most timeout_ns) until `expected` arrivals are on
 * the counter and takes them off; kernels behind it in the stream see all columns.
 * A rank may run ahead of another by less than one wait: outputs that are still being read when
 * the next forwards are issued need a second buffer (and its own counter).
 * The reference has no multi-GPU path (see nf4_sharded_linear_forward_dev). */
typedef struct nf4_peer_outputs {
    uint32_t struct_bytes;      /* sizeof(nf4_peer_outputs) */
    int32_t world, rank;
    void *y_full[8];
    uint64_t ldy_full;
    uint32_t *arrivals[8];
    uint32_t signal;
    uint32_t wait_expected;
    uint32_t *wait_arrivals;
} nf4_peer_outputs;
NF4_API int32_t nf4_linear_forward_scatter_dev(const nf4_linear_args *shard, const nf4_peer_outputs *peers,
                                               void *stream);
/* The same exchange for forwards of any size (the tensor-core kernel's included): the rank's forward
 * writes its columns into its OWN output in place (y = y_full[rank] + rank * d_out, ldy = ldy_full
 * in nf4_linear_forward_dev), then this call pushes those columns -- rows x d_out_shard elements of
 * elem_bytes -- into the same place of every other rank's output with peer stores (one pass over
 * the shard; no gather buffer, no placing copy) and, with peers->signal, adds one arrival to every
 * rank's counter when all of it is out.  d_out_shard * elem_bytes and the pitch must be multiples of
 * 16 bytes.  scratch_word: four bytes of device memory, zero at first use, left zero. */
NF4_API int32_t nf4_peer_push_columns_dev(const nf4_peer_outputs *peers, uint64_t rows, uint64_t d_out_shard,
                                          int32_t elem_bytes, uint32_t *scratch_word, void *stream);
NF4_API int32_t nf4_peer_arrivals_wait_dev(uint32_t *own_arrivals, uint32_t expected, uint32_t timeout_ns,
                                           void *stream);

/* Decode-sized forward for callers that cannot allocate or own device memory.
 * No counterpart in the reference (its forward allocates a fresh f32 weight on every call).
 *
 * Some hosts of this library only ever receive device pointers: a plug-in running inside
 * another runtime's memory pool, a serving loop in a latency-critical section where cudaMalloc
 * would synchronise the whole device, or an FFI shim with no allocator of its own.  Such a
 * caller cannot supply the workspace nf4_linear_forward_dev asks for.  This entry point takes
 * the same arguments (args->workspace / workspace_bytes are ignored) and keeps its scratch --
 * the adapter intermediate x*A^T and two flag words -- in a fixed array inside the library's device
 * image, nf4_linear_noalloc_scratch_bytes() = 4352 bytes, which every GPU that loads the library
 * holds until the process exits.  It calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits: the decode shapes only (rows <= 16, bf16 x/y, NF4_LAYOUT_OUT_IN, d_in a multiple of 256
 * and <= 4096) with rows * lora_rank * 4 <= 4096 bytes (e.g. 16 rows at rank 64); anything
 * larger is refused with NF4_ERR_INVALID_ARG / NF4_ERR_UNSUPPORTED and a message.
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call outside any stream capture.
 * All calls on a device share the one array, which keeps whatever the last call left in it
 * (its flag words start at zero with the library's device image and every call puts them back
 * to zero; the intermediate is rewritten by each call before it is read: callers clear nothing).  Two calls whose
 * kernels overlap on the GPU -- different streams, no dependency -- race on it; order them. */
NF4_API uint64_t nf4_linear_noalloc_scratch_bytes(void);
NF4_API int32_t nf4_linear_forward_noalloc_dev(const nf4_linear_args *args, void *stream);

/* ------------------------------------------------ resident weight handles -- */

/* An NF4 weight resident in device memory (what Nf4Linear holds in `packed`,
 * src/qwennet.rs:168-178).  Immutable after creation; free with nf4_weight_free. */
typedef struct nf4_weight nf4_weight;

/* Quantize host f32 values on the device and keep the result resident.
 * Nf4Linear::from_values, src/qwennet.rs:198-205 (double_quantization = 1 there). */
NF4_API int32_t nf4_weight_from_values_host(const float *values, uint64_t d_in, uint64_t d_out,
                                    int32_t layout, int32_t double_quantization,
                                    nf4_weight **out);
/* Upload an already-packed weight.  Nf4Linear::from_packed, src/qwennet.rs:182-194. */
NF4_API int32_t nf4_weight_from_packed_host(const uint8_t *packed, const float *absmax,
                                    const uint8_t *scale_codes, float scale_of_scales,
                                    uint64_t d_in, uint64_t d_out, int32_t layout,
                                    nf4_weight **out);
NF4_API void nf4_weight_free(nf4_weight *w);
NF4_API uint64_t nf4_weight_resident_bytes(const nf4_weight *w); /* src/quantize.rs:370-376 */
/* Copy the packed bytes / scales back (PartialEq and dequantize() on the Rust side). */
NF4_API int32_t nf4_weight_download_host(const nf4_weight *w, uint8_t *packed, float *absmax,
                                 uint8_t *scale_codes, float *scale_of_scales);
/* Nf4Linear::dequantized_weight, src/qwennet.rs:230-236. */
NF4_API int32_t nf4_weight_dequantize_host(const nf4_weight *w, float *out);

/* Keep a LoRA adapter resident beside the weight (QwenLinear::with_lora,
 * src/qwennet.rs:419-434; QloraLinear holds `adapter` next to `base`, :318-322).  The
 * factors are copied to the device once; later forwards that pass lora_a == NULL use them.
 * Factor orientation follows the weight's layout; element type is `io_dtype`.
 * Attaching again replaces the adapter; rank 0 detaches it. */
NF4_API int32_t nf4_weight_attach_lora_host(nf4_weight *w, const void *lora_a, const void *lora_b,
                                    uint32_t lora_rank, float lora_scale, int32_t io_dtype);

/* Forward with host activations: x [rows, d_in] -> y [rows, d_out], element type
 * `io_dtype`.  `lora_a`/`lora_b` (host, may be NULL) use the layout's orientation; when they are NULL and
 * an adapter of the same element type is attached to the weight, that adapter is used.  Any host
 * memory serves; with up to 16 rows a page-locked y that the device can address (cudaHostAlloc, or
 * cudaHostRegister with the mapped flag) is written by the kernel itself, which saves the copy
 * back (a quarter of the call's latency at these sizes). */
NF4_API int32_t nf4_weight_linear_forward_host(const nf4_weight *w, const void *x, uint64_t rows,
                                       int32_t io_dtype, const float *bias, const void *lora_a,
                                       const void *lora_b, uint32_t lora_rank, float lora_scale,
                                       void *y);

#ifdef __cplusplus
}
#endif
#endif /* NF4_B200_H */
