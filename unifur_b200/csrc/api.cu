// C ABI of the NF4 B200 library: argument checks, error reporting, host-pointer
// wrappers and resident weight handles.  Kernels live in the other .cu files.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "kernels.cuh"

namespace nf4 {

namespace {
thread_local std::string t_last_error;
std::atomic<uint64_t> g_launches{0};
}  // namespace

int32_t fail(int32_t code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return code;
}

int32_t check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return NF4_OK;
    const int32_t code = (e == cudaErrorMemoryAllocation) ? NF4_ERR_OOM
                         : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
                             ? NF4_ERR_NO_DEVICE
                             : NF4_ERR_CUDA;
    return fail(code, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int32_t ensure_dynamic_smem(const void *kernel, int bytes) {
    struct Done {
        const void *kernel;
        int device;
    };
    static std::mutex mu;
    static Done done[256];
    static int n_done = 0;
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_done; ++i)
        if (done[i].kernel == kernel && done[i].device == dev) return NF4_OK;
    NF4_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (n_done < 256) done[n_done++] = Done{kernel, dev};
    return NF4_OK;
}

void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

// Grow-only device scratch owned by one host thread; the host-pointer entry points
// stage through it so repeated calls do not pay cudaMalloc/cudaFree.
struct Arena {
    void *ptr = nullptr;
    size_t cap = 0;
    int device = -1;
    int32_t reserve(size_t bytes) {
        int dev = 0;
        NF4_CUDA_TRY(cudaGetDevice(&dev));
        if (ptr && dev == device && cap >= bytes) return NF4_OK;
        if (ptr) {
            cudaFree(ptr);
            ptr = nullptr;
            cap = 0;
        }
        size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
        NF4_CUDA_TRY(cudaMalloc(&ptr, want));
        cap = want;
        device = dev;
        return NF4_OK;
    }
    ~Arena() {
        // The CUDA context may already be gone at thread exit; ignore the result.
        if (ptr) cudaFree(ptr);
    }
};
thread_local Arena t_arena;

// A small zero-filled device buffer per host thread and device: the decode kernel's workspace
// (flag words that must be zero at first use and are left zero, then the adapter intermediate).
struct ZeroScratch {
    static constexpr size_t kMaxBytes = 16u << 20;  // larger workspaces are zeroed per call instead
    void *ptr = nullptr;
    size_t cap = 0;
    int device = -1;
    // `need` bytes whose first 256 are zero (the decode kernels leave them zero); grows when asked for more
    int32_t get(void **out, size_t need) {
        int dev = 0;
        NF4_CUDA_TRY(cudaGetDevice(&dev));
        if (!ptr || dev != device || need > cap) {
            if (ptr) cudaFree(ptr);
            ptr = nullptr;
            cap = need > 8192 ? align_up_pow2(need) : 8192;
            NF4_CUDA_TRY(cudaMalloc(&ptr, cap));
            NF4_CUDA_TRY(cudaMemset(ptr, 0, 8192));
            device = dev;
        }
        *out = ptr;
        return NF4_OK;
    }
    static size_t align_up_pow2(size_t v) {
        size_t p = 8192;
        while (p < v) p <<= 1;
        return p;
    }
    ~ZeroScratch() {
        if (ptr) cudaFree(ptr);
    }
};
thread_local ZeroScratch t_zero_scratch;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Carves aligned sub-buffers out of the arena.
struct Carver {
    uint8_t *base;
    size_t off = 0;
    explicit Carver(void *p) : base(static_cast<uint8_t *>(p)) {}
    template <class T>
    T *take(size_t count) {
        off = align_up(off, 256);
        T *p = reinterpret_cast<T *>(base + off);
        off += count * sizeof(T);
        return p;
    }
};

// ---- device-side failure flags ----------------------------------------------------
// Device addresses of the three kernels' flags, looked up once per device.
int32_t flag_ptrs(int **out3) {
    static std::mutex mu;
    static int *cache[64][3] = {};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NF4_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev][0]) {
        int *p0 = nullptr, *p1 = nullptr, *p2 = nullptr;
        NF4_TRY(decode_error_flag_ptr(&p0));
        NF4_TRY(decode2_error_flag_ptr(&p1));
        NF4_TRY(prefill_error_flag_ptr(&p2));
        cache[dev][1] = p1;
        cache[dev][2] = p2;
        cache[dev][0] = p0;
    }
    for (int i = 0; i < 3; ++i) out3[i] = cache[dev][i];
    return NF4_OK;
}

// Turns flag values already on the host into a status; flags that were set are cleared.
int32_t report_flags(int *const *ptrs, const int *v) {
    for (int i = 0; i < 3; ++i)
        if (v[i]) NF4_CUDA_TRY(cudaMemset(ptrs[i], 0, sizeof(int)));
    if (v[0] == 4)
        return fail(NF4_ERR_CUDA, "decode kernel: dynamic shared memory does not start where the kernel "
                                  "expects it; the launch produced no output");
    if (v[0] || v[1] || v[2])
        return fail(NF4_ERR_TIMEOUT, "a bounded device-side wait gave up (decode %d, decode split-K %d, "
                                     "prefill %d): the outputs of the calls since the last check are void",
                    v[0], v[1], v[2]);
    return NF4_OK;
}

// Three words of mapped host memory per device that the kernels' failure codes are written to
// as well as to the device flags: the host-pointer entry points look at them after their final
// synchronise, without a copy.  Set up at the first such call on a device.
int32_t host_flag_words(volatile int **out) {
    static std::mutex mu;
    static int *words[64] = {};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NF4_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        int *h = nullptr, *d = nullptr;
        NF4_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void **>(&h), 3 * sizeof(int), cudaHostAllocMapped));
        h[0] = h[1] = h[2] = 0;
        NF4_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&d), h, 0));
        NF4_TRY(decode_set_host_flag(d));
        NF4_TRY(decode2_set_host_flag(d + 1));
        NF4_TRY(prefill_set_host_flag(d + 2));
        words[dev] = h;
    }
    *out = words[dev];
    return NF4_OK;
}

// The host-pointer entry points work on the calling thread's own stream, so that calls from
// several host threads (each with its own staging arena) do not serialise on the default stream.
#define kHostStream cudaStreamPerThread

inline size_t dtype_bytes(int32_t dt) { return dt == NF4_DTYPE_F32 ? 4 : 2; }

int32_t validate_linear(const nf4_linear_args *a, bool needs_workspace = true) {
    if (!a) return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: null args");
    if (a->struct_bytes != sizeof(nf4_linear_args))
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: struct_bytes %u != %zu",
                    a->struct_bytes, sizeof(nf4_linear_args));
    if (a->layout != NF4_LAYOUT_OUT_IN && a->layout != NF4_LAYOUT_IN_OUT)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: bad layout %d", a->layout);
    if (a->io_dtype != NF4_DTYPE_BF16 && a->io_dtype != NF4_DTYPE_F32)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: bad io_dtype %d", a->io_dtype);
    if (a->y_f32 != 0 && a->y_f32 != 1)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: y_f32 must be 0 or 1");
    if (a->d_in == 0 || a->d_out == 0)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: zero d_in/d_out");
    if (a->rows && (!a->x || !a->y)) return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: null x/y");
    if (!a->packed) return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: null packed weight");
    if ((a->absmax != nullptr) == (a->scale_codes != nullptr))
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_linear_forward: give either absmax or scale_codes+scale_of_scales");
    if (a->scale_codes && !a->scale_of_scales)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: scale_codes without scale_of_scales");
    if ((a->lora_a != nullptr) != (a->lora_b != nullptr))
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: lora_a and lora_b go together");
    if (a->lora_a && a->lora_rank == 0)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: adapter with rank 0");
    if (a->ldy != 0 && a->ldy < a->d_out)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: ldy < d_out");
    const uint64_t need = nf4_linear_workspace_bytes(a->rows, a->d_in, a->d_out,
                                                     a->lora_a ? a->lora_rank : 0);
    if (!needs_workspace) return NF4_OK;
    if (need && (!a->workspace || a->workspace_bytes < need))
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: workspace %llu < %llu bytes",
                    (unsigned long long)a->workspace_bytes, (unsigned long long)need);
    if (need && (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward: workspace not 256-byte aligned");
    return NF4_OK;
}

}  // namespace
}  // namespace nf4

using namespace nf4;

struct nf4_weight {
    uint64_t d_in = 0, d_out = 0, len = 0, nblocks = 0;
    int32_t layout = 0;
    int device = 0;
    bool double_quantized = false;
    uint8_t *packed = nullptr;
    float *absmax = nullptr;
    uint8_t *scale_codes = nullptr;
    float *scale_of_scales = nullptr;  // one f32, device
    // resident adapter (optional)
    void *lora_a = nullptr, *lora_b = nullptr;
    uint32_t lora_rank = 0;
    float lora_scale = 0.0f;
    int32_t lora_dtype = 0;
};

// A weight lives on the device that was current when it was created: its kernels must be
// launched there.
static int32_t check_weight_device(const nf4_weight *w, const char *who) {
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device)
        return fail(NF4_ERR_INVALID_ARG, "%s: the weight lives on device %d, the current device is %d", who,
                    w->device, dev);
    return NF4_OK;
}

extern "C" {

int32_t nf4_version(void) { return 200; }

const char *nf4_last_error(void) { return t_last_error.c_str(); }

uint64_t nf4_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void nf4_levels(float out16[16]) { std::memcpy(out16, h_level_bits, sizeof(h_level_bits)); }

int32_t nf4_selfcheck_code_selection(uint64_t first_bits, uint64_t count, uint64_t *mismatches) {
    if (!mismatches) return fail(NF4_ERR_INVALID_ARG, "nf4_selfcheck_code_selection: null pointer");
    NF4_TRY(t_arena.reserve(256));
    unsigned long long *d = static_cast<unsigned long long *>(t_arena.ptr);
    NF4_CUDA_TRY(cudaMemsetAsync(d, 0, 8, 0));
    NF4_TRY(selfcheck_codes(first_bits, count, d, 0));
    unsigned long long h = 0;
    NF4_CUDA_TRY(cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost));
    *mismatches = h;
    return NF4_OK;
}

int32_t nf4_selfcheck_quantize_fast_path(uint64_t first_bits, uint64_t count, float absmax,
                                         uint64_t *mismatches) {
    if (!mismatches) return fail(NF4_ERR_INVALID_ARG, "nf4_selfcheck_quantize_fast_path: null pointer");
    NF4_TRY(t_arena.reserve(256));
    unsigned long long *d = static_cast<unsigned long long *>(t_arena.ptr);
    NF4_CUDA_TRY(cudaMemsetAsync(d, 0, 8, 0));
    NF4_TRY(selfcheck_fast(first_bits, count, absmax, d, 0));
    unsigned long long h = 0;
    NF4_CUDA_TRY(cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost));
    *mismatches = h;
    return NF4_OK;
}

int32_t nf4_device_status(int32_t *decode, int32_t *decode_split_k, int32_t *prefill) {
    int *ptrs[3];
    NF4_TRY(flag_ptrs(ptrs));
    int v[3] = {0, 0, 0};
    for (int i = 0; i < 3; ++i)
        NF4_CUDA_TRY(cudaMemcpy(&v[i], ptrs[i], sizeof(int), cudaMemcpyDeviceToHost));
    if (decode) *decode = v[0];
    if (decode_split_k) *decode_split_k = v[1];
    if (prefill) *prefill = v[2];
    return report_flags(ptrs, v);
}

int32_t nf4_selftest_bounded_wait(uint64_t limit_ns, uint64_t *waited_ns) {
    if (limit_ns == 0 || limit_ns > 1000000000ull)
        return fail(NF4_ERR_INVALID_ARG, "nf4_selftest_bounded_wait: limit must be 1 ns .. 1 s");
    NF4_TRY(t_arena.reserve(256));
    unsigned long long *d = static_cast<unsigned long long *>(t_arena.ptr);
    NF4_TRY(decode_selftest_wait((uint32_t)limit_ns, d, 0));
    unsigned long long h = 0;
    NF4_CUDA_TRY(cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost));
    if (waited_ns) *waited_ns = h;
    return nf4_device_status(nullptr, nullptr, nullptr);
}

uint64_t nf4_num_blocks(uint64_t len) { return (len + kBlock - 1) / kBlock; }

uint64_t nf4_packed_bytes(uint64_t len) { return (len + 1) / 2; }

uint64_t nf4_estimated_resident_bytes(uint64_t len, int32_t double_quantized) {
    const uint64_t blocks = nf4_num_blocks(len);
    return nf4_packed_bytes(len) + (double_quantized ? blocks + 4 : 4 * blocks);
}

// ---- device-pointer entry points ------------------------------------------

int32_t nf4_quantize_dev(const float *values, uint64_t len, uint8_t *packed, float *absmax,
                         void *stream) {
    return quantize_packed(values, len, packed, absmax, static_cast<cudaStream_t>(stream));
}

int32_t nf4_quantize_unpacked_dev(const float *values, uint64_t len, uint8_t *codes,
                                  float *absmax, void *stream) {
    return quantize_unpacked(values, len, codes, absmax, static_cast<cudaStream_t>(stream));
}

int32_t nf4_double_quantize_dev(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                                float *scale_of_scales, void *stream) {
    return double_quantize(absmax, nblocks, scale_codes, scale_of_scales,
                           static_cast<cudaStream_t>(stream));
}

int32_t nf4_dequantize_dev(const uint8_t *packed, uint64_t len, const float *absmax,
                           const uint8_t *scale_codes, const float *scale_of_scales, float *out,
                           void *stream) {
    return dequantize_packed(packed, len, absmax, scale_codes, scale_of_scales, out,
                             static_cast<cudaStream_t>(stream));
}

uint64_t nf4_quantize_transposed_workspace_bytes(uint64_t rows, uint64_t cols) {
    return (rows % 64 == 0 && cols % 4 == 0) ? 0 : rows * cols * sizeof(float);
}

int32_t nf4_quantize_transposed_dev(const void *src, int32_t src_dtype, uint64_t rows, uint64_t cols,
                                    uint8_t *packed, float *absmax, void *workspace,
                                    uint64_t workspace_bytes, void *stream) {
    if (src_dtype != NF4_DTYPE_F32 && src_dtype != NF4_DTYPE_BF16)
        return fail(NF4_ERR_INVALID_ARG, "nf4_quantize_transposed_dev: src_dtype must be NF4_DTYPE_F32 or NF4_DTYPE_BF16");
    return quantize_transposed(src, src_dtype == NF4_DTYPE_BF16, rows, cols, packed, absmax, workspace,
                               workspace_bytes, static_cast<cudaStream_t>(stream));
}

int32_t nf4_embedding_gather_dev(const uint8_t *packed, const float *absmax,
                                 const uint8_t *scale_codes, const float *scale_of_scales,
                                 uint64_t n_embedding, uint64_t d_model, const int64_t *ids,
                                 uint64_t n_ids, void *out, int32_t out_dtype, void *stream) {
    if (out_dtype != NF4_DTYPE_F32 && out_dtype != NF4_DTYPE_BF16)
        return fail(NF4_ERR_INVALID_ARG, "nf4_embedding_gather_dev: out_dtype must be NF4_DTYPE_F32 or NF4_DTYPE_BF16");
    return embedding_gather(packed, absmax, scale_codes, scale_of_scales, n_embedding, d_model, ids,
                            n_ids, out, out_dtype == NF4_DTYPE_BF16, static_cast<cudaStream_t>(stream));
}

int32_t nf4_dequantize_unpacked_dev(const uint8_t *codes, uint64_t len, const float *absmax,
                                    const uint8_t *scale_codes, const float *scale_of_scales,
                                    float *out, void *stream) {
    return dequantize_unpacked(codes, len, absmax, scale_codes, scale_of_scales, out,
                               static_cast<cudaStream_t>(stream));
}

uint64_t nf4_quantize_dequantize_workspace_bytes(uint64_t len) {
    // one code per byte + f32 absmax + u8 scale codes + scale of scales, each 256-aligned
    const uint64_t nb = nf4_num_blocks(len);
    return align_up(len, 256) + align_up(nb * 4, 256) + align_up(nb, 256) + 256;
}

int32_t nf4_quantize_dequantize_dev(const float *values, uint64_t len, int32_t double_quantization,
                                    float *out, void *workspace, uint64_t workspace_bytes,
                                    void *stream) {
    if (len == 0) return NF4_OK;
    if (!workspace || workspace_bytes < nf4_quantize_dequantize_workspace_bytes(len))
        return fail(NF4_ERR_INVALID_ARG, "nf4_quantize_dequantize: workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint64_t nb = nf4_num_blocks(len);
    Carver cv(workspace);
    uint8_t *codes = cv.take<uint8_t>(len);
    float *absmax = cv.take<float>(nb);
    uint8_t *scodes = cv.take<uint8_t>(nb);
    float *sos = cv.take<float>(1);
    NF4_TRY(quantize_unpacked(values, len, codes, absmax, s));  // the simulated form, :411
    if (double_quantization) {
        NF4_TRY(double_quantize(absmax, nb, scodes, sos, s));
        return dequantize_unpacked(codes, len, nullptr, scodes, sos, out, s);
    }
    return dequantize_unpacked(codes, len, absmax, nullptr, nullptr, out, s);
}

uint64_t nf4_linear_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out,
                                    uint32_t lora_rank) {

    uint64_t need = decode_workspace_bytes(rows, d_in, d_out, lora_rank);
    const uint64_t b = prefill_workspace_bytes(rows, d_in, d_out, lora_rank);
    const uint64_t c = generic_workspace_bytes(rows, d_in, d_out, lora_rank);
    const uint64_t d = decode2_workspace_bytes(rows, d_in, d_out, lora_rank);
    const uint64_t e = f32_rows_workspace_bytes(rows, d_in, d_out, lora_rank);
    if (d > need) need = d;
    if (b > need) need = b;
    if (c > need) need = c;
    if (e > need) need = e;
    return need;
}

int32_t nf4_linear_forward_dev(const nf4_linear_args *args, void *stream) {
    NF4_TRY(validate_linear(args));
    if (args->rows == 0) return NF4_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // rows <= 16: the warp-MMA kernel (d_in <= 4096, whole 256-slices), else the tcgen05 split-K
    // kernel; more rows: the tcgen05 GEMM; whatever none of them takes: the CUDA-core kernel.
    if (decode_supported(*args)) {
        return decode_forward(*args, s);
    }
    if (decode2_supported(*args)) {
        return decode2_forward(*args, s);
    }
    if (prefill_supported(*args) || prefill_in_out_supported(*args)) {
        return prefill_forward(*args, s);
    }
    if (f32_rows_supported(*args)) {
        return f32_rows_forward(*args, s);
    }
    return generic_forward(*args, s);
}

// SMs the decode kernel leaves alone (see nf4_reserve_sms)
static std::atomic<int> g_reserved_sms{0};

}  // extern "C"
uint32_t nf4::persistent_ctas() {
    const int r = g_reserved_sms.load(std::memory_order_relaxed);
    return (uint32_t)(kNumSMs - r);
}
extern "C" {

int32_t nf4_reserve_sms(int32_t count) {
    if (count < 0 || count > kNumSMs / 2)
        return fail(NF4_ERR_INVALID_ARG, "nf4_reserve_sms: count must be 0 ... %d", kNumSMs / 2);
    g_reserved_sms.store(count, std::memory_order_relaxed);
    return NF4_OK;
}

int32_t nf4_linear_forward_grouped_dev(const nf4_linear_args *args, uint32_t count, void *stream) {
    if (!args || count == 0 || count > 4)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_grouped_dev: count must be 1 ... 4");
    bool together = true;
    for (uint32_t i = 0; i < count; ++i) {
        if (args[i].struct_bytes != sizeof(nf4_linear_args))
            return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_grouped_dev: struct_bytes of element %u", i);
        NF4_TRY(validate_linear(&args[i]));
        together = together && decode_supported(args[i]);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (together && args[0].rows != 0) {
        bool taken = false;
        NF4_TRY(decode_forward_grouped(args, count, s, &taken));
        if (taken) {
            return NF4_OK;
        }
    }
    for (uint32_t i = 0; i < count; ++i) NF4_TRY(nf4_linear_forward_dev(&args[i], stream));
    return NF4_OK;
}

int32_t nf4_linear_forward_scatter_dev(const nf4_linear_args *shard, const nf4_peer_outputs *peers, void *stream) {
    if (!shard || !peers || peers->struct_bytes != sizeof(nf4_peer_outputs))
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_scatter_dev: null arguments or struct_bytes");
    if (peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_scatter_dev: world 1 ... 8, rank inside it");
    nf4_linear_args a = *shard;
    a.y = peers->y_full[peers->rank];  // (validation wants an output; the kernel writes to all of them)
    a.ldy = 0;
    NF4_TRY(validate_linear(&a));
    const uint64_t ldy = peers->ldy_full ? peers->ldy_full : (uint64_t)peers->world * a.d_out;
    if (ldy < (uint64_t)peers->world * a.d_out)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_scatter_dev: ldy_full < world * d_out");
    if (a.rows == 0) return NF4_OK;
    if (!decode_supported(a))
        return fail(NF4_ERR_UNSUPPORTED, "nf4_linear_forward_scatter_dev: only shapes the decode kernel takes "
                                         "(rows <= 16, bf16, W [d_out, d_in], d_in a multiple of 256)");
    if (!a.workspace || a.workspace_bytes < 256)
        return fail(NF4_ERR_INVALID_ARG, "nf4_linear_forward_scatter_dev: the workspace must hold 256 bytes at least");
    return decode_forward_scatter(a, peers->y_full, peers->arrivals, (uint32_t)peers->world, (uint32_t)peers->rank,
                                  ldy, peers->signal != 0, peers->wait_arrivals, peers->wait_expected,
                                  static_cast<cudaStream_t>(stream));
}

int32_t nf4_peer_push_columns_dev(const nf4_peer_outputs *peers, uint64_t rows, uint64_t d_out_shard,
                                  int32_t elem_bytes, uint32_t *scratch_word, void *stream) {
    if (!peers || peers->struct_bytes != sizeof(nf4_peer_outputs))
        return fail(NF4_ERR_INVALID_ARG, "nf4_peer_push_columns_dev: null arguments or struct_bytes");
    if (peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world)
        return fail(NF4_ERR_INVALID_ARG, "nf4_peer_push_columns_dev: world 1 ... 8, rank inside it");
    if (elem_bytes != 2 && elem_bytes != 4) return fail(NF4_ERR_INVALID_ARG, "nf4_peer_push_columns_dev: elem_bytes 2 or 4");
    const uint64_t ldy = peers->ldy_full ? peers->ldy_full : (uint64_t)peers->world * d_out_shard;
    return push_columns(peers->y_full, peers->arrivals, (uint32_t)peers->world, (uint32_t)peers->rank, rows,
                        d_out_shard * elem_bytes, ldy * elem_bytes, peers->signal != 0, scratch_word,
                        static_cast<cudaStream_t>(stream));
}

int32_t nf4_peer_arrivals_wait_dev(uint32_t *own_arrivals, uint32_t expected, uint32_t timeout_ns, void *stream) {
    if (!own_arrivals) return fail(NF4_ERR_INVALID_ARG, "nf4_peer_arrivals_wait_dev: null counter");
    return decode_peer_wait(own_arrivals, expected, timeout_ns, static_cast<cudaStream_t>(stream));
}

int32_t nf4_decode_share_plan(uint32_t rows, uint32_t d_in, uint32_t d_out, uint32_t lora_rank, uint32_t cta,
                              uint32_t *k0_k1_n0_n1) {
    if (!k0_k1_n0_n1) return fail(NF4_ERR_INVALID_ARG, "nf4_decode_share_plan: null output");
    const int32_t n = decode_share_plan(rows, d_in, d_out, lora_rank, cta, k0_k1_n0_n1);
    if (n < 0) return fail(NF4_ERR_INVALID_ARG, "nf4_decode_share_plan: not a shape of the decode kernel, or no such CTA");
    return n;
}

int32_t nf4_prefill_share_plan(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t cta, uint32_t *ctas,
                               uint32_t *segments, uint32_t capacity) {
    if (!segments && capacity) return fail(NF4_ERR_INVALID_ARG, "nf4_prefill_share_plan: null segments");
    const int32_t n = prefill_share_plan(rows, d_in, d_out, cta, ctas, segments, capacity);
    if (n < 0) return fail(NF4_ERR_INVALID_ARG, "nf4_prefill_share_plan: not a shape of the tensor-core kernel, or no such CTA");
    return n;
}

uint64_t nf4_linear_noalloc_scratch_bytes(void) { return decode_static_scratch_bytes(); }

int32_t nf4_linear_forward_noalloc_dev(const nf4_linear_args *args, void *stream) {
    NF4_TRY(validate_linear(args, /*needs_workspace=*/false));
    if (args->rows == 0) return NF4_OK;
    return decode_forward_static_scratch(*args, static_cast<cudaStream_t>(stream));
}

// ---- the adapter alone, its dense update, the merge ----------------------------------------

static int32_t check_lora(const void *a, const void *b, uint64_t d_in, uint64_t d_out, uint32_t rank,
                          int32_t layout, int32_t io_dtype, const char *who) {
    if (!a || !b) return fail(NF4_ERR_INVALID_ARG, "%s: null factors", who);
    if (rank == 0 || d_in == 0 || d_out == 0) return fail(NF4_ERR_INVALID_ARG, "%s: zero rank or dimension", who);
    if (layout != NF4_LAYOUT_OUT_IN && layout != NF4_LAYOUT_IN_OUT) return fail(NF4_ERR_INVALID_ARG, "%s: bad layout %d", who, layout);
    if (io_dtype != NF4_DTYPE_BF16 && io_dtype != NF4_DTYPE_F32) return fail(NF4_ERR_INVALID_ARG, "%s: bad io_dtype %d", who, io_dtype);
    return NF4_OK;
}

uint64_t nf4_lora_workspace_bytes(uint64_t rows, uint32_t lora_rank) { return lora_workspace_bytes(rows, lora_rank); }

int32_t nf4_lora_forward_dev(const void *x, uint64_t rows, uint64_t d_in, uint64_t d_out, const void *lora_a,
                             const void *lora_b, uint32_t lora_rank, float lora_scale, int32_t layout,
                             int32_t io_dtype, void *y, uint64_t ldy, void *workspace, uint64_t workspace_bytes,
                             void *stream) {
    NF4_TRY(check_lora(lora_a, lora_b, d_in, d_out, lora_rank, layout, io_dtype, "nf4_lora_forward_dev"));
    if (rows == 0) return NF4_OK;
    if (!x || !y) return fail(NF4_ERR_INVALID_ARG, "nf4_lora_forward_dev: null x/y");
    if (ldy != 0 && ldy < d_out) return fail(NF4_ERR_INVALID_ARG, "nf4_lora_forward_dev: ldy < d_out");
    if (!workspace || workspace_bytes < lora_workspace_bytes(rows, lora_rank))
        return fail(NF4_ERR_INVALID_ARG, "nf4_lora_forward_dev: workspace smaller than nf4_lora_workspace_bytes");
    return lora_forward(x, rows, d_in, d_out, lora_a, lora_b, lora_rank, lora_scale, layout, io_dtype, y,
                        ldy ? ldy : d_out, static_cast<float *>(workspace), static_cast<cudaStream_t>(stream));
}

int32_t nf4_lora_delta_weight_dev(const void *lora_a, const void *lora_b, uint64_t d_in, uint64_t d_out,
                                  uint32_t lora_rank, float lora_scale, int32_t layout, int32_t io_dtype,
                                  float *out, void *stream) {
    NF4_TRY(check_lora(lora_a, lora_b, d_in, d_out, lora_rank, layout, io_dtype, "nf4_lora_delta_weight_dev"));
    if (!out) return fail(NF4_ERR_INVALID_ARG, "nf4_lora_delta_weight_dev: null out");
    return lora_delta(lora_a, lora_b, nullptr, nullptr, nullptr, nullptr, d_in, d_out, lora_rank, lora_scale,
                      layout, io_dtype, out, static_cast<cudaStream_t>(stream));
}

int32_t nf4_qlora_merge_dev(const uint8_t *packed, const float *absmax, const uint8_t *scale_codes,
                            const float *scale_of_scales, uint64_t d_in, uint64_t d_out, int32_t layout,
                            const void *lora_a, const void *lora_b, uint32_t lora_rank, float lora_scale,
                            int32_t io_dtype, float *out, void *stream) {
    NF4_TRY(check_lora(lora_a, lora_b, d_in, d_out, lora_rank, layout, io_dtype, "nf4_qlora_merge_dev"));
    if (!packed || !out) return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_merge_dev: null packed/out");
    if ((absmax != nullptr) == (scale_codes != nullptr) || (scale_codes && !scale_of_scales))
        return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_merge_dev: give either absmax or scale_codes+scale_of_scales");
    return lora_delta(lora_a, lora_b, packed, absmax, scale_codes, scale_of_scales, d_in, d_out, lora_rank,
                      lora_scale, layout, io_dtype, out, static_cast<cudaStream_t>(stream));
}

// ---- backward of the QLoRA linear (base weight frozen) -----------------------------------------

uint64_t nf4_qlora_backward_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    // grad_x is a forward with d_in and d_out exchanged; then two [rows][rank] f32 intermediates
    // ... and one adapter factor transposed (bf16)
    const uint64_t widest = d_in > d_out ? d_in : d_out;
    return nf4_linear_workspace_bytes(rows, d_out, d_in, lora_rank) + 2 * lora_workspace_bytes(rows, lora_rank) +
           align_up((uint64_t)lora_rank * widest * 2, 256);
}

int32_t nf4_qlora_backward_dev(const nf4_linear_args *fwd, const void *grad_y, void *grad_x, void *grad_a,
                               void *grad_b, void *stream) {
    if (!fwd) return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_backward_dev: null args");
    if (fwd->struct_bytes != sizeof(nf4_linear_args))
        return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_backward_dev: struct_bytes %u != %zu", fwd->struct_bytes,
                    sizeof(nf4_linear_args));
    const uint32_t r = fwd->lora_a ? fwd->lora_rank : 0;
    if (fwd->rows == 0) return NF4_OK;
    if (!grad_y || !grad_x || (r && (!grad_a || !grad_b)))
        return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_backward_dev: null gradient buffer");
    const uint64_t need = nf4_qlora_backward_workspace_bytes(fwd->rows, fwd->d_in, fwd->d_out, r);
    if (need && (!fwd->workspace || fwd->workspace_bytes < need || (reinterpret_cast<uintptr_t>(fwd->workspace) & 255u)))
        return fail(NF4_ERR_INVALID_ARG, "nf4_qlora_backward_dev: workspace smaller than "
                                         "nf4_qlora_backward_workspace_bytes or not 256-byte aligned");
    // grad_x = grad_y W^T + s (grad_y B^T) A^T: one more NF4 linear over the same packed bytes read
    // in the other orientation, the adapter factors exchanging roles
    nf4_linear_args g = *fwd;
    g.layout = fwd->layout == NF4_LAYOUT_OUT_IN ? NF4_LAYOUT_IN_OUT : NF4_LAYOUT_OUT_IN;
    g.d_in = fwd->d_out;
    g.d_out = fwd->d_in;
    g.x = grad_y;
    g.y = grad_x;
    g.ldy = 0;
    g.y_f32 = 0;
    g.bias = nullptr;
    g.lora_a = fwd->lora_b;
    g.lora_b = fwd->lora_a;
    const uint64_t fw = nf4_linear_workspace_bytes(fwd->rows, fwd->d_out, fwd->d_in, r);
    g.workspace_bytes = fw;
    NF4_TRY(nf4_linear_forward_dev(&g, stream));
    if (!r) return NF4_OK;
    uint8_t *ws = static_cast<uint8_t *>(fwd->workspace) + fw;
    float *t = reinterpret_cast<float *>(ws);
    float *u = reinterpret_cast<float *>(ws + lora_workspace_bytes(fwd->rows, r));
    void *factor_t = ws + 2 * lora_workspace_bytes(fwd->rows, r);
    return lora_grads(fwd->x, grad_y, fwd->lora_a, fwd->lora_b, fwd->rows, fwd->d_in, fwd->d_out, r,
                      fwd->lora_scale, fwd->layout, fwd->io_dtype, grad_a, grad_b, t, u, factor_t,
                      static_cast<cudaStream_t>(stream));
}

// ---- column-sharded forward ------------------------------------------------------------------

uint64_t nf4_sharded_gather_bytes(uint64_t rows, uint64_t d_out_shard, int32_t world, int32_t io_dtype, int32_t y_f32) {
    const uint64_t eb = (y_f32 || io_dtype == NF4_DTYPE_F32) ? 4 : 2;
    return world > 0 ? (uint64_t)world * rows * d_out_shard * eb : 0;
}

int32_t nf4_sharded_linear_forward_dev(const nf4_linear_args *shard, void *nccl_comm, int32_t rank, int32_t world,
                                       void *gather_buffer, uint64_t gather_bytes, void *y_full,
                                       uint64_t ldy_full, void *stream) {
    NF4_TRY(validate_linear(shard));
    if (!nccl_comm || world < 1 || rank < 0 || rank >= world)
        return fail(NF4_ERR_INVALID_ARG, "nf4_sharded_linear_forward_dev: bad communicator, rank or world");
    if (shard->rows == 0) return NF4_OK;
    const uint64_t eb = (shard->y_f32 || shard->io_dtype == NF4_DTYPE_F32) ? 4 : 2;
    const uint64_t ldy_local = shard->ldy ? shard->ldy : shard->d_out;
    if (ldy_local != shard->d_out)
        return fail(NF4_ERR_INVALID_ARG, "nf4_sharded_linear_forward_dev: the local slab must be dense (ldy = d_out)");
    if (ldy_full == 0) ldy_full = shard->d_out * (uint64_t)world;
    if (ldy_full < shard->d_out * (uint64_t)world)
        return fail(NF4_ERR_INVALID_ARG, "nf4_sharded_linear_forward_dev: ldy_full < world * d_out of a shard");
    if (!gather_buffer || !y_full ||
        gather_bytes < nf4_sharded_gather_bytes(shard->rows, shard->d_out, world, shard->io_dtype, shard->y_f32))
        return fail(NF4_ERR_INVALID_ARG, "nf4_sharded_linear_forward_dev: gather buffer smaller than nf4_sharded_gather_bytes");
    NF4_TRY(nf4_linear_forward_dev(shard, stream));
    return gather_slabs(shard->y, gather_buffer, y_full, shard->rows, shard->d_out * eb, ldy_full * eb, nccl_comm,
                        world, static_cast<cudaStream_t>(stream));
}

// ---- host-pointer entry points ------------------------------------------------

int32_t nf4_quantize_host(const float *values, uint64_t len, uint8_t *packed, float *absmax) {
    if (len == 0) return NF4_OK;
    if (!values || !packed || !absmax)
        return fail(NF4_ERR_INVALID_ARG, "nf4_quantize_host: null pointer");
    const uint64_t nb = nf4_num_blocks(len), pb = nf4_packed_bytes(len);
    NF4_TRY(t_arena.reserve(align_up(len * 4, 256) + align_up(pb, 256) + align_up(nb * 4, 256)));
    Carver cv(t_arena.ptr);
    float *d_v = cv.take<float>(len);
    uint8_t *d_p = cv.take<uint8_t>(pb);
    float *d_a = cv.take<float>(nb);
    NF4_CUDA_TRY(cudaMemcpyAsync(d_v, values, len * 4, cudaMemcpyHostToDevice, kHostStream));
    NF4_TRY(quantize_packed(d_v, len, d_p, d_a, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(packed, d_p, pb, cudaMemcpyDeviceToHost, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(absmax, d_a, nb * 4, cudaMemcpyDeviceToHost, kHostStream));
    return check_cuda(cudaStreamSynchronize(kHostStream), "nf4_quantize_host sync");
}

int32_t nf4_double_quantize_host(const float *absmax, uint64_t nblocks, uint8_t *scale_codes,
                                 float *scale_of_scales) {
    if (!scale_of_scales) return fail(NF4_ERR_INVALID_ARG, "nf4_double_quantize_host: null pointer");
    if (nblocks == 0) {
        *scale_of_scales = 0.0f;
        return NF4_OK;
    }
    if (!absmax || !scale_codes)
        return fail(NF4_ERR_INVALID_ARG, "nf4_double_quantize_host: null pointer");
    NF4_TRY(t_arena.reserve(align_up(nblocks * 4, 256) + align_up(nblocks, 256) + 256));
    Carver cv(t_arena.ptr);
    float *d_a = cv.take<float>(nblocks);
    uint8_t *d_c = cv.take<uint8_t>(nblocks);
    float *d_s = cv.take<float>(1);
    NF4_CUDA_TRY(cudaMemcpyAsync(d_a, absmax, nblocks * 4, cudaMemcpyHostToDevice, kHostStream));
    NF4_TRY(double_quantize(d_a, nblocks, d_c, d_s, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(scale_codes, d_c, nblocks, cudaMemcpyDeviceToHost, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(scale_of_scales, d_s, 4, cudaMemcpyDeviceToHost, kHostStream));
    return check_cuda(cudaStreamSynchronize(kHostStream), "nf4_double_quantize_host sync");
}

int32_t nf4_dequantize_host(const uint8_t *packed, uint64_t len, const float *absmax,
                            const uint8_t *scale_codes, const float *scale_of_scales, float *out) {
    if (len == 0) return NF4_OK;
    if (!packed || !out) return fail(NF4_ERR_INVALID_ARG, "nf4_dequantize_host: null pointer");
    if ((absmax != nullptr) == (scale_codes != nullptr) || (scale_codes && !scale_of_scales))
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_dequantize_host: give either absmax or scale_codes+scale_of_scales");
    const uint64_t nb = nf4_num_blocks(len), pb = nf4_packed_bytes(len);
    NF4_TRY(t_arena.reserve(align_up(len * 4, 256) + align_up(pb, 256) + align_up(nb * 4, 256) + 256));
    Carver cv(t_arena.ptr);
    float *d_o = cv.take<float>(len);
    uint8_t *d_p = cv.take<uint8_t>(pb);
    float *d_a = cv.take<float>(nb);  // f32 scales, or the u8 codes in the same space
    float *d_s = cv.take<float>(1);
    NF4_CUDA_TRY(cudaMemcpyAsync(d_p, packed, pb, cudaMemcpyHostToDevice, kHostStream));
    if (absmax) {
        NF4_CUDA_TRY(cudaMemcpyAsync(d_a, absmax, nb * 4, cudaMemcpyHostToDevice, kHostStream));
        NF4_TRY(dequantize_packed(d_p, len, d_a, nullptr, nullptr, d_o, kHostStream));
    } else {
        NF4_CUDA_TRY(cudaMemcpyAsync(d_a, scale_codes, nb, cudaMemcpyHostToDevice, kHostStream));
        NF4_CUDA_TRY(cudaMemcpyAsync(d_s, scale_of_scales, 4, cudaMemcpyHostToDevice, kHostStream));
        NF4_TRY(dequantize_packed(d_p, len, nullptr, reinterpret_cast<uint8_t *>(d_a), d_s, d_o, kHostStream));
    }
    NF4_CUDA_TRY(cudaMemcpyAsync(out, d_o, len * 4, cudaMemcpyDeviceToHost, kHostStream));
    return check_cuda(cudaStreamSynchronize(kHostStream), "nf4_dequantize_host sync");
}

int32_t nf4_quantize_dequantize_host(const float *values, uint64_t len,
                                     int32_t double_quantization, float *out) {
    if (len == 0) return NF4_OK;
    if (!values || !out) return fail(NF4_ERR_INVALID_ARG, "nf4_quantize_dequantize_host: null pointer");
    const uint64_t ws = nf4_quantize_dequantize_workspace_bytes(len);
    NF4_TRY(t_arena.reserve(2 * align_up(len * 4, 256) + ws + 256));
    Carver cv(t_arena.ptr);
    float *d_v = cv.take<float>(len);
    float *d_o = cv.take<float>(len);
    uint8_t *d_w = cv.take<uint8_t>(ws);
    NF4_CUDA_TRY(cudaMemcpyAsync(d_v, values, len * 4, cudaMemcpyHostToDevice, kHostStream));
    NF4_TRY(nf4_quantize_dequantize_dev(d_v, len, double_quantization, d_o, d_w, ws, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(out, d_o, len * 4, cudaMemcpyDeviceToHost, kHostStream));
    return check_cuda(cudaStreamSynchronize(kHostStream), "nf4_quantize_dequantize_host sync");
}

// ---- resident weight handles -----------------------------------------------------

static int32_t weight_alloc(uint64_t d_in, uint64_t d_out, int32_t layout, bool dq,
                            nf4_weight **out) {
    if (!out) return fail(NF4_ERR_INVALID_ARG, "nf4_weight: null out");
    *out = nullptr;
    if (d_in == 0 || d_out == 0) return fail(NF4_ERR_INVALID_ARG, "nf4_weight: zero dimension");
    if (layout != NF4_LAYOUT_OUT_IN && layout != NF4_LAYOUT_IN_OUT)
        return fail(NF4_ERR_INVALID_ARG, "nf4_weight: bad layout %d", layout);
    nf4_weight *w = new (std::nothrow) nf4_weight();
    if (!w) return fail(NF4_ERR_OOM, "nf4_weight: host allocation failed");
    w->d_in = d_in;
    w->d_out = d_out;
    w->len = d_in * d_out;
    w->nblocks = nf4_num_blocks(w->len);
    w->layout = layout;
    w->double_quantized = dq;
    int32_t st = check_cuda(cudaGetDevice(&w->device), "cudaGetDevice");
    if (st == NF4_OK) st = check_cuda(cudaMalloc(&w->packed, nf4_packed_bytes(w->len)), "cudaMalloc packed");
    if (st == NF4_OK) st = check_cuda(cudaMalloc(&w->absmax, w->nblocks * 4), "cudaMalloc absmax");
    if (st == NF4_OK && dq) {
        st = check_cuda(cudaMalloc(&w->scale_codes, w->nblocks), "cudaMalloc scale codes");
        if (st == NF4_OK) st = check_cuda(cudaMalloc(&w->scale_of_scales, 256), "cudaMalloc sos");
    }
    if (st != NF4_OK) {
        nf4_weight_free(w);
        return st;
    }
    *out = w;
    return NF4_OK;
}

int32_t nf4_weight_from_values_host(const float *values, uint64_t d_in, uint64_t d_out,
                                    int32_t layout, int32_t double_quantization,
                                    nf4_weight **out) {
    if (!values) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_from_values_host: null values");
    nf4_weight *w = nullptr;
    NF4_TRY(weight_alloc(d_in, d_out, layout, double_quantization != 0, &w));
    int32_t st = t_arena.reserve(w->len * 4);
    if (st == NF4_OK) {
        float *d_v = static_cast<float *>(t_arena.ptr);
        st = check_cuda(cudaMemcpyAsync(d_v, values, w->len * 4, cudaMemcpyHostToDevice, kHostStream), "H2D values");
        if (st == NF4_OK) st = quantize_packed(d_v, w->len, w->packed, w->absmax, kHostStream);
        if (st == NF4_OK && w->double_quantized)
            st = double_quantize(w->absmax, w->nblocks, w->scale_codes, w->scale_of_scales, kHostStream);
        if (st == NF4_OK) st = check_cuda(cudaStreamSynchronize(kHostStream), "nf4_weight_from_values_host sync");
    }
    if (st == NF4_OK && w->double_quantized) {
        // The f32 scales are not part of a double-quantized weight (src/quantize.rs:304-307).
        cudaFree(w->absmax);
        w->absmax = nullptr;
    }
    if (st != NF4_OK) {
        nf4_weight_free(w);
        return st;
    }
    *out = w;
    return NF4_OK;
}

int32_t nf4_weight_from_packed_host(const uint8_t *packed, const float *absmax,
                                    const uint8_t *scale_codes, float scale_of_scales,
                                    uint64_t d_in, uint64_t d_out, int32_t layout,
                                    nf4_weight **out) {
    if (!packed) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_from_packed_host: null packed");
    if ((absmax != nullptr) == (scale_codes != nullptr))
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_weight_from_packed_host: give either absmax or scale_codes");
    nf4_weight *w = nullptr;
    NF4_TRY(weight_alloc(d_in, d_out, layout, scale_codes != nullptr, &w));
    int32_t st = check_cuda(cudaMemcpy(w->packed, packed, nf4_packed_bytes(w->len), cudaMemcpyHostToDevice), "H2D packed");
    if (st == NF4_OK && absmax)
        st = check_cuda(cudaMemcpy(w->absmax, absmax, w->nblocks * 4, cudaMemcpyHostToDevice), "H2D absmax");
    if (st == NF4_OK && scale_codes) {
        st = check_cuda(cudaMemcpy(w->scale_codes, scale_codes, w->nblocks, cudaMemcpyHostToDevice), "H2D scale codes");
        if (st == NF4_OK)
            st = check_cuda(cudaMemcpy(w->scale_of_scales, &scale_of_scales, 4, cudaMemcpyHostToDevice), "H2D sos");
        cudaFree(w->absmax);
        w->absmax = nullptr;
    }
    if (st != NF4_OK) {
        nf4_weight_free(w);
        return st;
    }
    *out = w;
    return NF4_OK;
}

void nf4_weight_free(nf4_weight *w) {
    if (!w) return;
    cudaFree(w->packed);
    cudaFree(w->absmax);
    cudaFree(w->scale_codes);
    cudaFree(w->scale_of_scales);
    cudaFree(w->lora_a);
    cudaFree(w->lora_b);
    delete w;
}

uint64_t nf4_weight_resident_bytes(const nf4_weight *w) {
    return w ? nf4_estimated_resident_bytes(w->len, w->double_quantized) : 0;
}

int32_t nf4_weight_download_host(const nf4_weight *w, uint8_t *packed, float *absmax,
                                 uint8_t *scale_codes, float *scale_of_scales) {
    if (!w) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_download_host: null weight");
    if (packed)
        NF4_CUDA_TRY(cudaMemcpy(packed, w->packed, nf4_packed_bytes(w->len), cudaMemcpyDeviceToHost));
    if (w->double_quantized) {
        if (absmax) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_download_host: weight is double-quantized, it has no f32 scales");
        if (scale_codes)
            NF4_CUDA_TRY(cudaMemcpy(scale_codes, w->scale_codes, w->nblocks, cudaMemcpyDeviceToHost));
        if (scale_of_scales)
            NF4_CUDA_TRY(cudaMemcpy(scale_of_scales, w->scale_of_scales, 4, cudaMemcpyDeviceToHost));
    } else {
        if (scale_codes || scale_of_scales)
            return fail(NF4_ERR_INVALID_ARG, "nf4_weight_download_host: weight has f32 scales, not u8 codes");
        if (absmax)
            NF4_CUDA_TRY(cudaMemcpy(absmax, w->absmax, w->nblocks * 4, cudaMemcpyDeviceToHost));
    }
    return NF4_OK;
}

int32_t nf4_weight_dequantize_host(const nf4_weight *w, float *out) {
    if (!w || !out) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_dequantize_host: null pointer");
    NF4_TRY(check_weight_device(w, "nf4_weight_dequantize_host"));
    NF4_TRY(t_arena.reserve(w->len * 4));
    float *d_o = static_cast<float *>(t_arena.ptr);
    NF4_TRY(dequantize_packed(w->packed, w->len, w->absmax, w->scale_codes, w->scale_of_scales, d_o, kHostStream));
    NF4_CUDA_TRY(cudaMemcpyAsync(out, d_o, w->len * 4, cudaMemcpyDeviceToHost, kHostStream));
    return check_cuda(cudaStreamSynchronize(kHostStream), "nf4_weight_dequantize_host sync");
}

int32_t nf4_weight_attach_lora_host(nf4_weight *w, const void *lora_a, const void *lora_b,
                                    uint32_t lora_rank, float lora_scale, int32_t io_dtype) {
    if (!w) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_attach_lora_host: null weight");
    NF4_TRY(check_weight_device(w, "nf4_weight_attach_lora_host"));
    cudaFree(w->lora_a);
    cudaFree(w->lora_b);
    w->lora_a = w->lora_b = nullptr;
    w->lora_rank = 0;
    if (lora_rank == 0) return NF4_OK;
    if (!lora_a || !lora_b) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_attach_lora_host: null factors");
    if (io_dtype != NF4_DTYPE_BF16 && io_dtype != NF4_DTYPE_F32)
        return fail(NF4_ERR_INVALID_ARG, "nf4_weight_attach_lora_host: bad io_dtype");
    const size_t eb = dtype_bytes(io_dtype);
    const size_t ab = (size_t)lora_rank * w->d_in * eb, bb = (size_t)lora_rank * w->d_out * eb;
    NF4_CUDA_TRY(cudaMalloc(&w->lora_a, ab));
    NF4_CUDA_TRY(cudaMalloc(&w->lora_b, bb));
    NF4_CUDA_TRY(cudaMemcpy(w->lora_a, lora_a, ab, cudaMemcpyHostToDevice));
    NF4_CUDA_TRY(cudaMemcpy(w->lora_b, lora_b, bb, cudaMemcpyHostToDevice));
    w->lora_rank = lora_rank;
    w->lora_scale = lora_scale;
    w->lora_dtype = io_dtype;
    return NF4_OK;
}

int32_t nf4_weight_linear_forward_host(const nf4_weight *w, const void *x, uint64_t rows,
                                       int32_t io_dtype, const float *bias, const void *lora_a,
                                       const void *lora_b, uint32_t lora_rank, float lora_scale,
                                       void *y) {
    if (!w) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_linear_forward_host: null weight");
    NF4_TRY(check_weight_device(w, "nf4_weight_linear_forward_host"));
    if (rows == 0) return NF4_OK;
    if (!x || !y) return fail(NF4_ERR_INVALID_ARG, "nf4_weight_linear_forward_host: null x/y");
    if (io_dtype != NF4_DTYPE_BF16 && io_dtype != NF4_DTYPE_F32)
        return fail(NF4_ERR_INVALID_ARG, "nf4_weight_linear_forward_host: bad io_dtype");
    if ((lora_a != nullptr) != (lora_b != nullptr))
        return fail(NF4_ERR_INVALID_ARG, "nf4_weight_linear_forward_host: lora_a and lora_b go together");
    const size_t eb = dtype_bytes(io_dtype);
    const bool resident = !lora_a && w->lora_rank && w->lora_dtype == io_dtype;
    if (resident) {
        lora_rank = w->lora_rank;
        lora_scale = w->lora_scale;
    }
    const uint32_t r = (lora_a || resident) ? lora_rank : 0;
    const uint64_t ws = nf4_linear_workspace_bytes(rows, w->d_in, w->d_out, r);
    const size_t xb = rows * w->d_in * eb, yb = rows * w->d_out * eb;
    const size_t ab = resident ? 0 : (size_t)r * w->d_in * eb;
    const size_t bb = resident ? 0 : (size_t)r * w->d_out * eb;
    NF4_TRY(t_arena.reserve(align_up(xb, 256) + align_up(yb, 256) + align_up(ab, 256) +
                            align_up(bb, 256) + align_up(w->d_out * 4, 256) + ws + 1024));
    Carver cv(t_arena.ptr);
    uint8_t *d_x = cv.take<uint8_t>(xb);
    uint8_t *d_y = cv.take<uint8_t>(yb);
    uint8_t *d_a = cv.take<uint8_t>(ab);
    uint8_t *d_b = cv.take<uint8_t>(bb);
    float *d_bias = cv.take<float>(w->d_out);
    uint8_t *d_ws = cv.take<uint8_t>(ws);
    NF4_CUDA_TRY(cudaMemcpyAsync(d_x, x, xb, cudaMemcpyHostToDevice, kHostStream));
    if (r && !resident) {
        NF4_CUDA_TRY(cudaMemcpyAsync(d_a, lora_a, ab, cudaMemcpyHostToDevice, kHostStream));
        NF4_CUDA_TRY(cudaMemcpyAsync(d_b, lora_b, bb, cudaMemcpyHostToDevice, kHostStream));
    }
    if (bias) NF4_CUDA_TRY(cudaMemcpyAsync(d_bias, bias, w->d_out * 4, cudaMemcpyHostToDevice, kHostStream));
    nf4_linear_args a;
    std::memset(&a, 0, sizeof(a));
    a.struct_bytes = sizeof(a);
    a.layout = w->layout;
    a.io_dtype = io_dtype;
    a.rows = rows;
    a.d_in = w->d_in;
    a.d_out = w->d_out;
    a.x = d_x;
    a.packed = w->packed;
    a.absmax = w->absmax;
    a.scale_codes = w->scale_codes;
    a.scale_of_scales = w->scale_of_scales;
    a.bias = bias ? d_bias : nullptr;
    a.lora_a = r ? (resident ? w->lora_a : (void *)d_a) : nullptr;
    a.lora_b = r ? (resident ? w->lora_b : (void *)d_b) : nullptr;
    a.lora_rank = r;
    a.lora_scale = lora_scale;
    a.y = d_y;
    // At decode sizes the two copies are half of the call's latency.  When y is page-locked memory
    // the device can address (cudaHostAlloc, cudaHostRegister with the mapped flag), the kernel
    // stores its results there itself: the copy back, a separate operation of some ten microseconds, goes.
    // (Not for the tensor-core GEMM of more rows, which stores through a tensor map, and where the
    // copies do not matter.)
    void *y_mapped = nullptr;
    if (rows <= 16) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, y) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
            y_mapped = attr.devicePointer;
        else
            (void)cudaGetLastError();  // pageable memory is reported as an error by older drivers: not one here
    }
    if (y_mapped) a.y = y_mapped;
    a.ldy = w->d_out;
    a.workspace = ws ? d_ws : nullptr;
    a.workspace_bytes = ws;
    void *kept = nullptr;
    if (ws && rows <= 16 && ws <= ZeroScratch::kMaxBytes) {
        // the decode workspace starts with flag words that must be zero: a buffer kept for it
        NF4_TRY(t_zero_scratch.get(&kept, ws));
        a.workspace = kept;
    } else if (ws) {
        NF4_CUDA_TRY(cudaMemsetAsync(d_ws, 0, 256, kHostStream));
    }
    volatile int *failed = nullptr;
    NF4_TRY(host_flag_words(&failed));  // (before the launch: the kernels write their failure codes there too)
    NF4_TRY(nf4_linear_forward_dev(&a, kHostStream));
    if (!y_mapped) NF4_CUDA_TRY(cudaMemcpyAsync(y, d_y, yb, cudaMemcpyDeviceToHost, kHostStream));
    NF4_TRY(check_cuda(cudaStreamSynchronize(kHostStream), "nf4_weight_linear_forward_host sync"));
    // ... and a wait that gave up in a kernel must not pass for a result
    if (failed[0] | failed[1] | failed[2]) {
        int *ptrs[3];
        NF4_TRY(flag_ptrs(ptrs));
        const int v[3] = {failed[0], failed[1], failed[2]};
        failed[0] = failed[1] = failed[2] = 0;
        if (kept) (void)cudaMemset(kept, 0, 256);  // a kernel that gave up may have left its flag words set
        return report_flags(ptrs, v);
    }
    return NF4_OK;
}

}  // extern "C"
