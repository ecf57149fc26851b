/*
 * CPU oracle for the NF4 quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference crate's
 * src/quantize.rs (and the two forwards in src/qwennet.rs).  It exists so the
 * CUDA kernels can be checked bit-for-bit; the shipped library never links,
 * loads or calls it.  Only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark may use it.
 *
 * Parity pinning: the reference itself is Rust and cannot be compiled on a
 * machine without a Rust toolchain, so this restatement is pinned against the
 * deterministic known-answer tests the reference carries (level table,
 * level*0.75 round trip, the -4.25/2.0 block, all-zero block, ragged 69,
 * byte-count formulae, packed == simulated) -- see tests/test_oracle_kat.py.
 * The GEMM part of the forward lives in third-party crates (burn-ndarray 0.21.0
 * -> ndarray 0.17.2 -> matrixmultiply 0.3.11) whose summation order is not
 * pinned by any reference test: for the matmul the oracle accumulates in f64
 * and parity there is tolerance-based ("parity unpinned" for absolute GEMM
 * bits; every quantize/dequantize result is pinned).
 *
 * Build: -O2 -ffp-contract=off, no fast-math.  Rust f32 arithmetic is strict
 * IEEE-754 without contraction; f32::max is fmaxf, f32::round is roundf.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define NF4O_BLOCK 64

/* src/quantize.rs:37 */
size_t nf4o_block_size(void) { return NF4O_BLOCK; }

/* src/quantize.rs:49-66 -- the sixteen levels, written as the f64 originals of
 * src/quantize.rs:845-862 and narrowed to f32 exactly as that test does. */
static const double k_levels_f64[16] = {
    -1.0,
    -0.6961928009986877,
    -0.5250730514526367,
    -0.39491748809814453,
    -0.28444138169288635,
    -0.18477343022823334,
    -0.09105003625154495,
    0.0,
    0.07958029955625534,
    0.16093020141124725,
    0.24611230194568634,
    0.33791524171829224,
    0.44070982933044434,
    0.5626170039176941,
    0.7229568362236023,
    1.0,
};

static float level(int i) { return (float)k_levels_f64[i]; }

void nf4o_levels(float *out16)
{
    for (int i = 0; i < 16; ++i) out16[i] = level(i);
}

/* src/quantize.rs:208-219 -- linear scan, strict '<', ties keep the lower
 * index, NaN compares false everywhere and so yields code 0. */
uint8_t nf4o_nearest_level_code(float v)
{
    int best = 0;
    float best_dist = INFINITY;
    for (int i = 0; i < 16; ++i) {
        float d = fabsf(v - level(i));
        if (d < best_dist) {
            best_dist = d;
            best = i;
        }
    }
    return (uint8_t)best;
}

void nf4o_nearest_level_codes(const float *v, size_t n, uint8_t *out)
{
    for (size_t i = 0; i < n; ++i) out[i] = nf4o_nearest_level_code(v[i]);
}

size_t nf4o_num_blocks(size_t len) { return (len + NF4O_BLOCK - 1) / NF4O_BLOCK; }

/* src/quantize.rs:99-124 -- Nf4Tensor::quantize: one code per byte, one absmax
 * per chunk of 64 over the FLAT slice (the last chunk may be short). */
void nf4o_quantize_simulated(const float *values, size_t len, uint8_t *codes, float *absmax)
{
    size_t nb = nf4o_num_blocks(len);
    for (size_t b = 0; b < nb; ++b) {
        size_t lo = b * NF4O_BLOCK;
        size_t hi = lo + NF4O_BLOCK < len ? lo + NF4O_BLOCK : len;
        float am = 0.0f;
        for (size_t i = lo; i < hi; ++i) am = fmaxf(am, fabsf(values[i])); /* :103 */
        for (size_t i = lo; i < hi; ++i) {
            if (am == 0.0f)                                               /* :109-110 */
                codes[i] = nf4o_nearest_level_code(0.0f);
            else
                codes[i] = nf4o_nearest_level_code(values[i] / am);      /* :112 */
        }
        absmax[b] = am;
    }
}

/* src/quantize.rs:262-279 -- PackedNf4Tensor::quantize: pairs inside each block,
 * low nibble first, a lone last code leaves the high nibble 0. */
void nf4o_pack_codes(const uint8_t *codes, size_t len, uint8_t *packed)
{
    size_t nb = nf4o_num_blocks(len);
    size_t w = 0;
    for (size_t b = 0; b < nb; ++b) {
        size_t lo = b * NF4O_BLOCK;
        size_t hi = lo + NF4O_BLOCK < len ? lo + NF4O_BLOCK : len;
        for (size_t i = lo; i < hi; i += 2) {
            uint8_t low = codes[i];
            uint8_t high = (i + 1 < hi) ? codes[i + 1] : 0;
            packed[w++] = (uint8_t)(low | (uint8_t)(high << 4));
        }
    }
}

void nf4o_quantize_packed(const float *values, size_t len, uint8_t *packed, float *absmax,
                          uint8_t *scratch_codes)
{
    nf4o_quantize_simulated(values, len, scratch_codes, absmax);
    nf4o_pack_codes(scratch_codes, len, packed);
}

/* src/quantize.rs:129-149 and :284-309 -- with_double_quantization. */
void nf4o_double_quantize(const float *absmax, size_t nblocks, uint8_t *scale_codes,
                          float *scale_of_scales)
{
    float max_scale = 0.0f;
    for (size_t b = 0; b < nblocks; ++b) max_scale = fmaxf(max_scale, absmax[b]);
    for (size_t b = 0; b < nblocks; ++b) {
        if (max_scale == 0.0f) {
            scale_codes[b] = 0;
        } else {
            float q = roundf(absmax[b] / max_scale * 255.0f);  /* :300 divide, multiply, round */
            if (q < 0.0f) q = 0.0f;                             /* clamp(0, 255); NaN -> 0 as `as u8` does */
            if (q > 255.0f) q = 255.0f;
            scale_codes[b] = (q != q) ? 0 : (uint8_t)q;
        }
    }
    *scale_of_scales = max_scale;
}

/* src/quantize.rs:170-175 and :341-351 -- block_scale. */
float nf4o_block_scale_dq(uint8_t code, float scale_of_scales)
{
    return (float)code / 255.0f * scale_of_scales; /* divide first, then multiply */
}

/* src/quantize.rs:355-366 -- PackedNf4Tensor::dequantize.  Exactly one of
 * (absmax) or (scale_codes, scale_of_scales) describes the scales. */
void nf4o_dequantize_packed(const uint8_t *packed, size_t len, const float *absmax,
                            const uint8_t *scale_codes, float scale_of_scales, float *out)
{
    size_t nb = nf4o_num_blocks(len);
    for (size_t b = 0; b < nb; ++b) {
        float scale = absmax ? absmax[b] : nf4o_block_scale_dq(scale_codes[b], scale_of_scales);
        size_t lo = b * NF4O_BLOCK;
        size_t hi = lo + NF4O_BLOCK < len ? lo + NF4O_BLOCK : len;
        for (size_t i = lo; i < hi; ++i) {
            uint8_t byte = packed[i / 2];                          /* :330-337 */
            uint8_t c = (i % 2 == 0) ? (uint8_t)(byte & 0x0F) : (uint8_t)(byte >> 4);
            out[i] = level(c) * scale;                             /* :362 */
        }
    }
}

/* src/quantize.rs:178-185 -- Nf4Tensor::dequantize (one code per byte). */
void nf4o_dequantize_simulated(const uint8_t *codes, size_t len, const float *absmax,
                               const uint8_t *scale_codes, float scale_of_scales, float *out)
{
    size_t nb = nf4o_num_blocks(len);
    for (size_t b = 0; b < nb; ++b) {
        float scale = absmax ? absmax[b] : nf4o_block_scale_dq(scale_codes[b], scale_of_scales);
        size_t lo = b * NF4O_BLOCK;
        size_t hi = lo + NF4O_BLOCK < len ? lo + NF4O_BLOCK : len;
        for (size_t i = lo; i < hi; ++i) out[i] = level(codes[i]) * scale;
    }
}

/* src/quantize.rs:370-376, :391-399 -- byte accounting. */
size_t nf4o_estimated_resident_bytes(size_t len, int double_quantized)
{
    size_t blocks = nf4o_num_blocks(len);
    size_t scale_bytes = double_quantized ? blocks + 4 : 4 * blocks;
    return (len + 1) / 2 + scale_bytes;
}

/* src/quantize.rs:190-200 -- Nf4Tensor::bits_per_value. */
double nf4o_bits_per_value_simulated(size_t len, int double_quantized)
{
    if (len == 0) return 0.0;
    double payload = 4.0 * (double)len;
    double blocks = (double)nf4o_num_blocks(len);
    double scales = double_quantized ? 8.0 * blocks + 32.0 : 32.0 * blocks;
    return (payload + scales) / (double)len;
}

/* src/quantize.rs:404-416 -- quantize_dequantize_tensor on a flat buffer.
 * `work` holds len code bytes, nblocks floats and nblocks bytes. */
void nf4o_quantize_dequantize(const float *values, size_t len, int double_quantization,
                              float *out, uint8_t *work_codes, float *work_absmax,
                              uint8_t *work_scale_codes)
{
    nf4o_quantize_simulated(values, len, work_codes, work_absmax);
    if (double_quantization) {
        float sos;
        nf4o_double_quantize(work_absmax, nf4o_num_blocks(len), work_scale_codes, &sos);
        nf4o_dequantize_simulated(work_codes, len, NULL, work_scale_codes, sos, out);
    } else {
        nf4o_dequantize_simulated(work_codes, len, work_absmax, NULL, 0.0f, out);
    }
}

/* qwennet.rs:238-241 with the weight layout pinned by qwennet.rs:2196-2211:
 * W is [d_in, d_out] row-major and y[r][o] = sum_i x[r][i] * W[i][o] (+ bias[o]).
 * Accumulates in f64 (the reference's f32 summation order lives in the
 * un-vendored matrixmultiply crate and is not pinned). */
void nf4o_linear_in_out(const float *x, size_t rows, size_t d_in, size_t d_out, const float *w,
                        const float *bias, double *y)
{
    for (size_t r = 0; r < rows; ++r) {
        double *yr = y + r * d_out;
        for (size_t o = 0; o < d_out; ++o) yr[o] = bias ? (double)bias[o] : 0.0;
        for (size_t i = 0; i < d_in; ++i) {
            double xv = (double)x[r * d_in + i];
            const float *wr = w + i * d_out;
            for (size_t o = 0; o < d_out; ++o) yr[o] += xv * (double)wr[o];
        }
    }
}

/* The [d_out, d_in] ("K-contiguous") orientation used by the measured
 * configurations: y[r][o] = sum_i x[r][i] * W[o][i]. */
void nf4o_linear_out_in(const float *x, size_t rows, size_t d_in, size_t d_out, const float *w,
                        const float *bias, double *y)
{
    for (size_t r = 0; r < rows; ++r) {
        for (size_t o = 0; o < d_out; ++o) {
            const float *wr = w + o * d_in;
            const float *xr = x + r * d_in;
            double acc = 0.0;
            for (size_t i = 0; i < d_in; ++i) acc += (double)xr[i] * (double)wr[i];
            y[r * d_out + o] = acc + (bias ? (double)bias[o] : 0.0);
        }
    }
}

/* src/quantize.rs:620-624 -- LoraAdapter::forward: ((x A) B) * (scaling as f32)
 * with A [d_in, rank], B [rank, d_out]; the scale is applied last. */
void nf4o_lora_forward(const float *x, size_t rows, size_t d_in, size_t rank, size_t d_out,
                       const float *a, const float *b, double scaling, double *y)
{
    double s = (double)(float)scaling;
    for (size_t r = 0; r < rows; ++r) {
        double t[512];
        for (size_t j = 0; j < rank && j < 512; ++j) {
            double acc = 0.0;
            for (size_t i = 0; i < d_in; ++i) acc += (double)x[r * d_in + i] * (double)a[i * rank + j];
            t[j] = acc;
        }
        for (size_t o = 0; o < d_out; ++o) {
            double acc = 0.0;
            for (size_t j = 0; j < rank && j < 512; ++j) acc += t[j] * (double)b[j * d_out + o];
            y[r * d_out + o] = acc * s;
        }
    }
}

/* src/quantize.rs:629-634 -- delta_weight = (A B) * scaling, [d_in, d_out]. */
void nf4o_lora_delta_weight(size_t d_in, size_t rank, size_t d_out, const float *a,
                            const float *b, double scaling, double *dw)
{
    double s = (double)(float)scaling;
    for (size_t i = 0; i < d_in; ++i)
        for (size_t o = 0; o < d_out; ++o) {
            double acc = 0.0;
            for (size_t j = 0; j < rank; ++j) acc += (double)a[i * rank + j] * (double)b[j * d_out + o];
            dw[i * d_out + o] = acc * s;
        }
}

/* qwennet.rs:2567-2575 -- the integer LCG the reference uses for fixtures:
 * bit-reproducible inputs in any language. */
void nf4o_lcg_fill(uint64_t *state, float *out, size_t n)
{
    uint64_t s = *state;
    for (size_t i = 0; i < n; ++i) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        uint16_t bits = (uint16_t)(s >> 48);
        out[i] = ((float)bits / (float)65535 - 0.5f) * 0.1f;
    }
    *state = s;
}

/* Round an f32 to the bf16 grid, nearest-even, as src/precision.rs:95-127
 * specifies (finite inputs; overflow goes to infinity). */
float nf4o_round_bf16(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return x; /* inf / nan pass through */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    u &= 0xFFFF0000u;
    float r;
    memcpy(&r, &u, 4);
    return r;
}
