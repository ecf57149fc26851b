// Shared device/host helpers of the NF4 B200 library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nf4_b200.h"
#include "nf4_tables.inc"

namespace nf4 {

constexpr int kBlock = NF4_BLOCK_SIZE;  // values per quantization block
constexpr int kNumSMs = 148;            // B200

// ---- error plumbing (defined in api.cu) ------------------------------------
int32_t fail(int32_t code, const char *fmt, ...);
int32_t check_cuda(cudaError_t e, const char *what);
void count_launch(uint64_t n = 1);

#define NF4_CUDA_TRY(expr)                                         \
    do {                                                           \
        int32_t _st = ::nf4::check_cuda((expr), #expr);            \
        if (_st != NF4_OK) return _st;                             \
    } while (0)

#define NF4_TRY(expr)                  \
    do {                               \
        int32_t _st = (expr);          \
        if (_st != NF4_OK) return _st; \
    } while (0)

// ---- tables -----------------------------------------------------------------
static __device__ __constant__ const uint32_t c_level_bits[16] = {NF4_LEVEL_BITS_LIST};
// the same levels rounded to f16 (bit patterns)
static __device__ __constant__ const uint32_t c_level_f16_bits[16] = {NF4_LEVEL_F16_BITS_LIST};
static const uint32_t h_level_bits[16] = {NF4_LEVEL_BITS_LIST};
static const uint32_t h_threshold_bits[15] = {NF4_THRESHOLD_BITS_LIST};

// Decision thresholds as compile-time immediates (bit patterns from nf4_tables.inc).
struct ThresholdBits {
    uint32_t t[15];
};
__host__ __device__ constexpr ThresholdBits threshold_bits() { return {{NF4_THRESHOLD_BITS_LIST}}; }

template <int I>
__device__ __forceinline__ float T() {
    constexpr ThresholdBits tb = threshold_bits();
    return __uint_as_float(tb.t[I]);
}

// Code of an already-normalised value.  Equals the reference's sixteen-way scan
// (strict '<', lower index on ties) for NaN (code 0) and for every v with
// |v| <= 65536: there the scan's answer is the number of thresholds T_i with
// v >= T_i, found here by a four-step bisection on immediates.  (For much larger |v|
// the f32 differences v - L_i collapse onto each other and the scan drifts back to
// code 0; the quantizer never gets there, because |x| <= absmax makes
// |x / absmax| <= 1 and inf / inf is NaN.)
__device__ __forceinline__ uint32_t code_of_normalized(float v) {
    const bool b3 = v >= T<7>();
    const float t2 = b3 ? T<11>() : T<3>();
    const bool b2 = v >= t2;
    const float t1 = b3 ? (b2 ? T<13>() : T<9>()) : (b2 ? T<5>() : T<1>());
    const bool b1 = v >= t1;
    const float t0hi = b2 ? (b1 ? T<14>() : T<12>()) : (b1 ? T<10>() : T<8>());
    const float t0lo = b2 ? (b1 ? T<6>() : T<4>()) : (b1 ? T<2>() : T<0>());
    const float t0 = b3 ? t0hi : t0lo;
    const bool b0 = v >= t0;
    return (b3 ? 8u : 0u) | (b2 ? 4u : 0u) | (b1 ? 2u : 0u) | (b0 ? 1u : 0u);
}

// The reference's literal scan; used by the self-check kernel only.
__device__ __forceinline__ uint32_t code_by_scan(float v) {
    uint32_t best = 0;
    float best_dist = __int_as_float(0x7f800000);
    #pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float d = fabsf(__fsub_rn(v, __uint_as_float(c_level_bits[i])));
        if (d < best_dist) {
            best_dist = d;
            best = i;
        }
    }
    return best;
}

// Code of one raw value given its block's absmax (src/quantize.rs:109-112).
__device__ __forceinline__ uint32_t code_of(float x, float absmax) {
    if (absmax == 0.0f) return 7u;  // nearest level to 0.0
    return code_of_normalized(__fdiv_rn(x, absmax));
}

// ---- fast code selection ------------------------------------------------------------------
// Thirty-two uniform cells over [-1, 1); a cell holds at most one decision threshold.  One word
// per cell: the f32 threshold inside the cell with its low four mantissa bits replaced by the
// number of thresholds below the cell (the threshold moves by < 9e-7), or 1.7e38 | count for a
// cell that holds none.
static __device__ __constant__ const uint32_t c_cell_table[32] = {NF4_CELL_TABLE_LIST};

// Code of x / absmax without the division, when that is provably safe.
//   q = x * rcp with rcp = fl(1 / absmax) lies within 1.8e-7 of the correctly rounded quotient
//   (|x| <= absmax, both roundings <= 2^-24 relative).  The cell of q names the only threshold
//   that can matter; when q is more than 3e-6 away from the table's (slightly moved) copy of
//   it, q and the exact quotient are on the same side of the true threshold and the code is
//   `count + (q >= threshold)`.  Otherwise -- next to a threshold, NaN, or a scale outside
//   [1e-30, 1e30] where rcp is not trustworthy (the caller starts `unsure` as true for those)
//   -- the exact path decides.
// `cells` is the table in shared memory (32 words, one bank each: no conflicts).  Cell rounding
// can put q in a neighbouring cell only within 2e-6 of a cell edge, and no threshold is within
// 1e-4 of an edge, so the count is unaffected.
// Out of line on purpose: taken for a few values in a million, and inlining sixteen copies of
// the division and the bisection doubles the quantize kernel's register count.
static __device__ __noinline__ uint32_t code_of_exact(float x, float absmax) { return code_of(x, absmax); }

// `unsure` is set (never cleared) when the value sits next to a threshold or is NaN; the caller
// then redoes its values with code_of_exact.  Keeping the decision out of this function leaves
// the common path branch-free.
__device__ __forceinline__ uint32_t code_of_fast(float x, float rcp, const uint32_t *cells,
                                                 bool &unsure) {
    const float q = __fmul_rn(x, rcp);
    int c = __float2int_rz(fmaf(q, 16.0f, 16.0f));  // NaN -> 0
    c = min(max(c, 0), 31);
    const uint32_t e = cells[c];
    const float d = q - __uint_as_float(e);
    unsure |= !(fabsf(d) > 3e-6f);
    return (e & 15u) + (d >= 0.0f ? 1u : 0u);
}

// Scale of a double-quantized block: divide first, then multiply (src/quantize.rs:348).
__device__ __forceinline__ float dq_scale(uint32_t code, float scale_of_scales) {
    return __fmul_rn(__fdiv_rn((float)code, 255.0f), scale_of_scales);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace nf4
