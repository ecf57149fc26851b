// Prefill path: y[M, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T) for many rows of x,
// W stored as packed NF4 [N, K] with 64-blocks along K.  A dense contraction: tensor-core
// bound, built on tcgen05.mma with the dequantised weight operand and the accumulator in
// tensor memory (TMEM) and the activations in shared memory.
//
// Roles inside one persistent CTA (one per SM, 864 threads):
//   warp 0      TMA producer: x tiles [256 rows x 64 k] (f16, 128B-swizzled, K-major) into a
//               4-deep shared-memory ring; after the K loop the same ring carries the LoRA
//               intermediate T (bf16 hi / lo halves) and a second small ring the matching
//               128 x 64 tiles of LoRA B, so the adapter is just more k-steps (with both
//               operands in shared memory).
//   warp 1      owns TMEM (alloc/dealloc); one of its threads issues the tcgen05.mma of the even
//               k-stages, one thread of warp 6 those of the odd ones.  Issuing a stage's MMAs
//               holds the thread for about as long as they run, and waits, fences and commits
//               separate two batches; with two threads the second has done its waiting while
//               the first issues, and only a short hand-over is left.
//   warps 2-5, 23-26  epilogue: TMEM -> registers -> (* row scale, + bias) -> bf16/f32 ->
//               shared -> TMA store.
//   warps 7-22  dequantisers, four groups of 128 threads taking every fourth k-stage.  A thread
//               owns one weight row (= one TMEM lane; a warp may only touch the lane quarter its
//               number names): it reads the row's 32 packed bytes and the block scale straight
//               from global memory (L2), expands the nibbles with byte-permute lookups held in
//               registers, multiplies by the scale in f16x2 and writes the 64 f16 values into
//               its lane of an eight-deep ring of TMEM columns with tcgen05.st.
//
// Why the weight operand lives in TMEM.  An MMA of 128 x 256 x 16 with both operands in shared
// memory reads 12 KB per 128 cycles, and the TMA and the dequantisers write as much again: more
// than the 128 B/clk a shared memory delivers, so the k-stage was bound by shared-memory traffic.
// With the 128-row operand in TMEM the shared memory carries only the activation tile (written
// once, read once), and the dequantised weight never touches it.  The price: the accumulator
// (256 columns) and the weight ring (8 x 32 columns) share the 512 TMEM columns, so there is one
// accumulator and the MMAs of the next tile wait while the epilogue reads it out.
//
// The MMA computes D[n, m] = sum_k W[n, k] x[m, k]: weight rows are the MMA's M (TMEM lanes),
// activation rows its N (256 accumulator columns).  Both operands are f16 with f32 accumulation:
// rounding the dequantised weight to bf16 instead would cost ~1.6e-3 relative error, above the
// 1e-3 parity bar, while f16 costs ~3e-4.  The bf16 activations are converted to f16 by a
// pre-pass (exact for every value inside f16's range; a row whose largest magnitude exceeds 32768
// or lies below 2^-8 is divided by a power of two that the epilogue multiplies back), which also
// produces the LoRA intermediate.
//
// The other orientation (W [K][N] with the 64-blocks along N, the reference's own; f32 or bf16
// activations) comes through the same GEMM at more than 16 rows: three small kernels first write the
// transposed nibbles, the scales as f16 [N / 64][K] and the adapter factors in this kernel's
// orientation into the workspace (the nibbles exactly; the scales with the rounding the dequantisers
// apply anyway).  A weight row's scale then changes with every k: a lane loads the pair of scales of
// k = 2 lane, 2 lane + 1 of its stage (one 128-byte line per warp) and the warp hands them round
// with shuffles while it multiplies (template parameter PERK).  f32 activations are converted to f16
// directly, every row divided by its own power of two.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

__device__ int g_prefill_error = 0;  // set when a bounded wait gives up
__device__ int *g_prefill_error_host = nullptr;  // the same, in mapped host memory (set by the host-pointer entry points)


namespace {

constexpr int BM = 128;        // weight rows per tile (MMA M, TMEM lanes)
constexpr int BN = 256;        // activation rows per tile (MMA N, accumulator columns)
constexpr int BK = 64;         // k per stage = one quantization block = one 128B swizzle row
constexpr int kXStages = 4;    // shared-memory ring of activation tiles
constexpr int kLoraStages = 2; // shared-memory ring of LoRA B tiles (adapter k-stages)
constexpr int kAStages = 8;    // TMEM ring of dequantised weight stages
constexpr int kAStageCols = BK / 2;  // 32 columns: two f16 per 32-bit cell
constexpr int kAccCols = BN;   // the accumulator: columns [0, 256); the weight ring follows
constexpr int kTmemCols = 512;
constexpr int kXTileBytes = BN * BK * 2;   // 32 KB: activations, written by TMA
constexpr int kLoraTileBytes = BM * BK * 2;  // 16 KB: 128 rows of LoRA B x 64 ranks, written by TMA

constexpr int kEpiBytes = 64 * 1024;       // output staging: a whole tile of bf16, half a tile of f32
constexpr int kThreads = 27 * 32;
constexpr int kFirstExpanderWarp = 7;      // sixteen warps
constexpr int kFirstEpilogueWarpB = 23;    // the second set of four epilogue warps
constexpr int kExpanderGroups = 4;         // of four warps (one per TMEM lane quarter) each
constexpr uint64_t kInOutMinRows = 17;     // the other weight orientation comes here from this many rows on

// barrier slots
constexpr int kBarXFull = 0, kBarXEmpty = kBarXFull + kXStages, kBarAFull = kBarXEmpty + kXStages,
              kBarAEmpty = kBarAFull + kAStages, kBarAccFull = kBarAEmpty + kAStages,
              kBarAccEmpty = kBarAccFull + 1, kBarIssued = kBarAccEmpty + 1, kBarLEmpty = kBarIssued + 2,
              kNumBars = kBarLEmpty + kLoraStages;

struct PrefillParams {
    const uint8_t *codes;
    const float *absmax;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const float *bias;
    const float *row_scale;       // [M] power-of-two factor each activation row was divided by
    // Weights that came in the other orientation ([d_in][d_out], blocks along d_out) are repacked
    // before the GEMM: `codes` then holds the transposed nibbles, and a weight's scale depends on
    // k, not on the k-stage: scales_t[n / 64][k] as f16, already divided by the weight's power of two.
    const __half *scales_t;
    uint32_t M, N, K, rank;
    uint32_t lora_chunks;  // ceil(rank / 64); T is [M][2 * 64 * lora_chunks] (hi halves, then lo)
    uint32_t m_tiles, n_tiles;
    // Work of a CTA: first its share of the `sk_tiles` tiles whose k-stages all CTAs divide
    // evenly between them (a tile can be split between neighbouring CTAs), then `dp_rounds`
    // whole tiles.  A CTA that multiplies the leading stages of a tile leaves its accumulator
    // in `partial` ([CTA][BN][BM] f32) and raises its word of `sk_flags`; the CTA that multiplies
    // the last stages adds those and finishes the tile.
    uint32_t sk_tiles, dp_rounds;
    float *partial;
    uint32_t *sk_flags;
    uint32_t wait_ns;  // bound of the wait for a neighbour's flag
};

// This CTA's list of segments (tile, main k-stages [b, e)), in the order they are worked on: the
// shared tiles from the last to the first -- a piece without a tile's last stage comes first and
// waits for nobody; the piece with the last stage of a tile that a neighbour began comes last of
// them -- then the whole tiles.
struct WorkList {
    uint64_t u0, u1;   // this CTA's range of main stages of the shared tiles
    uint32_t ks;       // main stages per tile
    uint32_t t_first, t_last, n_shared, n_seg, sk_tiles, cta, ctas;

    __host__ __device__ void init(const PrefillParams &p, uint32_t k_stages, uint32_t cta_, uint32_t ctas_) {
        ks = k_stages;
        cta = cta_;
        ctas = ctas_;
        sk_tiles = p.sk_tiles;
        const uint64_t all = (uint64_t)p.sk_tiles * ks;
        u0 = all * cta / ctas;
        u1 = all * (cta + 1) / ctas;
        n_shared = 0;
        t_first = t_last = 0;
        if (u1 > u0) {
            t_first = (uint32_t)(u0 / ks);
            t_last = (uint32_t)((u1 - 1) / ks);
            n_shared = t_last - t_first + 1;
        }
        n_seg = n_shared + p.dp_rounds;
    }
    __host__ __device__ static uint64_t range_begin(uint64_t all, uint32_t c, uint32_t n) { return all * c / n; }
    __host__ __device__ void get(uint32_t j, uint32_t &tile, uint32_t &b, uint32_t &e) const {
        if (j < n_shared) {
            tile = t_last - j;
            const uint64_t t0 = (uint64_t)tile * ks;
            b = (uint32_t)((u0 > t0 ? u0 : t0) - t0);
            e = (uint32_t)((u1 < t0 + ks ? u1 : t0 + ks) - t0);
        } else {
            tile = sk_tiles + (j - n_shared) * ctas + cta;
            b = 0;
            e = ks;
        }
    }
};

// ---- descriptors -----------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 B apart,
// 8-row groups 1024 B apart (SBO), version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                              // LBO (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                    // SBO, bits [32,46)
    d |= (uint64_t)1 << 46;                              // descriptor version
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16: f32 accumulate, K-major A and B.
// a_fmt / b_fmt: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m,
                                                  uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- TMEM load (32 lanes x 32-bit, 16 consecutive columns) -------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,"
        "%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// ---- TMEM store (32 lanes x 32-bit, 32 consecutive columns) ------------------------------
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&a)[16],
                                          const uint32_t (&b)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,"
        "%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]),
        "r"(a[7]), "r"(a[8]), "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]),
        "r"(a[15]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]),
        "r"(b[7]), "r"(b[8]), "r"(b[9]), "r"(b[10]), "r"(b[11]), "r"(b[12]), "r"(b[13]), "r"(b[14]),
        "r"(b[15])
        : "memory");
}

// ---- nibble -> f16 expansion with byte-permute lookups --------------------------------
// The sixteen f16 levels are split into a table of high bytes and a table of low bytes, four
// registers each.  One prmt looks four nibbles up in an 8-entry half table; a third prmt picks,
// per nibble, the half its top bit names; a last pair interleaves high and low bytes.
struct LevelTables {
    uint32_t hi[4], lo[4];
};

__device__ __forceinline__ LevelTables make_level_tables() {
    LevelTables t;
    #pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t h = 0, l = 0;
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t bits = __half_as_ushort(
                __float2half_rn(__uint_as_float(c_level_bits[4 * q + i])));
            h |= (bits >> 8) << (8 * i);
            l |= (bits & 0xffu) << (8 * i);
        }
        t.hi[q] = h;
        t.lo[q] = l;
    }
    return t;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Four nibbles (bits 0..15 of `w4`) -> two f16x2 registers {e0,e1}, {e2,e3}.
__device__ __forceinline__ void expand4(const LevelTables &t, uint32_t w4, uint32_t &out01,
                                        uint32_t &out23) {
    const uint32_t sel = w4 & 0x7777u;
    const uint32_t pick = ((w4 & 0x8888u) >> 1) | 0x3210u;
    const uint32_t h = prmt(prmt(t.hi[0], t.hi[1], sel), prmt(t.hi[2], t.hi[3], sel), pick);
    const uint32_t l = prmt(prmt(t.lo[0], t.lo[1], sel), prmt(t.lo[2], t.lo[3], sel), pick);
    out01 = prmt(l, h, 0x5140u);
    out23 = prmt(l, h, 0x7362u);
}

__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Half a stage of one weight row: 16 packed bytes + scale -> 16 registers of f16x2.
__device__ __forceinline__ void expand_half(const LevelTables &t, const uint4 &c, float scale,
                                            uint32_t (&out)[16]) {
    const __half2 s2 = __float2half2_rn(scale);
    const uint32_t s = *reinterpret_cast<const uint32_t *>(&s2);
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a, b, c2, d;
        expand4(t, w[i], a, b);
        expand4(t, w[i] >> 16, c2, d);
        out[4 * i + 0] = hmul2(a, s);
        out[4 * i + 1] = hmul2(b, s);
        out[4 * i + 2] = hmul2(c2, s);
        out[4 * i + 3] = hmul2(d, s);
    }
}

// The same with a scale per k: lane j of the warp holds the f16 pair of scales of k = 2j, 2j + 1
// of this stage (`pairs`); `first` is the pair that goes with out[0].
__device__ __forceinline__ void expand_half_per_k(const LevelTables &t, const uint4 &c, uint32_t pairs,
                                                  int first, uint32_t (&out)[16]) {
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a, b, c2, d;
        expand4(t, w[i], a, b);
        expand4(t, w[i] >> 16, c2, d);
        out[4 * i + 0] = hmul2(a, __shfl_sync(0xffffffffu, pairs, first + 4 * i + 0));
        out[4 * i + 1] = hmul2(b, __shfl_sync(0xffffffffu, pairs, first + 4 * i + 1));
        out[4 * i + 2] = hmul2(c2, __shfl_sync(0xffffffffu, pairs, first + 4 * i + 2));
        out[4 * i + 3] = hmul2(d, __shfl_sync(0xffffffffu, pairs, first + 4 * i + 3));
    }
}

struct RowStage {
    uint4 c0, c1;  // the row's 64 packed codes of one k-stage
    float scale;   // PERK: the bits of this lane's pair of f16 scales
};

// The tensor-core GEMM scales the expanded levels in f16, so block scales must sit inside f16's
// normal range (6.1e-5 .. 65504).  Both kernels therefore work with scales divided by 2^e, e the
// exponent of the weight's first block scale (the scales of one weight lie within a few powers of
// two of each other), and the outputs are multiplied back by 2^e: the pre-pass folds 2^e into the
// rows' factors and 2^-e into the adapter intermediate.  Powers of two: every step is exact.
__device__ __forceinline__ int weight_exponent(const float *absmax, const uint8_t *scale_codes,
                                               const float *scale_of_scales) {
    const float s0 = absmax ? __ldg(absmax) : dq_scale(__ldg(scale_codes), __ldg(scale_of_scales));
    if (!(s0 > 0.0f) || s0 >= __int_as_float(0x7f800000)) return 0;
    int e;
    frexpf(s0, &e);  // s0 = f * 2^e, f in [0.5, 1)
    return min(max(e, -100), 100);
}

template <bool YF32, bool PERK>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_t,
               const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_y,
               const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled operand tiles
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *x_ring = smem;                                   // kXStages activation tiles
    uint8_t *lora_ring = x_ring + kXStages * kXTileBytes;     // kLoraStages tiles of LoRA B
    uint8_t *epi = lora_ring + kLoraStages * kLoraTileBytes;  // output staging, 64 KB
    constexpr int kStageRows = kEpiBytes / (BM * (YF32 ? 4 : 2));  // activation rows per staging pass
    uint64_t *bars = reinterpret_cast<uint64_t *>(epi + kEpiBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
    float *row_scales = reinterpret_cast<float *>(bars + kNumBars + 2);  // BN factors of the tile's rows

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t bar0 = ptx::smem_addr(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    const uint32_t k_stages = p.K / BK;
    const uint32_t lora_stages = 2 * p.lora_chunks;  // adapter k-stages per tile: hi and lo halves of T
    WorkList wl;
    wl.init(p, k_stages, blockIdx.x, gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kXStages; ++s) {
            ptx::mbar_init(bar(kBarXFull + s), 1);
            ptx::mbar_init(bar(kBarXEmpty + s), 1);
        }
        for (int s = 0; s < kAStages; ++s) {
            ptx::mbar_init(bar(kBarAFull + s), 4);  // the four warps writing the stage
            ptx::mbar_init(bar(kBarAEmpty + s), 1);
        }
        ptx::mbar_init(bar(kBarAccFull), 1);
        ptx::mbar_init(bar(kBarAccEmpty), 8);
        ptx::mbar_init(bar(kBarIssued + 0), 1);
        ptx::mbar_init(bar(kBarIssued + 1), 1);
        for (int s = 0; s < kLoraStages; ++s) ptx::mbar_init(bar(kBarLEmpty + s), 1);
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tmap(&tmap_x);
        ptx::prefetch_tmap(&tmap_y);
        if (p.lora_chunks) {
            ptx::prefetch_tmap(&tmap_t);
            ptx::prefetch_tmap(&tmap_b);
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_acc = tmem_base;             // columns [0, 256)
    const uint32_t tmem_a = tmem_base + kAccCols;    // kAStages x 32 columns

    bool ok = true;

    if (warp == 0) {
        // ============================ TMA producer ============================
        if (lane == 0) {
            // the f16 activations and T come from the pre-pass, which may still be running: this
            // kernel is its programmatic dependent (the dequantisers start on the weights at once)
            ptx::pdl_wait();
            uint32_t cnt = 0, lcnt = 0;
            for (uint32_t seg = 0; seg < wl.n_seg && ok; ++seg) {
                uint32_t tile, kb, ke;
                wl.get(seg, tile, kb, ke);
                const uint32_t m0 = (tile % p.m_tiles) * BN, n0 = (tile / p.m_tiles) * BM;
                // the adapter's stages follow a tile's last main stage
                const uint32_t k_end = ke == k_stages ? k_stages + lora_stages : ke;
                for (uint32_t ks = kb; ks < k_end; ++ks, ++cnt) {
                    const uint32_t s = cnt % kXStages, ph = (cnt / kXStages) & 1u;
                    if (!ptx::mbar_wait_suspended(bar(kBarXEmpty + s), ph ^ 1u)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst = ptx::smem_addr(x_ring + s * kXTileBytes);
                    if (ks < k_stages) {
                        ptx::mbar_arrive_expect_tx(bar(kBarXFull + s), kXTileBytes);
                        ptx::tma_load_2d(dst, &tmap_x, (int32_t)(ks * BK), (int32_t)m0,
                                         bar(kBarXFull + s));
                    } else {
                        // adapter stage: a tile of T beside the activations' ring slot and the
                        // matching 128 x 64 tile of LoRA B (ranks beyond the adapter's read as
                        // zero) as the MMA's other shared-memory operand
                        const uint32_t j = ks - k_stages;
                        const uint32_t ls = lcnt % kLoraStages, lph = (lcnt / kLoraStages) & 1u;
                        ++lcnt;
                        if (!ptx::mbar_wait_suspended(bar(kBarLEmpty + ls), lph ^ 1u)) {
                            ok = false;
                            break;
                        }
                        ptx::mbar_arrive_expect_tx(bar(kBarXFull + s), kXTileBytes + kLoraTileBytes);
                        ptx::tma_load_2d(dst, &tmap_t, (int32_t)(j * BK), (int32_t)m0, bar(kBarXFull + s));
                        ptx::tma_load_2d(ptx::smem_addr(lora_ring + ls * kLoraTileBytes), &tmap_b,
                                         (int32_t)((j % p.lora_chunks) * BK), (int32_t)n0,
                                         bar(kBarXFull + s));
                    }
                }
            }
            if (!ok) NF4_REPORT_FAILURE(g_prefill_error, g_prefill_error_host, 1);
        }
    } else if (warp == 1 || warp == 6) {
        // ============================= MMA issuers =============================
        // Thread `me` (0: warp 1, 1: warp 6) issues the stages whose global counter has its
        // parity.  Stage c may only be issued after stage c - 1 has been (hand-over barrier
        // kBarIssued + parity of c - 1), which keeps the MMAs of the accumulator in order.
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            constexpr uint32_t idesc_main = make_idesc(0, 0, BM, BN);  // f16 x f16
            constexpr uint32_t idesc_lora = make_idesc(1, 1, BM, BN);  // bf16 x bf16
            const uint32_t x_addr = ptx::smem_addr(x_ring);
            uint32_t cnt = 0, a_next = 0, l_next = 0;  // stages, main stages, adapter stages so far
            for (uint32_t seg = 0; seg < wl.n_seg && ok; ++seg) {
                uint32_t tile, kb, ke;
                wl.get(seg, tile, kb, ke);
                const uint32_t k_end = ke == k_stages ? k_stages + lora_stages : ke;
                for (uint32_t ks = kb; ks < k_end; ++ks, ++cnt) {
                    // the weight ring counts main stages only, the LoRA ring adapter stages only
                    const bool main_stage = ks < k_stages;
                    const uint32_t acnt = a_next, lcnt = l_next;
                    if (main_stage) ++a_next;
                    else ++l_next;
                    if ((cnt & 1u) != me) continue;
                    const uint32_t sx = cnt % kXStages, phx = (cnt / kXStages) & 1u;
                    const uint32_t sa = acnt % kAStages, pha = (acnt / kAStages) & 1u;
                    const uint32_t ls = lcnt % kLoraStages;
                    // the epilogue must have read the previous segment out of the accumulator
                    if (ks == kb && !ptx::mbar_wait_suspended(bar(kBarAccEmpty), (seg & 1u) ^ 1u)) {
                        ok = false;
                        break;
                    }
                    if (!ptx::mbar_wait_suspended(bar(kBarXFull + sx), phx)) {
                        ok = false;
                        break;
                    }
                    if (main_stage && !ptx::mbar_wait_suspended(bar(kBarAFull + sa), pha)) {
                        ok = false;
                        break;
                    }
                    // hand-over: the other thread has issued stage cnt - 1 (its (cnt-1)/2-th)
                    if (cnt > 0 &&
                        !ptx::mbar_wait_suspended(bar(kBarIssued + (me ^ 1u)), ((cnt - 1) >> 1) & 1u)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint64_t bdesc = make_kmajor_sw128_desc(x_addr + sx * kXTileBytes);
                    const uint32_t a_cols = tmem_a + sa * kAStageCols;
                    if (main_stage) {
                        // 16 k = 8 TMEM columns of the weight stage = 32 bytes inside the
                        // activation tile's swizzled row (+2 in the encoded address)
                        ptx::mma_ts_f16(tmem_acc, a_cols, bdesc, idesc_main, ks != kb ? 1u : 0u);
                        ptx::mma_ts_f16(tmem_acc, a_cols + 8, bdesc + 2, idesc_main, 1u);
                        ptx::mma_ts_f16(tmem_acc, a_cols + 16, bdesc + 4, idesc_main, 1u);
                        ptx::mma_ts_f16(tmem_acc, a_cols + 24, bdesc + 6, idesc_main, 1u);
                    } else {
                        const uint32_t chunk = (ks - k_stages) % p.lora_chunks;
                        const uint32_t left = p.rank - chunk * 64;
                        const uint32_t nk16 = ((left < 64 ? left : 64) + 15) / 16;
                        const uint64_t adesc =
                            make_kmajor_sw128_desc(ptx::smem_addr(lora_ring) + ls * kLoraTileBytes);
                        for (uint32_t j = 0; j < nk16; ++j)
                            ptx::mma_ss_f16(tmem_acc, adesc + 2 * j, bdesc + 2 * j, idesc_lora, 1u);
                    }
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(bar(kBarIssued + me));
                    ptx::tc_commit(bar(kBarXEmpty + sx));
                    ptx::tc_commit(main_stage ? bar(kBarAEmpty + sa) : bar(kBarLEmpty + ls));
                    if (ks + 1 == k_end) ptx::tc_commit(bar(kBarAccFull));
                }
            }
            if (!ok) NF4_REPORT_FAILURE(g_prefill_error, g_prefill_error_host, 2);
        }
    } else if (warp < 6 || warp >= kFirstEpilogueWarpB) {
        // ============================== epilogue ==============================
        // The MMAs of the next tile wait for the accumulator, so it is read out as fast as eight
        // warps can (two per TMEM lane quarter, each taking half of the columns): the whole tile
        // (bf16) or half of it (f32) goes through one 64 KB staging buffer, two TMEM loads in
        // flight per warp, and the accumulator is handed back before the last values are
        // converted; the TMA store of the tile then overlaps the next tile's MMAs.
        const uint32_t set = warp >= kFirstEpilogueWarpB ? 1u : 0u;
        const uint32_t q = warp & 3u;  // TMEM lane quarter this warp may touch
        const uint32_t row_in_tile = q * 32 + lane;
        const uint32_t epi_thread = set * 128 + (warp - (set ? kFirstEpilogueWarpB : 2)) * 32 + lane;
        const uint32_t epi_leader = (warp == 2 && lane == 0);
        const uint32_t acc_lane = tmem_acc + ((q * 32) << 16);
        // this warp's eight 16-column TMEM loads of a tile: within every staging pass the first
        // set takes the first half of the pass's activation rows, the second set the other half
        constexpr uint32_t kHalfRows = kStageRows / 2, kPerPass = kHalfRows / 16;
        constexpr uint32_t kLoads = BN / 2 / 16;
        auto col_of = [&](uint32_t k) {
            return (k / kPerPass) * kStageRows + set * kHalfRows + (k % kPerPass) * 16;
        };
        ptx::pdl_wait();  // the rows' factors come from the pre-pass, which also cleared the flags
        float *own_partial = p.partial + (size_t)blockIdx.x * (BM * BN) + row_in_tile;
        for (uint32_t seg = 0; seg < wl.n_seg && ok; ++seg) {
            const uint32_t i = seg;  // the accumulator's barriers alternate per segment
            uint32_t tile, kb, ke;
            wl.get(seg, tile, kb, ke);
            const uint32_t n0 = (tile / p.m_tiles) * BM, m0 = (tile % p.m_tiles) * BN;
            const uint32_t n = n0 + row_in_tile;
            if (ke != k_stages) {
                // The leading stages of a tile that a neighbour finishes: the raw sums go to this
                // CTA's place in global memory ([activation row][weight row]: a warp's stores are
                // whole lines; a thread's values 64 bytes in a row were measured 15 % slower over
                // the whole GEMM), then the flag goes up.
                ok = ptx::mbar_wait_suspended(bar(kBarAccFull), i & 1u);
                if (!ok) break;
                ptx::tc_fence_after();
                uint32_t v[16];
                for (uint32_t k = 0; k < kLoads; ++k) {
                    tmem_ld16(acc_lane + col_of(k), v);
                    ptx::tmem_wait_ld();
                    float *dst = own_partial + (size_t)col_of(k) * BM;
                    #pragma unroll
                    for (int r = 0; r < 16; ++r) dst[r * BM] = __uint_as_float(v[r]);
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(kBarAccEmpty));
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (epi_leader) {
                    __threadfence();
                    atomicExch(p.sk_flags + blockIdx.x, 1u);
                }
                continue;
            }
            // a tile whose leading stages other CTAs multiplied: the CTAs before this one, back to
            // the one that began the tile
            uint32_t first_helper = blockIdx.x;
            if (kb != 0) {
                const uint64_t all = (uint64_t)wl.sk_tiles * k_stages, t0 = (uint64_t)tile * k_stages;
                do {
                    --first_helper;
                } while (first_helper > 0 && WorkList::range_begin(all, first_helper, gridDim.x) > t0);
            }
            const float bias = (p.bias && n < p.N) ? __ldg(p.bias + n) : 0.0f;
            // the rows' factors go to shared memory while the MMAs still run: a global load per
            // value inside the read-out would wait for L2 every time (the L1 left beside 227 KB
            // of shared memory is small and the dequantisers stream through it)
            row_scales[epi_thread] = m0 + epi_thread < p.M ? __ldg(p.row_scale + m0 + epi_thread) : 1.0f;
            ok = ptx::mbar_wait_suspended(bar(kBarAccFull), i & 1u);
            if (!ok) break;
            ptx::tc_fence_after();
            uint32_t va[16], vb[16];
            tmem_ld16(acc_lane + col_of(0), va);
            // staging layout: [kStageRows activation rows][BM weight rows]
            auto stage_chunk = [&](const uint32_t (&v)[16], uint32_t col) {
                const uint32_t r0 = col % kStageRows;
                // the factors first, as vectors: a load per value between the stores could not be
                // moved ahead of them (both are shared memory) and each would wait out its latency
                float rs[16];
                #pragma unroll
                for (int r4 = 0; r4 < 4; ++r4) {
                    const float4 f4 = reinterpret_cast<const float4 *>(row_scales + col)[r4];
                    rs[4 * r4 + 0] = f4.x;
                    rs[4 * r4 + 1] = f4.y;
                    rs[4 * r4 + 2] = f4.z;
                    rs[4 * r4 + 3] = f4.w;
                }
                #pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const float f = fmaf(__uint_as_float(v[r]), rs[r], bias);
                    if (YF32)
                        reinterpret_cast<float *>(epi)[(r0 + r) * BM + row_in_tile] = f;
                    else
                        reinterpret_cast<__nv_bfloat16 *>(epi)[(r0 + r) * BM + row_in_tile] =
                            __float2bfloat16_rn(f);
                }
            };
            // the helpers' sums for sixteen activation rows of this thread's weight row
            auto add_helpers = [&](uint32_t (&v)[16], uint32_t col) {
                for (uint32_t h = first_helper; h < blockIdx.x; ++h) {
                    const float *src = p.partial + (size_t)h * (BM * BN) + (size_t)col * BM + row_in_tile;
                    float part[16];
                    #pragma unroll
                    for (int r = 0; r < 16; ++r) part[r] = __ldcg(src + r * BM);
                    #pragma unroll
                    for (int r = 0; r < 16; ++r) v[r] = __float_as_uint(__uint_as_float(v[r]) + part[r]);
                }
            };
            if (first_helper != blockIdx.x && epi_leader) {
                // bounded wait for the helpers' flags (they dumped before anything else they did)
                const uint64_t t_begin = ptx::global_timer_ns();
                for (uint32_t h = first_helper; h < blockIdx.x && ok; ++h) {
                    while (ptx::ld_acquire_gpu_u32(p.sk_flags + h) == 0u) {
                        if (ptx::global_timer_ns() - t_begin > (uint64_t)p.wait_ns) {
                            ok = false;
                            break;
                        }
                        __nanosleep(64);
                    }
                }
                if (!ok) NF4_REPORT_FAILURE(g_prefill_error, g_prefill_error_host, 5);  // the sums are wrong; the flag says so
                ok = true;  // the read-out goes on (every role must finish its segments)
            }
            for (uint32_t k = 0; k < kLoads; k += 2) {
                if (k % kPerPass == 0) {
                    // the TMA store that last read the staging buffer must be done with it
                    if (epi_leader) ptx::tma_store_wait_read<0>();
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                }
                ptx::tmem_wait_ld();
                tmem_ld16(acc_lane + col_of(k + 1), vb);
                if (first_helper != blockIdx.x) add_helpers(va, col_of(k));
                stage_chunk(va, col_of(k));
                ptx::tmem_wait_ld();
                if (first_helper != blockIdx.x) add_helpers(vb, col_of(k + 1));
                if (k + 2 < kLoads) {
                    tmem_ld16(acc_lane + col_of(k + 2), va);
                } else {
                    // this warp's part of the accumulator is read: hand it back to the MMA threads
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(kBarAccEmpty));
                }
                stage_chunk(vb, col_of(k + 1));
                if ((k + 2) % kPerPass == 0) {
                    ptx::fence_proxy_async();
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (epi_leader) {
                        ptx::tma_store_2d(&tmap_y, ptx::smem_addr(epi), (int32_t)n0,
                                          (int32_t)(m0 + (k / kPerPass) * kStageRows));
                        ptx::tma_store_commit();
                    }
                }
            }
        }
        if (epi_leader) ptx::tma_store_wait<0>();
        if (!ok && lane == 0) NF4_REPORT_FAILURE(g_prefill_error, g_prefill_error_host, 3);
    } else if (warp >= kFirstExpanderWarp && warp < kFirstEpilogueWarpB) {
        // ============================ dequantisers ============================
        // Four groups of four warps; group g takes the main stages (adapter stages need no
        // dequantiser) whose running number over this CTA's tiles is g modulo 4.
        // Within a group the warp's number modulo 4 names the TMEM lane quarter it may write, and
        // the lane the weight row: 32 packed bytes + the scale in, 64 f16 values out, stored as
        // 32 TMEM columns (two f16 per cell, even k in the low half) of the stage's ring slot.
        const uint32_t group = (warp - kFirstExpanderWarp) >> 2;
        const uint32_t q = warp & 3u;
        const uint32_t row_in_tile = q * 32 + lane;
        const LevelTables tables = make_level_tables();
        const float sos = p.scale_codes ? __ldg(p.scale_of_scales) : 0.0f;
        // block scales are used divided by a power of two (see weight_exponent)
        const float w_down = ldexpf(1.0f, -weight_exponent(p.absmax, p.scale_codes, p.scale_of_scales));
        const uint32_t blocks_per_row = p.K / 64;
        const uint32_t total = (uint32_t)(wl.u1 - wl.u0) + p.dp_rounds * k_stages;  // main stages of this CTA
        const uint32_t lane_base = tmem_a + ((q * 32) << 16);

        // Stage positions are walked, not divided out: a 64-bit division per stage costs more
        // than the expansion itself.
        struct Pos {
            uint32_t cnt, seg, ks, ke, n;  // running main-stage number, segment, stage in tile, the segment's end, weight row
        };
        auto enter = [&](Pos &pos, uint32_t over) {  // to segment pos.seg, `over` stages in
            uint32_t tile, kb, ke;
            wl.get(pos.seg, tile, kb, ke);
            pos.ks = kb + over;
            pos.ke = ke;
            pos.n = (tile / p.m_tiles) * BM + row_in_tile;
        };
        auto settle = [&](Pos &pos) {
            while (pos.ks >= pos.ke) {
                const uint32_t over = pos.ks - pos.ke;
                if (++pos.seg >= wl.n_seg) {  // past the last segment
                    pos.cnt = total;
                    return;
                }
                enter(pos, over);
            }
        };
        auto advance = [&](Pos &pos) {
            pos.cnt += kExpanderGroups;
            pos.ks += kExpanderGroups;
            settle(pos);
        };
        auto fetch = [&](const Pos &pos, RowStage &rs) {
            rs.c0 = rs.c1 = make_uint4(0, 0, 0, 0);
            rs.scale = 0.0f;
            if (pos.cnt >= total) return;
            const uint32_t ks = pos.ks, n = pos.n;
            if (n >= p.N) return;
            const uint4 *src = reinterpret_cast<const uint4 *>(
                p.codes + (size_t)n * (p.K / 2) + (size_t)ks * 32);
            rs.c0 = __ldg(src);
            rs.c1 = __ldg(src + 1);
            if constexpr (PERK) {
                // the warp's 32 weight rows lie in one 64-block of the original rows: one 128-byte
                // line of scales for the stage, a pair per lane
                const uint32_t *line = reinterpret_cast<const uint32_t *>(
                    p.scales_t + (size_t)((n - lane) >> 6) * p.K + (size_t)ks * BK);
                rs.scale = __uint_as_float(__ldg(line + lane));
            } else {
                const size_t blk = (size_t)n * blocks_per_row + ks;
                rs.scale = (p.absmax ? __ldg(p.absmax + blk) : dq_scale(__ldg(p.scale_codes + blk), sos)) * w_down;
            }
        };
        auto emit = [&](const Pos &pos, const RowStage &rs) -> bool {
            const uint32_t cnt = pos.cnt;
            const uint32_t s = cnt % kAStages, ph = (cnt / kAStages) & 1u;
            const uint32_t dst = lane_base + s * kAStageCols;
            uint32_t lo[16], hi[16];
            if constexpr (PERK) {
                expand_half_per_k(tables, rs.c0, __float_as_uint(rs.scale), 0, lo);
                expand_half_per_k(tables, rs.c1, __float_as_uint(rs.scale), 16, hi);
            } else {
                expand_half(tables, rs.c0, rs.scale, lo);
                expand_half(tables, rs.c1, rs.scale, hi);
            }
            if (!ptx::mbar_wait_suspended(bar(kBarAEmpty + s), ph ^ 1u)) return false;
            ptx::tc_fence_after();
            tmem_st32(dst, lo, hi);
            ptx::tmem_wait_st();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kBarAFull + s));
            return true;
        };

        // software pipeline over this group's stages (group, group + 4, group + 8, ...): the
        // loads of a stage are in flight while the stages before it are expanded
        constexpr int kDepth = 2;
        Pos pe{group, 0, 0, 0, 0};
        if (wl.n_seg == 0) pe.cnt = total;
        else {
            enter(pe, group);
            settle(pe);
        }
        Pos pf = pe;
        RowStage rs[kDepth];
        #pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            fetch(pf, rs[d]);
            advance(pf);
        }
        while (pe.cnt < total && ok) {
            #pragma unroll
            for (int d = 0; d < kDepth; ++d) {
                if (ok && pe.cnt < total) {
                    ok = emit(pe, rs[d]);
                    advance(pe);
                    fetch(pf, rs[d]);
                    advance(pf);
                }
            }
        }
        if (!ok && lane == 0) NF4_REPORT_FAILURE(g_prefill_error, g_prefill_error_host, 4);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- pre-pass: f16 activations, row scales and the LoRA intermediate ---------------------
// One CTA per 16 rows of x, sixteen warps splitting K.  x is read once:
//   1. xh[m][k] = f16(x[m][k]) is written at once (exact inside f16's range) while the row
//      maxima are collected; row_scale[m] = 1, or the power of two that brings a row whose
//      largest magnitude exceeds 32768 or lies below 2^-8 to [16384, 32768), in which case that
//      row is converted again as f16(x / row_scale) at the end (rare).
//   2. with an adapter: T = lora_scale * (x A^T) / row_scale, written as bf16 hi / lo halves:
//      T[m][c] for c < 64*chunks holds bf16(T), T[m][64*chunks + c] holds bf16(T - bf16(T));
//      columns beyond the rank are zero.  The same registers of x feed warp MMAs against A.
// k is walked in 32-wide pieces; inside a piece thread t owns k = 8t .. 8t+7 so that both
// operands are read with 16-byte loads (a consistent permutation of k on A and B).  The loads
// of the next piece are in flight while a piece is multiplied.
constexpr int kTThreads = 512;
constexpr int kTWarps = kTThreads / 32;
constexpr int kTPartStride = 72;  // floats per row of a warp's partial sums (64 + padding against bank conflicts)
constexpr int kTPartBytes = kTWarps * 16 * kTPartStride * 4;

struct PrepassPiece {
    uint4 xa, xb;   // rows g and g + 8 of the slab
    uint4 bv[8];    // rows 8u + g of this 64-rank chunk of A
};

// Running maxima of |bf16|, a pair at a time; a NaN leaves the maximum as it is (max.bf16x2
// returns the other operand).
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t w, uint32_t mx) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(w & 0x7fff7fffu), "r"(mx));
    return d;
}
// The larger half of such a pair as an f32 pattern; 0 if only NaNs were seen.
__device__ __forceinline__ uint32_t bf16x2_larger_bits(uint32_t mx) {
    const uint32_t lo = mx << 16, hi = mx & 0xffff0000u;
    const uint32_t a = lo <= 0x7f800000u ? lo : 0u, b = hi <= 0x7f800000u ? hi : 0u;
    return max(a, b);
}

__device__ __forceinline__ uint4 bf16x8_to_f16x8(const uint4 &v, float is) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
    #pragma unroll
    for (int q = 0; q < 4; ++q) {
        const __half2 h = __floats2half2_rn(__uint_as_float(w[q] << 16) * is,
                                            __uint_as_float(w[q] & 0xffff0000u) * is);
        o[q] = *reinterpret_cast<const uint32_t *>(&h);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// MODE 1 (XH_READY): the activations arrive as the f16 copy itself (made, with the row scales, by
// x_f32_to_f16_row) and the adapter factor as f16: only T is computed, with f16 MMAs.
// MODE 2 (T_ONLY): the product alone, t32[m][j] = sum_k x[m][k] a[j][k] in f32, for callers outside
// the GEMM (the adapter's gradients): no copy of x, no scales.
template <int MODE>
__global__ void __launch_bounds__(kTThreads)
prefill_prepass_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a,
                       uint32_t M, uint32_t K, uint32_t rank, uint32_t chunks, float scale,
                       __half *__restrict__ xh, float *__restrict__ row_scale,
                       __nv_bfloat16 *__restrict__ t_out, const float *__restrict__ absmax,
                       const uint8_t *__restrict__ scale_codes, const float *__restrict__ scale_of_scales,
                       uint32_t *__restrict__ sk_flags, uint32_t n_flags, float *__restrict__ t32) {
    constexpr bool XH_READY = MODE == 1, T_ONLY = MODE == 2;
    // the warps' partial sums of T: [warp][16 rows][64 ranks, padded to 72], summed in warp order
    extern __shared__ __align__(16) float part[];
    __shared__ uint32_t row_max_bits[16];
    __shared__ float inv_scale[16];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t m0 = blockIdx.x * 16;
    const uint32_t rows = min(16u, M - m0);
    ptx::pdl_launch_dependents();  // the GEMM may set itself up and start on the weights
    // the GEMM's CTAs raise these once this kernel has completed (their readers and writers wait for that)
    if (blockIdx.x == 0)
        for (uint32_t i = threadIdx.x; i < n_flags; i += kTThreads) sk_flags[i] = 0;
    const int w_exp = T_ONLY ? 0 : weight_exponent(absmax, scale_codes, scale_of_scales);
    const float w_up = ldexpf(1.0f, w_exp), w_down = ldexpf(1.0f, -w_exp);
    const bool row_a = g < rows, row_b = g + 8 < rows;
    const uint32_t pieces = (K + 31) / 32, n_it = (pieces + kTWarps - 1) / kTWarps;
    const size_t off_a = (size_t)(m0 + g) * K, off_b = (size_t)(m0 + g + 8) * K;

    if (threadIdx.x < 16) row_max_bits[threadIdx.x] = 0;
    __syncthreads();
    uint32_t mx_a = 0, mx_b = 0;

    const uint32_t passes = chunks ? chunks : 1u;
    for (uint32_t chunk = 0; chunk < passes; ++chunk) {
        float acc[8][4];
        #pragma unroll
        for (int u = 0; u < 8; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;

        // piece `it` of this warp starts at k = (warp + 16 it) * 32; this thread's 8 values at + 8t
        auto k_of = [&](uint32_t it) { return (warp + kTWarps * it) * 32 + 8 * t; };
        auto load = [&](PrepassPiece &pc, uint32_t it) {
            const uint32_t k = k_of(it);
            const bool in = it < n_it && k + 8 <= K && (!XH_READY || rank != 0);
            pc.xa = pc.xb = make_uint4(0, 0, 0, 0);
            if (in && row_a) pc.xa = __ldg(reinterpret_cast<const uint4 *>(x + off_a + k));
            if (in && row_b) pc.xb = __ldg(reinterpret_cast<const uint4 *>(x + off_b + k));
            #pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t j = chunk * 64 + 8 * u + g;
                pc.bv[u] = make_uint4(0, 0, 0, 0);
                if (in && j < rank) pc.bv[u] = __ldg(reinterpret_cast<const uint4 *>(a + (size_t)j * K + k));
            }
        };
        auto process = [&](const PrepassPiece &pc, uint32_t it) {
            const uint32_t k = k_of(it);
            if (MODE == 0 && chunk == 0 && it < n_it && k + 8 <= K) {
                if (row_a) {
                    mx_a = bf16x2_absmax(pc.xa.x, bf16x2_absmax(pc.xa.y, mx_a));
                    mx_a = bf16x2_absmax(pc.xa.z, bf16x2_absmax(pc.xa.w, mx_a));
                    *reinterpret_cast<uint4 *>(xh + off_a + k) = bf16x8_to_f16x8(pc.xa, 1.0f);
                }
                if (row_b) {
                    mx_b = bf16x2_absmax(pc.xb.x, bf16x2_absmax(pc.xb.y, mx_b));
                    mx_b = bf16x2_absmax(pc.xb.z, bf16x2_absmax(pc.xb.w, mx_b));
                    *reinterpret_cast<uint4 *>(xh + off_b + k) = bf16x8_to_f16x8(pc.xb, 1.0f);
                }
            }
            if (rank) {
                #pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (XH_READY) {
                        ptx::mma_16816_f16(acc[u], pc.xa.x, pc.xb.x, pc.xa.y, pc.xb.y, pc.bv[u].x, pc.bv[u].y);
                        ptx::mma_16816_f16(acc[u], pc.xa.z, pc.xb.z, pc.xa.w, pc.xb.w, pc.bv[u].z, pc.bv[u].w);
                    } else {
                        ptx::mma_16816_bf16(acc[u], pc.xa.x, pc.xb.x, pc.xa.y, pc.xb.y, pc.bv[u].x, pc.bv[u].y);
                        ptx::mma_16816_bf16(acc[u], pc.xa.z, pc.xb.z, pc.xa.w, pc.xb.w, pc.bv[u].z, pc.bv[u].w);
                    }
                }
            }
        };
        PrepassPiece p0, p1;
        load(p0, 0);
        for (uint32_t it = 0; it < n_it; it += 2) {
            load(p1, it + 1);
            process(p0, it);
            load(p0, it + 2);
            process(p1, it + 1);
        }

        if (MODE == 0 && chunk == 0) {
            atomicMax(&row_max_bits[g], bf16x2_larger_bits(mx_a));
            atomicMax(&row_max_bits[g + 8], bf16x2_larger_bits(mx_b));
        }
        if (rank) {
            #pragma unroll
            for (int u = 0; u < 8; ++u) {
                float *mine = part + warp * (16 * kTPartStride);
                *reinterpret_cast<float2 *>(mine + g * kTPartStride + 8 * u + 2 * t) = make_float2(acc[u][0], acc[u][1]);
                *reinterpret_cast<float2 *>(mine + (g + 8) * kTPartStride + 8 * u + 2 * t) =
                    make_float2(acc[u][2], acc[u][3]);
            }
        }
        __syncthreads();
        if (MODE != 0 && chunk == 0) {
            if (threadIdx.x < 16) inv_scale[threadIdx.x] = 1.0f;  // the rows arrive scaled, or stay as they are
            __syncthreads();
        }
        if (MODE == 0 && chunk == 0) {
            if (threadIdx.x < 16) {
                const float mx = __uint_as_float(row_max_bits[threadIdx.x]);
                float sc = 1.0f;
                if ((mx > 32768.0f || (mx < 0.00390625f && mx >= 1.1754944e-38f)) && mx < __int_as_float(0x7f800000)) {
                    int e;
                    frexpf(mx, &e);             // mx = f * 2^e with f in [0.5, 1)
                    sc = ldexpf(1.0f, e - 15 < -100 ? -100 : e - 15);  // mx / sc lands in [16384, 32768)
                }
                inv_scale[threadIdx.x] = 1.0f / sc;  // exact: sc is a power of two
                if (threadIdx.x < rows) row_scale[m0 + threadIdx.x] = sc * w_up;  // both factors of the outputs
            }
            __syncthreads();
            // rows beyond f16's range: convert again, scaled
            for (uint32_t r = 0; r < rows; ++r) {
                const float is = inv_scale[r];
                if (is == 1.0f) continue;
                for (uint32_t c = threadIdx.x; c < K / 8; c += kTThreads) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * K) + c);
                    reinterpret_cast<uint4 *>(xh + (size_t)(m0 + r) * K)[c] = bf16x8_to_f16x8(v, is);
                }
            }
        }
        if (rank) {
            const uint32_t ld_t = 2 * 64 * chunks;
            for (uint32_t i = threadIdx.x; i < 16 * 64; i += kTThreads) {
                const uint32_t r = i >> 6, c = i & 63u;
                if (m0 + r < M) {
                    float sum = 0.0f;
                    #pragma unroll
                    for (int w = 0; w < kTWarps; ++w) sum += part[w * (16 * kTPartStride) + r * kTPartStride + c];
                    if (T_ONLY) {
                        if (chunk * 64 + c < rank) t32[(size_t)(m0 + r) * rank + chunk * 64 + c] = sum;
                        continue;
                    }
                    const float v = sum * scale * inv_scale[r] * w_down;
                    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
                    const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
                    t_out[(size_t)(m0 + r) * ld_t + chunk * 64 + c] = hi;
                    t_out[(size_t)(m0 + r) * ld_t + 64 * chunks + chunk * 64 + c] = lo;
                }
            }
        }
        __syncthreads();
    }
}

// ---- weights in the other orientation: repacking before the GEMM ---------------------------
// W [d_in][d_out] with the 64-blocks along d_out (the reference's Burn layout) is brought into the
// form the GEMM's dequantisers read: codes_t[n][k / 2] (the same nibbles, transposed, so exact) and
// scales_t[n / 64][k] (f16 of scale / 2^e, the rounding the GEMM applies to a scale anyway).

struct RepackParams {
    const uint8_t *codes;
    const float *absmax;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const void *a, *b;          // adapter factors A [K][r], B [r][N], or null
    uint8_t *codes_t;
    __half *scales_t;
    uint16_t *a_t;
    __nv_bfloat16 *b_t;
    uint32_t K, N, r;
    int32_t factors_out_in;     // the factors come as A [r][K], B [N][r] (else A [K][r], B [r][N])
    uint32_t code_cols, code_rows, code_blocks;   // CTAs of the nibbles: columns of 128 n x groups of kRepackTiles k-tiles
    uint32_t scale_cols, scale_blocks;            // CTAs of the scales: 32 x 32 tiles
    uint32_t adapter_blocks;
    const float *x32;           // f32 activations [x_rows][K] to convert, or null
    __half *xh;
    float *row_scale;
    uint32_t x_rows;
};
constexpr uint32_t kRepackTiles = 4;  // 64-row tiles of nibbles one CTA walks, the next one's loads in flight

// Nibbles: 64 rows (k) x 128 columns (n) per tile through shared memory; a thread turns 16 rows of
// one byte column (two n) into the 8 bytes each of those two weight rows gets.
__device__ __forceinline__ void repack_codes_block(const RepackParams &p, uint32_t block, uint8_t (*tile)[64][80]) {
    const uint32_t n0 = (block % p.code_cols) * 128, kt0 = (block / p.code_cols) * kRepackTiles, t = threadIdx.x;
    const uint32_t k_tiles = p.K / 64;
    const uint32_t n_it = min(kRepackTiles, k_tiles - kt0);
    const uint32_t r = t >> 2, seg = t & 3u;  // loads: 16 bytes = 32 columns of row r per thread
    const bool in = n0 + seg * 32 < p.N;
    auto load = [&](uint32_t it) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (in)
            v = __ldg(reinterpret_cast<const uint4 *>(p.codes + (size_t)((kt0 + it) * 64 + r) * (p.N / 2) + n0 / 2 +
                                                      seg * 16));
        return v;
    };
    const uint32_t bc = t & 63u, kq = t >> 6;  // byte column and quarter of the rows
    uint4 v = load(0);
    for (uint32_t it = 0; it < n_it; ++it) {
        uint8_t(*cur)[80] = tile[it & 1u];
        *reinterpret_cast<uint4 *>(&cur[r][seg * 16]) = v;
        __syncthreads();
        if (it + 1 < n_it) v = load(it + 1);
        if (n0 + 2 * bc < p.N) {
            uint32_t e0 = 0, e1 = 0, o0 = 0, o1 = 0;  // even column: k 0..7, 8..15 of the quarter; odd column
            #pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t b0 = cur[kq * 16 + j][bc], b1 = cur[kq * 16 + 8 + j][bc];
                e0 |= (b0 & 15u) << (4 * j);
                o0 |= (b0 >> 4) << (4 * j);
                e1 |= (b1 & 15u) << (4 * j);
                o1 |= (b1 >> 4) << (4 * j);
            }
            const size_t at = (size_t)(n0 + 2 * bc) * (p.K / 2) + ((kt0 + it) * 64 + kq * 16) / 2;
            *reinterpret_cast<uint2 *>(p.codes_t + at) = make_uint2(e0, e1);
            *reinterpret_cast<uint2 *>(p.codes_t + at + p.K / 2) = make_uint2(o0, o1);
        }
    }
}

// scales_t[b][k] = f16(scale(k, b) / 2^e), scale(k, b) the scale of block k * (N / 64) + b.
__device__ __forceinline__ void repack_scales_block(const RepackParams &p, uint32_t block, float (*tile)[33]) {
    const uint32_t blocks_per_row = p.N / 64;
    const int w_exp = weight_exponent(p.absmax, p.scale_codes, p.scale_of_scales);
    const float w_down = ldexpf(1.0f, -w_exp);
    const float sos = p.scale_codes ? __ldg(p.scale_of_scales) : 0.0f;
    const uint32_t b0 = (block % p.scale_cols) * 32, k0 = (block / p.scale_cols) * 32;
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
    for (uint32_t r = ty; r < 32; r += 8) {
        const uint32_t k = k0 + r, b = b0 + tx;
        float v = 0.0f;
        if (k < p.K && b < blocks_per_row) {
            const size_t blk = (size_t)k * blocks_per_row + b;
            v = (p.absmax ? __ldg(p.absmax + blk) : dq_scale(__ldg(p.scale_codes + blk), sos)) * w_down;
        }
        tile[r][tx] = v;
    }
    __syncthreads();
    for (uint32_t r = ty; r < 32; r += 8) {
        const uint32_t b = b0 + r, k = k0 + tx;
        if (k < p.K && b < blocks_per_row) p.scales_t[(size_t)b * p.K + k] = __float2half_rn(tile[tx][r]);
    }
}

// The adapter factors in the orientation and types the pre-pass and the GEMM read them in.
// From A [d_in][r], B [r][d_out] of type T:
//   bf16: a_t[j][k] = A[k][j], b_t[n][j] = B[j][n] (rank_out = r): exact.
//   f32:  a_t[j][k] = a_t[r + j][k] = f16(A[k][j]); b_t[n][j] = bf16(B[j][n]), b_t[n][r + j] = the
//         bf16 of what that rounding left: as an adapter of rank 2 r whose intermediate holds every
//         column twice, B enters the product with sixteen bits of mantissa.
template <class T>
__device__ __forceinline__ void repack_adapter_block(const RepackParams &p, uint32_t block) {
    constexpr bool kF32 = sizeof(T) == 4;
    const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
    const uint32_t r = p.r, rank_out = kF32 ? 2 * r : r;
    const uint64_t i = (uint64_t)block * blockDim.x + threadIdx.x;
    const uint64_t na = (uint64_t)r * p.K, nb = (uint64_t)p.N * r;
    if (i < na) {
        const uint32_t j = (uint32_t)(i / p.K), k = (uint32_t)(i % p.K);
        const size_t at = p.factors_out_in ? (size_t)j * p.K + k : (size_t)k * r + j;
        if constexpr (kF32) {
            const __half h = __float2half_rn(a[at]);
            p.a_t[i] = __half_as_ushort(h);
            p.a_t[na + i] = __half_as_ushort(h);
        } else {
            p.a_t[i] = reinterpret_cast<const uint16_t *>(a)[at];
        }
    } else if (i < na + nb) {
        const uint64_t e = i - na;
        const uint32_t n = (uint32_t)(e / r), j = (uint32_t)(e % r);
        const size_t at = p.factors_out_in ? (size_t)n * r + j : (size_t)j * p.N + n;
        if constexpr (kF32) {
            const float v = b[at];
            const __nv_bfloat16 hi = __float2bfloat16_rn(v);
            p.b_t[(size_t)n * rank_out + j] = hi;
            p.b_t[(size_t)n * rank_out + r + j] = __float2bfloat16_rn(v - __bfloat162float(hi));
        } else {
            p.b_t[(size_t)n * rank_out + j] = b[at];
        }
    }
}

// f32 activations: xh[m][k] = f16(x[m][k] / sc), sc the power of two that brings the row's largest
// finite magnitude into [16384, 32768) (any row, so small activations keep their bits too);
// row_scale[m] = sc * 2^e with e the weight's exponent.  One CTA of 256 threads per row.
__device__ __forceinline__ void x_f32_to_f16_row(const float *__restrict__ x, uint32_t m, uint32_t K,
                                                 __half *__restrict__ xh, float *__restrict__ row_scale,
                                                 const float *__restrict__ absmax,
                                                 const uint8_t *__restrict__ scale_codes,
                                                 const float *__restrict__ scale_of_scales, uint32_t *mx_bits) {
    const float4 *row = reinterpret_cast<const float4 *>(x + (size_t)m * K);
    if (threadIdx.x == 0) *mx_bits = 0;
    __syncthreads();
    uint32_t mx = 0;
    for (uint32_t c = threadIdx.x; c < K / 4; c += 256) {
        const float4 v = __ldg(row + c);
        const uint32_t b[4] = {__float_as_uint(v.x) & 0x7fffffffu, __float_as_uint(v.y) & 0x7fffffffu,
                               __float_as_uint(v.z) & 0x7fffffffu, __float_as_uint(v.w) & 0x7fffffffu};
        #pragma unroll
        for (int q = 0; q < 4; ++q)
            if (b[q] < 0x7f800000u) mx = max(mx, b[q]);
    }
    #pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    if ((threadIdx.x & 31u) == 0) atomicMax(mx_bits, mx);
    __syncthreads();
    const float largest = __uint_as_float(*mx_bits);
    float sc = 1.0f;
    if (largest >= 1.1754944e-38f) {  // a normal number
        int e;
        frexpf(largest, &e);
        e = e - 15 < -100 ? -100 : e - 15;  // 1 / sc stays finite
        sc = ldexpf(1.0f, e);
    }
    const float is = 1.0f / sc;
    if (threadIdx.x == 0)
        row_scale[m] = sc * ldexpf(1.0f, weight_exponent(absmax, scale_codes, scale_of_scales));
    uint2 *out = reinterpret_cast<uint2 *>(xh + (size_t)m * K);
    for (uint32_t c = threadIdx.x; c < K / 4; c += 256) {
        const float4 v = __ldg(row + c);
        const __half2 lo = __floats2half2_rn(v.x * is, v.y * is), hi = __floats2half2_rn(v.z * is, v.w * is);
        out[c] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
}

// One launch for everything in front of the pre-pass: the first code_blocks CTAs take the nibbles,
// the next scale_blocks the scales, the next adapter_blocks the adapter, the last x_rows one row of
// f32 activations each.
template <class T>
__global__ void __launch_bounds__(256) repack_kernel(const RepackParams p) {
    __shared__ __align__(16) uint8_t smem[2 * 64 * 80];
    uint32_t b = blockIdx.x;
    if (b < p.code_blocks) return repack_codes_block(p, b, reinterpret_cast<uint8_t(*)[64][80]>(smem));
    b -= p.code_blocks;
    if (b < p.scale_blocks) return repack_scales_block(p, b, reinterpret_cast<float(*)[33]>(smem));
    b -= p.scale_blocks;
    if (b < p.adapter_blocks) return repack_adapter_block<T>(p, b);
    b -= p.adapter_blocks;
    x_f32_to_f16_row(p.x32, b, p.K, p.xh, p.row_scale, p.absmax, p.scale_codes, p.scale_of_scales,
                     reinterpret_cast<uint32_t *>(smem));
}

// ---- host side -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D row-major tensor [rows][cols] with row pitch `pitch_bytes`; box = [box_rows][box_cols].
int32_t make_map(CUtensorMap *map, CUtensorMapDataType dt, uint32_t elem_bytes, const void *base,
                 uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows,
                 uint32_t box_cols, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(NF4_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NF4_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return NF4_OK;
}

uint32_t lora_chunks_of(uint32_t rank) { return (rank + 63) / 64; }

}  // namespace

bool prefill_supported(const nf4_linear_args &a) {
    if (a.layout != NF4_LAYOUT_OUT_IN) return false;
    if (a.io_dtype != NF4_DTYPE_BF16 && a.io_dtype != NF4_DTYPE_F32) return false;
    const bool f32 = a.io_dtype == NF4_DTYPE_F32;
    if (a.rows <= 16) return false;  // the decode kernel's territory
    if (a.d_in % 64 != 0 || a.d_in >= (1ull << 31) || a.d_out >= (1ull << 31) || a.rows >= (1ull << 31))
        return false;
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;
    const uint64_t ybytes = (a.y_f32 || f32) ? 4 : 2;
    if ((ldy * ybytes) % 16 != 0 || !aligned16(a.y) || !aligned16(a.x) || !aligned16(a.packed))
        return false;
    if (a.lora_a && f32) {
        // f32 factors are converted into the workspace and enter as an adapter of twice the rank
        if (2 * a.lora_rank > 256 || (2 * a.lora_rank) % 8 != 0) return false;
    } else if (a.lora_a) {
        // LoRA B is read by TMA: rows (rank * 2 bytes) must be a multiple of 16 bytes
        if (a.lora_rank > 256 || a.lora_rank % 8 != 0 || !aligned16(a.lora_b)) return false;
        if (a.d_in % 8 != 0 || !aligned16(a.lora_a)) return false;
    }
    return true;
}

namespace {
// How the tiles are shared out: `grid` CTAs; the first `sk_tiles` tiles are divided by k-stages
// (every CTA the same number of stages, a tile possibly split between neighbours), the other
// grid * dp_rounds tiles go out whole.  With a tile count that is a multiple of the grid nothing
// is split.  Otherwise the last round of whole tiles would leave most CTAs idle (896 tiles on 148
// CTAs: seven rounds for 6.05 rounds of work), so the last full round and the remainder are
// divided by stages instead.  Fewer tiles than SMs: divided as long as a CTA keeps 24 stages.
struct Sharing {
    uint32_t grid, sk_tiles, dp_rounds;
};
Sharing share_tiles(uint64_t rows, uint64_t d_in, uint64_t d_out) {
    const uint64_t tiles = ((rows + BN - 1) / BN) * ((d_out + BM - 1) / BM), ks = d_in / BK;
    Sharing sh;
    uint64_t grid = kNumSMs;
    if (tiles < grid) {
        const uint64_t by_stages = tiles * ks / 24;
        grid = by_stages < grid ? by_stages : grid;
        if (grid < tiles) grid = tiles;
    }
    sh.grid = (uint32_t)grid;
    if (tiles % grid == 0) {
        sh.sk_tiles = 0;
        sh.dp_rounds = (uint32_t)(tiles / grid);
    } else {
        sh.dp_rounds = tiles / grid >= 1 ? (uint32_t)(tiles / grid - 1) : 0u;
        sh.sk_tiles = (uint32_t)(tiles - (uint64_t)sh.dp_rounds * grid);
    }
    return sh;
}

struct WorkspaceLayout {
    uint64_t off_xh, off_scale, off_t, off_flags, off_partial, bytes;
    uint64_t off_a_t, off_b_t;             // the adapter factors as the GEMM reads them (f32 factors, other orientation)
    uint64_t off_codes_t, off_scales_t;    // the repacked weight (other orientation)
};
enum Extra { kPlain = 0, kFactors = 1, kFactorsAndWeight = 2 };
// f16 copy of x | row scales | T (bf16 hi/lo) | flags and partial sums of the split tiles; d_in is
// bounded so that rows * d_in * 2 fits
WorkspaceLayout workspace_layout(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank,
                                 Extra extra = kPlain) {
    auto up = [](uint64_t v) { return (v + 255) / 256 * 256; };
    WorkspaceLayout w;
    w.off_xh = 0;
    w.off_scale = up(rows * d_in * 2);
    w.off_t = w.off_scale + up(rows * 4);
    w.off_flags = w.off_t + up(rows * 2ull * 64 * lora_chunks_of(lora_rank) * 2);
    const Sharing sh = share_tiles(rows, d_in, d_out);
    w.off_partial = w.off_flags + up((uint64_t)sh.grid * 4);
    w.bytes = w.off_partial + (sh.sk_tiles ? (uint64_t)sh.grid * BM * BN * 4 : 0);
    w.off_codes_t = w.off_scales_t = w.off_a_t = w.off_b_t = 0;
    if (extra >= kFactors) {  // `lora_rank` is the rank the GEMM sees (twice the adapter's for f32 factors)
        w.off_a_t = up(w.bytes);
        w.off_b_t = w.off_a_t + up((uint64_t)lora_rank * d_in * 2);
        w.bytes = w.off_b_t + up(d_out * (uint64_t)lora_rank * 2);
    }
    if (extra >= kFactorsAndWeight) {
        w.off_codes_t = up(w.bytes);
        w.off_scales_t = w.off_codes_t + up(d_in * d_out / 2);
        w.bytes = w.off_scales_t + up((d_out / 64) * d_in * 2);
    }
    return w;
}
}  // namespace

uint64_t prefill_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    if (rows <= 16 || d_in % 64 != 0 || d_in == 0 || d_out == 0) return 0;
    // f32 factors at worst; the other orientation where its shapes allow it
    return workspace_layout(rows, d_in, d_out, 2 * lora_rank, d_out % 64 == 0 ? kFactorsAndWeight : kFactors).bytes;
}

// The reference's orientation (W [d_in][d_out], blocks along d_out) at more than 16 rows: repacked
// into the workspace, then the same GEMM.  Fewer rows stay with the CUDA-core strip kernel, whose
// f32 arithmetic is the reference's own.
bool prefill_in_out_supported(const nf4_linear_args &a) {
    if (a.layout != NF4_LAYOUT_IN_OUT) return false;
    if (a.io_dtype != NF4_DTYPE_BF16 && a.io_dtype != NF4_DTYPE_F32) return false;
    if (a.rows < kInOutMinRows) return false;
    if (a.d_in % 64 != 0 || a.d_out % 64 != 0 || a.d_in >= (1ull << 31) || a.d_out >= (1ull << 31) ||
        a.rows >= (1ull << 31))
        return false;
    const bool f32 = a.io_dtype == NF4_DTYPE_F32;
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;
    const uint64_t ybytes = (a.y_f32 || f32) ? 4 : 2;
    if ((ldy * ybytes) % 16 != 0 || !aligned16(a.y) || !aligned16(a.x) || !aligned16(a.packed)) return false;
    if (a.lora_a) {
        const uint32_t rank = f32 ? 2 * a.lora_rank : a.lora_rank;  // as the GEMM sees it
        if (rank > 256 || rank % 8 != 0) return false;
    }
    return true;
}

int32_t prefill_forward(const nf4_linear_args &a, cudaStream_t stream) {
    const bool repacked = a.layout == NF4_LAYOUT_IN_OUT;
    if (!(repacked ? prefill_in_out_supported(a) : prefill_supported(a)))
        return fail(NF4_ERR_UNSUPPORTED, "prefill_forward: unsupported shape");
    const bool x_f32 = a.io_dtype == NF4_DTYPE_F32;
    const bool y_f32 = a.y_f32 || x_f32;
    const Extra extra = repacked ? kFactorsAndWeight : x_f32 ? kFactors : kPlain;
    PrefillParams p{};
    p.codes = a.packed;
    p.absmax = a.absmax;
    p.scale_codes = a.scale_codes;
    p.scale_of_scales = a.scale_of_scales;
    p.bias = a.bias;
    p.M = (uint32_t)a.rows;
    p.N = (uint32_t)a.d_out;
    p.K = (uint32_t)a.d_in;
    p.rank = a.lora_a ? a.lora_rank : 0;
    if (x_f32) p.rank *= 2;  // see repack_adapter_block
    p.lora_chunks = lora_chunks_of(p.rank);
    p.m_tiles = (p.M + BN - 1) / BN;
    p.n_tiles = (p.N + BM - 1) / BM;
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;

    const WorkspaceLayout wl = workspace_layout(p.M, p.K, p.N, p.rank, extra);
    if (a.workspace_bytes < wl.bytes) return fail(NF4_ERR_INVALID_ARG, "prefill_forward: workspace too small");
    const Sharing sh = share_tiles(p.M, p.K, p.N);
    p.sk_tiles = sh.sk_tiles;
    p.dp_rounds = sh.dp_rounds;
    p.wait_ns = 1000000000u;
    uint8_t *ws = static_cast<uint8_t *>(a.workspace);
    __half *xh = reinterpret_cast<__half *>(ws + wl.off_xh);
    float *row_scale = reinterpret_cast<float *>(ws + wl.off_scale);
    __nv_bfloat16 *t = reinterpret_cast<__nv_bfloat16 *>(ws + wl.off_t);
    p.row_scale = row_scale;
    p.sk_flags = reinterpret_cast<uint32_t *>(ws + wl.off_flags);
    p.partial = reinterpret_cast<float *>(ws + wl.off_partial);
    const void *lora_a = a.lora_a, *lora_b = a.lora_b;
    if (extra != kPlain) {  // the other orientation, f32 tensors, or both: one launch in front of the pre-pass
        RepackParams rp{};
        rp.factors_out_in = !repacked;
        rp.codes = a.packed;
        rp.absmax = a.absmax;
        rp.scale_codes = a.scale_codes;
        rp.scale_of_scales = a.scale_of_scales;
        rp.codes_t = ws + wl.off_codes_t;
        rp.scales_t = reinterpret_cast<__half *>(ws + wl.off_scales_t);
        rp.K = p.K;
        rp.N = p.N;
        rp.code_cols = (p.N + 127) / 128;
        rp.code_rows = (p.K / 64 + kRepackTiles - 1) / kRepackTiles;
        rp.code_blocks = repacked ? rp.code_cols * rp.code_rows : 0;
        rp.scale_cols = (p.N / 64 + 31) / 32;
        rp.scale_blocks = repacked ? rp.scale_cols * ((p.K + 31) / 32) : 0;
        if (p.rank) {
            rp.a = a.lora_a;
            rp.b = a.lora_b;
            rp.r = a.lora_rank;
            rp.a_t = reinterpret_cast<uint16_t *>(ws + wl.off_a_t);
            rp.b_t = reinterpret_cast<__nv_bfloat16 *>(ws + wl.off_b_t);
            rp.adapter_blocks = (uint32_t)(((uint64_t)a.lora_rank * (p.K + p.N) + 255) / 256);
            lora_a = rp.a_t;
            lora_b = rp.b_t;
        }
        if (x_f32) {
            rp.x32 = static_cast<const float *>(a.x);
            rp.xh = xh;
            rp.row_scale = row_scale;
            rp.x_rows = p.M;
        }
        const uint32_t blocks = rp.code_blocks + rp.scale_blocks + rp.adapter_blocks + rp.x_rows;
        if (x_f32) repack_kernel<float><<<blocks, 256, 0, stream>>>(rp);
        else repack_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(rp);
        count_launch();
        if (repacked) {
            p.codes = rp.codes_t;
            p.scales_t = rp.scales_t;
        }
        NF4_CUDA_TRY(cudaGetLastError());
    }
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(prefill_prepass_kernel<1>), kTPartBytes));
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(prefill_prepass_kernel<0>), kTPartBytes));
    if (x_f32) {
        prefill_prepass_kernel<1><<<(p.M + 15) / 16, kTThreads, kTPartBytes, stream>>>(
            reinterpret_cast<const __nv_bfloat16 *>(xh), static_cast<const __nv_bfloat16 *>(lora_a), p.M, p.K, p.rank,
            p.lora_chunks, a.lora_scale, xh, row_scale, t, a.absmax, a.scale_codes, a.scale_of_scales, p.sk_flags,
            sh.grid, nullptr);
    } else {
        prefill_prepass_kernel<0><<<(p.M + 15) / 16, kTThreads, kTPartBytes, stream>>>(
            static_cast<const __nv_bfloat16 *>(a.x), static_cast<const __nv_bfloat16 *>(lora_a), p.M, p.K, p.rank,
            p.lora_chunks, a.lora_scale, xh, row_scale, t, a.absmax, a.scale_codes, a.scale_of_scales, p.sk_flags,
            sh.grid, nullptr);
    }
    count_launch();
    NF4_CUDA_TRY(cudaGetLastError());

    CUtensorMap map_x, map_t, map_b, map_y;
    NF4_TRY(make_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, p.M, p.K, (uint64_t)p.K * 2, BN, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B));
    map_t = map_b = map_x;
    if (p.rank) {
        const uint32_t ld_t = 2 * 64 * p.lora_chunks;
        NF4_TRY(make_map(&map_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, p.M, ld_t, (uint64_t)ld_t * 2, BN,
                         BK, CU_TENSOR_MAP_SWIZZLE_128B));
        // LoRA B [N][rank]: columns beyond the rank and rows beyond N read as zero
        NF4_TRY(make_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lora_b, p.N, p.rank,
                         (uint64_t)p.rank * 2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B));
    }
    if (y_f32)
        NF4_TRY(make_map(&map_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.y, p.M, p.N, ldy * 4, kEpiBytes / (BM * 4), BM,
                         CU_TENSOR_MAP_SWIZZLE_NONE));
    else
        NF4_TRY(make_map(&map_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, p.M, p.N, ldy * 2, kEpiBytes / (BM * 2), BM,
                         CU_TENSOR_MAP_SWIZZLE_NONE));

    const uint32_t grid = sh.grid;
    const size_t smem = 1024 + kXStages * kXTileBytes + kLoraStages * kLoraTileBytes + kEpiBytes +
                        kNumBars * 8 + 16 + BN * 4 + 64;
    auto go = [&](auto kernel) -> int32_t {
        NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), (int)smem));
        return launch_maybe_overlapped(kernel, dim3(grid), dim3(kThreads), smem, stream, true, map_x, map_t, map_b,
                                       map_y, p);
    };
    if (repacked) NF4_TRY(y_f32 ? go(prefill_kernel<true, true>) : go(prefill_kernel<false, true>));
    else NF4_TRY(y_f32 ? go(prefill_kernel<true, false>) : go(prefill_kernel<false, false>));
    count_launch();
    return check_cuda(cudaGetLastError(), "prefill_kernel launch");
}


namespace {
// dst[j][k] = src[k][j] for a bf16 factor [K][r]
__global__ void __launch_bounds__(256)
transpose_factor_kernel(const uint16_t *__restrict__ src, uint16_t *__restrict__ dst, uint64_t K, uint32_t r) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= K * r) return;
    const uint64_t j = i / K, k = i % K;
    dst[i] = src[k * r + j];
}
}  // namespace

// t32[m][j] = sum_k x[m][k] F(k, j) for bf16 x [rows][k] on the warp MMAs of the pre-pass; the factor is
// f [rank][k] (`k_major` false) or f [k][rank], which is transposed into `scratch` (rank * k * 2 bytes)
// first.  Declines shapes its 16-byte loads do not cover.
int32_t adapter_intermediate_bf16(const void *x, const void *f, bool k_major, uint64_t rows, uint64_t k, uint32_t rank,
                                  float *t32, void *scratch, cudaStream_t stream) {
    if (k % 8 != 0 || rows == 0 || rows >= (1ull << 31) || k >= (1ull << 31) || rank == 0 || !aligned16(x) ||
        (k_major ? !scratch || !aligned16(scratch) : !aligned16(f)))
        return NF4_ERR_UNSUPPORTED;
    if (k_major) {
        transpose_factor_kernel<<<(unsigned)((k * rank + 255) / 256), 256, 0, stream>>>(
            static_cast<const uint16_t *>(f), static_cast<uint16_t *>(scratch), k, rank);
        count_launch();
        f = scratch;
    }
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(prefill_prepass_kernel<2>), kTPartBytes));
    prefill_prepass_kernel<2><<<(unsigned)((rows + 15) / 16), kTThreads, kTPartBytes, stream>>>(
        static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(f), (uint32_t)rows, (uint32_t)k, rank,
        lora_chunks_of(rank), 1.0f, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, t32);
    count_launch();
    return check_cuda(cudaGetLastError(), "adapter intermediate launch");
}

int32_t prefill_set_host_flag(int *mapped) {
    return check_cuda(cudaMemcpyToSymbol(g_prefill_error_host, &mapped, sizeof(mapped)), "setting the mapped failure word");
}

// The sharing of the tiles as the kernel will see it, for inspection on the host: the number of
// CTAs and, for CTA `cta`, its segments (tile, first main k-stage, one past the last) in the order
// it works on them.  Returns the number of segments (at most `cap` are written), or -1.
int32_t prefill_share_plan(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t cta, uint32_t *ctas,
                           uint32_t *segments, uint32_t cap) {
    if (rows <= 16 || d_in % BK != 0 || d_in == 0 || d_out == 0) return -1;
    const Sharing sh = share_tiles(rows, d_in, d_out);
    if (ctas) *ctas = sh.grid;
    if (cta >= sh.grid) return -1;
    PrefillParams p{};
    p.sk_tiles = sh.sk_tiles;
    p.dp_rounds = sh.dp_rounds;
    WorkList wl;
    wl.init(p, (uint32_t)(d_in / BK), cta, sh.grid);
    for (uint32_t j = 0; j < wl.n_seg && j < cap; ++j) {
        uint32_t tile, b, e;
        wl.get(j, tile, b, e);
        segments[3 * j] = tile;
        segments[3 * j + 1] = b;
        segments[3 * j + 2] = e;
    }
    return (int32_t)wl.n_seg;
}

int32_t prefill_error_flag_ptr(int **dev_ptr) {
    return check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(dev_ptr), g_prefill_error),
                      "address of the prefill error flag");
}

}  // namespace nf4
