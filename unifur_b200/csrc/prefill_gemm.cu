// Prefill path: y[M, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T) for many rows of x,
// W stored as packed NF4 [N, K] with 64-blocks along K.  A dense contraction: tensor-core
// bound, built on tcgen05.mma with both operands in shared memory and the accumulators in
// tensor memory (TMEM).
//
// Roles inside one persistent CTA (one per SM, 768 threads):
//   warp 0      TMA producer: x tiles [256 rows x 64 k] (f16, 128B-swizzled, K-major) into a
//               3-deep shared-memory ring; after the K loop the same ring carries the LoRA
//               intermediate T (bf16 hi / lo halves) so the adapter is just more k-steps.
//   warp 1      owns TMEM (alloc/dealloc); one of its threads issues the tcgen05.mma of the even
//               k-stages, one thread of warp 7 those of the odd ones.  Issuing a stage's MMAs
//               holds the thread for about as long as they run, and ~400 cycles of waits,
//               fences and commits separate two batches; with two threads the second has done
//               its waiting while the first issues, and only a short hand-over is left.
//   warp 6      idle.
//   warps 2-5   epilogue: TMEM -> registers -> (* row scale, + bias) -> bf16/f32 -> shared ->
//               TMA store.
//   warps 8-23  dequantisers, two groups of 256 threads.  Two threads share one weight row of
//               a stage: each reads 16 packed bytes and the block scale straight from global
//               memory (L2), expands the nibbles with byte-permute lookups held in registers,
//               multiplies by the scale in f16x2 and writes its 32 f16 values into the row's
//               128B-swizzled place in the weight tile in shared memory.  (The expansion is a
//               dependent chain of ~120 instructions per thread: it is the number of warps that
//               hides its latency, so the work is cut fine.)
//
// Tile shapes.  A tile is one 128-row weight half against a 256-row activation tile, with the
// accumulator double-buffered in TMEM so that the epilogue overlaps the next tile; the two
// dequantiser groups take alternate k-stages.  A second shape (two halves per tile, one TMEM
// accumulator and one dequantiser group each, eight MMAs per k-stage reading the activation
// tile twice) is kept behind an environment switch for measurements: it halves the activation
// bytes per flop but is slower, because the k-stage is bound by shared-memory traffic.
//
// The MMA computes D[n, m] = sum_k W[n, k] x[m, k]: weight rows are the MMA's M (TMEM lanes),
// activation rows its N (256 accumulator columns).  Both operands are f16 with f32 accumulation:
// rounding the dequantised weight to bf16 instead would cost ~1.6e-3 relative error, above the
// 1e-3 parity bar, while f16 costs ~3e-4.  The bf16 activations are converted to f16 by a
// pre-pass (exact for every value inside f16's range; a row whose magnitude exceeds 32768 is
// divided by a power of two that the epilogue multiplies back), which also produces the LoRA
// intermediate.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

__device__ int g_prefill_error = 0;  // set when a bounded wait gives up

#ifdef NF4_PREFILL_TIMING
// Optional instrumentation (off in the shipped build): SM-clock timestamps of CTA 0.
__device__ long long g_prefill_ts[128];
#define NF4_PTS(i) do { if (blockIdx.x == 0) g_prefill_ts[(i)] = clock64(); } while (0)
#else
#define NF4_PTS(i) do { } while (0)
#endif

namespace {

constexpr int BM = 128;        // weight rows per tile (MMA M, TMEM lanes)
constexpr int BN = 256;        // activation rows per tile (MMA N, accumulator columns)
constexpr int BK = 64;         // k per stage = one quantization block = one 128B swizzle row
constexpr int kHalves = 2;     // 128-row weight halves per tile on large problems
constexpr int kWStages = 3;    // shared-memory ring of dequantised weight stages (kHalves tiles each)
constexpr int kMaxXStages = 3; // shared-memory ring of activation tiles
constexpr int kAccCols = BN;   // one accumulator; two of them fill the 512 TMEM columns
constexpr int kTmemCols = 512;
constexpr int kXTileBytes = BN * BK * 2;   // 32 KB: activations, written by TMA
constexpr int kWTileBytes = BM * BK * 2;   // 16 KB: dequantised weights, written by the expanders
constexpr int kWStageBytes = kHalves * kWTileBytes;

constexpr int kEpiRows = 32;               // activation rows per epilogue chunk
constexpr int kThreads = 24 * 32;
constexpr int kFirstExpanderWarp = 8;
constexpr int kExpanderWarpsPerGroup = 8;
constexpr uint32_t kSpin = 1u << 22;

// barrier slots
constexpr int kBarXFull = 0, kBarXEmpty = kBarXFull + kMaxXStages, kBarWFull = kBarXEmpty + kMaxXStages,
              kBarWEmpty = kBarWFull + kWStages, kBarAccFull = kBarWEmpty + kWStages,
              kBarAccEmpty = kBarAccFull + 2, kBarIssued = kBarAccEmpty + 2, kNumBars = kBarIssued + 2;

struct PrefillParams {
    const uint8_t *codes;
    const float *absmax;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const float *bias;
    const __nv_bfloat16 *lora_b;  // [N][rank]
    const float *row_scale;       // [M] power-of-two factor each activation row was divided by
    uint32_t M, N, K, rank;
    uint32_t lora_chunks;  // ceil(rank / 64); T is [M][2 * 64 * lora_chunks] (hi halves, then lo)
    uint32_t m_tiles, n_tiles;  // n_tiles counts groups of `halves` * 128 weight rows
    uint32_t halves;            // 2: two 128-row halves per tile; 1: one, accumulator double-buffered
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

// ---- TMEM load (32 lanes x 32-bit, 32 consecutive columns) ------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,"
        "%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
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
#ifdef NF4_PREFILL_FAKE_EXPAND  // measurement aid: what the stage costs without the expansion
    #pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = w[i & 3] ^ s;
    return;
#endif
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

struct RowStage {
    uint4 c;  // this thread's 32 packed codes of one k-stage
    float scale;
};

template <bool YF32>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_t,
               const __grid_constant__ CUtensorMap tmap_y, const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled operand tiles
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kXStages = kMaxXStages;
    uint8_t *x_ring = smem;                                   // kXStages activation tiles
    uint8_t *w_ring = smem + kXStages * kXTileBytes;          // kWStages weight stages
    uint8_t *epi = w_ring + kWStages * kWStageBytes;          // 2 staging buffers
    constexpr int kEpiBufBytes = kEpiRows * BM * (YF32 ? 4 : 2);
    uint64_t *bars = reinterpret_cast<uint64_t *>(epi + 2 * kEpiBufBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t bar0 = ptx::smem_addr(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    const uint32_t k_stages = p.K / BK;
    const uint32_t stages_per_tile = k_stages + 2 * p.lora_chunks;
    const uint32_t total_tiles = p.m_tiles * p.n_tiles;
    const uint32_t my_tiles = blockIdx.x < total_tiles
                                  ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kXStages; ++s) {
            ptx::mbar_init(bar(kBarXFull + s), 1);
            ptx::mbar_init(bar(kBarXEmpty + s), 1);
        }
        for (int s = 0; s < kWStages; ++s) {
            ptx::mbar_init(bar(kBarWFull + s), kExpanderWarpsPerGroup * p.halves);  // the warps writing the stage
            ptx::mbar_init(bar(kBarWEmpty + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(bar(kBarAccFull + b), 1);
            ptx::mbar_init(bar(kBarAccEmpty + b), 4);
            ptx::mbar_init(bar(kBarIssued + b), 1);
        }
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
        ptx::prefetch_tmap(&tmap_x);
        ptx::prefetch_tmap(&tmap_y);
        if (p.lora_chunks) ptx::prefetch_tmap(&tmap_t);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;  // two accumulators: columns [0,256) and [256,512)

    bool ok = true;

    if (warp == 0) {
        // ============================ TMA producer ============================
        if (lane == 0) {
            uint32_t cnt = 0;
            for (uint32_t i = 0; i < my_tiles && ok; ++i) {
                const uint32_t tile = blockIdx.x + i * gridDim.x;
                const uint32_t m0 = (tile % p.m_tiles) * BN;
                for (uint32_t ks = 0; ks < stages_per_tile; ++ks, ++cnt) {
                    const uint32_t s = cnt % kXStages, ph = (cnt / kXStages) & 1u;
                    if (!ptx::mbar_wait_bounded(bar(kBarXEmpty + s), ph ^ 1u, kSpin)) {
                        ok = false;
                        break;
                    }
                    if (cnt >= 20 && cnt < 28) NF4_PTS(cnt - 20);
                    ptx::mbar_arrive_expect_tx(bar(kBarXFull + s), kXTileBytes);
                    const uint32_t dst = ptx::smem_addr(x_ring + s * kXTileBytes);
                    if (ks < k_stages)
                        ptx::tma_load_2d(dst, &tmap_x, (int32_t)(ks * BK), (int32_t)m0,
                                         bar(kBarXFull + s));
                    else
                        ptx::tma_load_2d(dst, &tmap_t, (int32_t)((ks - k_stages) * BK), (int32_t)m0,
                                         bar(kBarXFull + s));
                }
            }
            if (!ok) atomicExch(&g_prefill_error, 1);
        }
    } else if (warp == 1 || warp == 7) {
        // ============================= MMA issuers =============================
        // Thread `me` (0: warp 1, 1: warp 7) issues the stages whose global counter has its
        // parity.  Stage c may only be issued after stage c - 1 has been (hand-over barrier
        // kBarIssued + parity of c - 1), which keeps the MMAs of an accumulator in order.
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            constexpr uint32_t idesc_main = make_idesc(0, 0, BM, BN);  // f16 x f16
            constexpr uint32_t idesc_lora = make_idesc(1, 1, BM, BN);  // bf16 x bf16
            const uint32_t x_addr = ptx::smem_addr(x_ring), w_addr = ptx::smem_addr(w_ring);
            uint32_t cnt = 0;
            for (uint32_t i = 0; i < my_tiles && ok; ++i) {
                // two halves: both accumulators belong to this tile; one half: they alternate
                const uint32_t buf = p.halves == 2 ? 0u : (i & 1u), use = p.halves == 2 ? i : (i >> 1);
                const uint32_t tile = blockIdx.x + i * gridDim.x;
                const uint32_t n0 = (tile / p.m_tiles) * BM * p.halves;
                const uint32_t halves_here = (p.halves == 2 && n0 + BM < p.N) ? 2u : 1u;
                for (uint32_t ks = 0; ks < stages_per_tile; ++ks, ++cnt) {
                    if ((cnt & 1u) != me) continue;
                    const uint32_t sx = cnt % kXStages, phx = (cnt / kXStages) & 1u;
                    const uint32_t sw = cnt % kWStages, phw = (cnt / kWStages) & 1u;
                    if (cnt >= 20 && cnt < 28) NF4_PTS(16 + 4 * (cnt - 20));
                    // the epilogue must have drained this accumulator's previous tile
                    if (ks == 0 &&
                        !ptx::mbar_wait_bounded(bar(kBarAccEmpty + buf), (use & 1u) ^ 1u, kSpin)) {
                        ok = false;
                        break;
                    }
                    if (!ptx::mbar_wait_bounded(bar(kBarXFull + sx), phx, kSpin)) {
                        ok = false;
                        break;
                    }
                    if (cnt >= 20 && cnt < 28) NF4_PTS(17 + 4 * (cnt - 20));
                    if (!ptx::mbar_wait_bounded(bar(kBarWFull + sw), phw, kSpin)) {
                        ok = false;
                        break;
                    }
                    // hand-over: the other thread has issued stage cnt - 1 (its (cnt-1)/2-th)
                    if (cnt > 0 &&
                        !ptx::mbar_wait_bounded(bar(kBarIssued + (me ^ 1u)), ((cnt - 1) >> 1) & 1u, kSpin)) {
                        ok = false;
                        break;
                    }
                    if (cnt >= 20 && cnt < 28) NF4_PTS(18 + 4 * (cnt - 20));
                    ptx::tc_fence_after();
                    const uint64_t bdesc = make_kmajor_sw128_desc(x_addr + sx * kXTileBytes);
                    for (uint32_t h = 0; h < halves_here; ++h) {
                        const uint32_t acc = tmem_base + (p.halves == 2 ? h : buf) * kAccCols;
                        const uint64_t adesc =
                            make_kmajor_sw128_desc(w_addr + sw * kWStageBytes + h * kWTileBytes);
                        if (ks < k_stages) {
                            // +32 bytes of K inside the swizzled row = +2 in the encoded address
                            ptx::mma_ss_f16(acc, adesc, bdesc, idesc_main, ks != 0 ? 1u : 0u);
                            ptx::mma_ss_f16(acc, adesc + 2, bdesc + 2, idesc_main, 1u);
                            ptx::mma_ss_f16(acc, adesc + 4, bdesc + 4, idesc_main, 1u);
                            ptx::mma_ss_f16(acc, adesc + 6, bdesc + 6, idesc_main, 1u);
                        } else {
                            const uint32_t chunk = (ks - k_stages) % p.lora_chunks;
                            const uint32_t left = p.rank - chunk * 64;
                            const uint32_t nk16 = ((left < 64 ? left : 64) + 15) / 16;
                            for (uint32_t j = 0; j < nk16; ++j)
                                ptx::mma_ss_f16(acc, adesc + 2 * j, bdesc + 2 * j, idesc_lora, 1u);
                        }
                    }
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(bar(kBarIssued + me));
                    ptx::tc_commit(bar(kBarXEmpty + sx));
                    ptx::tc_commit(bar(kBarWEmpty + sw));
                    if (ks + 1 == stages_per_tile) ptx::tc_commit(bar(kBarAccFull + buf));
                    if (cnt >= 20 && cnt < 28) NF4_PTS(19 + 4 * (cnt - 20));
                }
            }
            if (!ok) atomicExch(&g_prefill_error, 2);
        }
    } else if (warp < 6) {
        // ============================== epilogue ==============================
        const uint32_t q = warp & 3u;  // TMEM lane quarter this warp may touch
        const uint32_t row_in_tile = q * 32 + lane;
        const uint32_t epi_leader = (warp == 2 && lane == 0);
        for (uint32_t i = 0; i < my_tiles && ok; ++i) {
            const uint32_t tile = blockIdx.x + i * gridDim.x;
            const uint32_t n00 = (tile / p.m_tiles) * BM * p.halves, m0 = (tile % p.m_tiles) * BN;
            const uint32_t buf = p.halves == 2 ? 0u : (i & 1u), use = p.halves == 2 ? i : (i >> 1);
            const uint32_t halves_here = (p.halves == 2 && n00 + BM < p.N) ? 2u : 1u;
            ok = ptx::mbar_wait_bounded(bar(kBarAccFull + buf), use & 1u, kSpin);
            if (!ok) break;
            ptx::tc_fence_after();
            for (uint32_t h = 0; h < halves_here; ++h) {
                const uint32_t n0 = n00 + h * BM;
                const uint32_t n = n0 + row_in_tile;
                const float bias = (p.bias && n < p.N) ? __ldg(p.bias + n) : 0.0f;
                const uint32_t acc = tmem_base + (p.halves == 2 ? h : buf) * kAccCols;
                for (uint32_t c = 0; c < BN / kEpiRows; ++c) {
                    uint8_t *ebuf = epi + (c & 1u) * kEpiBufBytes;
                    // the TMA store that last read this buffer must be done with it
                    if (epi_leader) ptx::tma_store_wait_read<1>();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    uint32_t v[32];
                    tmem_ld32(acc + ((q * 32) << 16) + c * kEpiRows, v);
                    ptx::tmem_wait_ld();
                    if (c == BN / kEpiRows - 1 && h + 1 == halves_here) {
                        // accumulators fully read: hand them back to the MMA warp
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bar(kBarAccEmpty + buf));
                    }
                    // staging layout: [kEpiRows activation rows][BM weight rows]
                    #pragma unroll
                    for (int r = 0; r < 32; ++r) {
                        const uint32_t m = m0 + c * kEpiRows + r;
                        const float rs = m < p.M ? __ldg(p.row_scale + m) : 1.0f;
                        const float f = fmaf(__uint_as_float(v[r]), rs, bias);
                        if (YF32)
                            reinterpret_cast<float *>(ebuf)[r * BM + row_in_tile] = f;
                        else
                            reinterpret_cast<__nv_bfloat16 *>(ebuf)[r * BM + row_in_tile] =
                                __float2bfloat16_rn(f);
                    }
                    ptx::fence_proxy_async();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (epi_leader) {
                        ptx::tma_store_2d(&tmap_y, ptx::smem_addr(ebuf), (int32_t)n0,
                                          (int32_t)(m0 + c * kEpiRows));
                        ptx::tma_store_commit();
                    }
                }
            }
        }
        if (epi_leader) ptx::tma_store_wait<0>();
        if (!ok && lane == 0) atomicExch(&g_prefill_error, 3);
    } else if (warp >= kFirstExpanderWarp) {
        // ============================ dequantisers ============================
        // Two groups of 256 threads: with two halves per tile each group owns a half and takes
        // every stage; with one half they take alternate stages.  Two threads share a weight
        // row: 16 packed bytes + the scale in, 32 f16 values out, written as four 16-byte chunks
        // at the 128B-swizzled positions the MMA's shared-memory descriptor expects.
        const uint32_t group = (warp - kFirstExpanderWarp) / kExpanderWarpsPerGroup;  // 0 or 1
        const uint32_t half = p.halves == 2 ? group : 0u;
        const uint32_t row_in_tile = ((warp - kFirstExpanderWarp) % kExpanderWarpsPerGroup) * 16 + (lane >> 1);
        const uint32_t side = lane & 1u;  // which 32 of the row's 64 weights
        const LevelTables tables = make_level_tables();
        const float sos = p.scale_codes ? __ldg(p.scale_of_scales) : 0.0f;
        const uint32_t blocks_per_row = p.K / 64;
        const uint32_t total = my_tiles * stages_per_tile;
        const uint32_t row_off = (row_in_tile >> 3) * 1024 + (row_in_tile & 7u) * 128;
        const uint32_t swz = row_in_tile & 7u;

        // Stage positions are walked, not divided out: a 64-bit division per stage costs more
        // than the expansion itself.
        struct Pos {
            uint32_t cnt, i, ks, n;  // global stage counter, tile number, stage in tile, weight row
        };
        const uint32_t step = p.halves == 2 ? 1u : 2u;
        auto row_of_tile = [&](uint32_t i) {
            const uint32_t tile = blockIdx.x + i * gridDim.x;
            return (tile / p.m_tiles) * BM * p.halves + half * BM + row_in_tile;
        };
        auto advance = [&](Pos &q) {
            q.cnt += step;
            q.ks += step;
            while (q.ks >= stages_per_tile) {
                q.ks -= stages_per_tile;
                ++q.i;
                q.n = row_of_tile(q.i);
            }
        };
        auto fetch = [&](const Pos &q, RowStage &rs) {
            rs.c = make_uint4(0, 0, 0, 0);
            rs.scale = 0.0f;
            if (q.cnt >= total) return;
            const uint32_t ks = q.ks, n = q.n;
            if (n >= p.N || ks >= k_stages) return;  // adapter stages are read when emitted
#ifdef NF4_PREFILL_FAKE_FETCH  // measurement aid: what the stage costs without the global loads
            rs.c = make_uint4(n, ks, n ^ ks, 7u);
            rs.scale = 1.0f;
            return;
#endif
            rs.c = __ldg(reinterpret_cast<const uint4 *>(
                p.codes + (size_t)n * (p.K / 2) + (size_t)ks * 32 + side * 16));
            const size_t blk = (size_t)n * blocks_per_row + ks;
            rs.scale = p.absmax ? __ldg(p.absmax + blk) : dq_scale(__ldg(p.scale_codes + blk), sos);
        };
        auto emit = [&](const Pos &q, const RowStage &rs) -> bool {
            const uint32_t cnt = q.cnt, ks = q.ks;
            const uint32_t s = cnt % kWStages, ph = (cnt / kWStages) & 1u;
            uint32_t out[16];
            if (ks < k_stages) {
                expand_half(tables, rs.c, rs.scale, out);
            } else {
                // this thread's half of one 64-wide chunk of this row of LoRA B (bf16 pairs),
                // zero beyond the rank
                const uint32_t n = q.n;
                const uint32_t chunk = (ks - k_stages) % p.lora_chunks;
                const uint32_t left = p.rank - chunk * 64;
                const uint16_t *src = reinterpret_cast<const uint16_t *>(p.lora_b) +
                                      (size_t)n * p.rank + chunk * 64;
                #pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const uint32_t col = side * 32 + 2 * e;
                    uint32_t lo = 0, hi = 0;
                    if (n < p.N) {
                        if (col < left) lo = __ldg(src + col);
                        if (col + 1 < left) hi = __ldg(src + col + 1);
                    }
                    out[e] = lo | (hi << 16);
                }
            }
            if ((warp == 8 || warp == 16) && lane == 0 && cnt >= 20 && cnt < 28) NF4_PTS(64 + 4 * (cnt - 20));
            if (!ptx::mbar_wait_bounded(bar(kBarWEmpty + s), ph ^ 1u, kSpin)) return false;
            if ((warp == 8 || warp == 16) && lane == 0 && cnt >= 20 && cnt < 28) NF4_PTS(65 + 4 * (cnt - 20));
            uint8_t *wrow = w_ring + s * kWStageBytes + half * kWTileBytes + row_off;
            #pragma unroll
            for (uint32_t c = 0; c < 4; ++c)
                *reinterpret_cast<uint4 *>(wrow + (((side * 4 + c) ^ swz) << 4)) =
                    make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
            ptx::fence_proxy_async();  // the tensor core reads this tile through the async proxy
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kBarWFull + s));
            if ((warp == 8 || warp == 16) && lane == 0 && cnt >= 20 && cnt < 28) NF4_PTS(66 + 4 * (cnt - 20));
            return true;
        };

        // four-deep software pipeline over this group's stages (the loads of a stage are in
        // flight for three emits): every stage with two halves, stages group, group + 2,
        // group + 4, ... with one
        constexpr int kDepth = 4;
        Pos pe{0, 0, 0, row_of_tile(0)};
        if (p.halves != 2 && group) {  // the second group starts one stage in
            pe.cnt = 1;
            pe.ks = 1;
            while (pe.ks >= stages_per_tile) {
                pe.ks -= stages_per_tile;
                ++pe.i;
                pe.n = row_of_tile(pe.i);
            }
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
#ifdef NF4_PREFILL_TIMING
                    if ((warp == 8 || warp == 16) && lane == 0 && pe.cnt - step >= 20 && pe.cnt - step < 28)
                        NF4_PTS(67 + 4 * (pe.cnt - step - 20));
#endif
                }
            }
        }
        if (!ok && lane == 0) atomicExch(&g_prefill_error, 4);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- pre-pass: f16 activations, row scales and the LoRA intermediate ---------------------
// One CTA per 16 rows of x.
//   1. row_scale[m] = 1, or the power of two that brings a row whose magnitude exceeds 32768
//      back under it; xh[m][k] = f16(x[m][k] / row_scale[m]) (exact inside f16's range).
//   2. with an adapter: T = lora_scale * (x A^T) / row_scale, written as bf16 hi / lo halves:
//      T[m][c] for c < 64*chunks holds bf16(T), T[m][64*chunks + c] holds bf16(T - bf16(T));
//      columns beyond the rank are zero.  Eight warps split K and use warp MMAs.
constexpr int kTThreads = 256;

__global__ void __launch_bounds__(kTThreads)
prefill_prepass_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a,
                       uint32_t M, uint32_t K, uint32_t rank, uint32_t chunks, float scale,
                       __half *__restrict__ xh, float *__restrict__ row_scale,
                       __nv_bfloat16 *__restrict__ t_out) {
    __shared__ float red[16][64 + 1];
    __shared__ uint32_t row_max_bits[16];
    __shared__ float inv_scale[16];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t m0 = blockIdx.x * 16;
    const uint32_t rows = min(16u, M - m0);

    // ---- 1. row maxima -> scales -> f16 copy (K is a multiple of 8, rows are 16-byte aligned)
    if (threadIdx.x < 16) row_max_bits[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t vec_per_row = K / 8;
    for (uint32_t i = threadIdx.x; i < rows * vec_per_row; i += kTThreads) {
        const uint32_t r = i / vec_per_row, c = i % vec_per_row;
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * K) + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t mx = 0;
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            // |bf16| as the top half of an f32 pattern; NaNs are left out of the maximum
            const uint32_t lo = (w[q] << 16) & 0x7fff0000u, hi = w[q] & 0x7fff0000u;
            if (lo <= 0x7f800000u) mx = max(mx, lo);
            if (hi <= 0x7f800000u) mx = max(mx, hi);
        }
        atomicMax(&row_max_bits[r], mx);
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        const float mx = __uint_as_float(row_max_bits[threadIdx.x]);
        float sc = 1.0f;
        if (mx > 32768.0f && mx < __int_as_float(0x7f800000)) {
            int e;
            frexpf(mx, &e);             // mx = f * 2^e with f in [0.5, 1)
            sc = ldexpf(1.0f, e - 15);  // mx / sc lands in [16384, 32768)
        }
        inv_scale[threadIdx.x] = 1.0f / sc;  // exact: sc is a power of two
        if (threadIdx.x < rows) row_scale[m0 + threadIdx.x] = sc;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < rows * vec_per_row; i += kTThreads) {
        const uint32_t r = i / vec_per_row, c = i % vec_per_row;
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * K) + c);
        const float is = inv_scale[r];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __half2 h = __floats2half2_rn(__uint_as_float(w[q] << 16) * is,
                                                __uint_as_float(w[q] & 0xffff0000u) * is);
            o[q] = *reinterpret_cast<const uint32_t *>(&h);
        }
        reinterpret_cast<uint4 *>(xh + (size_t)(m0 + r) * K)[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (rank == 0) return;

    // ---- 2. T = scale * x A^T / row_scale ----
    const uint32_t ld_t = 2 * 64 * chunks;
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        for (uint32_t i = threadIdx.x; i < 16 * 65; i += kTThreads) (&red[0][0])[i] = 0.0f;
        __syncthreads();
        float acc[8][4];
        #pragma unroll
        for (int u = 0; u < 8; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;
        // k is walked in 32-wide pieces; inside a piece thread t owns k = 8t .. 8t+7 so that
        // both operands are read with 16-byte loads (a consistent permutation of k on A and B)
        for (uint32_t k0 = warp * 32; k0 < K; k0 += 8 * 32) {
            uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
            if (k0 + 8 * t + 8 <= K) {
                if (m0 + g < M) xa = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + g) * K + k0 + 8 * t));
                if (m0 + g + 8 < M) xb = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + g + 8) * K + k0 + 8 * t));
            }
            #pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t j = chunk * 64 + 8 * u + g;
                uint4 bv = make_uint4(0, 0, 0, 0);
                if (j < rank && k0 + 8 * t + 8 <= K)
                    bv = __ldg(reinterpret_cast<const uint4 *>(a + (size_t)j * K + k0 + 8 * t));
                ptx::mma_16816_bf16(acc[u], xa.x, xb.x, xa.y, xb.y, bv.x, bv.y);
                ptx::mma_16816_bf16(acc[u], xa.z, xb.z, xa.w, xb.w, bv.z, bv.w);
            }
        }
        #pragma unroll
        for (int u = 0; u < 8; ++u) {
            atomicAdd(&red[g][8 * u + 2 * t], acc[u][0]);
            atomicAdd(&red[g][8 * u + 2 * t + 1], acc[u][1]);
            atomicAdd(&red[g + 8][8 * u + 2 * t], acc[u][2]);
            atomicAdd(&red[g + 8][8 * u + 2 * t + 1], acc[u][3]);
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < 16 * 64; i += kTThreads) {
            const uint32_t r = i >> 6, c = i & 63u;
            if (m0 + r < M) {
                const float v = red[r][c] * scale * inv_scale[r];
                const __nv_bfloat16 hi = __float2bfloat16_rn(v);
                const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
                t_out[(size_t)(m0 + r) * ld_t + chunk * 64 + c] = hi;
                t_out[(size_t)(m0 + r) * ld_t + 64 * chunks + chunk * 64 + c] = lo;
            }
        }
        __syncthreads();
    }
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
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_BF16) return false;
    if (a.rows <= 16) return false;  // the decode kernel's territory
    if (a.d_in % 64 != 0 || a.d_in >= (1ull << 31) || a.d_out >= (1ull << 31) || a.rows >= (1ull << 31))
        return false;
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;
    const uint64_t ybytes = a.y_f32 ? 4 : 2;
    if ((ldy * ybytes) % 16 != 0 || !aligned16(a.y) || !aligned16(a.x) || !aligned16(a.packed))
        return false;
    if (a.lora_a) {
        if (a.lora_rank > 256) return false;
        if (a.d_in % 8 != 0 || !aligned16(a.lora_a)) return false;
    }
    return true;
}

namespace {
struct WorkspaceLayout {
    uint64_t off_xh, off_scale, off_t, bytes;
};
// f16 copy of x | row scales | T (bf16 hi/lo); d_in is bounded so that rows * d_in * 2 fits
WorkspaceLayout workspace_layout(uint64_t rows, uint64_t d_in, uint32_t lora_rank) {
    auto up = [](uint64_t v) { return (v + 255) / 256 * 256; };
    WorkspaceLayout w;
    w.off_xh = 0;
    w.off_scale = up(rows * d_in * 2);
    w.off_t = w.off_scale + up(rows * 4);
    w.bytes = w.off_t + up(rows * 2ull * 64 * lora_chunks_of(lora_rank) * 2);
    return w;
}
}  // namespace

uint64_t prefill_workspace_bytes(uint64_t rows, uint64_t d_in, uint32_t lora_rank) {
    if (rows <= 16 || d_in % 64 != 0) return 0;
    return workspace_layout(rows, d_in, lora_rank).bytes;
}

int32_t prefill_forward(const nf4_linear_args &a, cudaStream_t stream) {
    if (!prefill_supported(a)) return fail(NF4_ERR_UNSUPPORTED, "prefill_forward: unsupported shape");
    PrefillParams p{};
    p.codes = a.packed;
    p.absmax = a.absmax;
    p.scale_codes = a.scale_codes;
    p.scale_of_scales = a.scale_of_scales;
    p.bias = a.bias;
    p.lora_b = static_cast<const __nv_bfloat16 *>(a.lora_b);
    p.M = (uint32_t)a.rows;
    p.N = (uint32_t)a.d_out;
    p.K = (uint32_t)a.d_in;
    p.rank = a.lora_a ? a.lora_rank : 0;
    p.lora_chunks = lora_chunks_of(p.rank);
    p.m_tiles = (p.M + BN - 1) / BN;
    // One 128-row half per tile by default.  Two halves per tile (NF4_PREFILL_HALVES=2) halve the
    // activation bytes per flop, but on B200 the k-stage is bound by shared-memory traffic (MMA
    // operand reads + TMA writes + dequantiser stores), not by the activation stream: measured
    // 547 against 601 TFLOP/s on the 2048 x 14336 x 4096 shape.
    static const int halves_env = [] {
        const char *e = std::getenv("NF4_PREFILL_HALVES");  // measurement knob: 1 or 2
        return e ? std::atoi(e) : 0;
    }();
    p.halves = halves_env == 2 ? 2u : 1u;
    p.n_tiles = (p.N + BM * p.halves - 1) / (BM * p.halves);
    const uint64_t ldy = a.ldy ? a.ldy : a.d_out;

    const WorkspaceLayout wl = workspace_layout(p.M, p.K, p.rank);
    uint8_t *ws = static_cast<uint8_t *>(a.workspace);
    __half *xh = reinterpret_cast<__half *>(ws + wl.off_xh);
    float *row_scale = reinterpret_cast<float *>(ws + wl.off_scale);
    __nv_bfloat16 *t = reinterpret_cast<__nv_bfloat16 *>(ws + wl.off_t);
    p.row_scale = row_scale;
    prefill_prepass_kernel<<<(p.M + 15) / 16, kTThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(a.x), static_cast<const __nv_bfloat16 *>(a.lora_a), p.M, p.K,
        p.rank, p.lora_chunks, a.lora_scale, xh, row_scale, t);
    count_launch();
    NF4_CUDA_TRY(cudaGetLastError());

    CUtensorMap map_x, map_t, map_y;
    NF4_TRY(make_map(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, p.M, p.K, (uint64_t)p.K * 2, BN, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B));
    map_t = map_x;
    if (p.rank) {
        const uint32_t ld_t = 2 * 64 * p.lora_chunks;
        NF4_TRY(make_map(&map_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, p.M, ld_t, (uint64_t)ld_t * 2, BN,
                         BK, CU_TENSOR_MAP_SWIZZLE_128B));
    }
    if (a.y_f32)
        NF4_TRY(make_map(&map_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.y, p.M, p.N, ldy * 4, kEpiRows, BM,
                         CU_TENSOR_MAP_SWIZZLE_NONE));
    else
        NF4_TRY(make_map(&map_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, p.M, p.N, ldy * 2, kEpiRows, BM,
                         CU_TENSOR_MAP_SWIZZLE_NONE));

    const uint32_t total_tiles = p.m_tiles * p.n_tiles;
    const uint32_t grid = total_tiles < (uint32_t)kNumSMs ? total_tiles : (uint32_t)kNumSMs;
    const size_t smem = 1024 + kMaxXStages * kXTileBytes + kWStages * kWStageBytes +
                        2 * kEpiRows * BM * (a.y_f32 ? 4 : 2) +
                        kNumBars * 8 + 64;
    if (a.y_f32) {
        static bool configured = false;
        if (!configured) {
            NF4_CUDA_TRY(cudaFuncSetAttribute(prefill_kernel<true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = true;
        }
        prefill_kernel<true><<<grid, kThreads, smem, stream>>>(map_x, map_t, map_y, p);
    } else {
        static bool configured = false;
        if (!configured) {
            NF4_CUDA_TRY(cudaFuncSetAttribute(prefill_kernel<false>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = true;
        }
        prefill_kernel<false><<<grid, kThreads, smem, stream>>>(map_x, map_t, map_y, p);
    }
    count_launch();
    return check_cuda(cudaGetLastError(), "prefill_kernel launch");
}

#ifdef NF4_PREFILL_TIMING
extern "C" __attribute__((visibility("default"))) int nf4_debug_prefill_timestamps(long long *out128) {
    return (int)cudaMemcpyFromSymbol(out128, g_prefill_ts, sizeof(long long) * 128);
}
#endif

int32_t prefill_error_flag(int *host_value) {
    return check_cuda(cudaMemcpyFromSymbol(host_value, g_prefill_error, sizeof(int)),
                      "read prefill error flag");
}

}  // namespace nf4
