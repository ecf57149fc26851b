// Decode path, tcgen05 version: y[M<=16, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T) with
// W packed NF4 [N, K], 64-blocks along K.  HBM-bound; every byte of W is read once.
//
// Where it is used: shapes the warp-MMA decode kernel does not take (d_in above 4096, e.g. an
// 18944-wide down projection).  Measured on B200, a tcgen05.mma whose A operand sits in TMEM
// costs ~130-150 cycles whatever N is, so one MMA per 2048 weights bounds this kernel near
// 10 us for the 11008 x 4096 layer; the warp-MMA kernel is faster wherever both apply.
//
// Work split.  The weight is cut into units of 128 rows x 128 k (two quantization blocks); the
// units, in row-tile-major order, are dealt out in equal contiguous runs, one run per SM (a run
// is ~37 blocks for the 11008 x 4096 layer, within 3 % of perfectly even).  A run covers parts
// of at most a few row-tiles ("segments"); each segment accumulates in its own 16 TMEM columns.
//
// Data movement.  A producer warp streams tiles of 128 rows x 256 k (128 packed bytes per row,
// 128B-swizzled so that the per-row reads below are bank-conflict free) and the matching block
// scales through a shared-memory ring with tiled TMA loads; x's k-range is converted to f16 once
// per CTA into shared memory in the canonical K-major 128B-swizzled layout the MMA reads.
//
// Math.  Sixteen expander warps: warp w serves TMEM lane quarter w % 4 and, of every 4-block
// tile, block w / 4.  A thread owns one weight row: it reads the row's 32 packed bytes, looks
// byte pairs up in a 256-entry half2 table replicated per lane (no bank conflicts), multiplies
// by the block scale in f16x2 and writes the 64 f16 values into its TMEM lane (tcgen05.st).
// Four threads (one per block of a tile) issue the MMAs: A = weight block from TMEM (128 rows),
// B = x from shared memory (16 columns, rows >= M are zero), D = f32 accumulators in TMEM (two
// per issuer and segment, so consecutive MMAs of an issuer do not chain).
//
// Finish (four warps).  A segment that spans the whole K is finished in place (+bias, +LoRA, convert, store).
// Otherwise its 128 x 16 partial goes to a scratch slot; the last CTA to arrive for a row-tile
// (one counter per row-tile) adds the slots in a fixed order and finishes the tile, so results
// do not depend on timing.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

__device__ int g_decode2_error = 0;  // set when a bounded wait gives up
__device__ int *g_decode2_error_host = nullptr;  // the same, in mapped host memory (set by the host-pointer entry points)


namespace {

constexpr int kRowsPerTile = 128;
// one TMA tile = 4 quantization blocks = 128 bytes per row
constexpr int kCodeStageBytes = kRowsPerTile * 128;
constexpr int kScaleStageBytes = kRowsPerTile * 16;
constexpr int kStageBytes = kCodeStageBytes + kScaleStageBytes;
constexpr int kMaxCodeStages = 6;
constexpr int kASlots = 8;                  // TMEM ring of dequantised blocks (32 columns each)
constexpr int kMaxSegments = 2;             // row-tiles one run may touch
constexpr int kAccCols = 16;                // one accumulator: 128 rows x 16 activation rows
constexpr int kAccPerSeg = 8;               // independent accumulators a segment's MMAs rotate over
constexpr int kTmemCols = 512;
constexpr int kExpanderWarps = 16;
constexpr int kIssuerWarps = 4;             // one MMA-issuing thread per expander group
constexpr int kWarpTma = kExpanderWarps;
constexpr int kWarpIssuer0 = kExpanderWarps + 1;
constexpr int kWarpFinish0 = kWarpIssuer0 + kIssuerWarps;   // 21: warps 21..24 = lane quarters 1,2,3,0
constexpr int kThreads = (kWarpFinish0 + 4) * 32;
constexpr int kLutBytes = 256 * 32 * 4;
constexpr int kXBlockBytes = 16 * 128;      // 16 rows x 64 f16
constexpr int kMaxXBlocks = 56;
constexpr int kMaxRank = 64;
constexpr int kSmemLimit = 227 * 1024;

struct Decode2Params {
    const __nv_bfloat16 *x;
    const float *bias;
    const float *t;  // [M][rank] f32 = x A^T, or null
    const __nv_bfloat16 *lora_b;
    void *y;
    float *partials;   // [(grid + row_tiles)][16][128] f32
    int *counters;     // [row_tiles], zero at launch
    const float *scale_of_scales;
    uint64_t ldy;
    uint32_t y_f32;
    uint32_t M, K, N, rank;
    float lora_scale;
    uint32_t kb;          // K / 64
    uint32_t units_per_tile;  // ceil(kb / 2)
    uint32_t total_units;
    uint32_t row_tiles;
    uint32_t code_stages;
    uint32_t x_blocks;    // blocks of x kept in shared memory
    uint32_t off_x, off_ring;  // offsets inside dynamic shared memory
};

struct Segment {
    uint32_t rt, kb0, kb1;  // row tile, block range [kb0, kb1)
};

__device__ __forceinline__ uint32_t run_start(uint32_t c, uint32_t units, uint32_t grid) {
    return (uint32_t)(((uint64_t)c * units) / grid);
}

// CTA whose run holds unit u (runs start at floor(c * units / grid)).
__device__ __forceinline__ uint32_t cta_of_unit(uint32_t u, uint32_t units, uint32_t grid) {
    uint32_t c = (uint32_t)(((uint64_t)u * grid) / units);
    while (c + 1 < grid && run_start(c + 1, units, grid) <= u) ++c;
    while (c > 0 && run_start(c, units, grid) > u) --c;
    return c;
}

// Segment `i` of the run [u0, u1): returns false when the run has fewer segments.
__device__ __forceinline__ bool segment_of(const Decode2Params &p, uint32_t u0, uint32_t u1,
                                           uint32_t i, Segment &s) {
    const uint32_t rt_first = u0 / p.units_per_tile;
    const uint32_t rt = rt_first + i;
    const uint32_t tile_u0 = rt * p.units_per_tile, tile_u1 = tile_u0 + p.units_per_tile;
    if (tile_u0 >= u1) return false;
    const uint32_t a = max(u0, tile_u0), b = min(u1, tile_u1);
    s.rt = rt;
    s.kb0 = 2 * (a - tile_u0);
    s.kb1 = min(2 * (b - tile_u0), p.kb);
    return true;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,"
        "%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

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

// barrier slots
constexpr int kBarCodeFull = 0, kBarCodeEmpty = kBarCodeFull + kMaxCodeStages,
              kBarAFull = kBarCodeEmpty + kMaxCodeStages, kBarAEmpty = kBarAFull + kASlots,
              kBarSegDone = kBarAEmpty + kASlots, kBarLut = kBarSegDone + kMaxSegments;  // one more after it

// The lookup table in its shared-memory form -- entry (byte, lane) = half2 {level[byte & 15],
// level[byte >> 4]}, one copy per lane so no two lanes ever share a bank -- built at compile
// time and brought in with a single bulk copy.
struct LutImage {
    uint32_t v[256 * 32];
};
constexpr LutImage make_lut_image() {
    constexpr uint32_t h[16] = {NF4_LEVEL_F16_BITS_LIST};
    LutImage t{};
    for (int byte = 0; byte < 256; ++byte)
        for (int lane = 0; lane < 32; ++lane)
            t.v[byte * 32 + lane] = h[byte & 15] | (h[byte >> 4] << 16);
    return t;
}
__device__ __align__(128) const LutImage g_lut_image = make_lut_image();

template <bool DQ>
__global__ void __launch_bounds__(kThreads, 1)
decode2_kernel(const __grid_constant__ CUtensorMap tmap_codes,
               const __grid_constant__ CUtensorMap tmap_scales, const Decode2Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem);                       // 32 KB
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kLutBytes);          // < 512 B
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kLutBytes + 512);
    int *last_flag = reinterpret_cast<int *>(smem + kLutBytes + 520);
    float *t_s = reinterpret_cast<float *>(smem + kLutBytes + 1024);          // [16][64] f32
    uint8_t *x_s = smem + p.off_x;                                            // x_blocks * 2 KB
    uint8_t *ring = smem + p.off_ring;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t grid = gridDim.x, cta = blockIdx.x;
    const uint32_t u0 = run_start(cta, p.total_units, grid);
    const uint32_t u1 = run_start(cta + 1, p.total_units, grid);
    const uint32_t S = p.code_stages;
    const uint32_t bar0 = ptx::smem_addr(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    // x's block range kept in shared memory: slot(kb) = (kb - x_base) mod p.kb
    Segment seg0;
    segment_of(p, u0, u1, 0, seg0);
    const uint32_t x_base = (p.x_blocks == p.kb) ? 0u : seg0.kb0;

    auto issue_stage = [&](uint32_t st, uint32_t rt, uint32_t g4) {
        const uint32_t s = st % S;
        uint8_t *dst = ring + s * kStageBytes;
        ptx::mbar_arrive_expect_tx(bar(kBarCodeFull + s), kStageBytes);
        ptx::tma_load_2d(ptx::smem_addr(dst), &tmap_codes, (int32_t)(g4 * 128),
                         (int32_t)(rt * kRowsPerTile), bar(kBarCodeFull + s));
        // scales: f32 -> the tile's 4 blocks; u8 -> the 16-block group holding them
        const int32_t sx = DQ ? (int32_t)((g4 * 4) & ~15u) : (int32_t)(g4 * 4);
        ptx::tma_load_2d(ptx::smem_addr(dst + kCodeStageBytes), &tmap_scales, sx,
                         (int32_t)(rt * kRowsPerTile), bar(kBarCodeFull + s));
    };

    // ------------------------------- set-up -------------------------------
    if (warp == kWarpTma) {
        if (lane == 0) {
            for (uint32_t s = 0; s < S; ++s) {
                ptx::mbar_init(bar(kBarCodeFull + s), 1);
                ptx::mbar_init(bar(kBarCodeEmpty + s), kExpanderWarps);
            }
            for (int s = 0; s < kASlots; ++s) {
                ptx::mbar_init(bar(kBarAFull + s), 4);
                ptx::mbar_init(bar(kBarAEmpty + s), 1);
            }
            for (int s = 0; s < kMaxSegments; ++s) ptx::mbar_init(bar(kBarSegDone + s), kIssuerWarps);
            ptx::mbar_init(bar(kBarLut), 1);
            ptx::fence_mbar_init();
            ptx::fence_proxy_async();
        }
        // let the expanders' few requests for x leave first: once ~100 KB of bulk copies are
        // queued per SM, a late request waits microseconds behind them
        asm volatile("bar.sync 3, %0;" ::"n"((kExpanderWarps + 1) * 32) : "memory");
        if (lane == 0) {
            // nothing else touches the ring or the table before the set-up barrier below, so
            // the first requests leave right away
            ptx::mbar_arrive_expect_tx(bar(kBarLut), kLutBytes);
            ptx::bulk_g2s(ptx::smem_addr(lut), &g_lut_image, kLutBytes, bar(kBarLut));
            uint32_t st = 0;
            Segment sg;
            for (uint32_t i = 0; st < S && segment_of(p, u0, u1, i, sg); ++i)
                for (uint32_t g4 = sg.kb0 / 4; g4 * 4 < sg.kb1 && st < S; ++g4, ++st)
                    issue_stage(st, sg.rt, g4);
        }
    } else if (warp == kWarpIssuer0) {
        ptx::tmem_alloc(ptx::smem_addr(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    } else if (warp < kExpanderWarps) {
        // ---- x's k-range -> f16, canonical K-major 128B-swizzled rows (16 rows per block) ----
        // one 16-byte chunk (8 values) per thread and step, four loads in flight; rows >= M are zero
        const uint32_t chunks = p.x_blocks * 16 * 8;
        constexpr uint32_t nthreads = kExpanderWarps * 32;
        bool released = false;
        for (uint32_t base = tid; base < chunks; base += 4 * nthreads) {
            uint4 v[4];
            #pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = base + u * nthreads;
                const uint32_t slot = i >> 7, row = (i >> 3) & 15u, c = i & 7u;
                uint32_t kb = slot + x_base;
                if (kb >= p.kb) kb -= p.kb;
                v[u] = make_uint4(0, 0, 0, 0);
                if (i < chunks && row < p.M)
                    v[u] = __ldg(reinterpret_cast<const uint4 *>(
                        p.x + (size_t)row * p.K + (size_t)kb * 64 + c * 8));
            }
            if (!released) {  // first batch of loads is out: release the producer
                asm volatile("bar.arrive 3, %0;" ::"n"((kExpanderWarps + 1) * 32) : "memory");
                released = true;
            }
            #pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = base + u * nthreads;
                if (i >= chunks) break;
                const uint32_t slot = i >> 7, row = (i >> 3) & 15u, c = i & 7u;
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                uint32_t h[4];
                #pragma unroll
                for (int q = 0; q < 4; ++q)
                    h[q] = pack_h2(__uint_as_float(w[q] << 16), __uint_as_float(w[q] & 0xffff0000u));
                uint8_t *dst = x_s + slot * kXBlockBytes + (row >> 3) * 1024 + (row & 7u) * 128 +
                               ((c ^ (row & 7u)) << 4);
                *reinterpret_cast<uint4 *>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
            }
        }
        if (!released) asm volatile("bar.arrive 3, %0;" ::"n"((kExpanderWarps + 1) * 32) : "memory");
        ptx::fence_proxy_async();  // x_s is read by the tensor core through the async proxy
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + kMaxSegments * kAccPerSeg * kAccCols;

    bool ok = true;

    if (warp == kWarpTma) {
        // ============================== TMA producer ==============================
        if (lane == 0) {
            uint32_t st = 0;
            Segment sg;
            for (uint32_t i = 0; ok && segment_of(p, u0, u1, i, sg); ++i) {
                for (uint32_t g4 = sg.kb0 / 4; g4 * 4 < sg.kb1; ++g4, ++st) {
                    if (st < S) continue;  // requested before the set-up barrier
                    const uint32_t s = st % S, ph = (st / S) & 1u;
                    if (!ptx::mbar_wait_bounded(bar(kBarCodeEmpty + s), ph ^ 1u)) {
                        ok = false;
                        break;
                    }
                    issue_stage(st, sg.rt, g4);
                }
            }
            if (!ok) NF4_REPORT_FAILURE(g_decode2_error, g_decode2_error_host, 1);
        }
    } else if (warp >= kWarpIssuer0 && warp < kWarpIssuer0 + kIssuerWarps) {
        // ============================== MMA issuers ==============================
        // Issuing a tcgen05.mma costs its thread ~100 cycles, far more than a 128 x 16 x 16
        // MMA takes to run, so four threads issue side by side: issuer g takes the blocks
        // kb % 4 == g (the ones expander group g writes) and owns two accumulators per segment.
        if (lane == 0) {
            const uint32_t g = warp - kWarpIssuer0;
            // f16 x f16 -> f32, M = 128, N = 16, both K-major
            constexpr uint32_t idesc = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t xs_addr = ptx::smem_addr(x_s);
            uint32_t bc_base = 0;
            Segment sg;
            for (uint32_t i = 0; ok && segment_of(p, u0, u1, i, sg); ++i) {
                uint32_t lb = 0;
                for (uint32_t kb = (sg.kb0 & ~3u) + g; kb < sg.kb1; kb += 4) {
                    if (kb < sg.kb0) continue;
                    const uint32_t bc = bc_base + (kb - sg.kb0);
                    const uint32_t slot = bc % kASlots, ph = (bc / kASlots) & 1u;
                    if (!ptx::mbar_wait_bounded(bar(kBarAFull + slot), ph)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t xslot = kb >= x_base ? kb - x_base : kb + p.kb - x_base;
                    const uint64_t bdesc = make_kmajor_sw128_desc(xs_addr + xslot * kXBlockBytes);
                    const uint32_t acc = tmem_base + (i * kAccPerSeg + g * 2 + (lb & 1u)) * kAccCols;
                    const uint32_t a = tmem_a + slot * 32;
                    const uint32_t first = lb >= 2 ? 1u : 0u;
                    ptx::mma_ts_f16(acc, a, bdesc, idesc, first);
                    ptx::mma_ts_f16(acc, a + 8, bdesc + 2, idesc, 1u);
                    ptx::mma_ts_f16(acc, a + 16, bdesc + 4, idesc, 1u);
                    ptx::mma_ts_f16(acc, a + 24, bdesc + 6, idesc, 1u);
                    ptx::tc_commit(bar(kBarAEmpty + slot));
                    ++lb;
                }
                if (ok) ptx::tc_commit(bar(kBarSegDone + i));
                bc_base += sg.kb1 - sg.kb0;
            }
            if (!ok) NF4_REPORT_FAILURE(g_decode2_error, g_decode2_error_host, 2);
        }
    } else if (warp < kExpanderWarps) {
        // ================================ expanders ================================
        const uint32_t q = warp & 3u, grp = warp >> 2;   // TMEM lane quarter, block within a tile
        const uint32_t row = q * 32 + lane;              // row inside the 128-row tile = TMEM lane
        const float sos = DQ ? __ldg(p.scale_of_scales) : 0.0f;
        const uint32_t *lut_lane = lut + lane;
        const uint32_t swz = row & 7u;
        uint32_t st = 0, bc_base = 0;
        ok = ptx::mbar_wait_bounded(bar(kBarLut), 0);
        Segment sg;
        for (uint32_t i = 0; ok && segment_of(p, u0, u1, i, sg); ++i) {
            for (uint32_t g4 = sg.kb0 / 4; g4 * 4 < sg.kb1; ++g4, ++st) {
                const uint32_t s = st % S, ph = (st / S) & 1u;
                if (!ptx::mbar_wait_bounded(bar(kBarCodeFull + s), ph)) {
                    ok = false;
                    break;
                }
                const uint32_t kb = g4 * 4 + grp;
                if (kb >= sg.kb0 && kb < sg.kb1) {
                    const uint8_t *stage = ring + s * kStageBytes;
                    const uint8_t *rowp = stage + row * 128;
                    const uint4 c0 = *reinterpret_cast<const uint4 *>(rowp + (((2 * grp) ^ swz) << 4));
                    const uint4 c1 = *reinterpret_cast<const uint4 *>(rowp + (((2 * grp + 1) ^ swz) << 4));
                    float scale;
                    if (DQ)
                        scale = dq_scale(stage[kCodeStageBytes + row * 16 + (kb & 15u)], sos);
                    else
                        scale = reinterpret_cast<const float *>(stage + kCodeStageBytes)[row * 4 + grp];
                    const uint32_t s2 = pack_h2(scale, scale);
                    const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    uint32_t out[32];
                    #pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        #pragma unroll
                        for (int b = 0; b < 4; ++b)
                            out[4 * e + b] = hmul2(lut_lane[((w[e] >> (8 * b)) & 0xffu) << 5], s2);
                    }
                    const uint32_t bc = bc_base + (kb - sg.kb0);
                    const uint32_t slot = bc % kASlots, pha = (bc / kASlots) & 1u;
                    if (!ptx::mbar_wait_bounded(bar(kBarAEmpty + slot), pha ^ 1u)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    tmem_st32(tmem_a + ((q * 32) << 16) + slot * 32, out);
                    ptx::tmem_wait_st();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(kBarAFull + slot));
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(kBarCodeEmpty + s));
            }
            bc_base += sg.kb1 - sg.kb0;
        }
        if (!ok && lane == 0) NF4_REPORT_FAILURE(g_decode2_error, g_decode2_error_host, 3);
    } else if (warp >= kWarpFinish0) {
        // ================================= finish =================================
        // Four dedicated warps (one per TMEM lane quarter) finish a segment as soon as its MMAs
        // are done, so only the last segment's finish is exposed at the end of the kernel.
        const uint32_t q = warp & 3u;
        const uint32_t row = q * 32 + lane;  // TMEM lane = row inside the 128-row tile
        const uint32_t ftid = (warp - kWarpFinish0) * 32 + lane;
        Segment sg;
        // this thread's LoRA-B rows (one per segment) are fetched now, long before they are needed
        uint4 lbq[kMaxSegments][2];
        const bool lb_in_regs = p.rank == 16;
        #pragma unroll
        for (int i = 0; i < kMaxSegments; ++i) {
            lbq[i][0] = lbq[i][1] = make_uint4(0, 0, 0, 0);
            if (lb_in_regs && segment_of(p, u0, u1, i, sg)) {
                const uint32_t n = sg.rt * kRowsPerTile + row;
                if (n < p.N) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(p.lora_b + (size_t)n * 16);
                    lbq[i][0] = __ldg(src);
                    lbq[i][1] = __ldg(src + 1);
                }
            }
        }
        // T = x A^T comes from the pre-pass, which may still be running (programmatic dependent
        // launch): wait for it here, with this kernel's streaming already under way
        if (p.rank) {
            ptx::pdl_wait();
            for (uint32_t i = ftid; i < p.M * p.rank; i += 128) t_s[i] = __ldcg(p.t + i);
            asm volatile("bar.sync 2, 128;" ::: "memory");
        }
        #pragma unroll
        for (uint32_t i = 0; i < (uint32_t)kMaxSegments; ++i) {
            if (!segment_of(p, u0, u1, i, sg)) break;
            if (ok) ok = ptx::mbar_wait_bounded(bar(kBarSegDone + i), 0);
            ptx::tc_fence_after();
            float v[16];
            #pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = 0.0f;
            // issuer g wrote accumulator 2g (and 2g+1 when it had a second block in the segment)
            #pragma unroll
            for (uint32_t g = 0; g < 4; ++g) {
                const uint32_t first_kb = (sg.kb0 & ~3u) + g + ((((sg.kb0 & ~3u) + g) < sg.kb0) ? 4u : 0u);
                const uint32_t cnt = first_kb < sg.kb1 ? (sg.kb1 - first_kb + 3) / 4 : 0u;
                for (uint32_t a = 0; a < (cnt < 2u ? cnt : 2u); ++a) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((q * 32) << 16) + (i * kAccPerSeg + g * 2 + a) * kAccCols, r);
                    ptx::tmem_wait_ld();
                    #pragma unroll
                    for (int m = 0; m < 16; ++m) v[m] += ok ? __uint_as_float(r[m]) : 0.0f;
                }
            }
            const bool whole = sg.kb0 == 0 && sg.kb1 == p.kb;
            bool finish = whole;
            uint32_t c_first = cta, c_last = cta;
            bool own_in_memory = false;
            if (!whole) {
                c_first = cta_of_unit(sg.rt * p.units_per_tile, p.total_units, grid);
                c_last = cta_of_unit((sg.rt + 1) * p.units_per_tile - 1, p.total_units, grid);
                const int others = (int)(c_last - c_first);
                // everyone else already in?  then this CTA finishes the tile straight from its
                // registers and never writes its own partial
                if (ftid == 0) *last_flag = (atomicAdd(p.counters + sg.rt, 0) == others) ? 1 : 0;
                asm volatile("bar.sync 2, 128;" ::: "memory");
                finish = *last_flag != 0;
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (!finish) {
                    float *dst = p.partials + (size_t)(cta + sg.rt) * (16 * kRowsPerTile);
                    #pragma unroll
                    for (int m = 0; m < 16; ++m) dst[m * kRowsPerTile + row] = v[m];
                    __threadfence();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (ftid == 0) *last_flag = (atomicAdd(p.counters + sg.rt, 1) == others) ? 1 : 0;
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    finish = *last_flag != 0;
                    own_in_memory = true;
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                }
                if (finish) {
                    __threadfence();
                    float own[16];
                    #pragma unroll
                    for (int m = 0; m < 16; ++m) {
                        own[m] = v[m];
                        v[m] = 0.0f;
                    }
                    // fixed order c_first .. c_last, whoever happens to be last
                    for (uint32_t c = c_first; c <= c_last; ++c) {
                        if (c == cta && !own_in_memory) {
                            #pragma unroll
                            for (int m = 0; m < 16; ++m) v[m] += own[m];
                        } else {
                            const float *src = p.partials + (size_t)(c + sg.rt) * (16 * kRowsPerTile);
                            #pragma unroll
                            for (int m = 0; m < 16; ++m) v[m] += __ldcg(src + m * kRowsPerTile + row);
                        }
                    }
                }
            }
            const uint32_t n = sg.rt * kRowsPerTile + row;
            if (finish && n < p.N) {
                const float b = p.bias ? __ldg(p.bias + n) : 0.0f;
                float dot[16];
                #pragma unroll
                for (int m = 0; m < 16; ++m) dot[m] = 0.0f;
                if (lb_in_regs) {
                    const uint32_t w[8] = {lbq[i][0].x, lbq[i][0].y, lbq[i][0].z, lbq[i][0].w,
                                           lbq[i][1].x, lbq[i][1].y, lbq[i][1].z, lbq[i][1].w};
                    #pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) {
                        const float bj = __uint_as_float((j & 1u) ? (w[j >> 1] & 0xffff0000u) : (w[j >> 1] << 16));
                        #pragma unroll
                        for (uint32_t m = 0; m < 16; ++m)
                            if (m < p.M) dot[m] = fmaf(t_s[m * 16 + j], bj, dot[m]);
                    }
                } else {
                    for (uint32_t j = 0; j < p.rank; ++j) {
                        const float bj = __bfloat162float(p.lora_b[(size_t)n * p.rank + j]);
                        #pragma unroll
                        for (uint32_t m = 0; m < 16; ++m)
                            if (m < p.M) dot[m] = fmaf(t_s[m * p.rank + j], bj, dot[m]);
                    }
                }
                #pragma unroll
                for (uint32_t m = 0; m < 16; ++m) {
                    if (m >= p.M) break;
                    const float o = fmaf(dot[m], p.lora_scale, v[m]) + b;  // scale applied last
                    const size_t idx = (size_t)m * p.ldy + n;
                    if (p.y_f32) static_cast<float *>(p.y)[idx] = o;
                    else static_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(o);
                }
            }
        }
        if (!ok && lane == 0) NF4_REPORT_FAILURE(g_decode2_error, g_decode2_error_host, 4);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == kWarpIssuer0) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

int32_t make_map(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(NF4_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NF4_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return NF4_OK;
}

struct Plan {
    Decode2Params p;
    uint32_t grid, smem_bytes;
    uint64_t off_counters, off_partials, ws_bytes;
};

uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

bool shape_ok(uint64_t rows, uint64_t d_in, uint64_t d_out, bool dq, uint32_t rank) {
    if (rows == 0 || rows > 16) return false;
    if (d_in % 64 != 0 || d_in > (1u << 20) || d_out >= (1ull << 31)) return false;
    const uint32_t kb = (uint32_t)(d_in / 64);
    // TMA needs 16-byte row pitches for the scale tensor
    if (!dq && kb % 4 != 0) return false;
    if (dq && kb % 16 != 0) return false;
    if (rank > (uint32_t)kMaxRank) return false;
    return true;
}

bool make_plan(uint64_t rows, uint64_t d_in, uint64_t d_out, bool dq, uint32_t rank, Plan &pl) {
    if (!shape_ok(rows, d_in, d_out, dq, rank)) return false;
    Decode2Params &p = pl.p;
    p = Decode2Params{};
    p.M = (uint32_t)rows;
    p.K = (uint32_t)d_in;
    p.N = (uint32_t)d_out;
    p.rank = rank;
    p.kb = p.K / 64;
    p.units_per_tile = (p.kb + 1) / 2;
    p.row_tiles = (p.N + kRowsPerTile - 1) / kRowsPerTile;
    const uint64_t units = (uint64_t)p.row_tiles * p.units_per_tile;
    if (units >= (1ull << 31)) return false;
    p.total_units = (uint32_t)units;
    uint32_t grid = p.total_units < (uint32_t)kNumSMs ? p.total_units : (uint32_t)kNumSMs;
    // a run may not need more x blocks than fit, nor more segments than accumulators
    for (;;) {
        const uint32_t run = (p.total_units + grid - 1) / grid;           // units
        const uint32_t blocks = run * 2 < p.kb ? run * 2 : p.kb;
        const uint32_t segs = run >= p.units_per_tile
                                  ? (run + p.units_per_tile - 1) / p.units_per_tile + 1 : 2;
        if (blocks <= (uint32_t)kMaxXBlocks && segs <= (uint32_t)kMaxSegments) {
            p.x_blocks = blocks;
            break;
        }
        if (p.kb <= (uint32_t)kMaxXBlocks && segs > (uint32_t)kMaxSegments) {
            // many short row-tiles per run: more CTAs (several waves) keep the segment count down
            const uint32_t want = (p.total_units + (kMaxSegments - 1) * p.units_per_tile - 1) /
                                  ((kMaxSegments - 1) * p.units_per_tile);
            if (want <= grid) return false;
            grid = want;
            continue;
        }
        if (blocks > (uint32_t)kMaxXBlocks) {
            const uint32_t want = (p.total_units + kMaxXBlocks / 2 - 1) / (kMaxXBlocks / 2);
            if (want <= grid) return false;
            grid = want;
            continue;
        }
        return false;
    }
    pl.grid = grid;
    p.off_x = kLutBytes + 1024 + 16 * kMaxRank * 4;
    p.off_x = round_up(p.off_x, 1024);
    p.off_ring = round_up(p.off_x + p.x_blocks * kXBlockBytes, 1024);
    uint32_t stages = kMaxCodeStages;
    while (stages >= 2 && 1024 + p.off_ring + stages * kStageBytes > (uint32_t)kSmemLimit) --stages;
    if (stages < 2) return false;
    p.code_stages = stages;
    pl.smem_bytes = 1024 + p.off_ring + stages * kStageBytes;
    auto up = [](uint64_t v) { return (v + 255) / 256 * 256; };
    pl.off_counters = up((uint64_t)16 * kMaxRank * 4);
    pl.off_partials = pl.off_counters + up((uint64_t)p.row_tiles * 4);
    pl.ws_bytes = pl.off_partials + (uint64_t)(grid + p.row_tiles) * 16 * kRowsPerTile * 4;
    return true;
}

template <bool DQ>
int32_t launch(const CUtensorMap &mc, const CUtensorMap &ms, const Plan &pl, cudaStream_t stream) {
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(decode2_kernel<DQ>), kSmemLimit));
    count_launch();
    return launch_maybe_overlapped(decode2_kernel<DQ>, dim3(pl.grid), dim3(kThreads), pl.smem_bytes,
                                   stream, pl.p.rank != 0, mc, ms, pl.p);
}

}  // namespace


// lora_t_small lives in decode_gemv.cu
int32_t lora_t_small(const void *x, const void *a, uint32_t rows, uint32_t K, uint32_t rank,
                     float *t_out, cudaStream_t stream, bool chained);

bool decode2_supported(const nf4_linear_args &a) {
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_BF16) return false;
    const bool dq = a.scale_codes != nullptr;
    const void *scales = dq ? (const void *)a.scale_codes : (const void *)a.absmax;
    if (!aligned16(a.x) || !aligned16(a.packed) || !aligned16(scales)) return false;
    // the adapter factors are read with 16-byte loads: views at odd offsets go to the general kernel
    if (a.lora_a && (!aligned16(a.lora_a) || !aligned16(a.lora_b))) return false;
    if (reinterpret_cast<uintptr_t>(a.y) & (a.y_f32 ? 3u : 1u)) return false;
    Plan pl;
    return make_plan(a.rows, a.d_in, a.d_out, dq, a.lora_a ? a.lora_rank : 0, pl);
}

uint64_t decode2_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    // the scale form is not known here: size for whichever of the two plans is larger
    uint64_t need = 0;
    Plan pl;
    if (make_plan(rows, d_in, d_out, false, lora_rank, pl)) need = pl.ws_bytes;
    if (make_plan(rows, d_in, d_out, true, lora_rank, pl) && pl.ws_bytes > need) need = pl.ws_bytes;
    return need;
}

int32_t decode2_forward(const nf4_linear_args &a, cudaStream_t stream) {
    const bool dq = a.scale_codes != nullptr;
    Plan pl;
    if (!make_plan(a.rows, a.d_in, a.d_out, dq, a.lora_a ? a.lora_rank : 0, pl))
        return fail(NF4_ERR_UNSUPPORTED, "decode2_forward: unsupported shape");
    Decode2Params &p = pl.p;
    uint8_t *ws = static_cast<uint8_t *>(a.workspace);
    float *t = reinterpret_cast<float *>(ws);
    p.counters = reinterpret_cast<int *>(ws + pl.off_counters);
    p.partials = reinterpret_cast<float *>(ws + pl.off_partials);
    p.x = static_cast<const __nv_bfloat16 *>(a.x);
    p.bias = a.bias;
    p.lora_b = static_cast<const __nv_bfloat16 *>(a.lora_b);
    p.y = a.y;
    p.y_f32 = (uint32_t)a.y_f32;
    p.ldy = a.ldy ? a.ldy : a.d_out;
    p.lora_scale = a.lora_scale;
    p.scale_of_scales = a.scale_of_scales;
    NF4_CUDA_TRY(cudaMemsetAsync(p.counters, 0, (size_t)p.row_tiles * 4, stream));
    if (p.rank) {
        NF4_TRY(lora_t_small(a.x, a.lora_a, p.M, p.K, p.rank, t, stream, false));
        p.t = t;
    }
    CUtensorMap mc, ms;
    NF4_TRY(make_map(&mc, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.packed, p.N, p.K / 2, p.K / 2,
                     kRowsPerTile, 128, CU_TENSOR_MAP_SWIZZLE_128B));
    if (dq)
        NF4_TRY(make_map(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.scale_codes, p.N, p.kb, p.kb,
                         kRowsPerTile, 16, CU_TENSOR_MAP_SWIZZLE_NONE));
    else
        NF4_TRY(make_map(&ms, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.absmax, p.N, p.kb, (uint64_t)p.kb * 4,
                         kRowsPerTile, 4, CU_TENSOR_MAP_SWIZZLE_NONE));
    return dq ? launch<true>(mc, ms, pl, stream) : launch<false>(mc, ms, pl, stream);
}

int32_t decode2_set_host_flag(int *mapped) {
    return check_cuda(cudaMemcpyToSymbol(g_decode2_error_host, &mapped, sizeof(mapped)), "setting the mapped failure word");
}

int32_t decode2_error_flag_ptr(int **dev_ptr) {
    return check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(dev_ptr), g_decode2_error),
                      "address of the split-K decode error flag");
}

}  // namespace nf4
