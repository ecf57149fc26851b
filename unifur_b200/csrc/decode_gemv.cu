// Decode path: y[M<=16, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T), W stored as
// packed NF4 [N, K] with 64-blocks along K.  HBM-bound: the kernel exists to stream
// nibbles + scales once at full bandwidth.
//
// Data movement.  One CTA per SM owns a contiguous range of W rows.  Its sixteen warps split K
// into slices of 256 (four 64-blocks); when K is short the warps left over take other 16-row
// tiles.  Every warp streams its own slice with TMA: one lane asks for a 2-D box of
// 16 rows x 128 bytes of nibbles (128-byte swizzle) and a box of 16 rows x 4 f32 block scales,
// both into the warp's private ring of two tiles, and the box's arrival is counted on the
// warp's own mbarrier.  No warp ever waits for another while the weights stream: there is no
// producer warp and no CTA-wide barrier inside a pass.  The tensor maps cover this GPU's weight
// only and every load goes to one CTA.  The requests for the first tiles (and the loads of the
// adapter's A factor) are made BEFORE the kernel waits for its predecessor in the stream
// (programmatic dependent launch): weights are immutable, so they may be fetched while the
// kernel that produces x is still running.
//
// Math.  Dequantisation is a shared-memory table lookup: one packed byte (two codes) indexes a
// 256-entry table of half2 {level[lo], level[hi]}, replicated once per lane so that no two lanes
// share a bank; entries sit 256 bytes apart from the start of dynamic shared memory, so one byte
// permute (code byte into bits 8..15 above the lane's offset) forms the address and the table's
// base rides in the load's immediate: two instructions per pair of weights.  The looked-up
// register IS the A operand of a warp MMA (m16n8k16, f16 in / f32 accumulate) with W rows on
// the MMA's M side (MMA row g holds tile row 2g, row g+8 holds 2g+1: the rows a half-warp reads
// then fall into different banks of the swizzled box) and the <=16 activation rows on its N
// side.  Each warp keeps its slice of x as f16 B-fragments in registers for the whole kernel.
// A block's four MMAs accumulate in one chain and the result is scaled by the block's f32
// absmax (or its double-quantized decode) -- the scale never touches the f16 path.
//
// Adapter.  T = x A^T ([M][rank] f32) is needed by every CTA but costs rank * K * 2 bytes of A to
// compute, so it is computed once per launch: the first rank / 8 CTAs each take eight rows of A
// (their warps hold the matching slices of x already: sixteen bf16 MMAs per warp), write their
// columns of T to the workspace and count themselves in on a flag word there.  A CTA picks T up
// before the last tile of its first pass -- by then the producers have long finished -- with a
// bounded wait on the flag.  The last CTA to have read T puts the flag words back to zero, which
// is the state the workspace must have at first use.
//
// Longer K, several forwards, several GPUs.  d_in above 4096 is cut into parts that groups of
// CTAs multiply (SPLIT: the parts' sums meet in the workspace, the last CTA of a row range adds
// them in a fixed order).  Forwards that share x run as one launch whose CTAs are shared out
// between them (decode_group_kernel).  A column-sharded layer's kernel can store its columns
// into every rank's output over NVLink and signal the ranks (PEERS).
//
// Reduction.  When a warp has multiplied a tile it parks the tile's partial sums (four f32 per
// lane and eight activation rows) in its own row of a parking area in shared memory.  After a
// pass of tiles (all of a CTA's rows in the usual case) every warp takes one (tile, eight
// activation rows) job: it sums the K-warps' partials in a fixed order (so results do not depend
// on timing), adds the LoRA term with one bf16 MMA pair per sixteen ranks (LoRA-B rows x T, T split
// into bf16 high and low parts) and the bias, converts and stores.
//
// Code size.  The tile loop is rolled and nothing in it is replicated per tile: the kernel is
// launched once per forward and runs for microseconds, so code that is executed once is fetched
// from memory every time, and a 90 KB kernel (the tile body unrolled five times) spent most of
// its time waiting for instructions.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

// Set when the launch's shared-memory window is not where the kernel expects it (4) or a
// bounded wait gives up (5: a tile, 6: the adapter intermediate, 7: the ranks' arrivals).  Read
// and cleared by nf4_device_status().
__device__ int g_decode_error = 0;
__device__ int *g_decode_error_host = nullptr;  // the same, in mapped host memory (set by the host-pointer entry points)

int32_t lora_t_small(const void *x, const void *a, uint32_t rows, uint32_t K, uint32_t rank,
                     float *t_out, cudaStream_t stream, bool chained);

namespace {

constexpr int kTileRows = 16;
constexpr int kChunk = 64;         // one quantization block of K
constexpr int kSliceChunks = 4;    // blocks per K-slice
constexpr int kSliceK = kSliceChunks * kChunk;
constexpr int kMaxSlices = 16;     // slices of K a CTA multiplies (its sixteen warps)
constexpr int kMaxParts = 8;       // parts of K that CTAs share out: K <= 8 * 16 * 256
constexpr int kMaxRank = 64;
constexpr uint32_t kFlagBytes = 256;  // workspace: [ready, done] words, then T
constexpr uint32_t kWin0 = 1024;   // shared-window address of dynamic shared memory
constexpr uint32_t kCodesSlot = kTileRows * 128;  // one K-slice of one tile: nibbles
constexpr uint32_t kScaleSlot = kTileRows * 16;   // ... and its block scales
constexpr uint32_t kParkSlots = 10; // (tile, eight activation rows) results a warp can park per pass
constexpr uint32_t kGapRows = 256;  // LoRA-B rows the table's gaps hold (one row of up to 128 bytes each)

// One CTA per SM: sixteen warps, one K-slice each.  Two tiles per warp ring: with 148 CTAs that is
// ~70 KB per SM in flight, about what HBM bandwidth times latency needs; deeper rings only queue
// requests up in the memory system and make every other load (x, the adapter) wait behind them
// (four tiles per ring measured 13.8 us per forward against 10.1 us with two).
struct Cfg {
    static constexpr int kWarps = 16;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kSlices = 1;  // K-slices per warp
    static constexpr int kRing = 2;    // tiles per warp ring
    static constexpr uint32_t kLutStride = 256;  // bytes between table entries (128 used)
    static constexpr uint32_t kLutBytes = 256 * kLutStride;
    static constexpr uint32_t kCodesTile = kSlices * kCodesSlot;
    static constexpr uint32_t kScaleTile = kSlices * kScaleSlot;
    // byte offsets from the start of dynamic shared memory
    static constexpr uint32_t kOffCodes = kLutBytes;
    static constexpr uint32_t kOffScales = kOffCodes + kWarps * kRing * kCodesTile;
    static constexpr uint32_t kOffBars = kOffScales + kWarps * kRing * kScaleTile;
    // [warps][2][8][8] f32: a producer's slices of a unit of T (8 KB).  The upper half is where T
    // itself arrives later, asked for by warp 0, which is among the readers of the slices.
    static constexpr uint32_t kOffRed = kOffBars + 512;
    static constexpr uint32_t kOffT = kOffRed + 4096;
    static constexpr uint32_t kTBytes = 16 * kMaxRank * 4;
    static constexpr uint32_t kOffDq = kOffT + kTBytes;
    static constexpr uint32_t kOffPark = kOffDq + 1024;              // [warps][kParkSlots][32 lanes] float4
    static constexpr uint32_t kSmemBytes = kOffPark + kWarps * kParkSlots * 512;
    static_assert(kWarps * kRing * 8 <= 512, "barrier room");
    static_assert((kWin0 + kOffCodes) % 1024 == 0, "swizzled boxes need 1024-byte alignment");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory");
};

struct DecodeParams {
    const __nv_bfloat16 *x;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const float *bias;
    float *t_global;       // [part][M][rank] f32 = x A^T over the part's K, written by the producer CTAs (workspace)
    uint32_t *flags;       // [0] producers that have published, [1] CTAs that have read T, [2...] arrival counters
    uint32_t n_prod;       // CTAs of a K-part that compute T (each takes the units cta, cta + n_prod, ...; a unit is 8 columns)
    uint32_t n_prod_all;   // ... of all K-parts: the count the readers of T wait for
    // K longer than sixteen slices is split into kparts parts of part_slices slices; part i is
    // multiplied by the CTAs i * cpp ... (i + 1) * cpp - 1, which share the rows like the CTAs of
    // an unsplit launch do.  The parts' results meet in `partial` ([part][M][N] f32); the CTA
    // that arrives last for a row range (a byte counter per range after the two flag words) adds
    // them in the order of the parts and writes y.
    uint32_t kparts, part_slices, cpp;
    float *partial;
    const __nv_bfloat16 *lora_a;
    const __nv_bfloat16 *lora_b;
    void *y;
    uint64_t ldy;
    uint32_t y_f32;
    uint32_t y_pair;       // bf16 y whose even columns are 4-byte aligned in every row
    // Sharded layer whose ranks write their columns straight into every rank's output (PEERS):
    // dest[d] is rank d's output as mapped into this process, already at this rank's first
    // column, with row stride ldy; arrive[d] is rank d's arrival counter.
    // signal: when the kernel's last CTA is done it makes the launch's stores visible system-wide
    // and adds one to every rank's counter (word 63 of `flags` counts the CTAs that are done).
    // wait_on: before it reads x, every CTA waits (bounded) until wait_expected arrivals are on
    // this rank's counter -- x is the output of a sharded layer -- and the last CTA takes them off.
    void *dest[8];
    uint32_t *arrive[8];
    uint32_t n_dest, signal;
    uint32_t *wait_on;
    uint32_t wait_expected;
    uint32_t M, K, N, rank;
    float lora_scale;
    // CTA c owns rows_base rows, and gran more if light_front <= c < light_front + rows_extra;
    // ranges start on multiples of gran
    uint32_t gran, rows_base, rows_extra, light_front;
    uint32_t kw;          // K-slices of 256
    uint32_t kwarps;      // warps along K
    uint32_t rw_shift;    // 1 << rw_shift groups of warps take different tiles (kwarps << rw_shift <= warps)
    uint32_t pass_tiles;  // tiles per warp between two reductions
    uint32_t piece_shift; // a LoRA-B row is 1 << piece_shift pieces of 16 bytes
    uint8_t warp_rg[16];  // per warp: its group along rows (0xff: the warp has no work)
    uint8_t warp_kpos[16];  // per warp: its position along K
    uint32_t nchunks;
    uint32_t wait_ns;     // bound of every wait
};

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t pair) {
    return pack_f16x2(bf16_bits_to_float(pair & 0xffffu), __uint_as_float(pair & 0xffff0000u));
}

// Waits for a phase of an mbarrier, at most `limit_ns`; false when the time ran out.
__device__ __forceinline__ bool wait_phase(uint32_t bar, uint32_t parity, uint32_t limit_ns) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::global_timer_ns();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(2000u)
            : "memory");
        if (ok) return true;
        if (ptx::global_timer_ns() - t0 > (uint64_t)limit_ns) return false;
    }
}

// The sixteen f16 levels, read with plain loads when the table is built (a table in constant
// memory would be read with a different index per lane, which the constant cache serialises; a
// chain of selects on immediates costs sixty instructions that are fetched cold at every launch).
__device__ const uint32_t g_level_f16[16] = {NF4_LEVEL_F16_BITS_LIST};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA's share of one forward.  `bid` of `nctas`: the CTA's number among the CTAs of this
// forward (a launch can hold several forwards).  SPLIT: K is longer than a CTA's sixteen slices
// and groups of CTAs multiply parts of it.  The descriptors and `p` are kernel parameters.
template <int NT, bool DQ, bool SPLIT, bool PEERS = false>
__device__ __forceinline__ void decode_body(const CUtensorMap *tm_codes, const CUtensorMap *tm_scales,
                                            const DecodeParams &p, const uint32_t bid, const uint32_t nctas) {
    using C = Cfg;
    constexpr int kWarps = C::kWarps, kThreads = C::kThreads, SL = C::kSlices, kRing = C::kRing;
    constexpr int NC = SL * kSliceChunks;  // 64-blocks of K a warp owns
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (ptx::smem_addr(smem) != kWin0) {
        // the table's base is an immediate of the lookups: nothing can run from another address
        if (tid == 0) NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 4);
        return;
    }
    if (lane == 0) {  // the descriptors are on their way while the table is built
        ptx::prefetch_tmap(tm_codes);
        if (!DQ) ptx::prefetch_tmap(tm_scales);
    }
    float *red_s = reinterpret_cast<float *>(smem + C::kOffRed);
    float *t_s = reinterpret_cast<float *>(smem + C::kOffT);     // [SL][M][rank]
    float *dq_s = reinterpret_cast<float *>(smem + C::kOffDq);   // code / 255 for the 256 codes
    // LoRA-B rows of a pass live in the table's gaps (the unused upper half of each 256-byte row)
    const uint8_t *lora_s = smem + 128;                             // row i at + i * 256 bytes
    // parking place of a tile's partial sums: element (warp, slot, lane) is one float4
    float *park_s = reinterpret_cast<float *>(smem + C::kOffPark);
    constexpr uint32_t kParkWarp = kParkSlots * 128;                // floats per warp

    // this CTA's part of K and, within the part's CTAs, its rows
    const uint32_t part = SPLIT ? bid / p.cpp : 0u;
    const uint32_t cta = bid - part * p.cpp;
    const uint32_t part_s0 = SPLIT ? part * p.part_slices : 0u;
    const uint32_t part_s1 = SPLIT ? min(p.kw, part_s0 + p.part_slices) : p.kw;
    const uint32_t past = cta > p.light_front ? cta - p.light_front : 0u;
    const uint32_t n0 = cta * p.rows_base + min(past, p.rows_extra) * p.gran;
    const uint32_t n1 = n0 + p.rows_base + (cta >= p.light_front && past < p.rows_extra ? p.gran : 0u);
    const uint32_t ntiles = (n1 - n0 + kTileRows - 1) / kTileRows;

    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t rw = 1u << p.rw_shift;
    const uint32_t rg = p.warp_rg[warp];        // which tiles: rg, rg + rw, ...
    const bool active = rg != 0xffu;
    const uint32_t kpos = p.warp_kpos[warp];    // which K-slices: kpos * SL ...
    const uint32_t slice0 = part_s0 + kpos * SL;
    const uint32_t nsl = (active && slice0 < part_s1) ? min((uint32_t)SL, part_s1 - slice0) : 0u;  // slices this warp owns
    // (a K-warp without slices in this part -- the last part can be shorter -- has no tiles; its
    // parking place is zeroed once, so that the sums over the K-warps need not know)
    const uint32_t my_tiles = (nsl && rg < ntiles) ? (ntiles - rg + rw - 1) >> p.rw_shift : 0u;
    const uint32_t k0 = slice0 * kSliceK;

    const uint32_t bar0 = kWin0 + C::kOffBars + warp * kRing * 8u;
    const uint32_t codes0 = kWin0 + C::kOffCodes + warp * kRing * C::kCodesTile;
    const uint32_t scales0 = kWin0 + C::kOffScales + warp * kRing * C::kScaleTile;
    const uint8_t *codes_ring = smem + C::kOffCodes + warp * kRing * C::kCodesTile;
    const uint8_t *scales_ring = smem + C::kOffScales + warp * kRing * C::kScaleTile;

    // ---- this warp's barriers and its first tiles (nothing here depends on the predecessor):
    // lane (slot, slice) asks for its box, so the requests of all slots leave in one instruction ----
    auto request = [&](uint32_t j, uint32_t sl) {
        // K-slice sl of this warp's tile number j goes to slot j % kRing
        const uint32_t slot = j & (kRing - 1);
        const int32_t row0 = (int32_t)(n0 + (rg + j * rw) * kTileRows);
        const uint32_t bar = bar0 + 8 * slot;
        ptx::mbar_arrive_expect_tx(bar, DQ ? kCodesSlot : kCodesSlot + kScaleSlot);
        ptx::tma_load_2d(codes0 + slot * C::kCodesTile + sl * kCodesSlot, tm_codes,
                         (int32_t)((slice0 + sl) * 128u), row0, bar);
        if (!DQ)
            ptx::tma_load_2d(scales0 + slot * C::kScaleTile + sl * kScaleSlot, tm_scales,
                             (int32_t)((slice0 + sl) * 4u), row0, bar);
    };
    if (active && nsl == 0) {
        #pragma unroll 1
        for (uint32_t i = lane; i < kParkSlots * 32u; i += 32)
            reinterpret_cast<float4 *>(park_s + warp * kParkWarp)[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    // ---- the lookup table: each byte value's entry, one copy per lane ----
    {
        // thread (byte, half) writes sixteen lanes' copies
        const uint32_t byte = tid >> 1, half = tid & 1u;
        const uint32_t entry = __ldg(g_level_f16 + (byte & 15u)) | (__ldg(g_level_f16 + (byte >> 4)) << 16);
        const uint4 v = make_uint4(entry, entry, entry, entry);
        #pragma unroll
        for (int i = 0; i < 4; ++i)  // rotated by the byte so that a warp's stores spread over the banks
            *reinterpret_cast<uint4 *>(smem + byte * 256u + half * 64u + ((i + byte) & 3u) * 16u) = v;
    }
    if (DQ && tid < 256) dq_s[tid] = __fdiv_rn((float)tid, 255.0f);

    // ---- pass plan (the same for every warp): pass_tiles tiles per warp, then a reduction ----
    const uint32_t max_tiles = (ntiles + rw - 1) >> p.rw_shift;  // tiles of the busiest warp

    // LoRA-B rows of one pass of tiles, staged by everyone with 16-byte asynchronous copies
    auto stage_lora_b = [&](uint32_t tile0) {  // tile0: warp-local number of the pass's first tile
        if (p.rank) {
            const uint32_t r0 = n0 + ((tile0 * kTileRows) << p.rw_shift);
            if (r0 < n1) {
                const uint32_t rows = min(n1 - r0, (p.pass_tiles * kTileRows) << p.rw_shift);
                const uint8_t *src = reinterpret_cast<const uint8_t *>(p.lora_b + (size_t)r0 * p.rank);
                for (uint32_t q = tid; q < rows << p.piece_shift; q += kThreads) {
                    const uint32_t row = q >> p.piece_shift, piece = q - (row << p.piece_shift);
                    ptx::cp_async_16(kWin0 + 128u + row * 256u + piece * 16u, src + (size_t)q * 16u);
                }
            }
        }
        ptx::cp_async_commit();
    };
    stage_lora_b(0);

    if (nsl) {
        if (lane < (uint32_t)kRing) {
            ptx::mbar_init(bar0 + 8 * lane, nsl);
            ptx::fence_mbar_init();
        }
        __syncwarp();
        if (lane < (uint32_t)(kRing * SL)) {
            const uint32_t j = lane / SL, sl = lane % SL;
            if (j < my_tiles && sl < nsl) request(j, sl);
        }
    }
    uint32_t req_j = my_tiles < (uint32_t)kRing ? my_tiles : (uint32_t)kRing;  // tiles requested so far

    // ---- a producer CTA's unit of T: eight rows of the adapter factor A (row 8 * j8 + g in the
    // lanes of group g) against the warps' K-slice number h (unit = j8 * SL + h).  The lane loads
    // its sixteen consecutive k of each 64-block, the same k it holds of x, so that A's rows and
    // x's rows are the two operands of a bf16 MMA with the same order of k. ----
    const bool producer = p.rank != 0 && cta < p.n_prod;
    const bool t_warp = producer && active && rg == 0;
    uint4 araw[kSliceChunks][2];
    auto load_a = [&](uint32_t unit) {
        const uint32_t j = (unit / SL) * 8u + g, h = unit % SL;
        #pragma unroll
        for (int c = 0; c < kSliceChunks; ++c) {
            araw[c][0] = araw[c][1] = make_uint4(0, 0, 0, 0);
            if (t_warp && h < nsl) {
                const uint4 *src = reinterpret_cast<const uint4 *>(
                    p.lora_a + (size_t)j * p.K + k0 + (h * kSliceChunks + c) * kChunk + 16 * t);
                araw[c][0] = __ldg(src);
                araw[c][1] = __ldg(src + 1);
            }
        }
    };
    if (producer) load_a(cta);
    __syncthreads();  // the table is in place

    // ---- from here on the kernel reads what its predecessor wrote ----
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    if (PEERS && p.wait_on) {
        if (tid == 0) {
            const uint64_t t0 = ptx::global_timer_ns();
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_on) : "memory");
                if (v >= p.wait_expected) break;
                if (ptx::global_timer_ns() - t0 > (uint64_t)p.wait_ns) {
                    NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 7);
                    break;
                }
            }
        }
        __syncthreads();
    }

    // One K-slice of T^T = A x^T for the unit's eight rows of A and eight rows of x (raw bf16,
    // exact products, f32 sums): the lane gets T[m][j] for j = 8 * j8 + g, m = 8u + 2t and + 1.
    auto dot_slice = [&](const uint4 (&xr)[4][2]) -> float2 {
        float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        #pragma unroll
        for (int c = 0; c < kSliceChunks; ++c) {
            const uint32_t aw[8] = {araw[c][0].x, araw[c][0].y, araw[c][0].z, araw[c][0].w,
                                    araw[c][1].x, araw[c][1].y, araw[c][1].z, araw[c][1].w};
            const uint32_t xw[8] = {xr[c][0].x, xr[c][0].y, xr[c][0].z, xr[c][0].w,
                                    xr[c][1].x, xr[c][1].y, xr[c][1].z, xr[c][1].w};
            #pragma unroll
            for (int j = 0; j < 4; ++j)
                ptx::mma_16816_bf16(d, aw[2 * j], 0u, aw[2 * j + 1], 0u, xw[2 * j], xw[2 * j + 1]);
        }
        return make_float2(d[0], d[1]);
    };
    // this warp's K-slice `half` of x row m, raw: the lane's sixteen consecutive k of each 64-block
    auto load_x = [&](uint4 (&xr)[4][2], uint32_t m, uint32_t half) {
        #pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            xr[cc][0] = xr[cc][1] = make_uint4(0, 0, 0, 0);
            if (m < p.M && half < nsl) {
                const uint4 *src = reinterpret_cast<const uint4 *>(
                    p.x + (size_t)m * p.K + k0 + (half * 4 + cc) * kChunk + 16 * t);
                // (x that other GPUs stored into while this kernel waited is read past the L1)
                xr[cc][0] = PEERS ? __ldcg(src) : __ldg(src);
                xr[cc][1] = PEERS ? __ldcg(src + 1) : __ldg(src + 1);
            }
        }
    };

    // x becomes f16 (the MMA's operand type).  A bf16 value is an f16 value exactly as long as
    // its magnitude is inside f16's normal range, which activations usually are; a warp whose
    // slice of an activation row has its largest magnitude at 2^16 or above, or below 2^-7, first
    // divides that slice by the power of two that brings the largest magnitude to [2^14, 2^15)
    // and multiplies the row's partial sums back when it parks them (both exact).
    uint32_t xf[NT][NC][4][2];  // this warp's slices of x as f16 B-fragments
    float2 tpart[NT];           // a producer's first unit of T: this lane's part
    float col_scale[NT][2];     // factors of this lane's accumulator columns (activation rows 2t, 2t + 1)
    bool rescaled = false;      // some row of this warp's slice was divided (warp-uniform)
    const uint32_t h_first = cta % SL;
    uint4 xraw_all[NT][SL][4][2];  // every row's loads leave before the first is looked at
    #pragma unroll
    for (int u = 0; u < NT; ++u) {
        #pragma unroll
        for (int half = 0; half < SL; ++half) load_x(xraw_all[u][half], 8 * u + g, half);
    }
    #pragma unroll
    for (int u = 0; u < NT; ++u) {
        tpart[u] = make_float2(0.0f, 0.0f);
        float row_scale = 1.0f;
        #pragma unroll
        for (int half = 0; half < SL; ++half) {
            const uint4 (&xraw)[4][2] = xraw_all[u][half];
            if (producer && (uint32_t)half == h_first) tpart[u] = dot_slice(xraw);
            // the row's largest magnitude in this slice, as bf16 pairs (NaNs are left out)
            __nv_bfloat162 mx2 = __float2bfloat162_rn(0.0f);
            #pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const uint32_t w[8] = {xraw[cc][0].x, xraw[cc][0].y, xraw[cc][0].z, xraw[cc][0].w,
                                       xraw[cc][1].x, xraw[cc][1].y, xraw[cc][1].z, xraw[cc][1].w};
                #pragma unroll
                for (int i = 0; i < 8; ++i)
                    mx2 = __hmax2(mx2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
            }
            uint32_t mx = *reinterpret_cast<const uint32_t *>(&mx2);
            mx = max(mx & 0xffffu, mx >> 16);  // non-negative bf16 values order like their bit patterns
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const int ex = (int)(mx >> 7);  // biased exponent: 127 is 2^0, 255 is infinity
            const bool odd = mx != 0u && ex != 255 && (ex > 142 || ex < 120);
            if (__any_sync(0xffffffffu, odd)) {  // rare: the whole warp takes the scaling conversion
                int k = odd ? ex - 141 : 0;  // the largest magnitude goes to [2^14, 2^15)
                k = max(k, -100);
                const float down = __int_as_float((127 - k) << 23);
                row_scale = __int_as_float((127 + k) << 23);
                rescaled = true;
                #pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const uint32_t w[8] = {xraw[cc][0].x, xraw[cc][0].y, xraw[cc][0].z, xraw[cc][0].w,
                                           xraw[cc][1].x, xraw[cc][1].y, xraw[cc][1].z, xraw[cc][1].w};
                    #pragma unroll
                    for (int i = 0; i < 8; ++i)
                        xf[u][half * 4 + cc][i >> 1][i & 1] =
                            pack_f16x2(bf16_bits_to_float(w[i] & 0xffffu) * down, __uint_as_float(w[i] & 0xffff0000u) * down);
                }
            } else {
                #pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const uint32_t w[8] = {xraw[cc][0].x, xraw[cc][0].y, xraw[cc][0].z, xraw[cc][0].w,
                                           xraw[cc][1].x, xraw[cc][1].y, xraw[cc][1].z, xraw[cc][1].w};
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) xf[u][half * 4 + cc][i >> 1][i & 1] = bf16x2_to_f16x2(w[i]);
                }
            }
        }
        // the factor of activation row 8u + 2t + b sits in the lanes whose g is 2t + b
        col_scale[u][0] = __shfl_sync(0xffffffffu, row_scale, (2u * t) * 4u);
        col_scale[u][1] = __shfl_sync(0xffffffffu, row_scale, (2u * t + 1u) * 4u);
    }

    if (producer) {
        // Unit (j8, h) of T: every warp's K-slice h of sum_k x[m][k] A[j][k] for eight j; the
        // slices meet in shared memory, where the first warps add them in a fixed order (one
        // output per thread) and write the unit's columns of half h.  The first unit was
        // multiplied while x passed through the registers; a CTA that has more units (fewer CTAs
        // than units: short matrices) reads x again for them.
        constexpr uint32_t kOut = 64 * NT;  // (u, j, m) outputs of a unit
        for (uint32_t unit = cta; unit < (p.rank >> 3) * SL; unit += p.n_prod) {
            const uint32_t j8 = unit / SL, h = unit % SL;
            if (unit != cta) {
                __syncthreads();  // the slices of the unit before have been read
                load_a(unit);
                #pragma unroll
                for (int u = 0; u < NT; ++u) {
                    uint4 xraw[4][2];
                    load_x(xraw, 8 * u + g, h);
                    tpart[u] = dot_slice(xraw);
                }
            }
            #pragma unroll
            for (int u = 0; u < NT; ++u)
                *reinterpret_cast<float2 *>(red_s + warp * kOut + (u * 8 + g) * 8 + 2 * t) =
                    t_warp ? tpart[u] : make_float2(0.0f, 0.0f);
            __syncthreads();
            if (tid < kOut) {
                float v = 0.0f;
                #pragma unroll
                for (uint32_t w = 0; w < (uint32_t)kWarps; ++w) v += red_s[w * kOut + tid];
                const uint32_t m = (tid >> 6) * 8u + (tid & 7u), j = j8 * 8u + ((tid >> 3) & 7u);
                if (m < p.M) p.t_global[((size_t)(part * SL + h) * p.M + m) * p.rank + j] = v;
            }
        }
        if (tid < kOut) {
            // the writers meet (a barrier of their own), then one of them publishes
            asm volatile("bar.sync 1, %0;" ::"n"(kOut) : "memory");
            if (tid == 0) {
                __threadfence();
                atomicAdd(p.flags, 1u);
            }
        }
    }

    // Warp 0 brings T into shared memory shortly before the first pass ends.  Its lane 0 reads
    // the producers' count one tile early (the load is in flight while that tile is multiplied),
    // waits -- bounded -- only if the count is not there yet, then the warp issues asynchronous
    // copies that the end-of-pass wait collects.
    bool lost = false;   // a wait of this warp ran out: results are void, the flag is set
    uint32_t seen = 0;   // lane 0 of warp 0: the producers' count as last read
    uint32_t done_old = 0xffffffffu;  // lane 0 of warp 0: CTAs that had read T before this one
    auto peek_t = [&]() {
        if (lane == 0) seen = ld_acquire_gpu(p.flags);
    };
    auto fetch_t = [&]() {
        uint32_t ok = 1;
        if (lane == 0 && seen != p.n_prod_all) {
            const uint64_t t0 = ptx::global_timer_ns();
            while (ld_acquire_gpu(p.flags) != p.n_prod_all) {
                if (ptx::global_timer_ns() - t0 > (uint64_t)p.wait_ns) {
                    ok = 0;
                    NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 6);
                    break;
                }
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) lost = true;
        const uint32_t n = SL * p.M * p.rank;
        const float *t_part = p.t_global + (size_t)part * n;  // this part's share of T
        if ((n & 3u) == 0) {
            for (uint32_t i = lane * 4; i < n; i += 128) ptx::cp_async_16(kWin0 + C::kOffT + i * 4u, t_part + i);
        } else {
            for (uint32_t i = lane; i < n; i += 32) t_s[i] = __ldcg(t_part + i);
        }
        ptx::cp_async_commit();
    };

    const float sos = DQ ? __ldg(p.scale_of_scales) : 0.0f;
    // table entry of a code byte, relative to the table: {0, 0, byte, lane * 4}
    const uint32_t lane_word = lane * 4u;
    auto lut_at = [&](uint32_t word, int byte) -> uint32_t {
        const uint32_t addr = __byte_perm(word, lane_word, 0x7604u | ((uint32_t)byte << 4));
        uint32_t v;
        asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(kWin0));
        return v;
    };
    // byte offsets of this lane's first 8 bytes in rows 2g and 2g + 1 of a swizzled box; the
    // 32-byte block c of the row is at (offset ^ (c << 5))
    const uint32_t off_lo = (2 * g) * 128u + ((((t >> 1) ^ ((2 * g) & 7u))) << 4) + (t & 1u) * 8u;
    const uint32_t off_hi = (2 * g + 1) * 128u + ((((t >> 1) ^ ((2 * g + 1) & 7u))) << 4) + (t & 1u) * 8u;

    // double-quantized scales come straight from global memory, one tile ahead
    uint32_t dq_lo[SL], dq_hi[SL];
    #pragma unroll
    for (int sl = 0; sl < SL; ++sl) dq_lo[sl] = dq_hi[sl] = 0;
    auto fetch_dq = [&](uint32_t j) {
        if (DQ && j < my_tiles) {
            const uint32_t row = n0 + (rg + j * rw) * kTileRows + 2 * g;
            const uint32_t r_lo = min(row, p.N - 1), r_hi = min(row + 1, p.N - 1);
            #pragma unroll
            for (int sl = 0; sl < SL; ++sl) {
                if ((uint32_t)sl < nsl) {
                    dq_lo[sl] = __ldg(reinterpret_cast<const uint32_t *>(p.scale_codes + (size_t)r_lo * p.nchunks + (slice0 + sl) * 4u));
                    dq_hi[sl] = __ldg(reinterpret_cast<const uint32_t *>(p.scale_codes + (size_t)r_hi * p.nchunks + (slice0 + sl) * 4u));
                }
            }
        }
    };
    fetch_dq(0);

    uint32_t use_j = 0;  // tiles consumed so far

    #pragma unroll 1
    for (uint32_t tile0 = 0; tile0 < max_tiles; tile0 += p.pass_tiles) {  // a pass: tiles tile0 ... of every warp
        const uint32_t left = my_tiles - use_j;
        const uint32_t mine = left < p.pass_tiles ? left : p.pass_tiles;  // tiles of this warp in this pass
        const bool t_pass = tile0 == 0 && p.rank != 0 && warp == 0;  // this warp fetches T in this pass
        if (t_pass && mine < 2) peek_t();
        if (t_pass && mine == 0) fetch_t();

        #pragma unroll 1
        for (uint32_t q = 0; q < mine; ++q) {
            if (t_pass && q + 2 == mine) peek_t();
            if (t_pass && q + 1 == mine) fetch_t();
            const uint32_t slot = use_j & (kRing - 1);
            if (!lost && !wait_phase(bar0 + 8 * slot, (use_j / kRing) & 1u, p.wait_ns)) {
                lost = true;
                if (lane == 0) NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 5);
            }
            float acc[NT][4];
            #pragma unroll
            for (int u = 0; u < NT; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;
            #pragma unroll
            for (int sl = 0; sl < SL; ++sl) {
                if ((uint32_t)sl < nsl) {
                    const uint8_t *cs = codes_ring + slot * C::kCodesTile + sl * kCodesSlot;
                    uint2 w0[kSliceChunks], w1[kSliceChunks];
                    #pragma unroll
                    for (int c = 0; c < kSliceChunks; ++c) {
                        w0[c] = *reinterpret_cast<const uint2 *>(cs + (off_lo ^ ((uint32_t)c << 5)));
                        w1[c] = *reinterpret_cast<const uint2 *>(cs + (off_hi ^ ((uint32_t)c << 5)));
                    }
                    float s_lo[kSliceChunks], s_hi[kSliceChunks];
                    if (DQ) {
                        #pragma unroll
                        for (int c = 0; c < kSliceChunks; ++c) {
                            s_lo[c] = __fmul_rn(dq_s[(dq_lo[sl] >> (8 * c)) & 0xffu], sos);
                            s_hi[c] = __fmul_rn(dq_s[(dq_hi[sl] >> (8 * c)) & 0xffu], sos);
                        }
                    } else {
                        const uint8_t *ss = scales_ring + slot * C::kScaleTile + sl * kScaleSlot + g * 32u;
                        const float4 a = *reinterpret_cast<const float4 *>(ss);
                        const float4 b = *reinterpret_cast<const float4 *>(ss + 16u);
                        s_lo[0] = a.x; s_lo[1] = a.y; s_lo[2] = a.z; s_lo[3] = a.w;
                        s_hi[0] = b.x; s_hi[1] = b.y; s_hi[2] = b.z; s_hi[3] = b.w;
                    }
                    if (sl + 1 == SL || (uint32_t)sl + 1 == nsl) {
                        // every lane holds the last of the tile in registers: refill the slot
                        ++use_j;
                        fetch_dq(use_j);
                        __syncwarp();
                        if (req_j < my_tiles) {
                            if (lane < nsl) request(req_j, lane);
                            ++req_j;
                        }
                    }

                    #pragma unroll
                    for (int c = 0; c < kSliceChunks; ++c) {
                        float blk[NT][4];
                        #pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t x0 = (j < 2) ? w0[c].x : w0[c].y;
                            const uint32_t x1 = (j < 2) ? w1[c].x : w1[c].y;
                            const int b = 2 * (j & 1);
                            const uint32_t a0 = lut_at(x0, b), a1 = lut_at(x1, b);
                            const uint32_t a2 = lut_at(x0, b + 1), a3 = lut_at(x1, b + 1);
                            #pragma unroll
                            for (int u = 0; u < NT; ++u) {
                                const uint32_t b0 = xf[u][sl * kSliceChunks + c][j][0];
                                const uint32_t b1 = xf[u][sl * kSliceChunks + c][j][1];
                                if (j == 0) ptx::mma_16816_f16_zero(blk[u], a0, a1, a2, a3, b0, b1);
                                else ptx::mma_16816_f16(blk[u], a0, a1, a2, a3, b0, b1);
                            }
                        }
                        #pragma unroll
                        for (int u = 0; u < NT; ++u) {
                            #pragma unroll
                            for (int r = 0; r < 4; ++r)
                                acc[u][r] = fmaf(blk[u][r], r < 2 ? s_lo[c] : s_hi[c], acc[u][r]);
                        }
                    }
                }
            }
            if (rescaled) {
                #pragma unroll
                for (int u = 0; u < NT; ++u) {
                    #pragma unroll
                    for (int r = 0; r < 4; ++r) acc[u][r] *= col_scale[u][r & 1];
                }
            }
            // park the tile's partial sums: slot q * NT + u of this warp, one float4 per lane
            #pragma unroll
            for (int u = 0; u < NT; ++u)
                *reinterpret_cast<float4 *>(park_s + warp * kParkWarp + (q * NT + u) * 128u + lane * 4u) =
                    make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
        }

        // ================= end of a pass: reduce, finish and store its rows =================
        ptx::cp_async_wait<0>();  // this thread's pieces of the pass's LoRA-B rows (and of T)
        // T has left global memory: count this CTA out (the count comes back while the pass is
        // finished; it is looked at when the kernel ends)
        if (t_pass && lane == 0) done_old = atomicAdd(p.flags + 1, 1u);
        __syncthreads();

        // ---- a warp per (tile, eight activation rows): sum the K-warps' partials in a fixed
        // order, add the adapter term (one bf16 MMA pair per sixteen ranks: B rows x T, T split
        // into bf16 high and low parts so that its f32 value survives), bias, convert, store ----
        const uint32_t pass_tile0 = tile0 << p.rw_shift;
        const uint32_t tiles_in_pass = min(ntiles - pass_tile0, p.pass_tiles << p.rw_shift);
        const uint32_t pass_row0 = n0 + pass_tile0 * kTileRows;
        const uint32_t pass_rows = min(n1 - pass_row0, tiles_in_pass * (uint32_t)kTileRows);
        #pragma unroll 1
        for (uint32_t job = warp; job < tiles_in_pass * NT; job += kWarps) {
            const uint32_t ti = job / NT, u = job - ti * NT;
            const uint32_t trg = ti & (rw - 1), q = ti >> p.rw_shift;  // the warps that hold this tile, and where
            // four K-warps at a time (a fixed order of additions: results do not depend on timing)
            const float *src = park_s + (trg * p.kwarps) * kParkWarp + (q * NT + u) * 128u + lane * 4u;
            auto ld4 = [&](uint32_t w) -> float4 {
                return w < p.kwarps ? *reinterpret_cast<const float4 *>(src + w * kParkWarp)
                                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            };
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            #pragma unroll
            for (int w4 = 0; w4 < kWarps; w4 += 4) {
                const float4 pa = ld4(w4), pb = ld4(w4 + 1), pc = ld4(w4 + 2), pd = ld4(w4 + 3);
                v[0] += (pa.x + pb.x) + (pc.x + pd.x);
                v[1] += (pa.y + pb.y) + (pc.y + pd.y);
                v[2] += (pa.z + pb.z) + (pc.z + pd.z);
                v[3] += (pa.w + pb.w) + (pc.w + pd.w);
            }
            // this lane's outputs: rows 2g, 2g+1 of the tile, activation rows m0, m0 + 1
            const uint32_t row_a = ti * kTileRows + 2u * g, m0 = u * 8u + 2u * t;
            if (p.rank) {
                float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const __nv_bfloat16 *lb0 = reinterpret_cast<const __nv_bfloat16 *>(lora_s + (size_t)row_a * 256u);
                const __nv_bfloat16 *lb1 = reinterpret_cast<const __nv_bfloat16 *>(lora_s + (size_t)(row_a + 1) * 256u);
                const float *tm = t_s + (u * 8u + g) * p.rank;  // B operand: column m = 8u + g of T^T
                const bool m_ok = u * 8u + g < p.M;
                #pragma unroll 1
                for (uint32_t k16 = 0; k16 < p.rank; k16 += 16) {
                    const uint32_t ka = k16 + 2u * t, kb = ka + 8u;
                    const bool oka = ka < p.rank, okb = kb < p.rank;
                    const uint32_t a0 = oka ? *reinterpret_cast<const uint32_t *>(lb0 + ka) : 0u;
                    const uint32_t a1 = oka ? *reinterpret_cast<const uint32_t *>(lb1 + ka) : 0u;
                    const uint32_t a2 = okb ? *reinterpret_cast<const uint32_t *>(lb0 + kb) : 0u;
                    const uint32_t a3 = okb ? *reinterpret_cast<const uint32_t *>(lb1 + kb) : 0u;
                    const float2 ta = (oka && m_ok) ? *reinterpret_cast<const float2 *>(tm + ka) : make_float2(0.0f, 0.0f);
                    const float2 tb = (okb && m_ok) ? *reinterpret_cast<const float2 *>(tm + kb) : make_float2(0.0f, 0.0f);
                    const __nv_bfloat162 ha = __floats2bfloat162_rn(ta.x, ta.y), hb = __floats2bfloat162_rn(tb.x, tb.y);
                    const __nv_bfloat162 la = __floats2bfloat162_rn(ta.x - __low2float(ha), ta.y - __high2float(ha));
                    const __nv_bfloat162 lb = __floats2bfloat162_rn(tb.x - __low2float(hb), tb.y - __high2float(hb));
                    ptx::mma_16816_bf16(d, a0, a1, a2, a3, *reinterpret_cast<const uint32_t *>(&ha),
                                        *reinterpret_cast<const uint32_t *>(&hb));
                    ptx::mma_16816_bf16(d, a0, a1, a2, a3, *reinterpret_cast<const uint32_t *>(&la),
                                        *reinterpret_cast<const uint32_t *>(&lb));
                }
                #pragma unroll
                for (int r = 0; r < 4; ++r) v[r] = fmaf(d[r], p.lora_scale, v[r]);  // scale applied last
            }
            // v[0], v[2]: rows 2g and 2g + 1 for activation row m0 (neighbours in y); v[1], v[3]: for m0 + 1
            const uint32_t col = pass_row0 + row_a;
            const bool two = row_a + 1 < pass_rows;
            const bool pair = p.y_pair && two && (col & 1u) == 0;  // one 32-bit store for the two rows
            #pragma unroll
            for (int b = 0; b < 2; ++b) {
                if (row_a >= pass_rows || m0 + b >= p.M) continue;
                float o0 = v[b], o1 = v[b + 2];
                if (SPLIT) {  // this part's share of the sums; bias and conversion come later
                    float *dst = p.partial + ((size_t)part * p.M + m0 + b) * p.N + col;
                    dst[0] = o0;
                    if (two) dst[1] = o1;
                    continue;
                }
                if (p.bias) {
                    o0 += __ldg(p.bias + col);
                    if (two) o1 += __ldg(p.bias + col + 1);
                }
                const size_t at = (size_t)(m0 + b) * p.ldy + col;
                const uint32_t n_dest = PEERS ? p.n_dest : 1u;
                for (uint32_t d = 0; d < n_dest; ++d) {  // (the same values to every rank's output)
                    void *yb = PEERS ? p.dest[d] : p.y;
                    if (p.y_f32) {
                        static_cast<float *>(yb)[at] = o0;
                        if (two) static_cast<float *>(yb)[at + 1] = o1;
                    } else if (pair) {
                        *reinterpret_cast<__nv_bfloat162 *>(static_cast<__nv_bfloat16 *>(yb) + at) = __floats2bfloat162_rn(o0, o1);
                    } else {
                        static_cast<__nv_bfloat16 *>(yb)[at] = __float2bfloat16_rn(o0);
                        if (two) static_cast<__nv_bfloat16 *>(yb)[at + 1] = __float2bfloat16_rn(o1);
                    }
                }
            }
        }
        if (tile0 + p.pass_tiles < max_tiles) {
            __syncthreads();  // the pass's LoRA-B rows and parked sums have been read
            stage_lora_b(tile0 + p.pass_tiles);
        }
    }
    ptx::cp_async_wait<0>();
    if (SPLIT) {
        // The parts of K meet: the CTA that arrives last for these rows adds the parts' sums in
        // the order of the parts (the result does not depend on who was last), adds the bias,
        // converts and writes y, and leaves the counter at zero.
        uint32_t *last_s = reinterpret_cast<uint32_t *>(red_s);
        __syncthreads();  // every partial sum of this CTA has been stored
        if (tid == 0) {
            __threadfence();
            const uint32_t sh = (cta & 3u) * 8u;
            uint32_t *counter = p.flags + 2 + (cta >> 2);
            const uint32_t old = (atomicAdd(counter, 1u << sh) >> sh) & 0xffu;
            if (old == p.kparts - 1) atomicSub(counter, p.kparts << sh);
            *last_s = old == p.kparts - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (*last_s) {
            __threadfence();
            const uint32_t rows = n1 - n0;
            for (uint32_t e = tid; e < rows * p.M; e += kThreads) {
                const uint32_t m = e / rows, col = n0 + (e - m * rows);
                float o = 0.0f;
                for (uint32_t q = 0; q < p.kparts; ++q) o += __ldcg(p.partial + ((size_t)q * p.M + m) * p.N + col);
                if (p.bias) o += __ldg(p.bias + col);
                const size_t at = (size_t)m * p.ldy + col;
                const uint32_t n_dest = PEERS ? p.n_dest : 1u;
                for (uint32_t d = 0; d < n_dest; ++d) {
                    void *yb = PEERS ? p.dest[d] : p.y;
                    if (p.y_f32) static_cast<float *>(yb)[at] = o;
                    else static_cast<__nv_bfloat16 *>(yb)[at] = __float2bfloat16_rn(o);
                }
            }
        }
    }
    if (PEERS && (p.signal || p.wait_on)) {
        // Every store of this CTA has been issued.  The CTAs count themselves out on a word of the
        // workspace; the last one takes the arrivals this launch waited for off this rank's
        // counter and, if the launch signals, makes the launch's stores visible to the other GPUs
        // (its fence follows the others' through the counter) and adds one to every rank's
        // arrival counter.  Launches without a signal rely on a later launch of the stream for it.
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            if (atomicAdd(p.flags + 63, 1u) == nctas - 1) {
                p.flags[63] = 0;
                if (p.wait_on) atomicSub(p.wait_on, p.wait_expected);
                if (p.signal) {
                    __threadfence_system();
                    for (uint32_t d = 0; d < p.n_dest; ++d) atomicAdd_system(p.arrive[d], 1u);
                }
            }
        }
    }
    if (done_old == nctas - 1) {
        // The last CTA to have read T re-arms the two flag words for the next launch: every other
        // CTA read the first before it counted itself in on the second, and the next launch
        // looks at them only after this one has completed, so no order is needed between them.
        *reinterpret_cast<uint2 *>(p.flags) = make_uint2(0u, 0u);
    }
}

template <int NT, bool DQ, bool SPLIT, bool PEERS>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_codes,
              const __grid_constant__ CUtensorMap tm_scales, const __grid_constant__ DecodeParams p) {
    decode_body<NT, DQ, SPLIT, PEERS>(&tm_codes, &tm_scales, p, blockIdx.x, gridDim.x);
}

// Waits (bounded) until `expected` CTAs of the ranks of a sharded layer have counted themselves in
// on this rank's arrival counter, then takes them off the counter: the kernels behind it in the
// stream find every rank's columns in this rank's output.
__global__ void peer_wait_kernel(uint32_t *counter, uint32_t expected, uint32_t limit_ns) {
    const uint64_t t0 = ptx::global_timer_ns();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= expected) break;
        if (ptx::global_timer_ns() - t0 > (uint64_t)limit_ns) {
            NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 7);
            return;
        }
        __nanosleep(100);
    }
    atomicSub(counter, expected);
}

// Several forwards of the same activations (projections that share their input) in one launch:
// forward i is multiplied by the CTAs cta0[i] ... cta0[i + 1] - 1, exactly as a launch of its own
// with that many CTAs would do it.
constexpr int kMaxGroup = 4;
struct GroupParams {
    CUtensorMap tm_codes[kMaxGroup];
    CUtensorMap tm_scales[kMaxGroup];
    DecodeParams p[kMaxGroup];
    uint32_t cta0[kMaxGroup + 1];
    uint32_t count;
};

template <int NT, bool DQ>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
decode_group_kernel(const __grid_constant__ GroupParams gp) {
    uint32_t i = 0;
    while (i + 1 < gp.count && blockIdx.x >= gp.cta0[i + 1]) ++i;
    decode_body<NT, DQ, false>(&gp.tm_codes[i], &gp.tm_scales[i], gp.p[i], blockIdx.x - gp.cta0[i],
                               gp.cta0[i + 1] - gp.cta0[i]);
}

// T[m][j] = sum_k x[m][k] * A[j][k]  (x, A bf16; f32 accumulate).  One 128-thread CTA per (j, m).
// Used for adapter ranks the decode kernel does not multiply itself.
__global__ void __launch_bounds__(128, 16)
lora_t_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a, uint32_t K,
              uint32_t rank, float *__restrict__ t_out) {
    const uint32_t j = blockIdx.x, m = blockIdx.y;
    const __nv_bfloat16 *xr = x + (size_t)m * K, *ar = a + (size_t)j * K;
    float acc = 0.0f;
    if ((K & 7u) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a)) & 15u) == 0) {
        const uint4 *x4 = reinterpret_cast<const uint4 *>(xr), *a4 = reinterpret_cast<const uint4 *>(ar);
        for (uint32_t i = threadIdx.x; i < K / 8; i += 128) {
            const uint4 xv = __ldg(x4 + i), av = __ldg(a4 + i);
            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, as[4] = {av.x, av.y, av.z, av.w};
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc = fmaf(bf16_bits_to_float(xs[q] & 0xffffu), bf16_bits_to_float(as[q] & 0xffffu), acc);
                acc = fmaf(bf16_bits_to_float(xs[q] >> 16), bf16_bits_to_float(as[q] >> 16), acc);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += 128)
            acc = fmaf(__bfloat162float(xr[i]), __bfloat162float(ar[i]), acc);
    }
    __shared__ float part[4];
    #pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) t_out[(size_t)m * rank + j] = (part[0] + part[1]) + (part[2] + part[3]);
}

uint32_t gcd_u32(uint32_t a, uint32_t b) {
    while (b) {
        uint32_t t = a % b;
        a = b;
        b = t;
    }
    return a;
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
    DecodeParams p;
    uint32_t grid;
};

// Fills the shape-dependent fields; false when the shape does not fit.
bool plan_shape(uint32_t M, uint32_t K, uint32_t N, uint32_t rank, uint32_t gran, Plan &pl,
                uint32_t max_ctas) {
    using C = Cfg;
    DecodeParams &p = pl.p;
    const uint32_t nt = M > 8 ? 2u : 1u;
    p.kw = K / kSliceK;
    p.kparts = (p.kw + kMaxSlices - 1) / kMaxSlices;
    p.part_slices = (p.kw + p.kparts - 1) / p.kparts;
    p.kwarps = (p.part_slices + C::kSlices - 1) / C::kSlices;
    p.rw_shift = 0;
    while ((p.kwarps << (p.rw_shift + 1)) <= (uint32_t)C::kWarps) ++p.rw_shift;
    const uint32_t rw = 1u << p.rw_shift;
    for (uint32_t w = 0; w < (uint32_t)C::kWarps; ++w) {
        const bool active = w < p.kwarps * rw;
        p.warp_rg[w] = active ? (uint8_t)(w / p.kwarps) : 0xffu;
        p.warp_kpos[w] = active ? (uint8_t)(w % p.kwarps) : 0u;
    }
    // Row ranges are whole tiles where the matrix allows it (a CTA multiplies a partial tile at
    // the cost of a whole one).  The CTAs that get one unit less are the producers of T, which
    // have that work on top, and then the last ones, which tend to start last.
    if (N % kTileRows == 0 && kTileRows % gran == 0) gran = kTileRows;
    p.gran = gran;
    const uint64_t units = N / gran;
    const uint64_t tiles = ((uint64_t)N + kTileRows - 1) / kTileRows;
    const uint64_t per_part = (uint64_t)max_ctas / p.kparts;
    if (per_part == 0) return false;
    uint64_t ctas = tiles < per_part ? tiles : per_part;
    if (ctas > units) ctas = units;
    p.cpp = (uint32_t)ctas;
    pl.grid = (uint32_t)ctas * p.kparts;
    p.rows_base = (uint32_t)(units / ctas) * gran;
    p.rows_extra = (uint32_t)(units % ctas);
    // tiles per warp between two reductions: what the parking area and (with an adapter) the
    // table's gaps hold
    uint32_t pt = kParkSlots / nt;
    if (rank) {
        const uint32_t by_rows = kGapRows / (rw * kTileRows);
        if (by_rows == 0) return false;
        if (pt > by_rows) pt = by_rows;
        p.piece_shift = rank == 8 ? 0u : rank == 16 ? 1u : rank == 32 ? 2u : 3u;
    }
    p.pass_tiles = pt;
    const uint32_t t_units = (rank >> 3) * C::kSlices;
    p.n_prod = t_units < p.cpp ? t_units : p.cpp;
    p.n_prod_all = p.n_prod * p.kparts;
    const uint32_t light = p.cpp - p.rows_extra;
    p.light_front = rank ? (p.n_prod < light ? p.n_prod : light) : 0u;
    return true;
}

bool plan(const nf4_linear_args &a, Plan &pl, uint32_t max_ctas = 0) {
    if (max_ctas == 0) max_ctas = persistent_ctas();  // one CTA per SM, less what the host keeps free
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_BF16) return false;
    if (a.rows == 0 || a.rows > 16) return false;
    // whole slices of four blocks: the scale rows then have a 16-byte pitch, which TMA needs
    if (a.d_in % kSliceK != 0 || a.d_in > (uint64_t)kMaxParts * kMaxSlices * kSliceK) return false;
    if (a.d_out >= (1ull << 31)) return false;
    const bool dq = a.scale_codes != nullptr;
    const uint32_t rank = a.lora_a ? a.lora_rank : 0;
    // LoRA-B rows move in a power-of-two number of 16-byte pieces
    if (rank != 0 && rank != 8 && rank != 16 && rank != 32 && rank != 64) return false;
    const void *scales = dq ? (const void *)a.scale_codes : (const void *)a.absmax;
    if (!aligned16(a.x) || !aligned16(a.packed) || !aligned16(scales)) return false;
    if (rank && (!aligned16(a.lora_a) || !aligned16(a.lora_b))) return false;
    if (reinterpret_cast<uintptr_t>(a.y) & (a.y_f32 ? 3u : 1u)) return false;

    const uint32_t K = (uint32_t)a.d_in, N = (uint32_t)a.d_out, M = (uint32_t)a.rows;
    DecodeParams &p = pl.p;
    p = DecodeParams{};
    // CTA row ranges start where the CTA's LoRA-B rows are 16-byte aligned
    const uint32_t gran = rank ? 16u / gcd_u32(16u, rank * 2u) : 1u;
    if (N % gran != 0) return false;
    p.nchunks = K / kChunk;
    if (!plan_shape(M, K, N, rank, gran, pl, max_ctas)) return false;
    p.wait_ns = 1000000000u;
    p.x = static_cast<const __nv_bfloat16 *>(a.x);
    p.scale_codes = a.scale_codes;
    p.scale_of_scales = a.scale_of_scales;
    p.bias = a.bias;
    p.lora_a = static_cast<const __nv_bfloat16 *>(a.lora_a);
    p.lora_b = static_cast<const __nv_bfloat16 *>(a.lora_b);
    p.y = a.y;
    p.y_f32 = (uint32_t)a.y_f32;
    p.ldy = a.ldy ? a.ldy : a.d_out;
    p.y_pair = (!a.y_f32 && (reinterpret_cast<uintptr_t>(a.y) & 3u) == 0 && (p.ldy & 1u) == 0) ? 1u : 0u;
    p.M = M;
    p.K = K;
    p.N = N;
    p.rank = rank;
    p.lora_scale = a.lora_scale;
    return true;
}

template <int NT, bool DQ, bool SPLIT, bool PEERS>
int32_t launch_as(const CUtensorMap &mc, const CUtensorMap &ms, const Plan &pl, cudaStream_t stream) {
    using C = Cfg;
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(decode_kernel<NT, DQ, SPLIT, PEERS>), (int)C::kSmemBytes));
    count_launch();
    return launch_maybe_overlapped(decode_kernel<NT, DQ, SPLIT, PEERS>, dim3(pl.grid), dim3(C::kThreads),
                                   C::kSmemBytes, stream, true, mc, ms, pl.p);
}

template <int NT, bool DQ>
int32_t launch(const CUtensorMap &mc, const CUtensorMap &ms, const Plan &pl, cudaStream_t stream) {
    if (pl.p.n_dest)
        return pl.p.kparts > 1 ? launch_as<NT, DQ, true, true>(mc, ms, pl, stream)
                               : launch_as<NT, DQ, false, true>(mc, ms, pl, stream);
    return pl.p.kparts > 1 ? launch_as<NT, DQ, true, false>(mc, ms, pl, stream)
                           : launch_as<NT, DQ, false, false>(mc, ms, pl, stream);
}

// bytes of T in the workspace: a share per part of K (room for two where K is not split)
uint64_t t_bytes(uint64_t rows, uint32_t rank, uint32_t kparts) {
    return ((kparts > 2 ? kparts : 2u) * rows * rank * 4 + 255) / 256 * 256;
}

// `scratch`: kFlagBytes of flag words and counters (zero at first use, left zero), room for T,
// and, where K is split, for the parts' sums
int32_t prepare(const nf4_linear_args &a, Plan &pl, void *scratch, CUtensorMap &mc, CUtensorMap &ms) {
    DecodeParams &p = pl.p;
    const bool dq = a.scale_codes != nullptr;
    if (p.rank || p.kparts > 1 || p.signal || p.wait_on) {
        if (!scratch) return fail(NF4_ERR_INVALID_ARG, "decode_forward: this shape needs the workspace");
        p.flags = static_cast<uint32_t *>(scratch);
        p.t_global = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + kFlagBytes);
        p.partial = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + kFlagBytes + t_bytes(p.M, p.rank, p.kparts));
    }
    NF4_TRY(make_map(&mc, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.packed, p.N, p.K / 2, p.K / 2, kTileRows, 128,
                     CU_TENSOR_MAP_SWIZZLE_128B));
    if (dq) ms = mc;  // not used by the kernel
    else
        NF4_TRY(make_map(&ms, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.absmax, p.N, p.nchunks,
                         (uint64_t)p.nchunks * 4, kTileRows, 4, CU_TENSOR_MAP_SWIZZLE_NONE));
    return NF4_OK;
}

int32_t run(const nf4_linear_args &a, Plan &pl, void *scratch, cudaStream_t stream) {
    CUtensorMap mc, ms;
    NF4_TRY(prepare(a, pl, scratch, mc, ms));
    const DecodeParams &p = pl.p;
    const bool dq = a.scale_codes != nullptr;
    if (p.M <= 8) return dq ? launch<1, true>(mc, ms, pl, stream) : launch<1, false>(mc, ms, pl, stream);
    return dq ? launch<2, true>(mc, ms, pl, stream) : launch<2, false>(mc, ms, pl, stream);
}

}  // namespace

bool decode_supported(const nf4_linear_args &a) {
    Plan pl;
    return plan(a, pl);
}

uint64_t decode_workspace_bytes(uint64_t rows, uint64_t d_in, uint64_t d_out, uint32_t lora_rank) {
    if (rows == 0 || rows > 16) return 0;
    const uint64_t kw = d_in / kSliceK;
    const uint32_t kparts = (uint32_t)((kw + kMaxSlices - 1) / kMaxSlices);
    const bool split = d_in % kSliceK == 0 && kparts > 1 && kparts <= (uint32_t)kMaxParts;
    if (lora_rank == 0 && !split) return 0;
    uint64_t need = kFlagBytes + t_bytes(rows, lora_rank, split ? kparts : 1u);
    if (split) need += (uint64_t)kparts * rows * d_out * 4;  // the parts' sums
    return need;
}

// `chained` launches the pre-pass as a programmatic dependent of the kernel ahead of it; the
// kernel does not wait by itself, so callers pass false unless that kernel never writes x.
int32_t lora_t_small(const void *x, const void *a, uint32_t rows, uint32_t K, uint32_t rank,
                     float *t_out, cudaStream_t stream, bool chained) {
    count_launch();
    return launch_maybe_overlapped(lora_t_kernel, dim3(rank, rows), dim3(128), 0, stream, chained,
                                   static_cast<const __nv_bfloat16 *>(x),
                                   static_cast<const __nv_bfloat16 *>(a), K, rank, t_out);
}

template <int NT, bool DQ>
int32_t launch_group(const GroupParams &gp, cudaStream_t stream) {
    using C = Cfg;
    NF4_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(decode_group_kernel<NT, DQ>), (int)C::kSmemBytes));
    count_launch();
    return launch_maybe_overlapped(decode_group_kernel<NT, DQ>, dim3(gp.cta0[gp.count]), dim3(C::kThreads),
                                   C::kSmemBytes, stream, true, gp);
}

// Forwards that share x, rows, d_in and the scale form, as one launch; false (nothing launched,
// no error) when they do not fit together and the caller should launch them one by one.
int32_t decode_forward_grouped(const nf4_linear_args *a, uint32_t count, cudaStream_t stream, bool *taken) {
    *taken = false;
    if (count < 2 || count > (uint32_t)kMaxGroup) return NF4_OK;
    uint64_t tiles[kMaxGroup], all = 0;
    for (uint32_t i = 0; i < count; ++i) {
        if (a[i].x != a[0].x || a[i].rows != a[0].rows || a[i].d_in != a[0].d_in ||
            (a[i].scale_codes != nullptr) != (a[0].scale_codes != nullptr))
            return NF4_OK;
        if (a[i].d_in > (uint64_t)kMaxSlices * kSliceK) return NF4_OK;  // K shared out between CTAs: on its own
        tiles[i] = (a[i].d_out + kTileRows - 1) / kTileRows;
        all += tiles[i];
    }
    if (all == 0) return NF4_OK;
    // CTAs in proportion to the tiles, one at least
    const uint32_t n_sms = persistent_ctas();
    uint32_t ctas[kMaxGroup], sum = 0;
    for (uint32_t i = 0; i < count; ++i) {
        ctas[i] = (uint32_t)(tiles[i] * n_sms / all);
        if (ctas[i] == 0) ctas[i] = 1;
        sum += ctas[i];
    }
    while (sum > n_sms) {  // (only if several forwards were rounded up to one CTA)
        uint32_t big = 0;
        for (uint32_t i = 1; i < count; ++i) if (ctas[i] > ctas[big]) big = i;
        --ctas[big];
        --sum;
    }
    while (sum < n_sms) {  // the CTAs left over go where a CTA has the most tiles
        uint32_t worst = 0;
        for (uint32_t j = 1; j < count; ++j)
            if (tiles[j] * ctas[worst] > tiles[worst] * ctas[j]) worst = j;
        if (ctas[worst] >= tiles[worst]) break;
        ++ctas[worst];
        ++sum;
    }
    static thread_local GroupParams gp;
    gp.count = count;
    gp.cta0[0] = 0;
    for (uint32_t i = 0; i < count; ++i) {
        Plan pl;
        if (!plan(a[i], pl, ctas[i])) return NF4_OK;
        NF4_TRY(prepare(a[i], pl, a[i].workspace, gp.tm_codes[i], gp.tm_scales[i]));
        gp.p[i] = pl.p;
        gp.cta0[i + 1] = gp.cta0[i] + pl.grid;
    }
    *taken = true;
    const bool dq = a[0].scale_codes != nullptr;
    if (a[0].rows <= 8) return dq ? launch_group<1, true>(gp, stream) : launch_group<1, false>(gp, stream);
    return dq ? launch_group<2, true>(gp, stream) : launch_group<2, false>(gp, stream);
}

// The forward of one rank's column shard, stored into every rank's output.  `dest`: the outputs
// [rows, ldy] as mapped here, `arrive`: the ranks' arrival counters.
int32_t decode_forward_scatter(const nf4_linear_args &a, void *const *dest, uint32_t *const *arrive, uint32_t world,
                               uint32_t rank, uint64_t ldy, bool signal, uint32_t *wait_on, uint32_t wait_expected,
                               cudaStream_t stream) {
    Plan pl;
    if (world == 0 || world > 8 || rank >= world || !plan(a, pl))
        return fail(NF4_ERR_UNSUPPORTED, "decode_forward_scatter: decode shapes and up to eight ranks only");
    DecodeParams &p = pl.p;
    const size_t eb = a.y_f32 ? 4 : 2;
    p.ldy = ldy;
    p.n_dest = world;
    p.y_pair = (!a.y_f32 && (ldy & 1u) == 0 && ((rank * a.d_out) & 1u) == 0) ? 1u : 0u;
    for (uint32_t d = 0; d < world; ++d) {
        if (!dest[d] || !arrive[d]) return fail(NF4_ERR_INVALID_ARG, "decode_forward_scatter: null output or counter of rank %u", d);
        p.dest[d] = static_cast<uint8_t *>(dest[d]) + (size_t)rank * a.d_out * eb;
        p.arrive[d] = arrive[d];
        if (reinterpret_cast<uintptr_t>(p.dest[d]) & 3u) p.y_pair = 0;
    }
    p.signal = signal ? 1u : 0u;
    p.wait_on = wait_on;
    p.wait_expected = wait_expected;
    if ((signal || wait_on) && !a.workspace)
        return fail(NF4_ERR_INVALID_ARG, "decode_forward_scatter: signalling and waiting need the workspace (256 bytes at least)");
    return run(a, pl, a.workspace, stream);
}

int32_t decode_peer_wait(uint32_t *counter, uint32_t expected, uint32_t limit_ns, cudaStream_t stream) {
    peer_wait_kernel<<<1, 1, 0, stream>>>(counter, expected, limit_ns);
    count_launch();
    return check_cuda(cudaGetLastError(), "peer_wait_kernel launch");
}

// The row ranges and parts of K as the kernel will see them, for inspection on the host: for CTA
// `cta`, the part of K it multiplies ([k0, k1)) and its rows ([n0, n1)), by the kernel's own
// formulas.  Returns the number of CTAs, or -1 when the shape is not the kernel's.
int32_t decode_share_plan(uint32_t rows, uint32_t d_in, uint32_t d_out, uint32_t rank, uint32_t cta, uint32_t *out4) {
    if (rows == 0 || rows > 16 || d_in % kSliceK != 0 || d_in > (uint32_t)kMaxParts * kMaxSlices * kSliceK) return -1;
    if (rank != 0 && rank != 8 && rank != 16 && rank != 32 && rank != 64) return -1;
    Plan pl;
    pl.p = DecodeParams{};
    if (!plan_shape(rows, d_in, d_out, rank, 1, pl, persistent_ctas())) return -1;
    const DecodeParams &p = pl.p;
    if (cta >= pl.grid) return -1;
    const uint32_t part = p.kparts > 1 ? cta / p.cpp : 0u, c = cta - part * p.cpp;
    const uint32_t s0 = part * p.part_slices, s1 = p.kw < s0 + p.part_slices ? p.kw : s0 + p.part_slices;
    const uint32_t past = c > p.light_front ? c - p.light_front : 0u;
    const uint32_t n0 = c * p.rows_base + (past < p.rows_extra ? past : p.rows_extra) * p.gran;
    const uint32_t n1 = n0 + p.rows_base + (c >= p.light_front && past < p.rows_extra ? p.gran : 0u);
    out4[0] = s0 * kSliceK;
    out4[1] = s1 * kSliceK;
    out4[2] = n0;
    out4[3] = n1;
    return (int32_t)pl.grid;
}

int32_t decode_forward(const nf4_linear_args &a, cudaStream_t stream) {
    Plan pl;
    if (!plan(a, pl)) return fail(NF4_ERR_UNSUPPORTED, "decode_forward: unsupported shape");
    return run(a, pl, a.workspace, stream);
}

// ---- decode forward whose scratch is a fixed device array (no allocation anywhere) ----
// The adapter intermediate T = x A^T ([rows][rank] f32) and the two flag words its producers
// and readers meet on are the only scratch the decode path needs.  Here they live in a
// file-scope device array instead of a caller buffer.
constexpr uint32_t kStaticTBytes = 16 * kMaxRank * sizeof(float);  // 16 rows x rank 64
constexpr uint32_t kStaticScratchBytes = kFlagBytes + kStaticTBytes;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

uint64_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

int32_t decode_forward_static_scratch(const nf4_linear_args &a, cudaStream_t stream) {
    const uint64_t need = a.rows * (uint64_t)(a.lora_a ? a.lora_rank : 0) * sizeof(float);
    if (need > kStaticTBytes)
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_linear_forward_noalloc_dev: rows * rank * 4 = %llu bytes exceeds the %u bytes "
                    "the fixed scratch has for it", (unsigned long long)need, kStaticTBytes);
    Plan pl;
    if (!plan(a, pl) || pl.p.kparts > 1)
        return fail(NF4_ERR_UNSUPPORTED,
                    "nf4_linear_forward_noalloc_dev: only the decode shapes are served (rows <= 16, "
                    "bf16, W [d_out, d_in], d_in %% 256 == 0 and <= 4096, rank <= 64)");
    // In host code the array's name is only a handle: the device address has to be asked for,
    // once per device, with that device current.
    static std::mutex mu;
    static void *scratch_of_device[64] = {};
    int dev = 0;
    NF4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NF4_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_of_device[dev]) {
            void *ptr = nullptr;
            NF4_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
            scratch_of_device[dev] = ptr;
        }
        scratch = scratch_of_device[dev];
    }
    // The array starts zeroed (static storage) and every call leaves the flag words zero; T is
    // rewritten by each call before it is read: nothing to clear here.
    return run(a, pl, scratch, stream);
}

// A wait that nothing satisfies, with the caller's limit: exercises the bounded wait and the
// failure flag exactly as the decode kernel uses them, without hanging or trapping anything.
__global__ void selftest_wait_kernel(uint32_t limit_ns, unsigned long long *waited_ns) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = ptx::smem_addr(&bar);
    ptx::mbar_init(b, 1);
    ptx::fence_mbar_init();
    const uint64_t t0 = ptx::global_timer_ns();
    const bool ok = wait_phase(b, 0, limit_ns);  // phase 0 never completes: nobody arrives
    *waited_ns = ptx::global_timer_ns() - t0;
    if (!ok) NF4_REPORT_FAILURE(g_decode_error, g_decode_error_host, 5);
}

int32_t decode_selftest_wait(uint32_t limit_ns, unsigned long long *waited_ns_dev, cudaStream_t stream) {
    selftest_wait_kernel<<<1, 1, 0, stream>>>(limit_ns, waited_ns_dev);
    count_launch();
    return check_cuda(cudaGetLastError(), "selftest_wait_kernel launch");
}

int32_t decode_set_host_flag(int *mapped) {
    return check_cuda(cudaMemcpyToSymbol(g_decode_error_host, &mapped, sizeof(mapped)), "setting the mapped failure word");
}

int32_t decode_error_flag_ptr(int **dev_ptr) {
    return check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(dev_ptr), g_decode_error),
                      "address of the decode error flag");
}

}  // namespace nf4
