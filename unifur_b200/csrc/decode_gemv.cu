// Decode path: y[M<=16, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T), W stored as
// packed NF4 [N, K] with 64-blocks along K.  HBM-bound: the kernel exists to stream
// nibbles + scales once at full bandwidth.
//
// Data movement.  One CTA per SM owns a contiguous range of W rows; its sixteen warps split K
// (up to four 64-blocks each).  Every warp streams its own slice -- 16 rows x 128 bytes of
// nibbles per tile -- global -> shared with per-thread 16-byte asynchronous copies (cp.async,
// L2 only) into a private ring of a few tiles, rows on a padded stride so that the reads are
// bank-conflict free; the warps therefore share no barrier while the weights stream.  The block
// scales of all the CTA's rows are fetched once, whole lines at a time, at kernel start
// (fetched per warp and tile they cost one load/store-unit tag per 16 bytes, as many as the
// nibbles themselves).  A first version moved whole tiles with TMA bulk copies issued by a
// producer warp and met per tile on barriers; it was slower (18 us against 15 us per launch
// under the profiler), mostly for its per-tile rendezvous and reduction.
//
// Math.  Dequantisation is a shared-memory table lookup: one packed byte (two codes)
// indexes a 256-entry table of half2 {level[lo], level[hi]}, replicated once per
// lane so that no two lanes share a bank; entries sit 256 bytes apart and the table starts at
// shared-window address 0x10000, so that one byte permute (code byte into bits 8..15, lane
// offset below, the constant 0x0001 above) forms the whole address: two instructions per pair
// of weights.  The looked-up register IS the A operand of a warp MMA (m16n8k16, f16 in / f32
// accumulate), with W rows on the MMA's M side and the <=16 activation rows on its N side.
// Each warp keeps its slice of x as f16 B-fragments in registers for the whole kernel.  A
// block's four MMAs accumulate in one chain (the four blocks of a tile interleave) and the
// result is scaled by the block's f32 absmax (or its double-quantized decode) -- the scale
// never touches the f16 path.  What bounds the kernel is instruction issue at four warps per
// scheduler (one 512-thread CTA with ~120 registers per thread fills the register file).
//
// Reduction.  A warp keeps the partial sums of a pass of tiles in registers (a shift register:
// the tile being multiplied is slot 0).  At the end of a pass every warp parks them in its own
// shared-memory slot (the slots take the lookup table's place) and all threads sum the
// sixteen slots in warp order (so results do not depend on timing), add bias and the LoRA term
// (T = x A^T comes from a small pre-pass), convert and store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

__device__ int g_decode_error = 0;  // set when the launch gave too little shared memory or the one bounded wait gives up

#ifdef NF4_DECODE_TIMING
// Optional instrumentation (off in the shipped build): SM-clock timestamps of CTA 0.
__device__ long long g_decode_ts[64];
#define NF4_TS(i) do { if (blockIdx.x == 0 && lane == 0) g_decode_ts[(i)] = clock64(); } while (0)
#else
#define NF4_TS(i) do { } while (0)
#endif

namespace {

constexpr int kWarps = 16;           // all of them split K
constexpr int kDecodeThreads = kWarps * 32;
constexpr int kTileRows = 16;
constexpr int kChunk = 64;           // one quantization block of K
constexpr int kMaxChunksPerWarp = 4; // x fragments live in registers: K <= 16*4*64
constexpr int kMaxRing = 6;          // tiles per warp ring (one being read, the rest in flight)
constexpr uint32_t kLutWindow = 0x10000;  // shared-window address of the lookup table
constexpr int kLutStride = 256;      // bytes between table entries (128 used)
constexpr int kLutBytes = 256 * kLutStride;
constexpr int kMaxRank = 64;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kSmemLeftForPrepass = 3 * 1024;  // so that a CTA of the pre-pass can share the SM
constexpr int kSlots = kWarps;       // one reduction slot per warp

// tiles whose partial sums a warp keeps in registers between two reductions
template <int NT> struct PassTiles { static constexpr int value = NT == 1 ? 8 : 3; };

struct DecodeParams {
    const __nv_bfloat16 *x;
    const uint8_t *codes;
    const float *absmax;
    const uint8_t *scale_codes;
    const float *scale_of_scales;
    const float *bias;
    const float *t;  // [M][rank] f32 = x A^T, or null
    const __nv_bfloat16 *lora_b;
    void *y;
    uint32_t y_f32;
    uint64_t ldy;
    uint32_t M, K, N, rank;
    float lora_scale;
    uint32_t gran;            // CTA row ranges start on multiples of this
    uint32_t chunks_per_warp;
    uint32_t ring;            // tiles per warp ring
    uint32_t pass_tiles;      // tiles per reduction pass (<= PassTiles<NT>)
    uint32_t code_stride;     // bytes between rows of a warp's nibbles in shared memory
    uint32_t slot_bytes;      // one tile of one warp: its nibbles
    uint32_t vec_scales;      // the CTA's scales are staged in shared memory (else read from global)
    uint32_t scale_stride;    // bytes between rows of staged scales (padded)
    uint32_t scale_bytes_max; // room for them
    uint32_t lora_bytes_max;  // room for the CTA's LoRA-B rows
    uint32_t smem_bytes;      // dynamic shared memory of the launch (the kernel lays it out itself)
    uint32_t debug_no_request;  // timing build only: stream nothing after the first tiles
    uint32_t red_slot_bytes;
};

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

// sixteen bf16 (two 128-bit words) -> this lane's f16 B-fragments of one 64-chunk
__device__ __forceinline__ void convert_x(const uint4 &q0, const uint4 &q1, uint32_t (&xf)[4][2]) {
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t pair = w[2 * j + h];  // two bf16: k, k+1
            xf[j][h] = pack_f16x2(bf16_bits_to_float(pair & 0xffffu), bf16_bits_to_float(pair >> 16));
        }
    }
}

// Blocks until at most `n` of this thread's copy groups are in flight (n is small).
__device__ __forceinline__ void wait_groups(uint32_t n) {
    switch (n) {
        case 0: ptx::cp_async_wait<0>(); break;
        case 1: ptx::cp_async_wait<1>(); break;
        case 2: ptx::cp_async_wait<2>(); break;
        case 3: ptx::cp_async_wait<3>(); break;
        case 4: ptx::cp_async_wait<4>(); break;
        default: ptx::cp_async_wait<5>(); break;
    }
}

// FULL: d_in is exactly 4096, so every warp owns four 64-blocks and no per-chunk guard is needed.
// PT: tiles whose partial sums stay in registers between two reductions (>= p.pass_tiles).
// 120 registers x 512 threads and 3 KB short of all the shared memory: the pre-pass's small CTA
// fits on the SM beside this one.
template <int NT, bool DQ, bool FULL, int PT>
__global__ void __maxnreg__(120)
decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Layout by shared-window address: [start, 0x10000) rings of the first warps |
    // [0x10000, 0x20000) lookup table | [0x20000, ...) T, LoRA-B rows, rings of the other warps.
    const uint32_t win0 = ptx::smem_addr(smem_raw);
    uint8_t *smem = smem_raw + (kLutWindow - win0);  // generic pointer to the table
    uint8_t *high = smem + kLutBytes;
    float *t_s = reinterpret_cast<float *>(high);  // [M][rank]
    uint64_t *scale_bar = reinterpret_cast<uint64_t *>(high + 16 * kMaxRank * 4);  // scales have landed
    uint8_t *lora_raw = high + 16 * kMaxRank * 4 + 128;
    const __nv_bfloat16 *lora_s = reinterpret_cast<const __nv_bfloat16 *>(lora_raw);
    float *red = reinterpret_cast<float *>(smem);  // the reduction slots take the lookup table's place
    constexpr int kAccs = 1;  // a block's four MMAs run as one chain (the four blocks of a tile interleave)

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t ring_bytes = p.ring * p.slot_bytes;
    const uint32_t low_room = win0 < kLutWindow ? ((kLutWindow - win0) & ~127u) : 0u;
    const uint32_t low_warps = min((uint32_t)kWarps, low_room / ring_bytes);
    const uint32_t high_used = 16 * kMaxRank * 4 + 128 + p.lora_bytes_max + p.scale_bytes_max +
                               (kWarps - low_warps) * ring_bytes;
    if (win0 > kLutWindow || kLutWindow + kLutBytes + high_used > win0 + p.smem_bytes) {
        if (threadIdx.x == 0) atomicExch(&g_decode_error, 4);  // the launch gave too little room
        return;
    }
    uint8_t *ring = warp < low_warps
                        ? smem - low_room + (size_t)warp * ring_bytes
                        : lora_raw + p.lora_bytes_max + p.scale_bytes_max +
                              (size_t)(warp - low_warps) * ring_bytes;
    const uint32_t ring_addr = ptx::smem_addr(ring);
    uint8_t *scale_raw = lora_raw + p.lora_bytes_max;  // [rows of the CTA][scale_stride]
    const uint32_t R = p.ring, D = R - 1;  // D tiles in flight while one is read

    // rows owned by this CTA: units of `gran` rows, split evenly over the grid
    const uint64_t units = p.N / p.gran;
    const uint32_t n0 = (uint32_t)((uint64_t)blockIdx.x * units / gridDim.x) * p.gran;
    const uint32_t n1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * units / gridDim.x) * p.gran;
    const uint32_t ntiles = (n1 - n0 + kTileRows - 1) / kTileRows;
    if (warp == 0) NF4_TS(0);

    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t nchunks = p.K / kChunk;
    const uint32_t chunk0 = warp * p.chunks_per_warp;
    const bool active = FULL || chunk0 < nchunks;  // short K leaves the last warps without a slice
    const uint32_t my_chunks = FULL ? 4u : (active ? min(p.chunks_per_warp, nchunks - chunk0) : 0u);
    const bool vec_scales = FULL || p.vec_scales;
    const uint32_t code_row_bytes = p.K / 2;

    // Ask for one tile of this warp's slice: 16 rows x (32 bytes per chunk) of nibbles in
    // 16-byte pieces, then the rows' scales.  Rows past the CTA's range are left as they are:
    // their products land in accumulator rows that are never stored.
    // four-chunk slices: lane l copies piece (l & 7) of rows (l >> 3) + 4 i, i = 0..3
    const uint32_t lane_dst = (lane >> 3) * p.code_stride + (lane & 7u) * 16u;
    const uint8_t *lane_src = p.codes + (size_t)(n0 + (lane >> 3)) * code_row_bytes + chunk0 * 32u +
                              (lane & 7u) * 16u;
    uint32_t req_slot = 0, use_slot = 0;  // ring positions of the next request and the next tile read
    auto request_tile = [&](uint32_t tile) {
        const uint32_t row0 = n0 + tile * kTileRows;
        const uint32_t rows = min((uint32_t)kTileRows, n1 - row0);
        const uint32_t slot = ring_addr + req_slot * p.slot_bytes;
        req_slot = req_slot + 1 == R ? 0u : req_slot + 1;
        if (vec_scales) {
            const uint8_t *src = lane_src + (size_t)tile * (kTileRows * code_row_bytes);
            #pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
                if ((lane >> 3) + 4 * i < rows)
                    ptx::cp_async_16(slot + lane_dst + i * 4u * p.code_stride,
                                     src + (size_t)i * 4u * code_row_bytes);
            return;
        }
        const uint32_t pieces_per_row = my_chunks * 2u;
        const uint8_t *src0 = p.codes + (size_t)row0 * code_row_bytes + chunk0 * 32u;
        for (uint32_t q = lane; q < rows * pieces_per_row; q += 32) {
            const uint32_t row = q / pieces_per_row, piece = q - row * pieces_per_row;
            ptx::cp_async_16(slot + row * p.code_stride + piece * 16u,
                             src0 + (size_t)row * code_row_bytes + piece * 16u);
        }
    };

    // ---- x first (plain loads: nothing of this kernel's own is queued ahead of them).  The
    // pre-pass that this kernel may overlap is an ordinary launch: x was complete before it
    // started, so x is complete now. ----
    uint32_t xf[NT][kMaxChunksPerWarp][4][2];  // this warp's slice of x as f16 B-fragments
    {
        uint4 xraw[NT][kMaxChunksPerWarp][2];
        #pragma unroll
        for (int u = 0; u < NT; ++u) {
            const uint32_t m = 8 * u + g;
            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                xraw[u][c][0] = xraw[u][c][1] = make_uint4(0, 0, 0, 0);
                if (m < p.M && c < (int)my_chunks) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(
                        p.x + (size_t)m * p.K + (chunk0 + c) * kChunk + 16 * t);
                    xraw[u][c][0] = __ldg(src);
                    xraw[u][c][1] = __ldg(src + 1);
                }
            }
        }

        // ---- the CTA's block scales (whole rows), its LoRA-B rows and the first tiles ----
        if (tid == 0) {
            ptx::mbar_init(ptx::smem_addr(scale_bar), kDecodeThreads);
            ptx::fence_mbar_init();
        }
        if (vec_scales) {
            const uint32_t rows_cta = n1 - n0;
            if (DQ) {
                const uint32_t ppr = nchunks / 4;  // 4-byte pieces per row
                for (uint32_t q = tid; q < rows_cta * ppr; q += kDecodeThreads) {
                    const uint32_t row = q / ppr, pc = q - row * ppr;
                    ptx::cp_async_4(ptx::smem_addr(scale_raw) + row * p.scale_stride + pc * 4u,
                                    p.scale_codes + (size_t)(n0 + row) * nchunks + pc * 4u);
                }
            } else {
                const uint32_t ppr = nchunks / 4;  // 16-byte pieces per row
                for (uint32_t q = tid; q < rows_cta * ppr; q += kDecodeThreads) {
                    const uint32_t row = q / ppr, pc = q - row * ppr;
                    ptx::cp_async_16(ptx::smem_addr(scale_raw) + row * p.scale_stride + pc * 16u,
                                     p.absmax + (size_t)(n0 + row) * nchunks + pc * 4u);
                }
            }
        }
        if (p.rank) {
            const uint32_t pieces = (n1 - n0) * p.rank * 2u / 16u;
            const uint8_t *src = reinterpret_cast<const uint8_t *>(p.lora_b + (size_t)n0 * p.rank);
            for (uint32_t q = tid; q < pieces; q += kDecodeThreads)
                ptx::cp_async_16(ptx::smem_addr(lora_raw) + q * 16u, src + (size_t)q * 16u);
        }
        ptx::cp_async_commit();
        for (uint32_t d = 0; d < D; ++d) {
            if (active && d < ntiles) request_tile(d);
            ptx::cp_async_commit();
        }

        if (warp == 0) NF4_TS(2);
        #pragma unroll
        for (int u = 0; u < NT; ++u) {
            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) convert_x(xraw[u][c][0], xraw[u][c][1], xf[u][c]);
        }
#ifdef NF4_DECODE_TIMING
        if (xf[0][0][0][0] == 0x12345678u) NF4_TS(63);  // forces the conversion before the next stamp
#endif
        if (warp == 0) NF4_TS(3);
    }

    // ---- the lookup table: thread (byte, half) writes sixteen lanes' copies of its entry ----
    auto build_table = [&]() {
        const uint32_t byte = tid >> 1, half = tid & 1u;
        const uint32_t entry = c_level_f16_bits[byte & 15u] | (c_level_f16_bits[byte >> 4] << 16);
        const uint4 v = make_uint4(entry, entry, entry, entry);
        #pragma unroll
        for (int i = 0; i < 4; ++i)  // rotated by the byte so that a warp's stores spread over the banks
            *reinterpret_cast<uint4 *>(smem + byte * kLutStride + half * 64u + ((i + byte) & 3u) * 16u) = v;
    };
    build_table();
    if (warp == 0) NF4_TS(50);
    __syncthreads();
    // every thread's scale pieces report to one barrier when they land (no wait here)
    asm volatile("cp.async.mbarrier.arrive.noinc.shared.b64 [%0];" ::"r"(ptx::smem_addr(scale_bar)) : "memory");
    if (warp == 0) NF4_TS(1);

    const float sos = DQ ? __ldg(p.scale_of_scales) : 0.0f;
    // shared-window address of a table entry = {0x0001, code byte, lane * 4}
    const uint32_t lane_word = kLutWindow | (lane * 4u);
    auto lut_at = [&](uint32_t word, int byte) -> uint32_t {
        const uint32_t addr = __byte_perm(word, lane_word, 0x7604u | ((uint32_t)byte << 4));
        uint32_t v;
        asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
        return v;
    };
    const uint32_t slot_floats = p.red_slot_bytes / 4;
    const uint32_t first_pass_last = min(ntiles, p.pass_tiles) - 1;

    float acc[PT][NT][4];
    #pragma unroll
    for (int q = 0; q < PT; ++q) {
        #pragma unroll
        for (int u = 0; u < NT; ++u) acc[q][u][0] = acc[q][u][1] = acc[q][u][2] = acc[q][u][3] = 0.0f;
    }
    uint32_t pass_tile0 = 0;

    // One copy of the tile code; the accumulators work as a shift register: the tile being
    // multiplied is acc[0], older tiles of the pass move up.  The stream runs ahead across
    // pass boundaries.
    #pragma unroll 1
    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        if (active) {
            #pragma unroll
            for (int q = PT - 1; q > 0; --q) {
                #pragma unroll
                for (int u = 0; u < NT; ++u) {
                    #pragma unroll
                    for (int r = 0; r < 4; ++r) acc[q][u][r] = acc[q - 1][u][r];
                }
            }
            #pragma unroll
            for (int u = 0; u < NT; ++u) acc[0][u][0] = acc[0][u][1] = acc[0][u][2] = acc[0][u][3] = 0.0f;

            // The adapter intermediate comes from the pre-pass, which has had most of the
            // stream to finish: warp 0 asks for it one tile before it is needed.
            if (warp == 0 && p.rank && tile == first_pass_last) {
                ptx::pdl_wait();
                for (uint32_t i = lane; i < p.M * p.rank; i += 32)
                    ptx::cp_async_4(ptx::smem_addr(t_s + i), p.t + i);
                ptx::cp_async_commit();
            }
            // keep D tiles in flight, then wait for this one (groups retire in order)
            __syncwarp();  // every lane is done reading the slot about to be refilled
#ifdef NF4_DECODE_TIMING
            if (!p.debug_no_request)
#endif
            if (tile + D < ntiles) request_tile(tile + D);
            ptx::cp_async_commit();
            if (warp == 0 && tile < 8) NF4_TS(42 + tile);
            wait_groups(D);
            __syncwarp();  // the other lanes' pieces are visible too
            if (warp == 0 && tile < 8) NF4_TS(4 + 3 * tile);
            const uint8_t *st = ring + (size_t)use_slot * p.slot_bytes;
            use_slot = use_slot + 1 == R ? 0u : use_slot + 1;
            const uint8_t *codes_lo = st + g * p.code_stride + t * 8;
            const uint8_t *codes_hi = codes_lo + 8 * p.code_stride;

            float s_lo[kMaxChunksPerWarp], s_hi[kMaxChunksPerWarp];
            if (vec_scales) {
                if (tile == 0 && !ptx::mbar_wait_bounded(ptx::smem_addr(scale_bar), 0)) {
                    if (lane == 0) atomicExch(&g_decode_error, 5);
                }
                const uint8_t *sc = scale_raw + (size_t)(tile * kTileRows + g) * p.scale_stride;
                if (DQ) {
                    const uint32_t a = *reinterpret_cast<const uint32_t *>(sc + chunk0);
                    const uint32_t b = *reinterpret_cast<const uint32_t *>(sc + 8 * p.scale_stride + chunk0);
                    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        s_lo[c] = dq_scale((a >> (8 * c)) & 0xffu, sos);
                        s_hi[c] = dq_scale((b >> (8 * c)) & 0xffu, sos);
                    }
                } else {
                    const float4 a = *reinterpret_cast<const float4 *>(sc + chunk0 * 4);
                    const float4 b = *reinterpret_cast<const float4 *>(sc + 8 * p.scale_stride + chunk0 * 4);
                    s_lo[0] = a.x; s_lo[1] = a.y; s_lo[2] = a.z; s_lo[3] = a.w;
                    s_hi[0] = b.x; s_hi[1] = b.y; s_hi[2] = b.z; s_hi[3] = b.w;
                }
            } else {
                // odd slice widths: the scales come straight from global memory
                const uint32_t r_lo = min(n0 + tile * kTileRows + g, n1 - 1);
                const uint32_t r_hi = min(n0 + tile * kTileRows + g + 8, n1 - 1);
                #pragma unroll
                for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                    s_lo[c] = s_hi[c] = 0.0f;
                    if (c < (int)my_chunks) {
                        const size_t i_lo = (size_t)r_lo * nchunks + chunk0 + c;
                        const size_t i_hi = (size_t)r_hi * nchunks + chunk0 + c;
                        s_lo[c] = DQ ? dq_scale(__ldg(p.scale_codes + i_lo), sos) : __ldg(p.absmax + i_lo);
                        s_hi[c] = DQ ? dq_scale(__ldg(p.scale_codes + i_hi), sos) : __ldg(p.absmax + i_hi);
                    }
                }
            }

            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                if (c < (int)my_chunks) {
                    const uint2 w0 = *reinterpret_cast<const uint2 *>(codes_lo + c * 32);
                    const uint2 w1 = *reinterpret_cast<const uint2 *>(codes_hi + c * 32);
                    float blk[kAccs][NT][4];
                    #pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t x0 = (j < 2) ? w0.x : w0.y;
                        const uint32_t x1 = (j < 2) ? w1.x : w1.y;
                        const int b = 2 * (j & 1);
                        const uint32_t a0 = lut_at(x0, b), a1 = lut_at(x1, b);
                        const uint32_t a2 = lut_at(x0, b + 1), a3 = lut_at(x1, b + 1);
                        #pragma unroll
                        for (int u = 0; u < NT; ++u) {
                            if (j == 0)
                                ptx::mma_16816_f16_zero(blk[0][u], a0, a1, a2, a3, xf[u][c][j][0],
                                                        xf[u][c][j][1]);
                            else
                                ptx::mma_16816_f16(blk[0][u], a0, a1, a2, a3, xf[u][c][j][0],
                                                   xf[u][c][j][1]);
                        }
                    }
                    #pragma unroll
                    for (int u = 0; u < NT; ++u) {
                        #pragma unroll
                        for (int r = 0; r < 4; ++r)
                            acc[0][u][r] = fmaf(blk[0][u][r], r < 2 ? s_lo[c] : s_hi[c], acc[0][u][r]);
                    }
                }
            }
            if (warp == 0 && tile < 8) NF4_TS(5 + 3 * tile);
        }

        const uint32_t tiles_in_pass = tile + 1 - pass_tile0;
        if (tiles_in_pass < p.pass_tiles && tile + 1 < ntiles) continue;

        // ================= end of a pass: reduce, finish and store its rows =================
        // The reduction slots take the place of the lookup table, which is rebuilt afterwards
        // if more tiles follow; the rings keep filling meanwhile.
        if (warp == 0) NF4_TS(40);
        __syncthreads();  // nobody reads the table any more
        {
            // acc[q] holds the pass's tile number (tiles_in_pass - 1 - q)
            float *slot = red + warp * slot_floats;
            #pragma unroll
            for (int q = 0; q < PT; ++q) {
                if (q < (int)tiles_in_pass) {
                    const int ti = (int)tiles_in_pass - 1 - q;
                    #pragma unroll
                    for (int u = 0; u < NT; ++u) {
                        #pragma unroll
                        for (int r = 0; r < 4; ++r)
                            slot[((ti * NT + u) * 4 + r) * 32 + lane] = acc[q][u][r];
                    }
                }
            }
        }
        if (pass_tile0 == 0) {
            // first pass only: the LoRA-B rows and T must have landed; at most one copy group
            // (a tile's) is newer than T's
            if (tile + 1 == ntiles) ptx::cp_async_wait<0>();
            else ptx::cp_async_wait<1>();
        }
        __syncthreads();

        // ---- everyone: sum the sixteen slots in order, + adapter, + bias, convert, store ----
        // Thread o takes slot element o (conflict-free reads) and works out which output that
        // is: element = ((tile * NT + u) * 4 + r) * 32 + source lane.
        const uint32_t pass_row0 = n0 + pass_tile0 * kTileRows;
        const uint32_t pass_rows = min(n1 - pass_row0, tiles_in_pass * (uint32_t)kTileRows);
        for (uint32_t o = tid; o < tiles_in_pass * NT * 128u; o += kDecodeThreads) {
            const uint32_t src_lane = o & 31u, r = (o >> 5) & 3u, tu = o >> 7;
            const uint32_t ti = tu / NT, u = tu - ti * NT;
            const uint32_t rr = ti * kTileRows + (r >> 1) * 8u + (src_lane >> 2);
            const uint32_t m = u * 8u + (src_lane & 3u) * 2u + (r & 1u);
            if (rr >= pass_rows || m >= p.M) continue;
            float v = red[o];
            #pragma unroll
            for (int w = 1; w < kSlots; ++w) v += red[w * slot_floats + o];
            if (p.rank) {
                const __nv_bfloat16 *lb = lora_s + (size_t)(pass_row0 - n0 + rr) * p.rank;
                const float *tm = t_s + m * p.rank;
                float dot = 0.0f;
                if ((p.rank & 7u) == 0) {
                    for (uint32_t j = 0; j < p.rank; j += 8) {
                        const uint4 bq = *reinterpret_cast<const uint4 *>(lb + j);
                        const float4 t0 = *reinterpret_cast<const float4 *>(tm + j);
                        const float4 t1 = *reinterpret_cast<const float4 *>(tm + j + 4);
                        dot = fmaf(t0.x, bf16_bits_to_float(bq.x & 0xffffu), dot);
                        dot = fmaf(t0.y, bf16_bits_to_float(bq.x >> 16), dot);
                        dot = fmaf(t0.z, bf16_bits_to_float(bq.y & 0xffffu), dot);
                        dot = fmaf(t0.w, bf16_bits_to_float(bq.y >> 16), dot);
                        dot = fmaf(t1.x, bf16_bits_to_float(bq.z & 0xffffu), dot);
                        dot = fmaf(t1.y, bf16_bits_to_float(bq.z >> 16), dot);
                        dot = fmaf(t1.z, bf16_bits_to_float(bq.w & 0xffffu), dot);
                        dot = fmaf(t1.w, bf16_bits_to_float(bq.w >> 16), dot);
                    }
                } else {
                    for (uint32_t j = 0; j < p.rank; ++j) dot = fmaf(tm[j], __bfloat162float(lb[j]), dot);
                }
                v = fmaf(dot, p.lora_scale, v);  // scale applied last
            }
            if (p.bias) v += __ldg(p.bias + pass_row0 + rr);
            const size_t at = (size_t)m * p.ldy + pass_row0 + rr;
            if (p.y_f32) static_cast<float *>(p.y)[at] = v;
            else static_cast<__nv_bfloat16 *>(p.y)[at] = __float2bfloat16_rn(v);
        }
        if (warp == 0) NF4_TS(41);
        pass_tile0 = tile + 1;
        if (pass_tile0 < ntiles) {
            __syncthreads();  // the slots have been read
            build_table();
            __syncthreads();
            #pragma unroll
            for (int q = 0; q < PT; ++q) {
                #pragma unroll
                for (int u = 0; u < NT; ++u) acc[q][u][0] = acc[q][u][1] = acc[q][u][2] = acc[q][u][3] = 0.0f;
            }
        }
    }
    ptx::cp_async_wait<0>();
}

// T[m][j] = sum_k x[m][k] * A[j][k]  (x, A bf16; f32 accumulate).  One 128-thread CTA per (j, m):
// many short CTAs with at most 32 registers, so that one of them fits on an SM beside a GEMV CTA
// and the GEMV it overlaps with is not kept off the SMs the pre-pass occupies.
__global__ void __launch_bounds__(128, 16)
lora_t_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a, uint32_t K,
              uint32_t rank, float *__restrict__ t_out) {
    ptx::pdl_launch_dependents();  // the GEMV may start streaming weights right away
    const uint32_t j = blockIdx.x, m = blockIdx.y;
    const __nv_bfloat16 *xr = x + (size_t)m * K, *ar = a + (size_t)j * K;
    float acc = 0.0f;
    if ((K & 7u) == 0) {
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
uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

bool plan(const nf4_linear_args &a, DecodeParams &p, uint32_t &grid, uint32_t &smem_bytes) {
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_BF16) return false;
    if (a.rows == 0 || a.rows > 16) return false;
    if (a.d_in % kChunk != 0 || a.d_in > (uint64_t)kWarps * kMaxChunksPerWarp * kChunk) return false;
    if (a.d_out >= (1ull << 31)) return false;
    const bool dq = a.scale_codes != nullptr;
    const uint32_t rank = a.lora_a ? a.lora_rank : 0;
    if (rank > kMaxRank) return false;
    const void *scales = dq ? (const void *)a.scale_codes : (const void *)a.absmax;
    if (!aligned16(a.x) || !aligned16(a.packed) || !aligned16(scales)) return false;
    if (rank && !aligned16(a.lora_b)) return false;
    if (reinterpret_cast<uintptr_t>(a.y) & (a.y_f32 ? 3u : 1u)) return false;

    const uint32_t K = (uint32_t)a.d_in, N = (uint32_t)a.d_out, M = (uint32_t)a.rows;
    const uint32_t nchunks = K / kChunk;
    const uint32_t nt = M > 8 ? 2u : 1u;
    p = DecodeParams{};
    // CTA row ranges start where the CTA's LoRA-B rows are 16-byte aligned
    const uint32_t gran = rank ? 16u / gcd_u32(16u, rank * 2u) : 1u;
    if (N % gran != 0) return false;
    p.gran = gran;
    p.chunks_per_warp = (nchunks + kWarps - 1) / kWarps;
    p.vec_scales = (p.chunks_per_warp == 4 && nchunks % 4 == 0) ? 1u : 0u;
    p.code_stride = p.chunks_per_warp * 32u + 32u;  // 160 for four chunks: conflict-free 64-bit reads
    p.slot_bytes = kTileRows * p.code_stride;

    const uint64_t units = N / gran;
    grid = (uint32_t)(units < (uint64_t)kNumSMs ? units : (uint64_t)kNumSMs);
    const uint32_t max_rows = (uint32_t)(((units + grid - 1) / grid) * gran);
    const uint32_t max_tiles = (max_rows + kTileRows - 1) / kTileRows;
    const uint32_t pt_max = nt == 1 ? (uint32_t)PassTiles<1>::value : (uint32_t)PassTiles<2>::value;
    p.pass_tiles = max_tiles < pt_max ? max_tiles : pt_max;
    p.red_slot_bytes = p.pass_tiles * nt * 512u;
    p.lora_bytes_max = round_up(max_rows * rank * 2u, 128);
    // The kernel puts the table at shared-window address 0x10000 and the rings around it; with
    // the usual 1 KB reserved at the start of the window that leaves 63 KB below and
    // (227 - 127) KB above the table.
    const uint32_t low_room = (kLutWindow - 1024u) & ~127u;
    const uint32_t high_room = (uint32_t)(kSmemLimit - kSmemLeftForPrepass) + 1024u - (kLutWindow + (uint32_t)kLutBytes);
    p.scale_stride = nchunks * (dq ? 1u : 4u) + 16u;
    p.scale_bytes_max = p.vec_scales ? round_up(max_tiles * kTileRows * p.scale_stride, 128) : 0u;
    const uint32_t high_fixed = 16 * kMaxRank * 4 + 128 + p.lora_bytes_max + p.scale_bytes_max;
    static const int ring_env = [] {
        const char *e = std::getenv("NF4_DECODE_RING");  // experiment knob: tiles per warp ring
        return e ? std::atoi(e) : 0;
    }();
    uint32_t ring = 0;
    for (uint32_t r = 2; r <= (uint32_t)kMaxRing && r <= max_tiles + 1; ++r) {
        const uint32_t ring_bytes = r * p.slot_bytes;
        const uint32_t low_warps = low_room / ring_bytes < (uint32_t)kWarps ? low_room / ring_bytes : (uint32_t)kWarps;
        if (high_fixed + (kWarps - low_warps) * ring_bytes > high_room) break;
        if (ring_env >= 2 && r > (uint32_t)ring_env) break;
        ring = r;
    }
    if (ring < 2) {
        // a short matrix still needs two slots
        const uint32_t ring_bytes = 2 * p.slot_bytes;
        const uint32_t low_warps = low_room / ring_bytes < (uint32_t)kWarps ? low_room / ring_bytes : (uint32_t)kWarps;
        if (high_fixed + (kWarps - low_warps) * ring_bytes > high_room) return false;
        ring = 2;
    }
    p.ring = ring;
    if (kSlots * p.red_slot_bytes > (uint32_t)kLutBytes) return false;  // the slots reuse the table's room
    smem_bytes = kSmemLimit - kSmemLeftForPrepass;
    p.smem_bytes = smem_bytes;
    static const bool no_request = [] {
        const char *e = std::getenv("NF4_DEBUG_NO_REQUEST");  // read by the timing build only
        return e && e[0] == '1';
    }();
    p.debug_no_request = no_request ? 1u : 0u;
    p.x = static_cast<const __nv_bfloat16 *>(a.x);
    p.codes = a.packed;
    p.absmax = a.absmax;
    p.scale_codes = a.scale_codes;
    p.scale_of_scales = a.scale_of_scales;
    p.bias = a.bias;
    p.lora_b = static_cast<const __nv_bfloat16 *>(a.lora_b);
    p.y = a.y;
    p.y_f32 = (uint32_t)a.y_f32;
    p.ldy = a.ldy ? a.ldy : a.d_out;
    p.M = M;
    p.K = K;
    p.N = N;
    p.rank = rank;
    p.lora_scale = a.lora_scale;
    return true;
}

template <int NT, bool DQ, bool FULL, int PT>
int32_t launch_pt(const DecodeParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream) {
    static bool configured = false;  // benign race: the attribute is idempotent
    if (!configured) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<NT, DQ, FULL, PT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        configured = true;
    }
    count_launch();
    return launch_maybe_overlapped(decode_kernel<NT, DQ, FULL, PT>, dim3(grid), dim3(kDecodeThreads),
                                   smem_bytes, stream, p.rank != 0 && pdl_enabled(), p);
}

// the register budget holds 8 tiles of 8 activation rows or 3 tiles of 16; shorter passes get a
// kernel whose accumulator shift register is as short as they need
template <int NT, bool DQ, bool FULL>
int32_t launch_full(const DecodeParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream) {
    if constexpr (NT == 2) {
        return launch_pt<NT, DQ, FULL, PassTiles<2>::value>(p, grid, smem_bytes, stream);
    } else {
        if (p.pass_tiles <= 2) return launch_pt<NT, DQ, FULL, 2>(p, grid, smem_bytes, stream);
        if (p.pass_tiles <= 5) return launch_pt<NT, DQ, FULL, 5>(p, grid, smem_bytes, stream);
        return launch_pt<NT, DQ, FULL, PassTiles<1>::value>(p, grid, smem_bytes, stream);
    }
}

template <int NT, bool DQ>
int32_t launch(const DecodeParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream) {
    return p.K == (uint32_t)(kWarps * kMaxChunksPerWarp * kChunk)
               ? launch_full<NT, DQ, true>(p, grid, smem_bytes, stream)
               : launch_full<NT, DQ, false>(p, grid, smem_bytes, stream);
}

}  // namespace

bool decode_supported(const nf4_linear_args &a) {
    DecodeParams p;
    uint32_t grid, smem;
    return plan(a, p, grid, smem);
}

uint64_t decode_workspace_bytes(uint64_t rows, uint32_t lora_rank) {
    if (rows == 0 || rows > 16 || lora_rank == 0) return 0;
    return (rows * lora_rank * 4 + 255) / 256 * 256;
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

int32_t decode_forward(const nf4_linear_args &a, cudaStream_t stream) {
    DecodeParams p;
    uint32_t grid, smem;
    if (!plan(a, p, grid, smem)) return fail(NF4_ERR_UNSUPPORTED, "decode_forward: unsupported shape");
    if (p.rank) {
        float *t = static_cast<float *>(a.workspace);
        NF4_TRY(lora_t_small(a.x, a.lora_a, p.M, p.K, p.rank, t, stream, false));
        p.t = t;
    }
    const bool dq = a.scale_codes != nullptr;
    if (p.M <= 8) return dq ? launch<1, true>(p, grid, smem, stream) : launch<1, false>(p, grid, smem, stream);
    return dq ? launch<2, true>(p, grid, smem, stream) : launch<2, false>(p, grid, smem, stream);
}

#ifdef NF4_DECODE_TIMING
extern "C" __attribute__((visibility("default"))) int nf4_debug_decode_timestamps(long long *out64) {
    return (int)cudaMemcpyFromSymbol(out64, g_decode_ts, sizeof(long long) * 64);
}
#endif

// ---- decode forward whose scratch is a fixed device array (no allocation anywhere) ----
// The adapter intermediate T = x A^T ([rows][rank] f32) is the only scratch the decode
// path needs.  Here it lives in a file-scope device array instead of a caller buffer.
constexpr uint32_t kStaticScratchBytes = 16 * kMaxRank * sizeof(float);  // 16 rows x rank 64
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

uint64_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

int32_t decode_forward_static_scratch(const nf4_linear_args &a, cudaStream_t stream) {
    DecodeParams p;
    uint32_t grid, smem;
    if (!plan(a, p, grid, smem))
        return fail(NF4_ERR_UNSUPPORTED,
                    "nf4_linear_forward_noalloc_dev: only the decode shapes are served (rows <= 16, "
                    "bf16, W [d_out, d_in], d_in %% 64 == 0 and <= 4096, rank <= 64)");
    const uint64_t need = (uint64_t)p.M * p.rank * sizeof(float);
    if (need > kStaticScratchBytes)
        return fail(NF4_ERR_INVALID_ARG,
                    "nf4_linear_forward_noalloc_dev: rows * rank * 4 = %llu bytes exceeds the fixed "
                    "scratch of %u bytes", (unsigned long long)need, kStaticScratchBytes);
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
    if (p.rank) {
        float *t = static_cast<float *>(scratch);  // fully rewritten by the pre-pass: no clearing needed
        NF4_TRY(lora_t_small(a.x, a.lora_a, p.M, p.K, p.rank, t, stream, false));
        p.t = t;
    }
    const bool dq = a.scale_codes != nullptr;
    if (p.M <= 8) return dq ? launch<1, true>(p, grid, smem, stream) : launch<1, false>(p, grid, smem, stream);
    return dq ? launch<2, true>(p, grid, smem, stream) : launch<2, false>(p, grid, smem, stream);
}

int32_t decode_error_flag(int *host_value) {
    return check_cuda(cudaMemcpyFromSymbol(host_value, g_decode_error, sizeof(int)),
                      "read decode error flag");
}

}  // namespace nf4
