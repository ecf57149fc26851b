// Decode path: y[M<=16, N] = x * dequant(W)^T (+bias) (+ s * (x A^T) B^T), W stored as
// packed NF4 [N, K] with 64-blocks along K.  HBM-bound: the kernel exists to stream
// nibbles + scales once at full bandwidth.
//
// Data movement.  One CTA per SM owns a contiguous range of W rows.  A producer warp
// streams 16-row tiles (packed bytes, block scales, LoRA-B rows) global -> shared with
// untiled TMA bulk copies that complete on an mbarrier; every row lands on a padded
// stride so the consumers' shared-memory reads are bank-conflict free.  Whole tiles
// are requested as soon as a ring slot is free, which keeps ~150 KB per SM in flight.
//
// Math.  Dequantisation is a shared-memory table lookup: one packed byte (two codes)
// indexes a 256-entry table of half2 {level[lo], level[hi]}, replicated once per
// lane so that no two lanes share a bank.  The looked-up register IS the A operand of
// a warp MMA (m16n8k16, f16 in / f32 accumulate), with W rows on the MMA's M side and
// the <=16 activation rows on its N side.  The sixteen consumer warps split K; each
// keeps its slice of x as f16 B-fragments in registers for the whole kernel.  A block's
// four MMAs accumulate into a scratch accumulator that is then scaled by the block's
// f32 absmax (or its double-quantized decode) -- the scale never touches the f16 path.
// Each warp parks its partial sums in its own slice of a shared-memory slot and the
// producer warp finishes each tile: sum the slices in warp order (so results do not
// depend on timing), + bias, + LoRA (T = x A^T comes from a small pre-pass), convert, store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "kernels.cuh"
#include "ptx.cuh"

namespace nf4 {

__device__ int g_decode_error = 0;  // set when a bounded wait gives up

#ifdef NF4_DECODE_TIMING
// Optional instrumentation (off in the shipped build): SM-clock timestamps of CTA 0.
__device__ long long g_decode_ts[64];
#define NF4_TS(i) do { if (blockIdx.x == 0 && lane == 0) g_decode_ts[(i)] = clock64(); } while (0)
#else
#define NF4_TS(i) do { } while (0)
#endif

namespace {

constexpr int kMaxConsumerWarps = 16;
constexpr int kTileRows = 16;
constexpr int kChunk = 64;           // one quantization block of K
constexpr int kMaxChunksPerWarp = 4; // x fragments live in registers: K <= 16*4*64
constexpr int kMaxStages = 8;
constexpr int kLutBytes = 256 * 32 * 4;
constexpr int kMaxRank = 64;
constexpr int kSmemLimit = 227 * 1024;

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
    uint32_t consumer_warps;  // warps that split K
    uint32_t chunks_per_warp;
    uint32_t stages;
    uint32_t code_stride;   // bytes between rows of packed codes in shared memory
    uint32_t scale_stride;  // bytes between rows of scales in shared memory
    uint32_t scale_row_bytes;
    uint32_t scale_per_row;  // 1: one bulk copy per row (padded); 0: one copy per tile
    uint32_t stage_bytes;
    uint32_t off_scales, off_lora;  // offsets inside a stage
    uint32_t off_red, off_stages;   // offsets inside dynamic shared memory
};

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

// Producer warp: request one 16-row tile (packed bytes, block scales, LoRA-B rows) into its ring
// slot.  Lane r copies row r; lane 31 issues the copies that cover the whole tile.
template <bool DQ>
__device__ __forceinline__ void issue_tile(const DecodeParams &p, uint32_t tile, uint32_t n0,
                                           uint32_t n1, uint32_t S, uint8_t *stage_base,
                                           uint32_t bar_full, uint32_t lane) {
    const uint32_t s = tile % S;
    const uint32_t row0 = n0 + tile * kTileRows;
    const uint32_t rows = min((uint32_t)kTileRows, n1 - row0);
    const uint32_t code_row_bytes = p.K / 2;
    uint8_t *st = stage_base + (size_t)s * p.stage_bytes;
    const uint32_t bar = bar_full + 8 * s;
    const uint32_t lora_bytes = p.rank ? rows * p.rank * 2u : 0u;
    if (lane == 0)
        ptx::mbar_arrive_expect_tx(bar, rows * (code_row_bytes + p.scale_row_bytes) + lora_bytes);
    __syncwarp();
    if (lane < rows) {
        const uint32_t r = row0 + lane;
        ptx::bulk_g2s(ptx::smem_addr(st + lane * p.code_stride),
                      p.codes + (size_t)r * code_row_bytes, code_row_bytes, bar);
        if (p.scale_per_row) {
            const uint8_t *src = DQ ? p.scale_codes + (size_t)r * p.scale_row_bytes
                                    : reinterpret_cast<const uint8_t *>(p.absmax) +
                                          (size_t)r * p.scale_row_bytes;
            ptx::bulk_g2s(ptx::smem_addr(st + p.off_scales + lane * p.scale_stride), src,
                          p.scale_row_bytes, bar);
        }
    }
    if (lane == 31) {
        if (!p.scale_per_row) {
            const uint8_t *src = DQ ? p.scale_codes + (size_t)row0 * p.scale_row_bytes
                                    : reinterpret_cast<const uint8_t *>(p.absmax) +
                                          (size_t)row0 * p.scale_row_bytes;
            ptx::bulk_g2s(ptx::smem_addr(st + p.off_scales), src, rows * p.scale_row_bytes, bar);
        }
        if (lora_bytes)
            ptx::bulk_g2s(ptx::smem_addr(st + p.off_lora), p.lora_b + (size_t)row0 * p.rank,
                          lora_bytes, bar);
    }
}

template <int NT, bool DQ>
__global__ void __launch_bounds__((kMaxConsumerWarps + 2) * 32, 1)
decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kLutBytes);  // full[8], done[8], red_free[2]
    float *t_s = reinterpret_cast<float *>(smem + kLutBytes + 256);    // [M][rank]
    float *red = reinterpret_cast<float *>(smem + p.off_red);          // [2][warps][16][MP]
    uint8_t *stage_base = smem + p.off_stages;
    constexpr int MP = 8 * NT;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t S = p.stages;
    const uint32_t red_slot_floats = p.consumer_warps * kTileRows * MP;

    // rows owned by this CTA: units of `gran` rows, split evenly over the grid
    const uint64_t units = p.N / p.gran;
    const uint32_t n0 = (uint32_t)((uint64_t)blockIdx.x * units / gridDim.x) * p.gran;
    const uint32_t n1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * units / gridDim.x) * p.gran;
    const uint32_t ntiles = (n1 - n0 + kTileRows - 1) / kTileRows;

    const uint32_t bar_full = ptx::smem_addr(bars), bar_done = ptx::smem_addr(bars + kMaxStages);
    const uint32_t bar_red_free = ptx::smem_addr(bars + 2 * kMaxStages);
    const uint32_t bar_epi_done = ptx::smem_addr(bars + 2 * kMaxStages + 2);
    if (warp == 0) NF4_TS(0);

    // Consumers ask for their slice of x before anything else: once the producer's bulk copies
    // saturate the memory system, a late request would queue behind ~150 KB per SM.
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t nchunks = p.K / kChunk;
    const uint32_t chunk0 = warp * p.chunks_per_warp;
    uint4 xraw[NT][kMaxChunksPerWarp][2];
    if (warp < p.consumer_warps) {
        #pragma unroll
        for (int u = 0; u < NT; ++u) {
            const uint32_t m = 8 * u + g;
            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                const uint32_t kc = chunk0 + c;
                xraw[u][c][0] = xraw[u][c][1] = make_uint4(0, 0, 0, 0);
                if (m < p.M && c < (int)p.chunks_per_warp && kc < nchunks) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(
                        p.x + (size_t)m * p.K + kc * kChunk + 16 * t);
                    xraw[u][c][0] = __ldg(src);
                    xraw[u][c][1] = __ldg(src + 1);
                }
            }
        }
    }

    // x slice of this warp as f16 B-fragments, converted as soon as it arrives
    uint32_t xf[NT][kMaxChunksPerWarp][4][2];
    if (warp < p.consumer_warps) {
        // x slice of this warp as f16 B-fragments: xf[u][c][j] = {b0, b1}
        #pragma unroll
        for (int u = 0; u < NT; ++u) {
            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                const uint4 q0 = xraw[u][c][0], q1 = xraw[u][c][1];
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    #pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t pair = w[2 * j + h];  // two bf16: k, k+1
                        xf[u][c][j][h] = pack_f16x2(bf16_bits_to_float(pair & 0xffffu),
                                                    bf16_bits_to_float(pair >> 16));
                    }
                }
            }
        }

        if (warp == 0) NF4_TS(7);
        asm volatile("bar.arrive 3, %0;" ::"r"((p.consumer_warps + 1) * 32) : "memory");
    }

    if (warp == p.consumer_warps) {
        // ========================= producer warp =========================
        // The barriers are this warp's to set up, so the first loads leave before the other
        // warps have finished building the lookup table.
        if (lane == 0) {
            for (uint32_t s = 0; s < S; ++s) {
                ptx::mbar_init(bar_full + 8 * s, 1);
                ptx::mbar_init(bar_done + 8 * s, p.consumer_warps);
                ptx::mbar_init(bar_epi_done + 8 * s, 1);
            }
            ptx::mbar_init(bar_red_free, 1);
            ptx::mbar_init(bar_red_free + 8, 1);
            ptx::fence_mbar_init();
            ptx::fence_proxy_async();
        }
        __syncwarp();
        // hold the bulk copies back until the consumers HAVE their x: requests issued behind
        // ~150 KB of queued weight traffic per SM were seen to take ~4 us to come back
        asm volatile("bar.sync 3, %0;" ::"r"((p.consumer_warps + 1) * 32) : "memory");
        // Only the first tile is requested now.  Asking for everything at once makes every tile,
        // the first included, arrive together after the whole ~150 KB burst (~4 us); with one to
        // two tiles in flight the first is there after ~1 us and the rest keep ahead of the math.
        issue_tile<DQ>(p, 0, n0, n1, S, stage_base, bar_full, lane);
    } else if (warp < p.consumer_warps) {
        // ---- consumers build the lookup table while the first tiles are in flight ----
        const uint32_t nthreads = p.consumer_warps * 32;
        for (uint32_t i = tid; i < 256 * 32; i += nthreads) {
            const uint32_t byte = i >> 5;
            lut[i] = pack_f16x2(__uint_as_float(c_level_bits[byte & 15u]),
                                __uint_as_float(c_level_bits[byte >> 4]));
        }
    }
    __syncthreads();
    if (warp == 0) NF4_TS(1);

    if (warp == p.consumer_warps) {
        // Producer: keep `ahead + 1` tiles in flight, in order.  A tile is requested once the
        // tile `ahead + 1` before it has landed and its ring slot's previous tile is finished.
        const uint32_t ahead = S >= 4 ? 3u : S - 1u;
        bool ok = true;
        for (uint32_t n = 1; n < ntiles && ok; ++n) {
            if (n > ahead) {
                const uint32_t w = n - ahead - 1;
                ok = ptx::mbar_wait_bounded(bar_full + 8 * (w % S), (w / S) & 1u);
            }
            if (ok && n >= S) ok = ptx::mbar_wait_bounded(bar_epi_done + 8 * (n % S), ((n / S) - 1) & 1u);
            if (!ok) break;
            ptx::fence_proxy_async();
            issue_tile<DQ>(p, n, n0, n1, S, stage_base, bar_full, lane);
        }
        if (!ok && lane == 0) atomicExch(&g_decode_error, 3);
    } else if (warp == p.consumer_warps + 1) {
        // ========================= epilogue warp =========================
        // T = x A^T comes from the pre-pass, which may still be running: wait for it here,
        // after this kernel's own loads have long been issued
        if (p.rank) {
            ptx::pdl_wait();
            for (uint32_t i = lane; i < p.M * p.rank; i += 32) t_s[i] = __ldcg(p.t + i);
        }
        __syncwarp();
        // Finish tiles in order: sum the warps' partials in a fixed order (so the result does
        // not depend on timing), add bias and the adapter term, convert, store; then hand the
        // reduction slot back and refill the tile's ring slot.
        bool ok = true;
        for (uint32_t tile = 0; tile < ntiles && ok; ++tile) {
            const uint32_t s = tile % S;
            ok = ptx::mbar_wait_bounded(bar_done + 8 * s, (tile / S) & 1u);
            if (!ok) break;
            const uint32_t row0 = n0 + tile * kTileRows;
            const uint32_t rows = min((uint32_t)kTileRows, n1 - row0);
            const float *rs = red + (tile & 1u) * red_slot_floats;
            const __nv_bfloat16 *lb = reinterpret_cast<const __nv_bfloat16 *>(
                stage_base + (size_t)s * p.stage_bytes + p.off_lora);
            for (uint32_t idx = lane; idx < (uint32_t)kTileRows * MP; idx += 32) {
                const uint32_t row = idx & 15u, m = idx >> 4;
                if (m < p.M && row < rows) {
                    float v = 0.0f;
                    for (uint32_t w = 0; w < p.consumer_warps; ++w)
                        v += rs[(w * kTileRows + row) * MP + m];
                    if (p.rank) {
                        float dot = 0.0f;
                        for (uint32_t j = 0; j < p.rank; ++j)
                            dot = fmaf(t_s[m * p.rank + j], __bfloat162float(lb[row * p.rank + j]),
                                       dot);
                        v = fmaf(dot, p.lora_scale, v);  // scale applied last
                    }
                    if (p.bias) v += __ldg(p.bias + row0 + row);
                    const size_t o = (size_t)m * p.ldy + row0 + row;
                    if (p.y_f32) static_cast<float *>(p.y)[o] = v;
                    else static_cast<__nv_bfloat16 *>(p.y)[o] = __float2bfloat16_rn(v);
                }
            }
            __syncwarp();
            if (tile < 8) NF4_TS(6 + 3 * tile);
            if (lane == 0) {
                ptx::mbar_arrive(bar_red_free + 8 * (tile & 1u));
                ptx::mbar_arrive(bar_epi_done + 8 * s);
            }
        }
        NF4_TS(3);
        if (!ok && lane == 0) atomicExch(&g_decode_error, 1);
    } else if (warp < p.consumer_warps) {
        // ========================= consumer warps =========================
        const float sos = DQ ? __ldg(p.scale_of_scales) : 0.0f;

        if (warp == 0) NF4_TS(2);
        const uint32_t *lut_lane = lut + lane;
        auto lut_at = [&](uint32_t word, int byte) -> uint32_t {
            return lut_lane[((word >> (8 * byte)) & 0xffu) << 5];
        };

        bool ok = true;
        for (uint32_t tile = 0; tile < ntiles; ++tile) {
            const uint32_t s = tile % S;
            ok = ptx::mbar_wait_bounded(bar_full + 8 * s, (tile / S) & 1u);
            if (!ok) break;
            if (warp == 0 && tile < 8) NF4_TS(4 + 3 * tile);
            const uint8_t *st = stage_base + (size_t)s * p.stage_bytes;
            const uint8_t *codes_lo = st + g * p.code_stride + t * 8;
            const uint8_t *codes_hi = codes_lo + 8 * p.code_stride;
            const uint8_t *sc_lo = st + p.off_scales + g * p.scale_stride;
            const uint8_t *sc_hi = sc_lo + 8 * p.scale_stride;

            float acc[NT][4];
            #pragma unroll
            for (int u = 0; u < NT; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;

            #pragma unroll
            for (int c = 0; c < kMaxChunksPerWarp; ++c) {
                const uint32_t kc = chunk0 + c;
                if (c < (int)p.chunks_per_warp && kc < nchunks) {
                    const uint2 w0 = *reinterpret_cast<const uint2 *>(codes_lo + kc * 32);
                    const uint2 w1 = *reinterpret_cast<const uint2 *>(codes_hi + kc * 32);
                    float s_lo, s_hi;
                    if (DQ) {
                        s_lo = dq_scale(sc_lo[kc], sos);
                        s_hi = dq_scale(sc_hi[kc], sos);
                    } else {
                        s_lo = reinterpret_cast<const float *>(sc_lo)[kc];
                        s_hi = reinterpret_cast<const float *>(sc_hi)[kc];
                    }
                    float blk[NT][4];
                    #pragma unroll
                    for (int u = 0; u < NT; ++u) blk[u][0] = blk[u][1] = blk[u][2] = blk[u][3] = 0.0f;
                    #pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t x0 = (j < 2) ? w0.x : w0.y;
                        const uint32_t x1 = (j < 2) ? w1.x : w1.y;
                        const int b = 2 * (j & 1);
                        const uint32_t a0 = lut_at(x0, b), a1 = lut_at(x1, b);
                        const uint32_t a2 = lut_at(x0, b + 1), a3 = lut_at(x1, b + 1);
                        #pragma unroll
                        for (int u = 0; u < NT; ++u)
                            ptx::mma_16816_f16(blk[u], a0, a1, a2, a3, xf[u][c][j][0],
                                               xf[u][c][j][1]);
                    }
                    #pragma unroll
                    for (int u = 0; u < NT; ++u) {
                        acc[u][0] = fmaf(blk[u][0], s_lo, acc[u][0]);
                        acc[u][1] = fmaf(blk[u][1], s_lo, acc[u][1]);
                        acc[u][2] = fmaf(blk[u][2], s_hi, acc[u][2]);
                        acc[u][3] = fmaf(blk[u][3], s_hi, acc[u][3]);
                    }
                }
            }
            if (warp == 0 && tile < 8) NF4_TS(5 + 3 * tile);
            // this warp's partial sums go to its own slice of the tile's reduction slot; the
            // slot is free once the epilogue has summed the tile two before this one
            if (tile >= 2) {
                ok = ptx::mbar_wait_bounded(bar_red_free + 8 * (tile & 1u), ((tile >> 1) - 1) & 1u);
                if (!ok) break;
            }
            float *rs = red + (tile & 1u) * red_slot_floats + warp * kTileRows * MP;
            #pragma unroll
            for (int u = 0; u < NT; ++u) {
                *reinterpret_cast<float2 *>(rs + g * MP + 8 * u + 2 * t) =
                    make_float2(acc[u][0], acc[u][1]);
                *reinterpret_cast<float2 *>(rs + (g + 8) * MP + 8 * u + 2 * t) =
                    make_float2(acc[u][2], acc[u][3]);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_done + 8 * s);
        }
        if (!ok && lane == 0) atomicExch(&g_decode_error, 2);
    }
}

// T[m][j] = sum_k x[m][k] * A[j][k]  (x, A bf16; f32 accumulate).  One CTA per (j, m).
__global__ void __launch_bounds__(128)
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
uint32_t lcm_u32(uint32_t a, uint32_t b) { return a / gcd_u32(a, b) * b; }
uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

bool plan(const nf4_linear_args &a, DecodeParams &p, uint32_t &grid, uint32_t &smem_bytes) {
    if (a.layout != NF4_LAYOUT_OUT_IN || a.io_dtype != NF4_DTYPE_BF16) return false;
    if (a.rows == 0 || a.rows > 16) return false;
    if (a.d_in % kChunk != 0 || a.d_in > (uint64_t)kMaxConsumerWarps * kMaxChunksPerWarp * kChunk)
        return false;
    if (a.d_out >= (1ull << 31)) return false;
    const bool dq = a.scale_codes != nullptr;
    const uint32_t rank = a.lora_a ? a.lora_rank : 0;
    if (rank > kMaxRank) return false;
    const void *scales = dq ? (const void *)a.scale_codes : (const void *)a.absmax;
    if (!aligned16(a.x) || !aligned16(a.packed) || !aligned16(scales)) return false;
    if (rank && !aligned16(a.lora_b)) return false;
    if (reinterpret_cast<uintptr_t>(a.y) & (a.y_f32 ? 3u : 1u)) return false;

    const uint32_t K = (uint32_t)a.d_in, N = (uint32_t)a.d_out;
    const uint32_t nchunks = K / kChunk;
    p = DecodeParams{};
    p.scale_row_bytes = nchunks * (dq ? 1u : 4u);
    uint32_t gran = 16u / gcd_u32(16u, p.scale_row_bytes);
    if (rank) gran = lcm_u32(gran, 16u / gcd_u32(16u, rank * 2u));
    if (N % gran != 0) return false;
    p.gran = gran;
    p.chunks_per_warp = (nchunks + kMaxConsumerWarps - 1) / kMaxConsumerWarps;
    p.consumer_warps = (nchunks + p.chunks_per_warp - 1) / p.chunks_per_warp;
    p.code_stride = round_up(K / 2, 128) + 32;
    p.scale_per_row = (p.scale_row_bytes % 16u == 0) ? 1u : 0u;
    p.scale_stride = p.scale_per_row ? round_up(p.scale_row_bytes, 128) + 16 : p.scale_row_bytes;
    p.off_scales = kTileRows * p.code_stride;
    p.off_lora = round_up(p.off_scales + kTileRows * p.scale_stride, 128);
    p.stage_bytes = round_up(p.off_lora + kTileRows * rank * 2u, 128);

    const uint64_t units = N / gran;
    grid = (uint32_t)(units < (uint64_t)kNumSMs ? units : (uint64_t)kNumSMs);
    const uint32_t max_rows = (uint32_t)(((units + grid - 1) / grid) * gran);
    const uint32_t max_tiles = (max_rows + kTileRows - 1) / kTileRows;
    const uint32_t mp = a.rows > 8 ? 16u : 8u;
    const uint32_t fixed = kLutBytes + 256 + 16 * kMaxRank * 4;  // lut, barriers, T
    const uint32_t red_bytes = 2u * p.consumer_warps * kTileRows * mp * 4u;  // two reduction slots
    uint32_t stages = max_tiles < (uint32_t)kMaxStages ? max_tiles : (uint32_t)kMaxStages;
    while (stages >= 1) {
        p.off_red = fixed;
        p.off_stages = round_up(p.off_red + red_bytes, 128);
        smem_bytes = p.off_stages + stages * p.stage_bytes;
        if (smem_bytes <= (uint32_t)kSmemLimit) break;
        --stages;
    }
    if (stages == 0) return false;
    p.stages = stages;
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
    p.M = (uint32_t)a.rows;
    p.K = K;
    p.N = N;
    p.rank = rank;
    p.lora_scale = a.lora_scale;
    return true;
}

template <int NT, bool DQ>
int32_t launch(const DecodeParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream) {
    static bool configured = false;  // benign race: the attribute is idempotent
    if (!configured) {
        NF4_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<NT, DQ>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
        configured = true;
    }
    count_launch();
    return launch_maybe_overlapped(decode_kernel<NT, DQ>, dim3(grid), dim3((p.consumer_warps + 2) * 32),
                                   smem_bytes, stream, p.rank != 0 && pdl_enabled(), p);
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

int32_t lora_t_small(const void *x, const void *a, uint32_t rows, uint32_t K, uint32_t rank,
                     float *t_out, cudaStream_t stream) {
    lora_t_kernel<<<dim3(rank, rows), 128, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x),
                                                         static_cast<const __nv_bfloat16 *>(a), K,
                                                         rank, t_out);
    count_launch();
    return check_cuda(cudaGetLastError(), "lora_t_kernel launch");
}

int32_t decode_forward(const nf4_linear_args &a, cudaStream_t stream) {
    DecodeParams p;
    uint32_t grid, smem;
    if (!plan(a, p, grid, smem)) return fail(NF4_ERR_UNSUPPORTED, "decode_forward: unsupported shape");
    if (p.rank) {
        float *t = static_cast<float *>(a.workspace);
        NF4_TRY(lora_t_small(a.x, a.lora_a, p.M, p.K, p.rank, t, stream));
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
        NF4_TRY(lora_t_small(a.x, a.lora_a, p.M, p.K, p.rank, t, stream));
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
