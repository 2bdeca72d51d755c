// Projection GEMMs on the 5th-generation tensor cores: C = epilogue(A * W^T), A [M,K] and W [N,K] both K-contiguous,
// 16-bit operands (bf16 or fp16), fp32 accumulation in tensor memory.
//
// Exact tier: the same pipeline with fp32 operands split into two TF32 pieces each (x = hi + lo, hi = x rounded to
// TF32, lo = x - hi rounded to TF32, what is dropped is below 2^-21 |x|).  A arrives as [lo | hi] (2K columns), W as
// [hi | lo | hi] (3K columns); the k loop runs over the 3K columns of W and takes A's hi columns a second time for
// the last third, so one accumulator sums lo*hi, then hi*lo, then hi*hi (small terms first) on kind::tf32 MMAs.  Per
// k block of 128 bytes the timeline is the one of the 16-bit kernel; there are six times as many k blocks.
//
// One persistent CTA per SM, 320 threads in three roles:
//   warp 0      TMA producer: one lane streams 128 x 64 tiles of A and BN x 64 tiles of W (128-byte swizzle) into a
//               shared-memory ring, completion counted in bytes on an mbarrier per stage
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M 128, N = BN, K 16, four per stage) from shared-memory
//               descriptors into one of two TMEM accumulators; tcgen05.commit releases the stage to the producer and,
//               after the last k block, hands the accumulator to the epilogue.  This warp also owns TMEM alloc/free.
//   warps 2-9   epilogue: warp w owns TMEM lanes 32*(w%4).. (its hardware quadrant), the two warps of a quadrant take
//               alternate 32-column blocks.  A block goes TMEM -> registers (one accumulator row per lane) -> a
//               swizzled 32 x 128-byte shared-memory tile -> global memory by a TMA tile store, which coalesces the
//               rows and clips at the matrix edge.  For the residual epilogue the same tile is first filled by a TMA
//               load of R (prefetched one block ahead), updated in place and stored back.
// The epilogue costs a few dozen instructions per block and no address arithmetic per element, so it keeps up
// with the tensor pipe; the MMA warp fills the other accumulator meanwhile.
//
// K is walked in order and never split and every output is produced by exactly one accumulator, so a row of C does
// not depend on M or on the other rows of the batch (engine/include/shv_cuda.h:31-34, engine/cuda/gemm.cuh:5-10).
// No load uses cluster multicast: weight tiles are fetched per CTA and served from L2.
//
// Every mbarrier wait is bounded.  A wait that gives up raises a CTA-wide abort flag and a device status word; all
// roles then leave their loops, the CTA waits for TMA copies that may still be in flight, frees its TMEM and returns.
// The host reads the status word (shvk_gemm_tc_status) and fails the batch.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"
#include "status_words.cuh"
#include "tc_ptx.cuh"

#include <cuda.h>
#include <stdlib.h>

#include <atomic>
#include <string.h>

namespace sb {
namespace {

constexpr int TILE_M = 128, ROW_BYTES = 128, MAX_BN = 240, ACC_COLS = 256;   // an operand stage row is 128 bytes: 64 16-bit or 32 fp32 elements
constexpr int A_BYTES = TILE_M * ROW_BYTES, B_BYTES = MAX_BN * ROW_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_TILE = 32 * 128;                               // 32 rows x 128 bytes
constexpr int BAR_BYTES = 512;
static_assert(STAGE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
// Shape of one kernel variant: operand ring depth, epilogue warps (4 or 8), output tiles in flight per epilogue warp.
template <int STAGES_, int EPI_WARPS_, int NBUF_> struct Shape {
    static constexpr int STAGES = STAGES_, EPI_WARPS = EPI_WARPS_, NBUF = NBUF_;
    static constexpr int NTHREADS = 64 + 32 * EPI_WARPS;
    static constexpr int EPI_BYTES = EPI_WARPS * NBUF * EPI_TILE;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024 /* alignment slack */;
    static_assert((2 * STAGES + 4 + EPI_WARPS * NBUF) * 8 <= BAR_BYTES && SMEM_BYTES <= 232448, "shape does not fit");
};
constexpr uint32_t SPIN_LIMIT = 1u << 22;   // polls of ~64 ns each before a wait gives up (about a quarter second)

enum : int { EPI_PLAIN = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_SPLIT16 = 3 };

__device__ int g_tc_status = 0;   // 0 ok; else 1 + role of the wait that gave up

struct TcParams {
    int M, N, K, BN, n_tiles, m_tiles;
    const float* bias;
    float r_div;
    uint32_t idesc;
    int tile_k;     // operand elements per 128-byte stage row: 64 (16-bit) or 32 (fp32 read as TF32)
    int tf32;       // 1: kind::tf32 MMAs on split fp32 operands
    int a_wrap;     // exact tier: A has a_wrap columns ([lo | hi]); k beyond them takes the second half again.  0: none
    int split_n;    // EPI_SPLIT16: columns below go to the fp16 output, the rest (fp32, + bias) to C at column n - split_n
    int m_major;    // tile order: 1 = a CTA finishes all column tiles of a row block before its next row block
    uint32_t spin_limit;   // polls before a wait gives up (SPIN_LIMIT; the starved test launch passes a small number)
    int starve;     // test launch only: the producer withholds the first operand stage of its first tile
    int probe;      // timing probes of a development build (see probe_bits): 2 no epilogue work, 4 no MMA, 8 no W load,
                    // 16 no A load, 32 column-tile-major order always, 64 padding columns left unwritten, 128 no L2 hints
};

// Timing probes exist only in a build compiled with -DSHVK_DEV_PROBES (never the shipped libraries): there the plan
// takes the bits from the SHVK_TC_PROBE environment variable.  Otherwise this is the constant 0 and every probe branch
// below is dead code, so no environment variable can change what the kernel computes.
#ifdef SHVK_DEV_PROBES
__host__ __device__ __forceinline__ int probe_bits(const TcParams& p) { return p.probe; }
#else
__host__ __device__ __forceinline__ constexpr int probe_bits(const TcParams&) { return 0; }
#endif

using namespace tc;

struct TcMaps {
    CUtensorMap a, w;             // operands, 128-byte swizzle
    CUtensorMap c_full, c_half;   // output: boxes of 32 rows x (32 | 16) accumulator columns
    CUtensorMap r_full, r_half;   // EPI_RESID: residual input (fp32), same boxes; EPI_SPLIT16: the fp16 output, dense boxes
};

// Writes one epilogue block into its shared-memory tile.  Lane = accumulator row, r = its 32 (or 16) fp32 columns.
//   fp32 tiles, 32 columns: 128-byte rows, 16-byte chunk j of row l at chunk j ^ (l & 7) (the TMA 128-byte swizzle,
//                           which also makes these stores bank-conflict free); 16 columns: dense 64-byte rows
//   EPI_RESID: the tile already holds R (TMA load); v = R + acc / r_div overwrites it in place
//   EPI_SPLIT16: blocks left of split_n are rounded to fp16 (saturating) into dense 64-byte (32-byte) rows; the others
//               are plain fp32 blocks (+ bias)
//   EPI_SWIGLU: adjacent accumulator columns are (gate, up): silu(gate) * up in storage type T, dense rows (16-bit T:
//               hardware exp; T = float, the exact tier: expf and a true division, 64-byte rows)
template <typename T, int EPI>
__device__ __forceinline__ void stage_block(const TcParams& p, uint32_t tile, int lane, bool full, int n, const uint32_t* r) {
    if (EPI == EPI_SPLIT16 && n < p.split_n) {
        const uint32_t row = tile + uint32_t(lane) * (full ? 64u : 32u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < 2 || full) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(o[e]) : "f"(__uint_as_float(r[8 * j + 2 * e + 1])),
                        "f"(__uint_as_float(r[8 * j + 2 * e])));
                }
                sts128u(row + 16u * j, o[0], o[1], o[2], o[3]);
            }
        }
    } else if constexpr (EPI == EPI_SWIGLU && sizeof(T) == 4) {
        const uint32_t row = tile + uint32_t(lane) * (full ? 64u : 32u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < 2 || full) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = silu_f(__uint_as_float(r[8 * j + 2 * e])) * __uint_as_float(r[8 * j + 2 * e + 1]);
                sts128(row + 16u * j, v[0], v[1], v[2], v[3]);
            }
        }
    } else if constexpr (EPI == EPI_SWIGLU) {
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < 4 || full) {
                // hardware exp / reciprocal: the product is rounded to 16 bits right after
                const float g0 = __uint_as_float(r[4 * j]), g1 = __uint_as_float(r[4 * j + 2]);
                const float a = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(r[4 * j + 1]);
                const float b = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(r[4 * j + 3]);
                o[j] = pack2<T>(a, b);
            }
        }
        if (full) {
            sts128u(tile + lane * 32, o[0], o[1], o[2], o[3]);
            sts128u(tile + lane * 32 + 16, o[4], o[5], o[6], o[7]);
        } else {
            sts128u(tile + lane * 16, o[0], o[1], o[2], o[3]);
        }
    } else {
        const uint32_t row = tile + uint32_t(lane) * (full ? 128u : 64u);
        const uint32_t sw = full ? uint32_t(lane & 7) : 0u;
        float4 rr[8];
        if constexpr (EPI == EPI_RESID) {
            // all residual loads first: a store in between would hold back every load behind it
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (j < 4 || full) rr[j] = lds128(row + ((uint32_t(j) ^ sw) << 4));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < 4 || full) {
                const uint32_t addr = row + ((uint32_t(j) ^ sw) << 4);
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                       __uint_as_float(r[4 * j + 3]));
                if constexpr (EPI == EPI_RESID) {
                    if (p.r_div != 1.0f) {
                        v.x = rr[j].x + v.x / p.r_div; v.y = rr[j].y + v.y / p.r_div; v.z = rr[j].z + v.z / p.r_div; v.w = rr[j].w + v.w / p.r_div;
                    } else {
                        v.x = rr[j].x + v.x; v.y = rr[j].y + v.y; v.z = rr[j].z + v.z; v.w = rr[j].w + v.w;
                    }
                } else if (p.bias) {
                    if (n + 4 * j < p.N) {
                        const float4 b = *reinterpret_cast<const float4*>(p.bias + n + 4 * j);
                        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                    }
                }
                sts128(addr, v.x, v.y, v.z, v.w);
            }
        }
    }
}

// The it-th tile of this CTA; false past the end.  Row-block-major order (m_major) lets one CTA write whole rows of
// C within a few tiles' time, which DRAM takes about a third faster than column tiles of many row blocks interleaved.
__device__ __forceinline__ bool tile_at(const TcParams& p, long long it, int& mt, int& nt) {
    if (p.m_major) {
        const long long round = it / p.n_tiles;
        const long long m = round * gridDim.x + blockIdx.x;
        nt = int(it - round * p.n_tiles);
        mt = int(m);
        return m < p.m_tiles;
    }
    const long long tile = blockIdx.x + it * gridDim.x;
    mt = int(tile / p.n_tiles);
    nt = int(tile - (long long)mt * p.n_tiles);
    return tile < (long long)p.m_tiles * p.n_tiles;
}

template <typename T, int EPI, typename SH>
__global__ void __launch_bounds__(SH::NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ TcMaps maps, const TcParams p) {
    constexpr int STAGES = SH::STAGES, EPI_WARPS = SH::EPI_WARPS, NBUF = SH::NBUF, EPI_BYTES = SH::EPI_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_base = base + STAGES * STAGE_BYTES;       // output tiles of 4 KB, 1024-byte aligned
    const uint32_t bars = epi_base + EPI_BYTES;                  // full[S], empty[S], acc_full[2], acc_empty[2], r[8][2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto accf_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acce_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    auto r_bar = [&](int ew, int b) { return bars + 8u * (2 * STAGES + 4 + NBUF * ew + b); };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), EPI_WARPS); }
        for (int e = 0; e < EPI_WARPS; ++e)
            for (int b = 0; b < NBUF; ++b) mbar_init(r_bar(e, b), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abortp = &abort_flag;

    const int nk = p.K / p.tile_k;
    const uint32_t stage_tx = uint32_t(A_BYTES + p.BN * ROW_BYTES);

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int mt, nt;
            const uint64_t pol_w = policy_evict_last();
            const bool hint = !(probe_bits(p) & 128);
            for (long long it = 0; ok && tile_at(p, it, mt, nt); ++it) {
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                    if (p.starve && it == 0 && kb == 0) {           // test launch: this stage never fills
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                    const int kw = kb * p.tile_k;
                    const int ka = p.a_wrap && kw >= p.a_wrap ? kw - (p.a_wrap >> 1) : kw;
                    const bool la = !(probe_bits(p) & 16), lw = !(probe_bits(p) & 8);
                    if (la || lw) {
                        mbar_expect_tx(full_bar(stage), (la ? uint32_t(A_BYTES) : 0u) + (lw ? stage_tx - uint32_t(A_BYTES) : 0u));
                        if (la) tma_load_2d(sa, &maps.a, ka, mt * TILE_M, full_bar(stage));
                        if (lw) {
                            if (hint) tma_load_2d_hint(sb_, &maps.w, kw, nt * p.BN, full_bar(stage), pol_w);
                            else tma_load_2d(sb_, &maps.w, kw, nt * p.BN, full_bar(stage));
                        }
                    } else {
                        mbar_arrive(full_bar(stage));
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(&g_tc_status, 0, 1); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            int mt, nt;
            for (long long it = 0; ok && tile_at(p, it, mt, nt); ++it) {
                if (!mbar_wait(acce_bar(acc), acc_phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc * ACC_COLS);
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abortp, p.spin_limit)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb_);
                    if (p.tf32) {
#pragma unroll
                        for (int k = 0; k < ROW_BYTES / 32; ++k)       // 8 fp32 elements = 32 bytes = 2 descriptor units
                            tc_mma_tf32(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc, uint32_t((kb | k) != 0));
                    } else {
#pragma unroll
                        for (int k = 0; k < ROW_BYTES / 32; ++k)       // 16 elements = 32 bytes = 2 descriptor units
                            if (!(probe_bits(p) & 4)) tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc, uint32_t((kb | k) != 0));
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(accf_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(&g_tc_status, 0, 2); }
        }
    } else {
        // ------------------------------------------------------------------------------------------ epilogue
        constexpr int PER_QUAD = EPI_WARPS / 4;                      // warps sharing a TMEM quadrant take alternate blocks
        const int ew = warp - 2, quad = warp & 3, half = ew >> 2;
        const int nblk = (p.BN + 31) >> 5;
        uint32_t tiles[NBUF], rbars[NBUF], rphase[NBUF];
#pragma unroll
        for (int i = 0; i < NBUF; ++i) {
            tiles[i] = epi_base + uint32_t(NBUF * ew + i) * EPI_TILE;
            rbars[i] = r_bar(ew, i);
            rphase[i] = 0u;
        }
        const bool active = half < nblk && !(probe_bits(p) & 2);          // this warp has blocks to write
        const uint64_t pol_c = policy_evict_first();
        const bool hint = !(probe_bits(p) & 128);
        uint32_t nb = 0;                                            // blocks done by this warp; tile buffer = nb % NBUF
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        // lane 0 only: TMA load of R for block (tile, blk) into tile buffer b
        auto load_r = [&](int mt, int nt, int blk, int b) {
            const int c = blk << 5;
            const bool full = p.BN - c >= 32;
            mbar_expect_tx(rbars[b], full ? 4096u : 2048u);
            tma_load_2d(tiles[b], full ? &maps.r_full : &maps.r_half, nt * p.BN + c, mt * TILE_M + quad * 32, rbars[b]);
        };
        int mt, nt;
        if (EPI == EPI_RESID && active && lane == 0 && tile_at(p, 0, mt, nt)) load_r(mt, nt, half, 0);

        for (long long it = 0; ok && tile_at(p, it, mt, nt); ++it) {
            if (!mbar_wait(accf_bar(acc), acc_phase, abortp, p.spin_limit)) { ok = false; break; }
            tc_fence_after();
            const int m0 = mt * TILE_M + quad * 32;
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * ACC_COLS);
            uint32_t ra[32], rb[32];
            auto fetch = [&](int blk, uint32_t* r) {
                const int c = blk << 5;
                tc_ld16(taddr + uint32_t(c), r);
                if (p.BN - c >= 32) tc_ld16(taddr + uint32_t(c + 16), r + 16);
            };
            // one block: (prefetch the next R), wait for R / for the tile buffer, stage, TMA store
            auto emit = [&](int blk, const uint32_t* r) -> bool {
                const int b = int(nb % uint32_t(NBUF)), bn_ = int((nb + 1u) % uint32_t(NBUF));
                const int c = blk << 5;
                const bool full = p.BN - c >= 32;
                const int n = nt * p.BN + c;
                if constexpr (EPI == EPI_RESID) {
                    if (lane == 0) {
                        int mt2 = mt, nt2 = nt, nblk2 = blk + PER_QUAD;
                        bool more = true;
                        if (nblk2 >= nblk) { more = tile_at(p, it + 1, mt2, nt2); nblk2 = half; }
                        if (more) {
                            bulk_wait_read<NBUF - 2>();           // the store that last read the next buffer is done with it
                            load_r(mt2, nt2, nblk2, bn_);
                        }
                    }
                    if (!mbar_wait(rbars[b], rphase[b], abortp, p.spin_limit)) return false;
                    rphase[b] ^= 1u;
                } else {
                    if (lane == 0) bulk_wait_read<NBUF - 1>();    // the store that last used this buffer has left it
                    __syncwarp();
                }
                stage_block<T, EPI>(p, tiles[b], lane, full, n, r);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    const bool low = EPI == EPI_SPLIT16 && n < p.split_n;         // this block goes to the fp16 output
                    const int x = EPI == EPI_SWIGLU ? (n >> 1) : (EPI == EPI_SPLIT16 && !low ? n - p.split_n : n);
                    const CUtensorMap* cm = low ? (full ? &maps.r_full : &maps.r_half) : (full ? &maps.c_full : &maps.c_half);
                    if (hint) tma_store_2d_hint(cm, x, m0, tiles[b], pol_c);
                    else tma_store_2d(cm, x, m0, tiles[b]);
                    bulk_commit();
                }
                ++nb;
                return true;
            };
            if (active) {
                int blk = half;
                fetch(blk, ra);
                while (true) {
                    tc_wait_ld();
                    if (blk + PER_QUAD < nblk) fetch(blk + PER_QUAD, rb);
                    if (!emit(blk, ra)) { ok = false; break; }
                    blk += PER_QUAD;
                    if (blk >= nblk) break;
                    tc_wait_ld();
                    if (blk + PER_QUAD < nblk) fetch(blk + PER_QUAD, ra);
                    if (!emit(blk, rb)) { ok = false; break; }
                    blk += PER_QUAD;
                    if (blk >= nblk) break;
                }
                if (!ok) break;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (lane == 0) bulk_wait_all();                             // stores must have left shared memory before exit
        if (!ok && lane == 0 && !*abortp) { *abortp = 1; atomicCAS(&g_tc_status, 0, 3); }
    }

    __syncthreads();
    if (abort_flag) {
        // A role gave up: copies already issued may still land in this CTA's shared memory.  Give them time (bounded)
        // before the block retires; nothing here waits on another thread.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return EncodeTiledFn(nullptr);
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// Row-major matrix [rows][cols] of elem_bytes-wide elements, row pitch ld elements, box box_rows x box_cols.
bool make_map(CUtensorMap* map, const void* ptr, int elem_bytes, long long rows, long long cols, long long ld, int box_rows,
              int box_cols, bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(ld) * cuuint64_t(elem_bytes)};
    const cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    // 16-bit operands (bf16 or fp16 alike) travel as opaque 16-bit elements
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct HostPlan {
    CUtensorMap map_a, map_w;       // 128 bytes each, 64-byte aligned
    TcParams p;
    void* C; long long ldc; int c_dtype;
    const float* R; long long ldr;
    void* C16; long long ldc16;     // EPI_SPLIT16: the fp16 output
    int epi, ab_dtype, valid;
};
static_assert(sizeof(HostPlan) <= 512, "plan must fit the caller's 512-byte buffer");

// Accumulator width (multiple of 16, 64..240) with the least time per row block.  Per 16-deep k step one MMA costs
// bn/2 tensor cycles and moves 32*(128+bn) bytes out of shared memory at 128 bytes per cycle, so a tile costs
// max(bn/2, (128+bn)/4); padded columns of the last tile count in full.  Ties go to the wider tile.
int choose_bn(int n) {
    int best = MAX_BN;
    long long best_cost = -1;
    for (int bn = MAX_BN; bn >= 64; bn -= 16) {
        const long long tiles = (n + bn - 1) / bn;
        const long long per_tile = 2 * bn > 128 + bn ? 2 * bn : 128 + bn;    // 4 x max(bn/2, (128+bn)/4)
        const long long cost = tiles * per_tile;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <typename T, int EPI, typename SH> int launch_tc(const TcMaps& maps, const TcParams& p, cudaStream_t s) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    // one bit per device ordinal: the dynamic shared memory opt-in is per device.  Engines of several devices launch
    // from their own threads, hence the atomic; setting the attribute twice is harmless.
    static std::atomic<unsigned long long> attr_done{0};
    if (dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<T, EPI, SH>, cudaFuncAttributeMaxDynamicSharedMemorySize, SH::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        if (dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long total = (long long)p.m_tiles * p.n_tiles;
    const unsigned grid = unsigned(total < sms ? total : sms);
    TcParams q = p;
    // whole row blocks per CTA once there are enough of them to keep every SM equally busy (under 1/8 idle at the tail)
    q.m_major = p.n_tiles > 1 && p.m_tiles >= 8ll * grid && !(probe_bits(p) & 32);
    gemm_tc_kernel<T, EPI, SH><<<grid, SH::NTHREADS, SH::SMEM_BYTES, s>>>(maps, q);
    return int(cudaGetLastError());
}

// Three operand stages, eight epilogue warps, two output tiles in flight per warp.  Measured on the in-projection
// shape (M = 657k, N = 2316, K = 384): <3,8,2> 1.72 ms, <3,4,4> 1.66 ms, <2,8,4> 1.99 ms, so the epilogue is not limited
// by its own pipeline depth, and a two-stage operand ring starves the tensor pipe.
using ShapeDefault = Shape<3, 8, 2>;

}  // namespace
}  // namespace sb

static int plan_impl(const shvk_gemm_args* g, int ab_dtype, void* host_plan, int split_col, void* C16, long long ldc16);

extern "C" int shvk_gemm_tc_plan(const shvk_gemm_args* g, int ab_dtype, void* host_plan) {
    return plan_impl(g, ab_dtype, host_plan, 0, nullptr, 0);
}

extern "C" int shvk_gemm_tc_plan_split16(const shvk_gemm_args* g, int ab_dtype, int split_col, void* C16, long long ldc16,
                                         void* host_plan) {
    // columns [0, split_col) leave as fp16 rows of C16, the rest as fp32 (+ bias) at column n - split_col of C
    if (!g || !C16 || split_col <= 0 || split_col >= g->N || (split_col & 31) || (ldc16 & 7) || ldc16 < split_col ||
        (reinterpret_cast<uintptr_t>(C16) & 15) || g->swiglu || g->R || g->c_dtype != sb::DT_F32 || ab_dtype == sb::DT_F32)
        return int(cudaErrorInvalidValue);
    return plan_impl(g, ab_dtype, host_plan, split_col, C16, ldc16);
}

static int plan_impl(const shvk_gemm_args* g, int ab_dtype, void* host_plan, int split_col, void* C16, long long ldc16) {
    using namespace sb;
    if (!g || !host_plan || (reinterpret_cast<uintptr_t>(host_plan) & 63)) return int(cudaErrorInvalidValue);
    if (ab_dtype != DT_BF16 && ab_dtype != DT_F16 && ab_dtype != DT_F32) return int(cudaErrorInvalidValue);
    const bool split = ab_dtype == DT_F32;              // exact tier: A = [lo | hi] (2K fp32), W = [hi | lo | hi] (3K fp32)
    const int tile_k = split ? 32 : 64;
    const int align = split ? 3 : 7;                    // 16-byte pitches
    if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->K % tile_k || (g->lda & align) || (g->ldw & align) || (g->N & 3) ||
        (split && (g->lda < 2ll * g->K || g->ldw < 3ll * g->K)) ||
        ((reinterpret_cast<uintptr_t>(g->A) | reinterpret_cast<uintptr_t>(g->W) | reinterpret_cast<uintptr_t>(g->C)) & 15) ||
        (g->R && ((g->ldr & 3) || (reinterpret_cast<uintptr_t>(g->R) & 15))) || g->act != 0)
        return int(cudaErrorInvalidValue);
    // supported epilogues: fp32 C (+ bias), fp32 C = R + acc / r_div, SwiGLU into 16-bit C (fp32 C in the exact tier)
    int epi;
    if (g->swiglu) {
        if ((g->N & 7) || (g->c_dtype == DT_F32) != split || g->R || g->bias || (g->ldc & (split ? 3 : 7))) return int(cudaErrorInvalidValue);
        epi = EPI_SWIGLU;
    } else {
        if (g->c_dtype != DT_F32 || (g->ldc & 3) || (g->R && g->bias)) return int(cudaErrorInvalidValue);
        epi = g->R ? EPI_RESID : (split_col ? EPI_SPLIT16 : EPI_PLAIN);
    }
    HostPlan* hp = static_cast<HostPlan*>(host_plan);
    memset(hp, 0, sizeof(HostPlan));
    const int bn = choose_bn(g->N);
    const int eb = split ? 4 : 2;
    if (!make_map(&hp->map_a, g->A, eb, g->M, split ? 2ll * g->K : g->K, g->lda, TILE_M, tile_k, true)) return int(cudaErrorNotSupported);
    if (!make_map(&hp->map_w, g->W, eb, g->N, split ? 3ll * g->K : g->K, g->ldw, bn, tile_k, true)) return int(cudaErrorNotSupported);
    TcParams& p = hp->p;
    p.M = g->M; p.N = g->N; p.K = split ? 3 * g->K : g->K; p.BN = bn;
    p.tile_k = tile_k; p.tf32 = split ? 1 : 0; p.a_wrap = split ? 2 * g->K : 0;
    p.n_tiles = (g->N + bn - 1) / bn;
    p.m_tiles = (g->M + TILE_M - 1) / TILE_M;
    p.bias = g->bias;
    p.r_div = g->r_div == 0.0f ? 1.0f : g->r_div;
    const uint32_t fmt = split ? 2u : (ab_dtype == DT_BF16 ? 1u : 0u);      // f16 0, bf16 1, tf32 2
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), both K-major, N/8 at bit 17,
    // M/16 at bit 24
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(TILE_M >> 4) << 24);
#ifdef SHVK_DEV_PROBES
    { const char* e = getenv("SHVK_TC_PROBE"); p.probe = e ? atoi(e) : 0; }
#else
    p.probe = 0;
#endif
    p.spin_limit = SPIN_LIMIT;
    p.starve = 0;
    hp->C = g->C; hp->ldc = g->ldc; hp->c_dtype = g->c_dtype;
    hp->R = g->R; hp->ldr = g->ldr;
    hp->C16 = C16; hp->ldc16 = ldc16;
    p.split_n = split_col;
    if (split_col && (bn & 31)) return int(cudaErrorInvalidValue);      // a 32-column block must not straddle the split
    hp->epi = epi;
    hp->ab_dtype = ab_dtype;
    hp->valid = 0x5b200;
    return 0;
}

// `rows` <= the M the plan was made for; rows beyond `rows` are neither read for the residual nor written (the output
// tensor maps are encoded for exactly `rows` rows, so the TMA stores clip there).
namespace sb {
namespace {
int launch_rows(const void* host_plan, int rows, void* stream, int starve, uint32_t spin_limit) {
    const HostPlan* hp = static_cast<const HostPlan*>(host_plan);
    if (!hp || hp->valid != 0x5b200 || rows > hp->p.M) return int(cudaErrorInvalidValue);
    if (rows <= 0) return 0;
    TcParams p = hp->p;
    p.starve = starve;
    p.spin_limit = spin_limit;
    p.M = rows;
    p.m_tiles = (rows + TILE_M - 1) / TILE_M;
    TcMaps maps;
    maps.a = hp->map_a;
    maps.w = hp->map_w;
    bool ok;
    if (hp->epi == EPI_SWIGLU) {
        const int cb = hp->c_dtype == DT_F32 ? 4 : 2;
        ok = make_map(&maps.c_full, hp->C, cb, rows, p.N / 2, hp->ldc, 32, 16, false) &&
             make_map(&maps.c_half, hp->C, cb, rows, p.N / 2, hp->ldc, 32, 8, false);
        maps.r_full = maps.c_full;
        maps.r_half = maps.c_half;
    } else {
        // up to seven padding columns right of N are written too where the last column tile covers them (zeros: the
        // weight rows there read as zero fill); a row that ended inside a 32-byte sector would cost a DRAM
        // read-modify-write per row
        const int n_c = p.N - (hp->epi == EPI_SPLIT16 ? p.split_n : 0);        // columns that go to C
        const bool pad = (hp->epi == EPI_PLAIN || hp->epi == EPI_SPLIT16) && hp->ldc - n_c < 8 &&
                         hp->ldc - n_c <= (long long)p.n_tiles * p.BN - p.N && !(probe_bits(p) & 64);
        const long long c_cols = pad ? hp->ldc : n_c;
        ok = make_map(&maps.c_full, hp->C, 4, rows, c_cols, hp->ldc, 32, 32, true) &&
             make_map(&maps.c_half, hp->C, 4, rows, c_cols, hp->ldc, 32, 16, false);
        if (hp->epi == EPI_RESID)
            ok = ok && make_map(&maps.r_full, hp->R, 4, rows, p.N, hp->ldr, 32, 32, true) &&
                 make_map(&maps.r_half, hp->R, 4, rows, p.N, hp->ldr, 32, 16, false);
        else if (hp->epi == EPI_SPLIT16)
            ok = ok && make_map(&maps.r_full, hp->C16, 2, rows, p.split_n, hp->ldc16, 32, 32, false) &&
                 make_map(&maps.r_half, hp->C16, 2, rows, p.split_n, hp->ldc16, 32, 16, false);
        else { maps.r_full = maps.c_full; maps.r_half = maps.c_half; }
    }
    if (!ok) return int(cudaErrorNotSupported);
    cudaStream_t s = cudaStream_t(stream);
    if (hp->epi == EPI_PLAIN) return launch_tc<float, EPI_PLAIN, ShapeDefault>(maps, p, s);
    if (hp->epi == EPI_SPLIT16) return launch_tc<float, EPI_SPLIT16, ShapeDefault>(maps, p, s);
    if (hp->epi == EPI_RESID) return launch_tc<float, EPI_RESID, ShapeDefault>(maps, p, s);
    if (hp->c_dtype == DT_F32) return launch_tc<float, EPI_SWIGLU, ShapeDefault>(maps, p, s);
    if (hp->c_dtype == DT_BF16) return launch_tc<__nv_bfloat16, EPI_SWIGLU, ShapeDefault>(maps, p, s);
    return launch_tc<__half, EPI_SWIGLU, ShapeDefault>(maps, p, s);
}
}  // namespace
}  // namespace sb

extern "C" int shvk_gemm_tc_rows(const void* host_plan, int rows, void* stream) {
    return sb::launch_rows(host_plan, rows, stream, 0, sb::SPIN_LIMIT);
}

// Test launch: every CTA's producer withholds the first operand stage of its first tile, so the MMA role's wait on
// that stage runs out after `polls` polls (clamped to 256 .. 2^22); the CTA then takes its abort path (status word
// set, roles leave, copies in flight given time to land, tensor memory freed) and returns.  C is left partly written.
extern "C" int shvk_gemm_tc_rows_starved(const void* host_plan, int rows, int polls, void* stream) {
    const uint32_t lim = polls < 256 ? 256u : (uint32_t(polls) > sb::SPIN_LIMIT ? sb::SPIN_LIMIT : uint32_t(polls));
    return sb::launch_rows(host_plan, rows, stream, 1, lim);
}

extern "C" int shvk_gemm_tc(const void* host_plan, void* stream) {
    const sb::HostPlan* hp = static_cast<const sb::HostPlan*>(host_plan);
    if (!hp) return int(cudaErrorInvalidValue);
    return shvk_gemm_tc_rows(host_plan, hp->p.M, stream);
}

extern "C" int shvk_gemm_tc_status(int* status_out) {
    int v = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&v, sb::g_tc_status, sizeof(int));
    if (status_out) *status_out = v;
    return int(e);
}

namespace sb {
// Device address of this file's status word on the current device (looked up per call: it is cheap and stays right
// across a device reset).
int* gemm_tc_status_word() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_tc_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
}  // namespace sb
