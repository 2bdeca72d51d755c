// Projection GEMMs on the 5th-generation tensor cores: C = epilogue(A * W^T), A [M,K] and W [N,K] both K-contiguous,
// 16-bit operands (bf16 or fp16), fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, 320 threads in three roles:
//   warp 0      TMA producer: one lane streams 128 x 64 tiles of A and BN x 64 tiles of W (128-byte swizzle) into a
//               4-deep shared-memory ring, completion counted in bytes on an mbarrier per stage
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M 128, N = BN, K 16, four per stage) from shared-memory
//               descriptors into one of two TMEM accumulators; tcgen05.commit releases the stage to the producer and,
//               after the last k block, hands the accumulator to the epilogue.  This warp also owns TMEM alloc/free.
//   warps 2-9   epilogue: warp w reads TMEM lanes 32*(w%4).. (its hardware quadrant; two warps per quadrant take
//               alternate 32-column blocks), transposes each block through shared memory, applies bias / SiLU /
//               residual / SwiGLU and writes C coalesced, while the MMA warp already fills the other accumulator.
// K is walked in order and never split and every output is produced by exactly one accumulator, so a row of C does
// not depend on M or on the other rows of the batch (engine/include/shv_cuda.h:31-34, engine/cuda/gemm.cuh:5-10).
// No load uses cluster multicast: weight tiles are fetched per CTA and served from L2.
//
// Every mbarrier wait is bounded.  A wait that gives up raises a CTA-wide abort flag and a device status word; all
// roles then leave their loops, the CTA waits for TMA copies that may still be in flight, frees its TMEM and returns.
// The host reads the status word (shvk_gemm_tc_status) and fails the batch.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

namespace sb {
namespace {

constexpr int TILE_M = 128, TILE_K = 64, MAX_BN = 240, ACC_COLS = 256, STAGES = 4, EPI_WARPS = 8, NTHREADS = 64 + 32 * EPI_WARPS;
constexpr int A_BYTES = TILE_M * TILE_K * 2, B_BYTES = MAX_BN * TILE_K * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGE_PITCH = 36;                                  // floats per staged row: 16-byte aligned, conflict-free
constexpr int EPI_BYTES = EPI_WARPS * 32 * STAGE_PITCH * 4;      // one 32 x 32 fp32 transpose buffer per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + EPI_BYTES;
constexpr uint32_t SPIN_LIMIT = 1u << 22;   // polls of ~64 ns each before a wait gives up (about a quarter second)

__device__ int g_tc_status = 0;   // 0 ok; else 1 + role of the wait that gave up

struct TcParams {
    int M, N, K, BN, n_tiles, m_tiles;
    void* C; long long ldc; int c_dtype;
    const float* bias; int act;
    const float* R; long long ldr; float r_div;
    int swiglu;
    uint32_t idesc;
    int probe;      // timing probes (SHVK_TC_PROBE, development only): 1 no global stores, 2 no epilogue work, 4 no MMA, 8 no W load, 16 no A load
};

// ---------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the phase did not complete within the poll budget or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored with the 128-byte swizzle: rows of 128 bytes, groups of
// 8 rows 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= uint64_t((addr & 0x3ffffu) >> 4);           // start address, bits [0,14)
    d |= uint64_t(1) << 16;                          // leading byte offset (16-byte units), bits [16,30)
    d |= uint64_t(1024 >> 4) << 32;                  // stride byte offset, bits [32,46)
    d |= uint64_t(1) << 46;                          // version, bits [46,48)
    d |= uint64_t(2) << 61;                          // SWIZZLE_128B, bits [61,64)
    return d;
}

// Epilogue of one 32-row x (16 or 32)-column block held by one warp, one accumulator row per lane.  The block is
// transposed through the warp's private shared-memory buffer so that global traffic is coalesced: in the second phase
// a lane owns four consecutive columns and eight lanes cover a row, so every 128-bit access of a warp touches whole
// 32-byte sectors of four rows (a lane-per-row store would touch 32 rows with 16 bytes each).
template <typename T>
__device__ __forceinline__ void epilogue_block(const TcParams& p, float* stage, long long m0, int n0, int ncols, int lane,
                                               const uint32_t (&r)[32]) {
    float* mine = stage + lane * STAGE_PITCH;
    if (p.swiglu) {
        // (gate, up) pairs sit in adjacent accumulator columns of this lane's row: combine before the transpose
        const int nout = ncols >> 1;                                  // 8 or 16 outputs per row
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (4 * q < nout) {
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    o[j] = silu_f(__uint_as_float(r[8 * q + 2 * j])) * __uint_as_float(r[8 * q + 2 * j + 1]);
                *reinterpret_cast<float4*>(mine + 4 * q) = make_float4(o[0], o[1], o[2], o[3]);
            }
        }
        __syncwarp();
        const int lanes_per_row = nout >> 2;                          // 2 or 4 lanes of four outputs
        const int rows_per_pass = 32 / lanes_per_row;
        const int sub = lane % lanes_per_row, rsel = lane / lanes_per_row;
        const int col = (n0 >> 1) + 4 * sub;                          // output column
        for (int r0 = 0; r0 < 32; r0 += rows_per_pass) {
            const int row = r0 + rsel;
            const long long m = m0 + row;
            if (m < p.M && 2 * col < p.N) {
                const float4 v = *reinterpret_cast<const float4*>(stage + row * STAGE_PITCH + 4 * sub);
                store_quad<T>(static_cast<T*>(p.C) + m * p.ldc + col, v.x, v.y, v.z, v.w);
            }
        }
        __syncwarp();
        return;
    }
#pragma unroll
    for (int q = 0; q < 8; ++q)
        if (4 * q < ncols)
            *reinterpret_cast<float4*>(mine + 4 * q) = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                   __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
    __syncwarp();
    const int lanes_per_row = ncols >> 2;                             // 4 or 8
    const int rows_per_pass = 32 / lanes_per_row;
    const int sub = lane % lanes_per_row, rsel = lane / lanes_per_row;
    const int n = n0 + 4 * sub;
    const bool col_ok = n < p.N;                                      // N is a multiple of 4: a quad is all in or all out
    float4 bias = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (p.bias && col_ok) bias = *reinterpret_cast<const float4*>(p.bias + n);
    // residual rows first, all passes at once: R may alias C, so the compiler cannot move these loads above the stores
    // of an earlier pass by itself, and one dependent global load per pass would serialise on memory latency
    float4 res[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        res[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const int row = k * rows_per_pass + rsel;
        const long long m = m0 + row;
        if (p.R && k * rows_per_pass < 32 && m < p.M && col_ok) res[k] = *reinterpret_cast<const float4*>(p.R + m * p.ldr + n);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int row = k * rows_per_pass + rsel;
        const long long m = m0 + row;
        if (k * rows_per_pass < 32 && m < p.M && col_ok) {
            float4 v = *reinterpret_cast<const float4*>(stage + row * STAGE_PITCH + 4 * sub);
            v.x += bias.x; v.y += bias.y; v.z += bias.z; v.w += bias.w;
            if (p.act == 1) { v.x = silu_f(v.x); v.y = silu_f(v.y); v.z = silu_f(v.z); v.w = silu_f(v.w); }
            if (p.R) {
                const float4 rr = res[k];
                if (p.r_div != 1.0f) {
                    v.x = rr.x + v.x / p.r_div; v.y = rr.y + v.y / p.r_div; v.z = rr.z + v.z / p.r_div; v.w = rr.w + v.w / p.r_div;
                } else {
                    v.x = rr.x + v.x; v.y = rr.y + v.y; v.z = rr.z + v.z; v.w = rr.w + v.w;
                }
            }
            if (!(p.probe & 1)) store_quad<T>(static_cast<T*>(p.C) + m * p.ldc + n, v.x, v.y, v.z, v.w);
        }
    }
    __syncwarp();
}

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;           // full[4], empty[4], acc_full[2], acc_empty[2]
    const uint32_t epi_base = bars + 256;                        // four per-warp transpose buffers
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto accf_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acce_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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

    const int nk = p.K / TILE_K;
    const long long total = (long long)p.m_tiles * p.n_tiles;
    const uint32_t stage_tx = uint32_t(A_BYTES + p.BN * TILE_K * 2);

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                const int mt = int(tile / p.n_tiles), nt = int(tile - (long long)mt * p.n_tiles);
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) { ok = false; break; }
                    const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                    const bool la = !(p.probe & 16), lw = !(p.probe & 8);
                    if (la || lw) {
                        mbar_expect_tx(full_bar(stage), (la ? uint32_t(A_BYTES) : 0u) + (lw ? stage_tx - uint32_t(A_BYTES) : 0u));
                        if (la) tma_load_2d(sa, &map_a, kb * TILE_K, mt * TILE_M, full_bar(stage));
                        if (lw) tma_load_2d(sb_, &map_w, kb * TILE_K, nt * p.BN, full_bar(stage));
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
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                if (!mbar_wait(acce_bar(acc), acc_phase ^ 1u, abortp)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc * ACC_COLS);
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abortp)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb_);
#pragma unroll
                    for (int k = 0; k < TILE_K / 16; ++k)          // 16 elements = 32 bytes = 2 descriptor units
                        if (!(p.probe & 4)) tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc, uint32_t((kb | k) != 0));
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
        const int quad = warp & 3;                                  // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            const int mt = int(tile / p.n_tiles), nt = int(tile - (long long)mt * p.n_tiles);
            if (!mbar_wait(accf_bar(acc), acc_phase, abortp)) { ok = false; break; }
            tc_fence_after();
            const long long m0 = (long long)mt * TILE_M + quad * 32;
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * ACC_COLS);
            float* stage = reinterpret_cast<float*>(smem_raw + (epi_base - smem_u32(smem_raw))) + (warp - 2) * 32 * STAGE_PITCH;
            // The two warps of a quadrant take alternate 32-column blocks.  The TMEM read of the next block is issued
            // before the current one is transposed and written, so its latency hides behind the stores.
            const int nblk = (p.BN + 31) >> 5;
            const int half = (warp - 2) >> 2;
            uint32_t ra[32], rb[32];
            auto fetch = [&](int blk, uint32_t (&r)[32]) {
                const int c = blk << 5;
                if (p.probe & 32) return;
                tc_ld16(taddr + uint32_t(c), *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
                if (p.BN - c >= 32) tc_ld16(taddr + uint32_t(c + 16), *reinterpret_cast<uint32_t(*)[16]>(&r[16]));
            };
            auto emit = [&](int blk, const uint32_t (&r)[32]) {
                const int c = blk << 5;
                if (p.probe & 64) return;
                epilogue_block<T>(p, stage, m0, nt * p.BN + c, p.BN - c >= 32 ? 32 : 16, lane, r);
            };
            int blk = (p.probe & 2) ? nblk : half;
            if (blk < nblk) fetch(blk, ra);
            while (blk < nblk) {
                tc_wait_ld();
                if (blk + 2 < nblk) fetch(blk + 2, rb);
                emit(blk, ra);
                blk += 2;
                if (blk >= nblk) break;
                tc_wait_ld();
                if (blk + 2 < nblk) fetch(blk + 2, ra);
                emit(blk, rb);
                blk += 2;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
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

struct HostPlan {
    CUtensorMap map_a, map_w;       // 128 bytes each, 64-byte aligned
    TcParams p;
    int ab_dtype;
    int valid;
};
static_assert(sizeof(HostPlan) <= 512, "plan must fit the caller's 512-byte buffer");

// Accumulator width (multiple of 16, 64..256) with the least time per row block.  Per 16-deep k step one MMA costs
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

bool make_map(CUtensorMap* map, const void* ptr, long long rows, int k, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    const cuuint32_t box[2] = {cuuint32_t(TILE_K), cuuint32_t(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    // bf16 and fp16 are both moved as opaque 16-bit elements
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace sb

extern "C" int shvk_gemm_tc_plan(const shvk_gemm_args* g, int ab_dtype, void* host_plan) {
    using namespace sb;
    if (!g || !host_plan || (reinterpret_cast<uintptr_t>(host_plan) & 63)) return int(cudaErrorInvalidValue);
    if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return int(cudaErrorInvalidValue);
    if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->K % TILE_K || (g->lda & 7) || (g->ldw & 7) ||
        ((reinterpret_cast<uintptr_t>(g->A) | reinterpret_cast<uintptr_t>(g->W)) & 15) || (g->N & 3) || (g->swiglu && (g->N & 7)) ||
        (g->ldc & 3) || (g->R && (g->ldr & 3)) || (reinterpret_cast<uintptr_t>(g->C) & 15))
        return int(cudaErrorInvalidValue);
    HostPlan* hp = static_cast<HostPlan*>(host_plan);
    memset(hp, 0, sizeof(HostPlan));
    const int bn = choose_bn(g->N);
    if (!make_map(&hp->map_a, g->A, g->M, g->K, g->lda, TILE_M)) return int(cudaErrorNotSupported);
    if (!make_map(&hp->map_w, g->W, g->N, g->K, g->ldw, bn)) return int(cudaErrorNotSupported);
    TcParams& p = hp->p;
    p.M = g->M; p.N = g->N; p.K = g->K; p.BN = bn;
    p.n_tiles = (g->N + bn - 1) / bn;
    p.m_tiles = (g->M + TILE_M - 1) / TILE_M;
    p.C = g->C; p.ldc = g->ldc; p.c_dtype = g->c_dtype;
    p.bias = g->bias; p.act = g->act;
    p.R = g->R; p.ldr = g->ldr; p.r_div = g->r_div == 0.0f ? 1.0f : g->r_div;
    p.swiglu = g->swiglu;
    { const char* e = getenv("SHVK_TC_PROBE"); p.probe = e ? atoi(e) : 0; }
    const uint32_t fmt = ab_dtype == DT_BF16 ? 1u : 0u;
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), both K-major, N/8 at bit 17,
    // M/16 at bit 24
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(TILE_M >> 4) << 24);
    hp->ab_dtype = ab_dtype;
    hp->valid = 0x5b200;
    return 0;
}

namespace sb {
namespace {
template <typename T> int launch_tc(const HostPlan& hp, int M, cudaStream_t s) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    static unsigned long long attr_done = 0;   // one bit per device ordinal: dynamic shared memory opt-in is per device
    if (dev < 64 && !((attr_done >> dev) & 1ull)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_done |= 1ull << dev;
    }
    TcParams p = hp.p;
    p.M = M;
    p.m_tiles = (M + TILE_M - 1) / TILE_M;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long total = (long long)p.m_tiles * p.n_tiles;
    const unsigned grid = unsigned(total < sms ? total : sms);
    gemm_tc_kernel<T><<<grid, NTHREADS, SMEM_BYTES, s>>>(hp.map_a, hp.map_w, p);
    return int(cudaGetLastError());
}
}  // namespace
}  // namespace sb

// `rows` <= the M the plan was made for (the tensor map covers the planned extent; rows beyond `rows` are not written).
extern "C" int shvk_gemm_tc_rows(const void* host_plan, int rows, void* stream) {
    using namespace sb;
    const HostPlan* hp = static_cast<const HostPlan*>(host_plan);
    if (!hp || hp->valid != 0x5b200 || rows > hp->p.M) return int(cudaErrorInvalidValue);
    if (rows <= 0) return 0;
    SB_DISPATCH_DTYPE(hp->p.c_dtype, T, return launch_tc<T>(*hp, rows, cudaStream_t(stream)));
    return int(cudaErrorInvalidValue);
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
