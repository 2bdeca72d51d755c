// SwiGLU feed-forward block of the 16-bit modes in one kernel: h += down(silu(gate(xn)) * up(xn)), the hidden layer
// never leaving the SM.
//
// Per 128-row block of xn (a persistent CTA per SM walks the row blocks):
//   the block's xn rows (128 x 384, six swizzled k-block tiles, 96 KB) are brought into shared memory once;
//   for each slab j of 64 hidden units (15 slabs):
//     up(j)    acc_up[128 x 128]  = xn . W_up[128 j .. 128 j + 127]^T          6 k blocks x 4 MMAs (M 128, N 128, K 16)
//              the rows of W_up are (gate, up) interleaved, so columns (2 i, 2 i + 1) of acc_up are one hidden unit
//     drain(j) eight epilogue warps read acc_up, form silu(gate) * up, round to the storage type and write the
//              128 x 64 tile straight into shared memory in the swizzled K-major layout an MMA A operand has
//     down(j)  acc_down[128 x 384] += hid(j) . W_down[:, 64 j .. 64 j + 63]^T    3 x 4 MMAs (N 128 each)
//   after the last slab the epilogue adds acc_down to the residual rows of h: a 32 x 32 block leaves tensor memory one
//   row per lane, is turned through a swizzled shared-memory tile, and residual loads (prefetched into registers) and
//   stores run coalesced, eight lanes per 128-byte row segment.
// Tensor memory: acc_up in columns 0-127, acc_down in columns 128-511 (all 512).  The MMA thread issues
// up(j), down(j - 1), up(j + 1), ...: the tensor pipe works on down(j - 1) while the epilogue drains acc_up of slab j.
// Weight tiles of both matrices travel through one ring of six 16 KB stages in the order they are consumed.
//
// Arithmetic is the one of the two-kernel path (gemm_tc up with SwiGLU epilogue, gemm_tc down with residual epilogue):
// k in ascending order in blocks of 16, one accumulator per output, the same SwiGLU formula and rounding of the hidden
// layer; a row of h depends on no other row.
//
// Every mbarrier wait is bounded (status word of the tensor-core GEMMs, shvk_gemm_tc_status).  No multicast loads.
//
// Replaces two gemm<T> launches of the reference (engine/cuda/engine.cu:434-440; epilogues gemm.cuh:33-51) and the
// hidden-layer round trip through HBM between them.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"
#include "status_words.cuh"
#include "tc_ptx.cuh"
#include "tma_utils.cuh"

#include <atomic>
#include <stdlib.h>
#include <string.h>

namespace sb {
namespace {
using namespace tc;

constexpr int TILE = 128, TILE_K = 64, KB_UP = kD / TILE_K;              // 6 k blocks of the up projection
constexpr int SLABS = kDFF / 64;                                          // 15 slabs of 64 hidden units
constexpr int N_DOWN = kD / TILE;                                         // 3 column groups of the down projection
constexpr int TILE_BYTES = TILE * TILE_K * 2;                             // 16 KB: every operand tile here
constexpr int XN_BYTES = KB_UP * TILE_BYTES, W_STAGES = 6, HID_BUFS = 2;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = XN_BYTES + W_STAGES * TILE_BYTES + HID_BUFS * TILE_BYTES + BAR_BYTES + 1024;
constexpr int NTHREADS = 352, EPI_WARPS = 8;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr uint32_t ACC_UP = 0, ACC_DOWN = 128;                            // tensor-memory columns
static_assert(kD % TILE_K == 0 && kDFF % 64 == 0 && kD % TILE == 0, "shapes");
static_assert((2 * W_STAGES + 2 + 2 + 2 * HID_BUFS + 3) * 8 <= BAR_BYTES && SMEM_BYTES <= 232448, "shared memory budget");
static_assert(EPI_WARPS * 4096 <= HID_BUFS * TILE_BYTES, "the output staging tiles live in the hidden-layer buffers");

struct FfnMaps {
    CUtensorMap x;        // xn [rows][384], box 128 x 64
    CUtensorMap wu;       // W_up [1920][384] (gate / up rows interleaved), box 128 x 64
    CUtensorMap wd;       // W_down [384][960], box 128 x 64
};
// Timing probes of a development build (-DSHVK_DEV_PROBES, SHVK_FFN_PROBE; never the shipped libraries): 1 no SwiGLU
// arithmetic, 2 no acc_up loads, 4 no up MMAs, 8 no down MMAs, 16 no residual epilogue work.  The bits travel in the
// kernel parameters (constant bank), so reading them costs nothing in the loops they switch.
#ifdef SHVK_DEV_PROBES
#define FFN_PROBE(bit) (p.probe & (bit))
#else
#define FFN_PROBE(bit) 0
#endif
struct FfnParams {
    int probe;
    int rows, m_tiles;
    uint32_t idesc;
    float* h;
    uint32_t spin_limit;
    int starve;      // test launch only: the producer withholds the first weight tile of its first row block
};

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
ffn_fused_kernel(const __grid_constant__ FfnMaps maps, const FfnParams p, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t xn_base = base;                                   // six k-block tiles [128 rows][128 bytes]
    const uint32_t w_base = base + XN_BYTES;                         // ring of weight tiles [128 rows][128 bytes]
    const uint32_t hid_base = w_base + W_STAGES * TILE_BYTES;        // two hidden-layer tiles [128 rows][128 bytes]
    const uint32_t bars = hid_base + HID_BUFS * TILE_BYTES;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto wfull_bar = [&](int s) { return bars + 8u * s; };
    auto wempty_bar = [&](int s) { return bars + 8u * (W_STAGES + s); };
    const uint32_t xfull_bar = bars + 8u * (2 * W_STAGES), xempty_bar = xfull_bar + 8u;
    const uint32_t accu_full = xfull_bar + 16u, accu_empty = xfull_bar + 24u;
    auto hfull_bar = [&](int b) { return xfull_bar + 32u + 8u * b; };
    auto hempty_bar = [&](int b) { return xfull_bar + 48u + 8u * b; };
    const uint32_t accd_full = xfull_bar + 64u, accd_empty = xfull_bar + 72u;
    const uint32_t staging_free = xfull_bar + 80u;                   // every epilogue warp's output stores have left the staging tiles

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < W_STAGES; ++s) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 1); }
        mbar_init(xfull_bar, 1); mbar_init(xempty_bar, 1);
        mbar_init(accu_full, 1); mbar_init(accu_empty, EPI_WARPS);
        for (int b = 0; b < HID_BUFS; ++b) { mbar_init(hfull_bar(b), EPI_WARPS); mbar_init(hempty_bar(b), 1); }
        mbar_init(accd_full, 1); mbar_init(accd_empty, EPI_WARPS);
        mbar_init(staging_free, EPI_WARPS);
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

    if (warp == 0) {
        if (lane == 0) {                                             // ---- weight tiles, in the order the MMA thread consumes them
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t pol_w = policy_evict_last();
            bool withheld = !p.starve;
            auto put = [&](const CUtensorMap* map, int k0, int row0) -> bool {
                if (!mbar_wait(wempty_bar(stage), phase ^ 1u, abortp, p.spin_limit)) return false;
                if (!withheld) {                                     // test launch: this stage never fills
                    withheld = true;
                    if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
                    return true;
                }
                mbar_expect_tx(wfull_bar(stage), uint32_t(TILE_BYTES));
                tma_load_2d_hint(w_base + stage * TILE_BYTES, map, k0, row0, wfull_bar(stage), pol_w);
                if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
                return true;
            };
            for (int mt = blockIdx.x; ok && mt < p.m_tiles; mt += gridDim.x) {
                for (int j = 0; ok && j <= SLABS; ++j) {
                    if (j < SLABS)
                        for (int kb = 0; ok && kb < KB_UP; ++kb) ok = put(&maps.wu, kb * TILE_K, j * TILE);
                    if (j >= 1)
                        for (int c = 0; ok && c < N_DOWN; ++c) ok = put(&maps.wd, (j - 1) * 64, c * TILE);
                }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 1); }
        }
    } else if (warp == 2) {
        if (lane == 0) {                                             // ---- the row block's xn rows, once per block
            uint32_t n = 0;
            bool ok = true;
            for (int mt = blockIdx.x; ok && mt < p.m_tiles; mt += gridDim.x, ++n) {
                if (!mbar_wait(xempty_bar, (n & 1u) ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                mbar_expect_tx(xfull_bar, uint32_t(XN_BYTES));
                for (int kb = 0; kb < KB_UP; ++kb) tma_load_2d(xn_base + kb * TILE_BYTES, &maps.x, kb * TILE_K, mt * TILE, xfull_bar);
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 4); }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                             // ---- MMA issue
            int stage = 0;
            uint32_t phase = 0, n = 0, slab = 0;                     // slab: slabs started by this CTA so far
            uint32_t hpar = 0;                                       // bit b: parity of the down products issued from hidden-layer buffer b
            bool ok = true;
            auto take = [&]() -> bool {                              // next weight tile of the ring
                if (!mbar_wait(wfull_bar(stage), phase, abortp, p.spin_limit)) return false;
                tc_fence_after();
                return true;
            };
            auto release = [&]() {
                tc_commit(wempty_bar(stage));
                if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
            };
            for (int mt = blockIdx.x; ok && mt < p.m_tiles; mt += gridDim.x, ++n) {
                if (!mbar_wait(xfull_bar, n & 1u, abortp, p.spin_limit)) { ok = false; break; }
                tc_fence_after();
                for (int j = 0; ok && j <= SLABS; ++j) {
                    if (j < SLABS) {                                 // up(j)
                        if (!mbar_wait(accu_empty, (slab & 1u) ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                        tc_fence_after();
                        for (int kb = 0; kb < KB_UP; ++kb) {
                            if (!take()) { ok = false; break; }
                            const uint64_t da = smem_desc_sw128(xn_base + kb * TILE_BYTES), db = smem_desc_sw128(w_base + stage * TILE_BYTES);
#pragma unroll
                            for (int k = 0; k < TILE_K / 16; ++k)
                                if (!FFN_PROBE(4)) tc_mma_f16(tmem_base + ACC_UP, da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc, uint32_t((kb | k) != 0));
                            release();
                        }
                        if (!ok) break;
                        tc_commit(accu_full);
                        ++slab;
                        if (j == SLABS - 1) tc_commit(xempty_bar);   // the block's last up product has read the xn tile
                    }
                    if (j >= 1) {                                    // down(j - 1)
                        const int jj = j - 1, hb = jj & 1;
                        if (jj == 0 && !mbar_wait(accd_empty, (n & 1u) ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                        if (!mbar_wait(hfull_bar(hb), (hpar >> hb) & 1u, abortp, p.spin_limit)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = smem_desc_sw128(hid_base + hb * TILE_BYTES);
                        for (int c = 0; c < N_DOWN; ++c) {
                            if (!take()) { ok = false; break; }
                            const uint64_t db = smem_desc_sw128(w_base + stage * TILE_BYTES);
#pragma unroll
                            for (int k = 0; k < TILE_K / 16; ++k)
                                if (!FFN_PROBE(8)) tc_mma_f16(tmem_base + ACC_DOWN + uint32_t(c * TILE), da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc,
                                           uint32_t((jj | k) != 0));
                            release();
                        }
                        if (!ok) break;
                        tc_commit(hempty_bar(hb));
                        hpar ^= 1u << hb;
                        if (jj == SLABS - 1) tc_commit(accd_full);
                    }
                }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 2); }
        }
    } else {
        // ------------------------------------------------------------------------------------------ epilogue
        const int ew = warp - 3, quad = warp & 3, half = ew >> 2;
        const int row = quad * 32 + lane;                            // row of the block this lane owns (its tensor-memory lane)
        const uint32_t tlane = tmem_base + (uint32_t(quad * 32) << 16);
        // this lane's 64 bytes of the hidden-layer tile: 16-byte chunks 4 half .. 4 half + 3 of row `row`, chunk c at c ^ (row & 7)
        const uint32_t hid_row = uint32_t(row >> 3) * 1024u + uint32_t(row & 7) * 128u;
        const uint32_t stage_tile = hid_base + uint32_t(ew) * 4096u; // output staging: 32 rows x 128 bytes, swizzled
        uint32_t slab = 0, n = 0;
        uint32_t hpar = 0;                                           // bit b: parity of the fills of hidden-layer buffer b so far
        bool ok = true;
        for (int mt = blockIdx.x; ok && mt < p.m_tiles; mt += gridDim.x, ++n) {
            // the block's residual rows (128 x 1536 bytes) are asked into L2 now, fifteen slabs before the epilogue reads them:
            // its loads then wait for L2, not for DRAM
            for (int id = ew * 32 + lane; id < TILE * (kD * 4 / 128); id += EPI_WARPS * 32) {
                const int prow = id / (kD * 4 / 128), seg = id - prow * (kD * 4 / 128);
                if (mt * TILE + prow < p.rows)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(p.h + (long long)(mt * TILE + prow) * kD + seg * 32));
            }
            for (int j = 0; j < SLABS; ++j, ++slab) {
                const int hb = j & 1;
                if (!mbar_wait(accu_full, slab & 1u, abortp, p.spin_limit)) { ok = false; break; }
                tc_fence_after();
                uint32_t r[64];
                if (!FFN_PROBE(2)) {
                    tc_ld32(tlane + ACC_UP + uint32_t(half * 64), r);
                    tc_ld32(tlane + ACC_UP + uint32_t(half * 64 + 32), r + 32);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) r[i] = 0x3f000000u + uint32_t(i);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accu_empty);              // the next up product may overwrite acc_up
                uint32_t o[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = r[i];
                if (!FFN_PROBE(1))
#pragma unroll
                for (int i = 0; i < 16; ++i) {                       // the arithmetic of gemm_tc's SwiGLU epilogue
                    const float g0 = __uint_as_float(r[4 * i]), g1 = __uint_as_float(r[4 * i + 2]);
                    const float a = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(r[4 * i + 1]);
                    const float b = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(r[4 * i + 3]);
                    o[i] = pack2<T>(a, b);
                }
                // the down product that last read this buffer (two slabs ago) must be complete
                if (!mbar_wait(hempty_bar(hb), ((hpar >> hb) & 1u) ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                hpar ^= 1u << hb;
                const uint32_t dst = hid_base + uint32_t(hb) * TILE_BYTES + hid_row;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    sts128u(dst + ((uint32_t(4 * half + c) ^ uint32_t(row & 7)) << 4), o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                fence_proxy_async();                                 // the tensor core reads this tile through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(hfull_bar(hb));
            }
            if (!ok) break;
            // ---- h += acc_down: twelve 32-column blocks per row quadrant, alternate blocks to the quadrant's two warps.
            // A block leaves tensor memory with one row per lane; it is turned through the warp's staging tile so that
            // residual loads and stores are coalesced: lane -> (row rr + 4 i, 16-byte column group c4), eight lanes per row.
            const int m0 = mt * TILE + quad * 32;
            const int rr = lane >> 3, c4 = lane & 7;
            float* hblk = p.h + (long long)(m0 + rr) * kD + 4 * c4;
            float4 resa[8], resb[8];                                 // residuals of this warp's next two blocks
            auto load_res = [&](int blk, float4 (&res)[8]) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    res[i] = m0 + rr + 4 * i < p.rows ? *reinterpret_cast<const float4*>(hblk + (long long)(4 * i) * kD + 32 * blk)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
            };
            // one block: tensor memory -> staging tile (a row per lane) -> coalesced add and store
            auto emit = [&](int blk, const float4 (&res)[8]) {
                uint32_t r[32];
                tc_ld32(tlane + ACC_DOWN + uint32_t(32 * blk), r);
                tc_wait_ld();
                __syncwarp();                                        // the previous block's reads of the tile are done
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    sts128u(stage_tile + uint32_t(lane) * 128u + ((uint32_t(q) ^ uint32_t(lane & 7)) << 4), r[4 * q], r[4 * q + 1],
                            r[4 * q + 2], r[4 * q + 3]);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = rr + 4 * i;
                    const float4 a = lds128(stage_tile + uint32_t(row) * 128u + ((uint32_t(c4) ^ uint32_t(row & 7)) << 4));
                    if (m0 + row < p.rows)
                        *reinterpret_cast<float4*>(hblk + (long long)(4 * i) * kD + 32 * blk) =
                            make_float4(res[i].x + a.x, res[i].y + a.y, res[i].z + a.z, res[i].w + a.w);
                }
            };
            load_res(half, resa);
            load_res(half + 2, resb);
            if (!mbar_wait(accd_full, n & 1u, abortp, p.spin_limit)) { ok = false; break; }
            tc_fence_after();
            // both hidden-layer buffers are free now (every down product of the block is complete): they hold the
            // staging tiles of the eight warps.  Six blocks per warp, residuals fetched two blocks ahead.
            if (!FFN_PROBE(16)) {
#pragma unroll 1
                for (int blk = half; blk < kD / 32; blk += 4) {
                    emit(blk, resa);
                    if (blk + 4 < kD / 32) load_res(blk + 4, resa);
                    emit(blk + 2, resb);
                    if (blk + 6 < kD / 32) load_res(blk + 6, resb);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(accd_empty);                             // the next block's down products may overwrite acc_down
                mbar_arrive(staging_free);                           // this warp's staging tile is hidden-layer space again ...
            }
            // ... once every epilogue warp is done with its own (the tiles of the next block's hidden layer span them all)
            if (!mbar_wait(staging_free, n & 1u, abortp, p.spin_limit)) { ok = false; break; }
        }
        if (!ok && lane == 0 && !*abortp) { *abortp = 1; atomicCAS(status, 0, 3); }
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

struct HostPlan {
    CUtensorMap map_x, map_wu, map_wd;   // 128 bytes each, 64-byte aligned
    FfnParams p;
    long long max_rows;
    int ab_dtype, valid;
};
static_assert(sizeof(HostPlan) <= 512, "plan must fit the caller's 512-byte buffer");

template <typename T> int launch_ffn(const FfnMaps& maps, const FfnParams& p, int* status, cudaStream_t s) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    static std::atomic<unsigned long long> attr_done{0};
    if (dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
        const cudaError_t e = cudaFuncSetAttribute(ffn_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        if (dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned grid = unsigned(p.m_tiles < sms ? p.m_tiles : sms);
    FfnParams q = p;
    q.probe = 0;
#ifdef SHVK_DEV_PROBES
    { const char* e = getenv("SHVK_FFN_PROBE"); q.probe = e ? atoi(e) : 0; }
#endif
    ffn_fused_kernel<T><<<grid, NTHREADS, SMEM_BYTES, s>>>(maps, q, status);
    return int(cudaGetLastError());
}

}  // namespace
}  // namespace sb

extern "C" int shvk_ffn_fused_plan(const void* xn, long long max_rows, const void* w_up, const void* w_down, float* h, int ab_dtype,
                                   void* host_plan) {
    using namespace sb;
    if (!xn || !w_up || !w_down || !h || !host_plan || max_rows <= 0 || (reinterpret_cast<uintptr_t>(host_plan) & 63))
        return int(cudaErrorInvalidValue);
    if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return int(cudaErrorInvalidValue);
    if ((reinterpret_cast<uintptr_t>(xn) | reinterpret_cast<uintptr_t>(w_up) | reinterpret_cast<uintptr_t>(w_down) |
         reinterpret_cast<uintptr_t>(h)) & 15)
        return int(cudaErrorInvalidValue);
    HostPlan* hp = static_cast<HostPlan*>(host_plan);
    memset(hp, 0, sizeof(HostPlan));
    if (!tma::make_map_2d(&hp->map_x, xn, 2, max_rows, kD, kD, TILE, TILE_K, true) ||
        !tma::make_map_2d(&hp->map_wu, w_up, 2, 2 * kDFF, kD, kD, TILE, TILE_K, true) ||
        !tma::make_map_2d(&hp->map_wd, w_down, 2, kD, kDFF, kDFF, TILE, TILE_K, true))
        return int(cudaErrorNotSupported);
    FfnParams& p = hp->p;
    const uint32_t fmt = ab_dtype == DT_BF16 ? 1u : 0u;
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), both K-major, N/8 at bit 17, M/16 at bit 24
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(TILE >> 3) << 17) | (uint32_t(TILE >> 4) << 24);
    p.h = h;
    p.spin_limit = SPIN_LIMIT;
    p.starve = 0;
    hp->max_rows = max_rows;
    hp->ab_dtype = ab_dtype;
    hp->valid = 0x5b202;
    return 0;
}

static int ffn_launch_rows(const void* host_plan, int rows, void* stream, int starve, uint32_t spin_limit);

extern "C" int shvk_ffn_fused(const void* host_plan, int rows, void* stream) {
    return ffn_launch_rows(host_plan, rows, stream, 0, sb::SPIN_LIMIT);
}

// Test launch: every CTA's producer withholds the first weight tile of its first row block, so the MMA thread's wait on
// that stage runs out after `polls` polls (clamped to 256 .. 2^22); the CTA takes its abort path (status word of the
// tensor-core GEMMs set, every role leaves its loop, tensor memory freed) and returns.  h is left partly updated.
extern "C" int shvk_ffn_fused_starved(const void* host_plan, int rows, int polls, void* stream) {
    const uint32_t lim = polls < 256 ? 256u : (uint32_t(polls) > sb::SPIN_LIMIT ? sb::SPIN_LIMIT : uint32_t(polls));
    return ffn_launch_rows(host_plan, rows, stream, 1, lim);
}

static int ffn_launch_rows(const void* host_plan, int rows, void* stream, int starve, uint32_t spin_limit) {
    using namespace sb;
    const HostPlan* hp = static_cast<const HostPlan*>(host_plan);
    if (!hp || hp->valid != 0x5b202 || rows > hp->max_rows) return int(cudaErrorInvalidValue);
    if (rows <= 0) return 0;
    int* status = gemm_tc_status_word();
    if (!status) return int(cudaErrorInvalidSymbol);
    FfnMaps maps;
    maps.x = hp->map_x; maps.wu = hp->map_wu; maps.wd = hp->map_wd;
    FfnParams p = hp->p;
    p.starve = starve;
    p.spin_limit = spin_limit;
    p.rows = rows;
    p.m_tiles = (rows + TILE - 1) / TILE;
    cudaStream_t s = cudaStream_t(stream);
    return hp->ab_dtype == DT_BF16 ? launch_ffn<__nv_bfloat16>(maps, p, status, s) : launch_ffn<__half>(maps, p, status, s);
}
