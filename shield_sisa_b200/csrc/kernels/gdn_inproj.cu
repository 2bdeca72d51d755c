// GDN in-projection for the 16-bit modes, fused with everything between the projection and the recurrence:
// causal short conv (k = 4, bias) + SiLU on q, k, v, SiLU on the output gate, log decay and beta from a | b.
//
// The product is computed transposed on the tensor cores: D[channel][token] = W'[channel][:] . xn[token][:], the 128
// channels of a tile on the MMA rows (= tensor-memory lanes) and the tokens of a clip on the accumulator columns.
// An epilogue thread therefore owns ONE channel and finds consecutive tokens in consecutive registers, so the
// 4-tap causal convolution runs along registers (three carried values, no shuffles, no shared memory), and what
// leaves the kernel is not the fp32 projection [321][2316] but the bf16 operand tiles the scan multiplies with, in the
// chunk-blocked layout of gdn_pt_layout.cuh: 1.56 MB per clip written here and read once by the scan, instead of
// 2.97 MB each way.  Stores need no staging: a thread writes the 32 contiguous bytes of its channel row of a chunk,
// a warp 1 KB contiguous.
//
// Channel tiles (rows of W', permuted from the reference's fused layout [q | k | v | gate | a | b] by
// shvk_gdn_inproj_row_order): tile 3h = [q_h | k_h], 3h + 1 = v_h, 3h + 2 = gate_h for head h; tile 18 = [a | b | 0].
// Token tiles per clip: tokens 0..175 (accumulator 0) and 176..335 (accumulator 1; 321.. are written as zeros).
// One work item = (clip, channel tile) = both token tiles; items are dealt round-robin to the persistent CTAs, so
// neighbouring CTAs work on the same clip and share its xn rows in L2.
//
// Roles (320 threads): warp 0 TMA producer (W' tile 128 x 64 and xn tile N x 64 per stage, 128-byte swizzle, no
// multicast), warp 1 MMA issuer (tcgen05.mma M 128, N 176 / 160, K 16) and owner of tensor memory, warps 2-5 epilogue
// of accumulator 0, warps 6-9 epilogue of accumulator 1.  The conv history of token 176 is tokens 173..175, which
// the second group reads from accumulator 0 before that is released.  K is walked in order and never split; a token's
// column depends on no other token of the batch, so clips stay independent bitwise.
//
// Every mbarrier wait is bounded (status word of the tensor-core GEMM, shvk_gemm_tc_status).
//
// Replaces, together with gdn_scan_t.cu: gemm<T> in-projection (engine/cuda/engine.cu:418) + launch_gdn_prep
// (engine/cuda/seq.cu:72-104); oracle: oracle/shieldv_ref.py:142-150,186-193.
#include "device_utils.cuh"
#include "gdn_pt_layout.cuh"
#include "shv_seq_kernels.h"
#include "status_words.cuh"
#include "tc_ptx.cuh"
#include "tma_utils.cuh"

#include <atomic>
#include <string.h>

namespace sb {
namespace {
using namespace tc;

constexpr int TILE_M = 128, TILE_K = 64, N0 = 176, N1 = 160, M_TILES = 19, KBLOCKS = kD / TILE_K;
constexpr int W_ROWS = M_TILES * TILE_M;                         // 2432 rows of W' (2316 used)
constexpr int A_BYTES = TILE_M * TILE_K * 2, B_BYTES = N0 * TILE_K * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4, BAR_BYTES = 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
constexpr int NTHREADS = 320;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
static_assert(N0 + N1 == pt::TOK_PAD && N0 % pt::CHUNK == 0, "token tiles cover the padded clip in whole chunks");
static_assert(STAGE_BYTES % 1024 == 0 && A_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert((2 * STAGES + 4) * 8 <= BAR_BYTES && SMEM_BYTES <= 232448, "shared memory budget");

struct InprojMaps {
    CUtensorMap w;        // W' [2432][384], box 128 x 64
    CUtensorMap x0, x1;   // xn [rows][384], boxes 176 x 64 and 160 x 64
};
struct InprojParams {
    int B;
    uint32_t idesc0, idesc1;
    const float *conv_w, *conv_b, *a_log, *dt_bias;
    uint8_t* pt;
    uint32_t spin_limit;
};

// x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)) with the hardware tanh: absolute error ~5e-4 |x|, below the bf16 rounding
// that follows
__device__ __forceinline__ float silu_tanh(float x) {
    float th;
    const float hx = 0.5f * x;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(hx));
    return fmaf(hx, th, hx);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void stg128(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

enum : int { KIND_CONV = 0, KIND_SILU = 1, KIND_GATES = 2 };

struct ChanConst {            // what the epilogue thread knows about its channel
    float4 w;                 // conv taps: tap j multiplies x[t - 3 + j]
    float bias;
    float rate, dtb;          // KIND_GATES, decay rows: -exp(A_log), dt_bias
    bool is_beta, active;     // KIND_GATES: beta row; lane has a channel at all
};

// One token tile of one channel: NCOLS accumulator columns starting at tensor-memory address taddr, tokens TOK0 ..
// TOK0 + NCOLS - 1 of the clip, written to this channel's rows of the chunk blocks starting at dst (chunk TOK0 / 16).
// x1, x2, x3: raw projections of tokens TOK0 - 1, - 2, - 3 (KIND_CONV).
template <int KIND, int TOK0, int NCOLS>
__device__ __forceinline__ void emit_tile(uint32_t taddr, uint8_t* dst, const ChanConst& cc, float x1, float x2, float x3) {
    constexpr int NB = (NCOLS + 31) / 32;
    uint32_t r[2][32];
    tc_ld32(taddr, r[0]);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        tc_wait_ld();
        if (b + 1 < NB) {
            if (NCOLS - 32 * (b + 1) >= 32) tc_ld32(taddr + uint32_t(32 * (b + 1)), r[(b + 1) & 1]);
            else tc_ld16(taddr + uint32_t(32 * (b + 1)), r[(b + 1) & 1]);
        }
        const int ncol = NCOLS - 32 * b >= 32 ? 32 : 16;          // compile-time after unrolling
        const uint32_t* in = r[b & 1];
        if (KIND == KIND_GATES) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < ncol) {
                    const float raw = __uint_as_float(in[j]);
                    float o;
                    if (cc.is_beta) {
                        o = __fdividef(1.0f, 1.0f + __expf(-raw));
                    } else {
                        const float ax = raw + cc.dtb;
                        o = cc.rate * (ax > 15.0f ? ax : __logf(1.0f + __expf(ax)));
                    }
                    v[j] = (TOK0 + 32 * b + j < kTok) ? o : 0.0f;
                }
            }
            if (cc.active) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (16 * c < ncol) {
                        uint8_t* row = dst + (long long)(2 * b + c) * pt::BLOCK_BYTES;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            stg128(row + 16 * q, __float_as_uint(v[16 * c + 4 * q]), __float_as_uint(v[16 * c + 4 * q + 1]),
                                   __float_as_uint(v[16 * c + 4 * q + 2]), __float_as_uint(v[16 * c + 4 * q + 3]));
                    }
                }
            }
        } else {
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                if (j < ncol) {
                    float y[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float raw = __uint_as_float(in[j + e]);
                        float a = raw;
                        if (KIND == KIND_CONV) {
                            a = fmaf(cc.w.x, x3, cc.bias);
                            a = fmaf(cc.w.y, x2, a);
                            a = fmaf(cc.w.z, x1, a);
                            a = fmaf(cc.w.w, raw, a);
                            x3 = x2; x2 = x1; x1 = raw;
                        }
                        y[e] = (TOK0 + 32 * b + j + e < kTok) ? silu_tanh(a) : 0.0f;
                    }
                    o[j >> 1] = pack_bf16(y[0], y[1]);
                }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (16 * c < ncol) {
                    uint8_t* row = dst + (long long)(2 * b + c) * pt::BLOCK_BYTES;
                    stg128(row, o[8 * c], o[8 * c + 1], o[8 * c + 2], o[8 * c + 3]);
                    stg128(row + 16, o[8 * c + 4], o[8 * c + 5], o[8 * c + 6], o[8 * c + 7]);
                }
            }
        }
    }
}

__global__ void __launch_bounds__(NTHREADS, 1)
gdn_inproj_kernel(const __grid_constant__ InprojMaps maps, const InprojParams p, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;           // full[S], empty[S], acc_full[2], acc_empty[2]
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
        mbar_init(accf_bar(0), 1); mbar_init(accf_bar(1), 1);
        mbar_init(acce_bar(0), 8);                                // both epilogue groups read accumulator 0
        mbar_init(acce_bar(1), 4);
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
    const long long items = (long long)p.B * M_TILES;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t pol_w = policy_evict_last();
            for (long long item = blockIdx.x; ok && item < items; item += gridDim.x) {
                const int clip = int(item / M_TILES), m = int(item - (long long)clip * M_TILES);
                for (int tt = 0; ok && tt < 2; ++tt) {
                    const int row0 = clip * kTok + tt * N0;
                    const uint32_t tx = uint32_t(A_BYTES + (tt ? N1 : N0) * TILE_K * 2);
                    for (int kb = 0; kb < KBLOCKS; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                        const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                        mbar_expect_tx(full_bar(stage), tx);
                        tma_load_2d_hint(sa, &maps.w, kb * TILE_K, m * TILE_M, full_bar(stage), pol_w);
                        tma_load_2d(sb_, tt ? &maps.x1 : &maps.x0, kb * TILE_K, row0, full_bar(stage));
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 1); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (long long item = blockIdx.x; ok && item < items; item += gridDim.x) {
                for (int tt = 0; ok && tt < 2; ++tt) {
                    if (!mbar_wait(acce_bar(tt), acc_phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + uint32_t(tt * 256);
                    const uint32_t idesc = tt ? p.idesc1 : p.idesc0;
                    for (int kb = 0; kb < KBLOCKS; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, abortp, p.spin_limit)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sa = base + stage * STAGE_BYTES, sb_ = sa + A_BYTES;
                        const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb_);
#pragma unroll
                        for (int k = 0; k < TILE_K / 16; ++k)
                            tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, uint32_t((kb | k) != 0));
                        tc_commit(empty_bar(stage));
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    tc_commit(accf_bar(tt));
                }
                acc_phase ^= 1u;
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 2); }
        }
    } else {
        // ------------------------------------------------------------------------------------------ epilogue
        const int ew = warp - 2, quad = warp & 3, half = ew >> 2;    // half 0: tokens 0..175, half 1: tokens 176..335
        const int r = quad * 32 + lane;                              // channel row within the tile
        const uint32_t tlane = tmem_base + (uint32_t(quad * 32) << 16);
        uint32_t acc_phase = 0;
        bool ok = true;
        for (long long item = blockIdx.x; ok && item < items; item += gridDim.x) {
            const int clip = int(item / M_TILES), m = int(item - (long long)clip * M_TILES);
            const int type = m % 3;
            int head = m / 3;
            ChanConst cc;
            cc.w = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            cc.bias = 0.0f; cc.rate = 0.0f; cc.dtb = 0.0f; cc.is_beta = false; cc.active = true;
            int section = 0;
            if (m == M_TILES - 1) {
                cc.active = r < 12;
                cc.is_beta = r >= 6;
                head = cc.active ? (r < 6 ? r : r - 6) : 0;
                cc.rate = -expf(__ldg(p.a_log + head));
                cc.dtb = __ldg(p.dt_bias + head);
                section = cc.is_beta ? pt::BETA_OFF : pt::DEC_OFF;
            } else if (type == 0) {
                const int ci = (r < kDK ? 0 : kD) + head * kDK + (r & (kDK - 1));
                cc.w = __ldg(reinterpret_cast<const float4*>(p.conv_w) + ci);
                cc.bias = __ldg(p.conv_b + ci);
                section = pt::Q_OFF + r * 32;
            } else if (type == 1) {
                const int ci = 2 * kD + head * kDV + r;
                cc.w = __ldg(reinterpret_cast<const float4*>(p.conv_w) + ci);
                cc.bias = __ldg(p.conv_b + ci);
                section = pt::V_OFF + r * 32;
            } else {
                section = pt::G_OFF + r * 32;
            }
            uint8_t* dst = p.pt + ((long long)clip * kHeads + head) * pt::HEAD_BYTES + section;

            if (!mbar_wait(accf_bar(0), acc_phase, abortp, p.spin_limit)) { ok = false; break; }
            tc_fence_after();
            if (half == 0) {
                if (m == M_TILES - 1) { if (quad == 0) emit_tile<KIND_GATES, 0, N0>(tlane, dst, cc, 0.0f, 0.0f, 0.0f); }
                else if (type == 2) emit_tile<KIND_SILU, 0, N0>(tlane, dst, cc, 0.0f, 0.0f, 0.0f);
                else emit_tile<KIND_CONV, 0, N0>(tlane, dst, cc, 0.0f, 0.0f, 0.0f);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce_bar(0));
            } else {
                uint32_t hr[16];                                     // tokens 160..175: the last three are the conv history
                tc_ld16(tlane + uint32_t(N0 - 16), hr);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce_bar(0));
                if (!mbar_wait(accf_bar(1), acc_phase, abortp, p.spin_limit)) { ok = false; break; }
                tc_fence_after();
                uint8_t* dst1 = dst + (long long)(N0 / pt::CHUNK) * pt::BLOCK_BYTES;
                const float x1 = __uint_as_float(hr[15]), x2 = __uint_as_float(hr[14]), x3 = __uint_as_float(hr[13]);
                if (m == M_TILES - 1) { if (quad == 0) emit_tile<KIND_GATES, N0, N1>(tlane + 256u, dst1, cc, 0.0f, 0.0f, 0.0f); }
                else if (type == 2) emit_tile<KIND_SILU, N0, N1>(tlane + 256u, dst1, cc, 0.0f, 0.0f, 0.0f);
                else emit_tile<KIND_CONV, N0, N1>(tlane + 256u, dst1, cc, x1, x2, x3);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce_bar(1));
            }
            acc_phase ^= 1u;
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
    CUtensorMap map_w, map_x0, map_x1;   // 128 bytes each, 64-byte aligned
    InprojParams p;
    long long max_rows;
    int valid;
};
static_assert(sizeof(HostPlan) <= 512, "plan must fit the caller's 512-byte buffer");

}  // namespace
}  // namespace sb

extern "C" int shvk_gdn_inproj_rows(void) { return sb::W_ROWS; }

extern "C" void shvk_gdn_inproj_row_order(int32_t* src_row) {
    using namespace sb;
    for (int m = 0; m < M_TILES; ++m)
        for (int r = 0; r < TILE_M; ++r) {
            int src = -1;
            const int head = m / 3, type = m % 3;
            if (m == M_TILES - 1) src = r < 12 ? kGA + r : -1;                       // a[6] | b[6]
            else if (type == 0) src = (r < kDK ? kGQ : kGK) + head * kDK + (r & (kDK - 1));
            else if (type == 1) src = kGV + head * kDV + r;
            else src = kGG + head * kDV + r;
            src_row[m * TILE_M + r] = src;
        }
}

extern "C" size_t shvk_gdn_pt_bytes(int B) { return B > 0 ? size_t(B) * size_t(sb::pt::CLIP_BYTES) : 0; }

extern "C" int shvk_gdn_inproj_plan(const void* xn, long long max_rows, const void* w_perm, const float* conv_w,
                                    const float* conv_b, const float* a_log, const float* dt_bias, void* pt_out, int ab_dtype,
                                    void* host_plan) {
    using namespace sb;
    if (!xn || !w_perm || !conv_w || !conv_b || !a_log || !dt_bias || !pt_out || !host_plan || max_rows <= 0 ||
        (reinterpret_cast<uintptr_t>(host_plan) & 63))
        return int(cudaErrorInvalidValue);
    if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return int(cudaErrorInvalidValue);
    if ((reinterpret_cast<uintptr_t>(xn) | reinterpret_cast<uintptr_t>(w_perm) | reinterpret_cast<uintptr_t>(pt_out) |
         reinterpret_cast<uintptr_t>(conv_w)) & 15)
        return int(cudaErrorInvalidValue);
    HostPlan* hp = static_cast<HostPlan*>(host_plan);
    memset(hp, 0, sizeof(HostPlan));
    if (!tma::make_map_2d(&hp->map_w, w_perm, 2, W_ROWS, kD, kD, TILE_M, TILE_K, true) ||
        !tma::make_map_2d(&hp->map_x0, xn, 2, max_rows, kD, kD, N0, TILE_K, true) ||
        !tma::make_map_2d(&hp->map_x1, xn, 2, max_rows, kD, kD, N1, TILE_K, true))
        return int(cudaErrorNotSupported);
    InprojParams& p = hp->p;
    const uint32_t fmt = ab_dtype == DT_BF16 ? 1u : 0u;
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), both K-major, N/8 at bit 17, M/16 at bit 24
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(TILE_M >> 4) << 24);
    p.idesc0 = common | (uint32_t(N0 >> 3) << 17);
    p.idesc1 = common | (uint32_t(N1 >> 3) << 17);
    p.conv_w = conv_w; p.conv_b = conv_b; p.a_log = a_log; p.dt_bias = dt_bias;
    p.pt = static_cast<uint8_t*>(pt_out);
    p.spin_limit = SPIN_LIMIT;
    hp->max_rows = max_rows;
    hp->valid = 0x5b201;
    return 0;
}

extern "C" int shvk_gdn_inproj(const void* host_plan, int B, void* stream) {
    using namespace sb;
    const HostPlan* hp = static_cast<const HostPlan*>(host_plan);
    if (!hp || hp->valid != 0x5b201 || (long long)B * kTok > hp->max_rows) return int(cudaErrorInvalidValue);
    if (B <= 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    static std::atomic<unsigned long long> attr_done{0};
    if (dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
        const cudaError_t e = cudaFuncSetAttribute(gdn_inproj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        if (dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int* status = gemm_tc_status_word();
    if (!status) return int(cudaErrorInvalidSymbol);
    InprojMaps maps;
    maps.w = hp->map_w; maps.x0 = hp->map_x0; maps.x1 = hp->map_x1;
    InprojParams p = hp->p;
    p.B = B;
    const long long items = (long long)B * M_TILES;
    const unsigned grid = unsigned(items < sms ? items : sms);
    gdn_inproj_kernel<<<grid, NTHREADS, SMEM_BYTES, cudaStream_t(stream)>>>(maps, p, status);
    return int(cudaGetLastError());
}
