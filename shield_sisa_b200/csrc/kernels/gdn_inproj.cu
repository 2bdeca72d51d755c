// GDN in-projection for the 16-bit modes, fused with everything between the projection and the recurrence:
// causal short conv (k = 4, bias) + SiLU on q, k, v, SiLU on the output gate, log decay and beta from a | b.
//
// The product is computed transposed on the tensor cores: D[channel][token] = W'[channel][:] . xn[token][:], the 128
// channels of a tile on the MMA rows (= tensor-memory lanes) and the tokens of a clip on the accumulator columns.
// An epilogue thread therefore owns ONE channel and finds consecutive tokens in consecutive registers, so the
// 4-tap causal convolution runs along registers (three carried values, no shuffles, no shared memory), and what
// leaves the kernel is not the fp32 projection [321][2316] but the 16-bit operand tiles the scan multiplies with, in the
// chunk-blocked layout of gdn_pt_layout.cuh: 1.56 MB per clip written here and read once by the scan, instead of
// 2.97 MB each way.  Stores need no staging: a thread writes the 32 contiguous bytes of its channel row of a chunk,
// a warp 1 KB contiguous.
//
// Channel tiles (rows of W', permuted from the reference's fused layout [q | k | v | gate | a | b] by
// shvk_gdn_inproj_row_order): tile 3h = [q_h | k_h], 3h + 1 = v_h, 3h + 2 = gate_h for head h; tile 18 = [a | b | 0].
// Token tiles per clip: tokens 0..175 and tokens 160..335 (176 columns each; the second tile computes tokens 160..175
// again only as the convolution's history and writes chunks 11..20; token slots 321.. are written as zeros).
// One work item = (clip, token tile) = all 19 channel tiles: the item's xn rows (176 x 384, 132 KB) are brought into
// shared memory ONCE and stay there while the 19 weight tiles stream past them through a five-stage ring, so the
// operand traffic out of L2 is 4.0 MB per clip instead of 8.6 MB with both operands streamed (which alone took
// 2.0 ms per launch at 4096 clips, more than the products).  Neighbouring CTAs take the two tiles of one clip.
//
// Roles (352 threads): warp 0 streams W' tiles (TMA, 128-byte swizzle, no multicast), warp 2 loads the xn tile of the
// next item as soon as the last product of the current one has read it, warp 1 issues tcgen05.mma (M 128, N 176,
// K 16) into one of two accumulators and owns tensor memory, warps 3-10 are the epilogue: two warps per lane quadrant,
// one for the first six chunks of the accumulator and one for the other five (it reads its three history columns
// from the neighbour's range).  K is walked in order and never split; a token's column depends on no other token of
// the batch, so clips stay independent bitwise.
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
#include <stdlib.h>
#include <string.h>

namespace sb {
namespace {
using namespace tc;

constexpr int TILE_M = 128, TILE_K = 64, NT = 176, TT_STRIDE = 160, M_TILES = 19, KBLOCKS = kD / TILE_K;
constexpr int W_ROWS = M_TILES * TILE_M;                         // 2432 rows of W' (2316 used)
constexpr int W_STAGE_BYTES = TILE_M * TILE_K * 2, W_STAGES = 5;
constexpr int XN_KB_BYTES = NT * TILE_K * 2, XN_BYTES = KBLOCKS * XN_KB_BYTES;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = XN_BYTES + W_STAGES * W_STAGE_BYTES + BAR_BYTES + 1024;
constexpr int NTHREADS = 352;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
static_assert(TT_STRIDE + NT == pt::TOK_PAD && TT_STRIDE % pt::CHUNK == 0 && NT % pt::CHUNK == 0, "token tiles cover the padded clip in whole chunks");
static_assert(XN_KB_BYTES % 1024 == 0 && W_STAGE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert((2 * W_STAGES + 6) * 8 <= BAR_BYTES && SMEM_BYTES <= 232448, "shared memory budget");

struct InprojMaps {
    CUtensorMap w;        // W' [2432][384], box 128 x 64
    CUtensorMap x;        // xn [rows][384], box 176 x 64
};
struct InprojParams {
    int B;
    uint32_t idesc;
    const float *conv_w, *conv_b, *a_log, *dt_bias;
    uint8_t* pt;
    uint32_t spin_limit;
    int starve;      // test launch only: the producer withholds the first weight tile of its first work item
    int qk_f16;      // q^T / k^T tiles in fp16 (fp16 mode) instead of bf16
    int probe;       // timing probes of a development build (-DSHVK_DEV_PROBES, SHVK_INPROJ_PROBE): 1 no global stores,
                     // 2 no activation arithmetic, 4 no tensor-memory loads, 8 no MMA.  Constant 0 in the shipped libraries.
};
// The probe bits travel in the kernel parameters (constant bank) and, to the tile functions, in bits 8+ of `flags`: a
// word in global memory would add a load in front of every tile and change the timings it is meant to explain.
// Cycle counters of the same builds: lane 0 of every warp adds clock64() differences to eight slots in shared memory
// (W producer: 0 wait for a free stage.  MMA thread: 0 wait for a drained accumulator, 1 for a weight stage, 2 for the
// token tile.  Epilogue warps: 0 wait for a full accumulator, 1 first tensor-memory load of a tile, 2 the later ones,
// 3 the whole tile.  All: 7 the role's loop.)  CTA 5 adds its totals to g_prof, read and cleared by
// shvk_dev_inproj_cycles.
#ifdef SHVK_DEV_PROBES
__device__ unsigned long long g_prof[11][8];
#define PROF_T() clock64()
#define PROF_ADD(slot, dt) do { if ((threadIdx.x & 31) == 0) prof_s[(threadIdx.x >> 5) * 8 + (slot)] += (unsigned long long)(dt); } while (0)
#define INPROJ_PROBE(bit) (probe_bits & (bit))
#define INPROJ_TILE_FLAGS(f) ((f) | (p.probe << 8))
#else
#define PROF_T() 0ll
#define PROF_ADD(slot, dt) do { } while (0)
#define INPROJ_PROBE(bit) 0
#define INPROJ_TILE_FLAGS(f) (f)
#endif

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
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    uint32_t r;                                                     // saturating: a finite fp16 even where fp32 exceeds 65504
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void stg128(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// One 32-byte store: a lane writes a whole sector, a warp 1 KB contiguous.  (Two 16-byte stores per row put 32 half-filled
// sectors per instruction through the L1 store path, twice the sector traffic for the same bytes.)
__device__ __forceinline__ void stg256(void* p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// What an epilogue does with its channel: q, k (conv + SiLU, stored in the mode's operand type: KIND_CONV_BF16 or
// KIND_CONV_F16), v (conv + SiLU, fp16), output gate (SiLU, fp16), a | b (log decay and beta, fp32).
enum : int { KIND_CONV_BF16 = 0, KIND_CONV_F16 = 1, KIND_SILU = 2, KIND_GATES = 3 };

struct ChanConst {            // what the epilogue thread knows about its channel
    float4 w;                 // conv taps: tap j multiplies x[t - 3 + j]
    float bias;
    float rate, dtb;          // KIND_GATES, decay rows: -exp(A_log), dt_bias
    bool is_beta, active;     // KIND_GATES: beta row; lane has a channel at all
    int half0;                // byte offset (0 or 16) of tokens 0-7 within the channel's 32-byte row of a chunk block
    int probe;                // probe bits of a development build, else 0
};

// Sixteen accumulator columns = one chunk of 16 tokens of one channel: activation, packing, and the channel's 32-byte
// (KIND_GATES: 64-byte) row of the chunk block at `row`.  nvalid: how many of the 16 token slots lie inside the clip
// (16 everywhere except in the clip's last chunk); the others are written as zeros.  x1, x2, x3: raw projections of the
// three tokens before this chunk (conv kinds), updated to the chunk's last three.
template <int KIND>
__device__ __forceinline__ void emit_chunk(const uint32_t (&in)[16], uint8_t* row, const ChanConst& cc, int nvalid,
                                           float& x1, float& x2, float& x3) {
    [[maybe_unused]] const int probe_bits = cc.probe;
    if (KIND == KIND_GATES) {
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            // beta rows: 1 / (1 + exp(-raw)); decay rows: rate * softplus(raw + dt_bias).  Both from one exponential and
            // without a branch: the rows of the two kinds sit in one warp, and a divergent branch per token would run
            // the sixteen tokens one after the other.
            const float raw = __uint_as_float(in[j]);
            const float ax = cc.is_beta ? -raw : raw + cc.dtb;
            const float e1 = 1.0f + __expf(ax);
            const float sp = cc.rate * (ax > 15.0f ? ax : __logf(e1));
            const float o = cc.is_beta ? __fdividef(1.0f, e1) : sp;
            v[j] = __float_as_uint(o);
        }
        if (nvalid < 16) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = j < nvalid ? v[j] : 0u;
        }
        if (cc.active) {
#pragma unroll
            for (int q = 0; q < 4; ++q) stg128(row + 16 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
    } else {
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            float y[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float raw = __uint_as_float(in[j + e]);
                float a = raw;
                if (KIND == KIND_CONV_BF16 || KIND == KIND_CONV_F16) {
                    a = fmaf(cc.w.x, x3, cc.bias);
                    a = fmaf(cc.w.y, x2, a);
                    a = fmaf(cc.w.z, x1, a);
                    a = fmaf(cc.w.w, raw, a);
                    x3 = x2; x2 = x1; x1 = raw;
                }
                y[e] = INPROJ_PROBE(2) ? raw : silu_tanh(a);
            }
            o[j >> 1] = KIND == KIND_CONV_BF16 ? pack_bf16(y[0], y[1]) : pack_f16(y[0], y[1]);
        }
        if (nvalid < 16) {                                        // the clip's last chunk: zero the token slots past its end
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (2 * i < nvalid ? (o[i] & 0x0000ffffu) : 0u) | (2 * i + 1 < nvalid ? (o[i] & 0xffff0000u) : 0u);
        }
        // the two 16-byte halves of the row trade places in rows 4-7 of every eight, so that the scan's ldmatrix reads
        // (eight rows of one half at a time) fall into eight different bank groups
        if (!INPROJ_PROBE(1)) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                w[i] = cc.half0 ? o[i + 4] : o[i];
                w[i + 4] = cc.half0 ? o[i] : o[i + 4];
            }
            stg256(row, w);
        } else if (o[0] == 0x12345678u && o[7] == 0x9abcdef0u) {
            stg128(row, o[0], o[1], o[2], o[3]);          // keeps the arithmetic alive
        }
    }
}

// One token tile of one channel: ncols accumulator columns (a multiple of 16) starting at tensor-memory address taddr,
// tokens tok0 .. tok0 + ncols - 1 of the clip, written to this channel's rows of the chunk blocks starting at dst (chunk
// tok0 / 16).  x1, x2, x3: raw projections of tokens tok0 - 1, - 2, - 3 (conv kinds).  A real loop over pairs of chunks,
// not unrolled over the tile: the body then stays resident in the instruction cache (fully unrolled, the eight epilogue
// warps spent more cycles waiting for instructions than issuing them).
template <int KIND>
__device__ __noinline__ void emit_tile(uint32_t taddr, uint8_t* dst, float4 cw, float bias, float rate, float dtb, int flags,
                                       int tok0, int ncols, bool has_hist, [[maybe_unused]] unsigned long long* prof_s) {
    // the channel constants travel as scalars (registers), not as a struct behind a pointer (local memory)
    ChanConst cc;
    cc.w = cw; cc.bias = bias; cc.rate = rate; cc.dtb = dtb;
    cc.is_beta = flags & 1; cc.active = flags & 2; cc.half0 = flags & 16; cc.probe = flags >> 8;
    [[maybe_unused]] const int probe_bits = cc.probe;
    uint32_t ra[16], rb[16];
    float x1 = 0.0f, x2 = 0.0f, x3 = 0.0f;
#ifdef SHVK_DEV_PROBES
    if (INPROJ_PROBE(4)) {
#pragma unroll
        for (int i = 0; i < 16; ++i) { ra[i] = 0x3f000000u + i; rb[i] = 0x3f100000u + i; }
#pragma unroll 1
        for (int c = 0; c < ncols; c += 32) {
            emit_chunk<KIND>(ra, dst + (long long)(c >> 4) * pt::BLOCK_BYTES, cc, kTok - (tok0 + c), x1, x2, x3);
            if (c + 16 >= ncols) break;
            emit_chunk<KIND>(rb, dst + (long long)((c >> 4) + 1) * pt::BLOCK_BYTES, cc, kTok - (tok0 + c + 16), x1, x2, x3);
        }
        return;
    }
#endif
    // The 16 columns before this warp's range hold its convolution history (their last three tokens).  They come with
    // the first chunk in ONE 32-column load: a tensor-memory load takes the better part of a microsecond to return while
    // the MMA pipe is busy, and a separate history load would put that wait in front of every tile.
    if (has_hist) tc_ld16x2(taddr - 16u, rb, ra);
    else tc_ld16(taddr, ra);
#pragma unroll 1
    for (int c = 0; c < ncols; c += 32) {
        { [[maybe_unused]] const long long ta = PROF_T(); tc_wait_ld(); PROF_ADD(c == 0 ? 1 : 2, PROF_T() - ta); }
        if (c == 0 && has_hist) { x1 = __uint_as_float(rb[15]); x2 = __uint_as_float(rb[14]); x3 = __uint_as_float(rb[13]); }
        if (c + 16 < ncols) tc_ld16(taddr + uint32_t(c + 16), rb);
        emit_chunk<KIND>(ra, dst + (long long)(c >> 4) * pt::BLOCK_BYTES, cc, kTok - (tok0 + c), x1, x2, x3);
        if (c + 16 >= ncols) break;
        { [[maybe_unused]] const long long ta = PROF_T(); tc_wait_ld(); PROF_ADD(2, PROF_T() - ta); }
        if (c + 32 < ncols) tc_ld16(taddr + uint32_t(c + 32), ra);
        emit_chunk<KIND>(rb, dst + (long long)((c >> 4) + 1) * pt::BLOCK_BYTES, cc, kTok - (tok0 + c + 16), x1, x2, x3);
    }
}

// Constants of channel row r of channel tile m, and where its rows of the chunk blocks start within a (clip, head).
struct ChanSite {
    float4 w;
    float bias, rate, dtb;
    int flags;      // 1 beta row, 2 lane has a channel, 16 = byte offset of tokens 0-7 within the row
    int head, section;
};
__device__ __forceinline__ ChanSite chan_site(const InprojParams& p, int m, int r) {
    ChanSite c;
    c.w = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    c.bias = 0.0f; c.rate = 0.0f; c.dtb = 0.0f;
    c.flags = 2 | (((r >> 2) & 1) << 4);
    c.head = m / 3;
    const int type = m % 3;
    if (m == M_TILES - 1) {
        const bool active = r < 12, is_beta = r >= 6;
        c.flags = (is_beta ? 1 : 0) | (active ? 2 : 0);
        c.head = active ? (r < 6 ? r : r - 6) : 0;
        c.rate = -expf(__ldg(p.a_log + c.head));
        c.dtb = __ldg(p.dt_bias + c.head);
        c.section = is_beta ? pt::BETA_OFF : pt::DEC_OFF;
    } else if (type == 0) {
        const int ci = (r < kDK ? 0 : kD) + c.head * kDK + (r & (kDK - 1));
        c.w = __ldg(reinterpret_cast<const float4*>(p.conv_w) + ci);
        c.bias = __ldg(p.conv_b + ci);
        c.section = pt::Q_OFF + r * 32;
    } else if (type == 1) {
        const int ci = 2 * kD + c.head * kDV + r;
        c.w = __ldg(reinterpret_cast<const float4*>(p.conv_w) + ci);
        c.bias = __ldg(p.conv_b + ci);
        c.section = pt::V_OFF + r * 32;
    } else {
        c.section = pt::G_OFF + r * 32;
    }
    return c;
}

__global__ void __launch_bounds__(NTHREADS, 1)
gdn_inproj_kernel(const __grid_constant__ InprojMaps maps, const InprojParams p, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t xn_base = base;                               // six k-block tiles [176 rows][128 bytes] of the item's xn rows
    const uint32_t w_base = base + XN_BYTES;                     // ring of W' k-block tiles [128 rows][128 bytes]
    const uint32_t bars = w_base + W_STAGES * W_STAGE_BYTES;     // wfull[S], wempty[S], accf[2], acce[2], xfull, xempty
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
#ifdef SHVK_DEV_PROBES
    __shared__ unsigned long long prof_arr[11 * 8];
    unsigned long long* prof_s = prof_arr;
    if (threadIdx.x < 88) prof_arr[threadIdx.x] = 0;
#else
    unsigned long long* prof_s = nullptr;
#endif
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto wfull_bar = [&](int s) { return bars + 8u * s; };
    auto wempty_bar = [&](int s) { return bars + 8u * (W_STAGES + s); };
    auto accf_bar = [&](int a) { return bars + 8u * (2 * W_STAGES + a); };
    auto acce_bar = [&](int a) { return bars + 8u * (2 * W_STAGES + 2 + a); };
    const uint32_t xfull_bar = bars + 8u * (2 * W_STAGES + 4), xempty_bar = bars + 8u * (2 * W_STAGES + 5);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < W_STAGES; ++s) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), 8); }
        mbar_init(xfull_bar, 1);
        mbar_init(xempty_bar, 1);
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
    [[maybe_unused]] const long long tk0 = PROF_T();
    const long long items = 2ll * p.B;                           // item = 2 * clip + token tile

    if (warp == 0) {
        if (lane == 0) {                                         // ---- W' tiles: 19 x 6 k-blocks per item through the ring
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t pol_w = policy_evict_last();
            for (long long item = blockIdx.x; ok && item < items; item += gridDim.x) {
                for (int m = 0; ok && m < M_TILES; ++m) {
                    for (int kb = 0; kb < KBLOCKS; ++kb) {
                        [[maybe_unused]] const long long tw0 = PROF_T();
                        if (!mbar_wait(wempty_bar(stage), phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                        PROF_ADD(0, PROF_T() - tw0);
                        if (p.starve && item == (long long)blockIdx.x && m == 0 && kb == 0) {   // test launch: this stage never fills
                            if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
                            continue;
                        }
                        mbar_expect_tx(wfull_bar(stage), uint32_t(W_STAGE_BYTES));
                        tma_load_2d_hint(w_base + stage * W_STAGE_BYTES, &maps.w, kb * TILE_K, m * TILE_M, wfull_bar(stage), pol_w);
                        if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 1); }
        }
    } else if (warp == 2) {
        if (lane == 0) {                                         // ---- the item's xn rows, once per item
            uint32_t n = 0;
            bool ok = true;
            for (long long item = blockIdx.x; ok && item < items; item += gridDim.x, ++n) {
                const int row0 = int(item >> 1) * kTok + int(item & 1) * TT_STRIDE;
                if (!mbar_wait(xempty_bar, (n & 1u) ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                mbar_expect_tx(xfull_bar, uint32_t(XN_BYTES));
                for (int kb = 0; kb < KBLOCKS; ++kb) tma_load_2d(xn_base + kb * XN_KB_BYTES, &maps.x, kb * TILE_K, row0, xfull_bar);
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 4); }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                         // ---- MMA issue
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0, n = 0;
            bool ok = true;
            [[maybe_unused]] const int probe_bits = p.probe;
            for (long long item = blockIdx.x; ok && item < items; item += gridDim.x, ++n) {
                { [[maybe_unused]] const long long tm2 = PROF_T();
                  if (!mbar_wait(xfull_bar, n & 1u, abortp, p.spin_limit)) { ok = false; break; }
                  PROF_ADD(2, PROF_T() - tm2); }
                for (int m = 0; ok && m < M_TILES; ++m) {
                    [[maybe_unused]] const long long tm0 = PROF_T();
                    if (!mbar_wait(acce_bar(acc), acc_phase ^ 1u, abortp, p.spin_limit)) { ok = false; break; }
                    PROF_ADD(0, PROF_T() - tm0);
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + uint32_t(acc * 256);
                    for (int kb = 0; kb < KBLOCKS; ++kb) {
                        [[maybe_unused]] const long long tm1 = PROF_T();
                        if (!mbar_wait(wfull_bar(stage), phase, abortp, p.spin_limit)) { ok = false; break; }
                        PROF_ADD(1, PROF_T() - tm1);
                        tc_fence_after();
                        const uint64_t da = smem_desc_sw128(w_base + stage * W_STAGE_BYTES), db = smem_desc_sw128(xn_base + kb * XN_KB_BYTES);
#pragma unroll
                        for (int k = 0; k < TILE_K / 16; ++k)
                            if (!INPROJ_PROBE(8)) tc_mma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), p.idesc, uint32_t((kb | k) != 0));
                        tc_commit(wempty_bar(stage));
                        if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    tc_commit(accf_bar(acc));
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
                if (ok) tc_commit(xempty_bar);                   // the item's last product has read the xn tile
            }
            if (!ok && !*abortp) { *abortp = 1; atomicCAS(status, 0, 2); }
        }
    } else {
        // ------------------------------------------------------------------------------------------ epilogue
        const int ew = warp - 3, quad = warp & 3, half = ew >> 2;    // half 0: the accumulator's first chunks, half 1: the rest
        const int r = quad * 32 + lane;                              // channel row within the tile
        const uint32_t tlane = tmem_base + (uint32_t(quad * 32) << 16);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (long long item = blockIdx.x; ok && item < items; item += gridDim.x) {
            const int clip = int(item >> 1), tt = int(item & 1);
            // this warp's columns of the accumulator: [col0, col0 + ncols), written from chunk `chunk0` on; its three
            // history tokens are the columns just before col0 (none at the start of the clip)
            const int col0 = half ? 96 : (tt ? 16 : 0);
            const int ncols = half ? 80 : (tt ? 80 : 96);
            const int tok0 = tt * TT_STRIDE + col0, chunk0 = tok0 >> 4;
            const bool has_hist = col0 > 0;
            ChanSite cur = chan_site(p, 0, r);
            for (int m = 0; m < M_TILES; ++m) {
                const ChanSite nxt = chan_site(p, m + 1 < M_TILES ? m + 1 : m, r);   // its loads fly during this tile's work
                [[maybe_unused]] const long long tp0 = PROF_T();
                if (!mbar_wait(accf_bar(acc), acc_phase, abortp, p.spin_limit)) { ok = false; break; }
                [[maybe_unused]] const long long tp1 = PROF_T();
                PROF_ADD(0, tp1 - tp0);
                tc_fence_after();
                const uint32_t tacc = tlane + uint32_t(acc * 256);
                uint8_t* dst = p.pt + ((long long)clip * kHeads + cur.head) * pt::HEAD_BYTES + cur.section + (long long)chunk0 * pt::BLOCK_BYTES;
                const int type = m % 3;
                if (m == M_TILES - 1) { if (quad == 0) emit_tile<KIND_GATES>(tacc + col0, dst, cur.w, cur.bias, cur.rate, cur.dtb, INPROJ_TILE_FLAGS(cur.flags), tok0, ncols, false, prof_s); }
                else if (type == 2) emit_tile<KIND_SILU>(tacc + col0, dst, cur.w, cur.bias, cur.rate, cur.dtb, INPROJ_TILE_FLAGS(cur.flags), tok0, ncols, false, prof_s);
                else if (type == 1 || p.qk_f16) emit_tile<KIND_CONV_F16>(tacc + col0, dst, cur.w, cur.bias, cur.rate, cur.dtb, INPROJ_TILE_FLAGS(cur.flags), tok0, ncols, has_hist, prof_s);
                else emit_tile<KIND_CONV_BF16>(tacc + col0, dst, cur.w, cur.bias, cur.rate, cur.dtb, INPROJ_TILE_FLAGS(cur.flags), tok0, ncols, has_hist, prof_s);
                PROF_ADD(3, PROF_T() - tp1);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                cur = nxt;
            }
        }
        if (!ok && lane == 0 && !*abortp) { *abortp = 1; atomicCAS(status, 0, 3); }
    }

    PROF_ADD(7, PROF_T() - tk0);
    __syncthreads();
#ifdef SHVK_DEV_PROBES
    if (threadIdx.x < 88 && blockIdx.x == 5) atomicAdd(&g_prof[threadIdx.x >> 3][threadIdx.x & 7], prof_arr[threadIdx.x]);
#endif
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
    CUtensorMap map_w, map_x;            // 128 bytes each, 64-byte aligned
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
        !tma::make_map_2d(&hp->map_x, xn, 2, max_rows, kD, kD, NT, TILE_K, true))
        return int(cudaErrorNotSupported);
    InprojParams& p = hp->p;
    const uint32_t fmt = ab_dtype == DT_BF16 ? 1u : 0u;
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), both K-major, N/8 at bit 17, M/16 at bit 24
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(NT >> 3) << 17) | (uint32_t(TILE_M >> 4) << 24);
    p.conv_w = conv_w; p.conv_b = conv_b; p.a_log = a_log; p.dt_bias = dt_bias;
    p.pt = static_cast<uint8_t*>(pt_out);
    p.spin_limit = SPIN_LIMIT;
    p.starve = 0;
    p.qk_f16 = ab_dtype == DT_F16;
    hp->max_rows = max_rows;
    hp->valid = 0x5b201;
    return 0;
}

static int inproj_launch(const void* host_plan, int B, void* stream, int starve, uint32_t spin_limit);

extern "C" int shvk_gdn_inproj(const void* host_plan, int B, void* stream) {
    return inproj_launch(host_plan, B, stream, 0, sb::SPIN_LIMIT);
}

// Test launch: every CTA's producer withholds the first weight tile of its first work item, so the MMA thread's wait on
// that stage runs out after `polls` polls (clamped to 256 .. 2^22); the CTA takes its abort path (status word of the
// tensor-core GEMMs set, every role leaves its loop, tensor memory freed) and returns.  The tiles are left partly written.
extern "C" int shvk_gdn_inproj_starved(const void* host_plan, int B, int polls, void* stream) {
    const uint32_t lim = polls < 256 ? 256u : (uint32_t(polls) > sb::SPIN_LIMIT ? sb::SPIN_LIMIT : uint32_t(polls));
    return inproj_launch(host_plan, B, stream, 1, lim);
}

static int inproj_launch(const void* host_plan, int B, void* stream, int starve, uint32_t spin_limit) {
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
    maps.w = hp->map_w; maps.x = hp->map_x;
    InprojParams p = hp->p;
    p.B = B;
    p.starve = starve;
    p.spin_limit = spin_limit;
    const long long items = 2ll * B;
    const unsigned grid = unsigned(items < sms ? items : sms);
#ifdef SHVK_DEV_PROBES
    {
        const char* e = getenv("SHVK_INPROJ_PROBE");
        p.probe = e ? atoi(e) : 0;
    }
#endif
    gdn_inproj_kernel<<<grid, NTHREADS, SMEM_BYTES, cudaStream_t(stream)>>>(maps, p, status);
    return int(cudaGetLastError());
}

#ifdef SHVK_DEV_PROBES
// Development builds only: the in-projection's cycle counters [11 warps][8 slots], read and cleared (synchronises the device).
extern "C" __attribute__((visibility("default"))) int shvk_dev_inproj_cycles(unsigned long long* out) {
    unsigned long long zero[88] = {0};
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, sb::g_prof, sizeof(zero));
    cudaMemcpyToSymbol(sb::g_prof, zero, sizeof(zero));
    return 0;
}
#endif
