// Fused GatedDeltaNet core for the 16-bit modes: the delta rule in chunks of 16 tokens on the tensor cores.
//
// Same inputs, outputs and fusion as gdn_scan.cu (TMA-staged slices of the projection P, conv + SiLU, L2 norms, gates,
// delta rule, gated RMSNorm), but the recurrence is evaluated 16 tokens at a time in its WY form, so that the 64 x 128
// state is touched by matrix products instead of per-token sweeps.  For a chunk with inclusive cumulative log decay
// c_i, e_i = exp(c_i), state S0 (keys x values) entering the chunk:
//     A = K K^T, B = Q K^T                                      (16 x 16, contraction over the 64 keys)
//     L_ij = beta_i exp(c_i - c_j) A_ij (j < i),  T = (I + L)^-1,  T2 = T diag(beta),  M_ij = exp(c_i - c_j) B_ij (j <= i)
//     R = K S0,  QS = Q S0                                       (16 x 128)
//     U = T2 (V - diag(e) R)                                    (16 x 128)
//     O = M U + diag(e) QS
//     S' = e_16 S0 + K^T diag(exp(c_16 - c_j)) U
// Everything is computed transposed (value dimension = MMA rows), which makes every hand-over between products a
// register-only repack: warp w owns value columns 32w .. 32w+31, keeps its slice of S^T (32 x 64, fp32) as the
// accumulator fragments of mma.sync.m16n8k16, and the accumulator layout of one product (rows = values, columns =
// tokens) is exactly the A-operand layout of the next.  Only K, Q, T2 and M pass through shared memory (bf16 tiles
// written once per chunk, read as B fragments), and the 16 x 16 triangular inverse is a 16-lane forward substitution
// in fp32.  k and q enter the tiles un-normalised; their L2 norms are the diagonals of the Gram products K K^T and
// Q Q^T and are applied as per-token scalars (rows of L and M, the decay factors of R, Q S0 and the state update).
// Operands are rounded to bf16, the state and all accumulation stay fp32: the error against the exact
// recurrence is a few 1e-3 relative on the delta-rule output (measured against the oracle in the tests), inside the
// 2e-2 budget of the 16-bit modes.  The exact tier keeps the per-token fp32 kernel of gdn_scan.cu.
//
// Schedule of one chunk (three CTA barriers): prep (conv + SiLU of two adjacent channels per thread, gates on
// warp 0) | Gram / inverse on warps 0 and 1 with the gated RMSNorm of the PREVIOUS chunk spread over all
// four warps, then R and Q S0 | U, O, state update, and each warp's share of sum(o^2) for the next chunk's norm.
// The TMA ring has three slots because a slot stays alive as the chunk's o tile and gate tile until that deferred
// norm is done.  Within a phase every shared-memory load is issued before the first tile store: the compiler keeps
// loads behind an earlier store to the same memory space, which would serialise otherwise independent tokens.
// A rotated loop (operand tiles of chunk + 1 computed into registers before the closing barrier of chunk) was measured
// and dropped: 32 more live registers under the 168 cap spill, 7.5 ms against 5.9 ms.
//
// Warp-level mma.sync rather than tcgen05: per 16-token chunk the products form a dependency chain five deep on tiles
// of 16 tokens; tcgen05 needs M >= 64 rows and an asynchronous issue / commit / tensor-memory round trip per link of
// that chain, which costs more than the products themselves.  tcgen05 carries the projections (gemm_tc.cu).
//
// Reference: engine/cuda/seq.cu:72-214 (gdn_prep + delta + gated_norm), oracle/shieldv_ref.py:121-163,186-197.
#include <type_traits>

#include "device_utils.cuh"
#include "gdn_scan_mma.cuh"
#include "status_words.cuh"
#include "tma_utils.cuh"

namespace sb {
namespace {

constexpr int TC = 16;
constexpr uint32_t WAIT_POLLS = 1u << 22;    // about a quarter second
constexpr int KB_PITCH = 72;                 // bf16 per row of the K / Q tiles (144 bytes: conflict-free fragment reads)
constexpr int KT_PITCH = 24;                 // bf16 per row of K^T, T2, M tiles (48 bytes)
constexpr int VT_PITCH = 20;                 // floats per row of V^T
constexpr int OT_PITCH = kDV + 4;            // floats per token row of the o tile: the fragment stores of a warp (eight value rows
                                             // x four token pairs) then fall into 32 different banks

__device__ int g_scan_mma_status = 0;

struct RawBuf {                              // TMA targets, one chunk
    float q[TC][kDK];                        // raw q projection
    float k[TC][kDK];                        // raw k projection
    float v[TC][kDV];                        // raw v; after prep reused as the chunk's output tile o[token][value], whose
                                             // padded rows (OT_PITCH) run 256 bytes into ab, dead by then
    float ab[TC][16];                        // a | b gate projections; after the gates are taken, the 16 x 16 matrix L (until the
                                             // inverse is done, before the o tile is written)
};
// Once q and k are converted, their two tiles (contiguous, 8 KB) receive the chunk's output-gate tile [16][128].
static_assert(sizeof(RawBuf) == 17408 && sizeof(RawBuf) % 128 == 0, "tile offsets must stay 128-byte aligned");
static_assert(TC * OT_PITCH * 4 <= int(sizeof(float) * TC * (kDV + 16)), "padded o tile must end inside v + ab");

struct MmaSmem {
    RawBuf raw[3];                           // ring: chunk c uses raw[c % 3] until its deferred gated norm is done
    float vt[kDV][VT_PITCH];                 // silu(conv v), transposed: [value][token]
    __nv_bfloat16 kb[TC][KB_PITCH];          // silu(conv k), un-normalised, [token][key]
    __nv_bfloat16 qb[TC][KB_PITCH];          // silu(conv q), un-normalised
    __nv_bfloat16 kt[kDK][KT_PITCH];         // the k tile transposed: [key][token]
    __nv_bfloat16 t2[TC][KT_PITCH];          // (I + L)^-1 diag(beta)
    __nv_bfloat16 mq[TC][KT_PITCH];          // decay-masked Q K^T
    float ssq[TC][4];                        // per token: each warp's share of sum(o^2) over its 32 value columns
    float iq[TC], ik[TC], beta[TC];          // 0.125/|q|, 1/|k|, beta (0 beyond the sequence end)
    float cum[TC], eg[TC], dj[TC];           // c_i, exp(c_i), exp(c_last - c_i)
    unsigned long long full[3], gfull[3];    // mbarriers: raw tiles / gate tile of the chunk in ring slot i landed
};
constexpr int MMA_SMEM_BYTES = int(sizeof(MmaSmem)) + 128;

struct MmaMaps {
    CUtensorMap qk;    // box 16 x 64
    CUtensorMap vg;    // box 16 x 128
    CUtensorMap ab;    // box 16 x 16
};

// x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)) with the hardware tanh: absolute error ~5e-4 |x|, below the bf16 rounding
// that follows every use in this kernel
__device__ __forceinline__ float silu_tanh(float x) {
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * x));
    const float hx = 0.5f * x;
    return fmaf(hx, th, hx);
}
// Two adjacent channels per thread.  Plain scalar pairs: the packed fma.rn.f32x2 / mul.rn.f32x2 forms were measured and
// executed no fewer instructions here (105.3 M against 103.3 M warp instructions on the same launch).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
// SiLU of two values at once
__device__ __forceinline__ float2 silu_tanh2(float2 x) {
    const float2 hx = fmul2(x, make_float2(0.5f, 0.5f));
    float2 th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th.x) : "f"(hx.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(th.y) : "f"(hx.y));
    return ffma2(hx, th, hx);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__global__ void __launch_bounds__(128, 3)
gdn_scan_mma_kernel(const __grid_constant__ MmaMaps maps, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                    const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ o_norm_w,
                    T* __restrict__ on) {
    extern __shared__ uint8_t mma_smem_raw[];
    MmaSmem& sm = *reinterpret_cast<MmaSmem*>((reinterpret_cast<uintptr_t>(mma_smem_raw) + 127) & ~uintptr_t(127));
    const int clip = blockIdx.x / kHeads, head = blockIdx.x % kHeads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;               // mma fragment coordinates
    const int row_base = clip * kTok;
    const int dvb = warp * 32;                           // this warp's value columns

    // prep role: two adjacent channels per thread (64-bit tile loads and stores).  Warp 0: q channels 2 lane, + 1;
    // warp 1: k channels; warps 2, 3: v columns 2 (tid - 64), + 1.  Conv tap j multiplies x[t - 3 + j].
    const int pc0 = warp == 0 ? 2 * lane : warp == 1 ? 2 * lane : 2 * (tid - 64);       // first channel within its stream
    const int cw0 = (warp == 0 ? 0 : warp == 1 ? 384 : 768) + head * (warp < 2 ? kDK : kDV) + pc0;
    // taps and bias of the channel pair are re-read per chunk (L1 hits, issued ahead of the TMA wait) rather than held
    // in ten registers across the whole recurrence
    const float4* cwp = reinterpret_cast<const float4*>(conv_w + cw0 * 4);
    const float2* cbp = reinterpret_cast<const float2*>(conv_b + cw0);
    float2 x1 = make_float2(0.0f, 0.0f), x2 = x1, x3 = x1;   // zero history = causal padding
    const float neg_rate = -expf(a_log[head]), dtb = dt_bias[head];

    // S^T slice of this warp as accumulator fragments: S[mi][nj][.] = values dvb + 16 mi + {g, g + 8}, keys 8 nj + 2t, + 1
    float S[2][8][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nj = 0; nj < 8; ++nj)
#pragma unroll
            for (int e = 0; e < 4; ++e) S[mi][nj][e] = 0.0f;

    const uint32_t bars0 = tma::smem_addr(&sm.full[0]), gbars0 = tma::smem_addr(&sm.gfull[0]);   // + 8 * ring slot
    auto issue = [&](int chunk) {                         // thread 0: q, k, v, a|b tiles of `chunk`
        RawBuf& b = sm.raw[chunk % 3];
        const uint32_t bar = bars0 + 8u * uint32_t(chunk % 3);
        const int row = row_base + chunk * TC;
        tma::mbar_expect_tx(bar, uint32_t(sizeof(RawBuf)));
        tma::load_2d(tma::smem_addr(&b.q[0][0]), &maps.qk, kGQ + head * kDK, row, bar);
        tma::load_2d(tma::smem_addr(&b.k[0][0]), &maps.qk, kGK + head * kDK, row, bar);
        tma::load_2d(tma::smem_addr(&b.v[0][0]), &maps.vg, kGV + head * kDV, row, bar);
        tma::load_2d(tma::smem_addr(&b.ab[0][0]), &maps.ab, kGA, row, bar);
    };
    if (tid == 0) {
        for (int i = 0; i < 3; ++i) { tma::mbar_init(bars0 + 8u * i, 1); tma::mbar_init(gbars0 + 8u * i, 1); }
        tma::fence_barrier_init();
        tma::fence_proxy_async();
        issue(0);
    }
    __syncthreads();

    constexpr int NCHUNK = (kTok + TC - 1) / TC;
    // Gated RMSNorm of chunk pc (its o tile and gate tile sit in ring slot pc % 3), tokens first .. first + count - 1
    // Loads and arithmetic run unconditionally (the tile rows exist), only the store is guarded, so the
    // unrolled tokens overlap.  Returns false if the gate tile never arrived.
    auto gated_norm = [&](int pc, int first, auto count_c) -> bool {
        constexpr int count = decltype(count_c)::value;   // compile-time, so a warp with few tokens does only their work
        RawBuf& pb = sm.raw[pc % 3];
        if (!tma::mbar_wait_bounded(gbars0 + 8u * uint32_t(pc % 3), uint32_t(pc / 3) & 1u, WAIT_POLLS)) return false;
        const float* ot = &pb.v[0][0];
        const float* gt_ = &pb.q[0][0];
        const float4 onw = __ldg(reinterpret_cast<const float4*>(o_norm_w + lane * 4));
        const int pnt = min(min(TC, kTok - pc * TC), first + count);
        // rows first .. first + count - 1 at constant offsets
        const float* op = ot + first * OT_PITCH + lane * 4;
        const float* gp = gt_ + first * kDV + lane * 4;
        const float* sp = &sm.ssq[first][0];
        T* dst = on + ((long long)row_base + pc * TC + first) * kVD + head * kDV + lane * 4;
#pragma unroll
        for (int k = 0; k < count; ++k) {
            const float4 o = *reinterpret_cast<const float4*>(op + k * OT_PITCH);
            const float4 gt = *reinterpret_cast<const float4*>(gp + k * kDV);
            const float4 pp = *reinterpret_cast<const float4*>(sp + 4 * k);   // the four warps' partial sums of o^2
            const float rstd = rsqrtf(((pp.x + pp.y) + (pp.z + pp.w)) * (1.0f / float(kDV)) + 1e-6f);
            if (first + k < pnt)
                store_quad<T>(dst + k * kVD, ((o.x * rstd) * onw.x) * silu_tanh(gt.x), ((o.y * rstd) * onw.y) * silu_tanh(gt.y),
                              ((o.z * rstd) * onw.z) * silu_tanh(gt.z), ((o.w * rstd) * onw.w) * silu_tanh(gt.w));
        }
        return true;
    };
    for (int chunk = 0; chunk < NCHUNK; ++chunk) {
        const int t0 = chunk * TC, nt = min(TC, kTok - t0);
        RawBuf& b = sm.raw[chunk % 3];
        (void)nt;
        if (tid == 0) {
            // ring slot (chunk + 1) % 3 was last used by chunk - 2, whose gated norm ended before the previous barrier
            tma::fence_proxy_async();
            if (chunk + 1 < NCHUNK) issue(chunk + 1);
        }
        const float4 w0 = __ldg(cwp), w1 = __ldg(cwp + 1);
        const float2 bc2 = __ldg(cbp);
        const float2 wx = make_float2(w0.x, w1.x), wy = make_float2(w0.y, w1.y), wz = make_float2(w0.z, w1.z), ww = make_float2(w0.w, w1.w);
        if (!tma::mbar_wait_bounded(bars0 + 8u * uint32_t(chunk % 3), uint32_t(chunk / 3) & 1u, WAIT_POLLS)) {
            if (tid == 0) atomicCAS(&g_scan_mma_status, 0, 1);
            return;                                       // every thread times out on the same barrier and leaves
        }
        // ---------------------------------------------------------------- prep: conv + SiLU -> bf16 operand tiles, gates
        // k and q go into the tiles un-normalised; their norms come out of the Gram products below and enter every
        // later formula as per-token scalars.
        if (warp < 2) {
            const float* src = warp == 0 ? &b.q[0][pc0] : &b.k[0][pc0];
            uint32_t* dst = reinterpret_cast<uint32_t*>(warp == 0 ? &sm.qb[0][pc0] : &sm.kb[0][pc0]);
            uint32_t kt0[TC / 2], kt1[TC / 2];             // warp 1: two rows of K^T, two tokens per word
            float2 prev = make_float2(0.0f, 0.0f);
            // all loads first: a tile store between them would order every later load behind it and serialise the tokens
            float2 rawv[TC];
#pragma unroll
            for (int i = 0; i < TC; ++i) rawv[i] = *reinterpret_cast<const float2*>(src + i * kDK);
#pragma unroll
            for (int i = 0; i < TC; ++i) {
                const float2 raw = rawv[i];
                float2 acc = ffma2(wx, x3, bc2);
                acc = ffma2(wy, x2, acc);
                acc = ffma2(wz, x1, acc);
                acc = ffma2(ww, raw, acc);
                const float2 val = silu_tanh2(acc);
                x3 = x2; x2 = x1; x1 = raw;
                dst[i * (KB_PITCH / 2)] = pack_bf16(val.x, val.y);
                if (warp == 1) {
                    if (i & 1) { kt0[i >> 1] = pack_bf16(prev.x, val.x); kt1[i >> 1] = pack_bf16(prev.y, val.y); }
                    prev = val;
                }
            }
            if (warp == 1) {
                uint4* r0 = reinterpret_cast<uint4*>(&sm.kt[pc0][0]);             // rows of 48 bytes: 16-byte aligned
                uint4* r1 = reinterpret_cast<uint4*>(&sm.kt[pc0 + 1][0]);
                r0[0] = make_uint4(kt0[0], kt0[1], kt0[2], kt0[3]); r0[1] = make_uint4(kt0[4], kt0[5], kt0[6], kt0[7]);
                r1[0] = make_uint4(kt1[0], kt1[1], kt1[2], kt1[3]); r1[1] = make_uint4(kt1[4], kt1[5], kt1[6], kt1[7]);
            }
        } else {
            const float* src = &b.v[0][pc0];
            float4* r0 = reinterpret_cast<float4*>(&sm.vt[pc0][0]);                // rows of 80 bytes: 16-byte aligned
            float4* r1 = reinterpret_cast<float4*>(&sm.vt[pc0 + 1][0]);
            float2 rawv[TC];
#pragma unroll
            for (int i = 0; i < TC; ++i) rawv[i] = *reinterpret_cast<const float2*>(src + i * kDV);
#pragma unroll
            for (int i4 = 0; i4 < TC / 4; ++i4) {
                float c0[4], c1[4];
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const float2 raw = rawv[4 * i4 + ii];
                    float2 acc = ffma2(wx, x3, bc2);
                    acc = ffma2(wy, x2, acc);
                    acc = ffma2(wz, x1, acc);
                    acc = ffma2(ww, raw, acc);
                    const float2 val = silu_tanh2(acc);
                    x3 = x2; x2 = x1; x1 = raw;
                    c0[ii] = val.x; c1[ii] = val.y;
                }
                r0[i4] = make_float4(c0[0], c0[1], c0[2], c0[3]);
                r1[i4] = make_float4(c1[0], c1[1], c1[2], c1[3]);
            }
        }
        if (warp == 0) {                                  // gates and the inclusive prefix sum of the log decays
            // tokens past the sequence end are made inert: beta = 0, no decay
            const bool valid = lane < nt;
            // hardware exp / log: absolute error ~1e-7 on the log decay and on beta, far below the bf16 operands
            const float ax = b.ab[lane & (TC - 1)][head] + dtb;
            float c = valid ? neg_rate * (ax > 15.0f ? ax : __logf(1.0f + __expf(ax))) : 0.0f;
            const float bt_ = valid ? __fdividef(1.0f, 1.0f + __expf(-b.ab[lane & (TC - 1)][6 + head])) : 0.0f;
#pragma unroll
            for (int o = 1; o < TC; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, c, o);
                if (lane >= o) c += up;
            }
            const float last = __shfl_sync(0xffffffffu, c, TC - 1);
            if (lane < TC) {
                sm.beta[lane] = bt_;
                sm.cum[lane] = c;
                sm.eg[lane] = __expf(c);
                sm.dj[lane] = __expf(last - c);
            }
        }
        __syncthreads();
        float* gtile = &b.q[0][0];                        // q and k are consumed: their 8 KB now take the gate tile
        float (*lf)[TC] = reinterpret_cast<float (*)[TC]>(&b.ab[0][0]);       // and the a|b tile takes L
        if (tid == 0) {
            tma::fence_proxy_async();
            const uint32_t gbar = gbars0 + 8u * uint32_t(chunk % 3);
            tma::mbar_expect_tx(gbar, uint32_t(TC * kDV * 4));
            tma::load_2d(tma::smem_addr(gtile), &maps.vg, kGG + head * kDV, row_base + t0, gbar);
        }
        const uint32_t* kbw = reinterpret_cast<const uint32_t*>(&sm.kb[0][0]);   // 36 words per token row
        const uint32_t* qbw = reinterpret_cast<const uint32_t*>(&sm.qb[0][0]);
        // ---------------------------------------------------------------- warp 0: norms of k, L, T2; warp 1: norms, masked Q K^T
        if (warp < 2) {
            // Gram products over the 64 keys: warp 0 K K^T; warp 1 Q K^T and the diagonal of Q Q^T
            float acc[2][4], dq[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) { acc[ni][e] = 0.0f; dq[ni][e] = 0.0f; }
            const uint32_t* xa = warp == 0 ? kbw : qbw;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint32_t a[4] = {xa[g * 36 + 8 * p + t], xa[(g + 8) * 36 + 8 * p + t], xa[g * 36 + 8 * p + t + 4],
                                       xa[(g + 8) * 36 + 8 * p + t + 4]};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    const uint32_t k0 = kbw[(8 * ni + g) * 36 + 8 * p + t], k1 = kbw[(8 * ni + g) * 36 + 8 * p + t + 4];
                    mma16816(acc[ni], a, k0, k1);
                    if (warp == 1) mma16816(dq[ni], a, qbw[(8 * ni + g) * 36 + 8 * p + t], qbw[(8 * ni + g) * 36 + 8 * p + t + 4]);
                }
            }
            // diagonal entries: row g sits in tile 0 at column 2t + e == g, row g + 8 in tile 1 at the same lane / slot
            if (t == (g >> 1)) {
                const bool odd = g & 1;                   // selects, not a runtime index: the fragments stay in registers
                if (warp == 0) {
                    sm.ik[g] = rsqrtf((odd ? acc[0][1] : acc[0][0]) + 1e-6f);
                    sm.ik[g + 8] = rsqrtf((odd ? acc[1][3] : acc[1][2]) + 1e-6f);
                } else {
                    sm.iq[g] = rsqrtf((odd ? dq[0][1] : dq[0][0]) + 1e-6f) * 0.125f;
                    sm.iq[g + 8] = rsqrtf((odd ? dq[1][3] : dq[1][2]) + 1e-6f) * 0.125f;
                }
            }
            __syncwarp();
            // acc[ni][0,1]: row i = g, columns j = 8 ni + 2t, + 1;  acc[ni][2,3]: row i = g + 8
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = g + (e >> 1) * 8, j = 8 * ni + 2 * t + (e & 1);
                    const bool keep = warp == 0 ? j < i : j <= i;
                    const float dec = __expf(keep ? sm.cum[i] - sm.cum[j] : 0.0f);
                    // warp 0: L_ij carries both key norms; warp 1: the key norm of column j is applied to U in the O product
                    const float f = warp == 0 ? sm.beta[i] * sm.ik[i] * sm.ik[j] : sm.iq[i];
                    acc[ni][e] = keep ? dec * acc[ni][e] * f : 0.0f;
                }
            if (warp == 0) {
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                    for (int e = 0; e < 4; ++e) lf[g + (e >> 1) * 8][8 * ni + 2 * t + (e & 1)] = acc[ni][e];
                __syncwarp();
                if (lane < TC) {                          // column `lane` of (I + L)^-1 by forward substitution
                    float x[TC];
#pragma unroll
                    for (int i = 0; i < TC; ++i) {
                        // four partial sums: the dependent chain per row is i / 4 long instead of i
                        float s0 = i == lane ? 1.0f : 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                        for (int j = 0; j < i; ++j) {
                            const float l = lf[i][j];
                            if ((j & 3) == 0) s0 = fmaf(-l, x[j], s0);
                            else if ((j & 3) == 1) s1 = fmaf(-l, x[j], s1);
                            else if ((j & 3) == 2) s2 = fmaf(-l, x[j], s2);
                            else s3 = fmaf(-l, x[j], s3);
                        }
                        x[i] = (s0 + s1) + (s2 + s3);
                    }
                    const float bc = sm.beta[lane];
#pragma unroll
                    for (int i = 0; i < TC; ++i) sm.t2[i][lane] = __float2bfloat16_rn(x[i] * bc);
                }
            } else {
                uint32_t* mw = reinterpret_cast<uint32_t*>(&sm.mq[0][0]);        // 12 words per row
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    mw[g * 12 + 4 * ni + t] = pack_bf16(acc[ni][0], acc[ni][1]);
                    mw[(g + 8) * 12 + 4 * ni + t] = pack_bf16(acc[ni][2], acc[ni][3]);
                }
            }
        }
        // meanwhile the previous chunk is finished: its gated RMSNorm, seven tokens each on warps 2 and 3 and two behind
        // the Gram work of warp 1 (warp 0 has the inverse)
        if (chunk > 0) {
            bool ok;
            if (warp == 0) ok = true;
            else if (warp == 1) ok = gated_norm(chunk - 1, 14, std::integral_constant<int, 2>());
            else ok = gated_norm(chunk - 1, 7 * (warp - 2), std::integral_constant<int, 7>());
            if (!ok) atomicCAS(&g_scan_mma_status, 0, 2);
        }
        // ---------------------------------------------------------------- R^T = S0^T K^T and (Q S0)^T, all warps
        float R[2][2][4], QS[2][2][4];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) { R[mi][ni][e] = 0.0f; QS[mi][ni][e] = 0.0f; }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t bk[2][2], bq[2][2];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                bk[ni][0] = kbw[(8 * ni + g) * 36 + 8 * p + t]; bk[ni][1] = kbw[(8 * ni + g) * 36 + 8 * p + t + 4];
                bq[ni][0] = qbw[(8 * ni + g) * 36 + 8 * p + t]; bq[ni][1] = qbw[(8 * ni + g) * 36 + 8 * p + t + 4];
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                // keys 16p .. 16p+15 of the state as an A fragment: two adjacent accumulator tiles, rounded to bf16
                const uint32_t sa[4] = {pack_bf16(S[mi][2 * p][0], S[mi][2 * p][1]), pack_bf16(S[mi][2 * p][2], S[mi][2 * p][3]),
                                        pack_bf16(S[mi][2 * p + 1][0], S[mi][2 * p + 1][1]),
                                        pack_bf16(S[mi][2 * p + 1][2], S[mi][2 * p + 1][3])};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    mma16816(R[mi][ni], sa, bk[ni][0], bk[ni][1]);
                    mma16816(QS[mi][ni], sa, bq[ni][0], bq[ni][1]);
                }
            }
        }
        __syncthreads();                                  // T2 and the masked Q K^T tile are in shared memory
        // ---------------------------------------------------------------- U^T = (V - diag(e) R)^T T2^T
        const uint32_t* t2w = reinterpret_cast<const uint32_t*>(&sm.t2[0][0]);   // 12 words per row
        const uint32_t* mqw = reinterpret_cast<const uint32_t*>(&sm.mq[0][0]);
        const uint32_t* ktw = reinterpret_cast<const uint32_t*>(&sm.kt[0][0]);
        // per-token scalars of this lane's tokens 8 ni + 2t, + 1, with the norms folded in:
        //   er = exp(c) / |k|  (R = K S0),  eq = exp(c) * 0.125 / |q|  (Q S0),  dj2 = exp(c_last - c) / |k|  (state update)
        float er[2][2], eq[2][2], dj2[2][2], ikt[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = 8 * ni + 2 * t + e;
                const float egv = sm.eg[tok], ikv = sm.ik[tok];
                er[ni][e] = egv * ikv;
                eq[ni][e] = egv * sm.iq[tok];
                dj2[ni][e] = sm.dj[tok] * ikv;
                ikt[ni][e] = ikv;
            }
        uint32_t bt[2][2], bm[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            bt[ni][0] = t2w[(8 * ni + g) * 12 + t]; bt[ni][1] = t2w[(8 * ni + g) * 12 + t + 4];
            bm[ni][0] = mqw[(8 * ni + g) * 12 + t]; bm[ni][1] = mqw[(8 * ni + g) * 12 + t + 4];
        }
        float* otile = &b.v[0][0];                        // raw v is consumed: the tile now collects o[token][value]
        float sq[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};    // sum of o^2 over this thread's value rows, per token 8 ni + 2t + e
        uint32_t da[2][4];                                // decay-scaled U^T as A fragments, for the state update
        // every shared-memory load of this phase is issued before its first o-tile store (a store would hold back the
        // loads behind it): V^T for both row halves and the K^T fragments of the state update
        float2 vv[2][2][2];
        uint32_t kf[8][2];
#pragma unroll
        for (int nj = 0; nj < 8; ++nj) { kf[nj][0] = ktw[(8 * nj + g) * 12 + t]; kf[nj][1] = ktw[(8 * nj + g) * 12 + t + 4]; }
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                vv[mi][ni][0] = *reinterpret_cast<const float2*>(&sm.vt[dvb + 16 * mi + g][8 * ni + 2 * t]);
                vv[mi][ni][1] = *reinterpret_cast<const float2*>(&sm.vt[dvb + 16 * mi + g + 8][8 * ni + 2 * t]);
            }
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
            const int r0 = dvb + 16 * mi + g, r1 = r0 + 8;
            uint32_t va[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                const float2 v0 = vv[mi][ni][0];
                const float2 v1 = vv[mi][ni][1];
                va[2 * ni] = pack_bf16(v0.x - er[ni][0] * R[mi][ni][0], v0.y - er[ni][1] * R[mi][ni][1]);
                va[2 * ni + 1] = pack_bf16(v1.x - er[ni][0] * R[mi][ni][2], v1.y - er[ni][1] * R[mi][ni][3]);
            }
            float U[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
                for (int e = 0; e < 4; ++e) U[ni][e] = 0.0f;
                mma16816(U[ni], va, bt[ni][0], bt[ni][1]);
            }
            uint32_t ua[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                ua[2 * ni] = pack_bf16(U[ni][0] * ikt[ni][0], U[ni][1] * ikt[ni][1]);      // U / |k| for the O product
                ua[2 * ni + 1] = pack_bf16(U[ni][2] * ikt[ni][0], U[ni][3] * ikt[ni][1]);
                da[mi][2 * ni] = pack_bf16(U[ni][0] * dj2[ni][0], U[ni][1] * dj2[ni][1]);
                da[mi][2 * ni + 1] = pack_bf16(U[ni][2] * dj2[ni][0], U[ni][3] * dj2[ni][1]);
            }
            // O^T = U^T M^T + diag(e) (Q S0)^T
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                float O[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma16816(O, ua, bm[ni][0], bm[ni][1]);
                const int tok = 8 * ni + 2 * t;
                const float o00 = O[0] + eq[ni][0] * QS[mi][ni][0], o01 = O[1] + eq[ni][1] * QS[mi][ni][1];
                const float o10 = O[2] + eq[ni][0] * QS[mi][ni][2], o11 = O[3] + eq[ni][1] * QS[mi][ni][3];
                otile[tok * OT_PITCH + r0] = o00;
                otile[(tok + 1) * OT_PITCH + r0] = o01;
                otile[tok * OT_PITCH + r1] = o10;
                otile[(tok + 1) * OT_PITCH + r1] = o11;
                sq[ni][0] = fmaf(o00, o00, fmaf(o10, o10, sq[ni][0]));
                sq[ni][1] = fmaf(o01, o01, fmaf(o11, o11, sq[ni][1]));
            }
        }
        // ---------------------------------------------------------------- S^T <- e_last S^T + (diag(d) U)^T K
        {
            const float elast = sm.eg[TC - 1];
#pragma unroll
            for (int nj = 0; nj < 8; ++nj) {
                const uint32_t b0 = kf[nj][0], b1 = kf[nj][1];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mi][nj][e] *= elast;
                    mma16816(S[mi][nj], da[mi], b0, b1);
                }
            }
        }
        // this warp's share of sum(o^2): reduce over the eight row groups g (lane bits 2-4), lanes 0-3 publish it
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = sq[ni][e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (g == 0) sm.ssq[8 * ni + 2 * t + e][warp] = v;
            }
        __syncthreads();                                  // o tile complete; operand tiles free for the next chunk
    }
    if (!gated_norm(NCHUNK - 1, 4 * warp, std::integral_constant<int, 4>())) atomicCAS(&g_scan_mma_status, 0, 2);
}

}  // namespace

int launch_gdn_scan_mma(const float* P, const float* conv_w, const float* conv_b, const float* a_log, const float* dt_bias,
                        const float* o_norm_w, void* on, int on_dtype, int B, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (reinterpret_cast<uintptr_t>(P) & 15) return int(cudaErrorInvalidValue);
    MmaMaps maps;
    const long long rows = (long long)B * kTok;
    if (!tma::make_map_f32(&maps.qk, P, rows, kGLD, kGLD, TC, kDK) || !tma::make_map_f32(&maps.vg, P, rows, kGLD, kGLD, TC, kDV) ||
        !tma::make_map_f32(&maps.ab, P, rows, kGLD, kGLD, TC, 16))
        return int(cudaErrorNotSupported);
    const unsigned grid = unsigned(B) * kHeads;
    if (on_dtype == DT_BF16) {
        const cudaError_t e = cudaFuncSetAttribute(gdn_scan_mma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        gdn_scan_mma_kernel<__nv_bfloat16><<<grid, 128, MMA_SMEM_BYTES, stream>>>(maps, conv_w, conv_b, a_log, dt_bias, o_norm_w,
                                                                                   static_cast<__nv_bfloat16*>(on));
    } else if (on_dtype == DT_F16) {
        const cudaError_t e = cudaFuncSetAttribute(gdn_scan_mma_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        gdn_scan_mma_kernel<__half><<<grid, 128, MMA_SMEM_BYTES, stream>>>(maps, conv_w, conv_b, a_log, dt_bias, o_norm_w,
                                                                           static_cast<__half*>(on));
    } else {
        return int(cudaErrorInvalidValue);
    }
    return int(cudaGetLastError());
}

int* gdn_scan_mma_status_word() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scan_mma_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

int gdn_scan_mma_status(int* status_out) {
    int v = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&v, g_scan_mma_status, sizeof(int));
    if (status_out) *status_out = v;
    return int(e);
}

}  // namespace sb
