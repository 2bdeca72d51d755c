// Fused GatedDeltaNet core: short conv + SiLU, q/k L2 norm, decay/beta gates, gated delta rule, gated RMSNorm.
//
// One CTA (128 threads) owns one (clip, head) and walks the 321 tokens in chunks of 16.
//
// Data movement.  The chunk's slices of the fused projection P (q 16x64, k 16x64, v 16x128, output gate 16x128, a|b
// 16x16, all fp32) are brought into shared memory by five TMA tile loads that complete on an mbarrier; the loads of
// chunk c+1 are issued before chunk c is processed (two buffers), so no thread ever waits on a global load inside
// the token loop.  Everything is then converted in place: conv+SiLU overwrites the raw q, k, v; the delta-rule output
// overwrites v; the gated norm reads it back with the gate tile and writes the result to global memory.
//
// Arithmetic.  The head's 64 x 128 state stays in registers for the whole sequence: thread (g, s) with g = tid / 4,
// s = tid % 4 holds 16 keys x 4 value columns of it, keys {16 j + 4 s + e : j, e < 4} (the four slices interleave at
// float4 granularity, so that the slices' 128-bit reads of one k or q row fall on distinct banks) and columns
// 4g .. 4g+3, as eight float2 pairs along the key dimension, so the
// update and the two contractions over keys run as packed fp32x2 FMAs (fma.rn.f32x2) whose k / q operands come
// straight out of 128-bit shared-memory loads (13 per token per thread), followed by a two-step shuffle reduction
// over the four key slices.  The L2 normalisations are folded into scalars: with kr, qr the un-normalised conv
// outputs and ik = 1/sqrt(|kr|^2 + 1e-6), iq = 0.125/sqrt(|qr|^2 + 1e-6),
//     pred = ik_t (S^T kr_t),  u = beta (v - a pred),  S <- a S + kr_t (ik_t u)^T,  o = iq_t (S^T qr_t),
// and the sweep that updates S also accumulates S^T kr_{t+1} for the next token's prediction (the one-pass
// formulation of engine/model/isa_impl.hpp:914-947).  The first token of a chunk predicts from the state directly.
//
// Same function as engine/cuda/seq.cu:72-214 (gdn_prep + delta + gated_norm) and oracle/shieldv_ref.py:121-163,186-197.
// SiLU uses the hardware exponential and reciprocal (relative error of a few 1e-7, far inside the 1e-4 budget of the
// exact tier); the gates, square roots and divisions of the norms are IEEE.
//
// A wait on a TMA barrier is bounded; if it gives up the CTA records it in a status word and returns.
#include "device_utils.cuh"

#include <atomic>
#include "shv_seq_kernels.h"
#include "tma_utils.cuh"
#include "status_words.cuh"

#include <stdlib.h>

namespace sb {
namespace {

constexpr int TC = 16;                       // tokens per chunk
constexpr uint32_t WAIT_POLLS = 1u << 22;    // about a quarter second

__device__ int g_scan_status = 0;

struct ChunkBuf {                            // one chunk of projections; every tile is the target of one TMA load
    float q[TC][kDK];                        // raw q  -> silu(conv q), un-normalised
    float k[TC][kDK];                        // raw k  -> silu(conv k), un-normalised (the look-ahead read of the last
                                             //           token runs one row past the tile, into v: discarded)
    float v[TC][kDV];                        // raw v  -> silu(conv v) -> delta-rule output o
    float g[TC][kDV];                        // output gate projection
    float ab[TC][16];                        // a[6] | b[6] | 4 pad columns
};
static_assert(sizeof(ChunkBuf) == 25600 && sizeof(ChunkBuf) % 128 == 0, "tile offsets must stay 128-byte aligned");

struct ScanSmem {
    ChunkBuf buf[2];
    float part[TC][4];                       // per-warp sums of squares (warps 0,1: q; warps 2,3: k)
    float iq[TC], ik[TC + 1];                // 0.125 / |q|, 1 / |k|  (ik[TC] only feeds a discarded look-ahead)
    float decay[TC], beta[TC];
    unsigned long long full[2];              // mbarriers: chunk data landed
};
constexpr int SCAN_SMEM_BYTES = int(sizeof(ScanSmem)) + 128;

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(*reinterpret_cast<uint64_t*>(&d))
        : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)), "l"(*reinterpret_cast<uint64_t*>(&c)));
    return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(*reinterpret_cast<uint64_t*>(&d))
        : "l"(*reinterpret_cast<uint64_t*>(&a)), "l"(*reinterpret_cast<uint64_t*>(&b)));
    return d;
}
__device__ __forceinline__ float quad_sum(float v) {      // over the four key slices (lanes differing in bits 0-1)
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
// x * sigmoid(x) with the hardware exp2 and reciprocal
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

struct ScanMaps {
    CUtensorMap qk;    // box 16 x 64
    CUtensorMap vg;    // box 16 x 128
    CUtensorMap ab;    // box 16 x 16
};

template <typename T>
__global__ void __launch_bounds__(128, 4)
gdn_scan_kernel(const __grid_constant__ ScanMaps maps, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ o_norm_w,
                T* __restrict__ on) {
    extern __shared__ uint8_t scan_smem_raw[];
    ScanSmem& sm = *reinterpret_cast<ScanSmem*>((reinterpret_cast<uintptr_t>(scan_smem_raw) + 127) & ~uintptr_t(127));
    const int clip = blockIdx.x / kHeads, head = blockIdx.x % kHeads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_base = clip * kTok;

    // prep role: q / k channel and v column of this thread, conv taps (tap j multiplies x[t - 3 + j])
    const bool is_k = tid >= kDK;
    const int qk_ch = tid & (kDK - 1);
    const int qk_w = (is_k ? 384 : 0) + head * kDK + qk_ch;
    const float4 wqk = *reinterpret_cast<const float4*>(conv_w + qk_w * 4);
    const float bqk = conv_b[qk_w];
    const int v_w = 768 + head * kDV + tid;
    const float4 wv = *reinterpret_cast<const float4*>(conv_w + v_w * 4);
    const float bv = conv_b[v_w];
    float x1 = 0.0f, x2 = 0.0f, x3 = 0.0f;   // raw q/k projection at t-1, t-2, t-3 (zero history = causal padding)
    float y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;   // raw v projection at t-1, t-2, t-3
    const float neg_rate = -expf(a_log[head]), dtb = dt_bias[head];

    // scan role: key slice ks (keys 16 j + 4 ks + e), value columns [4 cg, 4 cg + 4)
    const int ks = tid & 3, cg = tid >> 2;
    float2 S[8][4];                          // S[2 j + h][c] = state rows 16 j + 4 ks + 2 h, + 1 of column 4 cg + c
#pragma unroll
    for (int jp = 0; jp < 8; ++jp)
#pragma unroll
        for (int c = 0; c < 4; ++c) S[jp][c] = make_float2(0.0f, 0.0f);

    const uint32_t bar0 = tma::smem_addr(&sm.full[0]), bar1 = tma::smem_addr(&sm.full[1]);
    auto issue = [&](int chunk) {            // one thread: five tile loads of `chunk` into buffer chunk & 1
        ChunkBuf& b = sm.buf[chunk & 1];
        const uint32_t bar = (chunk & 1) ? bar1 : bar0;
        const int row = row_base + chunk * TC;
        tma::mbar_expect_tx(bar, uint32_t(sizeof(ChunkBuf)));
        tma::load_2d(tma::smem_addr(&b.q[0][0]), &maps.qk, kGQ + head * kDK, row, bar);
        tma::load_2d(tma::smem_addr(&b.k[0][0]), &maps.qk, kGK + head * kDK, row, bar);
        tma::load_2d(tma::smem_addr(&b.v[0][0]), &maps.vg, kGV + head * kDV, row, bar);
        tma::load_2d(tma::smem_addr(&b.g[0][0]), &maps.vg, kGG + head * kDV, row, bar);
        tma::load_2d(tma::smem_addr(&b.ab[0][0]), &maps.ab, kGA, row, bar);
    };
    if (tid == 0) {
        tma::mbar_init(bar0, 1);
        tma::mbar_init(bar1, 1);
        tma::fence_barrier_init();
        tma::fence_proxy_async();
        issue(0);
    }
    __syncthreads();

    constexpr int NCHUNK = (kTok + TC - 1) / TC;
    for (int chunk = 0; chunk < NCHUNK; ++chunk) {
        const int t0 = chunk * TC, nt = min(TC, kTok - t0);
        ChunkBuf& b = sm.buf[chunk & 1];
        // every thread is done with the other buffer (post of chunk - 1 ended at the barrier closing the last
        // iteration): refill it while this chunk is processed
        if (tid == 0 && chunk + 1 < NCHUNK) {
            tma::fence_proxy_async();
            issue(chunk + 1);
        }
        if (!tma::mbar_wait_bounded((chunk & 1) ? bar1 : bar0, uint32_t(chunk >> 1) & 1u, WAIT_POLLS)) {
            if (tid == 0) atomicCAS(&g_scan_status, 0, 1);
            return;                          // every thread of the CTA times out on the same barrier and leaves
        }
        // ---------------------------------------------------------------- prep, in place
#pragma unroll 4
        for (int i = 0; i < TC; ++i) {
            float* pqk = is_k ? &b.k[i][qk_ch] : &b.q[i][qk_ch];
            const float raw_qk = *pqk, raw_v = b.v[i][tid];
            float acc = wqk.x * x3;
            acc = fmaf(wqk.y, x2, acc);
            acc = fmaf(wqk.z, x1, acc);
            acc = fmaf(wqk.w, raw_qk, acc);
            const float val = silu_fast(acc + bqk);
            *pqk = val;
            x3 = x2; x2 = x1; x1 = raw_qk;
            float accv = wv.x * y3;
            accv = fmaf(wv.y, y2, accv);
            accv = fmaf(wv.z, y1, accv);
            accv = fmaf(wv.w, raw_v, accv);
            b.v[i][tid] = silu_fast(accv + bv);
            y3 = y2; y2 = y1; y1 = raw_v;
            const float ss = warp_sum(val * val);
            if (lane == 0) sm.part[i][warp] = ss;
        }
        if (tid < TC) {
            sm.decay[tid] = expf(neg_rate * softplus_f(b.ab[tid][head] + dtb));
            sm.beta[tid] = sigmoid_f(b.ab[tid][6 + head]);
        }
        __syncthreads();
        if (tid < 2 * TC) {
            const int i = tid & (TC - 1);
            if (tid < TC) sm.iq[i] = (1.0f / sqrtf(sm.part[i][0] + sm.part[i][1] + 1e-6f)) * 0.125f;
            else sm.ik[i] = 1.0f / sqrtf(sm.part[i][2] + sm.part[i][3] + 1e-6f);
        }
        if (tid == 2 * TC) sm.ik[TC] = 0.0f;
        __syncthreads();
        // ---------------------------------------------------------------- scan
        float pred[4];
        {
            float2 acc[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[c] = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int jq = 0; jq < 4; ++jq) {
                const float4 kk = *reinterpret_cast<const float4*>(&b.k[0][(jq * 4 + ks) * 4]);
                const float2 k01 = make_float2(kk.x, kk.y), k23 = make_float2(kk.z, kk.w);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    acc[c] = ffma2(S[2 * jq][c], k01, acc[c]);
                    acc[c] = ffma2(S[2 * jq + 1][c], k23, acc[c]);
                }
            }
            const float ik0 = sm.ik[0];
#pragma unroll
            for (int c = 0; c < 4; ++c) pred[c] = quad_sum(acc[c].x + acc[c].y) * ik0;
        }
        for (int i = 0; i < nt; ++i) {
            const float a = sm.decay[i], bik = sm.beta[i] * sm.ik[i];
            const float4 vv = *reinterpret_cast<const float4*>(&b.v[i][cg * 4]);
            const float2 a2 = make_float2(a, a);
            float2 u2[4], o2[4], n2[4];
            {
                // u = beta (v - a pred), pre-multiplied by 1/|k| because the state is updated with the raw k
                const float u0 = (vv.x - a * pred[0]) * bik, u1 = (vv.y - a * pred[1]) * bik;
                const float u2s = (vv.z - a * pred[2]) * bik, u3 = (vv.w - a * pred[3]) * bik;
                u2[0] = make_float2(u0, u0); u2[1] = make_float2(u1, u1);
                u2[2] = make_float2(u2s, u2s); u2[3] = make_float2(u3, u3);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) { o2[c] = make_float2(0.0f, 0.0f); n2[c] = make_float2(0.0f, 0.0f); }
#pragma unroll
            for (int jq = 0; jq < 4; ++jq) {
                const float4 kk = *reinterpret_cast<const float4*>(&b.k[i][(jq * 4 + ks) * 4]);
                const float4 qq = *reinterpret_cast<const float4*>(&b.q[i][(jq * 4 + ks) * 4]);
                const float4 kn = *reinterpret_cast<const float4*>(&b.k[0][0] + (i + 1) * kDK + (jq * 4 + ks) * 4);
                const float2 kp[2] = {make_float2(kk.x, kk.y), make_float2(kk.z, kk.w)};
                const float2 qp[2] = {make_float2(qq.x, qq.y), make_float2(qq.z, qq.w)};
                const float2 np[2] = {make_float2(kn.x, kn.y), make_float2(kn.z, kn.w)};
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 x = ffma2(kp[h], u2[c], fmul2(S[2 * jq + h][c], a2));
                        S[2 * jq + h][c] = x;
                        o2[c] = ffma2(x, qp[h], o2[c]);
                        n2[c] = ffma2(x, np[h], n2[c]);
                    }
            }
            const float iq = sm.iq[i], ikn = sm.ik[i + 1];
            float o[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                o[c] = quad_sum(o2[c].x + o2[c].y) * iq;
                pred[c] = quad_sum(n2[c].x + n2[c].y) * ikn;
            }
            // All four key slices now hold the sums; slice s stores column 4 cg + s over the v value that this quad
            // (and only this quad) read at the top of the iteration.
            b.v[i][tid] = ks == 0 ? o[0] : ks == 1 ? o[1] : ks == 2 ? o[2] : o[3];
        }
        __syncthreads();
        // ---------------------------------------------------------------- post: gated RMSNorm, warp per token
        for (int i = warp; i < nt; i += 4) {
            const long long row = (long long)row_base + t0 + i;
            const float4 o = *reinterpret_cast<const float4*>(&b.v[i][lane * 4]);
            const float4 g = *reinterpret_cast<const float4*>(&b.g[i][lane * 4]);
            const float4 w = *reinterpret_cast<const float4*>(o_norm_w + lane * 4);
            const float ss = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
            const float rstd = 1.0f / sqrtf(ss / float(kDV) + 1e-6f);
            store_quad<T>(on + row * kVD + head * kDV + lane * 4, ((o.x * rstd) * w.x) * silu_fast(g.x),
                          ((o.y * rstd) * w.y) * silu_fast(g.y), ((o.z * rstd) * w.z) * silu_fast(g.z),
                          ((o.w * rstd) * w.w) * silu_fast(g.w));
        }
        __syncthreads();                     // this buffer may be refilled from the next iteration on
    }
}

}  // namespace
}  // namespace sb

extern "C" int shvk_gdn_scan(const float* P, const float* conv_w, const float* conv_b, const float* a_log,
                             const float* dt_bias, const float* o_norm_w, void* on, int on_dtype, int B, void* stream) {
    using namespace sb;
    if (B <= 0) return 0;
    if (reinterpret_cast<uintptr_t>(P) & 15) return int(cudaErrorInvalidValue);
    // the three tensor maps depend on (P, rows) only: an engine thread launches with the same pair again and again, so
    // the last encoding is kept per thread
    struct Cached { const float* P = nullptr; long long rows = 0; ScanMaps maps; };
    static thread_local Cached cache;
    const long long rows = (long long)B * kTok;
    if (cache.P != P || cache.rows != rows) {
        cache.P = nullptr;
        if (!tma::make_map_f32(&cache.maps.qk, P, rows, kGLD, kGLD, TC, kDK) || !tma::make_map_f32(&cache.maps.vg, P, rows, kGLD, kGLD, TC, kDV) ||
            !tma::make_map_f32(&cache.maps.ab, P, rows, kGLD, kGLD, TC, 16))
            return int(cudaErrorNotSupported);
        cache.P = P; cache.rows = rows;
    }
    const unsigned grid = unsigned(B) * kHeads;
    int dev = 0;
    cudaGetDevice(&dev);
    SB_DISPATCH_DTYPE(on_dtype, T, {
        // the dynamic shared memory opt-in is per device and per instantiation; setting it twice is harmless
        static std::atomic<unsigned long long> attr_done{0};
        if (dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
            const cudaError_t e = cudaFuncSetAttribute(gdn_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM_BYTES);
            if (e != cudaSuccess) return int(e);
            if (dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
        }
        gdn_scan_kernel<T><<<grid, 128, SCAN_SMEM_BYTES, cudaStream_t(stream)>>>(cache.maps, conv_w, conv_b, a_log, dt_bias, o_norm_w,
                                                                                 static_cast<T*>(on));
    });
    return int(cudaGetLastError());
}

namespace sb {
int* gdn_scan_status_word() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scan_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
}  // namespace sb

// Combined status of the two scan kernels: 0, or the word of the kernel that reads the fp32 projection, or 16 + the word
// of the 16-bit kernel that reads operand tiles.
extern "C" int shvk_gdn_scan_status(int* status_out) {
    int v[2] = {0, 0};
    int* words[2] = {sb::gdn_scan_status_word(), sb::gdn_scan_t_status_word()};
    for (int i = 0; i < 2; ++i) {
        if (!words[i]) return int(cudaErrorInvalidSymbol);
        const cudaError_t e = cudaMemcpy(&v[i], words[i], sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return int(e);
    }
    if (status_out) *status_out = v[0] ? v[0] : v[1] ? 16 + v[1] : 0;
    return 0;
}
