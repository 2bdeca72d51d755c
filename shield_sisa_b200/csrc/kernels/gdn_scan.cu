// Fused GatedDeltaNet core: short conv + SiLU, q/k L2 norm, decay/beta gates, gated delta rule, gated RMSNorm.
//
// One CTA owns one (clip, head) and walks the 321 tokens in chunks of 16.  Thread c (128 threads) owns value
// column c of the head and keeps the 64 state entries S[0..63][c] in registers for the whole sequence, so the two
// contractions over the key dimension (the prediction S^T k and the readout S^T q) are private fma chains: no
// shuffle and no barrier sits inside the token loop.  Per chunk:
//   prep   threads 0-63 / 64-127 convolve + SiLU one q / k channel each (sliding window of the three previous raw
//          projections lives in registers across chunks), the 64-wide sums of squares are combined through shared
//          memory, normalised q (scaled by 1/8) and k go to shared memory; every thread convolves its own v column;
//          threads 0-15 evaluate decay and beta of one token each.
//   scan   u = beta (v - a * pred); S <- a S + k u^T; o = S^T q; and in the same sweep over the state the prediction
//          for the next token, S^T k_next (the formulation of engine/model/isa_impl.hpp:914-947).  The first token
//          of a chunk computes its prediction from the state directly.
//   post   one warp per token: rstd over the head's 128 outputs, times o_norm weight, times SiLU of the output gate
//          (read straight from the projection buffer), written in the storage type.
// Same arithmetic as engine/cuda/seq.cu:72-214 and oracle/shieldv_ref.py:121-163,186-197.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int TC = 16;   // tokens per chunk

struct ScanSmem {
    float q[TC][kDK];
    float k[TC + 1][kDK];          // row TC: unused slot that keeps the look-ahead read of the last token in bounds
    float v[TC][kDV];
    float o[TC][kDV];
    float part[TC][4];             // per-warp partial sums of squares (warps 0,1: q; warps 2,3: k)
    float decay[TC], beta[TC];
};

template <typename T>
__global__ void __launch_bounds__(128)
gdn_scan_kernel(const float* __restrict__ P, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ o_norm_w,
                T* __restrict__ on) {
    __shared__ __align__(16) ScanSmem sm;
    const int clip = blockIdx.x / kHeads, head = blockIdx.x % kHeads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* P0 = P + (long long)clip * kTok * kGLD;

    // q / k channel of this thread (prep role) and its conv taps; tap j multiplies x[t - 3 + j]
    const bool is_k = tid >= kDK;
    const int qk_ch = head * kDK + (tid & (kDK - 1));
    const int qk_col = (is_k ? kGK : kGQ) + qk_ch;
    const int qk_w = (is_k ? 384 : 0) + qk_ch;
    const float4 wqk = *reinterpret_cast<const float4*>(conv_w + qk_w * 4);
    const float bqk = conv_b[qk_w];
    // v column of this thread
    const int v_col = kGV + head * kDV + tid;
    const int v_w = 768 + head * kDV + tid;
    const float4 wv = *reinterpret_cast<const float4*>(conv_w + v_w * 4);
    const float bv = conv_b[v_w];
    float x1 = 0.0f, x2 = 0.0f, x3 = 0.0f;   // raw q/k projection at t-1, t-2, t-3
    float y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;   // raw v projection at t-1, t-2, t-3
    const float neg_rate = -expf(a_log[head]), dtb = dt_bias[head];

    float S[kDK];
#pragma unroll
    for (int j = 0; j < kDK; ++j) S[j] = 0.0f;

    for (int t0 = 0; t0 < kTok; t0 += TC) {
        const int nt = min(TC, kTok - t0);
        // ---------------------------------------------------------------- prep
        float val[TC];
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            float raw_qk = 0.0f, raw_v = 0.0f;
            if (i < nt) {
                const float* row = P0 + (long long)(t0 + i) * kGLD;
                raw_qk = row[qk_col];
                raw_v = row[v_col];
            }
            // zero history before t = 0 makes the skipped taps of the causal conv vanish
            float acc = wqk.x * x3;
            acc = fmaf(wqk.y, x2, acc);
            acc = fmaf(wqk.z, x1, acc);
            acc = fmaf(wqk.w, raw_qk, acc);
            val[i] = silu_f(acc + bqk);
            x3 = x2; x2 = x1; x1 = raw_qk;
            float accv = wv.x * y3;
            accv = fmaf(wv.y, y2, accv);
            accv = fmaf(wv.z, y1, accv);
            accv = fmaf(wv.w, raw_v, accv);
            sm.v[i][tid] = silu_f(accv + bv);
            y3 = y2; y2 = y1; y1 = raw_v;
            const float ss = warp_sum(val[i] * val[i]);
            if (lane == 0) sm.part[i][warp] = ss;
        }
        if (tid < nt) {
            const float* row = P0 + (long long)(t0 + tid) * kGLD;
            sm.decay[tid] = expf(neg_rate * softplus_f(row[kGA + head] + dtb));
            sm.beta[tid] = sigmoid_f(row[kGB + head]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            const float tot = is_k ? sm.part[i][2] + sm.part[i][3] : sm.part[i][0] + sm.part[i][1];
            const float inv = 1.0f / sqrtf(tot + 1e-6f);
            if (is_k) sm.k[i][tid - kDK] = val[i] * inv;
            else sm.q[i][tid] = (val[i] * inv) * 0.125f;
        }
        __syncthreads();
        // ---------------------------------------------------------------- scan
        float pred = 0.0f;
        {
            float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
            for (int j = 0; j < kDK; j += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(&sm.k[0][j]);
                p0 = fmaf(S[j], kk.x, p0); p1 = fmaf(S[j + 1], kk.y, p1);
                p2 = fmaf(S[j + 2], kk.z, p2); p3 = fmaf(S[j + 3], kk.w, p3);
            }
            pred = (p0 + p1) + (p2 + p3);
        }
        for (int i = 0; i < nt; ++i) {
            const float a = sm.decay[i];
            const float u = (sm.v[i][tid] - a * pred) * sm.beta[i];
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f, n0 = 0.0f, n1 = 0.0f, n2 = 0.0f, n3 = 0.0f;
#pragma unroll
            for (int j = 0; j < kDK; j += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(&sm.k[i][j]);
                const float4 qq = *reinterpret_cast<const float4*>(&sm.q[i][j]);
                const float4 kn = *reinterpret_cast<const float4*>(&sm.k[i + 1][j]);
                const float s0 = fmaf(kk.x, u, S[j] * a), s1 = fmaf(kk.y, u, S[j + 1] * a);
                const float s2 = fmaf(kk.z, u, S[j + 2] * a), s3 = fmaf(kk.w, u, S[j + 3] * a);
                S[j] = s0; S[j + 1] = s1; S[j + 2] = s2; S[j + 3] = s3;
                o0 = fmaf(s0, qq.x, o0); o1 = fmaf(s1, qq.y, o1); o2 = fmaf(s2, qq.z, o2); o3 = fmaf(s3, qq.w, o3);
                n0 = fmaf(s0, kn.x, n0); n1 = fmaf(s1, kn.y, n1); n2 = fmaf(s2, kn.z, n2); n3 = fmaf(s3, kn.w, n3);
            }
            sm.o[i][tid] = (o0 + o1) + (o2 + o3);
            pred = (n0 + n1) + (n2 + n3);
        }
        __syncthreads();
        // ---------------------------------------------------------------- post: gated RMSNorm, warp per token
        for (int i = warp; i < nt; i += 4) {
            const long long row = (long long)clip * kTok + t0 + i;
            const float4 o = *reinterpret_cast<const float4*>(&sm.o[i][lane * 4]);
            const float4 g = *reinterpret_cast<const float4*>(P + row * kGLD + kGG + head * kDV + lane * 4);
            const float4 w = *reinterpret_cast<const float4*>(o_norm_w + lane * 4);
            const float ss = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
            const float rstd = 1.0f / sqrtf(ss / float(kDV) + 1e-6f);
            store_quad<T>(on + row * kVD + head * kDV + lane * 4, ((o.x * rstd) * w.x) * silu_f(g.x),
                          ((o.y * rstd) * w.y) * silu_f(g.y), ((o.z * rstd) * w.z) * silu_f(g.z),
                          ((o.w * rstd) * w.w) * silu_f(g.w));
        }
        // the next chunk's prep writes v/part before its first barrier; o is rewritten only after two more barriers
    }
}

}  // namespace
}  // namespace sb

extern "C" int shvk_gdn_scan(const float* P, const float* conv_w, const float* conv_b, const float* a_log,
                             const float* dt_bias, const float* o_norm_w, void* on, int on_dtype, int B, void* stream) {
    if (B <= 0) return 0;
    const unsigned grid = unsigned(B) * sb::kHeads;
    SB_DISPATCH_DTYPE(on_dtype, T, (sb::gdn_scan_kernel<T><<<grid, 128, 0, cudaStream_t(stream)>>>(
                                       P, conv_w, conv_b, a_log, dt_bias, o_norm_w, static_cast<T*>(on))));
    return int(cudaGetLastError());
}
