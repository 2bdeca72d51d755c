// SISA attention for the readout row (token 320), one CTA per (clip, head).
//
// Only row 320 leaves the SISA block, so Q and C exist for that row alone while K, V, B, theta, alpha and forget
// cover all 321 rows (engine/cuda/engine.cu:445-453; engine/model/isa_impl.hpp:996-1069).  Phases:
//   1  per-token terms -softplus(alpha), logsigmoid(forget), theta[16] -> shared memory (fp32)
//   2  18 inclusive prefix sums over the 321 tokens, accumulated in double and rounded to fp32 per element (the
//      cumsum semantics both reference engines keep, seq.cu:249-258).  A warp scans one column: each lane sums 11
//      consecutive tokens, a shuffle scan combines the lane totals, all in double.
//   3  rotate C (row 320) by phi[320]; per token rotate B by phi[t], score = q.k/8 + softplus(lambda) *
//      exp(g_last - g_t) * (c_rot . b_rot) + (f_last - f_t); eight threads per token, 16 bytes of K each
//   4  softmax over the 321 scores, y = sum_t p_t v_t: eight threads per token row, 24 tokens per round
//
// Two row formats.  fp32 (exact tier): one row [K | V | B | theta | alpha | forget] of 1,072 floats per token.  16-bit
// modes: K, V, B travel as fp16 in a row of 960 halves (S16) and theta, alpha, forget as fp32 in a row of 112 floats
// (SG), 2,368 instead of 4,288 bytes per token; the arithmetic is the same fp32 arithmetic on the widened values.
#include "device_utils.cuh"

#include <cuda_fp16.h>
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int NT = 192, NCOL = 18, PER_LANE = 11;   // 32 * 11 = 352 >= 321
constexpr int VSLOTS = NT / 8;                       // tokens of the value sum in flight: eight threads share a token's 64 values
constexpr int kS16LD = 960, kSGLD = 112;             // row pitches of the split format; SG = [theta 96 | alpha 6 | forget 6 | pad 4]

// Eight consecutive K or B values of a token row, widened to fp32.
template <bool H16> struct Row8;
template <> struct Row8<false> {
    static __device__ __forceinline__ void load(const void* base, int i, float (&v)[8]) {
        const float4* p = static_cast<const float4*>(base) + 2 * i;
        const float4 a = p[0], b = p[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Row8<true> {
    static __device__ __forceinline__ void load(const void* base, int i, float (&v)[8]) {
        const uint4 u = static_cast<const uint4*>(base)[i];
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            v[2 * e] = f.x; v[2 * e + 1] = f.y;
        }
    }
};

// sin and cos of a phase: reduction to [-pi, pi] with 2 pi split in two (exact to about 1e-7 for the phases that occur,
// cumulative sums of theta over 321 tokens), then the hardware approximations (absolute error below 4e-7 on that range).
// sincosf costs about 45 instructions, and a token needs sixteen of them.
__device__ __forceinline__ void sincos_phase(float x, float& sn, float& cs) {
    const float k = rintf(x * 0.15915494309189535f);
    float r = fmaf(k, -6.2831854820251465f, x);       // fp32(2 pi) = 2 pi + 1.7484555e-7
    r = fmaf(k, 1.7484555e-7f, r);
    sn = __sinf(r);
    cs = __cosf(r);
}

// Four consecutive B values of a token row, widened to fp32.
template <bool H16> struct Row4;
template <> struct Row4<false> {
    static __device__ __forceinline__ void load(const void* base, int i, float (&v)[4]) {
        const float4 a = static_cast<const float4*>(base)[i];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
};
template <> struct Row4<true> {
    static __device__ __forceinline__ void load(const void* base, int i, float (&v)[4]) {
        const uint2 u = static_cast<const uint2*>(base)[i];
        const __half2* h = reinterpret_cast<const __half2*>(&u);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]);
        v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    }
};

// Four CTAs of 192 threads per SM: the phases of one CTA alternate between loads and scans, and more resident CTAs keep
// HBM busy through the scans.  B = 4096, 16-bit rows: a thread per token with sincosf and a value sum of one column per
// thread 1.18 ms (256 threads x 4 CTAs; 352 x 3 1.16, 352 x 2 1.45, 192 x 5 1.10); hardware sin / cos and 16-byte value
// reads 0.98 ms; eight threads per token in the score phase as well 0.73 ms (four, five and six CTAs per SM the same).
template <bool H16>
__global__ void __launch_bounds__(NT, 4)
sisa_attn_kernel(const void* __restrict__ Skvb, const float* __restrict__ Sgate, const float* __restrict__ QC,
                 const float* __restrict__ lambda_raw, float* __restrict__ Y) {
    using KV = typename std::conditional<H16, __half, float>::type;
    constexpr int LDK = H16 ? kS16LD : kSLD;                 // pitch of the K | V | B row (elements of KV)
    constexpr int LDG = H16 ? kSGLD : kSLD;                  // pitch of the theta | alpha | forget row (floats)
    constexpr int G0 = H16 ? 0 : kSTheta;                    // column of theta in that row
    const int clip = blockIdx.x / kHeads, head = blockIdx.x % kHeads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const KV* S0 = static_cast<const KV*>(Skvb) + (long long)clip * kTok * LDK;
    const float* SG0 = Sgate + (long long)clip * kTok * LDG;
    __shared__ float term[NCOL][kTok + 3];     // column-major: a scan walks one row of this array
    __shared__ float score[kTok];
    __shared__ __align__(16) float sq[kDK];
    __shared__ __align__(16) float sc[kState];
    __shared__ float red[NT / 32];
    __shared__ float ypart[NT / 32][kDK];

    // per-token terms: theta[16] of this head is one 64-byte run, alpha and forget are single floats
    for (int tk = tid; tk < kTok; tk += NT) {
        const float* row = SG0 + (long long)tk * LDG + G0;
        const float4* th = reinterpret_cast<const float4*>(row + head * kPairs);
        const float4 t0 = th[0], t1 = th[1], t2 = th[2], t3 = th[3];
        const float al = row[kSAlpha - kSTheta + head], fg = row[kSForget - kSTheta + head];
        term[0][tk] = -softplus_f(al);
        term[1][tk] = logsigmoid_f(fg);
        term[2][tk] = t0.x; term[3][tk] = t0.y; term[4][tk] = t0.z; term[5][tk] = t0.w;
        term[6][tk] = t1.x; term[7][tk] = t1.y; term[8][tk] = t1.z; term[9][tk] = t1.w;
        term[10][tk] = t2.x; term[11][tk] = t2.y; term[12][tk] = t2.z; term[13][tk] = t2.w;
        term[14][tk] = t3.x; term[15][tk] = t3.y; term[16][tk] = t3.z; term[17][tk] = t3.w;
    }
    if (tid < kDK) sq[tid] = QC[(long long)clip * kSQN + kSQ + head * kDK + tid];
    else if (tid < kDK + kState) sc[tid - kDK] = QC[(long long)clip * kSQN + kSC + head * kState + (tid - kDK)];
    __syncthreads();

    for (int c = warp; c < NCOL; c += NT / 32) {
        const int t0 = lane * PER_LANE;
        double loc[PER_LANE];
        double run = 0.0;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int t = t0 + i;
            run += t < kTok ? double(term[c][t]) : 0.0;
            loc[i] = run;
        }
        double incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const double base = incl - run;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int t = t0 + i;
            if (t < kTok) term[c][t] = float(base + loc[i]);
        }
    }
    __syncthreads();

    if (tid < kPairs) {
        float si, co;
        sincos_phase(term[2 + tid][kTok - 1], si, co);
        const float e = sc[2 * tid], o = sc[2 * tid + 1];
        __syncwarp(0x0000ffffu);
        sc[2 * tid] = e * co - o * si;
        sc[2 * tid + 1] = e * si + o * co;
    }
    __syncthreads();

    const float lam = softplus_f(lambda_raw[head]);
    const float g_last = term[0][kTok - 1], f_last = term[1][kTok - 1];
    // scores: eight threads per token (16 bytes of K and two of the sixteen state pairs each), VSLOTS tokens per round;
    // a warp then reads four whole rows per instruction instead of 32 different ones
    float lmax = -INFINITY;
    {
        const int part = tid & 7, slot = tid >> 3;
        float q8[8], c4[4];
#pragma unroll
        for (int e = 0; e < 8; ++e) q8[e] = sq[8 * part + e];
#pragma unroll
        for (int e = 0; e < 4; ++e) c4[e] = sc[4 * part + e];
#pragma unroll 2
        for (int t0 = 0; t0 < kTok; t0 += VSLOTS) {
            const int t = t0 + slot;
            float content = 0.0f, ssm = 0.0f;
            if (t < kTok) {
                float kk[8], bb[4];
                Row8<H16>::load(S0 + (long long)t * LDK + kSK + head * kDK, part, kk);
                Row4<H16>::load(S0 + (long long)t * LDK + kSB + head * kState, part, bb);
#pragma unroll
                for (int e = 0; e < 8; ++e) content = fmaf(q8[e], kk[e], content);
#pragma unroll
                for (int e = 0; e < 2; ++e) {             // pair 2 part + e: (bb[2e], bb[2e+1]) rotated by phi of that pair
                    float sn, cs;
                    sincos_phase(term[2 + 2 * part + e][t], sn, cs);
                    ssm = fmaf(c4[2 * e], bb[2 * e] * cs - bb[2 * e + 1] * sn, ssm);
                    ssm = fmaf(c4[2 * e + 1], bb[2 * e] * sn + bb[2 * e + 1] * cs, ssm);
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                content += __shfl_xor_sync(0xffffffffu, content, o);
                ssm += __shfl_xor_sync(0xffffffffu, ssm, o);
            }
            if (part == 0 && t < kTok) {
                float sv = content * 0.125f + (lam * expf(g_last - term[0][t])) * ssm;
                sv = sv + (f_last - term[1][t]);
                score[t] = sv;
                lmax = fmaxf(lmax, sv);
            }
        }
    }
    lmax = warp_max(lmax);
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float mx = red[0];
#pragma unroll
    for (int i = 1; i < NT / 32; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float lsum = 0.0f;
    for (int t = tid; t < kTok; t += NT) {
        const float e = expf(score[t] - mx);
        score[t] = e;
        lsum += e;
    }
    lsum = warp_sum(lsum);
    if (lane == 0) red[warp] = lsum;
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NT / 32; ++i) sum += red[i];
    const float inv = 1.0f / sum;
    // y = sum_t p_t v_t: eight threads share a token's 64 values (16 bytes each in the 16-bit format), VSLOTS tokens per
    // round; the token slots of a warp are added by shuffles, the warps through shared memory
    const int part = tid & 7, slot = tid >> 3;
    float y[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = 0.0f;
#pragma unroll 4
    for (int t = slot; t < kTok; t += VSLOTS) {
        float vv[8];
        Row8<H16>::load(S0 + (long long)t * LDK + kSV + head * kDK, part, vv);
        const float pt = score[t] * inv;
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = fmaf(pt, vv[e], y[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        y[e] += __shfl_xor_sync(0xffffffffu, y[e], 8);
        y[e] += __shfl_xor_sync(0xffffffffu, y[e], 16);
    }
    if (lane < 8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ypart[warp][8 * lane + e] = y[e];
    }
    __syncthreads();
    if (tid < kDK) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) acc += ypart[w][tid];
        Y[(long long)clip * kD + head * kDK + tid] = acc;
    }
}

}  // namespace
}  // namespace sb

extern "C" int shvk_sisa_attn(const float* S, const float* QC, const float* lambda_raw, float* Y, int B, void* stream) {
    if (B <= 0) return 0;
    sb::sisa_attn_kernel<false><<<unsigned(B) * sb::kHeads, sb::NT, 0, cudaStream_t(stream)>>>(S, S, QC, lambda_raw, Y);
    return int(cudaGetLastError());
}

extern "C" int shvk_sisa_attn_h16(const void* S16, const float* SG, const float* QC, const float* lambda_raw, float* Y, int B,
                                  void* stream) {
    if (B <= 0) return 0;
    if (!S16 || !SG || ((reinterpret_cast<uintptr_t>(S16) | reinterpret_cast<uintptr_t>(SG)) & 15)) return int(cudaErrorInvalidValue);
    sb::sisa_attn_kernel<true><<<unsigned(B) * sb::kHeads, sb::NT, 0, cudaStream_t(stream)>>>(S16, SG, QC, lambda_raw, Y);
    return int(cudaGetLastError());
}
