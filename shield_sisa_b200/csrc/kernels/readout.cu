// The readout row (token 320) of the SISA block and the classifier head, fp32 in every mode, in two kernels around
// the attention kernel:
//
//   readout_qc    xl = rmsnorm(h[320]) * w;  [Q | C] = xl . W_qc^T                                 (before sisa_attn)
//   readout_tail  x1 = h[320] + Y . W_O^T;  x2 = x1 + down(silu(gate(n)) * up(n)), n = rmsnorm(x1) * w;
//                 z = rmsnorm(x2) * w;  logit = w2 . silu(W0 z + b0) + b2                           (after sisa_attn)
//
// Only row 320 leaves the SISA block, so this work is B rows, not 321 B (engine/cuda/engine.cu:451-469;
// engine/model/isa_impl.hpp:1092-1133).  A CTA takes TB clips (16 when the batch is large enough to give every SM a
// CTA that way, else 4, 2 or 1) and walks the small matrix products one after the other with all activations of its
// clips in shared memory: a thread owns one or two output columns for all TB clips (TB or 2 TB accumulators), reads its
// weights coalesced from a [K][N] (transposed) copy that stays in L2, several steps of k in flight at a time, and the
// activations as 128-bit broadcast loads.  Every output is one fp32 FMA chain over k in ascending order, whatever the
// batch and whatever TB, so a clip's logit does not depend on its neighbours (engine/include/shv_cuda.h:31-34).
//
// Replaces two launch_rmsnorm, five gemm<float> and launch_head of the reference's run_classify
// (engine/cuda/engine.cu:451-469, engine/cuda/seq.cu:309-336).
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

#include <stdlib.h>

namespace sb {
namespace {

constexpr int XP = kD + 4, HP = kDFF + 4;     // row pitches (floats) of the shared-memory activation tiles

// acc[c][e] = sum_k X[c][k] * Wt[k][n0 + e], e < NC, for the TB clips of the tile; k ascending, one FMA chain per output.
template <int K, int NC, int TB>
__device__ __forceinline__ void dot_columns(const float* __restrict__ X, int xp, const float* __restrict__ Wt, int ldw, int n0,
                                            float (&acc)[TB][NC]) {
#pragma unroll
    for (int c = 0; c < TB; ++c)
#pragma unroll
        for (int e = 0; e < NC; ++e) acc[c][e] = 0.0f;
    const float* wp = Wt + n0;
    // The weights of D steps of four k are loaded before the first of them is used, so that D x 4 loads are in flight per
    // thread (with few clips per CTA the kernel is bound by the latency of exactly these loads).  This needs the registers
    // for them: the kernels are declared with a minimum number of CTAs per SM, because without one the assembler keeps the
    // register count low for occupancy by moving every load next to its use, which runs the steps one L2 round trip
    // after the other (B = 512: 0.27 ms for the tail kernel against 0.14 ms).
    constexpr int D = TB >= 8 ? 4 : 8;
    static_assert(K % (4 * D) == 0, "the k loop walks whole groups of steps");
#pragma unroll 1
    for (int k0 = 0; k0 < K; k0 += 4 * D) {
        float w[D][4][NC];
#pragma unroll
        for (int d = 0; d < D; ++d)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if constexpr (NC == 2) {
                    const float2 v = __ldg(reinterpret_cast<const float2*>(wp + (long long)(k0 + 4 * d + i) * ldw));
                    w[d][i][0] = v.x; w[d][i][1] = v.y;
                } else {
                    w[d][i][0] = __ldg(wp + (long long)(k0 + 4 * d + i) * ldw);
                }
            }
#pragma unroll
        for (int d = 0; d < D; ++d)
#pragma unroll
            for (int c = 0; c < TB; ++c) {
                const float4 x = *reinterpret_cast<const float4*>(X + c * xp + k0 + 4 * d);
#pragma unroll
                for (int e = 0; e < NC; ++e) {
                    acc[c][e] = fmaf(x.x, w[d][0][e], acc[c][e]);
                    acc[c][e] = fmaf(x.y, w[d][1][e], acc[c][e]);
                    acc[c][e] = fmaf(x.z, w[d][2][e], acc[c][e]);
                    acc[c][e] = fmaf(x.w, w[d][3][e], acc[c][e]);
                }
            }
    }
}

// out[c] = (in[c] * (1 / sqrt(mean(in[c]^2) + 1e-6))) * w over rows of 384 in shared memory; warp w takes clips w, w + 8.
// A row is read into registers before it is written, so out may be in.
template <int TB, int NT>
__device__ __forceinline__ void norm_rows(const float* in, float* out, const float* __restrict__ w, int warp, int lane) {
    for (int c = warp; c < TB; c += NT / 32) {
        float v[kD / 32];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < kD / 32; ++i) {
            v[i] = in[c * XP + lane + 32 * i];
            ss = fmaf(v[i], v[i], ss);
        }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / float(kD) + 1e-6f);
#pragma unroll
        for (int i = 0; i < kD / 32; ++i) out[c * XP + lane + 32 * i] = (v[i] * r) * __ldg(w + lane + 32 * i);
    }
}

template <int TB, int NT>
__global__ void __launch_bounds__(NT, NT <= 256 ? 2 : 1)
readout_qc_kernel(const float* __restrict__ h_last, long long ldh, const float* __restrict__ norm_w, const float* __restrict__ wqc_t,
                  float* __restrict__ QC, int B) {
    __shared__ __align__(16) float xs[TB * XP];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int clip0 = blockIdx.x * TB;
    for (int i = tid; i < TB * kD; i += NT) {
        const int c = i / kD, k = i - c * kD;
        xs[c * XP + k] = clip0 + c < B ? h_last[(long long)(clip0 + c) * ldh + k] : 0.0f;
    }
    __syncthreads();
    norm_rows<TB, NT>(xs, xs, norm_w, warp, lane);
    __syncthreads();
    for (int n0 = 2 * tid; n0 < kSQN; n0 += 2 * NT) {          // 576 columns = 288 pairs
        float acc[TB][2];
        dot_columns<kD, 2, TB>(xs, XP, wqc_t, kSQN, n0, acc);
#pragma unroll
        for (int c = 0; c < TB; ++c)
            if (clip0 + c < B) *reinterpret_cast<float2*>(QC + (long long)(clip0 + c) * kSQN + n0) = make_float2(acc[c][0], acc[c][1]);
    }
}

struct TailWeights {
    const float *wo_t;          // [384][384]   W_O transposed
    const float *ffn_norm_w;    // [384]
    const float *up_t;          // [384][1920]  gate / up rows interleaved (2j, 2j + 1), transposed
    const float *down_t;        // [960][384]   down projection transposed
    const float *final_norm_w;  // [384]
    const float *head_w0_t;     // [384][128]   head.0 transposed
    const float *head_b0;       // [128]
    const float *head_w2;       // [128]
    const float *head_b2;       // [1]
};

template <int TB, int NT>
__global__ void __launch_bounds__(NT, NT <= 256 ? 2 : 1)
readout_tail_kernel(const float* __restrict__ Y, const float* __restrict__ h_last, long long ldh, const TailWeights tw,
                    float* __restrict__ x2_out, float* __restrict__ logits, int B) {
    extern __shared__ __align__(16) float tail_smem[];
    float* x1 = tail_smem;                  // [TB][XP]  residual stream of the row
    float* xa = x1 + TB * XP;               // [TB][XP]  attention output, then normalised rows
    float* hid = xa + TB * XP;              // [TB][HP]  SwiGLU product; later the head's hidden layer [TB][128]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int clip0 = blockIdx.x * TB;
    for (int i = tid; i < TB * kD; i += NT) {
        const int c = i / kD, k = i - c * kD;
        const bool live = clip0 + c < B;
        xa[c * XP + k] = live ? Y[(long long)(clip0 + c) * kD + k] : 0.0f;
        x1[c * XP + k] = live ? h_last[(long long)(clip0 + c) * ldh + k] : 0.0f;
    }
    __syncthreads();
    // x1 = h + Y . W_O^T: 192 column pairs
    float keep[TB][2];
    if (tid < kD / 2) {
        dot_columns<kD, 2, TB>(xa, XP, tw.wo_t, kD, 2 * tid, keep);
#pragma unroll
        for (int c = 0; c < TB; ++c) {
            float2* p = reinterpret_cast<float2*>(x1 + c * XP + 2 * tid);
            const float2 r = *p;
            *p = make_float2(r.x + keep[c][0], r.y + keep[c][1]);
        }
    }
    __syncthreads();
    norm_rows<TB, NT>(x1, xa, tw.ffn_norm_w, warp, lane);
    __syncthreads();
    // hid[j] = silu(gate_j) * up_j: 960 (gate, up) column pairs
    for (int j = tid; j < kDFF; j += NT) {
        float acc[TB][2];
        dot_columns<kD, 2, TB>(xa, XP, tw.up_t, 2 * kDFF, 2 * j, acc);
#pragma unroll
        for (int c = 0; c < TB; ++c) hid[c * HP + j] = silu_f(acc[c][0]) * acc[c][1];
    }
    __syncthreads();
    // x2 = x1 + hid . W_down^T
    if (tid < kD / 2) {
        dot_columns<kDFF, 2, TB>(hid, HP, tw.down_t, kD, 2 * tid, keep);
#pragma unroll
        for (int c = 0; c < TB; ++c) {
            float2* p = reinterpret_cast<float2*>(x1 + c * XP + 2 * tid);
            const float2 r = *p;
            const float2 v = make_float2(r.x + keep[c][0], r.y + keep[c][1]);
            *p = v;
            if (x2_out && clip0 + c < B) *reinterpret_cast<float2*>(x2_out + (long long)(clip0 + c) * kD + 2 * tid) = v;
        }
    }
    __syncthreads();
    norm_rows<TB, NT>(x1, xa, tw.final_norm_w, warp, lane);
    __syncthreads();
    // head: 128 hidden units (one column per thread of the first four warps), then their weighted sum per clip
    float* hh = hid;                         // [TB][128]; the SwiGLU product is consumed
    if (tid < 128) {
        float acc[TB][1];
        dot_columns<kD, 1, TB>(xa, XP, tw.head_w0_t, 128, tid, acc);
        const float b0 = __ldg(tw.head_b0 + tid), w2 = __ldg(tw.head_w2 + tid);
#pragma unroll
        for (int c = 0; c < TB; ++c) hh[c * 128 + tid] = w2 * silu_f(acc[c][0] + b0);
    }
    __syncthreads();
    for (int c = warp; c < TB; c += NT / 32) {
        const float s = warp_sum((hh[c * 128 + lane] + hh[c * 128 + lane + 32]) + (hh[c * 128 + lane + 64] + hh[c * 128 + lane + 96]));
        if (lane == 0 && clip0 + c < B) logits[clip0 + c] = s + __ldg(tw.head_b2);
    }
}

constexpr int tail_smem_bytes(int tb) { return (2 * tb * XP + tb * HP) * int(sizeof(float)); }

// Clips and threads per CTA for a batch of B: 16 clips once that still gives every SM a CTA, else 4, 2 (the few hundred
// clips of a pipeline batch: at B = 512 two clips per CTA 0.087 ms for the tail kernel, one 0.144, four 0.108; two or four
// clips with 512 threads 0.121 / 0.089, four with 1024 0.122), else 1.  The arithmetic of an output does not depend on
// the choice (one FMA chain over k ascending in every form).
struct ReadoutShape { int tb, nt; };
ReadoutShape readout_shape(int B) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ReadoutShape r = B >= 16 * sms ? ReadoutShape{16, 256} : B >= 4 * sms ? ReadoutShape{4, 256} : B >= 2 * sms ? ReadoutShape{2, 256} : ReadoutShape{1, 256};
#ifdef SHVK_DEV_PROBES
    if (const char* e = getenv("SHVK_READOUT_TB")) { r.tb = atoi(e); r.nt = 256; }
    if (const char* e = getenv("SHVK_READOUT_NT")) r.nt = atoi(e);
#endif
    return r;
}

template <int TB, int NT>
int launch_qc(const float* h_last, long long ldh, const float* norm_w, const float* wqc_t, float* QC, int B, cudaStream_t s) {
    readout_qc_kernel<TB, NT><<<unsigned((B + TB - 1) / TB), NT, 0, s>>>(h_last, ldh, norm_w, wqc_t, QC, B);
    return int(cudaGetLastError());
}
template <int TB, int NT>
int launch_tail(const float* Y, const float* h_last, long long ldh, const TailWeights& tw, float* x2_out, float* logits, int B,
                cudaStream_t s) {
    const cudaError_t e = cudaFuncSetAttribute(readout_tail_kernel<TB, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, tail_smem_bytes(TB));
    if (e != cudaSuccess) return int(e);
    readout_tail_kernel<TB, NT><<<unsigned((B + TB - 1) / TB), NT, tail_smem_bytes(TB), s>>>(Y, h_last, ldh, tw, x2_out, logits, B);
    return int(cudaGetLastError());
}

// the shapes that are compiled: clips per CTA * 10000 + threads
#define SHVK_READOUT_SHAPES(X) X(16, 256) X(8, 256) X(4, 256) X(2, 256) X(1, 256)

}  // namespace
}  // namespace sb

extern "C" int shvk_readout_qc(const float* h_last, long long ldh, const float* norm_w, const float* wqc_t, float* QC, int B,
                               void* stream) {
    if (B <= 0) return 0;
    if (!h_last || !norm_w || !wqc_t || !QC) return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    const sb::ReadoutShape sh = sb::readout_shape(B);
    switch (sh.tb * 10000 + sh.nt) {
#define X(TB, NT) case TB * 10000 + NT: return sb::launch_qc<TB, NT>(h_last, ldh, norm_w, wqc_t, QC, B, s);
        SHVK_READOUT_SHAPES(X)
#undef X
        default: return int(cudaErrorInvalidValue);
    }
}

extern "C" int shvk_readout_tail(const float* Y, const float* h_last, long long ldh, const shvk_readout_weights* w, float* x2_out,
                                 float* logits, int B, void* stream) {
    if (B <= 0) return 0;
    if (!Y || !h_last || !w || !logits) return int(cudaErrorInvalidValue);
    const sb::TailWeights tw{w->wo_t, w->ffn_norm_w, w->up_t, w->down_t, w->final_norm_w, w->head_w0_t, w->head_b0, w->head_w2, w->head_b2};
    cudaStream_t s = cudaStream_t(stream);
    const sb::ReadoutShape sh = sb::readout_shape(B);
    switch (sh.tb * 10000 + sh.nt) {
#define X(TB, NT) case TB * 10000 + NT: return sb::launch_tail<TB, NT>(Y, h_last, ldh, tw, x2_out, logits, B, s);
        SHVK_READOUT_SHAPES(X)
#undef X
        default: return int(cudaErrorInvalidValue);
    }
}
