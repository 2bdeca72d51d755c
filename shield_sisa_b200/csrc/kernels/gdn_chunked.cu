// Long-sequence gated delta rule in chunked (WY / UT-transform) form on the tensor cores.
//
//   S_t = exp(g_t) S_{t-1} + k_t u_t^T,  u_t = beta_t (v_t - exp(g_t) S_{t-1}^T k_t),  o_t = S_t^T (scale q_t),  S_0 = 0
// for q, k [B,T,H,DK] (already L2-normalised, bf16), v [B,T,H,128] (bf16), log decay g and beta [B,T,H] (fp32): the
// recurrence of the reference's oracle (oracle/shieldv_ref.py:121-139, gated_delta_rule_recurrent), which the reference
// engines only evaluate token by token at T = 321 (engine/cuda/seq.cu:107-195).  This entry point is the long-T form.
//
// One CTA owns one (batch, head) sequence and walks it in blocks of 16 tokens with the same algebra and the same
// register-only hand-over between products as gdn_scan_mma.cu (see there): per block, with inclusive cumulative log
// decay c_i, e_i = exp(c_i),
//     L_ij = beta_i exp(c_i - c_j) (k_i . k_j)  (j < i),  T2 = (I + L)^-1 diag(beta),  M_ij = scale exp(c_i - c_j) (q_i . k_j)  (j <= i)
//     R = K S0,  U = T2 (V - diag(e) R),  O = M U + diag(scale e) Q S0,  S' = e_16 S0 + K^T diag(exp(c_16 - c_j)) U.
// The value dimension (128) is the MMA row dimension and is split over the warps of the CTA: four warps of 32 columns
// for DK = 64, eight warps of 16 columns for DK = 128, so that a warp's slice of S^T is 64 fp32 registers per lane in
// both cases.  Operands are bf16, the state and all accumulation fp32.  A caller's chunk size (e.g. 64) only groups
// these 16-token blocks: the result does not depend on it.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int CB = 16;                       // tokens per block
constexpr int CT_PITCH = 24;                 // bf16 per row of K^T, T2, M tiles
constexpr int CV_PITCH = 20;                 // floats per row of V^T
constexpr int CDV = 128;

template <int DK> struct ChunkSmem {
    static constexpr int KP = DK + 8;        // bf16 per token row of the K / Q tiles: conflict-free fragment reads
    __nv_bfloat16 kb[CB][KP];
    __nv_bfloat16 qb[CB][KP];
    __nv_bfloat16 kt[DK][CT_PITCH];
    float vt[CDV][CV_PITCH];
    __nv_bfloat16 t2[CB][CT_PITCH];
    __nv_bfloat16 mq[CB][CT_PITCH];
    float lf[CB][CB + 1];
    float otile[CB][CDV + 4];                // padded rows: the fragment stores of a warp fall into 32 different banks
    float beta[CB], cum[CB], eg[CB], dj[CB];
};

__device__ __forceinline__ uint32_t cpack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cmma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// DK = 64: MI = 2 row tiles per warp, 4 warps;  DK = 128: MI = 1, 8 warps.
template <int DK, typename TO>
__global__ void __launch_bounds__(DK == 64 ? 128 : 256)
gdn_chunked_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K, const __nv_bfloat16* __restrict__ V,
                   const float* __restrict__ G, const float* __restrict__ Beta, TO* __restrict__ O, int T, int H, float scale) {
    constexpr int MI = DK == 64 ? 2 : 1, NWARP = DK == 64 ? 4 : 8, NTHR = NWARP * 32;
    constexpr int KSTEP = DK / 16, NJ = DK / 8, KW = ChunkSmem<DK>::KP / 2;     // KW: 32-bit words per K / Q tile row
    extern __shared__ uint8_t chunk_smem_raw[];
    ChunkSmem<DK>& sm = *reinterpret_cast<ChunkSmem<DK>*>((reinterpret_cast<uintptr_t>(chunk_smem_raw) + 15) & ~uintptr_t(15));
    const int bh = blockIdx.x, bidx = bh / H, head = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int dvb = warp * 16 * MI;
    const long long tok_stride_k = (long long)H * DK, tok_stride_v = (long long)H * CDV;
    const __nv_bfloat16* Qs = Q + ((long long)bidx * T * H + head) * DK;
    const __nv_bfloat16* Ks = K + ((long long)bidx * T * H + head) * DK;
    const __nv_bfloat16* Vs = V + ((long long)bidx * T * H + head) * CDV;
    const float* Gs = G + (long long)bidx * T * H + head;
    const float* Bs = Beta + (long long)bidx * T * H + head;
    TO* Os = O + ((long long)bidx * T * H + head) * CDV;

    float S[MI][NJ][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int nj = 0; nj < NJ; ++nj)
#pragma unroll
            for (int e = 0; e < 4; ++e) S[mi][nj][e] = 0.0f;

    // global -> register prefetch of one block: 16-byte vectors of q and k rows (DK / 8 per row), v rows (16 per row).
    // Lanes run over the 16 tokens first (two adjacent vectors per token and warp instruction = whole 32-byte
    // sectors): the transposing stores into K^T and V^T then hit 16 different banks instead of one.
    constexpr int QK_VECS = CB * DK / 8, V_VECS = CB * CDV / 8;
    constexpr int QK_PER = (QK_VECS + NTHR - 1) / NTHR, V_PER = V_VECS / NTHR;
    uint4 pq[QK_PER], pk[QK_PER], pv[V_PER];
    float pgate = 0.0f, pbeta = 0.0f;
    auto prefetch = [&](int t0) {
#pragma unroll
        for (int r = 0; r < QK_PER; ++r) {
            const int idx = tid + r * NTHR, row = idx % CB, c8 = idx / CB;
            const bool ok = idx < QK_VECS && t0 + row < T;
            pq[r] = ok ? *reinterpret_cast<const uint4*>(Qs + (long long)(t0 + row) * tok_stride_k + c8 * 8) : make_uint4(0, 0, 0, 0);
            pk[r] = ok ? *reinterpret_cast<const uint4*>(Ks + (long long)(t0 + row) * tok_stride_k + c8 * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < V_PER; ++r) {
            const int idx = tid + r * NTHR, row = idx % CB, c8 = idx / CB;
            pv[r] = t0 + row < T ? *reinterpret_cast<const uint4*>(Vs + (long long)(t0 + row) * tok_stride_v + c8 * 8) : make_uint4(0, 0, 0, 0);
        }
        if (tid < CB) {                                   // tokens past the end are inert: no decay, beta = 0
            const bool ok = t0 + tid < T;
            pgate = ok ? Gs[(long long)(t0 + tid) * H] : 0.0f;
            pbeta = ok ? Bs[(long long)(t0 + tid) * H] : 0.0f;
        }
    };
    prefetch(0);

    const uint32_t* kbw = reinterpret_cast<const uint32_t*>(&sm.kb[0][0]);
    const uint32_t* qbw = reinterpret_cast<const uint32_t*>(&sm.qb[0][0]);
    const uint32_t* t2w = reinterpret_cast<const uint32_t*>(&sm.t2[0][0]);   // 12 words per row
    const uint32_t* mqw = reinterpret_cast<const uint32_t*>(&sm.mq[0][0]);
    const uint32_t* ktw = reinterpret_cast<const uint32_t*>(&sm.kt[0][0]);

    for (int t0 = 0; t0 < T; t0 += CB) {
        // ---------------------------------------------------------------- registers -> operand tiles
#pragma unroll
        for (int r = 0; r < QK_PER; ++r) {
            const int idx = tid + r * NTHR, row = idx % CB, c8 = idx / CB;
            if (idx < QK_VECS) {
                *reinterpret_cast<uint4*>(&sm.qb[row][c8 * 8]) = pq[r];
                *reinterpret_cast<uint4*>(&sm.kb[row][c8 * 8]) = pk[r];
                const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(&pk[r]);
#pragma unroll
                for (int e = 0; e < 8; ++e) sm.kt[c8 * 8 + e][row] = kv[e];
            }
        }
#pragma unroll
        for (int r = 0; r < V_PER; ++r) {
            const int idx = tid + r * NTHR, row = idx % CB, c8 = idx / CB;
            const __nv_bfloat16* vv = reinterpret_cast<const __nv_bfloat16*>(&pv[r]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sm.vt[c8 * 8 + e][row] = __bfloat162float(vv[e]);
        }
        if (warp == 0) {                                  // inclusive prefix sum of the log decays over the block
            float c = pgate;                              // lanes >= 16 hold 0
#pragma unroll
            for (int o = 1; o < CB; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, c, o);
                if (lane >= o) c += up;
            }
            const float last = __shfl_sync(0xffffffffu, c, CB - 1);
            if (lane < CB) {
                sm.beta[lane] = pbeta;
                sm.cum[lane] = c;
                sm.eg[lane] = __expf(c);
                sm.dj[lane] = __expf(last - c);
            }
        }
        if (t0 + CB < T) prefetch(t0 + CB);               // next block's loads fly while this one is computed
        __syncthreads();
        // ---------------------------------------------------------------- warp 0: L, T2;  warp 1: masked Q K^T
        if (warp < 2) {
            const uint32_t* xa = warp == 0 ? kbw : qbw;
            float acc[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[ni][e] = 0.0f;
#pragma unroll
            for (int p = 0; p < KSTEP; ++p) {
                const uint32_t a[4] = {xa[g * KW + 8 * p + t], xa[(g + 8) * KW + 8 * p + t], xa[g * KW + 8 * p + t + 4],
                                       xa[(g + 8) * KW + 8 * p + t + 4]};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
                    cmma(acc[ni], a, kbw[(8 * ni + g) * KW + 8 * p + t], kbw[(8 * ni + g) * KW + 8 * p + t + 4]);
            }
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = g + (e >> 1) * 8, j = 8 * ni + 2 * t + (e & 1);
                    const bool keep = warp == 0 ? j < i : j <= i;
                    const float dec = __expf(keep ? sm.cum[i] - sm.cum[j] : 0.0f);
                    const float rowf = warp == 0 ? sm.beta[i] : scale;
                    acc[ni][e] = keep ? dec * acc[ni][e] * rowf : 0.0f;
                }
            if (warp == 0) {
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sm.lf[g + (e >> 1) * 8][8 * ni + 2 * t + (e & 1)] = acc[ni][e];
                __syncwarp();
                if (lane < CB) {                          // column `lane` of (I + L)^-1 by forward substitution
                    float x[CB];
#pragma unroll
                    for (int i = 0; i < CB; ++i) {
                        // four partial sums: the dependent chain per row is i / 4 long instead of i
                        float s0 = i == lane ? 1.0f : 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                        for (int j = 0; j < i; ++j) {
                            const float l = sm.lf[i][j];
                            if ((j & 3) == 0) s0 = fmaf(-l, x[j], s0);
                            else if ((j & 3) == 1) s1 = fmaf(-l, x[j], s1);
                            else if ((j & 3) == 2) s2 = fmaf(-l, x[j], s2);
                            else s3 = fmaf(-l, x[j], s3);
                        }
                        x[i] = (s0 + s1) + (s2 + s3);
                    }
                    const float bc = sm.beta[lane];
#pragma unroll
                    for (int i = 0; i < CB; ++i) sm.t2[i][lane] = __float2bfloat16_rn(x[i] * bc);
                }
            } else {
                uint32_t* mw = reinterpret_cast<uint32_t*>(&sm.mq[0][0]);
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    mw[g * 12 + 4 * ni + t] = cpack(acc[ni][0], acc[ni][1]);
                    mw[(g + 8) * 12 + 4 * ni + t] = cpack(acc[ni][2], acc[ni][3]);
                }
            }
        }
        // ---------------------------------------------------------------- R^T = S0^T K^T, (Q S0)^T
        float R[MI][2][4], QS[MI][2][4];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) { R[mi][ni][e] = 0.0f; QS[mi][ni][e] = 0.0f; }
#pragma unroll
        for (int p = 0; p < KSTEP; ++p) {
            uint32_t bk[2][2], bq[2][2];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                bk[ni][0] = kbw[(8 * ni + g) * KW + 8 * p + t]; bk[ni][1] = kbw[(8 * ni + g) * KW + 8 * p + t + 4];
                bq[ni][0] = qbw[(8 * ni + g) * KW + 8 * p + t]; bq[ni][1] = qbw[(8 * ni + g) * KW + 8 * p + t + 4];
            }
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const uint32_t sa[4] = {cpack(S[mi][2 * p][0], S[mi][2 * p][1]), cpack(S[mi][2 * p][2], S[mi][2 * p][3]),
                                        cpack(S[mi][2 * p + 1][0], S[mi][2 * p + 1][1]), cpack(S[mi][2 * p + 1][2], S[mi][2 * p + 1][3])};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    cmma(R[mi][ni], sa, bk[ni][0], bk[ni][1]);
                    cmma(QS[mi][ni], sa, bq[ni][0], bq[ni][1]);
                }
            }
        }
        __syncthreads();
        // ---------------------------------------------------------------- U, O, state update
        float er[2][2], eq[2][2], dj2[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = 8 * ni + 2 * t + e;
                er[ni][e] = sm.eg[tok];
                eq[ni][e] = sm.eg[tok] * scale;
                dj2[ni][e] = sm.dj[tok];
            }
        uint32_t bt[2][2], bm[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            bt[ni][0] = t2w[(8 * ni + g) * 12 + t]; bt[ni][1] = t2w[(8 * ni + g) * 12 + t + 4];
            bm[ni][0] = mqw[(8 * ni + g) * 12 + t]; bm[ni][1] = mqw[(8 * ni + g) * 12 + t + 4];
        }
        uint32_t da[MI][4];
        // V^T for all row tiles is loaded before the first o-tile store (a store would hold back the loads behind it)
        float2 vv[MI][2][2];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                vv[mi][ni][0] = *reinterpret_cast<const float2*>(&sm.vt[dvb + 16 * mi + g][8 * ni + 2 * t]);
                vv[mi][ni][1] = *reinterpret_cast<const float2*>(&sm.vt[dvb + 16 * mi + g + 8][8 * ni + 2 * t]);
            }
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
            const int r0 = dvb + 16 * mi + g, r1 = r0 + 8;
            uint32_t va[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                const float2 v0 = vv[mi][ni][0];
                const float2 v1 = vv[mi][ni][1];
                va[2 * ni] = cpack(v0.x - er[ni][0] * R[mi][ni][0], v0.y - er[ni][1] * R[mi][ni][1]);
                va[2 * ni + 1] = cpack(v1.x - er[ni][0] * R[mi][ni][2], v1.y - er[ni][1] * R[mi][ni][3]);
            }
            float U[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
                for (int e = 0; e < 4; ++e) U[ni][e] = 0.0f;
                cmma(U[ni], va, bt[ni][0], bt[ni][1]);
            }
            uint32_t ua[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                ua[2 * ni] = cpack(U[ni][0], U[ni][1]);
                ua[2 * ni + 1] = cpack(U[ni][2], U[ni][3]);
                da[mi][2 * ni] = cpack(U[ni][0] * dj2[ni][0], U[ni][1] * dj2[ni][1]);
                da[mi][2 * ni + 1] = cpack(U[ni][2] * dj2[ni][0], U[ni][3] * dj2[ni][1]);
            }
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                float Oa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                cmma(Oa, ua, bm[ni][0], bm[ni][1]);
                const int tok = 8 * ni + 2 * t;
                sm.otile[tok][r0] = Oa[0] + eq[ni][0] * QS[mi][ni][0];
                sm.otile[tok + 1][r0] = Oa[1] + eq[ni][1] * QS[mi][ni][1];
                sm.otile[tok][r1] = Oa[2] + eq[ni][0] * QS[mi][ni][2];
                sm.otile[tok + 1][r1] = Oa[3] + eq[ni][1] * QS[mi][ni][3];
            }
        }
        {
            const float elast = sm.eg[CB - 1];
#pragma unroll
            for (int nj = 0; nj < NJ; ++nj) {
                const uint32_t b0 = ktw[(8 * nj + g) * 12 + t], b1 = ktw[(8 * nj + g) * 12 + t + 4];
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mi][nj][e] *= elast;
                    cmma(S[mi][nj], da[mi], b0, b1);
                }
            }
        }
        __syncthreads();
        // ---------------------------------------------------------------- o tile -> global, coalesced along the values
        for (int idx = tid; idx < CB * (CDV / 4); idx += NTHR) {
            const int row = idx / (CDV / 4), c4 = idx % (CDV / 4);
            if (t0 + row < T) {
                const float4 o = *reinterpret_cast<const float4*>(&sm.otile[row][c4 * 4]);
                store_quad<TO>(Os + (long long)(t0 + row) * tok_stride_v + c4 * 4, o.x, o.y, o.z, o.w);
            }
        }
        // the next iteration rewrites the operand tiles only; otile is rewritten after two more barriers
    }
}

template <int DK, typename TO>
int launch_chunked(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o, int B, int T, int H,
                   float scale, cudaStream_t s) {
    const int smem = int(sizeof(ChunkSmem<DK>)) + 16;
    const cudaError_t e = cudaFuncSetAttribute(gdn_chunked_kernel<DK, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    gdn_chunked_kernel<DK, TO><<<unsigned(B) * unsigned(H), DK == 64 ? 128 : 256, smem, s>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), g, beta,
        static_cast<TO*>(o), T, H, scale);
    return int(cudaGetLastError());
}

}  // namespace
}  // namespace sb

extern "C" int shvk_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o,
                                int o_dtype, int B, int T, int H, int DK, int DV, float scale, void* stream) {
    using namespace sb;
    if (B <= 0 || T <= 0 || H <= 0) return 0;
    if (DV != CDV || (DK != 64 && DK != 128) || (o_dtype != DT_F32 && o_dtype != DT_BF16)) return int(cudaErrorInvalidValue);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(o)) & 15)
        return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    if (DK == 64) {
        return o_dtype == DT_F32 ? launch_chunked<64, float>(q, k, v, g, beta, o, B, T, H, scale, s)
                                 : launch_chunked<64, __nv_bfloat16>(q, k, v, g, beta, o, B, T, H, scale, s);
    }
    return o_dtype == DT_F32 ? launch_chunked<128, float>(q, k, v, g, beta, o, B, T, H, scale, s)
                             : launch_chunked<128, __nv_bfloat16>(q, k, v, g, beta, o, B, T, H, scale, s);
}
