// Long-sequence gated delta rule in chunked (WY / UT-transform) form on the tensor cores.
//
//   S_t = exp(g_t) S_{t-1} + k_t u_t^T,  u_t = beta_t (v_t - exp(g_t) S_{t-1}^T k_t),  o_t = S_t^T (scale q_t),  S_0 = 0
// for q, k [B,T,H,DK] (already L2-normalised, bf16), v [B,T,H,128] (bf16), log decay g and beta [B,T,H] (fp32): the
// recurrence of the reference's oracle (oracle/shieldv_ref.py:121-139, gated_delta_rule_recurrent), which the reference
// engines only evaluate token by token at T = 321 (engine/cuda/seq.cu:107-195).  This entry point is the long-T form.
//
// Per block of 16 tokens, with inclusive cumulative log decay c_i, e_i = exp(c_i), state S0 entering the block:
//     L_ij = beta_i exp(c_i - c_j) (k_i . k_j)  (j < i),  T2 = (I + L)^-1 diag(beta),  M_ij = scale exp(c_i - c_j) (q_i . k_j)  (j <= i)
//     R = K S0,  U = T2 (V - diag(e) R),  O = M U + diag(scale e) Q S0,  S' = e_16 S0 + K^T diag(exp(c_16 - c_j)) U.
// T2 and M do not depend on the state, only R, U, O and S' do.  Two kernels, chunk-parallel where the algebra allows:
//
//   prep   one warp per block, all B x H x T/16 blocks at once: the two Gram products on mma.sync, the decay masks, the
//          16 x 16 triangular inverse (forward substitution over 16 lanes), T2 and M as bf16 tiles and the cumulative
//          decays into a workspace of 1,152 bytes per block
//   scan   one CTA per (batch, head) walks the blocks with the state resident: per block only the chain R -> U -> O and
//          the state update remain, every operand fragment read straight out of the staged K, Q, V, T2, M tiles with
//          ldmatrix (tiles arrive by cp.async into a three-slot ring, XOR-swizzled so the fragment reads are
//          conflict-free), one CTA barrier per block, the previous block's output rows written while the next block's
//          products run
//
// The value dimension (128) is the MMA row dimension and is split over the warps of the scan CTA: four warps of 32
// columns for DK = 64, eight warps of 16 columns for DK = 128, so that a warp's slice of S^T is 64 fp32 registers per lane
// in both cases; the hand-over between the products of a block stays in registers (the accumulator layout of one is the
// A-operand layout of the next).  Operands are bf16, the state and all accumulation fp32.  A caller's chunk size (e.g.
// 64) only groups these 16-token blocks: the result does not depend on it.
//
// Why not tcgen05 here: the chain of a block is three dependent products on 16-token tiles; tcgen05 wants M >= 64 rows
// per instruction and an asynchronous issue / commit / tensor-memory round trip per link.  With the state-independent
// half of the work moved into the chunk-parallel kernel, the sequential kernel is bound by the latency of that chain,
// not by the tensor pipe, and the whole computation by HBM (141 to 177 flop per byte, below the machine's ridge).
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int CB = 16;                       // tokens per block
constexpr int CDV = 128;
constexpr int WS_T2 = 0, WS_M = 512, WS_CUM = 1024, WS_BLOCK = 1152;   // workspace block: T2 | M (bf16 16 x 16) | c (fp32 16) | pad
constexpr int OT_PITCH = CDV + 4;            // floats per token row of the o tile (fragment stores fall into 32 banks)

__device__ __forceinline__ uint32_t cpack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ void cmma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
// 16-byte asynchronous copy global -> shared; `bytes` = 16, or 0 to fill the destination with zeros (tokens past T)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A tile of 16 token rows of ROWB bytes in shared memory: the 16-byte chunk c of row r sits at chunk c ^ (r & 7), so the
// eight rows of one ldmatrix read (same chunk column) fall into eight different bank groups.
template <int ROWB> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return uint32_t(row * ROWB + ((chunk ^ (row & 7)) << 4));
}

// ---------------------------------------------------------------------------------------------------- prep kernel
// (declared with a minimum of CTAs per SM: without one the assembler keeps the kernel at 40-48 registers by moving loads
// next to their uses)
template <int DK>
__global__ void __launch_bounds__(128, 4)
gdn_chunked_prep_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K, const float* __restrict__ G,
                        const float* __restrict__ Beta, uint8_t* __restrict__ ws, int T, int H, int NB, long long blocks,
                        float scale) {
    constexpr int ROWB = DK * 2, VPR = DK / 8, KSTEP = DK / 16;          // bytes and 16-byte vectors per tile row
    struct WarpSmem {
        __align__(16) uint8_t k[CB * ROWB], q[CB * ROWB];
        float lf[CB][CB + 1];
        float cum[CB], beta[CB];
        __align__(16) uint8_t out[WS_BLOCK];
    };
    extern __shared__ __align__(16) uint8_t prep_smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    WarpSmem& sm = reinterpret_cast<WarpSmem*>(prep_smem_raw)[warp];
    const long long blk = (long long)blockIdx.x * 4 + warp;
    if (blk >= blocks) return;
    const long long bh = blk / NB;
    const int c = int(blk - bh * NB), t0 = c * CB;
    const int bidx = int(bh / H), head = int(bh - (long long)bidx * H);
    const int g = lane >> 2, t = lane & 3, lm = lane >> 3, lr = lane & 7;
    const long long tok_stride = (long long)H * DK;
    const __nv_bfloat16* Ks = K + ((long long)bidx * T * H + head) * DK;
    const __nv_bfloat16* Qs = Q + ((long long)bidx * T * H + head) * DK;

    // K and Q rows of the block, 16-byte vectors, eight (DK = 64) or sixteen lanes per 128 / 256-byte row
#pragma unroll
    for (int i = 0; i < CB * VPR / 32; ++i) {
        const int v = lane + 32 * i, row = v / VPR, c8 = v % VPR;
        const bool ok = t0 + row < T;
        const uint4 z = make_uint4(0, 0, 0, 0);
        const uint4 kv = ok ? *reinterpret_cast<const uint4*>(Ks + (long long)(t0 + row) * tok_stride + c8 * 8) : z;
        const uint4 qv = ok ? *reinterpret_cast<const uint4*>(Qs + (long long)(t0 + row) * tok_stride + c8 * 8) : z;
        *reinterpret_cast<uint4*>(sm.k + tile_off<ROWB>(row, c8)) = kv;
        *reinterpret_cast<uint4*>(sm.q + tile_off<ROWB>(row, c8)) = qv;
    }
    // decays: inclusive prefix sum over the 16 tokens (both half-warps compute it); tokens past T are inert
    {
        const int tok = lane & (CB - 1);
        const bool ok = t0 + tok < T;
        float cs = ok ? G[((long long)bidx * T + t0 + tok) * H + head] : 0.0f;
        const float bt = ok ? Beta[((long long)bidx * T + t0 + tok) * H + head] : 0.0f;
#pragma unroll
        for (int o = 1; o < CB; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, cs, o);
            if (tok >= o) cs += up;
        }
        if (lane < CB) { sm.cum[lane] = cs; sm.beta[lane] = bt; }
    }
    __syncwarp();
    // Gram products over the keys: A = K K^T, Bm = Q K^T (16 x 16 each)
    float acc[2][4], accq[2][4];
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[ni][e] = 0.0f; accq[ni][e] = 0.0f; }
    const uint32_t k_s = smem_u32(sm.k), q_s = smem_u32(sm.q);
#pragma unroll
    for (int p = 0; p < KSTEP; ++p) {
        // matrices (tokens 0-7, keys lo), (tokens 8-15, keys lo), (tokens 0-7, keys hi), (tokens 8-15, keys hi) of k-step p:
        // the A fragment of [token][key]; as B fragments of the transposed product: (r[ni], r[ni + 2])
        const uint32_t off = tile_off<ROWB>((lm & 1) * 8 + lr, 2 * p + (lm >> 1));
        uint32_t kf[4], qf[4];
        ldsm4(k_s + off, kf);
        ldsm4(q_s + off, qf);
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            cmma(acc[ni], kf, kf[ni], kf[ni + 2]);
            cmma(accq[ni], qf, kf[ni], kf[ni + 2]);
        }
    }
    // acc[ni][0,1]: row i = g, columns j = 8 ni + 2t, + 1;  acc[ni][2,3]: row i = g + 8
    uint32_t* mw = reinterpret_cast<uint32_t*>(sm.out + WS_M);                 // 8 words per row
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) {
        float m[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = g + (e >> 1) * 8, j = 8 * ni + 2 * t + (e & 1);
            const float dec = __expf(j <= i ? sm.cum[i] - sm.cum[j] : 0.0f);
            sm.lf[i][j] = j < i ? sm.beta[i] * dec * acc[ni][e] : 0.0f;
            m[e] = j <= i ? scale * dec * accq[ni][e] : 0.0f;
        }
        mw[g * 8 + 4 * ni + t] = cpack(m[0], m[1]);
        mw[(g + 8) * 8 + 4 * ni + t] = cpack(m[2], m[3]);
    }
    __syncwarp();
    if (lane < CB) {                                      // column `lane` of (I + L)^-1 by forward substitution
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
        __nv_bfloat16* t2 = reinterpret_cast<__nv_bfloat16*>(sm.out + WS_T2);
#pragma unroll
        for (int i = 0; i < CB; ++i) t2[i * CB + lane] = __float2bfloat16_rn(x[i] * bc);
        reinterpret_cast<float*>(sm.out + WS_CUM)[lane] = sm.cum[lane];
        reinterpret_cast<float*>(sm.out + WS_CUM)[CB + lane] = 0.0f;
    }
    __syncwarp();
    uint4* dst = reinterpret_cast<uint4*>(ws + blk * WS_BLOCK);
    const uint4* src = reinterpret_cast<const uint4*>(sm.out);
    for (int i = lane; i < WS_BLOCK / 16; i += 32) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------------------- scan kernel
template <int DK> struct ScanStage {                      // one block's operands as they lie in shared memory
    __align__(16) uint8_t k[CB * DK * 2], q[CB * DK * 2];  // [token][key] bf16, swizzled rows of DK * 2 bytes
    __align__(16) uint8_t v[2][CB * 128];                  // [token][value] bf16 as two halves of 64 values (128-byte rows)
    __align__(16) uint8_t w[WS_BLOCK];                     // T2 | M | c of the block
};

// DK = 64: MI = 2 row tiles per warp, 4 warps;  DK = 128: MI = 1, 8 warps.
template <int DK, typename TO>
__global__ void __launch_bounds__(DK == 64 ? 128 : 256)
gdn_chunked_scan_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K, const __nv_bfloat16* __restrict__ V,
                        const uint8_t* __restrict__ ws, TO* __restrict__ O, int T, int H, int NB, float scale) {
    constexpr int MI = DK == 64 ? 2 : 1, NWARP = DK == 64 ? 4 : 8, NTHR = NWARP * 32;
    constexpr int KSTEP = DK / 16, NJ = DK / 8, ROWB = DK * 2, VPR = DK / 8, NSLOT = 3;
    struct Smem {
        ScanStage<DK> st[NSLOT];
        float ot[2][CB][OT_PITCH];
    };
    extern __shared__ __align__(128) uint8_t cscan_smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(cscan_smem_raw) + 127) & ~uintptr_t(127));
    const int bh = blockIdx.x, bidx = bh / H, head = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3, lm = lane >> 3, lr = lane & 7;
    const int dvb = warp * 16 * MI;
    const long long tok_stride_k = (long long)H * DK, tok_stride_v = (long long)H * CDV;
    const __nv_bfloat16* Qs = Q + ((long long)bidx * T * H + head) * DK;
    const __nv_bfloat16* Ks = K + ((long long)bidx * T * H + head) * DK;
    const __nv_bfloat16* Vs = V + ((long long)bidx * T * H + head) * CDV;
    const uint8_t* Ws = ws + (long long)bh * NB * WS_BLOCK;
    TO* Os = O + ((long long)bidx * T * H + head) * CDV;

    float S[MI][NJ][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int nj = 0; nj < NJ; ++nj)
#pragma unroll
            for (int e = 0; e < 4; ++e) S[mi][nj][e] = 0.0f;

    // asynchronous copies of block `c` into ring slot c % 3; every thread issues its share and commits one group
    auto issue = [&](int c) {
        if (c < NB) {
            ScanStage<DK>& st = sm.st[c % NSLOT];
            const int t0 = c * CB;
            for (int v = tid; v < CB * VPR; v += NTHR) {
                const int row = v / VPR, c8 = v % VPR;
                const int ok = t0 + row < T ? 16 : 0;
                const long long src = (long long)(ok ? t0 + row : 0) * tok_stride_k + c8 * 8;
                cp_async16(smem_u32(st.k) + tile_off<ROWB>(row, c8), Ks + src, ok);
                cp_async16(smem_u32(st.q) + tile_off<ROWB>(row, c8), Qs + src, ok);
            }
            for (int v = tid; v < CB * 16; v += NTHR) {
                const int row = v >> 4, c16 = v & 15;
                const int ok = t0 + row < T ? 16 : 0;
                cp_async16(smem_u32(st.v[c16 >> 3]) + tile_off<128>(row, c16 & 7), Vs + (long long)(ok ? t0 + row : 0) * tok_stride_v + c16 * 8, ok);
            }
            for (int v = tid; v < WS_BLOCK / 16; v += NTHR) cp_async16(smem_u32(st.w) + v * 16, Ws + (long long)c * WS_BLOCK + v * 16, 16);
        }
        cp_commit();                                      // an empty group past the end keeps the group count in step
    };
    // rows of a finished block from its o tile to global memory: 16 tokens x 128 values, eight values per thread and pass
    auto store_rows = [&](int c) {
        const float* ot = &sm.ot[c & 1][0][0];
        const int t0 = c * CB;
        for (int idx = tid; idx < CB * CDV / 8; idx += NTHR) {
            const int row = idx >> 4, c8 = idx & 15;
            if (t0 + row < T) {
                const float4 a = *reinterpret_cast<const float4*>(ot + row * OT_PITCH + c8 * 8);
                const float4 b = *reinterpret_cast<const float4*>(ot + row * OT_PITCH + c8 * 8 + 4);
                TO* dst = Os + (long long)(t0 + row) * tok_stride_v + c8 * 8;
                store_quad<TO>(dst, a.x, a.y, a.z, a.w);
                store_quad<TO>(dst + 4, b.x, b.y, b.z, b.w);
            }
        }
    };

    issue(0);
    issue(1);
    for (int c = 0; c < NB; ++c) {
        cp_wait<1>();                                     // this thread's copies of block c have landed (block c + 1 may still fly)
        __syncthreads();                                  // everyone's have; the o tile of block c - 1 is complete; slot (c + 2) % 3 is free
        issue(c + 2);
        if (c > 0) store_rows(c - 1);
        ScanStage<DK>& st = sm.st[c % NSLOT];
        const uint32_t k_s = smem_u32(st.k), q_s = smem_u32(st.q);
        const float* cum = reinterpret_cast<const float*>(st.w + WS_CUM);
        // ---------------------------------------------------------------- R^T = S0^T K^T and (Q S0)^T
        float R[MI][2][4], QS[MI][2][4];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) { R[mi][ni][e] = 0.0f; QS[mi][ni][e] = 0.0f; }
#pragma unroll
        for (int p = 0; p < KSTEP; ++p) {
            // B fragments [key][token]: matrices (tokens 0-7, keys lo), (tokens 0-7, keys hi), (tokens 8-15, keys lo),
            // (tokens 8-15, keys hi) -> (b0, b1) of token block 0, then of token block 1
            const uint32_t off = tile_off<ROWB>((lm >> 1) * 8 + lr, 2 * p + (lm & 1));
            uint32_t bk[4], bq[4];
            ldsm4(k_s + off, bk);
            ldsm4(q_s + off, bq);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const uint32_t sa[4] = {cpack(S[mi][2 * p][0], S[mi][2 * p][1]), cpack(S[mi][2 * p][2], S[mi][2 * p][3]),
                                        cpack(S[mi][2 * p + 1][0], S[mi][2 * p + 1][1]), cpack(S[mi][2 * p + 1][2], S[mi][2 * p + 1][3])};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    cmma(R[mi][ni], sa, bk[2 * ni], bk[2 * ni + 1]);
                    cmma(QS[mi][ni], sa, bq[2 * ni], bq[2 * ni + 1]);
                }
            }
        }
        // per-token scalars of this lane's tokens 8 ni + 2t, + 1
        float er[2][2], eq[2][2], dj[2][2];
        const float clast = cum[CB - 1];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float cv = cum[8 * ni + 2 * t + e];
                er[ni][e] = __expf(cv);
                eq[ni][e] = er[ni][e] * scale;
                dj[ni][e] = __expf(clast - cv);
            }
        // B fragments of T2 and M (row-major 16 x 16, 32-byte rows): matrices (rows 0-7, cols lo), (rows 0-7, cols hi),
        // (rows 8-15, cols lo), (rows 8-15, cols hi)
        uint32_t bt[4], bm[4];
        {
            const uint32_t off = uint32_t(((lm >> 1) * 8 + lr) * 32 + (lm & 1) * 16);
            ldsm4(smem_u32(st.w + WS_T2) + off, bt);
            ldsm4(smem_u32(st.w + WS_M) + off, bm);
        }
        // K^T fragments of the state update, B[token][key]: transposed reads; kf[q][2 h + c]: keys 16 q + 8 h + g, tokens 8 c + 2t, + 1
        uint32_t kf[KSTEP][4];
#pragma unroll
        for (int q = 0; q < KSTEP; ++q) ldsm4t(k_s + tile_off<ROWB>((lm & 1) * 8 + lr, 2 * q + (lm >> 1)), kf[q]);
        float* otile = &sm.ot[c & 1][0][0];
        uint32_t da[MI][4];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
            const int r0 = dvb + 16 * mi + g, r1 = r0 + 8;
            // V^T fragment A[value][token] of value rows dvb + 16 mi .. + 15: transposed reads of [token][value]; matrices
            // (tokens 0-7, values lo), (tokens 0-7, values hi), (tokens 8-15, values lo), (tokens 8-15, values hi)
            uint32_t vv[4];
            {
                const int val0 = dvb + 16 * mi;                      // multiple of 16: both 8-value chunks lie in one 64-value half
                ldsm4t(smem_u32(st.v[val0 >> 6]) + tile_off<128>((lm >> 1) * 8 + lr, ((val0 & 63) >> 3) + (lm & 1)), vv);
            }
            // vv[0]: value g, tokens 2t, +1 | vv[1]: value g + 8, same tokens | vv[2]: value g, tokens 8 + 2t | vv[3]: value g + 8
            uint32_t va[4];
            va[0] = cpack(bf_lo(vv[0]) - er[0][0] * R[mi][0][0], bf_hi(vv[0]) - er[0][1] * R[mi][0][1]);
            va[1] = cpack(bf_lo(vv[1]) - er[0][0] * R[mi][0][2], bf_hi(vv[1]) - er[0][1] * R[mi][0][3]);
            va[2] = cpack(bf_lo(vv[2]) - er[1][0] * R[mi][1][0], bf_hi(vv[2]) - er[1][1] * R[mi][1][1]);
            va[3] = cpack(bf_lo(vv[3]) - er[1][0] * R[mi][1][2], bf_hi(vv[3]) - er[1][1] * R[mi][1][3]);
            float U[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
                for (int e = 0; e < 4; ++e) U[ni][e] = 0.0f;
                cmma(U[ni], va, bt[2 * ni], bt[2 * ni + 1]);
            }
            uint32_t ua[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                ua[2 * ni] = cpack(U[ni][0], U[ni][1]);
                ua[2 * ni + 1] = cpack(U[ni][2], U[ni][3]);
                da[mi][2 * ni] = cpack(U[ni][0] * dj[ni][0], U[ni][1] * dj[ni][1]);
                da[mi][2 * ni + 1] = cpack(U[ni][2] * dj[ni][0], U[ni][3] * dj[ni][1]);
            }
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                float Oa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                cmma(Oa, ua, bm[2 * ni], bm[2 * ni + 1]);
                const int tok = 8 * ni + 2 * t;
                otile[tok * OT_PITCH + r0] = Oa[0] + eq[ni][0] * QS[mi][ni][0];
                otile[(tok + 1) * OT_PITCH + r0] = Oa[1] + eq[ni][1] * QS[mi][ni][1];
                otile[tok * OT_PITCH + r1] = Oa[2] + eq[ni][0] * QS[mi][ni][2];
                otile[(tok + 1) * OT_PITCH + r1] = Oa[3] + eq[ni][1] * QS[mi][ni][3];
            }
        }
        // ---------------------------------------------------------------- S^T <- e_last S^T + (diag(d) U)^T K
        {
            const float elast = __expf(clast);
#pragma unroll
            for (int nj = 0; nj < NJ; ++nj) {
                const uint32_t b0 = kf[nj >> 1][2 * (nj & 1)], b1 = kf[nj >> 1][2 * (nj & 1) + 1];
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mi][nj][e] *= elast;
                    cmma(S[mi][nj], da[mi], b0, b1);
                }
            }
        }
    }
    cp_wait<0>();
    __syncthreads();
    store_rows(NB - 1);
}

constexpr int prep_smem_bytes(int dk) { return 4 * (2 * CB * dk * 2 + CB * (CB + 1) * 4 + 2 * CB * 4 + WS_BLOCK + 64); }

template <int DK, typename TO>
int launch_chunked(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o, void* ws, int B, int T,
                   int H, float scale, cudaStream_t s) {
    const int NB = (T + CB - 1) / CB;
    const long long blocks = (long long)B * H * NB;
    // the struct sizes the kernels use (kept in one place: the kernels take their layout from the same templates)
    const int prep_smem = prep_smem_bytes(DK);
    cudaError_t e = cudaFuncSetAttribute(gdn_chunked_prep_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem);
    if (e != cudaSuccess) return int(e);
    gdn_chunked_prep_kernel<DK><<<unsigned((blocks + 3) / 4), 128, prep_smem, s>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), g, beta, static_cast<uint8_t*>(ws), T, H, NB, blocks, scale);
    e = cudaGetLastError();
    if (e != cudaSuccess) return int(e);
    const int scan_smem = 3 * int(sizeof(ScanStage<DK>)) + 2 * CB * OT_PITCH * 4 + 128;
    e = cudaFuncSetAttribute(gdn_chunked_scan_kernel<DK, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, scan_smem);
    if (e != cudaSuccess) return int(e);
    gdn_chunked_scan_kernel<DK, TO><<<unsigned(B) * unsigned(H), DK == 64 ? 128 : 256, scan_smem, s>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
        static_cast<const uint8_t*>(ws), static_cast<TO*>(o), T, H, NB, scale);
    return int(cudaGetLastError());
}

}  // namespace
}  // namespace sb

extern "C" size_t shvk_gdn_chunked_workspace_bytes(int B, int T, int H) {
    if (B <= 0 || T <= 0 || H <= 0) return 0;
    return size_t(B) * size_t(H) * size_t((T + sb::CB - 1) / sb::CB) * size_t(sb::WS_BLOCK);
}

extern "C" int shvk_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o,
                                int o_dtype, int B, int T, int H, int DK, int DV, float scale, void* workspace,
                                size_t workspace_bytes, void* stream) {
    using namespace sb;
    if (B <= 0 || T <= 0 || H <= 0) return 0;
    if (DV != CDV || (DK != 64 && DK != 128) || (o_dtype != DT_F32 && o_dtype != DT_BF16)) return int(cudaErrorInvalidValue);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(workspace)) & 15)
        return int(cudaErrorInvalidValue);
    if (!workspace || workspace_bytes < shvk_gdn_chunked_workspace_bytes(B, T, H)) return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    if (DK == 64) {
        return o_dtype == DT_F32 ? launch_chunked<64, float>(q, k, v, g, beta, o, workspace, B, T, H, scale, s)
                                 : launch_chunked<64, __nv_bfloat16>(q, k, v, g, beta, o, workspace, B, T, H, scale, s);
    }
    return o_dtype == DT_F32 ? launch_chunked<128, float>(q, k, v, g, beta, o, workspace, B, T, H, scale, s)
                             : launch_chunked<128, __nv_bfloat16>(q, k, v, g, beta, o, workspace, B, T, H, scale, s);
}
