// Gated delta rule + gated RMSNorm for the 16-bit modes, fed by the chunk-blocked 16-bit operand tiles of the fused
// in-projection (gdn_inproj.cu, layout in gdn_pt_layout.cuh): the delta rule in chunks of 16 tokens on the tensor cores,
// in two kernels.
//
// For a chunk with inclusive cumulative log decay c_i, e_i = exp(c_i), state S0 (keys x values) entering the chunk:
//     A = K K^T, B = Q K^T                                      (16 x 16, contraction over the 64 keys)
//     L_ij = beta_i exp(c_i - c_j) A_ij (j < i),  T = (I + L)^-1,  T2 = T diag(beta),  M_ij = exp(c_i - c_j) B_ij (j <= i)
//     R = K S0,  QS = Q S0                                       (16 x 128)
//     U = T2 (V - diag(e) R)                                    (16 x 128)
//     O = M U + diag(e) QS
//     S' = e_16 S0 + K^T diag(exp(c_16 - c_j)) U
// k and q arrive un-normalised; their L2 norms are the diagonals of the Gram products K K^T and Q Q^T and enter as
// per-token scalars.  Operands are in the mode's 16-bit type (the output type T: bf16 or fp16), the state and all
// accumulation fp32.
//
// gdn_chunk_prep_kernel: the first two lines above (T2, M, the decays and the norms) depend on nothing but the chunk's own
// tiles, so they are computed for all chunks of the batch at once, a warp per pair of chunks, and stored behind the
// chunk's tiles (the block's last 1,280 bytes).  The 16 x 16 triangular inverse is a forward substitution in fp32, one
// column per lane.
//
// gdn_scan_t_kernel: one CTA (four warps) owns one (clip, head) and walks its 21 chunk blocks.  A block (q^T, k^T, v^T,
// gate^T tiles, log decays, betas, and what the preparation added: 13,696 contiguous bytes) arrives by ONE bulk copy into
// a three-slot ring, two chunks ahead.  Nothing is converted or re-laid-out: every operand fragment of the chunk's
// products comes straight out of the landed tiles with ldmatrix (transposing where the product wants tokens along the
// contraction).  Everything is computed transposed (value dimension = MMA rows): warp w owns value columns
// 32w .. 32w+31, keeps its slice of S^T (32 x 64, fp32) as the accumulator fragments of mma.sync.m16n8k16 for the whole
// sequence, and the accumulator layout of one product is exactly the A-operand layout of the next, so every hand-over
// is a register repack; T2 and M are read as B fragments from the block.
// Schedule of one chunk (one CTA barrier): every warp finishes four tokens of the PREVIOUS chunk (its o tile times rstd
// and the norm weight -> `on`; o tile and sums of squares are double-buffered), then R and Q S0, U, O (times the output
// gate, into the o tile), the state update and its share of sum(o^2) | barrier.
//
// Token slots past the end of the clip hold zeros in every tile (the producer writes them), which makes them inert:
// beta = 0, no decay, zero keys and values.  Their output rows are not stored.
//
// Warp-level mma.sync rather than tcgen05: per 16-token chunk the products form a dependency chain four deep on tiles of
// 16 tokens; tcgen05 needs M >= 64 rows and an asynchronous issue / commit / tensor-memory round trip per link of that
// chain, which costs more than the products themselves.  tcgen05 carries the projections (gemm_tc.cu, gdn_inproj.cu).
//
// Reference: engine/cuda/seq.cu:107-214 (delta + gated_norm), oracle/shieldv_ref.py:121-163.
#include <type_traits>

#include "device_utils.cuh"
#include "gdn_pt_layout.cuh"
#include "shv_seq_kernels.h"
#include "status_words.cuh"
#include "tma_utils.cuh"

namespace sb {
namespace {

constexpr int TC = pt::CHUNK, NCHUNK = pt::NCHUNK, NSLOT = 3;
constexpr uint32_t WAIT_POLLS = 1u << 22;    // about a quarter second
constexpr int OT_PITCH = kDV + 4;            // floats per token row of the o tile: the fragment stores of a warp (eight value rows
                                             // x four token pairs) then fall into 32 different banks

__device__ int g_scan_t_status = 0;

struct BlockExt {                            // what the preparation kernel adds to a chunk block
    uint16_t t2[TC][TC];                     // (I + L)^-1 diag(beta), operand type
    uint16_t mq[TC][TC];                     // decay-masked Q K^T, operand type
    float eg[TC], dj[TC];                    // exp(c_i), exp(c_last - c_i)
    float ik[TC], iq[TC];                    // 1/|k|, 0.125/|q|
};
struct Block {                               // one chunk block as it lies in global memory
    uint16_t qt[kDK][TC], kt[kDK][TC];       // operand type of the mode
    uint16_t vt[kDV][TC], gt[kDV][TC];       // fp16
    float dec[TC], beta[TC];
    BlockExt ext;
};
static_assert(sizeof(BlockExt) == pt::EXT_BYTES && offsetof(Block, ext) == pt::EXT_OFF && sizeof(Block) == pt::BLOCK_BYTES,
              "chunk block layout");

struct Smem {
    Block blk[NSLOT];                        // ring: chunk c lands in blk[c % 3]
    float ot[2][TC][OT_PITCH];               // o * gate of chunk c in ot[c % 2], [token][value]; read back by the next chunk's norm
    float ssq[2][TC][4];                     // per token: each warp's share of sum(o^2) over its 32 value columns
    unsigned long long full[NSLOT];          // mbarriers: chunk block in ring slot i landed
};
constexpr int SMEM_BYTES = int(sizeof(Smem)) + 128;

struct PrepWarp {                            // the preparation kernel's shared memory, per warp = per pair of chunks
    uint16_t qt[kDK][TC], kt[kDK][TC];       // tiles of the chunk being worked on
    float dec[TC], beta[TC];
    float cw[TC];                            // its inclusive cumulative log decay
    float beta2[2][TC];                      // betas of both chunks, for the inverse
    float lf[2][TC][TC];                     // L of both chunks
    BlockExt out[2];                         // staged, then copied to the blocks in 16-byte pieces
    float pad[16];                           // size a multiple of 128
};
constexpr int PREP_WARPS = 4;
static_assert(sizeof(PrepWarp) % 128 == 0 && offsetof(PrepWarp, out) % 16 == 0 && offsetof(PrepWarp, dec) == 4096, "prep layout");
constexpr int PREP_SMEM_BYTES = PREP_WARPS * int(sizeof(PrepWarp)) + 128;
constexpr int PREP_CTAS_PER_SM = 4;                   // by registers

// Operand type of the products: the mode's 16-bit type (bf16 keeps fp32's range, fp16 has three more mantissa bits).
// The v^T and gate^T tiles are fp16 in both modes: they are only read element-wise and combined in fp32.
template <typename OP> __device__ __forceinline__ uint32_t pack_op(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_op<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_op<__half>(float lo, float hi) {
    uint32_t r;                                                     // saturating: a finite fp16 even where fp32 exceeds 65504
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 h2_floats(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
// D (16x8, fp32) += A (16x16, row) * B (16x8, col), operands in OP
template <typename OP> __device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Four 8 x 8 bf16 matrices; lane l supplies the address of row l % 8 of matrix l / 8.  Thread (g, t) receives from
// matrix i the pair [row g][2t, 2t + 1] (plain) or [rows 2t, 2t + 1][column g] (transposed).
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}


// ---------------------------------------------------------------------------------------------- chunk preparation
// The part of a chunk's work that does not depend on the recurrent state, for every chunk of the batch at once: from
// q^T, k^T, log decays and betas the Gram products K K^T, Q K^T and diag(Q Q^T) on the tensor cores, the key and query
// norms from their diagonals, the decay masks, the 16 x 16 triangular inverse (forward substitution, fp32, one column
// per lane) and T2, M, exp(c), exp(c_last - c) and the norms into the block's last 1,280 bytes.  Inside the scan this
// chain (about half of a chunk's critical path, most of it one warp's dependent instructions while the other three
// waited) ran 21 times in sequence per (clip, head); here half a million chunks are independent.
//
// A warp walks pairs of chunk blocks.  The Gram products and masks of the two chunks run one after the other on all 32
// lanes; the inverse, which has work for 16 lanes per chunk, runs once for both (lanes 0-15 the first chunk, 16-31 the
// second).  The tiles of the next chunk are fetched into registers while the current one is computed.

// One chunk: tiles (already in w.qt / w.kt / w.dec / w.beta) -> L in w.lf[slot], everything but T2 in w.out[slot]
template <typename T>
__device__ __forceinline__ void prep_chunk(PrepWarp& w, int slot, int lane) {
    const int g = lane >> 2, t = lane & 3;                // mma fragment coordinates
    const int lm = lane >> 3, lr = lane & 7;              // ldmatrix lane roles: matrix lane / 8, row lane % 8
    BlockExt& out = w.out[slot];
    const uint32_t kt_s = tma::smem_addr(&w.kt[0][0]), qt_s = tma::smem_addr(&w.qt[0][0]);
    // transposed fragment of keys 16p .. 16p+15 x all 16 tokens (in rows 4-7 of every eight the two token halves of a
    // row trade places: gdn_pt_layout.cuh)
    const uint32_t tr_off = uint32_t(((lm >> 1) * 8 + lr) * (TC * 2) + ((lm & 1) ^ ((lr >> 2) & 1)) * 16);
    // inclusive prefix sum of the log decays
    float c = w.dec[lane & (TC - 1)];
#pragma unroll
    for (int o = 1; o < TC; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, c, o);
        if ((lane & (TC - 1)) >= o) c += up;
    }
    const float last = __shfl_sync(0xffffffffu, c, TC - 1);
    if (lane < TC) {
        w.cw[lane] = c;
        w.beta2[slot][lane] = w.beta[lane];
        out.eg[lane] = __expf(c);
        out.dj[lane] = __expf(last - c);
    }
    // Gram products over the 64 keys: K K^T, Q K^T and the diagonal of Q Q^T
    float ak[2][4], aq[2][4], dq[2][4];
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) { ak[ni][e] = 0.0f; aq[ni][e] = 0.0f; dq[ni][e] = 0.0f; }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        uint32_t kf[4], qf[4];
        ldsm4t(kt_s + uint32_t(p * 16 * TC * 2) + tr_off, kf);
        ldsm4t(qt_s + uint32_t(p * 16 * TC * 2) + tr_off, qf);
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            mma16816<T>(ak[ni], kf, kf[ni], kf[ni + 2]);
            mma16816<T>(aq[ni], qf, kf[ni], kf[ni + 2]);
            mma16816<T>(dq[ni], qf, qf[ni], qf[ni + 2]);
        }
    }
    // diagonal entries: row g sits in tile 0 at column 2t + e == g, row g + 8 in tile 1 at the same lane / slot
    if (t == (g >> 1)) {
        const bool odd = g & 1;                           // selects, not a runtime index: the fragments stay in registers
        out.ik[g] = rsqrtf((odd ? ak[0][1] : ak[0][0]) + 1e-6f);
        out.ik[g + 8] = rsqrtf((odd ? ak[1][3] : ak[1][2]) + 1e-6f);
        out.iq[g] = rsqrtf((odd ? dq[0][1] : dq[0][0]) + 1e-6f) * 0.125f;
        out.iq[g + 8] = rsqrtf((odd ? dq[1][3] : dq[1][2]) + 1e-6f) * 0.125f;
    }
    __syncwarp();
    // a*[ni][0,1]: row i = g, columns j = 8 ni + 2t, + 1;  a*[ni][2,3]: row i = g + 8
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = g + (e >> 1) * 8, j = 8 * ni + 2 * t + (e & 1);
            // one exponential serves both masks: exp(c_i - c_j) below the diagonal, exp(0) on it
            const float dec = __expf(j <= i ? w.cw[i] - w.cw[j] : 0.0f);
            // L_ij carries both key norms; in M the key norm of column j is applied to U in the scan's O product
            const float fl = w.beta[i] * out.ik[i] * out.ik[j];
            ak[ni][e] = j < i ? dec * ak[ni][e] * fl : 0.0f;
            aq[ni][e] = j <= i ? dec * aq[ni][e] * out.iq[i] : 0.0f;
        }
    uint32_t* mw = reinterpret_cast<uint32_t*>(&out.mq[0][0]);               // 8 words per row
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
        for (int e = 0; e < 4; ++e) w.lf[slot][g + (e >> 1) * 8][8 * ni + 2 * t + (e & 1)] = ak[ni][e];
        mw[g * 8 + 4 * ni + t] = pack_op<T>(aq[ni][0], aq[ni][1]);
        mw[(g + 8) * 8 + 4 * ni + t] = pack_op<T>(aq[ni][2], aq[ni][3]);
    }
}

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32, PREP_CTAS_PER_SM)
gdn_chunk_prep_kernel(uint8_t* __restrict__ ptb, long long npairs) {
    extern __shared__ uint8_t prep_smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    PrepWarp& w = reinterpret_cast<PrepWarp*>((reinterpret_cast<uintptr_t>(prep_smem_raw) + 127) & ~uintptr_t(127))[warp];
    const long long stride = (long long)gridDim.x * PREP_WARPS;
    long long pair = (long long)blockIdx.x * PREP_WARPS + warp;
    if (pair >= npairs) return;                           // whole warps leave; the kernel has no CTA barrier

    uint4 v[8], vg = make_uint4(0u, 0u, 0u, 0u);          // q^T | k^T (4 KB from the start of a block) and dec | beta, in flight
    auto fetch = [&](long long blk) {
        const uint8_t* gb = ptb + blk * pt::BLOCK_BYTES;
        const uint4* g4 = reinterpret_cast<const uint4*>(gb);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = g4[lane + 32 * i];
        if (lane < 8) vg = reinterpret_cast<const uint4*>(gb + pt::DEC_OFF)[lane];
    };
    auto land = [&]() {                                   // registers -> the warp's tile buffer
        uint4* s4 = reinterpret_cast<uint4*>(&w.qt[0][0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s4[lane + 32 * i] = v[i];
        if (lane < 8) reinterpret_cast<uint4*>(w.dec)[lane] = vg;
        __syncwarp();
    };
    fetch(2 * pair);
    for (; pair < npairs; pair += stride) {
        land();
        fetch(2 * pair + 1);                              // flies during the first chunk's products
        prep_chunk<T>(w, 0, lane);
        __syncwarp();                                     // every lane is done with the tile buffer
        land();
        if (pair + stride < npairs) fetch(2 * (pair + stride));   // flies during the second chunk's products and the inverse
        prep_chunk<T>(w, 1, lane);
        __syncwarp();
        {
            // column `lane % 16` of (I + L)^-1 of chunk `lane / 16` by forward substitution
            const int h = lane >> 4, col = lane & (TC - 1);
            float x[TC];
#pragma unroll
            for (int i = 0; i < TC; ++i) {
                // four partial sums: the dependent chain per row is i / 4 long instead of i
                float s0 = i == col ? 1.0f : 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                for (int j = 0; j < i; ++j) {
                    const float l = w.lf[h][i][j];
                    if ((j & 3) == 0) s0 = fmaf(-l, x[j], s0);
                    else if ((j & 3) == 1) s1 = fmaf(-l, x[j], s1);
                    else if ((j & 3) == 2) s2 = fmaf(-l, x[j], s2);
                    else s3 = fmaf(-l, x[j], s3);
                }
                x[i] = (s0 + s1) + (s2 + s3);
            }
            const float bc = w.beta2[h][col];
#pragma unroll
            for (int i = 0; i < TC; ++i) w.out[h].t2[i][col] = uint16_t(pack_op<T>(x[i] * bc, 0.0f) & 0xffffu);
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4* so = reinterpret_cast<const uint4*>(&w.out[h]);
            uint4* o4 = reinterpret_cast<uint4*>(ptb + (2 * pair + h) * pt::BLOCK_BYTES + pt::EXT_OFF);
            for (int i = lane; i < pt::EXT_BYTES / 16; i += 32) o4[i] = so[i];
        }
        __syncwarp();                                     // the staged outputs are read before the next pair overwrites them
    }
}

// Cycle counters of a development build (-DSHVK_DEV_PROBES): every warp adds the clock() ticks between the phase
// boundaries of its chunk loop to eight slots (0 block landed, 1 deferred norm, 2 R and Q S0, 3 U and O, 4 state update,
// 5 sum of squares, 6 barrier); one CTA in 61 adds its totals to g_scan_cycles, read and cleared by shvk_dev_scan_cycles.
#ifdef SHVK_DEV_PROBES
__device__ unsigned long long g_scan_cycles[4][8];
#define SCAN_TICK(slot) do { const unsigned now_ = unsigned(clock()); ticks[slot] += now_ - tick0; tick0 = now_; } while (0)
#else
#define SCAN_TICK(slot) do { } while (0)
#endif

template <typename T>
__global__ void __launch_bounds__(128, 3)
gdn_scan_t_kernel(const uint8_t* __restrict__ ptb, const float* __restrict__ o_norm_w, T* __restrict__ on, int* __restrict__ status,
                  uint32_t wait_polls, int starve) {
    extern __shared__ uint8_t scan_t_smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(scan_t_smem_raw) + 127) & ~uintptr_t(127));
    const int clip = blockIdx.x / kHeads, head = blockIdx.x % kHeads;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;               // mma fragment coordinates
    const long long row_base = (long long)clip * kTok;
    const int dvb = warp * 32;                           // this warp's value columns
    const uint8_t* src = ptb + (long long)blockIdx.x * pt::HEAD_BYTES;
    // ldmatrix lane roles: matrix lane / 8, row lane % 8
    const int lm = lane >> 3, lr = lane & 7;

    // S^T slice of this warp as accumulator fragments: S[mi][nj][.] = values dvb + 16 mi + {g, g + 8}, keys 8 nj + 2t, + 1
    float S[2][8][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int nj = 0; nj < 8; ++nj)
#pragma unroll
            for (int e = 0; e < 4; ++e) S[mi][nj][e] = 0.0f;

    const uint32_t bars0 = tma::smem_addr(&sm.full[0]);   // + 8 * ring slot
    auto issue = [&](int chunk) {                         // thread 0: the block of `chunk`
        if (starve) return;
        const uint32_t bar = bars0 + 8u * uint32_t(chunk % NSLOT);
        tma::mbar_expect_tx(bar, uint32_t(pt::BLOCK_BYTES));
        tma::load_bulk(tma::smem_addr(&sm.blk[chunk % NSLOT]), src + (long long)chunk * pt::BLOCK_BYTES, uint32_t(pt::BLOCK_BYTES), bar);
    };
    if (tid == 0) {
        for (int i = 0; i < NSLOT; ++i) tma::mbar_init(bars0 + 8u * i, 1);
        tma::fence_barrier_init();
        tma::fence_proxy_async();
        issue(0);
        issue(1);
    }
    __syncthreads();

    const float4 onw = __ldg(reinterpret_cast<const float4*>(o_norm_w + lane * 4));   // once: a load here every chunk would wait on L2
    // The previous chunk's output: o tile times rstd times the norm weight, tokens first .. first + count - 1 of chunk pc.
    // Loads and arithmetic run unconditionally (the tile rows exist), only the store is guarded.
    auto finish_norm = [&](int pc, int first, auto count_c) {
        constexpr int count = decltype(count_c)::value;   // compile-time, so a warp with few tokens does only their work
        const int pnt = min(min(TC, kTok - pc * TC), first + count);
        const float* op = &sm.ot[pc & 1][first][lane * 4];
        const float* sp = &sm.ssq[pc & 1][first][0];
        T* dst = on + (row_base + pc * TC + first) * kVD + head * kDV + lane * 4;
#pragma unroll
        for (int k = 0; k < count; ++k) {
            const float4 o = *reinterpret_cast<const float4*>(op + k * OT_PITCH);
            const float4 pp = *reinterpret_cast<const float4*>(sp + 4 * k);   // the four warps' partial sums of o^2
            const float rstd = rsqrtf(((pp.x + pp.y) + (pp.z + pp.w)) * (1.0f / float(kDV)) + 1e-6f);
            if (first + k < pnt)
                store_quad<T>(dst + k * kVD, (o.x * rstd) * onw.x, (o.y * rstd) * onw.y, (o.z * rstd) * onw.z, (o.w * rstd) * onw.w);
        }
    };

#ifdef SHVK_DEV_PROBES
    unsigned ticks[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    unsigned tick0 = unsigned(clock());
#endif
    for (int chunk = 0; chunk < NCHUNK; ++chunk) {
        Block& b = sm.blk[chunk % NSLOT];
        if (tid == 0 && chunk + 2 < NCHUNK) {
            // ring slot (chunk + 2) % 3 was last read by chunk - 1, which ended at the previous barrier
            tma::fence_proxy_async();
            issue(chunk + 2);
        }
        if (!tma::mbar_wait_bounded(bars0 + 8u * uint32_t(chunk % NSLOT), uint32_t(chunk / NSLOT) & 1u, wait_polls)) {
            if (tid == 0) atomicCAS(status, 0, 1);
            return;                                       // every thread times out on the same barrier and leaves
        }
        SCAN_TICK(0);
        const uint32_t kt_s = tma::smem_addr(&b.kt[0][0]), qt_s = tma::smem_addr(&b.qt[0][0]);
        // transposed fragment of keys 16p .. 16p+15 x all 16 tokens: matrices (keys lo, tokens 0-7), (keys lo, tokens 8-15),
        // (keys hi, tokens 0-7), (keys hi, tokens 8-15) = A fragment of [token][key], and B fragments (r[ni], r[ni + 2])
        // (in rows 4-7 of every eight the two token halves of a row trade places: gdn_pt_layout.cuh)
        const uint32_t tr_off = uint32_t(((lm >> 1) * 8 + lr) * (TC * 2) + ((lm & 1) ^ ((lr >> 2) & 1)) * 16);
        // the previous chunk is finished first: four tokens per warp (its o tile and sums of squares lie in the other buffer)
        if (chunk > 0) finish_norm(chunk - 1, 4 * warp, std::integral_constant<int, 4>());
        SCAN_TICK(1);
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
            uint32_t bk[4], bq[4];
            ldsm4t(kt_s + uint32_t(p * 16 * TC * 2) + tr_off, bk);
            ldsm4t(qt_s + uint32_t(p * 16 * TC * 2) + tr_off, bq);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                // keys 16p .. 16p+15 of the state as an A fragment: two adjacent accumulator tiles, rounded to bf16
                const uint32_t sa[4] = {pack_op<T>(S[mi][2 * p][0], S[mi][2 * p][1]), pack_op<T>(S[mi][2 * p][2], S[mi][2 * p][3]),
                                        pack_op<T>(S[mi][2 * p + 1][0], S[mi][2 * p + 1][1]),
                                        pack_op<T>(S[mi][2 * p + 1][2], S[mi][2 * p + 1][3])};
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    mma16816<T>(R[mi][ni], sa, bk[ni], bk[ni + 2]);
                    mma16816<T>(QS[mi][ni], sa, bq[ni], bq[ni + 2]);
                }
            }
        }
        SCAN_TICK(2);
        // ---------------------------------------------------------------- U^T = (V - diag(e) R)^T T2^T
        const BlockExt& x = b.ext;                        // T2, M, decays and norms of this chunk, prepared ahead of the scan
        const uint32_t* t2w = reinterpret_cast<const uint32_t*>(&x.t2[0][0]);    // 8 words per row
        const uint32_t* mqw = reinterpret_cast<const uint32_t*>(&x.mq[0][0]);
        // per-token scalars of this lane's tokens 8 ni + 2t, + 1, with the norms folded in:
        //   er = exp(c) / |k|  (R = K S0),  eq = exp(c) * 0.125 / |q|  (Q S0),  dj2 = exp(c_last - c) / |k|  (state update)
        float er[2][2], eq[2][2], dj2[2][2], ikt[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = 8 * ni + 2 * t + e;
                const float egv = x.eg[tok], ikv = x.ik[tok];
                er[ni][e] = egv * ikv;
                eq[ni][e] = egv * x.iq[tok];
                dj2[ni][e] = x.dj[tok] * ikv;
                ikt[ni][e] = ikv;
            }
        uint32_t bt[2][2], bm[2][2];
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
            bt[ni][0] = t2w[(8 * ni + g) * 8 + t]; bt[ni][1] = t2w[(8 * ni + g) * 8 + t + 4];
            bm[ni][0] = mqw[(8 * ni + g) * 8 + t]; bm[ni][1] = mqw[(8 * ni + g) * 8 + t + 4];
        }
        float sq[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};    // sum of o^2 over this thread's value rows, per token 8 ni + 2t + e
        uint32_t da[2][4];                                // decay-scaled U^T as A fragments, for the state update
        // every shared-memory load of this phase is issued before its first o-tile store (a store would hold back the
        // loads behind it): V^T and gate^T for both row halves and the K^T fragments of the state update
        // plain fragments of rows r0 .. r0+15 x 16 tokens: matrices (rows lo, tokens 0-7), (rows lo, tokens 8-15),
        // (rows hi, tokens 0-7), (rows hi, tokens 8-15): r[ni + 2 h] = tokens 8 ni + 2t, + 1 of row r0 + 8 h + g
        const uint32_t pl_off = tr_off;                   // same four matrices, read without the transpose
        uint32_t vv[2][4], gg[2][4], kf[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ldsm4(kt_s + uint32_t(q * 16 * TC * 2) + pl_off, kf[q]);   // kf[q][2 h + c]: keys 16 q + 8 h + g, tokens 8 c + 2t
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
            ldsm4(tma::smem_addr(&b.vt[dvb + 16 * mi][0]) + pl_off, vv[mi]);
            ldsm4(tma::smem_addr(&b.gt[dvb + 16 * mi][0]) + pl_off, gg[mi]);
        }
        float* otile = &sm.ot[chunk & 1][0][0];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
            const int r0 = dvb + 16 * mi + g, r1 = r0 + 8;
            uint32_t va[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                const float2 v0 = h2_floats(vv[mi][ni]), v1 = h2_floats(vv[mi][ni + 2]);
                va[2 * ni] = pack_op<T>(v0.x - er[ni][0] * R[mi][ni][0], v0.y - er[ni][1] * R[mi][ni][1]);
                va[2 * ni + 1] = pack_op<T>(v1.x - er[ni][0] * R[mi][ni][2], v1.y - er[ni][1] * R[mi][ni][3]);
            }
            float U[2][4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
                for (int e = 0; e < 4; ++e) U[ni][e] = 0.0f;
                mma16816<T>(U[ni], va, bt[ni][0], bt[ni][1]);
            }
            uint32_t ua[4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                ua[2 * ni] = pack_op<T>(U[ni][0] * ikt[ni][0], U[ni][1] * ikt[ni][1]);      // U / |k| for the O product
                ua[2 * ni + 1] = pack_op<T>(U[ni][2] * ikt[ni][0], U[ni][3] * ikt[ni][1]);
                da[mi][2 * ni] = pack_op<T>(U[ni][0] * dj2[ni][0], U[ni][1] * dj2[ni][1]);
                da[mi][2 * ni + 1] = pack_op<T>(U[ni][2] * dj2[ni][0], U[ni][3] * dj2[ni][1]);
            }
            // O^T = U^T M^T + diag(e) (Q S0)^T, stored times the output gate; sum(o^2) is taken before the gate
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) {
                float O[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma16816<T>(O, ua, bm[ni][0], bm[ni][1]);
                const int tok = 8 * ni + 2 * t;
                const float o00 = O[0] + eq[ni][0] * QS[mi][ni][0], o01 = O[1] + eq[ni][1] * QS[mi][ni][1];
                const float o10 = O[2] + eq[ni][0] * QS[mi][ni][2], o11 = O[3] + eq[ni][1] * QS[mi][ni][3];
                const float2 g0 = h2_floats(gg[mi][ni]), g1 = h2_floats(gg[mi][ni + 2]);
                otile[tok * OT_PITCH + r0] = o00 * g0.x;
                otile[(tok + 1) * OT_PITCH + r0] = o01 * g0.y;
                otile[tok * OT_PITCH + r1] = o10 * g1.x;
                otile[(tok + 1) * OT_PITCH + r1] = o11 * g1.y;
                sq[ni][0] = fmaf(o00, o00, fmaf(o10, o10, sq[ni][0]));
                sq[ni][1] = fmaf(o01, o01, fmaf(o11, o11, sq[ni][1]));
            }
        }
        SCAN_TICK(3);
        // ---------------------------------------------------------------- S^T <- e_last S^T + (diag(d) U)^T K
        {
            const float elast = x.eg[TC - 1];
#pragma unroll
            for (int nj = 0; nj < 8; ++nj) {
                // keys 8 nj + g: fragment kf[nj / 2], row half nj % 2; tokens 2t, + 1 (b0) and 8 + 2t, + 1 (b1)
                const uint32_t b0 = kf[nj >> 1][2 * (nj & 1)], b1 = kf[nj >> 1][2 * (nj & 1) + 1];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[mi][nj][e] *= elast;
                    mma16816<T>(S[mi][nj], da[mi], b0, b1);
                }
            }
        }
        SCAN_TICK(4);
        // this warp's share of sum(o^2): reduce over the eight row groups g (lane bits 2-4), lanes 0-3 publish it
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = sq[ni][e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (g == 0) sm.ssq[chunk & 1][8 * ni + 2 * t + e][warp] = v;
            }
        SCAN_TICK(5);
        __syncthreads();                                  // the chunk's o tile is complete; its ring slot is free
        SCAN_TICK(6);
    }
#ifdef SHVK_DEV_PROBES
    if (lane == 0 && blockIdx.x % 61 == 7)
        for (int k = 0; k < 8; ++k) atomicAdd(&g_scan_cycles[warp][k], (unsigned long long)ticks[k]);
#endif
    finish_norm(NCHUNK - 1, 4 * warp, std::integral_constant<int, 4>());
}

template <typename T>
int launch(const void* ptb, const float* o_norm_w, void* on, int B, uint32_t polls, int starve, cudaStream_t stream) {
    const cudaError_t e = cudaFuncSetAttribute(gdn_scan_t_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    int* status = gdn_scan_t_status_word();
    if (!status) return int(cudaErrorInvalidSymbol);
    gdn_scan_t_kernel<T><<<unsigned(B) * kHeads, 128, SMEM_BYTES, stream>>>(static_cast<const uint8_t*>(ptb), o_norm_w,
                                                                            static_cast<T*>(on), status, polls, starve);
    return int(cudaGetLastError());
}

template <typename T>
int launch_prep(void* ptb, int B, cudaStream_t stream) {
    const cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    static_assert((kHeads * NCHUNK) % 2 == 0, "a clip's chunk blocks come in pairs");
    const long long npairs = (long long)B * kHeads * NCHUNK / 2;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long want = (npairs + PREP_WARPS - 1) / PREP_WARPS, cap = (long long)sms * PREP_CTAS_PER_SM;
    gdn_chunk_prep_kernel<T><<<unsigned(want < cap ? want : cap), PREP_WARPS * 32, PREP_SMEM_BYTES, stream>>>(
        static_cast<uint8_t*>(ptb), npairs);
    return int(cudaGetLastError());
}

int launch_any(const void* ptb, const float* o_norm_w, void* on, int on_dtype, int B, uint32_t polls, int starve, void* stream) {
    if (B <= 0) return 0;
    if (!ptb || !o_norm_w || !on || (reinterpret_cast<uintptr_t>(ptb) & 127) || (reinterpret_cast<uintptr_t>(on) & 7))
        return int(cudaErrorInvalidValue);
    if (on_dtype == DT_BF16) return launch<__nv_bfloat16>(ptb, o_norm_w, on, B, polls, starve, cudaStream_t(stream));
    if (on_dtype == DT_F16) return launch<__half>(ptb, o_norm_w, on, B, polls, starve, cudaStream_t(stream));
    return int(cudaErrorInvalidValue);
}

}  // namespace

int* gdn_scan_t_status_word() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scan_t_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

}  // namespace sb

extern "C" int shvk_gdn_chunk_prep(void* ptb, int op_dtype, int B, void* stream) {
    if (B <= 0) return 0;
    if (!ptb || (reinterpret_cast<uintptr_t>(ptb) & 127)) return int(cudaErrorInvalidValue);
    if (op_dtype == sb::DT_BF16) return sb::launch_prep<__nv_bfloat16>(ptb, B, cudaStream_t(stream));
    if (op_dtype == sb::DT_F16) return sb::launch_prep<__half>(ptb, B, cudaStream_t(stream));
    return int(cudaErrorInvalidValue);
}

extern "C" int shvk_gdn_scan_t(const void* ptb, const float* o_norm_w, void* on, int on_dtype, int B, void* stream) {
    return sb::launch_any(ptb, o_norm_w, on, on_dtype, B, sb::WAIT_POLLS, 0, stream);
}

extern "C" int shvk_gdn_scan_t_starved(const void* ptb, const float* o_norm_w, void* on, int on_dtype, int B, int polls,
                                       void* stream) {
    const uint32_t lim = polls < 256 ? 256u : (uint32_t(polls) > sb::WAIT_POLLS ? sb::WAIT_POLLS : uint32_t(polls));
    return sb::launch_any(ptb, o_norm_w, on, on_dtype, B, lim, 1, stream);
}

#ifdef SHVK_DEV_PROBES
// Development builds only: the scan's cycle counters [4 warps][8 slots], read and cleared (synchronises the device).
extern "C" __attribute__((visibility("default"))) int shvk_dev_scan_cycles(unsigned long long* out) {
    unsigned long long zero[32] = {0};
    if (cudaDeviceSynchronize() != cudaSuccess) return int(cudaGetLastError());
    cudaMemcpyFromSymbol(out, sb::g_scan_cycles, sizeof(zero));
    cudaMemcpyToSymbol(sb::g_scan_cycles, zero, sizeof(zero));
    return int(cudaGetLastError());
}
#endif
