// IEEE fp32 GEMM on CUDA cores: C = epilogue(A * W^T), A [M,K], W [N,K], both K-contiguous.
//
// The exact tier and the last-row projections (which stay fp32 in every mode) run here.  Each output element is one
// thread's fma chain over k = 0..K-1 in order, K is never split, and the tile shape is fixed, so a row of C is bitwise
// independent of M and of the other rows in the batch (the row-independence contract of engine/include/shv_cuda.h:31-34
// and the k-order rule of engine/cuda/gemm.cuh:5-10).
//
// Tile 128 x 128 x 16, 256 threads, 8 x 8 outputs per thread as two 4-wide groups 64 apart in each direction so that
// the shared-memory reads are float4 broadcasts (A side) and 256-byte contiguous runs (W side).
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, PITCH = BM + 4, NTHREADS = 256;

struct Tile {
    float a[2][BK][PITCH];
    float w[2][BK][PITCH];
};

__device__ __forceinline__ float4 load_row4(const float* base, long long ld, int row, int rows, int k) {
    if (row < rows) return *reinterpret_cast<const float4*>(base + (long long)row * ld + k);
    return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

template <typename T>
__device__ __forceinline__ void epilogue_quad(const shvk_gemm_args& g, int m, int n, float v0, float v1, float v2, float v3) {
    if (m >= g.M || n >= g.N) return;
    if (g.swiglu) {                                   // (gate, up) pairs -> column n/2
        T* c = static_cast<T*>(g.C) + (long long)m * g.ldc + (n >> 1);
        c[0] = from_float<T>(silu_f(v0) * v1);
        if (n + 2 < g.N) c[1] = from_float<T>(silu_f(v2) * v3);
        return;
    }
    float v[4] = {v0, v1, v2, v3};
    const int cnt = min(4, g.N - n);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (j >= cnt) break;
        float x = v[j];
        if (g.bias) x += g.bias[n + j];
        if (g.act == 1) x = silu_f(x);
        if (g.R) {
            const float r = g.R[(long long)m * g.ldr + n + j];
            x = g.r_div != 1.0f ? r + x / g.r_div : r + x;
        }
        v[j] = x;
    }
    T* c = static_cast<T*>(g.C) + (long long)m * g.ldc + n;
    if (cnt == 4 && ((g.ldc | n) & 3) == 0) store_quad<T>(c, v[0], v[1], v[2], v[3]);
    else
        for (int j = 0; j < cnt; ++j) c[j] = from_float<T>(v[j]);
}

template <typename T>
__global__ void __launch_bounds__(NTHREADS)
gemm_f32_kernel(const shvk_gemm_args g) {
    __shared__ __align__(16) Tile sm;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const float* A = static_cast<const float*>(g.A);
    const float* W = static_cast<const float*>(g.W);
    // global -> shared: float4 slot s of the 128 x 16 tile: row s / 4, k quad s % 4 (two slots per thread)
    const int lrow0 = tid >> 2, lk = (tid & 3) * 4;
    float4 ra[2], rw[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            ra[i] = load_row4(A, g.lda, m0 + lrow0 + i * 64, g.M, k0 + lk);
            rw[i] = load_row4(W, g.ldw, n0 + lrow0 + i * 64, g.N, k0 + lk);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lrow0 + i * 64;
            sm.a[buf][lk + 0][r] = ra[i].x; sm.a[buf][lk + 1][r] = ra[i].y;
            sm.a[buf][lk + 2][r] = ra[i].z; sm.a[buf][lk + 3][r] = ra[i].w;
            sm.w[buf][lk + 0][r] = rw[i].x; sm.w[buf][lk + 1][r] = rw[i].y;
            sm.w[buf][lk + 2][r] = rw[i].z; sm.w[buf][lk + 3][r] = rw[i].w;
        }
    };
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    const int nk = g.K / BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kb = 0; kb < nk; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&sm.a[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&sm.a[buf][k][64 + ty * 4]);
            const float4 w0 = *reinterpret_cast<const float4*>(&sm.w[buf][k][tx * 4]);
            const float4 w1 = *reinterpret_cast<const float4*>(&sm.w[buf][k][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        if (kb + 1 < nk) {
            stash(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        epilogue_quad<T>(g, m, n0 + tx * 4, acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        epilogue_quad<T>(g, m, n0 + 64 + tx * 4, acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
}

}  // namespace
}  // namespace sb

extern "C" int shvk_gemm_f32(const shvk_gemm_args* g, void* stream) {
    if (!g || g->M <= 0 || g->N <= 0) return 0;
    if (g->K <= 0 || g->K % sb::BK || (g->lda & 3) || (g->ldw & 3) || (g->swiglu && (g->N & 3)) ||
        ((reinterpret_cast<uintptr_t>(g->A) | reinterpret_cast<uintptr_t>(g->W)) & 15))
        return int(cudaErrorInvalidValue);
    const dim3 grid(unsigned((g->N + sb::BN - 1) / sb::BN), unsigned((g->M + sb::BM - 1) / sb::BM));
    SB_DISPATCH_DTYPE(g->c_dtype, T, (sb::gemm_f32_kernel<T><<<grid, sb::NTHREADS, 0, cudaStream_t(stream)>>>(*g)));
    return int(cudaGetLastError());
}
