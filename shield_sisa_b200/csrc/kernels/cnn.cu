// Frame encoder kernels: MobileNetV3-Large features of 320x180 RGB crops (engine/cuda/cnn.cu, engine.cu:338-403 of
// the reference; CPU form engine/model/isa_impl.hpp:558-851; oracle/shieldv_ref.py:380-392).
//
// Layout: activations float32, NHWC, so that a 1x1 convolution is a row GEMM over pixels and the depthwise and
// pooling kernels read 16-byte channel quads.  BatchNorm arrives folded into weights and biases.  Every kernel is
// deterministic and computes a frame independently of the other frames of the batch (fixed reduction splits).
#include "device_utils.cuh"
#include "shv_cnn_kernels.h"

#include <mutex>
#include <string>

namespace sb {
namespace {

constexpr int kImgH = 180, kImgW = 320, kStemH = 90, kStemW = 160, kStemC = 16, kMapH = 6, kMapW = 10, kMapC = 960;

__device__ __forceinline__ float relu6_shift(float x) { return fminf(fmaxf(x + 3.0f, 0.0f), 6.0f); }
__device__ __forceinline__ float activate(float x, int act) {
    if (act == SHVK_ACT_RELU) return fmaxf(x, 0.0f);
    if (act == SHVK_ACT_HSWISH) return x * relu6_shift(x) / 6.0f;
    if (act == SHVK_ACT_HSIGMOID) return relu6_shift(x) / 6.0f;
    return x;
}

// ---------------------------------------------------------------------------------------------------- stem
// One thread per output pixel, 16 output channels in registers; lookup table and the 27x16 filter in shared memory.
__global__ void __launch_bounds__(256)
stem_kernel(const uint8_t* __restrict__ frames, const float* __restrict__ lut, const float* __restrict__ w,
            const float* __restrict__ b, float* __restrict__ out, long long npix) {
    __shared__ float s_lut[3 * 256];
    __shared__ __align__(16) float s_w[27 * kStemC];
    __shared__ float s_b[kStemC];
    for (int i = threadIdx.x; i < 3 * 256; i += blockDim.x) s_lut[i] = lut[i];
    for (int i = threadIdx.x; i < 27 * kStemC; i += blockDim.x) s_w[i] = w[i];
    if (threadIdx.x < kStemC) s_b[threadIdx.x] = b[threadIdx.x];
    __syncthreads();
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= npix) return;
    const int ox = int(p % kStemW), oy = int((p / kStemW) % kStemH);
    const long long f = p / (kStemW * kStemH);
    const uint8_t* img = frames + f * (long long)(kImgH * kImgW * 3);
    float acc[kStemC];
#pragma unroll
    for (int c = 0; c < kStemC; ++c) acc[c] = 0.0f;
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
        const int iy = 2 * oy - 1 + ky;
        if (iy < 0 || iy >= kImgH) continue;
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
            const int ix = 2 * ox - 1 + kx;
            if (ix < 0 || ix >= kImgW) continue;
            const uint8_t* px = img + ((long long)iy * kImgW + ix) * 3;
#pragma unroll
            for (int ci = 0; ci < 3; ++ci) {
                const float x = s_lut[ci * 256 + px[ci]];
                const float4* wr = reinterpret_cast<const float4*>(s_w + ((ky * 3 + kx) * 3 + ci) * kStemC);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 wv = wr[q];
                    acc[4 * q + 0] = fmaf(wv.x, x, acc[4 * q + 0]);
                    acc[4 * q + 1] = fmaf(wv.y, x, acc[4 * q + 1]);
                    acc[4 * q + 2] = fmaf(wv.z, x, acc[4 * q + 2]);
                    acc[4 * q + 3] = fmaf(wv.w, x, acc[4 * q + 3]);
                }
            }
        }
    }
    float4* o = reinterpret_cast<float4*>(out + p * kStemC);
#pragma unroll
    for (int q = 0; q < 4; ++q)
        o[q] = make_float4(activate(acc[4 * q] + s_b[4 * q], SHVK_ACT_HSWISH), activate(acc[4 * q + 1] + s_b[4 * q + 1], SHVK_ACT_HSWISH),
                           activate(acc[4 * q + 2] + s_b[4 * q + 2], SHVK_ACT_HSWISH),
                           activate(acc[4 * q + 3] + s_b[4 * q + 3], SHVK_ACT_HSWISH));
}

// ---------------------------------------------------------------------------------------------------- depthwise
// One thread per (four adjacent output pixels of a row, channel quad): per filter row the input columns the four
// outputs share are loaded once ((4 - 1) * stride + K float4 loads for 4 * K taps), taps are visited row by row in the
// same order for every output, and positions outside the image contribute a zero.
constexpr int DW_PX = 4;
template <int KS, int S>
__global__ void __launch_bounds__(256)
depthwise_kernel(const float* __restrict__ in, const float* __restrict__ w, const float* __restrict__ b,
                 float* __restrict__ out, long long total, int H, int W, int C, int Ho, int Wo, int act) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int C4 = C >> 2, GX = (Wo + DW_PX - 1) / DW_PX;
    const int c = int(i % C4) * 4;
    const long long grp = i / C4;
    const int ox0 = int(grp % GX) * DW_PX, oy = int((grp / GX) % Ho);
    const long long f = grp / ((long long)GX * Ho);
    constexpr int PAD = (KS - 1) / 2, NIN = (DW_PX - 1) * S + KS;
    const float* img = in + f * (long long)H * W * C + c;
    float4 acc[DW_PX];
#pragma unroll
    for (int p = 0; p < DW_PX; ++p) acc[p] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int ky = 0; ky < KS; ++ky) {
        const int iy = oy * S - PAD + ky;
        if (iy < 0 || iy >= H) continue;
        const float* row = img + (long long)iy * W * C;
        float4 x[NIN];
#pragma unroll
        for (int j = 0; j < NIN; ++j) {
            const int ix = ox0 * S - PAD + j;
            x[j] = (ix >= 0 && ix < W) ? *reinterpret_cast<const float4*>(row + (long long)ix * C) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int kx = 0; kx < KS; ++kx) {
            const float4 k = __ldg(reinterpret_cast<const float4*>(w + (ky * KS + kx) * C + c));
#pragma unroll
            for (int p = 0; p < DW_PX; ++p) {
                const float4 v = x[p * S + kx];
                acc[p].x = fmaf(k.x, v.x, acc[p].x);
                acc[p].y = fmaf(k.y, v.y, acc[p].y);
                acc[p].z = fmaf(k.z, v.z, acc[p].z);
                acc[p].w = fmaf(k.w, v.w, acc[p].w);
            }
        }
    }
    const float4 bias = __ldg(reinterpret_cast<const float4*>(b + c));
    float* o = out + ((f * Ho + oy) * (long long)Wo + ox0) * C + c;
#pragma unroll
    for (int p = 0; p < DW_PX; ++p)
        if (ox0 + p < Wo)
            *reinterpret_cast<float4*>(o + (long long)p * C) =
                make_float4(activate(acc[p].x + bias.x, act), activate(acc[p].y + bias.y, act), activate(acc[p].z + bias.z, act),
                            activate(acc[p].w + bias.w, act));
}

// ---------------------------------------------------------------------------------------------------- squeeze-excite
// Stage 1: partial[f][s][c] = sum over the 64 pixels of group s, eight strided pixel rows per block combined in order.
constexpr int kSeGroup = 64;
__global__ void __launch_bounds__(256)
se_partial_kernel(const float* __restrict__ x, float* __restrict__ partial, int HW, int C, int S) {
    __shared__ float4 red[8][32];
    const int f = blockIdx.x, s = blockIdx.y, lane = threadIdx.x & 31, pg = threadIdx.x >> 5;
    const int c = (blockIdx.z * 32 + lane) * 4;
    const int p0 = s * kSeGroup, p1 = min(HW, p0 + kSeGroup);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (c < C)
        for (int p = p0 + pg; p < p1; p += 8) {
            const float4 v = *reinterpret_cast<const float4*>(x + ((long long)f * HW + p) * C + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    red[pg][lane] = acc;
    __syncthreads();
    if (pg == 0 && c < C) {
        float4 t = red[0][lane];
#pragma unroll
        for (int r = 1; r < 8; ++r) {
            const float4 v = red[r][lane];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        *reinterpret_cast<float4*>(partial + ((long long)f * S + s) * C + c) = t;
    }
}
// Stage 2, one block of 32 warps per frame: mean, fc1 + ReLU, fc2 + Hardsigmoid; a warp per output, lanes over the
// inputs, four weight loads in flight per lane (the block is one latency chain: with 8 warps it took 1.6 to 2.8 times as long).
__global__ void __launch_bounds__(1024)
se_gate_kernel(const float* __restrict__ partial, const float* __restrict__ w1, const float* __restrict__ b1,
               const float* __restrict__ w2, const float* __restrict__ b2, float* __restrict__ gate, int HW, int C, int CS,
               int S) {
    extern __shared__ float se_smem[];
    float* pooled = se_smem;          // [C]
    float* hid = se_smem + C;         // [CS]
    const int f = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float t = 0.0f;
        for (int s = 0; s < S; ++s) t += partial[((long long)f * S + s) * C + c];
        pooled[c] = t / float(HW);
    }
    __syncthreads();
    // four outputs per warp at a time: their weight loads are in flight together; each output keeps its own
    // lane-strided sum and shuffle reduction, so the result does not depend on the grouping
    for (int j0 = warp * 4; j0 < CS; j0 += nwarp * 4) {
        float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* wr[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) wr[r] = w1 + (long long)min(j0 + r, CS - 1) * C;
#pragma unroll 2
        for (int c = lane; c < C; c += 32) {
            const float p = pooled[c];
#pragma unroll
            for (int r = 0; r < 4; ++r) t[r] = fmaf(__ldg(wr[r] + c), p, t[r]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float v = warp_sum(t[r]);
            if (lane == 0 && j0 + r < CS) hid[j0 + r] = fmaxf(v + b1[j0 + r], 0.0f);
        }
    }
    __syncthreads();
    for (int c0 = warp * 4; c0 < C; c0 += nwarp * 4) {
        float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* wr[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) wr[r] = w2 + (long long)min(c0 + r, C - 1) * CS;
#pragma unroll 2
        for (int j = lane; j < CS; j += 32) {
            const float h = hid[j];
#pragma unroll
            for (int r = 0; r < 4; ++r) t[r] = fmaf(__ldg(wr[r] + j), h, t[r]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float v = warp_sum(t[r]);
            if (lane == 0 && c0 + r < C) gate[(long long)f * C + c0 + r] = activate(v + b2[c0 + r], SHVK_ACT_HSIGMOID);
        }
    }
}

// ---------------------------------------------------------------------------------------------------- 1x1 convolution
// Row GEMM on CUDA cores, 256 threads, k in slabs of 8, next slab fetched into registers while the current one is
// consumed.  One fma chain over k per output, so a pixel's result does not depend on the tile shape's row count.
// Tile shapes (pixels x output channels, per-thread outputs): 256 x 16 and 128 x 32 and 64 x 64 with 4 x 4 for the narrow
// layers (every thread has live columns), 128 x 128 with 8 x 8 for the wide ones (half the shared-memory reads per fma).
constexpr int PW_K = 8;
template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(256)
pointwise_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                 const float* __restrict__ gate, int gate_rows, const float* R, float* out, int M, int N, int K, int act, int col_tiles) {
    static_assert((BM / TM) * (BN / TN) == 256, "256 threads");
    constexpr int NX = BN / TN, PA = BM + 4, PB = BN + 4, SLOTS = (BM + BN) * 2, PER = (SLOTS + 255) / 256;
    __shared__ __align__(16) float sa[2][PW_K][PA];
    __shared__ __align__(16) float sw[2][PW_K][PB];
    const int tid = threadIdx.x, tx = tid % NX, ty = tid / NX;
    const long long m0 = (long long)(blockIdx.x / col_tiles) * BM;   // column tiles of a row tile are neighbours
    const int n0 = int(blockIdx.x % col_tiles) * BN;
    // loader slots: slot i covers row i / 2 (A rows first, then W rows), k quad i % 2
    const float* src[PER];
    const float* gsrc[PER];
    float4 reg[PER];
#pragma unroll
    for (int r = 0; r < PER; ++r) {
        const int i = tid + r * 256, row = i >> 1;
        src[r] = nullptr;
        gsrc[r] = nullptr;
        if (i < SLOTS) {
            if (row < BM) {
                const long long m = m0 + row;
                if (m < M) {
                    src[r] = A + m * K + (i & 1) * 4;
                    if (gate) gsrc[r] = gate + (m / gate_rows) * K + (i & 1) * 4;
                }
            } else if (n0 + row - BM < N) {
                src[r] = W + (long long)(n0 + row - BM) * K + (i & 1) * 4;
            }
        }
    }
    auto fetch = [&](int k0) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            reg[r] = src[r] ? *reinterpret_cast<const float4*>(src[r] + k0) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (gsrc[r]) {
                const float4 g = *reinterpret_cast<const float4*>(gsrc[r] + k0);
                reg[r].x *= g.x; reg[r].y *= g.y; reg[r].z *= g.z; reg[r].w *= g.w;
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int i = tid + r * 256, row = i >> 1, kq = (i & 1) * 4;
            if (i >= SLOTS) continue;
            float* dst = row < BM ? &sa[buf][kq][row] : &sw[buf][kq][row - BM];
            const int pitch = row < BM ? PA : PB;
            dst[0] = reg[r].x; dst[pitch] = reg[r].y; dst[2 * pitch] = reg[r].z; dst[3 * pitch] = reg[r].w;
        }
    };
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    const int nk = K / PW_K;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kb = 0; kb < nk; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * PW_K);
#pragma unroll
        for (int k = 0; k < PW_K; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int h = 0; h < TM / 4; ++h) {       // row groups of four, BM / 2 apart when there are two
                const float4 a = *reinterpret_cast<const float4*>(&sa[buf][k][h * (BM / 2) + ty * 4]);
                av[4 * h] = a.x; av[4 * h + 1] = a.y; av[4 * h + 2] = a.z; av[4 * h + 3] = a.w;
            }
#pragma unroll
            for (int h = 0; h < TN / 4; ++h) {
                const float4 w = *reinterpret_cast<const float4*>(&sw[buf][k][h * (BN / 2) + tx * 4]);
                wv[4 * h] = w.x; wv[4 * h + 1] = w.y; wv[4 * h + 2] = w.z; wv[4 * h + 3] = w.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        if (kb + 1 < nk) {
            stash(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int hj = 0; hj < TN / 4; ++hj) {
        const int n = n0 + hj * (BN / 2) + tx * 4;
        if (n >= N) continue;
        const float4 bv = bias ? __ldg(reinterpret_cast<const float4*>(bias + n)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const long long m = m0 + (i / 4) * (BM / 2) + ty * 4 + (i & 3);
            if (m >= M) continue;
            float4 v = make_float4(activate(acc[i][4 * hj] + bv.x, act), activate(acc[i][4 * hj + 1] + bv.y, act),
                                   activate(acc[i][4 * hj + 2] + bv.z, act), activate(acc[i][4 * hj + 3] + bv.w, act));
            if (R) {
                const float4 r = *reinterpret_cast<const float4*>(R + m * N + n);
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
            *reinterpret_cast<float4*>(out + m * N + n) = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------------- 1x1 convolution, TF32
// The same row GEMM on the tensor cores for the 16-bit modes: operands rounded to TF32 (10-bit mantissa, float32
// range) on their way into shared memory, mma.sync m16n8k8 with float32 accumulation, float32 in and out.  These layers
// have K = 16 .. 160 in all but five cases and move 30 of the encoder's 46 MB per frame: they are bound by HBM, not by
// the tensor pipe, which is why this is a register-fed mma kernel and not a TMA / tcgen05 pipeline (whose 64-wide K
// tiles most of these layers would not fill).  256 threads = WM x WN warps, k in slabs of 16 (zero-filled past K),
// tiles row-major with a 20-float pitch: fragment reads and the 16-byte stores are conflict-free.
constexpr int PT_K = 16, PT_PITCH = 20;
__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int BM, int BN, int WM, int WN>
__global__ void __launch_bounds__(256, (BM / WM / 16) * (BN / WN / 8) > 10 ? 2 : (BM / WM / 16) * (BN / WN / 8) > 5 ? 3 : 4)
pointwise_tf32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                      const float* __restrict__ gate, int gate_rows, const float* R, float* out, int M, int N, int K, int act, int col_tiles) {
    static_assert(WM * WN == 8, "eight warps");
    constexpr int MT = BM / WM / 16, NT = BN / WN / 8, ROWS = BM + BN, SLOTS = ROWS * 4, PER = (SLOTS + 255) / 256;
    __shared__ __align__(16) float tile[2][ROWS][PT_PITCH];      // rows 0 .. BM-1: pixels, then BN rows of W
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int wm = warp % WM, wn = warp / WM;
    const long long m0 = (long long)(blockIdx.x / col_tiles) * BM;   // column tiles of a row tile are neighbours
    const int n0 = int(blockIdx.x % col_tiles) * BN;
    // loader slots: slot i covers tile row i / 4, k quad i % 4
    const int kq = (tid & 3) * 4;
    float4 reg[PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int row = (tid >> 2) + r * 64;
            reg[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (k0 + kq >= K) continue;
            if (row < BM) {
                const long long m = m0 + row;
                if (m < M) {
                    reg[r] = *reinterpret_cast<const float4*>(A + m * K + k0 + kq);
                    if (gate) {
                        const float4 gv = *reinterpret_cast<const float4*>(gate + (m / gate_rows) * K + k0 + kq);
                        reg[r].x *= gv.x; reg[r].y *= gv.y; reg[r].z *= gv.z; reg[r].w *= gv.w;
                    }
                }
            } else if (row < ROWS && n0 + row - BM < N) {
                reg[r] = __ldg(reinterpret_cast<const float4*>(W + (long long)(n0 + row - BM) * K + k0 + kq));
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int row = (tid >> 2) + r * 64;
            if (row >= ROWS) continue;
            *reinterpret_cast<float4*>(&tile[buf][row][kq]) =
                make_float4(to_tf32(reg[r].x), to_tf32(reg[r].y), to_tf32(reg[r].z), to_tf32(reg[r].w));
        }
    };
    float acc[MT][NT][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi)
#pragma unroll
        for (int ni = 0; ni < NT; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.0f;
    const int nk = (K + PT_K - 1) / PT_K;
    const int rb = wm * (BM / WM), nb = BM + wn * (BN / WN);
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kb = 0; kb < nk; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * PT_K);
#pragma unroll
        for (int ks = 0; ks < PT_K / 8; ++ks) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
                const float* r0 = &tile[buf][rb + mi * 16 + g][ks * 8 + t];
                a[mi][0] = __float_as_uint(r0[0]);
                a[mi][1] = __float_as_uint(r0[8 * PT_PITCH]);
                a[mi][2] = __float_as_uint(r0[4]);
                a[mi][3] = __float_as_uint(r0[8 * PT_PITCH + 4]);
            }
#pragma unroll
            for (int ni = 0; ni < NT; ++ni) {
                const float* w0 = &tile[buf][nb + ni * 8 + g][ks * 8 + t];
                const uint32_t b0 = __float_as_uint(w0[0]), b1 = __float_as_uint(w0[4]);
#pragma unroll
                for (int mi = 0; mi < MT; ++mi) mma_tf32(acc[mi][ni], a[mi], b0, b1);
            }
        }
        if (kb + 1 < nk) {
            stash(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int ni = 0; ni < NT; ++ni) {
        const int n = n0 + wn * (BN / WN) + ni * 8 + 2 * t;
        if (n >= N) continue;
        const float2 bv = bias ? __ldg(reinterpret_cast<const float2*>(bias + n)) : make_float2(0.0f, 0.0f);
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const long long m = m0 + rb + mi * 16 + g + h * 8;
                if (m >= M) continue;
                float2 v = make_float2(activate(acc[mi][ni][2 * h] + bv.x, act), activate(acc[mi][ni][2 * h + 1] + bv.y, act));
                if (R) {
                    const float2 r = *reinterpret_cast<const float2*>(R + m * N + n);
                    v.x += r.x; v.y += r.y;
                }
                *reinterpret_cast<float2*>(out + m * N + n) = v;
            }
    }
}

// ---------------------------------------------------------------------------------------------------- 1x1 convolution, 16-bit
// The same row GEMM with the operands rounded to the mode's 16-bit type (bf16 or fp16) on their way into shared
// memory and mma.sync m16n8k16: twice the contraction depth per shared-memory fragment and per mma of the TF32 form,
// k slabs of 32.  Float32 in, float32 accumulation, float32 out.
constexpr int PH_K = 32, PH_PITCH = 20;                       // 16 words of operands + 4 of padding per tile row
template <typename HT> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <typename HT> __device__ __forceinline__ void mma_16bit(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_16bit<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16bit<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int BM, int BN, int WM, int WN, typename HT>
__global__ void __launch_bounds__(256, (BM / WM / 16) * (BN / WN / 8) > 8 ? 2 : ((BM / WM / 16) * (BN / WN / 8) > 5 || BM == 256) ? 3 : 4)
pointwise_h_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                   const float* __restrict__ gate, int gate_rows, const float* R, float* out, int M, int N, int K, int act, int col_tiles) {
    static_assert(WM * WN == 8, "eight warps");
    constexpr int MT = BM / WM / 16, NT = BN / WN / 8, ROWS = BM + BN, PER = (ROWS + 63) / 64;
    __shared__ __align__(16) uint32_t tile[2][ROWS][PH_PITCH];   // rows 0 .. BM-1: pixels, then BN rows of W; 16-bit pairs
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int wm = warp % WM, wn = warp / WM;
    const long long m0 = (long long)(blockIdx.x / col_tiles) * BM;   // column tiles of a row tile are neighbours
    const int n0 = int(blockIdx.x % col_tiles) * BN;
    // loader slots: slot r of a thread covers tile row tid / 4 + 64 r, eight input channels starting at (tid % 4) * 8
    const int k8 = (tid & 3) * 8;
    float4 lo[PER], hi[PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int row = (tid >> 2) + r * 64;
            lo[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            hi[r] = lo[r];
            if (k0 + k8 >= K) continue;
            if (row < BM) {
                const long long m = m0 + row;
                if (m < M) {
                    const float4* p = reinterpret_cast<const float4*>(A + m * K + k0 + k8);
                    lo[r] = p[0];
                    hi[r] = p[1];
                    if (gate) {
                        const float4* gp = reinterpret_cast<const float4*>(gate + (m / gate_rows) * K + k0 + k8);
                        const float4 g0 = gp[0], g1 = gp[1];
                        lo[r].x *= g0.x; lo[r].y *= g0.y; lo[r].z *= g0.z; lo[r].w *= g0.w;
                        hi[r].x *= g1.x; hi[r].y *= g1.y; hi[r].z *= g1.z; hi[r].w *= g1.w;
                    }
                }
            } else if (row < ROWS && n0 + row - BM < N) {
                const float4* p = reinterpret_cast<const float4*>(W + (long long)(n0 + row - BM) * K + k0 + k8);
                lo[r] = __ldg(p);
                hi[r] = __ldg(p + 1);
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            const int row = (tid >> 2) + r * 64;
            if (row >= ROWS) continue;
            *reinterpret_cast<uint4*>(&tile[buf][row][(tid & 3) * 4]) =
                make_uint4(pack_pair<HT>(lo[r].x, lo[r].y), pack_pair<HT>(lo[r].z, lo[r].w), pack_pair<HT>(hi[r].x, hi[r].y),
                           pack_pair<HT>(hi[r].z, hi[r].w));
        }
    };
    float acc[MT][NT][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi)
#pragma unroll
        for (int ni = 0; ni < NT; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.0f;
    const int nk = (K + PH_K - 1) / PH_K;
    const int rb = wm * (BM / WM), nb = BM + wn * (BN / WN);
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kb = 0; kb < nk; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < nk) fetch((kb + 1) * PH_K);
#pragma unroll
        for (int ks = 0; ks < PH_K / 16; ++ks) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
                const uint32_t* r0 = &tile[buf][rb + mi * 16 + g][ks * 8 + t];
                a[mi][0] = r0[0];
                a[mi][1] = r0[8 * PH_PITCH];
                a[mi][2] = r0[4];
                a[mi][3] = r0[8 * PH_PITCH + 4];
            }
#pragma unroll
            for (int ni = 0; ni < NT; ++ni) {
                const uint32_t* w0 = &tile[buf][nb + ni * 8 + g][ks * 8 + t];
                const uint32_t b0 = w0[0], b1 = w0[4];
#pragma unroll
                for (int mi = 0; mi < MT; ++mi) mma_16bit<HT>(acc[mi][ni], a[mi], b0, b1);
            }
        }
        if (kb + 1 < nk) {
            stash(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int ni = 0; ni < NT; ++ni) {
        const int n = n0 + wn * (BN / WN) + ni * 8 + 2 * t;
        if (n >= N) continue;
        const float2 bv = bias ? __ldg(reinterpret_cast<const float2*>(bias + n)) : make_float2(0.0f, 0.0f);
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const long long m = m0 + rb + mi * 16 + g + h * 8;
                if (m >= M) continue;
                float2 v = make_float2(activate(acc[mi][ni][2 * h] + bv.x, act), activate(acc[mi][ni][2 * h + 1] + bv.y, act));
                if (R) {
                    const float2 r = *reinterpret_cast<const float2*>(R + m * N + n);
                    v.x += r.x; v.y += r.y;
                }
                *reinterpret_cast<float2*>(out + m * N + n) = v;
            }
    }
}

// ---------------------------------------------------------------------------------------------------- 4x4 pooling
__global__ void __launch_bounds__(256)
pool_tokens_kernel(const float* __restrict__ in, float* __restrict__ out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    constexpr int C4 = kMapC / 4;
    const int c = int(i % C4) * 4, tok = int((i / C4) % 16);
    const long long f = i / (16 * C4);
    const int r = tok >> 2, q = tok & 3;
    const int y0 = (r * kMapH) / 4, y1 = ((r + 1) * kMapH + 3) / 4, x0 = (q * kMapW) / 4, x1 = ((q + 1) * kMapW + 3) / 4;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int y = y0; y < y1; ++y)
        for (int x = x0; x < x1; ++x) {
            const float4 v = *reinterpret_cast<const float4*>(in + ((f * kMapH + y) * kMapW + x) * kMapC + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    const float cnt = float((y1 - y0) * (x1 - x0));
    *reinterpret_cast<float4*>(out + (f * 16 + tok) * kMapC + c) = make_float4(acc.x / cnt, acc.y / cnt, acc.z / cnt, acc.w / cnt);
}

inline unsigned blocks_for(long long n, int per) { return unsigned((n + per - 1) / per); }
inline bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

}  // namespace
}  // namespace sb

extern "C" int shvk_cnn_stem(const uint8_t* frames, const float* lut, const float* w, const float* b, float* out, int F,
                             void* stream) {
    if (F <= 0) return 0;
    if (sb::misaligned(out)) return int(cudaErrorInvalidValue);
    const long long npix = (long long)F * sb::kStemH * sb::kStemW;
    sb::stem_kernel<<<sb::blocks_for(npix, 256), 256, 0, cudaStream_t(stream)>>>(frames, lut, w, b, out, npix);
    return int(cudaGetLastError());
}

extern "C" int shvk_cnn_depthwise(const float* in, const float* w, const float* b, float* out, int F, int H, int W, int C,
                                  int K, int stride, int Ho, int Wo, int act, void* stream) {
    if (F <= 0) return 0;
    const int pad = (K - 1) / 2;
    if ((K != 3 && K != 5) || (stride != 1 && stride != 2) || (C & 3) || H <= 0 || W <= 0 ||
        Ho != (H + 2 * pad - K) / stride + 1 || Wo != (W + 2 * pad - K) / stride + 1 || sb::misaligned(in) ||
        sb::misaligned(out) || sb::misaligned(w) || sb::misaligned(b))
        return int(cudaErrorInvalidValue);
    const long long total = (long long)F * Ho * ((Wo + sb::DW_PX - 1) / sb::DW_PX) * (C / 4);
    const unsigned grid = sb::blocks_for(total, 256);
    cudaStream_t s = cudaStream_t(stream);
    if (K == 3 && stride == 1) sb::depthwise_kernel<3, 1><<<grid, 256, 0, s>>>(in, w, b, out, total, H, W, C, Ho, Wo, act);
    else if (K == 3) sb::depthwise_kernel<3, 2><<<grid, 256, 0, s>>>(in, w, b, out, total, H, W, C, Ho, Wo, act);
    else if (stride == 1) sb::depthwise_kernel<5, 1><<<grid, 256, 0, s>>>(in, w, b, out, total, H, W, C, Ho, Wo, act);
    else sb::depthwise_kernel<5, 2><<<grid, 256, 0, s>>>(in, w, b, out, total, H, W, C, Ho, Wo, act);
    return int(cudaGetLastError());
}

extern "C" size_t shvk_cnn_se_partial_floats(int F, int HW, int C) {
    if (F <= 0 || HW <= 0 || C <= 0) return 0;
    return size_t(F) * size_t((HW + sb::kSeGroup - 1) / sb::kSeGroup) * size_t(C);
}

extern "C" int shvk_cnn_se_gate(const float* x, float* partial, const float* w1, const float* b1, const float* w2,
                                const float* b2, float* gate, int F, int HW, int C, int CS, void* stream) {
    if (F <= 0) return 0;
    if (HW <= 0 || C <= 0 || (C & 3) || CS <= 0 || !partial || sb::misaligned(x) || sb::misaligned(partial))
        return int(cudaErrorInvalidValue);
    const int S = (HW + sb::kSeGroup - 1) / sb::kSeGroup;
    if (S > 65535) return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    sb::se_partial_kernel<<<dim3(unsigned(F), unsigned(S), unsigned((C + 127) / 128)), 256, 0, s>>>(x, partial, HW, C, S);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return int(e);
    const size_t smem = size_t(C + CS) * sizeof(float);
    if (smem > 48 * 1024) return int(cudaErrorInvalidValue);
    sb::se_gate_kernel<<<unsigned(F), 1024, smem, s>>>(partial, w1, b1, w2, b2, gate, HW, C, CS, S);
    return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------- no-allocation gate
// Scratch for shvk_cnn_se_gate_static.  In host code the name below is only a handle for cudaGetSymbolAddress, never a
// device address: the address is looked up with the caller's device current (on every call: the lookup allocates
// nothing, costs a table walk, and stays right after a device reset) and that pointer is what the kernels get.
static __device__ __align__(256) float g_se_static_partial[SHVK_CNN_SE_STATIC_FLOATS];

void shv_cuda_set_error(const std::string& s);   // thread-local error string behind shv_cuda_last_error (api.cpp)

extern "C" int shvk_cnn_se_gate_static(const float* x, const float* w1, const float* b1, const float* w2, const float* b2,
                                       float* gate, int F, int HW, int C, int CS, void* stream) {
    if (F <= 0) return 0;
    if (HW <= 0 || C <= 0) {
        shv_cuda_set_error("shvk_cnn_se_gate_static: HW and C must be positive");
        return int(cudaErrorInvalidValue);
    }
    const size_t need = shvk_cnn_se_partial_floats(F, HW, C);
    if (need > size_t(SHVK_CNN_SE_STATIC_FLOATS)) {
        shv_cuda_set_error("shvk_cnn_se_gate_static: " + std::to_string(need) + " floats of partial sums (F x ceil(HW / 64) x C) "
                           "do not fit the built-in " + std::to_string(SHVK_CNN_SE_STATIC_FLOATS) +
                           "; use shvk_cnn_se_gate with caller scratch or fewer frames per call");
        return int(cudaErrorInvalidValue);
    }
    void* scratch = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&scratch, g_se_static_partial);   // the current device's copy of the array
    if (e != cudaSuccess) {
        shv_cuda_set_error(std::string("shvk_cnn_se_gate_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        return int(e);
    }
    return shvk_cnn_se_gate(x, static_cast<float*>(scratch), w1, b1, w2, b2, gate, F, HW, C, CS, stream);
}

namespace sb {
namespace {
bool pointwise_args_bad(const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R,
                        const float* out, int N, int K) {
    return K <= 0 || (K % PW_K) || (N & 3) || (gate && gate_rows <= 0) || misaligned(A) || misaligned(W) || misaligned(out) ||
           (R && misaligned(R)) || (b && misaligned(b)) || (gate && misaligned(gate));
}
// tile width: wide layers take 128 columns; narrow ones the width in {16, 32, 64} that pads N least (ties: wider)
int pointwise_tile_width(int N) {
    if (N >= 112) return 128;
    int bn = 64, best = 1 << 30;
    for (int c : {64, 32, 16}) {
        const int padded = (N + c - 1) / c * c;
        if (padded < best) { best = padded; bn = c; }
    }
    return bn;
}
}  // namespace
}  // namespace sb

extern "C" int shvk_cnn_pointwise(const float* A, const float* W, const float* b, const float* gate, int gate_rows,
                                  const float* R, float* out, int M, int N, int K, int act, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (sb::pointwise_args_bad(A, W, b, gate, gate_rows, R, out, N, K)) return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    const int bn = sb::pointwise_tile_width(N);
    const unsigned gy = unsigned((N + bn - 1) / bn);
    if (bn == 128)
        sb::pointwise_kernel<128, 128, 8, 8><<<sb::blocks_for(M, 128) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    else if (bn == 64)
        sb::pointwise_kernel<64, 64, 4, 4><<<sb::blocks_for(M, 64) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    else if (bn == 32)
        sb::pointwise_kernel<128, 32, 4, 4><<<sb::blocks_for(M, 128) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    else
        sb::pointwise_kernel<256, 16, 4, 4><<<sb::blocks_for(M, 256) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    return int(cudaGetLastError());
}

extern "C" int shvk_cnn_pointwise_tf32(const float* A, const float* W, const float* b, const float* gate, int gate_rows,
                                       const float* R, float* out, int M, int N, int K, int act, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (sb::pointwise_args_bad(A, W, b, gate, gate_rows, R, out, N, K)) return int(cudaErrorInvalidValue);
    cudaStream_t s = cudaStream_t(stream);
    // layers of 24, 40, 72 or 80 output channels: one tile spans the whole row, so a block reads its pixels once and
    // writes whole contiguous rows (power-of-two column tiles re-read A up to five times and write 64-byte row pieces)
    if (N == 24 || N == 40 || N == 72 || N == 80) {
        const unsigned gx = sb::blocks_for(M, 128);
        if (N == 24) sb::pointwise_tf32_kernel<128, 24, 8, 1><<<gx, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, 1);
        else if (N == 40) sb::pointwise_tf32_kernel<128, 40, 8, 1><<<gx, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, 1);
        else if (N == 72) sb::pointwise_tf32_kernel<128, 72, 8, 1><<<gx, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, 1);
        else sb::pointwise_tf32_kernel<128, 80, 8, 1><<<gx, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, 1);
        return int(cudaGetLastError());
    }
    const int bn = sb::pointwise_tile_width(N);
    const unsigned gy = unsigned((N + bn - 1) / bn);
    if (bn == 128) {
        // wide layers: 64-column tiles (80 registers, three blocks per SM; the 128 x 128 tile needs 128 registers and
        // measured 5 % slower over the encoder); 128 rows per block, 64 when that leaves less than two waves of blocks
        const unsigned gy64 = unsigned((N + 63) / 64);
        if ((long long)sb::blocks_for(M, 128) * gy64 >= 2LL * 3 * 148)
            sb::pointwise_tf32_kernel<128, 64, 4, 2><<<sb::blocks_for(M, 128) * gy64, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy64));
        else
            sb::pointwise_tf32_kernel<64, 64, 4, 2><<<sb::blocks_for(M, 64) * gy64, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy64));
    }
    else if (bn == 64)
        sb::pointwise_tf32_kernel<64, 64, 4, 2><<<sb::blocks_for(M, 64) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    else if (bn == 32)
        sb::pointwise_tf32_kernel<128, 32, 8, 1><<<sb::blocks_for(M, 128) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    else
        sb::pointwise_tf32_kernel<256, 16, 8, 1><<<sb::blocks_for(M, 256) * gy, 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(gy));
    return int(cudaGetLastError());
}

namespace sb {
namespace {
template <typename HT>
int launch_pointwise_h(const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R, float* out,
                       int M, int N, int K, int act, cudaStream_t s) {
#define SB_PH(BM_, BN_, WM_, WN_, GY_) \
    pointwise_h_kernel<BM_, BN_, WM_, WN_, HT><<<blocks_for(M, BM_) * unsigned(GY_), 256, 0, s>>>(A, W, b, gate, gate_rows, R, out, M, N, K, act, int(GY_))
    if (N == 24) SB_PH(128, 24, 8, 1, 1);
    else if (N == 40) SB_PH(128, 40, 8, 1, 1);
    else if (N == 72) SB_PH(128, 72, 8, 1, 1);
    else if (N == 80) SB_PH(128, 80, 8, 1, 1);
    else {
        const int bn = pointwise_tile_width(N);
        const unsigned gy = unsigned((N + bn - 1) / bn);
        if (bn == 128) {
            const unsigned gy64 = unsigned((N + 63) / 64);
            if ((long long)blocks_for(M, 128) * gy64 >= 2LL * 3 * 148) SB_PH(128, 64, 4, 2, gy64);
            else SB_PH(64, 64, 4, 2, gy64);
        } else if (bn == 64) SB_PH(64, 64, 4, 2, gy);
        else if (bn == 32) SB_PH(128, 32, 8, 1, gy);
        else SB_PH(256, 16, 8, 1, gy);
    }
#undef SB_PH
    return int(cudaGetLastError());
}
}  // namespace
}  // namespace sb

extern "C" int shvk_cnn_pointwise_h(const float* A, const float* W, const float* b, const float* gate, int gate_rows,
                                    const float* R, float* out, int M, int N, int K, int act, int ab_dtype, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (sb::pointwise_args_bad(A, W, b, gate, gate_rows, R, out, N, K)) return int(cudaErrorInvalidValue);
    if (ab_dtype == sb::DT_BF16)
        return sb::launch_pointwise_h<__nv_bfloat16>(A, W, b, gate, gate_rows, R, out, M, N, K, act, cudaStream_t(stream));
    if (ab_dtype == sb::DT_F16)
        return sb::launch_pointwise_h<__half>(A, W, b, gate, gate_rows, R, out, M, N, K, act, cudaStream_t(stream));
    return int(cudaErrorInvalidValue);
}

extern "C" int shvk_cnn_pool_tokens(const float* in, float* out, int F, void* stream) {
    if (F <= 0) return 0;
    if (sb::misaligned(in) || sb::misaligned(out)) return int(cudaErrorInvalidValue);
    const long long total = (long long)F * 16 * (sb::kMapC / 4);
    sb::pool_tokens_kernel<<<sb::blocks_for(total, 256), 256, 0, cudaStream_t(stream)>>>(in, out, total);
    return int(cudaGetLastError());
}
