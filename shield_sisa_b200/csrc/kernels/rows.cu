// Row-wise kernels of the residual stream: token assembly fused with the first RMSNorm, RMSNorm, token-slot store.
// One warp owns one row of 384 floats (three float4 per lane), so every access is a 512-byte coalesced segment
// and the mean of squares is a single shuffle reduction.
#include "device_utils.cuh"
#include "shv_seq_kernels.h"

namespace sb {
namespace {

constexpr int kWarpsPerBlock = 8;

// Exact-tier operand split: x = hi + lo with hi = x rounded to TF32 (10 mantissa bits) and lo = x - hi (exact in
// fp32) rounded to TF32 as well, so neither piece has bits the tensor core would drop.
__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}
// Output type tag of the norm kernels in the exact tier: the normalised row leaves as the split A operand [lo | hi] of
// the tensor-core GEMM that reads it (a row of 2 x 384 floats), with no fp32 copy and no split launch in between.
struct Tf32Split {};
template <typename T> struct OutRow { using type = T; static constexpr int pitch = kD; };
template <> struct OutRow<Tf32Split> { using type = float; static constexpr int pitch = 2 * kD; };
template <typename T> __device__ __forceinline__ void store_norm4(typename OutRow<T>::type* out, float a, float b, float c, float d) {
    store_quad<T>(out, a, b, c, d);
}
template <> __device__ __forceinline__ void store_norm4<Tf32Split>(float* out, float a, float b, float c, float d) {
    const float4 hi = make_float4(tf32_rna(a), tf32_rna(b), tf32_rna(c), tf32_rna(d));
    *reinterpret_cast<float4*>(out) = make_float4(tf32_rna(a - hi.x), tf32_rna(b - hi.y), tf32_rna(c - hi.z), tf32_rna(d - hi.w));
    *reinterpret_cast<float4*>(out + kD) = hi;
}

template <typename T>
__device__ __forceinline__ void norm_store(const float4 (&v)[3], const float* __restrict__ w, typename OutRow<T>::type* __restrict__ out, int lane) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 3; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / float(kD) + 1e-6f);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int c = i * 128 + lane * 4;
        const float4 g = *reinterpret_cast<const float4*>(w + c);
        store_norm4<T>(out + c, (v[i].x * r) * g.x, (v[i].y * r) * g.y, (v[i].z * r) * g.z, (v[i].w * r) * g.w);
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
assemble_norm_kernel(const float* const* __restrict__ tok_ptrs, const float* __restrict__ pos,
                     const float* __restrict__ readout, const float* __restrict__ norm_w, float* __restrict__ h,
                     typename OutRow<T>::type* __restrict__ xn, long long rows) {
    const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const long long clip = row / kTok;
    const int t = int(row - clip * kTok);
    float4 v[3];
    if (t == kTok - 1) {
#pragma unroll
        for (int i = 0; i < 3; ++i) v[i] = *reinterpret_cast<const float4*>(readout + i * 128 + lane * 4);
    } else {
        const float* tok = tok_ptrs[clip * kFrames + (t >> 4)] + (t & 15) * kD;
        const float* pe = pos + (long long)t * kD;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const float4 a = *reinterpret_cast<const float4*>(tok + i * 128 + lane * 4);
            const float4 p = *reinterpret_cast<const float4*>(pe + i * 128 + lane * 4);
            v[i] = make_float4(a.x + p.x, a.y + p.y, a.z + p.z, a.w + p.w);
        }
    }
    float* hr = h + row * kD;
#pragma unroll
    for (int i = 0; i < 3; ++i) *reinterpret_cast<float4*>(hr + i * 128 + lane * 4) = v[i];
    norm_store<T>(v, norm_w, xn + row * OutRow<T>::pitch, lane);
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w, typename OutRow<T>::type* __restrict__ out,
               long long ldo, long long rows) {
    const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* xr = x + row * ldx;
    float4 v[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) v[i] = *reinterpret_cast<const float4*>(xr + i * 128 + lane * 4);
    norm_store<T>(v, w, out + row * ldo, lane);
}

// Scatter of token blocks into the slot pool, flat over all 128-bit words of the batch: word i belongs to block
// i / 1536, so a warp's 32 consecutive words are one 512-byte segment of one block and of its slot.
constexpr int kBlockWords = 16 * kD / 4;
__global__ void __launch_bounds__(256)
store_tokens_kernel(const float4* __restrict__ src, const int32_t* __restrict__ slots, float4* __restrict__ pool, long long words) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= words) return;
    const long long f = i / kBlockWords;
    const int s = __ldg(slots + f);
    if (s >= 0) pool[(long long)s * kBlockWords + (i - f * kBlockWords)] = src[i];
}

// Exact-tier operand split: x = hi + lo with hi = x rounded to TF32 (10 mantissa bits) and lo = x - hi (exact in
// fp32) rounded to TF32 as well, so neither piece has bits the tensor core would drop.  One thread per four elements.
//   layout 0 (activations): out row = [lo | hi]        (2K)
//   layout 1 (weights):     out row = [hi | lo | hi]   (3K)
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ in, long long ld_in, int k4, long long rows, float* __restrict__ out, long long ld_out,
                  int K, int layout) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * k4) return;
    const long long r = i / k4;
    const int c = int(i - r * k4) * 4;
    const float4 x = *reinterpret_cast<const float4*>(in + r * ld_in + c);
    float4 hi, lo;
    hi.x = tf32_rna(x.x); hi.y = tf32_rna(x.y); hi.z = tf32_rna(x.z); hi.w = tf32_rna(x.w);
    lo.x = tf32_rna(x.x - hi.x); lo.y = tf32_rna(x.y - hi.y); lo.z = tf32_rna(x.z - hi.z); lo.w = tf32_rna(x.w - hi.w);
    float* o = out + r * ld_out + c;
    if (layout == 0) {
        *reinterpret_cast<float4*>(o) = lo;
        *reinterpret_cast<float4*>(o + K) = hi;
    } else {
        *reinterpret_cast<float4*>(o) = hi;
        *reinterpret_cast<float4*>(o + K) = lo;
        *reinterpret_cast<float4*>(o + 2 * K) = hi;
    }
}

// fp16 token blocks that were uploaded into the upper halves of their fp32 staging blocks, widened in place: one CTA per
// block of 16 x 384 tokens, every thread reads its eight halves before anyone writes (the floats of the first half of
// the block land on bytes other threads still have to read).
__global__ void __launch_bounds__(768)
expand_f16_tokens_kernel(float* __restrict__ stage) {
    float* blk = stage + (long long)blockIdx.x * (16 * kD);
    const uint4 u = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(blk) + 16 * kD * 2)[threadIdx.x];
    __syncthreads();
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
    float4* out = reinterpret_cast<float4*>(blk) + 2 * threadIdx.x;
    out[0] = make_float4(a.x, a.y, b.x, b.y);
    out[1] = make_float4(c.x, c.y, d.x, d.y);
}

}  // namespace
}  // namespace sb

extern "C" int shvk_expand_f16_tokens(float* stage, int blocks, void* stream) {
    if (blocks <= 0) return 0;
    if (!stage || (reinterpret_cast<uintptr_t>(stage) & 15)) return int(cudaErrorInvalidValue);
    sb::expand_f16_tokens_kernel<<<unsigned(blocks), 768, 0, cudaStream_t(stream)>>>(stage);
    return int(cudaGetLastError());
}

extern "C" int shvk_split_tf32(const float* in, long long ld_in, int K, long long rows, float* out, long long ld_out, int layout,
                               void* stream) {
    if (rows <= 0) return 0;
    if (!in || !out || K <= 0 || (K & 3) || (ld_in & 3) || (ld_out & 3) || (layout != 0 && layout != 1) ||
        ld_out < (layout ? 3ll : 2ll) * K || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15))
        return int(cudaErrorInvalidValue);
    const long long n = rows * (K / 4);
    sb::split_tf32_kernel<<<unsigned((n + 255) / 256), 256, 0, cudaStream_t(stream)>>>(in, ld_in, K / 4, rows, out, ld_out, K, layout);
    return int(cudaGetLastError());
}

extern "C" int shvk_assemble_norm(const float* const* tok_ptrs, const float* pos, const float* readout,
                                  const float* norm_w, float* h, void* xn, int xn_dtype, int B, void* stream) {
    if (B <= 0) return 0;
    const long long rows = (long long)B * sb::kTok;
    const unsigned grid = unsigned((rows + sb::kWarpsPerBlock - 1) / sb::kWarpsPerBlock);
    if (xn_dtype == SHVK_F32_SPLIT) {
        sb::assemble_norm_kernel<sb::Tf32Split><<<grid, sb::kWarpsPerBlock * 32, 0, cudaStream_t(stream)>>>(
            tok_ptrs, pos, readout, norm_w, h, static_cast<float*>(xn), rows);
        return int(cudaGetLastError());
    }
    SB_DISPATCH_DTYPE(xn_dtype, T, (sb::assemble_norm_kernel<T><<<grid, sb::kWarpsPerBlock * 32, 0, cudaStream_t(stream)>>>(
                                       tok_ptrs, pos, readout, norm_w, h, static_cast<T*>(xn), rows)));
    return int(cudaGetLastError());
}

extern "C" int shvk_rmsnorm(const float* x, long long ldx, const float* w, void* out, int out_dtype, long long ldo,
                            int rows, void* stream) {
    if (rows <= 0) return 0;
    const unsigned grid = unsigned((rows + sb::kWarpsPerBlock - 1) / sb::kWarpsPerBlock);
    if (out_dtype == SHVK_F32_SPLIT) {
        if (ldo < 2 * sb::kD || (ldo & 3)) return int(cudaErrorInvalidValue);
        sb::rmsnorm_kernel<sb::Tf32Split><<<grid, sb::kWarpsPerBlock * 32, 0, cudaStream_t(stream)>>>(x, ldx, w, static_cast<float*>(out), ldo, rows);
        return int(cudaGetLastError());
    }
    SB_DISPATCH_DTYPE(out_dtype, T, (sb::rmsnorm_kernel<T><<<grid, sb::kWarpsPerBlock * 32, 0, cudaStream_t(stream)>>>(
                                        x, ldx, w, static_cast<T*>(out), ldo, rows)));
    return int(cudaGetLastError());
}

extern "C" int shvk_store_tokens(const float* tokens, const int32_t* slots, float* pool, int F, void* stream) {
    if (F <= 0) return 0;
    const long long words = (long long)F * sb::kBlockWords;
    sb::store_tokens_kernel<<<unsigned((words + 255) / 256), 256, 0, cudaStream_t(stream)>>>(
        reinterpret_cast<const float4*>(tokens), slots, reinterpret_cast<float4*>(pool), words);
    return int(cudaGetLastError());
}
