// Device-side helpers shared by the sequence kernels: storage-type packing, transcendental formulas, reductions.
// Arithmetic follows the reference's definitions (engine/cuda/common.cuh:70-78): sigmoid = 1/(1+exp(-x)),
// silu = x/(1+exp(-x)), softplus with threshold 20, logsigmoid = min(x,0) - log1p(exp(-|x|)).  No fast-math.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace sb {

// Storage type codes used across the C launch layer.
enum : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

constexpr int kD = 384, kTok = 321, kHeads = 6, kDK = 64, kDV = 128, kVD = 768, kDFF = 960;
constexpr int kState = 32, kPairs = 16, kFrames = 20;
// Fused GDN input projection: [q 384 | k 384 | v 768 | gate 768 | a 6 | b 6], row pitch 2320 (model.hpp:13-14).
constexpr int kGQ = 0, kGK = 384, kGV = 768, kGG = 1536, kGA = 2304, kGB = 2310, kGN = 2316, kGLD = 2320;
// Fused SISA all-row projection: [K 384 | V 384 | B 192 | theta 96 | alpha 6 | forget 6], pitch 1072 (model.hpp:15-16).
constexpr int kSK = 0, kSV = 384, kSB = 768, kSTheta = 960, kSAlpha = 1056, kSForget = 1062, kSN = 1068, kSLD = 1072;
constexpr int kSQ = 0, kSC = 384, kSQN = 576;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Four consecutive outputs in storage type T (16, 8 or 8 bytes, address aligned accordingly).
template <typename T> __device__ __forceinline__ void store_quad(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store_quad<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store_quad<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}
template <> __device__ __forceinline__ void store_quad<__half>(__half* p, float a, float b, float c, float d) {
    __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }

}  // namespace sb

// Dispatch a launcher body over the storage type code.
#define SB_DISPATCH_DTYPE(code, T, ...)                                   \
    switch (code) {                                                       \
    case sb::DT_F32: { using T = float; __VA_ARGS__; break; }             \
    case sb::DT_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }    \
    case sb::DT_F16: { using T = __half; __VA_ARGS__; break; }            \
    default: return int(cudaErrorInvalidValue);                           \
    }
