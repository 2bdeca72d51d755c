/*
 * shv_cnn_kernels.h -- thin C launch layer over the sm_100a frame-encoder kernels of the SHIELD-V engine
 * (MobileNetV3-Large features on 320x180 crops, 4x4 pooling; the 960 -> 384 token projection is shvk_gemm_f32).
 *
 * Same conventions as shv_seq_kernels.h: every pointer is a device pointer, `stream` is a cudaStream_t passed as
 * void*, every function only enqueues work and returns a cudaError_t value (0 = success).  Activations are float32 in
 * NHWC order ([frame][row][column][channel]); BatchNorm is folded into weights and biases by the caller.
 * Activation codes: 0 none, 1 ReLU, 2 Hardswish (x * relu6(x + 3) / 6), 4 Hardsigmoid (relu6(x + 3) / 6).
 *
 * Each entry replaces one launcher of the reference engine; citations are to the reference tree.
 */
#ifndef SHV_CNN_KERNELS_H
#define SHV_CNN_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

enum { SHVK_ACT_NONE = 0, SHVK_ACT_RELU = 1, SHVK_ACT_HSWISH = 2, SHVK_ACT_HSIGMOID = 4 };

/* Stem: uint8 RGB crops [F][180][320][3] -> normalisation through lut ([3][256]: ((u / 255) - mean_c) / std_c)
 * -> 3x3 convolution, stride 2, padding 1, 16 output channels -> + b -> Hardswish -> out [F][90][160][16].
 * w: [27][16], tap-major: ((kh * 3 + kw) * 3 + ci) * 16 + co.
 * Replaces launch_stem (engine/cuda/cnn.cu:8-50,164-167). */
int shvk_cnn_stem(const uint8_t* frames, const float* lut, const float* w, const float* b, float* out, int F,
                  void* stream);

/* Depthwise KxK convolution (K 3 or 5, stride 1 or 2, padding (K-1)/2) + b + activation.
 * in [F][H][W][C] -> out [F][Ho][Wo][C]; w: [K*K][C] tap-major; C a multiple of 4.
 * Replaces launch_dw (engine/cuda/cnn.cu:52-95,169-179). */
int shvk_cnn_depthwise(const float* in, const float* w, const float* b, float* out, int F, int H, int W, int C, int K,
                       int stride, int Ho, int Wo, int act, void* stream);

/* Squeeze-excite gate of F frames: mean over the HW pixels of each channel, fc1 + ReLU, fc2 + Hardsigmoid.
 * x [F][HW][C]; w1 [CS][C], b1 [CS]; w2 [C][CS], b2 [C]; gate [F][C].  The mean is taken in two stages with a split
 * that depends only on HW (64-pixel groups, combined in order), so a frame's gate does not depend on F.
 * `partial` is scratch the caller provides: shvk_cnn_se_partial_floats(F, HW, C) floats; it need not be cleared.
 * Replaces launch_se_pool and the two squeeze-excite GEMMs (engine/cuda/cnn.cu:97-131,181-186;
 * engine/cuda/engine.cu:367-376). */
size_t shvk_cnn_se_partial_floats(int F, int HW, int C);
int shvk_cnn_se_gate(const float* x, float* partial, const float* w1, const float* b1, const float* w2, const float* b2,
                     float* gate, int F, int HW, int C, int CS, void* stream);

/* shvk_cnn_se_gate without caller-provided scratch and without any device allocation.  No counterpart in the reference
 * (its engine allocates the partial-sum buffer with the rest of its arena, engine/cuda/engine.cu:246-262).
 *
 * For callers that cannot allocate device memory when they need the gate: a host that handed the whole GPU to its own
 * memory pool at start-up, or a frame loop in which cudaMalloc's device-wide synchronisation and its chance of failing
 * are not acceptable.  The partial sums live in an array that is part of the library image: SHVK_CNN_SE_STATIC_FLOATS
 * floats (1 MiB) on every GPU that loads the library, held until the process exits.  The call is refused with
 * cudaErrorInvalidValue, and shv_cuda_last_error() says why, when shvk_cnn_se_partial_floats(F, HW, C) exceeds that
 * (the largest squeeze-excite layer of the encoder, 240 pixels x 672 channels, fits 97 frames).
 *
 * Every call looks up the array's address on the device that is current (cudaGetSymbolAddress: no allocation, and the
 * address stays right after a device reset); the first call on a device also makes the runtime load the library's
 * image there, so make that first call outside any stream capture.  All calls share the one array: it keeps whatever the
 * previous call left, which is harmless because every partial sum a call reads it has written first (nothing needs
 * clearing), but two calls whose kernels overlap on the GPU (different streams, or different host threads) race on
 * it and must be ordered by the caller.  Results are bitwise those of shvk_cnn_se_gate. */
#define SHVK_CNN_SE_STATIC_FLOATS (1 << 18)
int shvk_cnn_se_gate_static(const float* x, const float* w1, const float* b1, const float* w2, const float* b2, float* gate,
                            int F, int HW, int C, int CS, void* stream);

/* 1x1 convolution as a row GEMM: out[m][n] = act(sum_k (A[m][k] * gate[m / gate_rows][k]) * W[n][k] + b[n]) (+ R[m][n]).
 * A [M][K] (pitch K), W [N][K], out and R [M][N] (R may alias out); gate NULL = no squeeze-excite scaling, else
 * [M / gate_rows][K]; K a multiple of 8, N a multiple of 4.  Each output is one fma chain over k in order.
 * Replaces gemm<T> as used by the frame encoder (engine/cuda/engine.cu:351-355,378-382,398-400;
 * engine/cuda/gemm.cuh:16-29). */
int shvk_cnn_pointwise(const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R,
                       float* out, int M, int N, int K, int act, void* stream);

/* The same 1x1 convolution on the tensor cores with float32 range: A (after the gate) and W are rounded to TF32
 * (10-bit mantissa, float32 range), products accumulate in float32; inputs and outputs stay float32.  k is walked in
 * order in slabs of 16, never split.  The reference's 16-bit modes run these layers as 16-bit tensor-core GEMMs
 * (gemm_mma, engine/cuda/gemm.cuh:266-289). */
int shvk_cnn_pointwise_tf32(const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R,
                            float* out, int M, int N, int K, int act, void* stream);

/* And with A (after the gate) and W rounded to a 16-bit type (ab_dtype: SHVK_BF16 = 1 or SHVK_F16 = 2 of
 * shv_seq_kernels.h), m16n8k16 tensor-core products, float32 accumulation; inputs and outputs stay float32.  k is
 * walked in order in slabs of 32, never split.  This is the arithmetic of the reference's 16-bit modes for these
 * layers (gemm_mma, engine/cuda/gemm.cuh:266-289), without its 16-bit activation storage. */
int shvk_cnn_pointwise_h(const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R,
                         float* out, int M, int N, int K, int act, int ab_dtype, void* stream);

/* Adaptive 4x4 average pooling of the [F][6][10][960] feature map: token r*4+c averages rows floor(6r/4) ..
 * ceil(6(r+1)/4)-1 and columns floor(10c/4) .. ceil(10(c+1)/4)-1.  out [F][16][960].
 * Replaces launch_pool (engine/cuda/cnn.cu:133-160,188-191). */
int shvk_cnn_pool_tokens(const float* in, float* out, int F, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* SHV_CNN_KERNELS_H */
