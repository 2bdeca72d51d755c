/*
 * shv_seq_kernels.h -- thin C launch layer over the sm_100a sequence kernels of the SHIELD-V engine.
 *
 * Host C++ (engine.cpp, api.cpp) reaches the GPU only through these functions; they are also exported from
 * libshield_v_cuda.so so that a kernel can be driven and checked in isolation.  Plain pointers and sizes only:
 * every pointer is a device pointer unless stated otherwise, `stream` is a cudaStream_t passed as void*, every
 * function only enqueues work and returns a cudaError_t value (0 = success).  Storage type codes: 0 = float32,
 * 1 = bfloat16, 2 = float16.
 *
 * Each entry replaces one launcher (or a fused group of launchers) of the reference engine; citations are to the
 * reference tree.
 */
#ifndef SHV_SEQ_KERNELS_H
#define SHV_SEQ_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

enum { SHVK_F32 = 0, SHVK_BF16 = 1, SHVK_F16 = 2 };
/* Output code of shvk_assemble_norm / shvk_rmsnorm only: the normalised row leaves as the exact tier's split A operand,
 * a row of 2 x 384 floats [lo | hi] (x = hi + lo, both TF32-representable; see shvk_split_tf32). */
enum { SHVK_F32_SPLIT = 3 };

/* h[b*321 + t] = tokens(b, t/16, t%16) + pos[t] (t < 320), readout (t == 320), and in the same pass
 * xn = rmsnorm(h) * norm_w in storage type xn_dtype.  tok_ptrs: [B*20] device pointers to 16x384 fp32 blocks.
 * Replaces launch_assemble + the first launch_rmsnorm (engine/cuda/seq.cu:27-69, engine.cu:409,416). */
int shvk_assemble_norm(const float* const* tok_ptrs, const float* pos, const float* readout, const float* norm_w,
                       float* h, void* xn, int xn_dtype, int B, void* stream);

/* out[r] = (x[r] * (1/sqrt(mean(x[r]^2) + 1e-6))) * w over rows of 384; x row pitch ldx, out row pitch ldo
 * (elements).  Replaces launch_rmsnorm<T> (engine/cuda/seq.cu:44-69,356-359). */
int shvk_rmsnorm(const float* x, long long ldx, const float* w, void* out, int out_dtype, long long ldo, int rows,
                 void* stream);

/* Token blocks (16 x 384) that arrived as fp16 in the upper half (bytes 12,288 ..) of their 24,576-byte fp32 staging
 * blocks, widened to fp32 in place; `stage` points at the first of `blocks` consecutive staging blocks. */
int shvk_expand_f16_tokens(float* stage, int blocks, void* stream);

/* C = epilogue(A * W^T): A [M,K] row-major (pitch lda), W [N,K] row-major (pitch ldw) = Linear weight layout.
 * Epilogue, in this order: + bias[n]; SiLU if act == 1; residual C = R + v / r_div (R fp32, may alias C);
 * swiglu: columns (2j, 2j+1) = (gate, up), writes silu(gate)*up at column j.  Never splits K.
 * Replaces GemmParams / gemm<T> (engine/cuda/gemm.cuh:16-29,435; gemm.cu:76-109). */
typedef struct shvk_gemm_args {
    int M, N, K;
    const void* A; long long lda;
    const void* W; long long ldw;
    void* C; long long ldc; int c_dtype;
    const float* bias;
    int act;
    const float* R; long long ldr; float r_div;
    int swiglu;
} shvk_gemm_args;
/* IEEE fp32 FMA chain on CUDA cores, k in order (exact tier and the fp32-only last-row projections). A, W fp32. */
int shvk_gemm_f32(const shvk_gemm_args* g, void* stream);
/* tcgen05 tensor-core GEMM, A and W in ab_dtype (bf16 or fp16), fp32 accumulation in tensor memory, operands
 * staged by TMA.  Needs K % 64 == 0, 16-byte aligned operands and pitches.  shvk_gemm_tc_plan encodes the two TMA
 * tensor maps and the tile shape for exactly these operands into a host-side plan that launches reuse.  Plain fp32
 * output with ldc - N < 8: the padding columns N .. ldc-1 may be written with zeros (whole 32-byte sectors per row).
 * Exact tier (ab_dtype = SHVK_F32; replaces the SIMT class of engine/cuda/gemm.cuh:66-188 for the all-row GEMMs): fp32
 * operands split into two TF32 pieces each by shvk_split_tf32, A = [lo | hi] (lda >= 2K), W = [hi | lo | hi]
 * (ldw >= 3K), K % 32 == 0; one accumulator sums lo*hi, hi*lo, hi*hi over k in that fixed order (K never split, rows
 * independent), what is dropped is below 2^-21 of each product.  SwiGLU then writes fp32 (c_dtype SHVK_F32). */
int shvk_gemm_tc_plan(const shvk_gemm_args* g, int ab_dtype, void* host_plan /* >= 512 bytes, host, 64-byte aligned */);
/* x = hi + lo, hi = x rounded to TF32, lo = x - hi rounded to TF32; rows of K fp32 (K % 4 == 0, 16-byte aligned).
 * layout 0: out row = [lo | hi] (A operand of the exact tier), layout 1: out row = [hi | lo | hi] (W operand). */
int shvk_split_tf32(const float* in, long long ld_in, int K, long long rows, float* out, long long ld_out, int layout, void* stream);
/* Plain epilogue with a 16-bit part: output columns [0, split_col) are rounded to fp16 (saturating) into C16 (pitch
 * ldc16 halves), columns [split_col, N) go to g->C as fp32 (+ bias[n]) at column n - split_col.  split_col % 32 == 0,
 * 16-bit operands only, no residual / SwiGLU.  The SISA all-row projection of the 16-bit modes uses it with
 * split_col = 960: K | V | B leave in 16 bits, theta | alpha | forget in fp32 (the reference keeps the whole row in fp32,
 * engine/cuda/engine.cu:446-450). */
int shvk_gemm_tc_plan_split16(const shvk_gemm_args* g, int ab_dtype, int split_col, void* C16, long long ldc16, void* host_plan);
int shvk_gemm_tc(const void* host_plan, void* stream);
/* Same plan, first `rows` <= M rows only (a smaller batch in buffers sized for the planned M). */
int shvk_gemm_tc_rows(const void* host_plan, int rows, void* stream);
/* Device status word of the tensor-core path: nonzero after a bounded wait inside a kernel gave up. */
int shvk_gemm_tc_status(int* status_out);
/* Test launch of the same plan: the producer of every CTA withholds the first operand stage of its first tile, so the
 * MMA role's bounded wait runs out after `polls` polls (clamped to 256 .. 2^22).  The CTA then takes its abort path
 * (status word set, every role leaves its loop, tensor memory freed) and returns; C is left partly written.  Nothing
 * faults or spins without bound.  Exists so that a test can watch the abort path work. */
int shvk_gemm_tc_rows_starved(const void* host_plan, int rows, int polls, void* stream);

/* SwiGLU feed-forward block of the 16-bit modes in one launch: h += down(silu(gate(xn)) * up(xn)) with the hidden
 * layer kept on the SM (shared memory -> tensor core), instead of an up launch writing [rows][960] and a down launch
 * reading it back.  xn [max_rows][384] and the weights in ab_dtype (bf16 or fp16): w_up [1920][384] with (gate, up) rows
 * interleaved (engine/cuda/model.cpp:95-102), w_down [384][960]; h [max_rows][384] fp32, updated in place.  Same
 * arithmetic as the two shvk_gemm_tc launches it replaces (k in order, hidden layer rounded to ab_dtype), rows
 * independent.  The plan (512 bytes, host, 64-byte aligned) holds the TMA tensor maps for exactly these buffers.
 * Replaces the two FFN gemm<T> launches of the reference (engine/cuda/engine.cu:434-440). */
int shvk_ffn_fused_plan(const void* xn, long long max_rows, const void* w_up, const void* w_down, float* h, int ab_dtype,
                        void* host_plan);
int shvk_ffn_fused(const void* host_plan, int rows, void* stream);
int shvk_ffn_fused_starved(const void* host_plan, int rows, int polls, void* stream);   /* test launch, as shvk_gdn_inproj_starved */

/* The kernels' status words (tensor-core GEMMs, the scan that reads the fp32 projection, the 16-bit scan) are per
 * device and per process.  These two calls enqueue on `stream`: a copy of the SHVK_STATUS_WORDS words into host_words (pinned host memory, read it after
 * the stream has passed this point), and their reset to zero.  A scheduler fetches the words behind a batch's last
 * kernel, fails the batch if one is set, and clears them so that later batches run normally. */
enum { SHVK_STATUS_WORDS = 3 };
int shvk_status_fetch_async(int* host_words, void* stream);
int shvk_status_clear_async(void* stream);

/* GDN in-projection of the 16-bit modes, fused with the steps between projection and recurrence (causal conv k = 4 +
 * bias + SiLU on q, k, v; SiLU on the output gate; log decay and beta).  Computes W' xn^T on the tensor cores with the
 * channels on the MMA rows and writes bf16 operand tiles in chunk blocks of 16 tokens ("PT": per clip, head and chunk
 * q^T [64][16], k^T [64][16], v^T [128][16], gate^T [128][16], log decay [16], beta [16], and room for what
 * shvk_gdn_chunk_prep adds; shvk_gdn_pt_bytes(B) bytes for B clips), which shvk_gdn_scan_t consumes.  xn: [max_rows][384] in ab_dtype (bf16 or fp16), rows of clip c at
 * 321 c; w_perm: [shvk_gdn_inproj_rows()][384] in ab_dtype = the rows of the reference's fused in-projection weight
 * [q | k | v | gate | a | b] (engine/cuda/model.cpp:109-115) in the order shvk_gdn_inproj_row_order gives (source row
 * per row of w_perm, -1 = a zero row); conv_w [1536][4], conv_b [1536], a_log [6], dt_bias [6] fp32 as in the
 * reference.  The plan (512 bytes, host, 64-byte aligned) holds the TMA tensor maps for exactly these buffers.
 * Replaces the in-projection gemm<T> (engine/cuda/engine.cu:418) + launch_gdn_prep (engine/cuda/seq.cu:72-104). */
int shvk_gdn_inproj_rows(void);
void shvk_gdn_inproj_row_order(int32_t* src_row /* [shvk_gdn_inproj_rows()] */);
size_t shvk_gdn_pt_bytes(int B);
int shvk_gdn_inproj_plan(const void* xn, long long max_rows, const void* w_perm, const float* conv_w, const float* conv_b,
                         const float* a_log, const float* dt_bias, void* pt_out, int ab_dtype, void* host_plan);
int shvk_gdn_inproj(const void* host_plan, int B, void* stream);
/* Test launches of the two kernels above's kind (see shvk_gemm_tc_rows_starved): the producer withholds its first weight
 * tile, the MMA role's bounded wait runs out after `polls` polls, the CTAs take their abort path and return with the
 * status word of the tensor-core GEMMs set.  Outputs are left partly written.  Nothing faults or spins without bound. */
int shvk_gdn_inproj_starved(const void* host_plan, int B, int polls, void* stream);
/* Completes the chunk blocks of B clips in place with what the delta rule needs per chunk and that does not depend on
 * the recurrent state: the decay-masked Gram products, the key and query norms and the 16 x 16 triangular inverse of
 * the WY form (written to the last 1,280 bytes of every block; one warp per block, all blocks at once).  op_dtype: the
 * type of the q^T / k^T tiles (bf16 or fp16).  Must run between shvk_gdn_inproj and shvk_gdn_scan_t. */
int shvk_gdn_chunk_prep(void* pt, int op_dtype, int B, void* stream);
/* Gated delta rule + gated RMSNorm of one mixer over B clips from the completed PT tiles: 16-token chunks in WY form on
 * the tensor cores, the head's 64 x 128 state in accumulator fragments for the whole sequence.  on: [B*321][768] in
 * on_dtype (bf16 or fp16).  Replaces launch_delta + launch_gated_norm (engine/cuda/seq.cu:107-214,364-371). */
int shvk_gdn_scan_t(const void* pt, const float* o_norm_w, void* on, int on_dtype, int B, void* stream);
/* Test launch of the same kernel: no CTA ever issues the copy of its first chunk, so the wait for it runs out after
 * `polls` polls, the status word is set and every CTA returns without writing. */
int shvk_gdn_scan_t_starved(const void* pt, const float* o_norm_w, void* on, int on_dtype, int B, int polls, void* stream);

/* Fused GatedDeltaNet core of one mixer over B clips from the fp32 projection (the exact tier's path; the 16-bit
 * modes use shvk_gdn_inproj + shvk_gdn_scan_t): causal short conv (k=4, bias) + SiLU on q|k|v, L2 norm of q
 * (then * 0.125) and k, decay = exp(-exp(A_log) * softplus(a + dt_bias)), beta = sigmoid(b), the gated delta rule
 * from a zero state with the head's 64x128 state held in registers (operands staged by TMA), and the gated RMSNorm
 * ((o * rstd) * w) * silu(gate).  P: [B*321][2320] fp32 fused projection output; on: [B*321][768] storage type.
 * Replaces launch_gdn_prep + launch_delta + launch_gated_norm (engine/cuda/seq.cu:72-214,360-371). */
int shvk_gdn_scan(const float* P, const float* conv_w, const float* conv_b, const float* a_log, const float* dt_bias,
                  const float* o_norm_w, void* on, int on_dtype, int B, void* stream);
/* Device status word of the scan kernel: nonzero after a bounded wait on a TMA barrier gave up. */
int shvk_gdn_scan_status(int* status_out);

/* Long-sequence gated delta rule in chunked (WY / UT-transform) form on the tensor cores: the recurrence of
 * oracle/shieldv_ref.py:121-139 (gated_delta_rule_recurrent) for any T, zero initial state.  q, k: [B,T,H,DK] bf16,
 * already L2-normalised; v: [B,T,H,128] bf16; g (log decay) and beta: [B,T,H] fp32; o: [B,T,H,128] in o_dtype (fp32 or
 * bf16); DK 64 or 128; q is multiplied by `scale`.  Two launches: a chunk-parallel kernel that prepares, for every
 * block of 16 tokens, everything that does not depend on the state (Gram products, decay masks, the triangular
 * inverse), and a sequential kernel per (batch, head) that carries the state.  `workspace` (device memory, 16-byte
 * aligned, at least shvk_gdn_chunked_workspace_bytes(B, T, H) bytes, contents irrelevant before and after) holds what
 * the first kernel hands to the second: 1,152 bytes per block.  The reference has no long-T implementation (its
 * sequence length is the compile-time constant 321, engine/cuda/model.hpp:10); this is the stress configuration T = 2048. */
size_t shvk_gdn_chunked_workspace_bytes(int B, int T, int H);
int shvk_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const float* beta, void* o, int o_dtype,
                     int B, int T, int H, int DK, int DV, float scale, void* workspace, size_t workspace_bytes, void* stream);

/* SISA attention of the readout row per (clip, head): -softplus(alpha), logsigmoid(forget), theta prefix sums in
 * double rounded to fp32, pair rotation of B (all rows) and C (row 320), scores, softmax over 321 keys, y = P V.
 * S: [B*321][1072] fp32; QC: [B][576] fp32; Y: [B][384] fp32.
 * Replaces launch_sisa_attn (engine/cuda/seq.cu:217-306,372-374). */
int shvk_sisa_attn(const float* S, const float* QC, const float* lambda_raw, float* Y, int B, void* stream);
/* The same over the split row format of the 16-bit modes: S16 [B*321][960] fp16 = K | V | B, SG [B*321][112] fp32 =
 * theta 96 | alpha 6 | forget 6 | pad (2,368 instead of 4,288 bytes per token; written by a shvk_gemm_tc_plan_split16
 * launch with split_col 960).  Arithmetic as above on the widened values. */
int shvk_sisa_attn_h16(const void* S16, const float* SG, const float* QC, const float* lambda_raw, float* Y, int B, void* stream);

/* Readout row (token 320) of the SISA block, fp32 in every mode, part 1: xl = rmsnorm(h_last) * norm_w, then
 * QC = xl * W_qc^T.  h_last: row 320 of clip c at h_last + c * ldh (elements); wqc_t: [384][576] = [W_Q | W_C]
 * transposed; QC: [B][576].  Replaces launch_rmsnorm + gemm<float> (engine/cuda/engine.cu:451-452). */
int shvk_readout_qc(const float* h_last, long long ldh, const float* norm_w, const float* wqc_t, float* QC, int B, void* stream);
/* Part 2, after the attention: x1 = h_last + Y * W_O^T; x2 = x1 + down(silu(gate(n)) * up(n)) with n = rmsnorm(x1);
 * logit = head(rmsnorm(x2)).  All matrices transposed to [K][N] (fp32); up_t holds the (gate, up) output pairs of the
 * SwiGLU FFN in adjacent columns (2j, 2j + 1).  Y: [B][384]; x2_out: [B][384] or NULL; logits: [B].
 * Replaces three gemm<float>, one launch_rmsnorm and launch_head (engine/cuda/engine.cu:455-469, seq.cu:309-336). */
typedef struct shvk_readout_weights {
    const float* wo_t;          /* [384][384]  */
    const float* ffn_norm_w;    /* [384]       */
    const float* up_t;          /* [384][1920] */
    const float* down_t;        /* [960][384]  */
    const float* final_norm_w;  /* [384]       */
    const float* head_w0_t;     /* [384][128]  */
    const float* head_b0;       /* [128]       */
    const float* head_w2;       /* [128]       */
    const float* head_b2;       /* [1]         */
} shvk_readout_weights;
int shvk_readout_tail(const float* Y, const float* h_last, long long ldh, const shvk_readout_weights* w, float* x2_out,
                      float* logits, int B, void* stream);

/* pool[slots[f]] = tokens[f] (6144 floats) for slots[f] >= 0.  Replaces launch_store_tokens (seq.cu:338-351). */
int shvk_store_tokens(const float* tokens, const int32_t* slots, float* pool, int F, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* SHV_SEQ_KERNELS_H */
