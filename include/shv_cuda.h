/*
 * shv_cuda.h -- C ABI of libshield_v_cuda.so, the GPU engine of the SHIELD-V video detector, as exported by the
 * B200 (sm_100a) sequence engine.
 *
 * Binary-compatible with the reference library's header (engine/include/shv_cuda.h:61-159): same opaque handles,
 * struct layouts, constants, entry points and calling conventions, so a caller built against the reference header
 * (the AV service, gpu_bench, gpu_cli) links against this library unchanged.  Each declaration cites the reference
 * line it replaces.
 *
 * What this library computes: the frame encoder -- 320x180 RGB crop -> MobileNetV3-Large features -> 4x4 pooling ->
 * 16 tokens x 384 (float32 in every mode) -- and the sequence stages of SHIELD-V -- 20 frames x 16 tokens x 384
 * (frame embeddings before position embeddings) + readout token -> GDN-A -> GDN-B x2 -> SISA (readout row) ->
 * RMSNorm -> head -> one logit per window.  score = sigmoid(logit) in double on the caller's side; alert iff
 * score >= threshold.  A NaN logit means "unavailable" (failed job or non-finite result), never a score.
 * Windows take their 16x384 blocks from frames of the same request, from device token slots, or from host pointers.
 *
 * MODES  "fp32": IEEE fp32 everywhere (exact tier, always loadable).  "bf16" / "fp16": 16-bit operands for the
 * all-row projections on the tensor cores, fp32 accumulation; norms, the delta-rule recurrence, the residual stream
 * and every readout-row computation stay fp32, SISA prefix sums are double.  The strict library loads a 16-bit mode
 * only with a passing certificate line for these weights, this compute revision and this threshold in
 * "<weights>.cuda.cert"; libshield_v_cuda_experimental.so skips that check (benchmarks, offline certification).
 * SIDECAR "<weights>.json" (every mode): "output_sha256" must equal the weight file's SHA-256 and "threshold" must
 * be in (0, 1).
 *
 * ROW INDEPENDENCE  A window's logit is bitwise identical whatever else is in the batch: no split-K, one
 * accumulation order per output, per-row reductions in a fixed order, no atomics.
 *
 * THREADS AND LIFETIMES  Every function may be called concurrently on one model except shv_cuda_free.  Jobs run in
 * submission order; consecutive queued jobs are coalesced into one GPU batch up to the limits.  Buffers a request
 * points to (token blocks, logits_out) stay owned by the caller but must remain valid and untouched until the job
 * completes; the index arrays are copied at submit.  Each job is released exactly once with shv_cuda_job_free, which
 * waits for completion and for the callback to return.  Callbacks run on the worker thread; they may submit and
 * query jobs but must not call the synchronous functions, free their own job, or free the model.
 * Error strings are thread-local.  int functions return 0 on success, -1 on error.
 */
#ifndef SHV_CUDA_H
#define SHV_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define SHV_CUDA_API_VERSION 1          /* shv_cuda.h:74 */
#define SHV_CUDA_FRAME_BYTES 172800     /* shv_cuda.h:75: 180 x 320 x 3 uint8 RGB */
#define SHV_CUDA_TOKEN_FLOATS 6144      /* shv_cuda.h:76: 16 tokens x 384, one frame */
#define SHV_CUDA_WINDOW_FRAMES 20       /* shv_cuda.h:77 */

typedef struct shv_cuda_model shv_cuda_model;   /* shv_cuda.h:79 */
typedef struct shv_cuda_job shv_cuda_job;       /* shv_cuda.h:80 */

/* shv_cuda.h:82-89.  Ranges: max_frames, max_windows in [1, 4096]; max_host_tokens in [0, 2^20]. */
typedef struct shv_cuda_options {
    int max_frames;       /* frames per GPU batch; default 640 */
    int max_windows;      /* windows per GPU batch; default 512 */
    int max_host_tokens;  /* host-provided token blocks per GPU batch; default 2048 */
    int token_slots;      /* device token slots (0 = none); default 0 */
    int use_graphs;       /* CUDA graph per batch size class; default 1 */
    int max_delay_us;     /* wait up to this long for more jobs before launching; default 0 */
} shv_cuda_options;

void shv_cuda_default_options(shv_cuda_options* opt);                                     /* shv_cuda.h:91 */
shv_cuda_model* shv_cuda_load(const char* weights, const char* mode, int device);         /* shv_cuda.h:94 */
shv_cuda_model* shv_cuda_load_ex(const char* weights, const char* mode, int device,
                                 const shv_cuda_options* opt);                            /* shv_cuda.h:95 */
void shv_cuda_free(shv_cuda_model* m);                                                    /* shv_cuda.h:96 */

const char* shv_cuda_last_error(void);                                                    /* shv_cuda.h:98 */
const char* shv_cuda_mode(const shv_cuda_model* m);                                       /* shv_cuda.h:99 */
const char* shv_cuda_fingerprint(const shv_cuda_model* m);  /* SHA-256 hex of the weights    shv_cuda.h:100 */
double shv_cuda_threshold(const shv_cuda_model* m);                                       /* shv_cuda.h:101 */
const char* shv_cuda_compute_revision(void);                /* hash of the engine sources    shv_cuda.h:102 */
int shv_cuda_limits(const shv_cuda_model* m, int* max_frames, int* max_windows, int* max_host_tokens,
                    int* token_slots);                                                    /* shv_cuda.h:103 */
size_t shv_cuda_weight_bytes(const shv_cuda_model* m);                                    /* shv_cuda.h:104 */
size_t shv_cuda_device_bytes(const shv_cuda_model* m);                                    /* shv_cuda.h:105 */

/* Synchronous calls, split into GPU batches internally (shv_cuda.h:107-113).
 * rgb: n crops [180][320][3] uint8; tokens: n x 16 x 384 (encode_frames) or b x 20 x 16 x 384 (classify) fp32;
 * clips: b x 20 crops; logits: b fp32.  NaN outputs and -1 on failure. */
int shv_cuda_encode_frames(shv_cuda_model* m, const uint8_t* rgb, size_t n, float* tokens);
int shv_cuda_classify(shv_cuda_model* m, const float* tokens, size_t b, float* logits);
int shv_cuda_predict(shv_cuda_model* m, const uint8_t* clips, size_t b, float* logits);

typedef void (*shv_cuda_callback)(shv_cuda_job* job, int status /* 1 done, -1 failed */, void* user); /* :116 */

/* shv_cuda.h:118-135.  Window entry e = window*20 + frame position takes its 16x384 block from
 * window_frames[e] >= 0 (frame of this request), else window_slots[e] >= 0 (device token slot), else
 * window_tokens[e] (host pointer to 6144 fp32). */
typedef struct shv_cuda_request {
    const uint8_t* frames;
    size_t n_frames;
    float* tokens_out;
    const int32_t* store_slots;
    size_t n_windows;
    const int32_t* window_frames;
    const int32_t* window_slots;
    const float* const* window_tokens;
    float* logits_out;
    shv_cuda_callback callback;
    void* user;
} shv_cuda_request;

shv_cuda_job* shv_cuda_submit(shv_cuda_model* m, const shv_cuda_request* req);            /* shv_cuda.h:139 */
int shv_cuda_job_status(const shv_cuda_job* job);   /* 0 pending, 1 done, -1 failed          shv_cuda.h:140 */
int shv_cuda_job_wait(shv_cuda_job* job);           /* blocks; 0 done, -1 failed             shv_cuda.h:141 */
const char* shv_cuda_job_error(const shv_cuda_job* job);                                  /* shv_cuda.h:142 */
int shv_cuda_job_timing(const shv_cuda_job* job, double* queue_ms, double* run_ms, double* gpu_ms,
                        int* batch_frames, int* batch_windows);                           /* shv_cuda.h:145 */
void shv_cuda_job_free(shv_cuda_job* job);                                                /* shv_cuda.h:147 */

/* Pinned host memory (shv_cuda.h:150-151).  Token blocks and outputs that live in pinned memory are copied by DMA
 * straight from / to the caller's buffer, without the staging memcpy. */
void* shv_cuda_host_alloc(size_t bytes);
void shv_cuda_host_free(void* p);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* SHV_CUDA_H */
