/*
 * shv_cuda_b200.h -- entry points of libshield_v_cuda.so that the reference library does not have.
 *
 * The reference engine fills its device token slots only from frames it encodes itself (store_slots of a request,
 * engine/include/shv_cuda.h:122,54-59).  A caller that encodes frames elsewhere and keeps per-participant token
 * rings on the device needs another way in: shv_cuda_b200_upload_tokens.
 */
#ifndef SHV_CUDA_B200_H
#define SHV_CUDA_B200_H

#include "shv_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Copies n host token blocks (n x 6144 fp32, frame embeddings before positions) into device token slots
 * slots[0..n) (each in [0, token_slots), no duplicates within max_host_tokens consecutive entries).  Goes through the
 * job queue, so it is ordered against windows exactly like a store_slots request of the reference: windows submitted
 * earlier see the old contents, windows submitted later the new ones.  Blocks; 0 on success, -1 on error. */
int shv_cuda_b200_upload_tokens(shv_cuda_model* m, const float* tokens, size_t n, const int32_t* slots);

/* shv_cuda_classify (engine/include/shv_cuda.h:141) with the tokens handed over as IEEE fp16 instead of fp32:
 * tokens_f16 is [b][20][16][384] halves (12,288 bytes per frame block, 16-byte aligned), half the bytes to bring to the
 * device.  No counterpart in the reference, whose ABI fixes fp32 tokens; meant for callers whose frame embeddings are
 * already 16-bit and whose GPUs share one host's upload bandwidth.  The blocks are widened to fp32 on the device before
 * anything reads them, so the logits are those of shv_cuda_classify on the same values as fp32, in every mode (and
 * differ from those of the unrounded embeddings by what fp16 rounding of the inputs costs).  Blocks; 0 or -1. */
int shv_cuda_b200_classify_f16(shv_cuda_model* m, const uint16_t* tokens_f16, size_t b, float* logits);

/* Number of kernels one GPU batch launches (for launch accounting in benchmarks). */
int shv_cuda_b200_launches_per_batch(const shv_cuda_model* m);

/* Test hook, experimental library only (-1 in the certificate-checked library): the next `batches` GPU batches of a
 * 16-bit model run with one launch starved of its input (kind 1: a tensor-core GEMM, 2: the scan), so that the kernel's
 * bounded wait runs out, its status word is set and it returns.  Those batches fail (NaN logits) like any batch whose
 * kernels gave up; the scheduler then clears the status words and later batches run normally.  Nothing faults or
 * hangs: the wait is a poll loop with a limit, the kernel's ordinary abort path is what the test exercises. */
int shv_cuda_b200_test_starve(shv_cuda_model* m, int kind, int batches);

/* ---------------------------------------------------------------- several GPUs of one box behind one object
 * The reference's service engine owns one GPU model and gives every session a block of 24 device token slots out of
 * that model's pool (service/src/shield_av.cpp:824-850 load, :1013-1020 slot blocks, :556-577 submit;
 * service/include/shield_av.h:205-211).  shv_box is that for N GPUs in one process: one model per device (loaded side
 * by side; `opt` applies to each, its token_slots is replaced by the box's own sizing), sessions placed by
 * crc32(participant id) mod N -- spilling to the device with the most free blocks when the home device is full -- and
 * batches of independent clips cut into contiguous per-device shards.  Nothing crosses between devices.
 * max_sessions sizes the slot pools: each device can hold its even share of the sessions plus a quarter. */
typedef struct shv_box shv_box;
shv_box* shv_box_load(const char* weights, const char* mode, const int* devices, int n_devices, const shv_cuda_options* opt,
                      int max_sessions);
void shv_box_free(shv_box* box);                                     /* drains every device's queue first */
int shv_box_devices(const shv_box* box);
shv_cuda_model* shv_box_model(shv_box* box, int device_index);       /* the device's model, for queries and direct use */
int shv_box_home_device(const shv_box* box, const char* participant_id);   /* crc32(id) mod N, before any spill */
/* Places a session and takes a block of 24 token slots on its device: slots slot_base .. slot_base + 23 of
 * shv_box_model(box, *device_index).  -1 with "max_sessions reached" when every device is full. */
int shv_box_session_open(shv_box* box, const char* participant_id, int* device_index, int* slot_base);
int shv_box_session_close(shv_box* box, int device_index, int slot_base);
int shv_box_free_sessions(shv_box* box, int device_index);           /* free session blocks on that device */
/* shv_cuda_submit on the session's device. */
shv_cuda_job* shv_box_submit(shv_box* box, int device_index, const shv_cuda_request* req);
/* shv_cuda_classify over all devices: clip i goes to device floor(i * N / b) (shard sizes differ by at most one), the
 * shards run concurrently, logits arrive in clip order.  Bitwise the single-device result (row independence). */
int shv_box_classify(shv_box* box, const float* tokens, size_t b, float* logits);
/* The same box over stand-in entry points (tests drive placement, slot accounting and sharding without a GPU). */
typedef struct shv_box_ops {
    shv_cuda_model* (*load_ex)(const char* weights, const char* mode, int device, const shv_cuda_options* opt);
    void (*free_model)(shv_cuda_model* m);
    shv_cuda_job* (*submit)(shv_cuda_model* m, const shv_cuda_request* req);
    int (*classify)(shv_cuda_model* m, const float* tokens, size_t b, float* logits);
    const char* (*last_error)(void);
} shv_box_ops;
shv_box* shv_box_load_with(const shv_box_ops* ops, const char* weights, const char* mode, const int* devices, int n_devices,
                           const shv_cuda_options* opt, int max_sessions);

/* ---------------------------------------------------------------- engine core for harnesses
 * The reference's internal C++ engine API (engine/cuda/engine.hpp:20-62: make_engine, Engine::slot, Engine::classify,
 * set_dump_dir), which its kernel benchmark and dump tools compile against (bench/gpu_kbench.cu:55-103,
 * bench/gpu_dump.cu:16-36), as plain C so that a harness in any language can time classify on tokens that already
 * live in device memory, on a stream it owns.  No worker thread, no staging; NOT thread-safe (one driver thread).
 * max_windows may exceed the 4096 cap of the job API.  Every int function returns 0 or -1 (+ shv_cuda_last_error). */
typedef struct shvb_engine shvb_engine;
shvb_engine* shvb_engine_create(const char* weights, const char* mode, int device, int max_windows, int use_graphs);
/* The same with a frame budget: slots hold up to max_frames RGB crops and their tokens (shvb_engine_create gives 1). */
shvb_engine* shvb_engine_create_ex(const char* weights, const char* mode, int device, int max_frames, int max_windows,
                                   int use_graphs);
void shvb_engine_destroy(shvb_engine* e);
/* Frame encoder (Engine::encode, engine/cuda/engine.hpp:46): reads F uint8 RGB crops [F][180][320][3] from
 * shvb_engine_frames(e, slot) and writes their tokens [F][16][384] fp32 to shvb_engine_tokens(e, slot), on `stream`. */
uint8_t* shvb_engine_frames(shvb_engine* e, int slot);               /* device pointer, [max_frames][172800] */
float* shvb_engine_tokens(shvb_engine* e, int slot);                 /* device pointer, [max_frames][6144] */
int shvb_engine_encode(shvb_engine* e, int slot, int F, void* stream);
int shvb_engine_frame_bucket(const shvb_engine* e, int F);           /* size class a batch of F frames is padded to */
int shvb_engine_encode_launches(const shvb_engine* e);               /* kernels per encode */
/* shvb_engine_profile for one eager encode of F frames. */
int shvb_engine_profile_encode(shvb_engine* e, int slot, int F, void* stream, float* ms, int cap, char* names, int names_cap);
/* Points window w, frame f of `slot` (0 or 1) at d_tokens + (w*20 + f)*6144: B windows of device-resident tokens
 * [B][20][16][384] fp32; the entries of the padding windows up to B's size class point at engine-owned tokens, so a
 * buffer bound earlier may be freed.  The table upload is enqueued on `stream`. */
int shvb_engine_bind_tokens(shvb_engine* e, int slot, const float* d_tokens, int B, void* stream);
/* Enqueues the whole sequence stack for B windows on `stream`; logits land in shvb_engine_logits(e, slot)[0..B). */
int shvb_engine_classify(shvb_engine* e, int slot, int B, void* stream);
float* shvb_engine_logits(shvb_engine* e, int slot);                 /* device pointer, [max_windows] */
/* Waits for `stream`, then copies the first n logits of `slot` to host memory. */
int shvb_engine_read_logits(shvb_engine* e, int slot, float* host, int n, void* stream);
int shvb_engine_window_bucket(const shvb_engine* e, int B);          /* size class a batch of B is padded to */
int shvb_engine_launches(const shvb_engine* e);                      /* kernels per classify */
int shvb_engine_status(const shvb_engine* e);                        /* nonzero: a kernel's bounded wait gave up */
/* Test hook, as shv_cuda_b200_test_starve: the next `batches` classify calls starve one launch (16-bit modes). */
int shvb_engine_test_starve(shvb_engine* e, int kind, int batches);
size_t shvb_engine_bytes(const shvb_engine* e, int which);           /* 0 weights, 1 activations, 2 one slot */
/* One eager classify of B windows with a CUDA event after every launch.  Writes up to `cap` per-launch times
 * (milliseconds, launch order) to ms and the kernel names, separated by ';', to names (names_cap bytes).  Returns the
 * number of launches, or -1.  Synchronises the stream. */
int shvb_engine_profile(shvb_engine* e, int slot, int B, void* stream, float* ms, int cap, char* names, int names_cap);
/* Debug: classify writes raw float32 intermediates of window 0 (<name>.f32) into dir; "" turns it off. */
int shvb_engine_set_dump_dir(shvb_engine* e, const char* dir);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* SHV_CUDA_B200_H */
