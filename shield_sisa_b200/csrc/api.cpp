// C ABI of libshield_v_cuda.so over the sequence engine: asynchronous jobs, FIFO batch coalescing, two-slot
// pipelining, pinned staging, NaN-on-failure.  Contract: include/shv_cuda.h; behaviour follows the reference's
// scheduler (engine/cuda/api.cu:131-383,466-729) entry point by entry point:
//   * jobs run in submission order; the worker coalesces queued jobs while the batch limits hold and no job stores
//     into a token slot that an earlier job of the batch reads or stores (api.cu:208-232)
//   * while batch n computes on the compute stream, batch n+1 is staged and copied on the copy stream into the
//     other buffer set (api.cu:346-383)
//   * a failed batch fails all its jobs, whose logits become NaN; a non-finite logit is reported as NaN
//     (api.cu:177-181,334-338)
//   * shv_cuda_job_free waits for completion and for the callback to return before deleting (api.cu:194-203,630-637)
// Beyond the reference: host token blocks that live in pinned memory are DMA'd straight from the caller's buffer as
// contiguous runs (the reference stages every block through a memcpy), staging buffers are allocated on first use,
// and shv_cuda_b200_upload_tokens fills device token slots from host tokens.
//   * frames of a request are encoded first, their tokens stored into the token slots the request names, then the
//     windows of the batch are classified (api.cu:233-318): a window sees the frames and stores of its own request and
//     of every earlier request
#include "shv_cuda.h"
#include "shv_cuda_b200.h"
#include "engine.hpp"
#include "shv_seq_kernels.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <limits>
#include <mutex>
#include <thread>
#include <unordered_set>

#ifndef SHV_CUDA_REVISION
#define SHV_CUDA_REVISION "unversioned"
#endif

namespace {
using Clock = std::chrono::steady_clock;
thread_local std::string t_error;
constexpr float kNaN = std::numeric_limits<float>::quiet_NaN();
constexpr size_t kBlockFloats = SHV_CUDA_TOKEN_FLOATS, kBlockBytes = kBlockFloats * 4, kFrameBytes = SHV_CUDA_FRAME_BYTES;

void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error ") + cudaGetErrorString(e) + " in " + what);
}

bool host_pinned(const void* p, size_t bytes) {
    if (!p || !bytes) return false;
    for (const void* q : {p, static_cast<const void*>(static_cast<const uint8_t*>(p) + bytes - 1)}) {
        cudaPointerAttributes a{};
        if (cudaPointerGetAttributes(&a, q) != cudaSuccess) { cudaGetLastError(); return false; }
        if (a.type != cudaMemoryTypeHost) return false;
    }
    return true;
}

// A maximal run of host token blocks that are contiguous in memory, in window-entry order.
struct HostRun {
    const float* src;
    int blocks;
    bool pinned;
};
}  // namespace

struct shv_cuda_job {
    // request
    size_t n_windows = 0;
    const uint8_t* frames = nullptr;        // request frames [n_frames][172800], borrowed until completion
    size_t n_frames = 0;
    float* tokens_out = nullptr;            // optional: tokens of the request's frames
    bool frames_pinned = false, tokens_out_pinned = false;
    std::vector<int32_t> frame_store;       // per frame: token slot its tokens are stored into, -1 = none (may be empty)
    std::vector<int32_t> wframes;           // per entry: frame of this request, -1 = none (may be empty)
    int frame_off = 0;                      // first frame of this job in its batch
    std::vector<int32_t> wslots;            // per entry, -1 = host block or frame
    std::vector<HostRun> runs;              // host blocks in entry order
    int host_blocks = 0;
    float* logits_out = nullptr;
    std::vector<int32_t> store_slots;       // upload job: slot per host block
    shv_cuda_callback cb = nullptr;
    void* user = nullptr;
    // placement in its batch
    int window_off = 0;
    // completion
    mutable std::mutex m;
    std::condition_variable cv;
    int state = 0;              // 0 pending, 1 done, -1 failed
    bool released = false;      // callback has returned
    std::string error;
    Clock::time_point t_submit, t_start, t_done;
    float gpu_ms = 0.0f;
    int batch_frames = 0, batch_windows = 0;
};

namespace {

struct HostSide {                            // pinned companions of one engine slot
    float* tok_stage = nullptr;              // [max_host_tokens][6144], allocated on first unpinned block
    const float** tokptr = nullptr;          // [max_windows*20]
    int32_t* store = nullptr;                // [max_host_tokens]
    int32_t* d_store = nullptr;              // device copy
    float* logits = nullptr;                 // [max_windows]
    uint8_t* frames = nullptr;               // [max_frames][172800], allocated on first unpinned frame
    float* tokens_out = nullptr;             // [max_frames][6144], allocated on first unpinned tokens_out
    int32_t* fstore = nullptr;               // [max_frames] token slot per encoded frame
    int32_t* d_fstore = nullptr;             // device copy
    int* status = nullptr;                   // [SHVK_STATUS_WORDS] the kernels' status words as of the end of the batch
    cudaEvent_t copied = nullptr, start = nullptr, end = nullptr;
};

struct Batch {
    int slot = 0;
    std::vector<shv_cuda_job*> jobs;
    int windows = 0, frames = 0;
    bool failed = false;
    std::string error;
};

class Scheduler {
public:
    std::unique_ptr<shv::Engine> engine;
    std::string mode, fingerprint;
    double threshold = 0.0;
    int device = 0;
    shv_cuda_options opt{};
    size_t device_bytes = 0;
    float* d_pool = nullptr;
    long fail_every = 0;                     // test hook: fail every n-th batch on the host before any GPU work

    ~Scheduler() {
        for (HostSide& h : host_) {
            if (h.tok_stage) cudaFreeHost(h.tok_stage);
            if (h.tokptr) cudaFreeHost(h.tokptr);
            if (h.store) cudaFreeHost(h.store);
            if (h.d_store) cudaFree(h.d_store);
            if (h.logits) cudaFreeHost(h.logits);
            if (h.frames) cudaFreeHost(h.frames);
            if (h.tokens_out) cudaFreeHost(h.tokens_out);
            if (h.fstore) cudaFreeHost(h.fstore);
            if (h.d_fstore) cudaFree(h.d_fstore);
            if (h.status) cudaFreeHost(h.status);
            for (cudaEvent_t e : {h.copied, h.start, h.end})
                if (e) cudaEventDestroy(e);
        }
        if (d_pool) cudaFree(d_pool);
        engine.reset();
        if (compute_) cudaStreamDestroy(compute_);
        if (copy_) cudaStreamDestroy(copy_);
    }

    void start(const shv::HostModel& hm) {
        cuda_ok(cudaSetDevice(device), "cudaSetDevice");
        cuda_ok(cudaStreamCreateWithFlags(&compute_, cudaStreamNonBlocking), "stream");
        cuda_ok(cudaStreamCreateWithFlags(&copy_, cudaStreamNonBlocking), "stream");
        shv::EngineConfig ec;
        ec.max_frames = opt.max_frames;
        ec.max_windows = opt.max_windows;
        ec.use_graphs = opt.use_graphs != 0;
        ec.slots = 2;
        shv::Precision p;
        if (!shv::parse_precision(mode, &p)) throw std::runtime_error("unknown mode: " + mode);
        engine = shv::make_engine(hm, p, ec);
        host_.resize(size_t(ec.slots));
        const size_t Bm = size_t(opt.max_windows), Hm = size_t(std::max(opt.max_host_tokens, 1));
        for (HostSide& h : host_) {
            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.tokptr), Bm * 20 * sizeof(float*), cudaHostAllocDefault), "pinned alloc");
            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.store), Hm * 4, cudaHostAllocDefault), "pinned alloc");
            cuda_ok(cudaMalloc(reinterpret_cast<void**>(&h.d_store), Hm * 4), "device alloc");
            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.logits), Bm * 4, cudaHostAllocDefault), "pinned alloc");
            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.fstore), size_t(opt.max_frames) * 4, cudaHostAllocDefault), "pinned alloc");
            cuda_ok(cudaMalloc(reinterpret_cast<void**>(&h.d_fstore), size_t(opt.max_frames) * 4), "device alloc");
            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.status), SHVK_STATUS_WORDS * sizeof(int), cudaHostAllocDefault), "pinned alloc");
            std::memset(h.status, 0, SHVK_STATUS_WORDS * sizeof(int));
            cuda_ok(cudaEventCreateWithFlags(&h.copied, cudaEventDisableTiming), "event");
            cuda_ok(cudaEventCreate(&h.start), "event");
            cuda_ok(cudaEventCreate(&h.end), "event");
        }
        if (opt.token_slots > 0) {
            cuda_ok(cudaMalloc(reinterpret_cast<void**>(&d_pool), size_t(opt.token_slots) * kBlockBytes), "token slots");
            cuda_ok(cudaMemset(d_pool, 0, size_t(opt.token_slots) * kBlockBytes), "token slots");
        }
        device_bytes = engine->weight_bytes() + engine->activation_bytes() +
                       size_t(ec.slots) * (engine->slot_bytes() + Hm * 4 + size_t(opt.max_frames) * 4) + size_t(std::max(opt.token_slots, 0)) * kBlockBytes;
#ifdef SHV_CUDA_EXPERIMENTAL
        // test hook of the experimental library only: the certificate-checked library reads no environment
        if (const char* e = std::getenv("SHV_CUDA_FAIL_EVERY")) fail_every = std::atol(e);
#endif
        cuda_ok(cudaDeviceSynchronize(), "init");
        worker_ = std::thread([this] { loop(); });
    }

    void stop() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stopping_ = true;
        }
        wake_.notify_all();
        if (worker_.joinable()) worker_.join();
    }

    // Test hook: the worker arms the engine before its next batch (the engine has one driver thread).
    void request_starve(int kind, int batches) {
        if (kind != 1 && kind != 2) throw std::runtime_error("starve kind: 1 = tensor-core GEMM, 2 = scan");
        if (mode == "fp32") throw std::runtime_error("the starved test launches exist for the 16-bit modes only");
        std::lock_guard<std::mutex> lk(mu_);
        starve_kind_ = kind;
        starve_batches_ = batches;
    }

    // Host token blocks one batch may carry: the option's limit, and what a slot's device staging area holds.
    int block_cap() const { return std::min(opt.max_host_tokens, opt.max_windows * 20); }

    // false if the model is stopping (the job is not queued)
    bool enqueue(shv_cuda_job* j) {
        {
            std::lock_guard<std::mutex> lk(mu_);
            if (stopping_) return false;
            queue_.push_back(j);
        }
        wake_.notify_all();
        return true;
    }

private:
    cudaStream_t compute_ = nullptr, copy_ = nullptr;
    std::vector<HostSide> host_;
    std::mutex mu_;
    std::condition_variable wake_;
    std::deque<shv_cuda_job*> queue_;
    bool stopping_ = false;
    int starve_kind_ = 0, starve_batches_ = 0;
    std::thread worker_;
    long batches_ = 0;

    static void finish_job(shv_cuda_job* j, bool ok, const std::string& err, float gpu_ms, int frames, int windows) {
        if (!ok) {
            for (size_t i = 0; i < j->n_windows; ++i) j->logits_out[i] = kNaN;
            if (j->tokens_out) std::fill(j->tokens_out, j->tokens_out + j->n_frames * kBlockFloats, kNaN);
        }
        shv_cuda_callback cb;
        void* user;
        {
            std::lock_guard<std::mutex> lk(j->m);
            j->state = ok ? 1 : -1;
            j->error = ok ? std::string() : err;
            j->t_done = Clock::now();
            j->gpu_ms = gpu_ms;
            j->batch_frames = frames;
            j->batch_windows = windows;
            cb = j->cb;
            user = j->user;
            j->cv.notify_all();              // under the lock: job_free may delete *j as soon as it sees `released`
        }
        if (cb) cb(j, ok ? 1 : -1, user);
        std::lock_guard<std::mutex> lk(j->m);
        j->released = true;
        j->cv.notify_all();
    }

    // Pops queued jobs in order while the limits hold and no store hazard appears.  Caller holds mu_.
    void coalesce(std::vector<shv_cuda_job*>& out) {
        int windows = 0, blocks = 0, frames = 0;
        std::unordered_set<int32_t> read, stored;
        while (!queue_.empty()) {
            shv_cuda_job* j = queue_.front();
            if (!out.empty()) {
                if (windows + int(j->n_windows) > opt.max_windows || blocks + j->host_blocks > block_cap() ||
                    frames + int(j->n_frames) > opt.max_frames)
                    break;
                bool hazard = false;
                for (const std::vector<int32_t>* v : {&j->store_slots, &j->frame_store})
                    for (int32_t s : *v)
                        if (s >= 0 && (read.count(s) || stored.count(s))) { hazard = true; break; }
                if (hazard) break;
            }
            queue_.pop_front();
            out.push_back(j);
            windows += int(j->n_windows);
            blocks += j->host_blocks;
            frames += int(j->n_frames);
            for (const std::vector<int32_t>* v : {&j->store_slots, &j->frame_store})
                for (int32_t s : *v)
                    if (s >= 0) stored.insert(s);
            for (int32_t s : j->wslots)
                if (s >= 0) read.insert(s);
        }
    }

    Batch launch(int slot, std::vector<shv_cuda_job*>& jobs) {
        Batch b;
        b.slot = slot;
        b.jobs = jobs;
        const Clock::time_point t0 = Clock::now();
        HostSide& h = host_[size_t(slot)];
        const shv::Engine::Slot& d = engine->slot(slot);
        try {
            ++batches_;
            if (fail_every > 0 && batches_ % fail_every == 0) throw std::runtime_error("injected batch failure (SHV_CUDA_FAIL_EVERY)");
            int windows = 0, blocks = 0, stores = 0, frames = 0;
            bool frame_stores = false;
            for (shv_cuda_job* j : jobs) {
                j->t_start = t0;
                j->window_off = windows;
                j->frame_off = frames;
                if (j->n_frames) {                              // crops: pinned sources by DMA, the rest staged
                    uint8_t* dst = d.d_frames + size_t(frames) * kFrameBytes;
                    const size_t bytes = j->n_frames * kFrameBytes;
                    if (j->frames_pinned) {
                        cuda_ok(cudaMemcpyAsync(dst, j->frames, bytes, cudaMemcpyHostToDevice, copy_), "frame upload");
                    } else {
                        if (!h.frames)
                            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.frames), size_t(opt.max_frames) * kFrameBytes,
                                                  cudaHostAllocDefault), "pinned staging");
                        uint8_t* st = h.frames + size_t(frames) * kFrameBytes;
                        std::memcpy(st, j->frames, bytes);
                        cuda_ok(cudaMemcpyAsync(dst, st, bytes, cudaMemcpyHostToDevice, copy_), "frame upload");
                    }
                    for (size_t f = 0; f < j->n_frames; ++f) {
                        const int32_t sl = j->frame_store.empty() ? -1 : j->frame_store[f];
                        h.fstore[size_t(frames) + f] = sl;
                        frame_stores |= sl >= 0;
                    }
                }
                size_t e = 0;                                   // next window entry that takes a host block
                const size_t entries = j->n_windows * 20;
                auto from_frame = [&](size_t k) { return !j->wframes.empty() && j->wframes[k] >= 0; };
                int stored_here = 0;
                for (const HostRun& run : j->runs) {
                    float* dst = d.d_tok_stage + size_t(blocks) * kBlockFloats;
                    const size_t bytes = size_t(run.blocks) * kBlockBytes;
                    if (run.pinned) {
                        cuda_ok(cudaMemcpyAsync(dst, run.src, bytes, cudaMemcpyHostToDevice, copy_), "token upload");
                    } else {
                        if (!h.tok_stage)
                            cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.tok_stage),
                                                  size_t(std::max(opt.max_host_tokens, 1)) * kBlockBytes, cudaHostAllocDefault),
                                    "pinned staging");
                        float* st = h.tok_stage + size_t(blocks) * kBlockFloats;
                        std::memcpy(st, run.src, bytes);
                        cuda_ok(cudaMemcpyAsync(dst, st, bytes, cudaMemcpyHostToDevice, copy_), "token upload");
                    }
                    for (int i = 0; i < run.blocks; ++i) {
                        const float* dev_block = dst + size_t(i) * kBlockFloats;
                        if (!j->store_slots.empty()) {
                            h.store[blocks + i] = j->store_slots[size_t(stored_here++)];
                            ++stores;
                        } else {
                            h.store[blocks + i] = -1;
                            while (e < entries && (j->wslots[e] >= 0 || from_frame(e))) ++e;
                            h.tokptr[size_t(windows) * 20 + e] = dev_block;
                            ++e;
                        }
                    }
                    blocks += run.blocks;
                }
                for (size_t k = 0; k < entries; ++k) {
                    if (from_frame(k))
                        h.tokptr[size_t(windows) * 20 + k] = d.d_tokens + size_t(frames + j->wframes[k]) * kBlockFloats;
                    else if (j->wslots[k] >= 0)
                        h.tokptr[size_t(windows) * 20 + k] = d_pool + size_t(j->wslots[k]) * kBlockFloats;
                }
                windows += int(j->n_windows);
                frames += int(j->n_frames);
            }
            if (frame_stores)
                cuda_ok(cudaMemcpyAsync(h.d_fstore, h.fstore, size_t(frames) * 4, cudaMemcpyHostToDevice, copy_), "slot list upload");
            if (windows)
                cuda_ok(cudaMemcpyAsync(d.d_tokptr, h.tokptr, size_t(windows) * 20 * sizeof(float*), cudaMemcpyHostToDevice, copy_),
                        "pointer table upload");
            if (stores)
                cuda_ok(cudaMemcpyAsync(h.d_store, h.store, size_t(blocks) * 4, cudaMemcpyHostToDevice, copy_), "slot list upload");
            cuda_ok(cudaEventRecord(h.copied, copy_), "event");
            cuda_ok(cudaStreamWaitEvent(compute_, h.copied, 0), "event");
            cuda_ok(cudaEventRecord(h.start, compute_), "event");
            if (frames) engine->encode(slot, frames, compute_);
            if (frame_stores) cuda_ok(cudaError_t(shvk_store_tokens(d.d_tokens, h.d_fstore, d_pool, frames, compute_)), "token slot store");
            if (stores) cuda_ok(cudaError_t(shvk_store_tokens(d.d_tok_stage, h.d_store, d_pool, blocks, compute_)), "token slot store");
            if (windows) {
                engine->classify(slot, windows, compute_);
                cuda_ok(cudaMemcpyAsync(h.logits, d.d_logits, size_t(windows) * 4, cudaMemcpyDeviceToHost, compute_), "logit download");
            }
            for (shv_cuda_job* j : jobs) {
                if (!j->tokens_out || !j->n_frames) continue;
                if (!j->tokens_out_pinned && !h.tokens_out)
                    cuda_ok(cudaHostAlloc(reinterpret_cast<void**>(&h.tokens_out), size_t(opt.max_frames) * kBlockBytes,
                                          cudaHostAllocDefault), "pinned staging");
                float* dst = j->tokens_out_pinned ? j->tokens_out : h.tokens_out + size_t(j->frame_off) * kBlockFloats;
                cuda_ok(cudaMemcpyAsync(dst, d.d_tokens + size_t(j->frame_off) * kBlockFloats, j->n_frames * kBlockBytes,
                                        cudaMemcpyDeviceToHost, compute_), "token download");
            }
            cuda_ok(cudaError_t(shvk_status_fetch_async(h.status, compute_)), "status fetch");
            cuda_ok(cudaEventRecord(h.end, compute_), "event");
            b.windows = windows;
            b.frames = frames;
        } catch (const std::exception& e) {
            b.failed = true;
            b.error = e.what();
        }
        return b;
    }

    void retire(Batch& b) {
        HostSide& h = host_[size_t(b.slot)];
        float gpu_ms = 0.0f;
        if (!b.failed) {
            const cudaError_t e = cudaEventSynchronize(h.end);
            if (e != cudaSuccess) {
                b.failed = true;
                b.error = std::string("CUDA error: ") + cudaGetErrorString(e);
            } else {
                if (cudaEventElapsedTime(&gpu_ms, h.start, h.end) != cudaSuccess) { cudaGetLastError(); gpu_ms = 0.0f; }
                bool gave_up = false;
                for (int i = 0; i < SHVK_STATUS_WORDS; ++i) gave_up |= h.status[i] != 0;
                if (gave_up) {
                    // The words are shared by everything on this device: clear them behind the work already queued, so
                    // that batches launched from now on are judged on their own.  A batch that was already in flight
                    // fetched the set words and fails too.
                    b.failed = true;
                    b.error = "a kernel gave up waiting on its TMA / tensor-core pipeline (device status word set)";
                    if (shvk_status_clear_async(compute_) != 0) cudaGetLastError();
                    cudaStreamSynchronize(compute_);
                }
            }
        } else {
            cudaStreamSynchronize(compute_);
            cudaStreamSynchronize(copy_);
        }
        for (shv_cuda_job* j : b.jobs) {
            if (!b.failed) {
                for (size_t i = 0; i < j->n_windows; ++i) {
                    const float v = h.logits[size_t(j->window_off) + i];
                    j->logits_out[i] = std::isfinite(v) ? v : kNaN;
                }
                if (j->tokens_out && !j->tokens_out_pinned && j->n_frames)
                    std::memcpy(j->tokens_out, h.tokens_out + size_t(j->frame_off) * kBlockFloats, j->n_frames * kBlockBytes);
            }
            finish_job(j, !b.failed, b.error, gpu_ms, b.frames, b.windows);
        }
    }

    void loop() {
        if (cudaSetDevice(device) != cudaSuccess) cudaGetLastError();
        std::deque<Batch> inflight;
        const int nslots = int(host_.size());
        int next_slot = 0;
        for (;;) {
            std::vector<shv_cuda_job*> jobs;
            {
                std::unique_lock<std::mutex> lk(mu_);
                if (inflight.empty()) wake_.wait(lk, [&] { return stopping_ || !queue_.empty(); });
                if (queue_.empty() && inflight.empty() && stopping_) return;
                if (!queue_.empty() && int(inflight.size()) < nslots) {
                    if (opt.max_delay_us > 0 && inflight.empty()) {
                        const auto deadline = Clock::now() + std::chrono::microseconds(opt.max_delay_us);
                        wake_.wait_until(lk, deadline, [&] {
                            if (stopping_) return true;
                            size_t w = 0;
                            for (const shv_cuda_job* j : queue_) w += j->n_windows;
                            return w >= size_t(opt.max_windows);
                        });
                    }
                    coalesce(jobs);
                    if (!jobs.empty() && starve_batches_ > 0) {
                        engine->inject_wait_timeout(starve_kind_, starve_batches_);
                        starve_batches_ = 0;
                    }
                }
            }
            if (!jobs.empty()) {
                inflight.push_back(launch(next_slot, jobs));
                next_slot = (next_slot + 1) % nslots;
                if (int(inflight.size()) < nslots) {
                    std::lock_guard<std::mutex> lk(mu_);
                    if (!queue_.empty()) continue;            // stage a second batch before waiting on the first
                }
            }
            if (!inflight.empty()) {
                retire(inflight.front());
                inflight.pop_front();
            }
        }
    }
};

template <class F> int guarded(F&& f) {
    try {
        return f();
    } catch (const std::exception& e) {
        t_error = e.what();
        return -1;
    }
}

// Splits `n` host block pointers into maximal contiguous runs and classifies each run as pinned or pageable.
void add_runs(shv_cuda_job& j, const float* const* blocks, size_t n) {
    size_t i = 0;
    while (i < n) {
        size_t k = i + 1;
        while (k < n && blocks[k] == blocks[k - 1] + kBlockFloats) ++k;
        j.runs.push_back({blocks[i], int(k - i), host_pinned(blocks[i], (k - i) * kBlockBytes)});
        i = k;
    }
    j.host_blocks += int(n);
}

int wait_and_free(std::vector<shv_cuda_job*>& jobs) {
    int rc = 0;
    std::string err;
    for (shv_cuda_job* j : jobs) {
        if (shv_cuda_job_wait(j) != 0) {
            rc = -1;
            if (err.empty()) err = shv_cuda_job_error(j);
        }
        shv_cuda_job_free(j);
    }
    if (rc) t_error = err;
    return rc;
}

}  // namespace

struct shv_cuda_model {
    std::unique_ptr<Scheduler> sched;
};

// shared with engine_c.cpp
void shv_cuda_set_error(const std::string& s) { t_error = s; }

extern "C" {

void shv_cuda_default_options(shv_cuda_options* o) {
    if (!o) return;
    o->max_frames = 640;
    o->max_windows = 512;
    o->max_host_tokens = 2048;
    o->token_slots = 0;
    o->use_graphs = 1;
    o->max_delay_us = 0;
}

shv_cuda_model* shv_cuda_load_ex(const char* weights, const char* mode, int device, const shv_cuda_options* opt) {
    try {
        if (!weights) throw std::runtime_error("null weights path");
        auto s = std::unique_ptr<Scheduler>(new Scheduler());
        s->mode = mode ? mode : "fp32";
        shv::Precision p;
        if (!shv::parse_precision(s->mode, &p)) throw std::runtime_error("unknown mode '" + s->mode + "' (fp32, bf16, fp16)");
        shv_cuda_default_options(&s->opt);
        if (opt) s->opt = *opt;
        const shv_cuda_options& o = s->opt;
        if (o.max_frames < 1 || o.max_frames > 4096 || o.max_windows < 1 || o.max_windows > 4096 || o.max_host_tokens < 0 ||
            o.max_host_tokens > (1 << 20) || o.token_slots < 0 || o.max_delay_us < 0)
            throw std::runtime_error("invalid options");
        s->device = device;
        const shv::HostModel hm = shv::load_host_model(weights);
        s->fingerprint = hm.sha256;
        s->threshold = hm.threshold;
        shv::check_sidecar_sha(weights, hm.sha256);
#ifndef SHV_CUDA_EXPERIMENTAL
        if (p != shv::Precision::FP32) {
            const std::string why = shv::check_certificate(weights, hm.sha256, s->mode, SHV_CUDA_REVISION, hm.threshold);
            if (!why.empty()) throw std::runtime_error(why);
        }
#endif
        s->start(hm);
        auto* m = new shv_cuda_model();
        m->sched = std::move(s);
        t_error.clear();
        return m;
    } catch (const std::exception& e) {
        t_error = e.what();
        return nullptr;
    }
}

shv_cuda_model* shv_cuda_load(const char* weights, const char* mode, int device) {
    return shv_cuda_load_ex(weights, mode, device, nullptr);
}

void shv_cuda_free(shv_cuda_model* m) {
    if (!m) return;
    m->sched->stop();
    delete m;
}

const char* shv_cuda_last_error(void) { return t_error.c_str(); }
const char* shv_cuda_mode(const shv_cuda_model* m) { return m ? m->sched->mode.c_str() : ""; }
const char* shv_cuda_fingerprint(const shv_cuda_model* m) { return m ? m->sched->fingerprint.c_str() : ""; }
double shv_cuda_threshold(const shv_cuda_model* m) { return m ? m->sched->threshold : std::nan(""); }
const char* shv_cuda_compute_revision(void) { return SHV_CUDA_REVISION; }
int shv_cuda_limits(const shv_cuda_model* m, int* mf, int* mw, int* mh, int* ts) {
    if (!m) { t_error = "null model"; return -1; }
    const shv_cuda_options& o = m->sched->opt;
    if (mf) *mf = o.max_frames;
    if (mw) *mw = o.max_windows;
    if (mh) *mh = o.max_host_tokens;
    if (ts) *ts = o.token_slots;
    return 0;
}
size_t shv_cuda_weight_bytes(const shv_cuda_model* m) { return m ? m->sched->engine->weight_bytes() : 0; }
size_t shv_cuda_device_bytes(const shv_cuda_model* m) { return m ? m->sched->device_bytes : 0; }

shv_cuda_job* shv_cuda_submit(shv_cuda_model* m, const shv_cuda_request* r) {
    try {
        if (!m || !r) throw std::runtime_error("null argument");
        Scheduler& s = *m->sched;
        const shv_cuda_options& o = s.opt;
        if (r->n_frames > size_t(o.max_frames)) throw std::runtime_error("request has more frames than max_frames");
        if (r->n_windows > size_t(o.max_windows)) throw std::runtime_error("request has more windows than max_windows");
        if (r->n_frames && !r->frames) throw std::runtime_error("null frames");
        if (r->n_windows && !r->logits_out) throw std::runtime_error("null logits_out");
        if (!r->n_frames && !r->n_windows) throw std::runtime_error("empty request");
        auto j = std::unique_ptr<shv_cuda_job>(new shv_cuda_job());
        j->frames = r->frames;
        j->n_frames = r->n_frames;
        j->tokens_out = r->n_frames ? r->tokens_out : nullptr;
        if (r->store_slots && r->n_frames) {
            if (!s.d_pool) throw std::runtime_error("store_slots needs options.token_slots > 0");
            j->frame_store.assign(r->store_slots, r->store_slots + r->n_frames);
            std::unordered_set<int32_t> seen;
            for (int32_t sl : j->frame_store) {
                if (sl < -1 || sl >= o.token_slots) throw std::runtime_error("store slot out of range");
                if (sl >= 0 && !seen.insert(sl).second) throw std::runtime_error("duplicate store slot in one request");
            }
        }
        j->n_windows = r->n_windows;
        j->logits_out = r->logits_out;
        j->cb = r->callback;
        j->user = r->user;
        const size_t entries = r->n_windows * 20;
        j->wslots.assign(entries, -1);
        if (r->window_frames && r->n_frames) j->wframes.assign(entries, -1);
        std::vector<const float*> host;
        host.reserve(entries);
        for (size_t e = 0; e < entries; ++e) {
            const int32_t wf = r->window_frames ? r->window_frames[e] : -1;
            const int32_t ws = r->window_slots ? r->window_slots[e] : -1;
            if (wf >= 0) {
                if (size_t(wf) >= r->n_frames) throw std::runtime_error("window frame index out of range");
                j->wframes[e] = wf;
            } else if (ws >= 0) {
                if (!s.d_pool || ws >= o.token_slots) throw std::runtime_error("window slot out of range");
                j->wslots[e] = ws;
            } else {
                if (!r->window_tokens || !r->window_tokens[e]) throw std::runtime_error("window entry has no token source");
                host.push_back(r->window_tokens[e]);
            }
        }
        if (host.size() > size_t(o.max_host_tokens))
            throw std::runtime_error("request has more host token blocks than max_host_tokens");
        add_runs(*j, host.data(), host.size());
        j->frames_pinned = host_pinned(r->frames, r->n_frames * kFrameBytes);
        j->tokens_out_pinned = j->tokens_out && host_pinned(j->tokens_out, r->n_frames * kBlockBytes);
        j->t_submit = Clock::now();
        shv_cuda_job* raw = j.release();
        if (!s.enqueue(raw)) {
            delete raw;
            throw std::runtime_error("model is stopping");
        }
        t_error.clear();
        return raw;
    } catch (const std::exception& e) {
        t_error = e.what();
        return nullptr;
    }
}

int shv_cuda_job_status(const shv_cuda_job* j) {
    if (!j) return -1;
    std::lock_guard<std::mutex> lk(j->m);
    return j->state;
}
int shv_cuda_job_wait(shv_cuda_job* j) {
    if (!j) { t_error = "null job"; return -1; }
    std::unique_lock<std::mutex> lk(j->m);
    j->cv.wait(lk, [&] { return j->state != 0; });
    if (j->state < 0) { t_error = j->error; return -1; }
    return 0;
}
const char* shv_cuda_job_error(const shv_cuda_job* j) {
    if (!j) return "null job";
    std::lock_guard<std::mutex> lk(j->m);
    return j->error.c_str();
}
int shv_cuda_job_timing(const shv_cuda_job* j, double* queue_ms, double* run_ms, double* gpu_ms, int* bf, int* bw) {
    if (!j) return -1;
    std::lock_guard<std::mutex> lk(j->m);
    if (j->state == 0) return 1;
    auto ms = [](Clock::duration d) { return std::chrono::duration<double, std::milli>(d).count(); };
    if (queue_ms) *queue_ms = ms(j->t_start - j->t_submit);
    if (run_ms) *run_ms = ms(j->t_done - j->t_start);
    if (gpu_ms) *gpu_ms = j->gpu_ms;
    if (bf) *bf = j->batch_frames;
    if (bw) *bw = j->batch_windows;
    return 0;
}
void shv_cuda_job_free(shv_cuda_job* j) {
    if (!j) return;
    {
        std::unique_lock<std::mutex> lk(j->m);
        j->cv.wait(lk, [&] { return j->released; });
    }
    delete j;
}

void* shv_cuda_host_alloc(size_t bytes) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        t_error = "cudaHostAlloc failed";
        return nullptr;
    }
    return p;
}
void shv_cuda_host_free(void* p) {
    if (p) cudaFreeHost(p);
}

int shv_cuda_encode_frames(shv_cuda_model* m, const uint8_t* rgb, size_t n, float* tokens) {
    return guarded([&]() -> int {
        if (!m || (n && (!rgb || !tokens))) throw std::runtime_error("null argument");
        const size_t step = size_t(m->sched->opt.max_frames);
        std::vector<shv_cuda_job*> jobs;
        for (size_t off = 0; off < n; off += step) {
            shv_cuda_request r{};
            r.frames = rgb + off * kFrameBytes;
            r.n_frames = std::min(step, n - off);
            r.tokens_out = tokens + off * kBlockFloats;
            shv_cuda_job* j = shv_cuda_submit(m, &r);
            if (!j) {
                const std::string why = t_error;
                wait_and_free(jobs);
                std::fill(tokens, tokens + n * kBlockFloats, kNaN);
                throw std::runtime_error(why);
            }
            jobs.push_back(j);
        }
        return wait_and_free(jobs);
    });
}

int shv_cuda_predict(shv_cuda_model* m, const uint8_t* clips, size_t b, float* logits) {
    return guarded([&]() -> int {
        if (!m || (b && (!clips || !logits))) throw std::runtime_error("null argument");
        const shv_cuda_options& o = m->sched->opt;
        const size_t step = size_t(std::min(o.max_windows, o.max_frames / 20));
        if (step < 1) throw std::runtime_error("predict needs max_frames >= 20");
        std::vector<int32_t> idx(step * 20);
        for (size_t e = 0; e < idx.size(); ++e) idx[e] = int32_t(e);
        std::vector<shv_cuda_job*> jobs;
        for (size_t off = 0; off < b; off += step) {
            const size_t w = std::min(step, b - off);
            shv_cuda_request r{};
            r.frames = clips + off * 20 * kFrameBytes;
            r.n_frames = w * 20;
            r.n_windows = w;
            r.window_frames = idx.data();
            r.logits_out = logits + off;
            shv_cuda_job* j = shv_cuda_submit(m, &r);
            if (!j) {
                const std::string why = t_error;
                wait_and_free(jobs);
                std::fill(logits, logits + b, kNaN);
                throw std::runtime_error(why);
            }
            jobs.push_back(j);
        }
        return wait_and_free(jobs);
    });
}

int shv_cuda_classify(shv_cuda_model* m, const float* tokens, size_t b, float* logits) {
    return guarded([&]() -> int {
        if (!m || (b && (!tokens || !logits))) throw std::runtime_error("null argument");
        const shv_cuda_options& o = m->sched->opt;
        if (o.max_host_tokens < 20) throw std::runtime_error("classify needs max_host_tokens >= 20");
        const size_t step = size_t(std::max(1, std::min(o.max_windows, o.max_host_tokens / 20)));
        std::vector<shv_cuda_job*> jobs;
        std::vector<const float*> ptrs;
        for (size_t off = 0; off < b; off += step) {
            const size_t w = std::min(step, b - off);
            ptrs.resize(w * 20);
            for (size_t e = 0; e < w * 20; ++e) ptrs[e] = tokens + (off * 20 + e) * kBlockFloats;
            shv_cuda_request r{};
            r.n_windows = w;
            r.window_tokens = ptrs.data();
            r.logits_out = logits + off;
            shv_cuda_job* j = shv_cuda_submit(m, &r);
            if (!j) {
                const std::string why = t_error;
                wait_and_free(jobs);
                std::fill(logits, logits + b, kNaN);
                throw std::runtime_error(why);
            }
            jobs.push_back(j);
        }
        return wait_and_free(jobs);
    });
}

// ---------------------------------------------------------------- extensions (include/shv_cuda_b200.h)
int shv_cuda_b200_upload_tokens(shv_cuda_model* m, const float* tokens, size_t n, const int32_t* slots) {
    return guarded([&]() -> int {
        if (!m || (n && (!tokens || !slots))) throw std::runtime_error("null argument");
        Scheduler& s = *m->sched;
        if (!s.d_pool) throw std::runtime_error("upload_tokens needs options.token_slots > 0");
        if (s.block_cap() < 1) throw std::runtime_error("upload_tokens needs max_host_tokens >= 1");
        const size_t step = size_t(s.block_cap());
        std::vector<shv_cuda_job*> jobs;
        for (size_t off = 0; off < n; off += step) {
            const size_t cnt = std::min(step, n - off);
            auto j = std::unique_ptr<shv_cuda_job>(new shv_cuda_job());
            std::unordered_set<int32_t> seen;
            for (size_t i = 0; i < cnt; ++i) {
                const int32_t sl = slots[off + i];
                if (sl < 0 || sl >= s.opt.token_slots) throw std::runtime_error("store slot out of range");
                if (!seen.insert(sl).second) throw std::runtime_error("duplicate store slot in one request");
                j->store_slots.push_back(sl);
            }
            std::vector<const float*> ptrs(cnt);
            for (size_t i = 0; i < cnt; ++i) ptrs[i] = tokens + (off + i) * kBlockFloats;
            add_runs(*j, ptrs.data(), cnt);
            j->t_submit = Clock::now();
            shv_cuda_job* raw = j.release();
            if (!s.enqueue(raw)) {
                delete raw;
                wait_and_free(jobs);
                throw std::runtime_error("model is stopping");
            }
            jobs.push_back(raw);
        }
        return wait_and_free(jobs);
    });
}

int shv_cuda_b200_launches_per_batch(const shv_cuda_model* m) { return m ? m->sched->engine->launches_per_classify() : 0; }

int shv_cuda_b200_test_starve(shv_cuda_model* m, int kind, int batches) {
#ifdef SHV_CUDA_EXPERIMENTAL
    return guarded([&]() -> int {
        if (!m) throw std::runtime_error("null model");
        m->sched->request_starve(kind, batches);
        return 0;
    });
#else
    (void)m; (void)kind; (void)batches;
    t_error = "test hooks exist in the experimental library only";
    return -1;
#endif
}

}  // extern "C"
