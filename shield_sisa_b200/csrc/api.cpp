// C ABI of libshield_v_cuda.so (contract: include/shv_cuda.h) over the engine core: an asynchronous job pipeline.
//
//   caller threads           feeder thread                       GPU (copy stream | compute stream)     finisher thread
//   submit(job) -> pending   forms a batch from the head of      H2D of batch n+2 | kernels of batch n  waits for the oldest batch in
//                            `pending`, fills a free lane,       ...                                     flight, hands results to its
//                            enqueues copies + kernels           up to kLanes batches in flight          jobs, runs callbacks, frees the lane
//
// A lane is one set of buffers (an engine slot plus its pinned host companions).  With four lanes the copy engine runs
// up to three batches ahead of the kernels, and completing a batch (callbacks included) never holds up the staging of
// the next one.  Jobs run in submission order.  The feeder coalesces consecutive jobs while the batch limits hold and
// no job stores into a token slot that the batch already reads or stores; while the pipeline is not yet full it also
// closes a batch early (at an eighth of the limits), so that the first kernels of a burst start while the rest of the
// burst is still being uploaded; and a batch never carries more than an eighth of the limits in data that has to be
// uploaded first, so a stream of batches keeps copy engine and SMs busy together -- a single large synchronous call
// overlaps its own uploads and kernels this way.
// Within a batch: frames are encoded, their tokens stored into the slots the requests name, host token blocks
// uploaded (pinned runs by DMA straight from the caller's memory, the rest through a pinned staging copy), then all
// windows are classified together; a window sees the frames and stores of its own request and of every earlier one.
// A batch that fails (a CUDA error, a kernel whose bounded wait gave up) fails all its jobs: their outputs become NaN;
// a non-finite logit is reported as NaN.  shv_cuda_job_free returns only after the job's callback has.
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

#ifndef SHV_CUDA_REVISION
#define SHV_CUDA_REVISION "unversioned"
#endif

namespace {

using Clock = std::chrono::steady_clock;
constexpr int kLanes = 4;
constexpr size_t kTokFloats = SHV_CUDA_TOKEN_FLOATS, kTokBytes = kTokFloats * sizeof(float), kCropBytes = SHV_CUDA_FRAME_BYTES;
constexpr int kWin = SHV_CUDA_WINDOW_FRAMES;
const float kUnavailable = std::numeric_limits<float>::quiet_NaN();

thread_local std::string tls_error;

struct ApiError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw ApiError(std::string("CUDA error ") + cudaGetErrorString(e) + " in " + what);
}
void check(int e, const char* what) { check(cudaError_t(e), what); }

// True if [p, p + bytes) starts and ends in page-locked host memory, i.e. the copy engine can read or write it directly.
bool is_pinned(const void* p, size_t bytes) {
    if (!p || !bytes) return false;
    const uint8_t* ends[2] = {static_cast<const uint8_t*>(p), static_cast<const uint8_t*>(p) + bytes - 1};
    for (const uint8_t* q : ends) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, q) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        if (attr.type != cudaMemoryTypeHost) return false;
    }
    return true;
}

template <typename T> T* pinned_array(size_t n, const char* what) {
    void* p = nullptr;
    check(cudaHostAlloc(&p, std::max<size_t>(n, 1) * sizeof(T), cudaHostAllocDefault), what);
    return static_cast<T*>(p);
}

// Where one window entry (window w, frame position f) of a job takes its 16 x 384 block from.
enum class Src : uint8_t { Host, Slot, Frame };
struct Entry {
    Src src;
    int32_t index;      // Slot: token slot; Frame: frame of the job's own request; Host: ordinal among the job's host blocks
};
// Host token blocks that follow one another in memory travel as one copy.
struct Span {
    const float* first;
    int count;
    bool pinned;
    bool half;          // the blocks hold fp16 tokens (12,288 bytes each): shv_cuda_b200_classify_f16
};

}  // namespace

struct shv_cuda_job {
    // ---- what was asked (index arrays copied, buffers borrowed)
    const uint8_t* crops = nullptr;
    int n_crops = 0;
    bool crops_pinned = false;
    float* tokens_out = nullptr;
    bool tokens_out_pinned = false;
    std::vector<int32_t> crop_slot;         // per crop: token slot that receives its tokens, or -1 (empty = none)
    int n_windows = 0;
    std::vector<Entry> entries;             // n_windows * 20
    std::vector<Span> spans;                // the job's host blocks in entry order (or in upload order)
    int n_host = 0;
    std::vector<int32_t> host_slot;         // upload job: destination slot of every host block (empty otherwise)
    float* logits_out = nullptr;
    shv_cuda_callback callback = nullptr;
    void* user = nullptr;
    // ---- where it landed
    int first_window = 0, first_crop = 0;
    Clock::time_point submitted, started, finished;
    float gpu_ms = 0.0f;
    int batch_crops = 0, batch_windows = 0;
    // ---- completion: outcome 0 until the batch retires; `settled` once the callback has returned
    mutable std::mutex mu;
    std::condition_variable cv;
    int outcome = 0;
    bool settled = false;
    std::string why;

    void complete(bool ok, const std::string& error, float ms, int crops_in_batch, int windows_in_batch) {
        {
            std::lock_guard<std::mutex> g(mu);
            outcome = ok ? 1 : -1;
            why = ok ? std::string() : error;
            finished = Clock::now();
            gpu_ms = ms;
            batch_crops = crops_in_batch;
            batch_windows = windows_in_batch;
        }
        cv.notify_all();
        // the job cannot be freed before `settled`, so the callback may use the handle
        if (callback) callback(this, ok ? 1 : -1, user);
        {
            std::lock_guard<std::mutex> g(mu);
            settled = true;
            cv.notify_all();                // inside the lock: a waiter in job_free may delete the job the moment it wakes
        }
    }
};

namespace {

// One buffer set of the pipeline: engine slot `index` and the pinned host memory that goes with it.
struct Lane {
    int index = 0;
    const float** table = nullptr;       // [max_windows * 20] device addresses of the windows' blocks
    int32_t* block_slot = nullptr;       // [block cap] destination slot per uploaded host block (-1 = none)
    int32_t* d_block_slot = nullptr;
    int32_t* crop_slot = nullptr;        // [max_frames] destination slot per encoded crop
    int32_t* d_crop_slot = nullptr;
    float* logits = nullptr;             // [max_windows]
    int* status = nullptr;               // [SHVK_STATUS_WORDS] the kernels' status words behind the batch
    float* stage_tokens = nullptr;       // staging for pageable host blocks, made on first use
    uint8_t* stage_crops = nullptr;      // staging for pageable crops, made on first use
    float* stage_tokens_out = nullptr;   // staging for pageable tokens_out, made on first use
    cudaEvent_t uploaded = nullptr, begin = nullptr, end = nullptr;

    void release() {
        for (void* p : {static_cast<void*>(table), static_cast<void*>(block_slot), static_cast<void*>(crop_slot),
                        static_cast<void*>(logits), static_cast<void*>(status), static_cast<void*>(stage_tokens),
                        static_cast<void*>(stage_crops), static_cast<void*>(stage_tokens_out)})
            if (p) cudaFreeHost(p);
        if (d_block_slot) cudaFree(d_block_slot);
        if (d_crop_slot) cudaFree(d_crop_slot);
        for (cudaEvent_t e : {uploaded, begin, end})
            if (e) cudaEventDestroy(e);
    }
};

struct Flight {                           // a batch between launch and retirement
    Lane* lane = nullptr;
    std::vector<shv_cuda_job*> jobs;
    std::vector<std::pair<int, int>> half_runs;   // (first staging block, count) of the runs that arrived as fp16 tokens
    int windows = 0, crops = 0;
    bool launched = false;                // false: enqueueing threw; `error` says why
    std::string error;
};

class Pipeline {
public:
    std::unique_ptr<shv::Engine> engine;
    std::string mode, fingerprint;
    double threshold = 0.0;
    int device = 0;
    shv_cuda_options opt{};
    size_t device_bytes = 0;
    float* pool = nullptr;                // device token slots [token_slots][6144]

    ~Pipeline() {
        for (Lane& l : lanes_) l.release();
        if (pool) cudaFree(pool);
        engine.reset();
        for (cudaStream_t s : {compute_, copy_})
            if (s) cudaStreamDestroy(s);
    }

    int block_cap() const { return std::min(opt.max_host_tokens, opt.max_windows * kWin); }
    // What one batch should carry at most when everything it classifies has to be uploaded first: an eighth of the
    // limits (at least 256 windows / frames).  Uploads and kernels of a stream of such batches overlap batch by batch; one
    // batch of the full limit would keep the GPU idle for the whole of its upload.
    int upload_windows() const { return std::max(std::min(256, opt.max_windows), opt.max_windows / 8); }
    int upload_crops() const { return std::max(std::min(256, opt.max_frames), opt.max_frames / 8); }

    void start(const shv::HostModel& hm) {
        check(cudaSetDevice(device), "cudaSetDevice");
        check(cudaStreamCreateWithFlags(&compute_, cudaStreamNonBlocking), "stream");
        check(cudaStreamCreateWithFlags(&copy_, cudaStreamNonBlocking), "stream");
        shv::Precision prec;
        if (!shv::parse_precision(mode, &prec)) throw ApiError("unknown mode: " + mode);
        shv::EngineConfig cfg;
        cfg.max_frames = opt.max_frames;
        cfg.max_windows = opt.max_windows;
        cfg.use_graphs = opt.use_graphs != 0;
        cfg.slots = kLanes;
        cfg.max_host_blocks = block_cap();
        engine = shv::make_engine(hm, prec, cfg);
        const size_t nwin = size_t(opt.max_windows), nblk = size_t(std::max(block_cap(), 1)), ncrop = size_t(opt.max_frames);
        lanes_.resize(kLanes);
        for (int i = 0; i < kLanes; ++i) {
            Lane& l = lanes_[size_t(i)];
            l.index = i;
            l.table = pinned_array<const float*>(nwin * kWin, "pinned pointer table");
            l.block_slot = pinned_array<int32_t>(nblk, "pinned slot list");
            l.crop_slot = pinned_array<int32_t>(ncrop, "pinned slot list");
            l.logits = pinned_array<float>(nwin, "pinned logits");
            l.status = pinned_array<int>(SHVK_STATUS_WORDS, "pinned status words");
            std::fill(l.status, l.status + SHVK_STATUS_WORDS, 0);
            check(cudaMalloc(reinterpret_cast<void**>(&l.d_block_slot), nblk * sizeof(int32_t)), "device slot list");
            check(cudaMalloc(reinterpret_cast<void**>(&l.d_crop_slot), ncrop * sizeof(int32_t)), "device slot list");
            check(cudaEventCreateWithFlags(&l.uploaded, cudaEventDisableTiming), "event");
            check(cudaEventCreate(&l.begin), "event");
            check(cudaEventCreate(&l.end), "event");
            idle_.push_back(&l);
        }
        if (opt.token_slots > 0) {
            check(cudaMalloc(reinterpret_cast<void**>(&pool), size_t(opt.token_slots) * kTokBytes), "token slots");
            check(cudaMemset(pool, 0, size_t(opt.token_slots) * kTokBytes), "token slots");
            touched_.assign(size_t(opt.token_slots), 0);
        }
        device_bytes = engine->weight_bytes() + engine->activation_bytes() +
                       size_t(kLanes) * (engine->slot_bytes() + (nblk + ncrop) * sizeof(int32_t)) +
                       size_t(std::max(opt.token_slots, 0)) * kTokBytes;
#ifdef SHV_CUDA_EXPERIMENTAL
        // test hook of the experimental library only: the certificate-checked library reads no environment
        if (const char* e = std::getenv("SHV_CUDA_FAIL_EVERY")) fail_every_ = std::atol(e);
#endif
        check(cudaDeviceSynchronize(), "initialisation");
        feeder_ = std::thread([this] { feed(); });
        finisher_ = std::thread([this] { finish(); });
    }

    // Queues a job; false if the model is shutting down (the caller keeps the job).
    bool accept(shv_cuda_job* j) {
        {
            std::lock_guard<std::mutex> g(mu_);
            if (closing_) return false;
            pending_.push_back(j);
        }
        work_.notify_all();
        return true;
    }

    // Everything queued so far still runs; returns when both threads have ended.
    void shutdown() {
        {
            std::lock_guard<std::mutex> g(mu_);
            closing_ = true;
        }
        work_.notify_all();
        if (feeder_.joinable()) feeder_.join();
        if (finisher_.joinable()) finisher_.join();
    }

    // Test hook: the feeder arms the engine before its next batch (the engine has a single driver thread).
    void arm_starved_launch(int kind, int batches) {
        if (kind != 1 && kind != 2) throw ApiError("starve kind: 1 = tensor-core GEMM, 2 = scan");
        if (mode == "fp32") throw ApiError("the starved test launches exist for the 16-bit modes only");
        std::lock_guard<std::mutex> g(mu_);
        starve_kind_ = kind;
        starve_batches_ = batches;
    }

private:
    cudaStream_t compute_ = nullptr, copy_ = nullptr;
    std::vector<Lane> lanes_;
    std::mutex mu_;                          // guards everything below
    std::condition_variable work_;           // pending job, freed lane, launched batch, shutdown
    std::deque<shv_cuda_job*> pending_;
    std::deque<Lane*> idle_;
    std::deque<Flight> flying_;
    bool closing_ = false, feeder_done_ = false;
    int starve_kind_ = 0, starve_batches_ = 0;
    std::vector<uint8_t> touched_;           // per token slot, within the batch being formed: 1 read, 2 stored
    std::vector<int32_t> touched_list_;
    long launched_ = 0, fail_every_ = 0;
    std::thread feeder_, finisher_;

    // ------------------------------------------------------------------------------------------ batch formation
    // Would adding `j` to the batch being formed store into a slot the batch already touches?
    bool store_hazard(const shv_cuda_job* j) const {
        for (const std::vector<int32_t>* list : {&j->crop_slot, &j->host_slot})
            for (int32_t s : *list)
                if (s >= 0 && touched_[size_t(s)]) return true;
        return false;
    }
    void note_slots(const shv_cuda_job* j) {
        auto mark = [&](int32_t s, uint8_t how) {
            if (s < 0) return;
            if (!touched_[size_t(s)]) touched_list_.push_back(s);
            touched_[size_t(s)] |= how;
        };
        for (int32_t s : j->crop_slot) mark(s, 2);
        for (int32_t s : j->host_slot) mark(s, 2);
        for (const Entry& e : j->entries)
            if (e.src == Src::Slot) mark(e.index, 1);
    }
    // Moves the head of `pending_` into `out`.  Caller holds mu_.  A batch closes at the limits of the options, at a store
    // hazard, or -- counting only what must be uploaded (host token blocks, crops) -- at the per-batch upload budget;
    // windows that read device token slots cost no upload and coalesce up to the limit, except while the pipeline has
    // room to spare (`eager`), when a batch also closes at that many windows so that the first kernels start early.
    void take_batch(std::vector<shv_cuda_job*>& out, bool eager) {
        const int want_blocks = upload_windows() * kWin, want_crops = upload_crops();
        const int want_windows = eager ? upload_windows() : opt.max_windows;
        int windows = 0, blocks = 0, crops = 0;
        while (!pending_.empty()) {
            shv_cuda_job* j = pending_.front();
            if (!out.empty()) {
                if (windows + j->n_windows > opt.max_windows || blocks + j->n_host > block_cap() || crops + j->n_crops > opt.max_frames)
                    break;
                if (windows >= want_windows || crops >= want_crops || blocks >= want_blocks) break;
                if (pool && store_hazard(j)) break;
            }
            pending_.pop_front();
            out.push_back(j);
            windows += j->n_windows;
            blocks += j->n_host;
            crops += j->n_crops;
            if (pool) note_slots(j);
        }
        for (int32_t s : touched_list_) touched_[size_t(s)] = 0;
        touched_list_.clear();
    }

    // ------------------------------------------------------------------------------------------ feeder
    void feed() {
        if (cudaSetDevice(device) != cudaSuccess) cudaGetLastError();
        for (;;) {
            Flight f;
            {
                std::unique_lock<std::mutex> lk(mu_);
                work_.wait(lk, [&] { return (!pending_.empty() && !idle_.empty()) || (closing_ && pending_.empty()); });
                if (pending_.empty()) {
                    feeder_done_ = true;
                    lk.unlock();
                    work_.notify_all();
                    return;
                }
                if (opt.max_delay_us > 0 && flying_.empty()) {
                    // nothing to overlap with yet: give more jobs a moment to arrive, up to a full batch
                    const auto until = Clock::now() + std::chrono::microseconds(opt.max_delay_us);
                    work_.wait_until(lk, until, [&] {
                        long w = 0;
                        for (const shv_cuda_job* j : pending_) w += j->n_windows;
                        return closing_ || w >= opt.max_windows;
                    });
                }
                take_batch(f.jobs, int(flying_.size()) + 1 < kLanes);
                f.lane = idle_.front();
                idle_.pop_front();
                if (starve_batches_ > 0) {
                    engine->inject_wait_timeout(starve_kind_, starve_batches_);
                    starve_batches_ = 0;
                }
            }
            enqueue(f);
            {
                std::lock_guard<std::mutex> g(mu_);
                flying_.push_back(std::move(f));
            }
            work_.notify_all();
        }
    }

    // Copies + kernels of one batch into the streams.  Never blocks on the GPU.  On an exception the batch is marked
    // unlaunched; whatever was already enqueued only touches the lane's own buffers.
    void enqueue(Flight& f) {
        Lane& l = *f.lane;
        const shv::Engine::Slot& dev = engine->slot(l.index);
        const Clock::time_point now = Clock::now();
        try {
            if (fail_every_ > 0 && ++launched_ % fail_every_ == 0) throw ApiError("injected batch failure (SHV_CUDA_FAIL_EVERY)");
            int windows = 0, crops = 0, blocks = 0;
            bool crop_stores = false, block_stores = false;
            for (shv_cuda_job* j : f.jobs) {
                j->started = now;
                j->first_window = windows;
                j->first_crop = crops;
                if (j->n_crops) {
                    uint8_t* dst = dev.d_frames + size_t(crops) * kCropBytes;
                    const size_t bytes = size_t(j->n_crops) * kCropBytes;
                    const uint8_t* from = j->crops;
                    if (!j->crops_pinned) {
                        if (!l.stage_crops) l.stage_crops = pinned_array<uint8_t>(size_t(opt.max_frames) * kCropBytes, "pinned crop staging");
                        std::memcpy(l.stage_crops + size_t(crops) * kCropBytes, j->crops, bytes);
                        from = l.stage_crops + size_t(crops) * kCropBytes;
                    }
                    check(cudaMemcpyAsync(dst, from, bytes, cudaMemcpyHostToDevice, copy_), "crop upload");
                    for (int c = 0; c < j->n_crops; ++c) {
                        const int32_t s = j->crop_slot.empty() ? -1 : j->crop_slot[size_t(c)];
                        l.crop_slot[crops + c] = s;
                        crop_stores |= s >= 0;
                    }
                }
                // host blocks: one copy per contiguous span; remember where each block lands on the device
                const int first_block = blocks;
                for (const Span& sp : j->spans) {
                    if (sp.half) {
                        // fp16 tokens: each block lands in the upper half of its fp32 staging block (one strided copy per
                        // span) and is widened in place on the device before anything reads it
                        uint8_t* dst16 = reinterpret_cast<uint8_t*>(dev.d_tok_stage + size_t(blocks) * kTokFloats) + kTokBytes / 2;
                        const void* from16 = sp.first;
                        if (!sp.pinned) {
                            if (!l.stage_tokens) l.stage_tokens = pinned_array<float>(size_t(std::max(block_cap(), 1)) * kTokFloats, "pinned token staging");
                            std::memcpy(l.stage_tokens + size_t(blocks) * kTokFloats, sp.first, size_t(sp.count) * (kTokBytes / 2));
                            from16 = l.stage_tokens + size_t(blocks) * kTokFloats;
                        }
                        check(cudaMemcpy2DAsync(dst16, kTokBytes, from16, kTokBytes / 2, kTokBytes / 2, size_t(sp.count),
                                                cudaMemcpyHostToDevice, copy_), "token upload");
                        f.half_runs.emplace_back(blocks, sp.count);
                        blocks += sp.count;
                        continue;
                    }
                    float* dst = dev.d_tok_stage + size_t(blocks) * kTokFloats;
                    const size_t bytes = size_t(sp.count) * kTokBytes;
                    const float* from = sp.first;
                    if (!sp.pinned) {
                        if (!l.stage_tokens) l.stage_tokens = pinned_array<float>(size_t(std::max(block_cap(), 1)) * kTokFloats, "pinned token staging");
                        std::memcpy(l.stage_tokens + size_t(blocks) * kTokFloats, sp.first, bytes);
                        from = l.stage_tokens + size_t(blocks) * kTokFloats;
                    }
                    check(cudaMemcpyAsync(dst, from, bytes, cudaMemcpyHostToDevice, copy_), "token upload");
                    blocks += sp.count;
                }
                for (int b = 0; b < j->n_host; ++b) {
                    const int32_t s = j->host_slot.empty() ? -1 : j->host_slot[size_t(b)];
                    l.block_slot[first_block + b] = s;
                    block_stores |= s >= 0;
                }
                const float** row = l.table + size_t(windows) * kWin;
                for (size_t e = 0; e < j->entries.size(); ++e) {
                    const Entry& en = j->entries[e];
                    row[e] = en.src == Src::Host   ? dev.d_tok_stage + size_t(first_block + en.index) * kTokFloats
                             : en.src == Src::Slot ? pool + size_t(en.index) * kTokFloats
                                                   : dev.d_tokens + size_t(crops + en.index) * kTokFloats;
                }
                windows += j->n_windows;
                crops += j->n_crops;
            }
            if (crop_stores)
                check(cudaMemcpyAsync(l.d_crop_slot, l.crop_slot, size_t(crops) * sizeof(int32_t), cudaMemcpyHostToDevice, copy_), "slot list upload");
            if (block_stores)
                check(cudaMemcpyAsync(l.d_block_slot, l.block_slot, size_t(blocks) * sizeof(int32_t), cudaMemcpyHostToDevice, copy_), "slot list upload");
            if (windows)
                check(cudaMemcpyAsync(dev.d_tokptr, l.table, size_t(windows) * kWin * sizeof(float*), cudaMemcpyHostToDevice, copy_), "pointer table upload");
            check(cudaEventRecord(l.uploaded, copy_), "event");
            check(cudaStreamWaitEvent(compute_, l.uploaded, 0), "event");
            check(cudaEventRecord(l.begin, compute_), "event");
            for (const std::pair<int, int>& run : f.half_runs)
                check(shvk_expand_f16_tokens(dev.d_tok_stage + size_t(run.first) * kTokFloats, run.second, compute_), "token widening");
            if (crops) engine->encode(l.index, crops, compute_);
            if (crop_stores) check(shvk_store_tokens(dev.d_tokens, l.d_crop_slot, pool, crops, compute_), "token slot store");
            if (block_stores) check(shvk_store_tokens(dev.d_tok_stage, l.d_block_slot, pool, blocks, compute_), "token slot store");
            if (windows) {
                engine->classify(l.index, windows, compute_);
                check(cudaMemcpyAsync(l.logits, dev.d_logits, size_t(windows) * sizeof(float), cudaMemcpyDeviceToHost, compute_), "logit download");
            }
            for (shv_cuda_job* j : f.jobs) {
                if (!j->tokens_out || !j->n_crops) continue;
                float* to = j->tokens_out;
                if (!j->tokens_out_pinned) {
                    if (!l.stage_tokens_out) l.stage_tokens_out = pinned_array<float>(size_t(opt.max_frames) * kTokFloats, "pinned token staging");
                    to = l.stage_tokens_out + size_t(j->first_crop) * kTokFloats;
                }
                check(cudaMemcpyAsync(to, dev.d_tokens + size_t(j->first_crop) * kTokFloats, size_t(j->n_crops) * kTokBytes,
                                      cudaMemcpyDeviceToHost, compute_), "token download");
            }
            check(shvk_status_fetch_async(l.status, compute_), "status fetch");
            check(cudaEventRecord(l.end, compute_), "event");
            f.windows = windows;
            f.crops = crops;
            f.launched = true;
        } catch (const std::exception& e) {
            f.launched = false;
            f.error = e.what();
        }
    }

    // ------------------------------------------------------------------------------------------ finisher
    void finish() {
        if (cudaSetDevice(device) != cudaSuccess) cudaGetLastError();
        for (;;) {
            Flight f;
            {
                std::unique_lock<std::mutex> lk(mu_);
                work_.wait(lk, [&] { return !flying_.empty() || feeder_done_; });
                if (flying_.empty()) return;
                f = std::move(flying_.front());       // stays counted as in flight until its lane is returned below
            }
            retire(f);
            {
                std::lock_guard<std::mutex> g(mu_);
                flying_.pop_front();
                idle_.push_back(f.lane);
            }
            work_.notify_all();
        }
    }

    void retire(Flight& f) {
        Lane& l = *f.lane;
        bool ok = f.launched;
        std::string error = f.error;
        float ms = 0.0f;
        if (ok) {
            const cudaError_t e = cudaEventSynchronize(l.end);
            if (e != cudaSuccess) {
                ok = false;
                error = std::string("CUDA error: ") + cudaGetErrorString(e);
            } else if (cudaEventElapsedTime(&ms, l.begin, l.end) != cudaSuccess) {
                cudaGetLastError();
                ms = 0.0f;
            }
            if (ok && std::any_of(l.status, l.status + SHVK_STATUS_WORDS, [](int w) { return w != 0; })) {
                // The status words are shared by everything on this device.  Clear them behind the work already queued,
                // so that batches launched from now on are judged on their own; a batch that was already in flight has
                // fetched the set words and fails as well.
                ok = false;
                error = "a kernel gave up waiting on its TMA / tensor-core pipeline (device status word set)";
                if (shvk_status_clear_async(compute_) != 0) cudaGetLastError();
            }
        } else {
            // whatever part of the batch was enqueued must not outlive the buffers the jobs lent us
            cudaStreamSynchronize(copy_);
            cudaStreamSynchronize(compute_);
        }
        for (shv_cuda_job* j : f.jobs) {
            if (ok) {
                const float* got = l.logits + j->first_window;
                for (int w = 0; w < j->n_windows; ++w) j->logits_out[w] = std::isfinite(got[w]) ? got[w] : kUnavailable;
                if (j->tokens_out && !j->tokens_out_pinned && j->n_crops)
                    std::memcpy(j->tokens_out, l.stage_tokens_out + size_t(j->first_crop) * kTokFloats, size_t(j->n_crops) * kTokBytes);
            } else {
                for (int w = 0; w < j->n_windows; ++w) j->logits_out[w] = kUnavailable;
                if (j->tokens_out) std::fill(j->tokens_out, j->tokens_out + size_t(j->n_crops) * kTokFloats, kUnavailable);
            }
            j->complete(ok, error, ms, f.crops, f.windows);
        }
    }
};

// Host block pointers -> spans of consecutive memory, each marked pinned or pageable.
void group_spans(shv_cuda_job& j, const std::vector<const float*>& blocks, bool half = false) {
    const size_t step = half ? kTokFloats / 2 : kTokFloats, block_bytes = half ? kTokBytes / 2 : kTokBytes;   // in floats; bytes
    size_t at = 0;
    while (at < blocks.size()) {
        size_t end = at + 1;
        while (end < blocks.size() && blocks[end] == blocks[end - 1] + step) ++end;
        j.spans.push_back(Span{blocks[at], int(end - at), is_pinned(blocks[at], (end - at) * block_bytes), half});
        at = end;
    }
    j.n_host = int(blocks.size());
}

void require_distinct_slots(const std::vector<int32_t>& slots, int token_slots, bool allow_none) {
    std::vector<int32_t> seen;
    for (int32_t s : slots) {
        if (s == -1 && allow_none) continue;
        if (s < 0 || s >= token_slots) throw ApiError("store slot out of range");
        seen.push_back(s);
    }
    std::sort(seen.begin(), seen.end());
    if (std::adjacent_find(seen.begin(), seen.end()) != seen.end()) throw ApiError("duplicate store slot in one request");
}

// Waits for every job, frees it, and reports the first failure (0 or -1, error string set).
int settle_all(std::vector<shv_cuda_job*>& jobs) {
    bool failed = false;
    std::string first;
    for (shv_cuda_job* j : jobs) {
        if (shv_cuda_job_wait(j) != 0 && !failed) {
            failed = true;
            first = shv_cuda_job_error(j);
        }
        shv_cuda_job_free(j);
    }
    jobs.clear();
    if (failed) tls_error = first;
    return failed ? -1 : 0;
}

// A synchronous call over `total` items as a train of requests of at most `piece` items, all submitted before the
// first is waited for, so that the pipeline overlaps their uploads and kernels.  make(first, count, request) fills the
// request; on a refused submit everything already queued is waited for and `poison` marks the outputs.
template <typename Make, typename Poison, typename Submit>
int run_in_pieces(shv_cuda_model* m, size_t total, size_t piece, Make make, Poison poison, Submit submit) {
    std::vector<shv_cuda_job*> jobs;
    for (size_t first = 0; first < total; first += piece) {
        shv_cuda_request r{};
        make(first, std::min(piece, total - first), r);
        shv_cuda_job* j = submit(m, &r);
        if (!j) {
            const std::string why = tls_error;
            settle_all(jobs);
            poison();
            tls_error = why;
            return -1;
        }
        jobs.push_back(j);
    }
    const int rc = settle_all(jobs);
    if (rc == 0) tls_error.clear();
    return rc;
}

}  // namespace

struct shv_cuda_model {
    std::unique_ptr<Pipeline> pipe;
};

// shared with engine_c.cpp
void shv_cuda_set_error(const std::string& s) { tls_error = s; }

extern "C" {

void shv_cuda_default_options(shv_cuda_options* o) {
    if (!o) return;
    *o = shv_cuda_options{640, 512, 2048, 0, 1, 0};
}

shv_cuda_model* shv_cuda_load_ex(const char* weights, const char* mode, int device, const shv_cuda_options* opt) {
    try {
        if (!weights) throw ApiError("null weights path");
        std::unique_ptr<Pipeline> p(new Pipeline());
        p->mode = mode ? mode : "fp32";
        shv::Precision prec;
        if (!shv::parse_precision(p->mode, &prec)) throw ApiError("unknown mode '" + p->mode + "' (fp32, bf16, fp16)");
        shv_cuda_default_options(&p->opt);
        if (opt) p->opt = *opt;
        const shv_cuda_options& o = p->opt;
        const bool sane = o.max_frames >= 1 && o.max_frames <= 4096 && o.max_windows >= 1 && o.max_windows <= 4096 &&
                          o.max_host_tokens >= 0 && o.max_host_tokens <= (1 << 20) && o.token_slots >= 0 && o.max_delay_us >= 0;
        if (!sane) throw ApiError("invalid options");
        p->device = device;
        const shv::HostModel hm = shv::load_host_model(weights);
        p->fingerprint = hm.sha256;
        p->threshold = hm.threshold;
        shv::check_sidecar_sha(weights, hm.sha256);
#ifndef SHV_CUDA_EXPERIMENTAL
        if (prec != shv::Precision::FP32) {
            const std::string refusal = shv::check_certificate(weights, hm.sha256, p->mode, SHV_CUDA_REVISION, hm.threshold);
            if (!refusal.empty()) throw ApiError(refusal);
        }
#endif
        p->start(hm);
        shv_cuda_model* m = new shv_cuda_model();
        m->pipe = std::move(p);
        tls_error.clear();
        return m;
    } catch (const std::exception& e) {
        tls_error = e.what();
        return nullptr;
    }
}

shv_cuda_model* shv_cuda_load(const char* weights, const char* mode, int device) {
    return shv_cuda_load_ex(weights, mode, device, nullptr);
}

void shv_cuda_free(shv_cuda_model* m) {
    if (!m) return;
    m->pipe->shutdown();
    delete m;
}

const char* shv_cuda_last_error(void) { return tls_error.c_str(); }
const char* shv_cuda_mode(const shv_cuda_model* m) { return m ? m->pipe->mode.c_str() : ""; }
const char* shv_cuda_fingerprint(const shv_cuda_model* m) { return m ? m->pipe->fingerprint.c_str() : ""; }
double shv_cuda_threshold(const shv_cuda_model* m) { return m ? m->pipe->threshold : std::nan(""); }
const char* shv_cuda_compute_revision(void) { return SHV_CUDA_REVISION; }
size_t shv_cuda_weight_bytes(const shv_cuda_model* m) { return m ? m->pipe->engine->weight_bytes() : 0; }
size_t shv_cuda_device_bytes(const shv_cuda_model* m) { return m ? m->pipe->device_bytes : 0; }

int shv_cuda_limits(const shv_cuda_model* m, int* max_frames, int* max_windows, int* max_host_tokens, int* token_slots) {
    if (!m) {
        tls_error = "null model";
        return -1;
    }
    const shv_cuda_options& o = m->pipe->opt;
    const int values[4] = {o.max_frames, o.max_windows, o.max_host_tokens, o.token_slots};
    int* outs[4] = {max_frames, max_windows, max_host_tokens, token_slots};
    for (int i = 0; i < 4; ++i)
        if (outs[i]) *outs[i] = values[i];
    return 0;
}

// half_tokens: the request's window_tokens point at fp16 token blocks (12,288 bytes each) instead of fp32 ones.
static shv_cuda_job* submit_request(shv_cuda_model* m, const shv_cuda_request* r, bool half_tokens) {
    try {
        if (!m || !r) throw ApiError("null argument");
        Pipeline& p = *m->pipe;
        const shv_cuda_options& o = p.opt;
        if (r->n_frames > size_t(o.max_frames)) throw ApiError("request has more frames than max_frames");
        if (r->n_windows > size_t(o.max_windows)) throw ApiError("request has more windows than max_windows");
        if (r->n_frames && !r->frames) throw ApiError("null frames");
        if (r->n_windows && !r->logits_out) throw ApiError("null logits_out");
        if (!r->n_frames && !r->n_windows) throw ApiError("empty request");

        std::unique_ptr<shv_cuda_job> job(new shv_cuda_job());
        job->crops = r->frames;
        job->n_crops = int(r->n_frames);
        job->tokens_out = r->n_frames ? r->tokens_out : nullptr;
        job->n_windows = int(r->n_windows);
        job->logits_out = r->logits_out;
        job->callback = r->callback;
        job->user = r->user;
        if (r->n_frames && r->store_slots) {
            if (!p.pool) throw ApiError("store_slots needs options.token_slots > 0");
            job->crop_slot.assign(r->store_slots, r->store_slots + r->n_frames);
            require_distinct_slots(job->crop_slot, o.token_slots, true);
        }
        // every window entry names exactly one source, in this order of precedence: frame, slot, host pointer
        std::vector<const float*> host;
        job->entries.reserve(r->n_windows * kWin);
        for (size_t e = 0; e < r->n_windows * kWin; ++e) {
            const int32_t frame = r->window_frames ? r->window_frames[e] : -1;
            const int32_t slot = r->window_slots ? r->window_slots[e] : -1;
            if (frame >= 0) {
                if (size_t(frame) >= r->n_frames) throw ApiError("window frame index out of range");
                job->entries.push_back(Entry{Src::Frame, frame});
            } else if (slot >= 0) {
                if (!p.pool || slot >= o.token_slots) throw ApiError("window slot out of range");
                job->entries.push_back(Entry{Src::Slot, slot});
            } else {
                const float* block = r->window_tokens ? r->window_tokens[e] : nullptr;
                if (!block) throw ApiError("window entry has no token source");
                job->entries.push_back(Entry{Src::Host, int32_t(host.size())});
                host.push_back(block);
            }
        }
        if (host.size() > size_t(o.max_host_tokens)) throw ApiError("request has more host token blocks than max_host_tokens");
        group_spans(*job, host, half_tokens);
        job->crops_pinned = is_pinned(r->frames, r->n_frames * kCropBytes);
        job->tokens_out_pinned = job->tokens_out && is_pinned(job->tokens_out, r->n_frames * kTokBytes);
        job->submitted = Clock::now();
        if (!p.accept(job.get())) throw ApiError("model is stopping");
        tls_error.clear();
        return job.release();
    } catch (const std::exception& e) {
        tls_error = e.what();
        return nullptr;
    }
}

shv_cuda_job* shv_cuda_submit(shv_cuda_model* m, const shv_cuda_request* r) { return submit_request(m, r, false); }

int shv_cuda_job_status(const shv_cuda_job* j) {
    if (!j) return -1;
    std::lock_guard<std::mutex> g(j->mu);
    return j->outcome;
}

int shv_cuda_job_wait(shv_cuda_job* j) {
    if (!j) {
        tls_error = "null job";
        return -1;
    }
    std::unique_lock<std::mutex> lk(j->mu);
    while (j->outcome == 0) j->cv.wait(lk);
    if (j->outcome > 0) return 0;
    tls_error = j->why;
    return -1;
}

const char* shv_cuda_job_error(const shv_cuda_job* j) {
    if (!j) return "null job";
    std::lock_guard<std::mutex> g(j->mu);
    return j->why.c_str();
}

int shv_cuda_job_timing(const shv_cuda_job* j, double* queue_ms, double* run_ms, double* gpu_ms, int* batch_frames, int* batch_windows) {
    if (!j) return -1;
    std::lock_guard<std::mutex> g(j->mu);
    if (j->outcome == 0) return 1;                               // still pending: nothing to report yet
    using Ms = std::chrono::duration<double, std::milli>;
    if (queue_ms) *queue_ms = Ms(j->started - j->submitted).count();
    if (run_ms) *run_ms = Ms(j->finished - j->started).count();
    if (gpu_ms) *gpu_ms = double(j->gpu_ms);
    if (batch_frames) *batch_frames = j->batch_crops;
    if (batch_windows) *batch_windows = j->batch_windows;
    return 0;
}

void shv_cuda_job_free(shv_cuda_job* j) {
    if (!j) return;
    {
        std::unique_lock<std::mutex> lk(j->mu);
        while (!j->settled) j->cv.wait(lk);
    }
    delete j;
}

void* shv_cuda_host_alloc(size_t bytes) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) == cudaSuccess) return p;
    cudaGetLastError();
    tls_error = "cudaHostAlloc failed";
    return nullptr;
}

void shv_cuda_host_free(void* p) {
    if (p) cudaFreeHost(p);
}

int shv_cuda_encode_frames(shv_cuda_model* m, const uint8_t* rgb, size_t n, float* tokens) {
    if (!m || (n && (!rgb || !tokens))) {
        tls_error = "null argument";
        return -1;
    }
    const size_t piece = size_t(m->pipe->opt.max_frames);
    return run_in_pieces(
        m, n, piece,
        [&](size_t first, size_t count, shv_cuda_request& r) {
            r.frames = rgb + first * kCropBytes;
            r.n_frames = count;
            r.tokens_out = tokens + first * kTokFloats;
        },
        [&] { std::fill(tokens, tokens + n * kTokFloats, kUnavailable); }, shv_cuda_submit);
}

int shv_cuda_predict(shv_cuda_model* m, const uint8_t* clips, size_t b, float* logits) {
    if (!m || (b && (!clips || !logits))) {
        tls_error = "null argument";
        return -1;
    }
    const shv_cuda_options& o = m->pipe->opt;
    const size_t piece = size_t(std::min(o.max_windows, o.max_frames / kWin));
    if (b && piece < 1) {
        tls_error = "predict needs max_frames >= 20";
        return -1;
    }
    std::vector<int32_t> own_frames(std::max<size_t>(piece, 1) * kWin);   // window w, position f -> frame w * 20 + f of the same request
    for (size_t e = 0; e < own_frames.size(); ++e) own_frames[e] = int32_t(e);
    return run_in_pieces(
        m, b, std::max<size_t>(piece, 1),
        [&](size_t first, size_t count, shv_cuda_request& r) {
            r.frames = clips + first * kWin * kCropBytes;
            r.n_frames = count * kWin;
            r.n_windows = count;
            r.window_frames = own_frames.data();
            r.logits_out = logits + first;
        },
        [&] { std::fill(logits, logits + b, kUnavailable); }, shv_cuda_submit);
}

// shv_cuda_classify over fp32 tokens (block_floats = 6144) or, for the extension below, fp16 tokens (block_floats = 3072:
// a block of 6144 halves measured in floats).
static int classify_blocks(shv_cuda_model* m, const float* tokens, size_t block_floats, bool half_tokens, size_t b, float* logits) {
    if (!m || (b && (!tokens || !logits))) {
        tls_error = "null argument";
        return -1;
    }
    const shv_cuda_options& o = m->pipe->opt;
    if (b && o.max_host_tokens < kWin) {
        tls_error = "classify needs max_host_tokens >= 20";
        return -1;
    }
    // Pieces of at most a batch, and small enough that a large call becomes a train of requests whose uploads overlap
    // the kernels of the requests before them (the feeder closes batches early while the pipeline is filling).
    const size_t fit = size_t(std::max(1, std::min(o.max_windows, o.max_host_tokens / kWin)));
    const size_t piece = std::min(fit, size_t(m->pipe->upload_windows()));
    std::vector<std::vector<const float*>> ptrs;                 // one pointer list per request, alive until the call returns
    ptrs.reserve((b + piece - 1) / piece + 1);
    return run_in_pieces(
        m, b, piece,
        [&](size_t first, size_t count, shv_cuda_request& r) {
            ptrs.emplace_back(count * kWin);
            std::vector<const float*>& list = ptrs.back();
            for (size_t e = 0; e < list.size(); ++e) list[e] = tokens + (first * kWin + e) * block_floats;
            r.n_windows = count;
            r.window_tokens = list.data();
            r.logits_out = logits + first;
        },
        [&] { std::fill(logits, logits + b, kUnavailable); },
        [&](shv_cuda_model* mm, const shv_cuda_request* rr) { return submit_request(mm, rr, half_tokens); });
}

int shv_cuda_classify(shv_cuda_model* m, const float* tokens, size_t b, float* logits) {
    return classify_blocks(m, tokens, kTokFloats, false, b, logits);
}

// ---------------------------------------------------------------- extensions (include/shv_cuda_b200.h)
int shv_cuda_b200_classify_f16(shv_cuda_model* m, const uint16_t* tokens_f16, size_t b, float* logits) {
    if (tokens_f16 && (reinterpret_cast<uintptr_t>(tokens_f16) & 15)) {
        tls_error = "fp16 tokens must be 16-byte aligned";
        return -1;
    }
    return classify_blocks(m, reinterpret_cast<const float*>(tokens_f16), kTokFloats / 2, true, b, logits);
}

int shv_cuda_b200_upload_tokens(shv_cuda_model* m, const float* tokens, size_t n, const int32_t* slots) {
    try {
        if (!m || (n && (!tokens || !slots))) throw ApiError("null argument");
        Pipeline& p = *m->pipe;
        if (!p.pool) throw ApiError("upload_tokens needs options.token_slots > 0");
        if (p.block_cap() < 1) throw ApiError("upload_tokens needs max_host_tokens >= 1");
        const size_t piece = size_t(p.block_cap());
        // validate everything before anything is queued: a bad slot must not leave half the upload done
        std::vector<std::unique_ptr<shv_cuda_job>> ready;
        for (size_t first = 0; first < n; first += piece) {
            const size_t count = std::min(piece, n - first);
            std::unique_ptr<shv_cuda_job> job(new shv_cuda_job());
            job->host_slot.assign(slots + first, slots + first + count);
            require_distinct_slots(job->host_slot, p.opt.token_slots, false);
            std::vector<const float*> blocks(count);
            for (size_t i = 0; i < count; ++i) blocks[i] = tokens + (first + i) * kTokFloats;
            group_spans(*job, blocks);
            ready.push_back(std::move(job));
        }
        std::vector<shv_cuda_job*> queued;
        for (std::unique_ptr<shv_cuda_job>& job : ready) {
            job->submitted = Clock::now();
            if (!p.accept(job.get())) {
                settle_all(queued);
                throw ApiError("model is stopping");
            }
            queued.push_back(job.release());
        }
        const int rc = settle_all(queued);
        if (rc == 0) tls_error.clear();
        return rc;
    } catch (const std::exception& e) {
        tls_error = e.what();
        return -1;
    }
}

int shv_cuda_b200_launches_per_batch(const shv_cuda_model* m) { return m ? m->pipe->engine->launches_per_classify() : 0; }

int shv_cuda_b200_test_starve(shv_cuda_model* m, int kind, int batches) {
#ifdef SHV_CUDA_EXPERIMENTAL
    try {
        if (!m) throw ApiError("null model");
        m->pipe->arm_starved_launch(kind, batches);
        return 0;
    } catch (const std::exception& e) {
        tls_error = e.what();
        return -1;
    }
#else
    (void)m; (void)kind; (void)batches;
    tls_error = "test hooks exist in the experimental library only";
    return -1;
#endif
}

}  // extern "C"
