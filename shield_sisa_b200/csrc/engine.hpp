// Engine core: device-resident weights, activation arena, bucketed CUDA graphs, encode() and classify().
//
// Same internal C++ interface as the reference engine core (engine/cuda/engine.hpp:12-62): EngineConfig, the
// abstract Engine with encode / classify / slot / buckets / byte counters / set_dump_dir, and make_engine,
// parse_precision, precision_name.  A harness written against the reference's engine.hpp drives this engine as is.
// Difference: max_windows may exceed 4096 when the engine is used directly.
//
// NOT thread-safe: one thread drives an engine (the API worker).  Errors are std::runtime_error.
#pragma once
#include "model.hpp"

#include <cuda_runtime_api.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace shv {

enum class Precision { FP32 = 0, BF16 = 1, FP16 = 2 };

struct EngineConfig {
    int max_frames = 640;    // frames per batch whose tokens a slot can hold
    int max_windows = 512;   // windows per classify launch
    bool use_graphs = true;  // one CUDA graph per (slot, bucket); off for dumps and debugging
    int slots = 2;           // input/output buffer sets, so the scheduler can stage batch n+1 while n runs
    int max_host_blocks = -1;  // token blocks a slot's upload area holds (d_tok_stage); -1 = max_windows * 20
};

class Engine {
public:
    virtual ~Engine() = default;
    Precision precision() const { return prec_; }
    int max_frames() const { return cfg_.max_frames; }
    int max_windows() const { return cfg_.max_windows; }
    int slots() const { return cfg_.slots; }

    struct Slot {
        uint8_t* d_frames = nullptr;      // [max_frames][180][320][3] RGB crops to encode
        float* d_tokens = nullptr;        // [max_frames][16*384] tokens of encoded frames
        float* d_tok_stage = nullptr;     // [max_windows*20][16*384] tokens uploaded by the host
        const float** d_tokptr = nullptr; // [max_windows*20] device pointers to 16x384 token blocks
        float* d_logits = nullptr;        // [max_windows]
    };
    const Slot& slot(int i) const { return slots_[size_t(i)]; }

    // Enqueue on `s` and return without synchronising.  encode reads slot.d_frames[0 .. F) and writes the tokens of
    // frame f to slot.d_tokens + f*6144.  classify reads slot.d_tokptr[0 .. 20*B) and writes
    // slot.d_logits[0 .. B); with graphs on, B is padded to its bucket and the padding windows are computed from
    // whatever valid pointers the table holds, then ignored.
    virtual void encode(int slot, int F, cudaStream_t s) = 0;
    virtual void classify(int slot, int B, cudaStream_t s) = 0;
    int frame_bucket(int F) const;
    int window_bucket(int B) const;

    size_t weight_bytes() const { return weight_bytes_; }
    size_t activation_bytes() const { return act_bytes_; }
    size_t slot_bytes() const { return slot_bytes_; }
    // Debug: raw float32 intermediates of window 0 are written into dir by classify (graphs are bypassed).
    void set_dump_dir(const std::string& dir) { dump_dir_ = dir; }
    // Nonzero once a bounded wait inside a tensor-core kernel gave up; results of that batch are invalid.
    virtual int device_status() const = 0;
    // Test hook (16-bit modes): the next `batches` classify calls run eagerly and give one launch no input, so that its
    // bounded wait runs out, the kernel sets its status word and returns (kind 1: the tensor-core GEMM of the first
    // output projection, 2: the first scan).  Nothing faults or spins without bound; the batch's results are invalid.
    virtual void inject_wait_timeout(int kind, int batches) = 0;
    // Kernels launched by one classify of B windows (for launch accounting in benchmarks).
    virtual int launches_per_classify() const = 0;
    // One eager classify of B windows with a CUDA event after every launch: (kernel name, milliseconds) per launch,
    // in launch order.  Synchronises the stream.
    virtual std::vector<std::pair<std::string, float>> profile(int slot, int B, cudaStream_t s) = 0;
    // The same for one eager encode of F frames.
    virtual std::vector<std::pair<std::string, float>> profile_encode(int slot, int F, cudaStream_t s) = 0;
    virtual int launches_per_encode() const = 0;

protected:
    Precision prec_ = Precision::FP32;
    EngineConfig cfg_;
    std::vector<Slot> slots_;
    std::vector<int> fbuckets_, wbuckets_;
    size_t weight_bytes_ = 0, act_bytes_ = 0, slot_bytes_ = 0;
    std::string dump_dir_;
};

std::unique_ptr<Engine> make_engine(const HostModel& hm, Precision p, const EngineConfig& cfg);
const char* precision_name(Precision p);
bool parse_precision(const std::string& s, Precision* p);

}  // namespace shv
