// Plain-C face of the engine core (include/shv_cuda_b200.h, shvb_engine_*): what the reference's kernel benchmark
// does in C++ against engine.hpp (bench/gpu_kbench.cu:55-103), callable from any language.
#include "shv_cuda_b200.h"
#include "engine.hpp"

#include <cstring>

// defined in api.cpp: the thread-local error string behind shv_cuda_last_error
void shv_cuda_set_error(const std::string& s);

struct shvb_engine {
    std::unique_ptr<shv::Engine> eng;
    int device = 0;
    std::vector<const float*> table;
};

namespace {
template <class F> int guard(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        shv_cuda_set_error(e.what());
        return -1;
    }
}
void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error ") + cudaGetErrorString(e) + " in " + what);
}
}  // namespace

extern "C" {

shvb_engine* shvb_engine_create(const char* weights, const char* mode, int device, int max_windows, int use_graphs) {
    return shvb_engine_create_ex(weights, mode, device, 1, max_windows, use_graphs);
}

shvb_engine* shvb_engine_create_ex(const char* weights, const char* mode, int device, int max_frames, int max_windows,
                                   int use_graphs) {
    shvb_engine* out = nullptr;
    guard([&] {
        if (!weights) throw std::runtime_error("null weights path");
        shv::Precision p;
        if (!shv::parse_precision(mode ? mode : "fp32", &p)) throw std::runtime_error("unknown mode (fp32, bf16, fp16)");
        cuda_ok(cudaSetDevice(device), "cudaSetDevice");
        const shv::HostModel hm = shv::load_host_model(weights);
        shv::check_sidecar_sha(weights, hm.sha256);
        shv::EngineConfig cfg;
        cfg.max_frames = max_frames;
        cfg.max_windows = max_windows;
        cfg.use_graphs = use_graphs != 0;
        cfg.slots = 2;
        auto e = std::unique_ptr<shvb_engine>(new shvb_engine());
        e->eng = shv::make_engine(hm, p, cfg);
        e->device = device;
        out = e.release();
    });
    return out;
}

void shvb_engine_destroy(shvb_engine* e) { delete e; }

int shvb_engine_bind_tokens(shvb_engine* e, int slot, const float* d_tokens, int B, void* stream) {
    return guard([&] {
        if (!e || !d_tokens || slot < 0 || slot >= e->eng->slots() || B < 1 || B > e->eng->max_windows())
            throw std::runtime_error("bind_tokens: bad argument");
        // With graphs on, classify pads B up to its size class and the padding windows read the table too: point them
        // at memory the engine owns, so that no entry outlives a buffer the caller bound earlier and has freed since.
        const int padded = e->eng->window_bucket(B);
        e->table.resize(size_t(padded) * 20);
        for (size_t i = 0; i < size_t(B) * 20; ++i) e->table[i] = d_tokens + i * SHV_CUDA_TOKEN_FLOATS;
        for (size_t i = size_t(B) * 20; i < e->table.size(); ++i) e->table[i] = e->eng->slot(slot).d_tokens;
        cuda_ok(cudaMemcpyAsync(e->eng->slot(slot).d_tokptr, e->table.data(), e->table.size() * sizeof(float*),
                                cudaMemcpyHostToDevice, cudaStream_t(stream)), "pointer table upload");
        cuda_ok(cudaStreamSynchronize(cudaStream_t(stream)), "pointer table upload");   // the host table is reused
    });
}

int shvb_engine_classify(shvb_engine* e, int slot, int B, void* stream) {
    return guard([&] {
        if (!e) throw std::runtime_error("null engine");
        e->eng->classify(slot, B, cudaStream_t(stream));
    });
}

float* shvb_engine_logits(shvb_engine* e, int slot) {
    return e && slot >= 0 && slot < e->eng->slots() ? e->eng->slot(slot).d_logits : nullptr;
}
int shvb_engine_read_logits(shvb_engine* e, int slot, float* host, int n, void* stream) {
    return guard([&] {
        if (!e || !host || slot < 0 || slot >= e->eng->slots() || n < 0 || n > e->eng->max_windows())
            throw std::runtime_error("read_logits: bad argument");
        cuda_ok(cudaStreamSynchronize(cudaStream_t(stream)), "read_logits");
        cuda_ok(cudaMemcpy(host, e->eng->slot(slot).d_logits, size_t(n) * 4, cudaMemcpyDeviceToHost), "read_logits");
    });
}
uint8_t* shvb_engine_frames(shvb_engine* e, int slot) {
    return e && slot >= 0 && slot < e->eng->slots() ? e->eng->slot(slot).d_frames : nullptr;
}
float* shvb_engine_tokens(shvb_engine* e, int slot) {
    return e && slot >= 0 && slot < e->eng->slots() ? e->eng->slot(slot).d_tokens : nullptr;
}
int shvb_engine_encode(shvb_engine* e, int slot, int F, void* stream) {
    return guard([&] {
        if (!e) throw std::runtime_error("null engine");
        e->eng->encode(slot, F, cudaStream_t(stream));
    });
}
int shvb_engine_frame_bucket(const shvb_engine* e, int F) {
    int out = -1;
    guard([&] { out = e ? e->eng->frame_bucket(F) : -1; });
    return out;
}
int shvb_engine_encode_launches(const shvb_engine* e) { return e ? e->eng->launches_per_encode() : 0; }
int shvb_engine_window_bucket(const shvb_engine* e, int B) {
    int out = -1;
    guard([&] { out = e ? e->eng->window_bucket(B) : -1; });
    return out;
}
int shvb_engine_launches(const shvb_engine* e) { return e ? e->eng->launches_per_classify() : 0; }
int shvb_engine_status(const shvb_engine* e) { return e ? e->eng->device_status() : -1; }
int shvb_engine_test_starve(shvb_engine* e, int kind, int batches) {
    return guard([&] {
        if (!e) throw std::runtime_error("null engine");
        e->eng->inject_wait_timeout(kind, batches);
    });
}
size_t shvb_engine_bytes(const shvb_engine* e, int which) {
    if (!e) return 0;
    return which == 0 ? e->eng->weight_bytes() : which == 1 ? e->eng->activation_bytes() : e->eng->slot_bytes();
}
namespace {
int profile_any(shvb_engine* e, bool encode, int slot, int n_items, void* stream, float* ms, int cap, char* names, int names_cap) {
    int n = -1;
    guard([&] {
        if (!e || !ms || !names || cap < 1 || names_cap < 1) throw std::runtime_error("profile: bad argument");
        const auto rows = encode ? e->eng->profile_encode(slot, n_items, cudaStream_t(stream))
                                 : e->eng->profile(slot, n_items, cudaStream_t(stream));
        std::string joined;
        for (size_t i = 0; i < rows.size(); ++i) {
            if (int(i) < cap) ms[i] = rows[i].second;
            joined += (i ? ";" : "") + rows[i].first;
        }
        std::strncpy(names, joined.c_str(), size_t(names_cap) - 1);
        names[names_cap - 1] = 0;
        n = int(rows.size());
    });
    return n;
}
}  // namespace
int shvb_engine_profile(shvb_engine* e, int slot, int B, void* stream, float* ms, int cap, char* names, int names_cap) {
    return profile_any(e, false, slot, B, stream, ms, cap, names, names_cap);
}
int shvb_engine_profile_encode(shvb_engine* e, int slot, int F, void* stream, float* ms, int cap, char* names, int names_cap) {
    return profile_any(e, true, slot, F, stream, ms, cap, names, names_cap);
}
int shvb_engine_set_dump_dir(shvb_engine* e, const char* dir) {
    return guard([&] {
        if (!e) throw std::runtime_error("null engine");
        e->eng->set_dump_dir(dir ? dir : "");
    });
}

}  // extern "C"
