// Several GPUs of one box behind one object, in one process (include/shv_cuda_b200.h, shv_box_*).
//
// The reference's service engine owns exactly one GPU model and hands every session a block of 24 device token slots
// out of that model's pool (service/src/shield_av.cpp:824-850 load, :1013-1020 slot blocks, :556-577 submit;
// service/include/shield_av.h:205-211 cuda_device / max_sessions).  A box of N GPUs needs the same three things N
// times over and a rule that keeps a participant on one device, because its token ring lives there:
//   * one model per device, loaded concurrently, each with its own worker threads, streams and slot pool
//   * placement: CRC-32 of the participant id modulo the number of devices (the rule of
//     shield_sisa_b200/sharding.py device_of_participant); if that device's pool is exhausted, the device with the most
//     free blocks takes the session instead, so the box fills up completely before it refuses anyone
//   * requests of a session go to its device; whole batches of independent clips are cut into contiguous shards, one
//     per device, classified concurrently, and the logits land in the caller's array in clip order (host gather)
// No device ever reads another device's memory and nothing is exchanged between devices.
//
// The models are reached through a table of entry points (shv_box_ops).  The default table is this library's own
// shv_cuda_* functions; a test passes stand-ins and exercises placement, slot accounting and sharding without a GPU.
#include "shv_cuda_b200.h"

#include <algorithm>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

void shv_cuda_set_error(const std::string& s);     // api.cpp: the thread-local error string of the C ABI

namespace {

constexpr int kRing = 24;                          // token slots per session (the reference's NSLOT)

uint32_t crc32_ieee(const char* s) {               // reflected polynomial 0xEDB88320, as zlib.crc32
    static const std::vector<uint32_t> table = [] {
        std::vector<uint32_t> t(256);
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1u) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            t[i] = c;
        }
        return t;
    }();
    uint32_t c = 0xFFFFFFFFu;
    for (const unsigned char* p = reinterpret_cast<const unsigned char*>(s); *p; ++p) c = table[(c ^ *p) & 0xFFu] ^ (c >> 8);
    return c ^ 0xFFFFFFFFu;
}

const shv_box_ops kDefaultOps = {shv_cuda_load_ex, shv_cuda_free, shv_cuda_submit, shv_cuda_classify, shv_cuda_last_error};

struct DeviceSide {
    int ordinal = 0;
    shv_cuda_model* model = nullptr;
    std::vector<int> free_blocks;                  // indices of free 24-slot blocks, taken from the back
    std::string load_error;
};

}  // namespace

struct shv_box {
    shv_box_ops ops{};
    std::vector<DeviceSide> dev;
    int blocks_per_device = 0;
    std::mutex mu;                                 // guards the free lists
};

extern "C" {

shv_box* shv_box_load_with(const shv_box_ops* ops, const char* weights, const char* mode, const int* devices, int n_devices,
                           const shv_cuda_options* opt, int max_sessions) {
    try {
        if (!ops || !ops->load_ex || !ops->free_model || !ops->submit || !ops->classify || !ops->last_error)
            throw std::runtime_error("incomplete entry-point table");
        if (!devices || n_devices < 1 || n_devices > 64) throw std::runtime_error("a box has 1 to 64 devices");
        if (max_sessions < 0) throw std::runtime_error("max_sessions must not be negative");
        std::unique_ptr<shv_box> box(new shv_box());
        box->ops = *ops;
        box->dev.resize(size_t(n_devices));
        // every device can take its even share of the sessions plus a quarter: hashing does not spread them evenly
        const int share = (max_sessions + n_devices - 1) / n_devices;
        box->blocks_per_device = max_sessions ? std::min(max_sessions, share + share / 4 + 8) : 0;
        shv_cuda_options o;
        if (opt) o = *opt;
        else shv_cuda_default_options(&o);
        o.token_slots = box->blocks_per_device * kRing;
        std::vector<std::thread> loaders;
        for (int i = 0; i < n_devices; ++i) {
            DeviceSide& d = box->dev[size_t(i)];
            d.ordinal = devices[i];
            for (int b = box->blocks_per_device - 1; b >= 0; --b) d.free_blocks.push_back(b);
            loaders.emplace_back([&box, &d, weights, mode, o] {
                d.model = box->ops.load_ex(weights, mode, d.ordinal, &o);
                if (!d.model) d.load_error = box->ops.last_error();      // thread-local: read it on the loading thread
            });
        }
        for (std::thread& t : loaders) t.join();
        for (const DeviceSide& d : box->dev) {
            if (d.model) continue;
            const std::string why = "device " + std::to_string(d.ordinal) + ": " + d.load_error;
            for (DeviceSide& e : box->dev)
                if (e.model) box->ops.free_model(e.model);
            throw std::runtime_error(why);
        }
        shv_cuda_set_error("");
        return box.release();
    } catch (const std::exception& e) {
        shv_cuda_set_error(e.what());
        return nullptr;
    }
}

shv_box* shv_box_load(const char* weights, const char* mode, const int* devices, int n_devices, const shv_cuda_options* opt,
                      int max_sessions) {
    return shv_box_load_with(&kDefaultOps, weights, mode, devices, n_devices, opt, max_sessions);
}

void shv_box_free(shv_box* box) {
    if (!box) return;
    std::vector<std::thread> closers;                    // each model drains its own queue; do that side by side
    for (DeviceSide& d : box->dev)
        closers.emplace_back([box, &d] { box->ops.free_model(d.model); });
    for (std::thread& t : closers) t.join();
    delete box;
}

int shv_box_devices(const shv_box* box) { return box ? int(box->dev.size()) : 0; }

shv_cuda_model* shv_box_model(shv_box* box, int index) {
    return box && index >= 0 && index < int(box->dev.size()) ? box->dev[size_t(index)].model : nullptr;
}

int shv_box_home_device(const shv_box* box, const char* participant_id) {
    if (!box || !participant_id) return -1;
    return int(crc32_ieee(participant_id) % uint32_t(box->dev.size()));
}

int shv_box_session_open(shv_box* box, const char* participant_id, int* device_index, int* slot_base) {
    if (!box || !participant_id || !device_index || !slot_base) {
        shv_cuda_set_error("null argument");
        return -1;
    }
    std::lock_guard<std::mutex> g(box->mu);
    int pick = shv_box_home_device(box, participant_id);
    if (box->dev[size_t(pick)].free_blocks.empty()) {
        for (int i = 0; i < int(box->dev.size()); ++i)
            if (box->dev[size_t(i)].free_blocks.size() > box->dev[size_t(pick)].free_blocks.size()) pick = i;
    }
    DeviceSide& d = box->dev[size_t(pick)];
    if (d.free_blocks.empty()) {
        shv_cuda_set_error("max_sessions reached (device token slots)");
        return -1;
    }
    *device_index = pick;
    *slot_base = d.free_blocks.back() * kRing;
    d.free_blocks.pop_back();
    return 0;
}

int shv_box_session_close(shv_box* box, int device_index, int slot_base) {
    if (!box || device_index < 0 || device_index >= int(box->dev.size()) || slot_base < 0 || slot_base % kRing ||
        slot_base / kRing >= box->blocks_per_device) {
        shv_cuda_set_error("no such session block");
        return -1;
    }
    std::lock_guard<std::mutex> g(box->mu);
    std::vector<int>& fl = box->dev[size_t(device_index)].free_blocks;
    const int block = slot_base / kRing;
    if (std::find(fl.begin(), fl.end(), block) != fl.end()) {
        shv_cuda_set_error("session block is not in use");
        return -1;
    }
    fl.push_back(block);
    return 0;
}

int shv_box_free_sessions(shv_box* box, int device_index) {
    if (!box || device_index < 0 || device_index >= int(box->dev.size())) return -1;
    std::lock_guard<std::mutex> g(box->mu);
    return int(box->dev[size_t(device_index)].free_blocks.size());
}

shv_cuda_job* shv_box_submit(shv_box* box, int device_index, const shv_cuda_request* req) {
    if (!box || device_index < 0 || device_index >= int(box->dev.size())) {
        shv_cuda_set_error("no such device in this box");
        return nullptr;
    }
    return box->ops.submit(box->dev[size_t(device_index)].model, req);
}

int shv_box_classify(shv_box* box, const float* tokens, size_t b, float* logits) {
    if (!box || (b && (!tokens || !logits))) {
        shv_cuda_set_error("null argument");
        return -1;
    }
    const size_t n = box->dev.size();
    std::vector<int> rc(n, 0);
    std::vector<std::string> why(n);
    std::vector<std::thread> callers;
    // contiguous shards whose sizes differ by at most one clip, earlier devices take the extra one
    const size_t base = b / n, extra = b % n;
    size_t lo = 0;
    for (size_t i = 0; i < n; ++i) {
        const size_t count = base + (i < extra ? 1 : 0);
        if (count) {
            callers.emplace_back([box, i, lo, count, tokens, logits, &rc, &why] {
                rc[i] = box->ops.classify(box->dev[i].model, tokens + lo * SHV_CUDA_WINDOW_FRAMES * SHV_CUDA_TOKEN_FLOATS, count, logits + lo);
                if (rc[i]) why[i] = box->ops.last_error();
            });
        }
        lo += count;
    }
    for (std::thread& t : callers) t.join();
    for (size_t i = 0; i < n; ++i)
        if (rc[i]) {
            shv_cuda_set_error("device " + std::to_string(box->dev[i].ordinal) + ": " + why[i]);
            return -1;
        }
    return 0;
}

}  // extern "C"
