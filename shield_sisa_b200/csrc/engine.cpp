// Sequence engine core.  Launch order of one classify (B windows, M = 321*B rows), following the reference's
// run_classify (engine/cuda/engine.cu:406-470) with the memory-bound steps between GEMMs fused.
//
// 16-bit modes (24 launches):
//   assemble+norm -> h (fp32), xn
//   3 mixers (GDN-A once, GDN-B twice with the same weights, delta / sqrt(2)):
//       fused in-projection (W' xn^T on the tensor cores, conv + SiLU + gates in its epilogue) xn -> 16-bit operand tiles PT
//       | chunk preparation (per-chunk Gram products, masks, triangular inverse: the part of the chunked delta rule that
//       does not depend on the state) PT -> PT | scan (the state-dependent part, gated norm) PT -> on
//       | o-proj GEMM + residual -> h | norm h -> xn
//   2 FFNs: one kernel (up GEMM, SwiGLU into shared memory, down GEMM, residual) xn -> h | norm -> xn
//   SISA: all-row GEMM + bias -> K | V | B as fp16 rows, theta | alpha | forget as fp32 rows (both alias PT);
//       readout row: norm + Q/C projection, attention kernel, then W_O + residual, norm, FFN, head -> logits as one kernel.
// fp32 mode (28 launches): the same sequence with the in-projection as a GEMM writing P [M,2320] fp32 and the scan
//   reading it, the FFN as two GEMMs, S [M,1072] fp32; all-row GEMMs on the tensor cores with fp32 operands split into two
//   TF32 pieces each (the norm kernels write their rows already split, the other A operands are split by a launch of their
//   own).  Everything on the readout row is fp32 in every mode.
//
// encode (F frames, reference run_encode engine/cuda/engine.cu:338-403): stem -> 15 inverted-residual blocks
//   (expand 1x1 | depthwise | squeeze-excite gate | project 1x1 with the gate applied to its input rows, + residual)
//   -> 1x1 160 -> 960 -> 4x4 pooling -> 960 -> 384 token projection into slot.d_tokens.  float32 NHWC storage in every
//   mode; in the bf16 / fp16 modes the 1x1 convolutions round their operands to that type and multiply on the tensor cores.
//
// Storage policy (engine/cuda/engine.cu:150-164,213-219): h and the readout-row buffers are fp32 always; xn, on and the
// all-row weights are the storage type of the mode.  Departures in the 16-bit modes, all inside the 2e-2 tolerance and
// measured against the policy's own error: q, k, v, gate and the SISA K, V, B rows cross memory in 16 bits where the
// reference keeps fp32, and the FFN hidden layer does not cross memory at all.
#include "engine.hpp"
#include "shv_seq_kernels.h"
#include "shv_cnn_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>

namespace shv {

const char* precision_name(Precision p) {
    return p == Precision::FP32 ? "fp32" : p == Precision::BF16 ? "bf16" : p == Precision::FP16 ? "fp16" : "?";
}
bool parse_precision(const std::string& s, Precision* p) {
    for (Precision c : {Precision::FP32, Precision::BF16, Precision::FP16})
        if (s == precision_name(c)) { *p = c; return true; }
    return false;
}

namespace {

void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error ") + cudaGetErrorString(e) + " in " + what);
}
void launch_ok(int code, const char* what) { cuda_ok(cudaError_t(code), what); }

// Size classes a batch is padded to so that one captured graph serves a range of batch sizes: 1..6, then two steps
// per octave up to 16, four per octave above, capped by the configured maximum (which is always a class).
std::vector<int> size_classes(int maxv) {
    std::vector<int> out;
    for (int v : {1, 2, 3, 4, 5, 6, 8, 10, 12})
        if (v < maxv) out.push_back(v);
    for (int base = 16; base < maxv; base *= 2)
        for (int q = 4; q < 8; ++q) {
            const int v = base / 4 * q;
            if (v < maxv) out.push_back(v);
        }
    out.push_back(maxv);
    return out;
}
int class_of(const std::vector<int>& classes, int n) {
    for (int v : classes)
        if (v >= n) return v;
    throw std::runtime_error("batch larger than the configured maximum");
}

// Bump allocator over one device allocation, 256-byte granularity; `reserve` first, `commit` once, then `at`.
class Arena {
public:
    ~Arena() { if (base_) cudaFree(base_); }
    size_t reserve(size_t bytes) {
        const size_t off = size_;
        size_ = (size_ + bytes + 255) & ~size_t(255);
        return off;
    }
    void commit(const char* what) {
        cuda_ok(cudaMalloc(&base_, size_ ? size_ : 256), what);
        cuda_ok(cudaMemset(base_, 0, size_ ? size_ : 256), what);
    }
    template <typename U> U* at(size_t off) const { return reinterpret_cast<U*>(static_cast<uint8_t*>(base_) + off); }
    size_t size() const { return size_; }

private:
    void* base_ = nullptr;
    size_t size_ = 0;
};

int dtype_code(Precision p) { return p == Precision::FP32 ? SHVK_F32 : p == Precision::BF16 ? SHVK_BF16 : SHVK_F16; }
size_t dtype_bytes(Precision p) { return p == Precision::FP32 ? 4 : 2; }

// Exact tier: a weight matrix [rows][K] as the tensor-core GEMM's split operand [rows][hi | lo | hi], hi = w rounded
// to TF32 (10 mantissa bits, ties away), lo = w - hi (exact) rounded the same way.
float tf32_round(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return x;       // inf / nan stay
    u = (u + 0x1000u) & 0xffffe000u;
    std::memcpy(&x, &u, 4);
    return x;
}
std::vector<float> split_weight(const std::vector<float>& w, int K) {
    const size_t rows = w.size() / size_t(K);
    std::vector<float> out(rows * 3 * size_t(K));
    for (size_t r = 0; r < rows; ++r)
        for (int k = 0; k < K; ++k) {
            const float x = w[r * K + k], hi = tf32_round(x), lo = tf32_round(x - hi);
            float* o = &out[r * 3 * size_t(K)];
            o[k] = hi; o[K + k] = lo; o[2 * K + k] = hi;
        }
    return out;
}

std::vector<uint8_t> to_storage(const std::vector<float>& v, Precision p) {
    std::vector<uint8_t> out(v.size() * dtype_bytes(p));
    if (p == Precision::FP32) {
        std::memcpy(out.data(), v.data(), out.size());
    } else if (p == Precision::BF16) {
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(out.data());
        for (size_t i = 0; i < v.size(); ++i) d[i] = __float2bfloat16_rn(v[i]);
    } else {
        __half* d = reinterpret_cast<__half*>(out.data());
        for (size_t i = 0; i < v.size(); ++i) d[i] = __float2half_rn(v[i]);
    }
    return out;
}

struct GdnDev {
    const float *norm_w, *ffn_norm_w, *conv_w, *conv_b, *a_log, *dt_bias, *o_norm_w;
    const void *in_w, *o_proj, *ffn_up, *ffn_down;   // storage type
    const void* in_w_perm = nullptr;                 // 16-bit modes: in_w rows in the channel-tile order of the fused in-projection
};

struct CnnBlockDev {
    const float *exp_w = nullptr, *exp_b = nullptr, *dw_w = nullptr, *dw_b = nullptr, *se_w1 = nullptr, *se_b1 = nullptr;
    const float *se_w2 = nullptr, *se_b2 = nullptr, *proj_w = nullptr, *proj_b = nullptr;
};

// One all-row GEMM of the launch sequence: its argument block for the planned maximum row count and, in the 16-bit
// modes, the tensor-core plan (TMA maps) made once for these buffers.
struct Site {
    shvk_gemm_args args{};
    alignas(64) unsigned char plan[512];
    bool planned = false;
    const float* split_src = nullptr;    // exact tier: the fp32 A operand, split into args.A = [lo | hi] before every launch
};

class SeqEngine final : public Engine {
public:
    SeqEngine(const HostModel& hm, Precision p, const EngineConfig& cfg) {
        prec_ = p;
        cfg_ = cfg;
        if (cfg_.max_frames < 1 || cfg_.max_windows < 1 || cfg_.slots < 1 || cfg_.slots > 4)
            throw std::runtime_error("invalid engine configuration");
        if ((long long)cfg_.max_windows * NTOK > 0x7fffffffLL / 4) throw std::runtime_error("max_windows too large");
        if (cfg_.max_frames > 65535) throw std::runtime_error("max_frames too large");
        fbuckets_ = size_classes(cfg_.max_frames);
        wbuckets_ = size_classes(cfg_.max_windows);
        dt_ = dtype_code(p);
        cnn_ = fold_cnn(hm);
        upload(hm);
        allocate();
        plan_sites();
    }
    ~SeqEngine() override {
        for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
        if (capture_) cudaStreamDestroy(capture_);
    }

    void encode(int slot, int F, cudaStream_t s) override {
        if (F <= 0) return;
        if (slot < 0 || slot >= cfg_.slots) throw std::runtime_error("encode: bad slot");
        if (F > cfg_.max_frames) throw std::runtime_error("encode: too many frames");
        if (!cfg_.use_graphs || !dump_dir_.empty()) { run_encode(slot, F, s); return; }
        const int n = class_of(fbuckets_, F);
        launch_graph((1LL << 40) | ((long long)slot << 32) | (long long)n, s, [&](cudaStream_t cs) { run_encode(slot, n, cs); });
    }

    void classify(int slot, int B, cudaStream_t s) override {
        if (B <= 0) return;
        if (slot < 0 || slot >= cfg_.slots) throw std::runtime_error("classify: bad slot");
        if (B > cfg_.max_windows) throw std::runtime_error("classify: too many windows");
        if (starve_batches_ > 0) {                      // test hook: this batch runs eagerly with one starved launch
            --starve_batches_;
            run(slot, B, s, starve_kind_);
            return;
        }
        if (!cfg_.use_graphs || !dump_dir_.empty()) { run(slot, B, s); return; }
        const int n = class_of(wbuckets_, B);
        launch_graph(((long long)slot << 32) | (long long)n, s, [&](cudaStream_t cs) { run(slot, n, cs); });
    }

    int device_status() const override {
        int scan = 0, gemm = 0;
        if (shvk_gdn_scan_status(&scan) != 0) return -1;
        if (shvk_gemm_tc_status(&gemm) != 0) return -1;
        return scan ? 16 + scan : gemm;
    }
    void inject_wait_timeout(int kind, int batches) override {
        if (prec_ == Precision::FP32) throw std::runtime_error("the starved test launches exist for the 16-bit modes only");
        if (kind != 1 && kind != 2) throw std::runtime_error("starve kind: 1 = tensor-core GEMM, 2 = scan");
        starve_kind_ = kind;
        starve_batches_ = batches > 0 ? batches : 0;
    }
    // 16-bit modes: 24 kernels.  Exact tier: 23 (its feed-forward blocks are two GEMMs each) + a launch that splits the
    // A operand of the five GEMMs that do not read a normalised row (three o-projections, two FFN down projections)
    int launches_per_classify() const override { return prec_ == Precision::FP32 ? 28 : 24; }

    // One eager classify / encode with an event after every launch; returns (kernel name, milliseconds) per launch.
    std::vector<std::pair<std::string, float>> profile(int slot, int B, cudaStream_t s) override {
        if (B <= 0 || B > cfg_.max_windows || slot < 0 || slot >= cfg_.slots) throw std::runtime_error("profile: bad argument");
        return timed(s, [&] { run(slot, B, s); });
    }
    std::vector<std::pair<std::string, float>> profile_encode(int slot, int F, cudaStream_t s) override {
        if (F <= 0 || F > cfg_.max_frames || slot < 0 || slot >= cfg_.slots) throw std::runtime_error("profile: bad argument");
        return timed(s, [&] { run_encode(slot, F, s); });
    }
    int launches_per_encode() const override {
        int n = 4;                                       // stem, last conv, pooling, token projection
        for (const CnnBlock& b : cnn_.blocks) n += 2 + (b.has_expand ? 1 : 0) + (b.se ? 2 : 0);
        return n;
    }

private:
    int dt_ = SHVK_F32;
    Arena wts_, acts_;
    std::vector<std::unique_ptr<Arena>> slot_mem_;
    const float *pos_ = nullptr, *readout_ = nullptr;
    GdnDev gdn_[2]{};
    const float *s_attn_norm_ = nullptr, *s_b_all_ = nullptr, *s_lambda_ = nullptr;
    const float *s_ffn_norm_ = nullptr;
    const float *s_wqc_t_ = nullptr, *s_wo_t_ = nullptr, *s_up_t_ = nullptr, *s_down_t_ = nullptr;   // readout-row matrices, [K][N]
    const void* s_w_all_ = nullptr;
    const float *fn_w_ = nullptr, *h_w0t_ = nullptr, *h_b0_ = nullptr, *h_w2_ = nullptr, *h_b2_ = nullptr;
    // activations
    float *h_ = nullptr, *P_ = nullptr;
    void *xn_ = nullptr, *on_ = nullptr, *hid_ = nullptr;
    float* a2_ = nullptr;
    static constexpr int SB_COLS = 960, SG_LD = 112;    // SISA rows of the 16-bit modes: [K | V | B] fp16, [theta | alpha | forget | pad] fp32
    float *s16_ = nullptr, *sg_ = nullptr;
    float *qc_ = nullptr, *y_ = nullptr, *x2_ = nullptr;
    Site in_[2], oproj_[2], up_[2], down_[2], sisa_in_;
    alignas(64) unsigned char ffn_plan_[2][512];      // 16-bit modes: fused feed-forward block (TMA maps for xn, W_up, W_down)
    alignas(64) unsigned char inproj_plan_[2][512];   // 16-bit modes: fused in-projection (TMA maps for xn, W', PT = P_)
    int starve_kind_ = 0, starve_batches_ = 0;        // test hook: see inject_wait_timeout
    // frame encoder
    CnnHost cnn_;
    const float *lut_ = nullptr, *stem_w_ = nullptr, *stem_b_ = nullptr, *last_w_ = nullptr, *last_b_ = nullptr, *tokproj_ = nullptr;
    CnnBlockDev blk_[15];
    float *cx_ = nullptr, *ce_ = nullptr, *cd_ = nullptr, *se_part_ = nullptr, *se_gate_ = nullptr, *pooled_ = nullptr;
    std::map<long long, cudaGraphExec_t> graphs_;
    cudaStream_t capture_ = nullptr;
    cudaStream_t capture_stream() {
        if (!capture_) cuda_ok(cudaStreamCreateWithFlags(&capture_, cudaStreamNonBlocking), "capture stream");
        return capture_;
    }
    // Launches the graph stored under `key` into `s`, capturing `body` first if there is none yet.  Captured on a
    // stream the engine owns: the caller's stream may be the legacy default stream, which cannot be captured.
    template <typename Body> void launch_graph(long long key, cudaStream_t s, Body body) {
        auto it = graphs_.find(key);
        if (it == graphs_.end()) {
            cudaGraph_t g = nullptr;
            cudaStream_t cs = capture_stream();
            cuda_ok(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal), "graph capture");
            try {
                body(cs);
            } catch (...) {
                cudaStreamEndCapture(cs, &g);
                if (g) cudaGraphDestroy(g);
                throw;
            }
            cuda_ok(cudaStreamEndCapture(cs, &g), "graph capture");
            cudaGraphExec_t ex = nullptr;
            const cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
            cudaGraphDestroy(g);
            cuda_ok(e, "graph instantiate");
            it = graphs_.emplace(key, ex).first;
        }
        cuda_ok(cudaGraphLaunch(it->second, s), "graph launch");
    }
    std::vector<std::pair<std::string, cudaEvent_t>>* marks_ = nullptr;   // non-null only inside profile()

    template <typename Body> std::vector<std::pair<std::string, float>> timed(cudaStream_t s, Body body) {
        std::vector<std::pair<std::string, cudaEvent_t>> marks;
        cudaEvent_t t0 = nullptr;
        cuda_ok(cudaEventCreate(&t0), "event");
        cuda_ok(cudaEventRecord(t0, s), "event");
        marks_ = &marks;
        try {
            body();
        } catch (...) {
            marks_ = nullptr;
            for (auto& m : marks) cudaEventDestroy(m.second);
            cudaEventDestroy(t0);
            throw;
        }
        marks_ = nullptr;
        cuda_ok(cudaStreamSynchronize(s), "profile");
        std::vector<std::pair<std::string, float>> out;
        cudaEvent_t prev = t0;
        for (auto& m : marks) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, prev, m.second);
            out.emplace_back(m.first, ms);
            prev = m.second;
        }
        cudaEventDestroy(t0);
        for (auto& m : marks) cudaEventDestroy(m.second);
        return out;
    }

    void mark(const char* name, cudaStream_t s) {
        if (!marks_) return;
        cudaEvent_t e = nullptr;
        cuda_ok(cudaEventCreate(&e), "event");
        cuda_ok(cudaEventRecord(e, s), "event");
        marks_->emplace_back(name, e);
    }

    // ---------------------------------------------------------------- weights
    void upload(const HostModel& hm) {
        std::vector<uint8_t> host;
        struct Fix { const void** dst; size_t off; };
        std::vector<Fix> fixes;
        auto put = [&](const void** dst, const void* src, size_t bytes) {
            const size_t off = wts_.reserve(bytes);
            host.resize(wts_.size());
            std::memcpy(host.data() + off, src, bytes);
            fixes.push_back({dst, off});
        };
        auto f32 = [&](const float** dst, const std::vector<float>& v) {
            put(reinterpret_cast<const void**>(dst), v.data(), v.size() * 4);
        };
        auto stor = [&](const void** dst, const std::vector<float>& v) {
            const std::vector<uint8_t> b = to_storage(v, prec_);
            put(dst, b.data(), b.size());
        };
        f32(&pos_, hm.pos);
        f32(&readout_, hm.readout);
        const GdnHost* gh[2] = {&hm.gdn_a, &hm.gdn_b};
        for (int i = 0; i < 2; ++i) {
            GdnDev& g = gdn_[i];
            f32(&g.norm_w, gh[i]->norm_w); f32(&g.ffn_norm_w, gh[i]->ffn_norm_w);
            f32(&g.conv_w, gh[i]->conv_w); f32(&g.conv_b, gh[i]->conv_b);
            f32(&g.a_log, gh[i]->a_log); f32(&g.dt_bias, gh[i]->dt_bias); f32(&g.o_norm_w, gh[i]->o_norm_w);
            if (prec_ == Precision::FP32) {
                f32(reinterpret_cast<const float**>(&g.in_w), split_weight(gh[i]->in_w, D));
            } else {
                // rows of [q | k | v | gate | a | b] regrouped per head into the 128-row channel tiles of the fused
                // in-projection kernel; rows it does not use are zero
                const size_t perm_rows = size_t(shvk_gdn_inproj_rows());
                std::vector<int32_t> order(perm_rows, -1);
                shvk_gdn_inproj_row_order(order.data());
                std::vector<float> perm(order.size() * D, 0.0f);
                for (size_t r = 0; r < order.size(); ++r)
                    if (order[r] >= 0) std::memcpy(&perm[r * D], &gh[i]->in_w[size_t(order[r]) * D], D * sizeof(float));
                stor(&g.in_w_perm, perm);
            }
            if (prec_ == Precision::FP32) {
                f32(reinterpret_cast<const float**>(&g.o_proj), split_weight(gh[i]->o_proj, VD));
                f32(reinterpret_cast<const float**>(&g.ffn_up), split_weight(gh[i]->ffn_up, D));
                f32(reinterpret_cast<const float**>(&g.ffn_down), split_weight(gh[i]->ffn_down, DFF));
            } else {
                stor(&g.o_proj, gh[i]->o_proj);
                stor(&g.ffn_up, gh[i]->ffn_up); stor(&g.ffn_down, gh[i]->ffn_down);
            }
        }
        const SisaHost& sh = hm.sisa;
        f32(&s_attn_norm_, sh.attn_norm_w);
        if (prec_ == Precision::FP32) f32(reinterpret_cast<const float**>(&s_w_all_), split_weight(sh.w_all, D));
        else stor(&s_w_all_, sh.w_all);
        f32(&s_b_all_, sh.b_all); f32(&s_lambda_, sh.lambda_raw);
        f32(&s_ffn_norm_, sh.ffn_norm_w);
        // the readout-row kernels read their matrices column-wise across a warp: [K][N] copies
        auto transposed = [](const std::vector<float>& w, int n, int k) {
            std::vector<float> t(w.size());
            for (int r = 0; r < n; ++r)
                for (int c = 0; c < k; ++c) t[size_t(c) * n + r] = w[size_t(r) * k + c];
            return t;
        };
        f32(&s_wqc_t_, transposed(sh.w_qc, SQN, D)); f32(&s_wo_t_, transposed(sh.w_o, D, D));
        f32(&s_up_t_, transposed(sh.ffn_up, 2 * DFF, D)); f32(&s_down_t_, transposed(sh.ffn_down, D, DFF));
        f32(&fn_w_, hm.final_norm_w);
        std::vector<float> w0t(size_t(D) * 128);            // [D][128]: the head kernel reads consecutive outputs
        for (int o = 0; o < 128; ++o)
            for (int k = 0; k < D; ++k) w0t[size_t(k) * 128 + o] = hm.head_w0[size_t(o) * D + k];
        f32(&h_w0t_, w0t); f32(&h_b0_, hm.head_b0); f32(&h_w2_, hm.head_w2); f32(&h_b2_, hm.head_b2);
        f32(&lut_, cnn_.lut); f32(&stem_w_, cnn_.stem_w); f32(&stem_b_, cnn_.stem_b);
        for (int i = 0; i < 15; ++i) {
            const CnnBlock& b = cnn_.blocks[i];
            CnnBlockDev& d = blk_[i];
            if (b.has_expand) { f32(&d.exp_w, b.exp_w); f32(&d.exp_b, b.exp_b); }
            f32(&d.dw_w, b.dw_w); f32(&d.dw_b, b.dw_b);
            if (b.se) { f32(&d.se_w1, b.se_w1); f32(&d.se_b1, b.se_b1); f32(&d.se_w2, b.se_w2); f32(&d.se_b2, b.se_b2); }
            f32(&d.proj_w, b.proj_w); f32(&d.proj_b, b.proj_b);
        }
        f32(&last_w_, cnn_.last_w); f32(&last_b_, cnn_.last_b); f32(&tokproj_, hm.proj);
        wts_.commit("weight upload");
        cuda_ok(cudaMemcpy(wts_.at<void>(0), host.data(), host.size(), cudaMemcpyHostToDevice), "weight upload");
        for (const Fix& f : fixes) *f.dst = wts_.at<uint8_t>(f.off);
        weight_bytes_ = wts_.size();
    }

    // ---------------------------------------------------------------- buffers
    void allocate() {
        const size_t Bm = size_t(cfg_.max_windows), Mm = Bm * NTOK, Fm = size_t(cfg_.max_frames), ts = dtype_bytes(prec_);
        const size_t o_h = acts_.reserve(Mm * D * 4), o_p = acts_.reserve(Mm * GLD * 4), o_xn = acts_.reserve(prec_ == Precision::FP32 ? 256 : Mm * D * ts);   // exact tier: the norm kernels write into a2_
        // the hidden layer of the feed-forward blocks exists in memory only in the exact tier (the 16-bit modes keep it on the SM)
        const size_t o_on = acts_.reserve(Mm * VD * ts), o_hid = acts_.reserve(prec_ == Precision::FP32 ? Mm * DFF * ts : 0);
        const size_t o_qc = acts_.reserve(Bm * SQN * 4), o_y = acts_.reserve(Bm * D * 4), o_x2 = acts_.reserve(Bm * D * 4);
        // exact tier: the split A operand [lo | hi] of the GEMM about to run (widest: the FFN hidden layer)
        const size_t o_a2 = acts_.reserve(prec_ == Precision::FP32 ? Mm * 2 * DFF * 4 : 0);
        // frame encoder: block input / output X, expanded E, depthwise output Dd (largest layer of each kind), the
        // squeeze-excite partial sums and gates, the pooled map
        size_t x_fl = size_t(90) * 160 * 16, e_fl = size_t(60) * CNN_OUT, d_fl = 0, part_fl = 0;
        for (const CnnBlock& b : cnn_.blocks) {
            x_fl = std::max(x_fl, size_t(b.h_out) * b.w_out * b.out);
            if (b.has_expand) e_fl = std::max(e_fl, size_t(b.h_in) * b.w_in * b.exp);
            d_fl = std::max(d_fl, size_t(b.h_out) * b.w_out * b.exp);
            if (b.se) part_fl = std::max(part_fl, shvk_cnn_se_partial_floats(1, b.h_out * b.w_out, b.exp));
        }
        const size_t o_cx = acts_.reserve(Fm * x_fl * 4), o_ce = acts_.reserve(Fm * e_fl * 4), o_cd = acts_.reserve(Fm * d_fl * 4);
        const size_t o_sp = acts_.reserve(Fm * part_fl * 4), o_sg = acts_.reserve(Fm * CNN_OUT * 4);
        const size_t o_po = acts_.reserve(Fm * 16 * CNN_OUT * 4);
        acts_.commit("activation arena");
        cx_ = acts_.at<float>(o_cx); ce_ = acts_.at<float>(o_ce); cd_ = acts_.at<float>(o_cd);
        se_part_ = acts_.at<float>(o_sp); se_gate_ = acts_.at<float>(o_sg); pooled_ = acts_.at<float>(o_po);
        h_ = acts_.at<float>(o_h); P_ = acts_.at<float>(o_p);
        xn_ = acts_.at<void>(o_xn); on_ = acts_.at<void>(o_on);
        hid_ = prec_ == Precision::FP32 ? acts_.at<void>(o_hid) : nullptr;
        qc_ = acts_.at<float>(o_qc); y_ = acts_.at<float>(o_y); x2_ = acts_.at<float>(o_x2);
        a2_ = prec_ == Precision::FP32 ? acts_.at<float>(o_a2) : nullptr;
        act_bytes_ = acts_.size();

        slots_.resize(size_t(cfg_.slots));
        for (int i = 0; i < cfg_.slots; ++i) {
            slot_mem_.emplace_back(new Arena());
            Arena& a = *slot_mem_.back();
            const size_t o_frm = a.reserve(Fm * IMG_H * IMG_W * 3);
            const size_t stage_blocks = cfg_.max_host_blocks >= 0 ? size_t(std::max(cfg_.max_host_blocks, 1)) : Bm * FRAMES;
            const size_t o_tok = a.reserve(Fm * 16 * D * 4), o_stage = a.reserve(stage_blocks * 16 * D * 4);
            const size_t o_ptr = a.reserve(Bm * FRAMES * sizeof(float*)), o_log = a.reserve(Bm * 4);
            a.commit("slot buffers");
            Slot& sl = slots_[size_t(i)];
            sl.d_frames = a.at<uint8_t>(o_frm);
            sl.d_tokens = a.at<float>(o_tok);
            sl.d_tok_stage = a.at<float>(o_stage);
            sl.d_tokptr = a.at<const float*>(o_ptr);
            sl.d_logits = a.at<float>(o_log);
            // every table entry starts as a valid pointer: padding windows of a bucket dereference it
            std::vector<const float*> init(Bm * FRAMES, sl.d_tokens);
            cuda_ok(cudaMemcpy(sl.d_tokptr, init.data(), init.size() * sizeof(float*), cudaMemcpyHostToDevice), "slot init");
            slot_bytes_ = a.size();
        }
    }

    void make_site(Site& st, int N, int K, const void* A, const void* W, void* C, long long ldc, int c_dtype) {
        shvk_gemm_args& a = st.args;
        a.M = cfg_.max_windows * NTOK; a.N = N; a.K = K;
        a.A = A; a.lda = K; a.W = W; a.ldw = K;
        a.C = C; a.ldc = ldc; a.c_dtype = c_dtype;
        a.r_div = 1.0f;
        if (prec_ == Precision::FP32) {          // split operands: A = [lo | hi] in a2_, W = [hi | lo | hi]
            // the norm kernels write their rows into a2_ already split; the other operands are split by a launch of their own
            st.split_src = A == xn_ ? nullptr : static_cast<const float*>(A);
            a.A = a2_; a.lda = 2 * K; a.ldw = 3 * K;
        }
    }
    void plan_sites() {
        const float inv_div[2] = {1.0f, float(std::sqrt(2.0))};
        for (int i = 0; i < 2; ++i) {
            const GdnDev& g = gdn_[i];
            if (prec_ == Precision::FP32) make_site(in_[i], GN, D, xn_, g.in_w, P_, GLD, SHVK_F32);
            make_site(oproj_[i], D, VD, on_, g.o_proj, h_, D, SHVK_F32);
            oproj_[i].args.R = h_; oproj_[i].args.ldr = D; oproj_[i].args.r_div = inv_div[i];
            if (prec_ == Precision::FP32) {
                make_site(up_[i], 2 * DFF, D, xn_, g.ffn_up, hid_, DFF, dt_);
                up_[i].args.swiglu = 1;
                make_site(down_[i], D, DFF, hid_, g.ffn_down, h_, D, SHVK_F32);
                down_[i].args.R = h_; down_[i].args.ldr = D;
            }
        }
        make_site(sisa_in_, SN, D, xn_, s_w_all_, P_, SLD, SHVK_F32);
        sisa_in_.args.bias = s_b_all_;
        for (Site* st : {&oproj_[0], &oproj_[1]}) {
            launch_ok(shvk_gemm_tc_plan(&st->args, dt_, st->plan), "tensor-core GEMM plan");
            st->planned = true;
        }
        if (prec_ == Precision::FP32) {
            for (Site* st : {&up_[0], &up_[1], &down_[0], &down_[1]}) {
                launch_ok(shvk_gemm_tc_plan(&st->args, dt_, st->plan), "tensor-core GEMM plan");
                st->planned = true;
            }
            launch_ok(shvk_gemm_tc_plan(&sisa_in_.args, dt_, sisa_in_.plan), "tensor-core GEMM plan");
        } else {
            // 16-bit modes: K | V | B of the SISA projection leave as fp16 rows (S16), theta | alpha | forget as fp32 rows
            // (SG); both live where the mixers' operand tiles were
            s16_ = P_;
            sg_ = P_ + (size_t(cfg_.max_windows) * NTOK * SB_COLS / 2 + 3) / 4 * 4;     // halves -> floats, 16-byte aligned
            if ((sg_ - P_) + size_t(cfg_.max_windows) * NTOK * SG_LD > size_t(cfg_.max_windows) * NTOK * GLD)
                throw std::runtime_error("projection buffer too small for the SISA rows");
            sisa_in_.args.C = sg_; sisa_in_.args.ldc = SG_LD;
            launch_ok(shvk_gemm_tc_plan_split16(&sisa_in_.args, dt_, SB_COLS, s16_, SB_COLS, sisa_in_.plan), "tensor-core GEMM plan");
        }
        sisa_in_.planned = true;
        if (prec_ == Precision::FP32) {
            for (Site* st : {&in_[0], &in_[1]}) {
                launch_ok(shvk_gemm_tc_plan(&st->args, dt_, st->plan), "tensor-core GEMM plan");
                st->planned = true;
            }
            return;
        }
        // the chunk-blocked operand tiles of the in-projection live where the fp32 projection of the exact tier would
        if (shvk_gdn_pt_bytes(cfg_.max_windows) > size_t(cfg_.max_windows) * NTOK * GLD * 4)
            throw std::runtime_error("projection buffer too small for the operand tiles");
        for (int i = 0; i < 2; ++i)
            launch_ok(shvk_ffn_fused_plan(xn_, (long long)cfg_.max_windows * NTOK, gdn_[i].ffn_up, gdn_[i].ffn_down, h_, dt_, ffn_plan_[i]),
                      "feed-forward plan");
        for (int i = 0; i < 2; ++i)
            launch_ok(shvk_gdn_inproj_plan(xn_, (long long)cfg_.max_windows * NTOK, gdn_[i].in_w_perm, gdn_[i].conv_w, gdn_[i].conv_b,
                                           gdn_[i].a_log, gdn_[i].dt_bias, P_, dt_, inproj_plan_[i]), "in-projection plan");
    }
    void rows_gemm(const Site& st, int rows, cudaStream_t s) {
        if (st.planned) {
            if (st.split_src) {
                launch_ok(shvk_split_tf32(st.split_src, st.args.K, st.args.K, rows, a2_, 2 * st.args.K, 0, s), "operand split");
                mark("split_tf32", s);
            }
            launch_ok(shvk_gemm_tc_rows(st.plan, rows, s), "tensor-core GEMM");
        } else {
            shvk_gemm_args a = st.args;
            a.M = rows;
            launch_ok(shvk_gemm_f32(&a, s), "fp32 GEMM");
        }
    }
    // ---------------------------------------------------------------- debug dumps
    void dump(const char* name, const void* dev, size_t n, int dtype, cudaStream_t s) {
        if (dump_dir_.empty()) return;
        cuda_ok(cudaStreamSynchronize(s), "dump");
        std::vector<float> f(n);
        if (dtype == SHVK_F32) {
            cuda_ok(cudaMemcpy(f.data(), dev, n * 4, cudaMemcpyDeviceToHost), "dump");
        } else {
            std::vector<uint16_t> raw(n);
            cuda_ok(cudaMemcpy(raw.data(), dev, n * 2, cudaMemcpyDeviceToHost), "dump");
            for (size_t i = 0; i < n; ++i)
                f[i] = dtype == SHVK_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(raw.data())[i])
                                          : __half2float(reinterpret_cast<const __half*>(raw.data())[i]);
        }
        std::ofstream o(dump_dir_ + "/" + name + ".f32", std::ios::binary);
        o.write(reinterpret_cast<const char*>(f.data()), std::streamsize(n * 4));
    }

    // ---------------------------------------------------------------- frame encoder
    void run_encode(int slot, int F, cudaStream_t s) {
        const Slot& sl = slots_[size_t(slot)];
        // 1x1 convolutions: exact fma chains in fp32 mode, tensor-core products of operands rounded to the mode's 16-bit
        // type in the bf16 / fp16 modes
        const int ab = dt_;
        auto pointwise = [&](const float* A, const float* W, const float* b, const float* gate, int gate_rows, const float* R,
                             float* out, int M, int N, int K, int act, void* st) {
            if (prec_ == Precision::FP32) return shvk_cnn_pointwise(A, W, b, gate, gate_rows, R, out, M, N, K, act, st);
            return shvk_cnn_pointwise_h(A, W, b, gate, gate_rows, R, out, M, N, K, act, ab, st);
        };
        launch_ok(shvk_cnn_stem(sl.d_frames, lut_, stem_w_, stem_b_, cx_, F, s), "stem");
        mark("cnn.stem", s);
        dump("cnn_stem_f0", cx_, size_t(16) * 90 * 160, SHVK_F32, s);
        for (int i = 0; i < 15; ++i) {
            const CnnBlock& b = cnn_.blocks[i];
            const CnnBlockDev& d = blk_[i];
            const int hw_in = b.h_in * b.w_in, hw_out = b.h_out * b.w_out;
            const float* dw_in = cx_;
            if (b.has_expand) {
                launch_ok(pointwise(cx_, d.exp_w, d.exp_b, nullptr, 1, nullptr, ce_, F * hw_in, b.exp, b.in, b.act, s),
                          "expand");
                mark("cnn.expand", s);
                dw_in = ce_;
            }
            launch_ok(shvk_cnn_depthwise(dw_in, d.dw_w, d.dw_b, cd_, F, b.h_in, b.w_in, b.exp, b.k, b.stride, b.h_out, b.w_out,
                                         b.act, s), "depthwise");
            mark("cnn.depthwise", s);
            const float* gate = nullptr;
            if (b.se) {
                launch_ok(shvk_cnn_se_gate(cd_, se_part_, d.se_w1, d.se_b1, d.se_w2, d.se_b2, se_gate_, F, hw_out, b.exp, b.cs, s),
                          "squeeze-excite");
                mark("cnn.se_gate", s);
                gate = se_gate_;
            }
            launch_ok(pointwise(cd_, d.proj_w, d.proj_b, gate, hw_out, b.residual ? cx_ : nullptr, cx_, F * hw_out, b.out,
                                         b.exp, SHVK_ACT_NONE, s), "project");
            mark("cnn.project", s);
            if (!dump_dir_.empty()) {
                char name[32];
                std::snprintf(name, sizeof name, "cnn_block%02d_f0", i + 1);
                dump(name, cx_, size_t(b.out) * hw_out, SHVK_F32, s);
            }
        }
        launch_ok(pointwise(cx_, last_w_, last_b_, nullptr, 1, nullptr, ce_, F * 60, CNN_OUT, 160, SHVK_ACT_HSWISH, s),
                  "last conv");
        mark("cnn.last", s);
        dump("cnn_map_f0", ce_, size_t(60) * CNN_OUT, SHVK_F32, s);
        launch_ok(shvk_cnn_pool_tokens(ce_, pooled_, F, s), "pool");
        mark("cnn.pool", s);
        if (prec_ == Precision::FP32) {
            shvk_gemm_args a{};
            a.M = F * 16; a.N = D; a.K = CNN_OUT; a.A = pooled_; a.lda = CNN_OUT; a.W = tokproj_; a.ldw = CNN_OUT;
            a.C = sl.d_tokens; a.ldc = D; a.c_dtype = SHVK_F32; a.r_div = 1.0f;
            launch_ok(shvk_gemm_f32(&a, s), "token projection");
        } else {
            launch_ok(pointwise(pooled_, tokproj_, nullptr, nullptr, 1, nullptr, sl.d_tokens, F * 16, D, CNN_OUT, SHVK_ACT_NONE, s),
                      "token projection");
        }
        mark("cnn.token_proj", s);
        dump("tokens", sl.d_tokens, size_t(16) * D, SHVK_F32, s);
    }

    // ---------------------------------------------------------------- the launch sequence
    void run(int slot, int B, cudaStream_t s, int starve = 0) {
        const Slot& sl = slots_[size_t(slot)];
        const int M = B * NTOK;
        // exact tier: the normalised rows leave the norm kernels as the split A operand [lo | hi] of the GEMM that reads them
        void* const xn_out = prec_ == Precision::FP32 ? static_cast<void*>(a2_) : xn_;
        const int xn_code = prec_ == Precision::FP32 ? int(SHVK_F32_SPLIT) : dt_;
        const long long xn_ld = prec_ == Precision::FP32 ? 2 * D : D;
        launch_ok(shvk_assemble_norm(sl.d_tokptr, pos_, readout_, gdn_[0].norm_w, h_, xn_out, xn_code, B, s), "assemble");
        mark("assemble_norm", s);
        dump("h0", h_, size_t(NTOK) * D, SHVK_F32, s);
        for (int st = 0; st < 2; ++st) {
            const GdnDev& g = gdn_[st];
            const int reps = st == 0 ? 1 : 2;
            for (int r = 0; r < reps; ++r) {
                if (prec_ == Precision::FP32) {
                    rows_gemm(in_[st], M, s);
                    mark("gemm.in_proj", s);
                    launch_ok(shvk_gdn_scan(P_, g.conv_w, g.conv_b, g.a_log, g.dt_bias, g.o_norm_w, on_, dt_, B, s), "gdn scan");
                } else {
                    // projection + conv + SiLU + gates in one tensor-core kernel, bf16 operand tiles for the scan
                    launch_ok(shvk_gdn_inproj(inproj_plan_[st], B, s), "gdn in-projection");
                    mark("gdn_inproj", s);
                    // what the delta rule needs per chunk and that does not depend on the state, for all chunks at once
                    launch_ok(shvk_gdn_chunk_prep(P_, dt_, B, s), "gdn chunk preparation");
                    mark("gdn_prep", s);
                    if (starve == 2 && st == 0 && r == 0)
                        launch_ok(shvk_gdn_scan_t_starved(P_, g.o_norm_w, on_, dt_, B, 2048, s), "gdn scan (starved test launch)");
                    else
                        launch_ok(shvk_gdn_scan_t(P_, g.o_norm_w, on_, dt_, B, s), "gdn scan");
                }
                mark("gdn_scan", s);
                if (st == 0) dump("gdn_a.o_gated", on_, size_t(NTOK) * VD, dt_, s);
                if (starve == 1 && st == 0 && r == 0)
                    launch_ok(shvk_gemm_tc_rows_starved(oproj_[st].plan, M, 2048, s), "tensor-core GEMM (starved test launch)");
                else
                    rows_gemm(oproj_[st], M, s);
                mark("gemm.o_proj", s);
                const float* next_norm = r + 1 < reps ? g.norm_w : g.ffn_norm_w;
                launch_ok(shvk_rmsnorm(h_, D, next_norm, xn_out, xn_code, xn_ld, M, s), "rmsnorm");
                mark("rmsnorm", s);
            }
            if (prec_ == Precision::FP32) {
                rows_gemm(up_[st], M, s);
                mark("gemm.ffn_up", s);
                rows_gemm(down_[st], M, s);
                mark("gemm.ffn_down", s);
            } else {
                // up + SwiGLU + down + residual in one launch, the hidden layer staying on the SM
                launch_ok(shvk_ffn_fused(ffn_plan_[st], M, s), "feed-forward block");
                mark("ffn_fused", s);
            }
            dump(st == 0 ? "after_gdn_a" : "after_gdn_b", h_, size_t(NTOK) * D, SHVK_F32, s);
            const float* next_norm = st == 0 ? gdn_[1].norm_w : s_attn_norm_;
            launch_ok(shvk_rmsnorm(h_, D, next_norm, xn_out, xn_code, xn_ld, M, s), "rmsnorm");
            mark("rmsnorm", s);
        }
        float* S = P_;
        rows_gemm(sisa_in_, M, s);
        mark("gemm.sisa_in", s);
        const float* h_last = h_ + size_t(NTOK - 1) * D;
        const long long ld_last = (long long)NTOK * D;
        launch_ok(shvk_readout_qc(h_last, ld_last, s_attn_norm_, s_wqc_t_, qc_, B, s), "readout q / c");
        mark("readout.qc", s);
        if (prec_ == Precision::FP32) launch_ok(shvk_sisa_attn(S, qc_, s_lambda_, y_, B, s), "sisa attention");
        else launch_ok(shvk_sisa_attn_h16(s16_, sg_, qc_, s_lambda_, y_, B, s), "sisa attention");
        mark("sisa_attn", s);
        dump("sisa.y", y_, size_t(D), SHVK_F32, s);
        const shvk_readout_weights rw{s_wo_t_, s_ffn_norm_, s_up_t_, s_down_t_, fn_w_, h_w0t_, h_b0_, h_w2_, h_b2_};
        launch_ok(shvk_readout_tail(y_, h_last, ld_last, &rw, x2_, sl.d_logits, B, s), "readout tail");
        mark("readout.tail", s);
        dump("after_sisa_row", x2_, size_t(D), SHVK_F32, s);
        dump("logit", sl.d_logits, 1, SHVK_F32, s);
    }
};

}  // namespace

int Engine::frame_bucket(int F) const { return cfg_.use_graphs ? class_of(fbuckets_, F) : F; }
int Engine::window_bucket(int B) const { return cfg_.use_graphs ? class_of(wbuckets_, B) : B; }

std::unique_ptr<Engine> make_engine(const HostModel& hm, Precision p, const EngineConfig& cfg) {
    return std::unique_ptr<Engine>(new SeqEngine(hm, p, cfg));
}

}  // namespace shv
