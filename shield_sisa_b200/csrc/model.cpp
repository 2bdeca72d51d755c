// SHLDV001 reader and weight packing for the sequence engine.
//
// File format (reference tools/export_v.py:4-8): "SHLDV001", u32 tensor count, then per tensor: u32 name length,
// name, u32 rank, u32 dims[rank], u64 element count, float32 data; little endian.  Validation rules follow the
// reference loader (engine/cuda/model.cpp:137-179,278-279): bounded counts and sizes, finite values, no duplicate,
// missing or unexpected tensor, no trailing bytes.
// Compile without floating-point contraction: the position table must equal float32 (time + row) + col with two
// separate roundings (engine/cuda/model.cpp:216-227).
#include "model.hpp"
#include "sha256.hpp"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace shv {
namespace {

[[noreturn]] void fail(const std::string& why) { throw std::runtime_error(why); }

class TensorFile {
public:
    explicit TensorFile(const std::string& path) {
        std::ifstream in(path, std::ios::binary);
        if (!in) fail("cannot open weights: " + path);
        std::vector<char> bytes((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        size_ = bytes.size();
        Sha256 sha;
        sha.update(bytes.data(), bytes.size());
        digest_ = sha.hex();
        const char* p = bytes.data();
        const char* end = p + bytes.size();
        auto need = [&](size_t n, const char* what) {
            if (size_t(end - p) < n) fail(std::string("truncated weights (") + what + ")");
        };
        auto u32 = [&](const char* what) {
            need(4, what);
            uint32_t v;
            std::memcpy(&v, p, 4);
            p += 4;
            return v;
        };
        need(8, "magic");
        if (std::memcmp(p, "SHLDV001", 8) != 0) fail("not a SHLDV001 weight file: " + path);
        p += 8;
        const uint32_t count = u32("count");
        if (count == 0 || count > 10000) fail("invalid tensor count");
        uint64_t total = 0;
        for (uint32_t i = 0; i < count; ++i) {
            const uint32_t nlen = u32("name length");
            if (nlen == 0 || nlen > 4096) fail("invalid tensor name length");
            need(nlen, "name");
            std::string name(p, nlen);
            p += nlen;
            const uint32_t rank = u32("rank");
            if (rank > 8) fail("invalid tensor rank");
            HostTensor t;
            uint64_t elems = 1;
            for (uint32_t d = 0; d < rank; ++d) {
                const uint32_t dim = u32("dims");
                if (dim == 0 || dim > 10000000u || elems > 100000000ull / dim) fail("invalid tensor shape");
                t.shape.push_back(int(dim));
                elems *= dim;
            }
            need(8, "element count");
            uint64_t stated;
            std::memcpy(&stated, p, 8);
            p += 8;
            total += elems;
            if (stated != elems || total > 100000000ull) fail("invalid tensor size");
            need(elems * 4, "data");
            t.data.resize(elems);
            std::memcpy(t.data.data(), p, elems * 4);
            p += elems * 4;
            for (float v : t.data)
                if (!std::isfinite(v)) fail("non-finite value in tensor: " + name);
            if (!tensors_.emplace(name, std::move(t)).second) fail("duplicate tensor: " + name);
        }
        if (p != end) fail("trailing weight data");
    }

    // Takes the tensor out of the file map after checking its shape.
    std::vector<float> take(const std::string& name, std::initializer_list<int> shape) {
        auto it = tensors_.find(name);
        if (it == tensors_.end()) fail("missing tensor: " + name);
        if (it->second.shape != std::vector<int>(shape)) {
            std::ostringstream s;
            s << "bad shape for " << name << ": [";
            for (int d : it->second.shape) s << d << ",";
            s << "]";
            fail(s.str());
        }
        std::vector<float> out = std::move(it->second.data);
        tensors_.erase(it);
        return out;
    }
    HostTensor take_tensor(const std::string& name, std::initializer_list<int> shape) {
        HostTensor t;
        t.shape = shape;
        t.data = take(name, shape);
        return t;
    }
    const HostTensor* peek(const std::string& name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    void expect_empty() const {
        if (!tensors_.empty()) fail("unexpected tensor in weight file: " + tensors_.begin()->first);
    }
    const std::string& digest() const { return digest_; }
    size_t size() const { return size_; }

private:
    std::map<std::string, HostTensor> tensors_;
    std::string digest_;
    size_t size_ = 0;
};

std::string slurp(const std::string& path, const char* purpose) {
    std::ifstream in(path);
    if (!in) fail("cannot open " + path + purpose);
    std::stringstream ss;
    ss << in.rdbuf();
    return ss.str();
}

double sidecar_threshold(const std::string& json_path) {
    const std::string s = slurp(json_path, " (threshold)");
    const size_t key = s.find("\"threshold\"");
    if (key == std::string::npos) fail("no threshold in " + json_path);
    const size_t colon = s.find(':', key);
    if (colon == std::string::npos) fail("bad threshold in " + json_path);
    const double v = std::strtod(s.c_str() + colon + 1, nullptr);
    if (!(v > 0.0 && v < 1.0)) fail("threshold out of (0,1) in " + json_path);
    return v;
}

void place_rows(std::vector<float>& dst, int row0, const std::vector<float>& src) {
    std::memcpy(dst.data() + size_t(row0) * D, src.data(), src.size() * sizeof(float));
}

// rows (2j, 2j+1) = (gate_j, up_j): a SwiGLU pair lands in adjacent output columns of one GEMM
std::vector<float> pair_gate_up(const std::vector<float>& gate, const std::vector<float>& up) {
    std::vector<float> w(size_t(2) * DFF * D);
    for (int j = 0; j < DFF; ++j) {
        std::memcpy(&w[size_t(2 * j) * D], &gate[size_t(j) * D], D * sizeof(float));
        std::memcpy(&w[size_t(2 * j + 1) * D], &up[size_t(j) * D], D * sizeof(float));
    }
    return w;
}

GdnHost pack_gdn(TensorFile& f, const std::string& stage) {
    GdnHost g;
    const std::string m = stage + ".mixer.";
    g.norm_w = f.take(stage + ".norm.weight", {D});
    g.ffn_norm_w = f.take(stage + ".ffn_norm.weight", {D});
    g.in_w.assign(size_t(GLD) * D, 0.0f);
    place_rows(g.in_w, GQ, f.take(m + "q_proj.weight", {H * DK, D}));
    place_rows(g.in_w, GK, f.take(m + "k_proj.weight", {H * DK, D}));
    place_rows(g.in_w, GV, f.take(m + "v_proj.weight", {VD, D}));
    place_rows(g.in_w, GG, f.take(m + "g_proj.weight", {VD, D}));
    place_rows(g.in_w, GA, f.take(m + "a_proj.weight", {H, D}));
    place_rows(g.in_w, GB, f.take(m + "b_proj.weight", {H, D}));
    struct { const char* name; int width, first; } convs[3] = {{"q_conv1d", H * DK, 0}, {"k_conv1d", H * DK, 384}, {"v_conv1d", VD, 768}};
    g.conv_w.resize(size_t(1536) * 4);
    g.conv_b.resize(1536);
    for (const auto& c : convs) {
        const std::vector<float> w = f.take(m + c.name + ".weight", {c.width, 1, 4});
        const std::vector<float> b = f.take(m + c.name + ".bias", {c.width});
        std::memcpy(&g.conv_w[size_t(c.first) * 4], w.data(), w.size() * sizeof(float));
        std::memcpy(&g.conv_b[c.first], b.data(), b.size() * sizeof(float));
    }
    g.a_log = f.take(m + "A_log", {H});
    g.dt_bias = f.take(m + "dt_bias", {H});
    g.o_norm_w = f.take(m + "o_norm.weight", {DV});
    g.o_proj = f.take(m + "o_proj.weight", {D, VD});
    g.ffn_up = pair_gate_up(f.take(stage + ".ffn.gate.weight", {DFF, D}), f.take(stage + ".ffn.up.weight", {DFF, D}));
    g.ffn_down = f.take(stage + ".ffn.down.weight", {D, DFF});
    return g;
}

SisaHost pack_sisa(TensorFile& f) {
    SisaHost s;
    const std::string a = "sisa.attn.";
    s.attn_norm_w = f.take("sisa.attn_norm.weight", {D});
    s.w_all.assign(size_t(SLD) * D, 0.0f);
    s.b_all.assign(SLD, 0.0f);
    place_rows(s.w_all, SK, f.take(a + "W_K.weight", {D, D}));
    place_rows(s.w_all, SV, f.take(a + "W_V.weight", {D, D}));
    place_rows(s.w_all, SB, f.take(a + "W_B.weight", {H * DSTATE, D}));
    place_rows(s.w_all, ST_, f.take(a + "theta_proj.weight", {H * NPAIR, D}));
    place_rows(s.w_all, SA, f.take(a + "alpha_proj.weight", {H, D}));
    place_rows(s.w_all, SF, f.take(a + "forget_proj.weight", {H, D}));
    const std::vector<float> ab = f.take(a + "alpha_proj.bias", {H}), fb = f.take(a + "forget_proj.bias", {H});
    for (int i = 0; i < H; ++i) { s.b_all[SA + i] = ab[i]; s.b_all[SF + i] = fb[i]; }
    s.w_qc.assign(size_t(SQN) * D, 0.0f);
    place_rows(s.w_qc, SQ, f.take(a + "W_Q.weight", {D, D}));
    place_rows(s.w_qc, SC, f.take(a + "W_C.weight", {H * DSTATE, D}));
    s.w_o = f.take(a + "W_O.weight", {D, D});
    s.lambda_raw = f.take(a + "lambda_raw", {H});
    s.ffn_norm_w = f.take("sisa.ffn_norm.weight", {D});
    s.ffn_up = pair_gate_up(f.take("sisa.ffn.w_gate.weight", {DFF, D}), f.take("sisa.ffn.w_up.weight", {DFF, D}));
    s.ffn_down = f.take("sisa.ffn.w_down.weight", {D, DFF});
    return s;
}

// MobileNetV3-Large: validate names and shapes of the frame-encoder tensors and keep them verbatim.
void take_cnn(TensorFile& f, HostModel& hm) {
    struct Blk { int in, k, exp, out; bool se; };
    static const Blk blocks[15] = {
        {16, 3, 16, 16, false},   {16, 3, 64, 24, false},   {24, 3, 72, 24, false},  {24, 5, 72, 40, true},
        {40, 5, 120, 40, true},   {40, 5, 120, 40, true},   {40, 3, 240, 80, false}, {80, 3, 200, 80, false},
        {80, 3, 184, 80, false},  {80, 3, 184, 80, false},  {80, 3, 480, 112, true}, {112, 3, 672, 112, true},
        {112, 5, 672, 160, true}, {160, 5, 960, 160, true}, {160, 5, 960, 160, true}};
    auto conv_bn = [&](const std::string& pre, int out, int in, int k) {
        hm.cnn[pre + ".0.weight"] = f.take_tensor(pre + ".0.weight", {out, in, k, k});
        for (const char* leaf : {"weight", "bias", "running_mean", "running_var"})
            hm.cnn[pre + ".1." + leaf] = f.take_tensor(pre + ".1." + leaf, {out});
    };
    conv_bn("cnn.0", 16, 3, 3);
    for (int i = 0; i < 15; ++i) {
        const Blk& b = blocks[i];
        const std::string pre = "cnn." + std::to_string(i + 1) + ".block.";
        int idx = 0;
        if (b.exp != b.in) conv_bn(pre + std::to_string(idx++), b.exp, b.in, 1);
        conv_bn(pre + std::to_string(idx++), b.exp, 1, b.k);
        if (b.se) {
            const std::string se = pre + std::to_string(idx++);
            const HostTensor* fc1 = f.peek(se + ".fc1.weight");    // squeeze width comes from the file
            if (!fc1 || fc1->shape.size() != 4) fail("missing SE " + se);
            const int cs = fc1->shape[0];
            hm.cnn[se + ".fc1.weight"] = f.take_tensor(se + ".fc1.weight", {cs, b.exp, 1, 1});
            hm.cnn[se + ".fc1.bias"] = f.take_tensor(se + ".fc1.bias", {cs});
            hm.cnn[se + ".fc2.weight"] = f.take_tensor(se + ".fc2.weight", {b.exp, cs, 1, 1});
            hm.cnn[se + ".fc2.bias"] = f.take_tensor(se + ".fc2.bias", {b.exp});
        }
        conv_bn(pre + std::to_string(idx), b.out, b.exp, 1);
    }
    conv_bn("cnn.16", CNN_OUT, 160, 1);
}

}  // namespace

HostModel load_host_model(const std::string& path) {
    TensorFile f(path);
    HostModel hm;
    hm.path = path;
    hm.sha256 = f.digest();
    hm.file_bytes = f.size();
    hm.threshold = sidecar_threshold(path + ".json");

    take_cnn(f, hm);
    hm.proj = f.take("projection.weight", {D, CNN_OUT});

    const std::vector<float> te = f.take("time_embedding", {FRAMES, D}), re = f.take("row_embedding", {4, D}),
                             ce = f.take("col_embedding", {4, D});
    hm.pos.resize(size_t(320) * D);
    for (int t = 0; t < FRAMES; ++t)
        for (int r = 0; r < 4; ++r)
            for (int c = 0; c < 4; ++c)
                for (int j = 0; j < D; ++j) {
                    volatile float tr = te[size_t(t) * D + j] + re[size_t(r) * D + j];   // rounded before the second add
                    hm.pos[size_t(t * 16 + r * 4 + c) * D + j] = tr + ce[size_t(c) * D + j];
                }
    hm.readout = f.take("readout", {1, 1, D});
    hm.gdn_a = pack_gdn(f, "gdn_a");
    hm.gdn_b = pack_gdn(f, "gdn_b");
    hm.sisa = pack_sisa(f);
    hm.final_norm_w = f.take("final_norm.weight", {D});
    hm.head_w0 = f.take("head.0.weight", {128, D});
    hm.head_b0 = f.take("head.0.bias", {128});
    hm.head_w2 = f.take("head.2.weight", {1, 128});
    hm.head_b2 = f.take("head.2.bias", {1});
    f.expect_empty();
    return hm;
}

void check_sidecar_sha(const std::string& weights, const std::string& sha) {
    const std::string path = weights + ".json";
    const std::string s = slurp(path, "");
    std::string got;
    const size_t key = s.find("\"output_sha256\"");
    if (key != std::string::npos) {
        const size_t colon = s.find(':', key);
        const size_t q0 = colon == std::string::npos ? colon : s.find('"', colon + 1);
        const size_t q1 = q0 == std::string::npos ? q0 : s.find('"', q0 + 1);
        if (q1 != std::string::npos) got = s.substr(q0 + 1, q1 - q0 - 1);
    }
    if (got.empty()) fail("no output_sha256 in " + path + " (the sidecar must name its weight file)");
    if (got != sha)
        fail(path + " output_sha256 " + got + " does not match the weights' SHA-256 " + sha + " (sidecar of another export)");
}

std::string check_certificate(const std::string& weights, const std::string& sha, const std::string& mode,
                              const std::string& revision, double thr) {
    const std::string path = weights + ".cuda.cert";
    std::ifstream in(path);
    if (!in) return "mode " + mode + " needs a quality certificate: " + path + " not found";
    std::string line;
    if (!std::getline(in, line) || line != "SHIELDV_CUDA_CERT_V2")
        return "invalid certificate file " + path + " (expected SHIELDV_CUDA_CERT_V2; V1 lines do not bind the threshold)";
    bool other_threshold = false;
    double seen = std::nan("");
    while (std::getline(in, line)) {
        std::istringstream ls(line);
        std::string f_sha, f_mode, f_rev, verdict, tok;
        if (!(ls >> f_sha >> f_mode >> f_rev >> verdict)) continue;
        if (f_sha != sha || f_mode != mode || f_rev != revision || verdict != "PASS") continue;
        double t = std::nan("");
        while (ls >> tok)
            if (tok.compare(0, 10, "threshold=") == 0) {
                char* e = nullptr;
                const double v = std::strtod(tok.c_str() + 10, &e);
                if (e != tok.c_str() + 10 && *e == 0) t = v;
            }
        if (std::isfinite(t) && t == thr) return "";
        other_threshold = true;
        seen = t;
    }
    if (other_threshold) {
        char b[160];
        std::snprintf(b, sizeof b, "certified threshold %.17g, loaded threshold %.17g", seen, thr);
        return "mode " + mode + " certificate in " + path + " does not cover the threshold in " + weights + ".json (" + b + ")";
    }
    return "mode " + mode + " has no passing certificate for weights " + sha + " at compute revision " + revision + " in " + path;
}

// ---------------------------------------------------------------------------------------------------- frame encoder
namespace {

const std::vector<float>& cnn_tensor(const HostModel& hm, const std::string& name) {
    const auto it = hm.cnn.find(name);
    if (it == hm.cnn.end()) throw std::runtime_error("missing tensor " + name);
    return it->second.data;
}

// conv weight [out][per_out] followed by BatchNorm `bn`: scales the rows in place, returns the folded bias
std::vector<float> fold_batchnorm(const HostModel& hm, const std::string& bn, int out, int per_out, std::vector<float>& w) {
    const std::vector<float>&g = cnn_tensor(hm, bn + ".weight"), &beta = cnn_tensor(hm, bn + ".bias"),
                            &mean = cnn_tensor(hm, bn + ".running_mean"), &var = cnn_tensor(hm, bn + ".running_var");
    std::vector<float> b(size_t(out), 0.0f);
    for (int o = 0; o < out; ++o) {
        const double s = double(g[size_t(o)]) / std::sqrt(double(var[size_t(o)]) + 1e-3);
        for (int i = 0; i < per_out; ++i) {
            float& x = w[size_t(o) * per_out + i];
            x = float(double(x) * s);
        }
        b[size_t(o)] = float(double(beta[size_t(o)]) - double(mean[size_t(o)]) * s);
    }
    return b;
}

}  // namespace

CnnHost fold_cnn(const HostModel& hm) {
    struct Cfg { int in, k, exp, out; bool se; int act, stride; };
    static const Cfg table[15] = {
        {16, 3, 16, 16, false, 1, 1},   {16, 3, 64, 24, false, 1, 2},   {24, 3, 72, 24, false, 1, 1},
        {24, 5, 72, 40, true, 1, 2},    {40, 5, 120, 40, true, 1, 1},   {40, 5, 120, 40, true, 1, 1},
        {40, 3, 240, 80, false, 2, 2},  {80, 3, 200, 80, false, 2, 1},  {80, 3, 184, 80, false, 2, 1},
        {80, 3, 184, 80, false, 2, 1},  {80, 3, 480, 112, true, 2, 1},  {112, 3, 672, 112, true, 2, 1},
        {112, 5, 672, 160, true, 2, 2}, {160, 5, 960, 160, true, 2, 1}, {160, 5, 960, 160, true, 2, 1}};
    CnnHost c;
    // normalisation table: x = u / 255, y = x - mean, y / std, every step a float32 operation (prepare_clips of the
    // reference pipeline; engine/cuda/engine.cu:76-87)
    const float mean[3] = {0.485f, 0.456f, 0.406f}, stdv[3] = {0.229f, 0.224f, 0.225f};
    c.lut.resize(768);
    for (int ch = 0; ch < 3; ++ch)
        for (int u = 0; u < 256; ++u) {
            volatile float x = float(u) / 255.0f;
            volatile float y = x - mean[ch];
            c.lut[size_t(ch) * 256 + u] = y / stdv[ch];
        }
    {
        std::vector<float> w = cnn_tensor(hm, "cnn.0.0.weight");           // [16][3][3][3] = [co][ci][kh][kw]
        c.stem_b = fold_batchnorm(hm, "cnn.0.1", 16, 27, w);
        c.stem_w.resize(27 * 16);
        for (int co = 0; co < 16; ++co)
            for (int ci = 0; ci < 3; ++ci)
                for (int kh = 0; kh < 3; ++kh)
                    for (int kw = 0; kw < 3; ++kw)
                        c.stem_w[size_t(((kh * 3 + kw) * 3 + ci) * 16 + co)] = w[size_t(((co * 3 + ci) * 3 + kh) * 3 + kw)];
    }
    int h = 90, wd = 160;
    for (int i = 0; i < 15; ++i) {
        const Cfg& t = table[i];
        CnnBlock& b = c.blocks[i];
        b.in = t.in; b.k = t.k; b.exp = t.exp; b.out = t.out; b.se = t.se; b.act = t.act; b.stride = t.stride;
        b.has_expand = t.exp != t.in;
        b.residual = t.stride == 1 && t.in == t.out;
        const std::string pre = "cnn." + std::to_string(i + 1) + ".block.";
        int idx = 0;
        if (b.has_expand) {
            const std::string p = pre + std::to_string(idx++);
            b.exp_w = cnn_tensor(hm, p + ".0.weight");
            b.exp_b = fold_batchnorm(hm, p + ".1", t.exp, t.in, b.exp_w);
        }
        {
            const std::string p = pre + std::to_string(idx++);
            std::vector<float> w = cnn_tensor(hm, p + ".0.weight");        // [exp][1][k][k]
            b.dw_b = fold_batchnorm(hm, p + ".1", t.exp, t.k * t.k, w);
            b.dw_w.resize(size_t(t.k) * t.k * t.exp);
            for (int ch = 0; ch < t.exp; ++ch)
                for (int tap = 0; tap < t.k * t.k; ++tap) b.dw_w[size_t(tap) * t.exp + ch] = w[size_t(ch) * t.k * t.k + tap];
        }
        if (t.se) {
            const std::string p = pre + std::to_string(idx++);
            b.se_w1 = cnn_tensor(hm, p + ".fc1.weight");
            b.se_b1 = cnn_tensor(hm, p + ".fc1.bias");
            b.se_w2 = cnn_tensor(hm, p + ".fc2.weight");
            b.se_b2 = cnn_tensor(hm, p + ".fc2.bias");
            b.cs = int(b.se_b1.size());
        }
        {
            const std::string p = pre + std::to_string(idx);
            b.proj_w = cnn_tensor(hm, p + ".0.weight");
            b.proj_b = fold_batchnorm(hm, p + ".1", t.out, t.exp, b.proj_w);
        }
        b.h_in = h; b.w_in = wd;
        const int pad = (t.k - 1) / 2;
        h = (h + 2 * pad - t.k) / t.stride + 1;
        wd = (wd + 2 * pad - t.k) / t.stride + 1;
        b.h_out = h; b.w_out = wd;
    }
    if (h != 6 || wd != 10) throw std::runtime_error("unexpected frame-encoder output size");
    c.last_w = cnn_tensor(hm, "cnn.16.0.weight");
    c.last_b = fold_batchnorm(hm, "cnn.16.1", CNN_OUT, 160, c.last_w);
    return c;
}

}  // namespace shv
