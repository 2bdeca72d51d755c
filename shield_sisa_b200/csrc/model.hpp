// Host-side description of a loaded SHIELD-V weight file, laid out for the sequence kernels.
//
// Mirrors the types the reference engine exposes to its callers (engine/cuda/model.hpp:10-18,44-70): the same
// dimension constants, the same fused projection layouts and `load_host_model`, so code written against the
// reference's internal engine API compiles against this one.  The frame-encoder (MobileNetV3) tensors are validated
// and kept verbatim in `cnn`; `fold_cnn` turns them into the folded, NHWC-ordered form the encoder kernels read.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace shv {

constexpr int IMG_H = 180, IMG_W = 320, FRAMES = 20, TOK_PER_FRAME = 16, D = 384, NTOK = 321;
constexpr int H = 6, DK = 64, DV = 128, VD = H * DV, DFF = 960, DSTATE = 32, NPAIR = DSTATE / 2;
constexpr int CNN_OUT = 960;
// Fused GDN input projection, one output row per column: [q 384 | k 384 | v 768 | gate 768 | a 6 | b 6], the
// projection output has row pitch GLD.
constexpr int GQ = 0, GK = 384, GV = 768, GG = 1536, GA = 2304, GB = 2310, GN = 2316, GLD = 2320;
// SISA all-row projection: [K 384 | V 384 | B 192 | theta 96 | alpha 6 | forget 6], row pitch SLD.
constexpr int SK = 0, SV = 384, SB = 768, ST_ = 960, SA = 1056, SF = 1062, SN = 1068, SLD = 1072;
// SISA readout-row projection: [Q 384 | C 192].
constexpr int SQ = 0, SC = 384, SQN = 576;

struct HostTensor {
    std::vector<int> shape;
    std::vector<float> data;
};

struct GdnHost {
    std::vector<float> norm_w, ffn_norm_w;   // [D]
    std::vector<float> in_w;                 // [GLD][D], rows GN..GLD-1 zero
    std::vector<float> conv_w, conv_b;       // [1536][4] and [1536]: q | k | v channels
    std::vector<float> a_log, dt_bias;       // [H]
    std::vector<float> o_norm_w;             // [DV]
    std::vector<float> o_proj;               // [D][VD]
    std::vector<float> ffn_up;               // [2*DFF][D]: row 2j = gate_j, row 2j+1 = up_j
    std::vector<float> ffn_down;             // [D][DFF]
};

struct SisaHost {
    std::vector<float> attn_norm_w, ffn_norm_w;  // [D]
    std::vector<float> w_all, b_all;             // [SLD][D], [SLD] (bias only under alpha and forget)
    std::vector<float> w_qc;                     // [SQN][D]
    std::vector<float> w_o;                      // [D][D]
    std::vector<float> lambda_raw;               // [H]
    std::vector<float> ffn_up, ffn_down;         // [2*DFF][D] interleaved, [D][DFF]
};

struct HostModel {
    std::string path, sha256;
    double threshold = 0.0;
    size_t file_bytes = 0;
    std::map<std::string, HostTensor> cnn;   // frame-encoder tensors by file name, shapes validated
    std::vector<float> proj;                 // [D][960] token projection (frame encoder tail)
    std::vector<float> pos;                  // [320][D] = (time[t] + row[r]) + col[c] for token t*16 + r*4 + c
    std::vector<float> readout;              // [D]
    GdnHost gdn_a, gdn_b;
    SisaHost sisa;
    std::vector<float> final_norm_w, head_w0 /*[128][D]*/, head_b0 /*[128]*/, head_w2 /*[128]*/, head_b2 /*[1]*/;
};

// MobileNetV3-Large frame encoder with BatchNorm (eps 1e-3) folded into each convolution in double precision
// (w' = w g / sqrt(var + eps), b' = beta - mean g / sqrt(var + eps)), as engine/cuda/model.cpp:56-91,182-214 does.
struct CnnBlock {
    int in = 0, k = 0, exp = 0, out = 0, stride = 1, act = 1;   // act: 1 ReLU, 2 Hardswish
    bool se = false, has_expand = false, residual = false;
    int h_in = 0, w_in = 0, h_out = 0, w_out = 0, cs = 0;       // cs: squeeze width, read from the file
    std::vector<float> exp_w, exp_b;      // [exp][in], [exp]
    std::vector<float> dw_w, dw_b;        // [k*k][exp] tap-major, [exp]
    std::vector<float> se_w1, se_b1;      // [cs][exp], [cs]
    std::vector<float> se_w2, se_b2;      // [exp][cs], [exp]
    std::vector<float> proj_w, proj_b;    // [out][exp], [out]
};
struct CnnHost {
    std::vector<float> lut;               // [3][256]: ((u / 255) - mean_c) / std_c, each step rounded to float32
    std::vector<float> stem_w, stem_b;    // [27][16] with index ((kh*3 + kw)*3 + ci)*16 + co, [16]
    CnnBlock blocks[15];
    std::vector<float> last_w, last_b;    // [960][160], [960]
};
CnnHost fold_cnn(const HostModel& hm);

// Reads and validates a SHLDV001 file: every tensor of the architecture present with its exact shape, all values
// finite, nothing else in the file; hashes the file; reads "threshold" (must lie in (0,1)) from "<path>.json".
// Throws std::runtime_error with the reason on any violation.
HostModel load_host_model(const std::string& path);

// "output_sha256" of "<weights>.json" must name this weight file (throws otherwise).
void check_sidecar_sha(const std::string& weights, const std::string& sha256);

// Quality certificate rule for the 16-bit modes: "<weights>.cuda.cert", first line SHIELDV_CUDA_CERT_V2, must hold a
// line "<sha256> <mode> <revision> PASS ... threshold=<%.17g>" whose threshold equals `threshold` exactly.
// Returns "" when such a line exists, else the reason.
std::string check_certificate(const std::string& weights, const std::string& sha256, const std::string& mode,
                              const std::string& revision, double threshold);

}  // namespace shv
