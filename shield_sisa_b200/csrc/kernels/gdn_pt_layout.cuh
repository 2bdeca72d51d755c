// Layout of the chunk-blocked, transposed GDN projection ("PT") that the fused in-projection kernel (gdn_inproj.cu)
// writes and the 16-bit scan (gdn_scan_t.cu) reads.  Per clip and head the 321 tokens are padded to 21 chunks of 16;
// one chunk block is 13,696 contiguous bytes, so the scan fetches a chunk with a single bulk copy:
//
//   offset     0   q^T  [64 keys  ][16 tokens] 16-bit  silu(conv(q projection)), not yet L2-normalised   } the mode's type:
//           2048   k^T  [64 keys  ][16 tokens] 16-bit  silu(conv(k projection)), not yet L2-normalised   } bf16 or fp16
//           4096   v^T  [128 values][16 tokens] fp16   silu(conv(v projection))       } fp16 in both modes (saturating): read
//           8192   g^T  [128 values][16 tokens] fp16   silu(output-gate projection)   } element-wise only, combined in fp32
//          12288   log decay [16] fp32                -exp(A_log) * softplus(a + dt_bias)
//          12352   beta      [16] fp32                sigmoid(b)
//   added in place by the chunk preparation kernel (gdn_scan_t.cu) from the sections above; none of it depends on the
//   recurrent state, so it is computed for all chunks at once instead of inside the scan's serial walk:
//          12416   T2  [16][16] 16-bit   (I + L)^-1 diag(beta), L_ij = beta_i exp(c_i - c_j) k_i.k_j / (|k_i||k_j|) (j < i)
//          12928   M   [16][16] 16-bit   exp(c_i - c_j) q_i.k_j * 0.125 / |q_i| (j <= i)       } c = inclusive cumulative
//          13440   exp(c_i) [16] fp32, 13504 exp(c_16 - c_i) [16] fp32                          } log decay of the chunk
//          13568   1/|k_i| [16] fp32, 13632 0.125/|q_i| [16] fp32
//
// In the four bf16 tiles a row is 32 bytes = two halves of eight tokens; in rows 4-7 of every eight rows the halves
// trade places (tokens 8-15 first), which spreads the eight rows of one ldmatrix read over eight bank groups.
// Blocks are ordered [clip][head][chunk].  Token slots 321 .. 335 of a clip hold zeros in every section, which makes
// them inert in the recurrence (beta 0, no decay, zero keys and values) whatever the neighbouring clips contain.
#pragma once

namespace sb {
namespace pt {
constexpr int CHUNK = 16, NCHUNK = 21, TOK_PAD = CHUNK * NCHUNK;
constexpr int Q_OFF = 0, K_OFF = 2048, V_OFF = 4096, G_OFF = 8192, DEC_OFF = 12288, BETA_OFF = 12352;
constexpr int EXT_OFF = 12416, EXT_BYTES = 1280, BLOCK_BYTES = EXT_OFF + EXT_BYTES;
constexpr long long HEAD_BYTES = (long long)NCHUNK * BLOCK_BYTES, CLIP_BYTES = 6 * HEAD_BYTES;
static_assert(BLOCK_BYTES % 128 == 0, "chunk blocks stay 128-byte aligned");
}  // namespace pt
}  // namespace sb
