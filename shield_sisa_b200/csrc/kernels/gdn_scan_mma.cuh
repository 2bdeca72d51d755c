// Internal: launcher of the tensor-core (chunked) GatedDeltaNet scan used by shvk_gdn_scan in the 16-bit modes.
#pragma once
#include <cuda_runtime.h>

namespace sb {
// on_dtype: DT_BF16 or DT_F16.  Returns a cudaError_t value.
int launch_gdn_scan_mma(const float* P, const float* conv_w, const float* conv_b, const float* a_log, const float* dt_bias,
                        const float* o_norm_w, void* on, int on_dtype, int B, cudaStream_t stream);
int gdn_scan_mma_status(int* status_out);
}  // namespace sb
