// Reading and clearing the kernels' status words without stalling the device: both are enqueued on the caller's
// stream, so a scheduler fetches the words behind a batch's last kernel together with its logits and looks at them
// when the batch retires.
#include "shv_seq_kernels.h"
#include "status_words.cuh"

#include <cuda_runtime.h>

extern "C" int shvk_status_fetch_async(int* host_words, void* stream) {
    if (!host_words) return int(cudaErrorInvalidValue);
    int* words[SHVK_STATUS_WORDS] = {sb::gemm_tc_status_word(), sb::gdn_scan_status_word(), sb::gdn_scan_t_status_word()};
    for (int i = 0; i < SHVK_STATUS_WORDS; ++i) {
        if (!words[i]) return int(cudaErrorInvalidSymbol);
        const cudaError_t e = cudaMemcpyAsync(host_words + i, words[i], sizeof(int), cudaMemcpyDeviceToHost, cudaStream_t(stream));
        if (e != cudaSuccess) return int(e);
    }
    return 0;
}

extern "C" int shvk_status_clear_async(void* stream) {
    int* words[SHVK_STATUS_WORDS] = {sb::gemm_tc_status_word(), sb::gdn_scan_status_word(), sb::gdn_scan_t_status_word()};
    for (int i = 0; i < SHVK_STATUS_WORDS; ++i) {
        if (!words[i]) return int(cudaErrorInvalidSymbol);
        const cudaError_t e = cudaMemsetAsync(words[i], 0, sizeof(int), cudaStream_t(stream));
        if (e != cudaSuccess) return int(e);
    }
    return 0;
}
