// Internal: the per-device status words of the kernels whose waits are bounded.  A kernel whose wait on an mbarrier
// runs out sets its word (atomicCAS from 0) and returns; the host reads the words after a batch and fails the batch
// when one is set.  The words are per device and per process: every engine on a device shares them, so a wait that
// gives up in one engine fails the batches of all engines on that device that retire before the words are cleared.
#pragma once

namespace sb {
// Device address of each word on the current device, or nullptr if the lookup failed.  Looked up per call.
int* gemm_tc_status_word();        // gemm_tc.cu: 1 + role (producer, MMA issuer, epilogue) whose wait gave up
int* gdn_scan_status_word();       // gdn_scan.cu: 1 = wait for a chunk's TMA tiles
int* gdn_scan_t_status_word();     // gdn_scan_t.cu: 1 = wait for a chunk block
}  // namespace sb
