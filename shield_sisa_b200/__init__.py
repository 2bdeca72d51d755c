"""B200 (sm_100a) sequence engine of the SHIELD-V video detector: GatedDeltaNet + SISA stages behind the reference's
`shv_cuda_*` C ABI.

The product is the native library `lib/libshield_v_cuda.so` (C++17 host + hand-written CUDA); this package only
builds it (`build`), binds it with ctypes for tests and benchmarks (`binding`), writes synthetic weight files
(`weights`), splits work across the GPUs of a box (`sharding`) and drives streaming hops over device token rings (`live`).  There is no CPU fallback: every compute call
needs the native library and a CUDA device and raises if either is missing.
"""

__all__ = ["binding", "build", "live", "sharding", "weights"]
