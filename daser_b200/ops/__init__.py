"""ctypes bindings of the sm_100a kernels in ops/csrc (GEMM, attention, KV restore / save, elementwise)."""
