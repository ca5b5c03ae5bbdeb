"""zipage_b200 — B200 (sm_100a) kernels for Zipage's compressed-PagedAttention hot path.

`zipage_b200.kernel` mirrors the function names and arguments of the
reference's `zipage.kernel` package; every function launches hand-written CUDA
kernels through the C ABI of `libzipage_b200.so` (see include/zipage_b200.h).
"""
__version__ = "0.1.0"
