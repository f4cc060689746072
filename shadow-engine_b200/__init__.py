"""shadowzero_b200: B200 (sm_100a) kernels for ShadowZero's speculative-decoding verify step, behind a C ABI.

The product is `libshadowzero_b200.so` (sources in csrc/, interface in include/shadowzero_b200.h).  This package is the
thin Python host used by the tests and the benchmark: it loads the library through ctypes, keeps device memory in torch
tensors, and mirrors the reference's verify surface.  There is no CPU fallback: importing `lib` without the built
library raises.

The directory name has a hyphen, so load it with `__graft_entry__.load_package()`, which registers it as
`shadow_engine_b200`.
"""
from . import lib, moe, synth, model, ep, head, gguf_io, mma_cols  # noqa: F401
