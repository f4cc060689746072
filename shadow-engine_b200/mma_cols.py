"""Many-row dense projections on the tensor pipe: the host mirror of `sz_mma_cols` (the reference's `mma_cols_<type>` launch,
crates/shadowzero-cuda/src/session.rs:7276, kernels/matvec.cu:1182)."""
import ctypes as C

import torch

from . import lib as szlib
from .model import Tensor

Q8_0 = 8


class MmaCols:
    """A Q8_0 matrix [rows][cols / 32 * 34 bytes] resident on the GPU, applied to many token rows at once."""

    def __init__(self, w_bytes, rows, cols, max_tokens, device="cuda"):
        self.lib = szlib.load()
        self.w = w_bytes.to(device=device, dtype=torch.uint8).contiguous().reshape(-1)
        assert self.w.numel() == rows * (cols // 32) * 34
        self.rows, self.cols, self.max_tokens = rows, cols, max_tokens
        self.t = Tensor(Q8_0, 0, self.w.data_ptr(), rows, cols)
        need = C.c_int64()
        szlib.check(self.lib.sz_mma_cols_scratch_bytes(cols, max_tokens, C.byref(need)))
        self.scratch = torch.empty(need.value, dtype=torch.uint8, device=device)
        self.stream = torch.cuda.current_stream().cuda_stream
        szlib.check(self.lib.sz_mma_cols_status(self.scratch.data_ptr(), 1, None, self.stream))

    def __call__(self, x, out=None):
        """x: float32 [m][cols] (row stride a multiple of 4 floats) -> float32 [m][rows]."""
        m = x.shape[0]
        assert m <= self.max_tokens and x.shape[1] == self.cols and x.dtype == torch.float32 and x.stride(1) == 1
        y = out if out is not None else torch.empty((m, self.rows), dtype=torch.float32, device=x.device)
        szlib.check(self.lib.sz_mma_cols(C.byref(self.t), x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), m, self.scratch.data_ptr(),
                                         self.scratch.numel(), torch.cuda.current_stream().cuda_stream))
        return y

    def status(self):
        """Synchronises; raises if a bounded wait of a kernel ran out since the scratch was cleared."""
        code = C.c_int()
        szlib.check(self.lib.sz_mma_cols_status(self.scratch.data_ptr(), 0, C.byref(code), torch.cuda.current_stream().cuda_stream))
        return code.value
