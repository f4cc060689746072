"""The output projection over an EXL3 output.weight (struct sz_head): the exact head, or the head screened by the 2-bit proxy."""
import ctypes as C

import numpy as np
import torch

from . import lib as szlib
from . import moe as szmoe


class Head:
    """`blob`: the EXL3 blob of output.weight (uint8, torch or numpy), [cols = hidden -> rows = vocabulary] at `bits` bits.
    k_blk = 0 evaluates every 128-output block; k_blk > 0 builds the proxy and keeps k_blk blocks a row of the pass."""

    def __init__(self, blob, rows, cols, bits, k_blk=0, device="cuda:0", stream=0):
        self.lib = szlib.load()
        self.device = torch.device(device)
        self.rows, self.cols, self.bits, self.k_blk = rows, cols, bits, k_blk
        self.stream = stream
        t = blob if isinstance(blob, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(blob, dtype=np.uint8))
        self._blob, addr, _ = szmoe.place(t.reshape(1, -1), self.device, 12)   # header = 2 (rows + cols) + 4 bytes: 4 mod 16
        h = szlib.HeadC(rows=rows, cols=cols, bits=bits, k_blk=k_blk, weight=addr)
        n = C.c_int64()
        szlib.check(self.lib.sz_head_work_bytes(rows, cols, k_blk, C.byref(n)))
        self._work = torch.empty(n.value + 256, dtype=torch.uint8, device=self.device)
        h.work = self._work.data_ptr() + (-self._work.data_ptr()) % 256
        h.work_bytes = n.value
        if k_blk > 0:
            q2, sc = C.c_int64(), C.c_int64()
            szlib.check(self.lib.sz_head_proxy_bytes(rows, cols, C.byref(q2), C.byref(sc)))
            self.w_q2 = torch.empty(q2.value, dtype=torch.uint8, device=self.device)
            self.w_sc = torch.empty(sc.value // 2, dtype=torch.int16, device=self.device)
            h.w_q2, h.w_sc = self.w_q2.data_ptr(), self.w_sc.data_ptr()
        self.c = h
        szlib.check(self.lib.sz_head_work_init(C.byref(h), stream))
        if k_blk > 0:
            szlib.check(self.lib.sz_head_proxy_build(C.byref(h), stream))
        torch.cuda.synchronize(self.device)

    def plan(self, m, need_k=64):
        ku, ms, ls = C.c_int32(), C.c_int32(), C.c_int64()
        szlib.check(self.lib.sz_head_plan(C.byref(self.c), m, need_k, C.byref(ku), C.byref(ms), C.byref(ls)))
        return ku.value, ms.value, ls.value

    def top(self, x, need_k=64):
        """x: float32 [m, cols] on the device.  Returns (top uint32 [m, 128] as numpy, logits float32 [m, stride] tensor)."""
        m = x.shape[0]
        _, _, ls = self.plan(m, need_k)
        logits = torch.zeros((m, ls), dtype=torch.float32, device=self.device)
        top = torch.zeros((m, 128), dtype=torch.int32, device=self.device)
        szlib.check(self.lib.sz_head_top(C.byref(self.c), x.data_ptr(), x.stride(0), m, need_k, logits.data_ptr(), top.data_ptr(),
                                         self.stream))
        torch.cuda.synchronize(self.device)
        return top.cpu().numpy().view(np.uint32), logits

    def stage(self, what, dtype):
        """An intermediate buffer of the last `top` as a numpy array of `dtype` (see SZ_HEAD_* in the header)."""
        addr, n = C.c_uint64(), C.c_int64()
        szlib.check(self.lib.sz_head_stage(C.byref(self.c), what, C.byref(addr), C.byref(n)))
        off = addr.value - self._work.data_ptr()
        return self._work[off:off + n.value].cpu().numpy().view(dtype)
