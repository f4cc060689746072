"""Device-side MoE layer: holds the weights in HBM in the layout the kernels want and calls sz_moe_verify.

Mirrors the MoE part of the reference's GPU session (GpuSession::moe_router_batch + moe_batch_resident,
crates/shadowzero-cuda/src/session.rs:7868-7871, 8222-8285): every expert of the layer resident, routing on the device.
"""
import ctypes as C

import torch

from . import lib as szlib


def _is_exl3(ty):
    return 1020 < ty <= 1028


def place(t, device, lead=0):
    """Copies the uint8 / float32 host tensor `t` ([count, bytes] or flat) to `device` with every row starting at an address
    that is `lead` mod 16 from a 16-byte boundary, rows padded to a multiple of 16 bytes.  Returns (buffer, address, stride).

    An EXL3 blob is placed with lead = 16 - (header bytes mod 16), so that its trellis starts on a 16-byte boundary."""
    raw = t.contiguous().view(torch.uint8)
    rows = raw.reshape(t.shape[0], -1) if t.dim() > 1 else raw.reshape(1, -1)
    n = rows.shape[1]
    stride = (n + 15) // 16 * 16
    buf = torch.zeros(rows.shape[0] * stride + 32, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 16 + lead
    view = buf[off:off + rows.shape[0] * stride].view(rows.shape[0], stride)
    view[:, :n] = rows.to(device)
    return buf, buf.data_ptr() + off, stride


class MoeLayer:
    """One MoE layer resident on a GPU.  `L` is the description `synth.make_moe_layer` returns (torch tensors)."""

    def __init__(self, L, device="cuda:0", max_rows=szlib.MAX_VERIFY, shard=None):
        """`shard` = (first, count, with_shared): hold only experts [first, first + count) of the layer (expert parallelism);
        `with_shared` says whether this rank adds the shared expert's term (exactly one rank of a group does)."""
        self.lib = szlib.load()
        self.device = torch.device(device)
        self.shape = {k: L[k] for k in ("hidden", "n_expert", "top_k", "expert_ff", "shared_ff", "expert_type", "shared_type")}
        H, FF, SF = L["hidden"], L["expert_ff"], L["shared_ff"]
        self._keep = []
        c = szlib.MoeLayerC()
        for k, v in self.shape.items():
            setattr(c, k, v)

        def lead(ty, n_in, n_out):
            return (16 - (2 * n_in + 2 * n_out + 4) % 16) % 16 if _is_exl3(ty) else 0

        def put(t, ld=0):
            buf, addr, stride = place(t, self.device, ld)
            self._keep.append(buf)
            return addr, stride

        lo, hi = 0, L["n_expert"]
        if shard is not None:
            lo, hi = shard[0], shard[0] + shard[1]
            assert 0 <= lo < hi <= L["n_expert"]
            c.ep_first, c.ep_count, c.ep_shared = lo, hi - lo, int(bool(shard[2]))
        self.shard = shard
        c.router, _ = put(L["router"].reshape(1, -1))
        c.gate, c.gate_stride = put(L["gate"][lo:hi], lead(L["expert_type"], H, FF))
        c.up, c.up_stride = put(L["up"][lo:hi], lead(L["expert_type"], H, FF))
        c.down, c.down_stride = put(L["down"][lo:hi], lead(L["expert_type"], FF, H))
        if SF > 0 and (shard is None or shard[2]):
            c.shared_router, _ = put(L["shared_router"].reshape(1, -1))
            c.sh_gate, _ = put(L["sh_gate"].reshape(1, -1), lead(L["shared_type"], H, SF))
            c.sh_up, _ = put(L["sh_up"].reshape(1, -1), lead(L["shared_type"], H, SF))
            c.sh_down, _ = put(L["sh_down"].reshape(1, -1), lead(L["shared_type"], SF, H))
        self.c = c
        self.max_rows = max_rows
        n = C.c_int64()
        szlib.check(self.lib.sz_moe_scratch_bytes(C.byref(c), max_rows, C.byref(n)))
        self.scratch_bytes = n.value
        self.scratch = torch.empty(n.value + 256, dtype=torch.uint8, device=self.device)
        self.scratch_addr = self.scratch.data_ptr() + (-self.scratch.data_ptr()) % 256
        szlib.check(self.lib.sz_moe_scratch_init(self.scratch_addr, self.scratch_bytes, torch.cuda.current_stream(self.device).cuda_stream))

    def launches(self):
        return self.lib.sz_moe_launches(C.byref(self.c))

    def moe_batch(self, x, y=None, want_routing=False, stream=None):
        """y[j] = moe(x[j]); x: float32 [m, hidden] on the device.  Returns y (and route_idx int32 [m, k], route_w f64 [m, k])."""
        m = x.shape[0]
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == self.shape["hidden"]
        if y is None:
            y = torch.empty_like(x)
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        if want_routing:
            ridx = torch.empty((m, self.shape["top_k"]), dtype=torch.int32, device=self.device)
            rw = torch.empty((m, self.shape["top_k"]), dtype=torch.float64, device=self.device)
            a, b = ridx.data_ptr(), rw.data_ptr()
        else:
            a = b = 0
        szlib.check(self.lib.sz_moe_verify(C.byref(self.c), x.data_ptr(), m, y.data_ptr(), a, b, self.scratch_addr,
                                           self.scratch_bytes, st))
        return (y, ridx, rw) if want_routing else y

    def moe_rows(self, x, y=None, want_routing=False, stream=None):
        """The sublayer over many rows at once (`sz_moe_rows`): x float32 [rows, hidden], rows a multiple of 8 up to 256; every
        distinct expert is decoded once for all the rows that chose it.  The scratch of this form is made at the first call."""
        rows = x.shape[0]
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == self.shape["hidden"]
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        have = getattr(self, "_rows_scratch", None)
        if have is None or have[0] < rows:
            n = C.c_int64()
            szlib.check(self.lib.sz_moe_rows_scratch_bytes(C.byref(self.c), rows, C.byref(n)))
            buf = torch.empty(n.value + 256, dtype=torch.uint8, device=self.device)
            addr = buf.data_ptr() + (-buf.data_ptr()) % 256
            szlib.check(self.lib.sz_moe_rows_status(C.byref(self.c), rows, addr, None, st))
            self._rows_scratch = have = (rows, buf, addr, n.value)
        if y is None:
            y = torch.empty_like(x)
        if want_routing:
            ridx = torch.empty((rows, self.shape["top_k"]), dtype=torch.int32, device=self.device)
            rw = torch.empty((rows, self.shape["top_k"]), dtype=torch.float64, device=self.device)
            a, b = ridx.data_ptr(), rw.data_ptr()
        else:
            a = b = 0
        if have[0] != rows:   # the layout depends on the row count: a smaller batch gets a scratch of its own size class
            n = C.c_int64()
            szlib.check(self.lib.sz_moe_rows_scratch_bytes(C.byref(self.c), rows, C.byref(n)))
            szlib.check(self.lib.sz_moe_rows_status(C.byref(self.c), rows, have[2], None, st))
            nbytes = n.value
        else:
            nbytes = have[3]
        szlib.check(self.lib.sz_moe_rows(C.byref(self.c), x.data_ptr(), rows, y.data_ptr(), a, b, have[2], nbytes, st))
        return (y, ridx, rw) if want_routing else y

    def moe_rows_status(self, rows, stream=None):
        """Synchronises; 0 unless a bounded wait ran out (1) or the routing needed more windows than the scratch has (2)."""
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        code = C.c_int()
        szlib.check(self.lib.sz_moe_rows_status(C.byref(self.c), rows, self._rows_scratch[2], C.byref(code), st))
        return code.value

    def moe_partial(self, x, y_fix=None, stream=None):
        """This rank's share of moe(x[j]) as 64-bit fixed point (int64 [m, hidden]); the shares of all ranks sum, as integers,
        to the layer's output, which `finish` converts to float32."""
        m = x.shape[0]
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == self.shape["hidden"]
        if y_fix is None:
            y_fix = torch.empty((m, self.shape["hidden"]), dtype=torch.int64, device=self.device)
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        szlib.check(self.lib.sz_moe_verify_partial(C.byref(self.c), x.data_ptr(), m, y_fix.data_ptr(), self.scratch_addr,
                                                   self.scratch_bytes, st))
        return y_fix

    def push_partial(self, x, stream=None):
        """With a peer exchange attached: this rank's share goes into every rank's exchange buffer."""
        m = x.shape[0]
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        szlib.check(self.lib.sz_moe_verify_partial(C.byref(self.c), x.data_ptr(), m, 0, self.scratch_addr, self.scratch_bytes, st))

    def finish_exchange(self, m, y=None, stream=None):
        if y is None:
            y = torch.empty((m, self.shape["hidden"]), dtype=torch.float32, device=self.device)
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        szlib.check(self.lib.sz_moe_finish_exchange(C.byref(self.c), m, y.data_ptr(), st))
        return y

    def finish(self, y_fix, y=None, stream=None):
        m, H = y_fix.shape
        if y is None:
            y = torch.empty((m, H), dtype=torch.float32, device=self.device)
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        szlib.check(self.lib.sz_moe_finish(y_fix.data_ptr(), m, H, y.data_ptr(), st))
        return y

    def moe_batch_host(self, x_host, y_host, x_dev, y_dev, stream=None):
        """The host-buffer entry point: x_host / y_host are (pinned) CPU float32 tensors [m, hidden]."""
        m = x_host.shape[0]
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        szlib.check(self.lib.sz_moe_verify_host(C.byref(self.c), x_host.data_ptr(), m, y_host.data_ptr(), None, None,
                                                x_dev.data_ptr(), y_dev.data_ptr(), self.scratch_addr, self.scratch_bytes, st))
        return y_host
