"""sz_moe_verify_static: the entry point for hosts that cannot allocate scratch (an engine whose arena owns all device memory,
a plugin that may not call the CUDA allocator once running).  Its scratch is a fixed array inside the library, so the test
checks what such a host relies on: the same bytes as sz_moe_verify, call after call, and a clear refusal when a layer would
not fit.  The file sorts last so a run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

szlib, synth, moe = pkg.lib, pkg.synth, pkg.moe


def test_oversized_layers_are_refused_without_a_gpu():
    L = szlib.load()
    n = C.c_int64()
    szlib.check(L.sz_moe_static_scratch_max(C.byref(n)))
    assert n.value == 4 << 20
    c = szlib.MoeLayerC()
    for k, v in dict(hidden=4096, n_expert=64, top_k=16, expert_ff=1024, shared_ff=0, expert_type=szlib.TYPE_Q8_0,
                     shared_type=szlib.TYPE_Q8_0, router=4096, gate=4096, up=4096, down=4096, gate_stride=4096, up_stride=4096,
                     down_stride=4096).items():
        setattr(c, k, v)
    need = C.c_int64()
    szlib.check(L.sz_moe_scratch_bytes(C.byref(c), 8, C.byref(need)))
    assert need.value > n.value
    assert L.sz_moe_verify_static(C.byref(c), 4096, 8, 4096, 0, 0, 0) == szlib.E_SCRATCH
    assert b"4194304" in L.sz_last_error()


@pytest.mark.gpu
@pytest.mark.parametrize("ety,H,FF", [(szlib.TYPE_Q8_0, 512, 256), (szlib.TYPE_EXL3(3), 512, 256)])
def test_static_scratch_gives_the_same_bytes_twice_in_a_row(ety, H, FF):
    Ld = synth.make_moe_layer(H, 32, 4, FF, FF, ety, ety, seed=41)
    layer = moe.MoeLayer(Ld, "cuda:0")
    x = torch.randn(4, H, generator=torch.Generator().manual_seed(3)).cuda()
    want, widx, ww = layer.moe_batch(x, want_routing=True)   # the existing entry point, caller-provided scratch
    torch.cuda.synchronize()
    L = szlib.load()
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        y = torch.full_like(x, float("nan"))
        ridx = torch.full((4, 4), -1, dtype=torch.int32, device="cuda")
        rw = torch.zeros((4, 4), dtype=torch.float64, device="cuda")
        szlib.check(L.sz_moe_verify_static(C.byref(layer.c), x.data_ptr(), 4, y.data_ptr(), ridx.data_ptr(), rw.data_ptr(), st))
        torch.cuda.synchronize()
        assert torch.equal(ridx, widx) and torch.equal(rw, ww)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
        err = C.c_int(-1)
        szlib.check(L.sz_moe_static_status(C.byref(err), st))
        assert err.value == 0                      # no bounded wait ran out in the shared array's kernels
    # and against the CPU oracle directly, not only against the sibling entry point
    Ln = synth.to_numpy_layer(Ld)
    for j in range(4):
        ref, idx, _, _ = ob.moe(Ln, x[j].cpu().numpy(), threads=2)
        assert np.array_equal(idx, ridx[j].cpu().numpy())
        assert np.abs(y[j].cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-9) < 2e-4
    # the reset (after a failed call or a device reset) leaves the entry point usable with the same result
    szlib.check(L.sz_moe_static_reset())
    y2 = torch.full_like(x, float("nan"))
    szlib.check(L.sz_moe_verify_static(C.byref(layer.c), x.data_ptr(), 4, y2.data_ptr(), 0, 0, st))
    torch.cuda.synchronize()
    assert torch.equal(y2, y)
