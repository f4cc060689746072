"""The MoE sublayer over many rows at once (`sz_moe_rows`): every row's output is bit for bit what the verify pass's `sz_moe_verify`
gives for it, the routing is the same, and it agrees with the CPU restatement of Session::moe."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

szlib, synth, moe = pkg.lib, pkg.synth, pkg.moe

pytestmark = pytest.mark.gpu


def layer(hidden, n_expert, top_k, ff, seed):
    ty = szlib.TYPE_EXL3(3)
    return synth.make_moe_layer(hidden, n_expert, top_k, ff, ff, ty, ty, seed=seed)


@pytest.mark.parametrize("hidden,n_expert,top_k,ff,rows", [(512, 16, 4, 256, 64), (512, 16, 4, 256, 8), (1024, 64, 6, 512, 256), (2048, 512, 10, 512, 256),
                                                            (2048, 512, 10, 512, 40)])
def test_rows_at_once_equal_rows_of_verify_passes(hidden, n_expert, top_k, ff, rows):
    L = layer(hidden, n_expert, top_k, ff, 7)
    ml = moe.MoeLayer(L, "cuda:0")
    x = synth.normal((rows, hidden), 1.0, 9, "rows.x").cuda()
    y, ridx, rw = ml.moe_rows(x, want_routing=True)
    assert ml.moe_rows_status(rows) == 0
    for c in range(0, rows, 8):
        yc, ic, wc = ml.moe_batch(x[c:c + 8].contiguous(), want_routing=True)
        assert torch.equal(ridx[c:c + 8], ic) and torch.equal(rw[c:c + 8], wc)
        assert torch.equal(y[c:c + 8].view(torch.int32), yc.view(torch.int32)), "rows %d.." % c
    # and a second call on the same scratch gives the same bits (accumulators and tickets are left clean)
    y2 = ml.moe_rows(x)
    assert torch.equal(y.view(torch.int32), y2.view(torch.int32))


def test_windows_as_block_rows_of_one_launch_equal_a_launch_pair_a_window(monkeypatch):
    """The expert kernels take all windows of a call as block rows of one launch; SZ_ROWS_SERIAL=1 launches them one after the
    other: the same bits, the same status."""
    L = layer(2048, 512, 10, 512, 17)
    ml = moe.MoeLayer(L, "cuda:0")
    x = synth.normal((96, 2048), 1.0, 19, "rows.x3").cuda()
    got = []
    for flag in ("0", "1"):
        monkeypatch.setenv("SZ_ROWS_SERIAL", flag)
        got.append(ml.moe_rows(x).clone())
        assert ml.moe_rows_status(96) == 0
    assert torch.equal(got[0].view(torch.int32), got[1].view(torch.int32))


def test_rows_at_once_against_the_cpu_restatement():
    hidden, n_expert, top_k, ff, rows = 512, 32, 4, 256, 24
    L = layer(hidden, n_expert, top_k, ff, 11)
    ml = moe.MoeLayer(L, "cuda:0")
    x = synth.normal((rows, hidden), 1.0, 13, "rows.x2")
    y, ridx, _ = ml.moe_rows(x.cuda(), want_routing=True)
    Ln = synth.to_numpy_layer(L)
    for j in range(rows):
        want, idx, _, _ = ob.moe(Ln, x[j].numpy(), threads=2)
        assert list(idx) == list(ridx[j].cpu().numpy())
        got = y[j].cpu().numpy()
        assert float(np.abs(got - want).max() / np.abs(want).max()) < 2e-4


def test_what_the_form_does_not_take_is_refused():
    L = synth.make_moe_layer(512, 16, 4, 256, 256, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=3)
    ml = moe.MoeLayer(L, "cuda:0")
    with pytest.raises(szlib.SzError):
        ml.moe_rows(torch.zeros((16, 512), device="cuda"))      # EXL3 experts only
    L2 = layer(512, 16, 4, 256, 5)
    ml2 = moe.MoeLayer(L2, "cuda:0")
    with pytest.raises(szlib.SzError):
        ml2.moe_rows(torch.zeros((12, 512), device="cuda"))     # a multiple of 8
