"""Many-row dense projections on tcgen05 (`sz_mma_cols`) against the restated arithmetic of the reference's `mma_cols_<type>` family."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

szlib, synth, mc = pkg.lib, pkg.synth, pkg.mma_cols

pytestmark = pytest.mark.gpu


def make(rows, cols, seed):
    w = synth.normal((rows, cols), 0.02, seed, "mma_cols.w")
    return synth.quantize_q8_0(w)


@pytest.mark.parametrize("rows,cols,m", [(128, 256, 16), (128, 256, 1), (200, 512, 100), (512, 2048, 256), (384, 2048, 300), (96, 4096, 64),
                                         (1024, 2048, 700)])
def test_rows_of_many_tokens_match_the_f16_restatement(rows, cols, m):
    wb = make(rows, cols, 5)
    x = synth.normal((m, cols), 1.0, 7, "mma_cols.x")
    op = mc.MmaCols(wb, rows, cols, m)
    y = op(x.cuda())
    assert op.status() == 0
    want, mag = ob.mma_cols_q8(wb.numpy(), rows, cols, x.numpy())
    got = y.cpu().numpy().astype(np.float64)
    # f32 accumulation of `cols` products: each partial sum is off by at most 2^-23 of the magnitudes summed so far
    bound = cols * 2.0 ** -23 * mag + 1e-30
    worst = float(np.max(np.abs(got - want) / bound))
    assert worst < 1.0, "distance / bound = %g" % worst
    # and against the exact f32 weights and inputs the mode is the reference's "inexact" one: about 1e-3 of the magnitudes
    exact = x.numpy().astype(np.float64) @ ob.dequant(ob.Q8_0, wb.numpy()).reshape(rows, cols).astype(np.float64).T
    assert float(np.max(np.abs(got - exact) / mag)) < 2e-3


def test_strided_rows_and_a_second_call_reuse_the_scratch():
    rows, cols, m = 256, 1024, 40
    wb = make(rows, cols, 11)
    xbig = synth.normal((m, cols + 64), 1.0, 13, "mma_cols.xs").cuda()
    x = xbig[:, :cols]                                 # row stride cols + 64 floats
    ybig = torch.full((m, rows + 32), -7.0, device="cuda")
    op = mc.MmaCols(wb, rows, cols, 64)
    op(x, out=ybig[:, :rows])
    a = ybig[:, :rows].clone()
    assert bool((ybig[:, rows:] == -7.0).all())        # nothing written past the rows
    op(x[:9], out=ybig[:9, :rows])                     # fewer tokens: another tile width
    assert op.status() == 0
    assert torch.equal(ybig[:9, :rows], a[:9])         # a token's result does not depend on how many tokens share the tile
    want, mag = ob.mma_cols_q8(wb.numpy(), rows, cols, x.cpu().numpy())
    assert float(np.max(np.abs(a.cpu().numpy() - want) / (cols * 2.0 ** -23 * mag))) < 1.0


def test_arguments_are_checked():
    wb = make(128, 256, 3)
    op = mc.MmaCols(wb, 128, 256, 16)
    with pytest.raises(szlib.SzError):
        mc.MmaCols(make(128, 96, 3), 128, 96, 16)      # cols not a multiple of 256
    bad = pkg.model.Tensor(14, 0, op.w.data_ptr(), 128, 256)
    import ctypes as C
    rc = op.lib.sz_mma_cols(C.byref(bad), 256, 256, 256, 128, 1, op.scratch.data_ptr(), op.scratch.numel(), 0)
    assert rc == szlib.E_TYPE if hasattr(szlib, "E_TYPE") else rc != 0
