"""The MoE verify step on the GPU against the CPU oracle (Session::moe, forward.rs:1009-1034): routing indices bit-exact,
routing weights to f64 rounding, outputs within the reference's own GPU-vs-CPU tolerance."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, synth, moe = pkg.lib, pkg.synth, pkg.moe

# |gpu - cpu| <= 1e-4 * sum|w x| + 1e-6 is the reference's matvec bound (crates/shadowzero-cuda/tests/matvec.rs:1-5); for a whole
# MoE layer the yardstick is the forward-pass one: relative error below 5e-3 with identical routing
# (crates/shadowzero/tests/reference.rs:57-66).  The f32-accumulating kernels are far inside it:
REL_TOL = 2e-4


def run_case(H, ne, k, FF, SF, ety, sty, m, seed=1, x_scale=1.0, router_sigma=None):
    L = synth.make_moe_layer(H, ne, k, FF, SF, ety, sty, seed=seed, router_sigma=router_sigma)
    layer = moe.MoeLayer(L, "cuda:0")
    g = torch.Generator().manual_seed(seed * 77 + m)
    x = (torch.randn(m, H, generator=g) * x_scale).to(torch.bfloat16).to(torch.float32)  # bf16 values, as the verify rows are
    y, ridx, rw = layer.moe_batch(x.cuda(), want_routing=True)
    torch.cuda.synchronize()
    y, ridx, rw = y.cpu().numpy(), ridx.cpu().numpy(), rw.cpu().numpy()
    Ln = synth.to_numpy_layer(L)
    worst = 0.0
    for j in range(m):
        want, idx, w, _ = ob.moe(Ln, x[j].numpy(), threads=4)
        assert np.array_equal(idx, ridx[j]), (j, idx, ridx[j])
        assert np.abs(w - rw[j]).max() < 1e-12
        scale = max(np.abs(want).max(), 1e-9)
        worst = max(worst, np.abs(y[j] - want).max() / scale)
    assert worst < REL_TOL, worst
    return layer, x, y


@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_q8_0_tiny_model_shapes(m):
    # benchmark config 1's MoE: hidden 512, 32 experts top-4, FF 256, shared FF 512, Q8_0
    run_case(512, 32, 4, 256, 512, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, m)


@pytest.mark.parametrize("m", [1, 4, 7])
def test_iq3_s_experts(m):
    run_case(512, 64, 6, 256, 256, szlib.TYPE_IQ3_S, szlib.TYPE_IQ3_S, m, seed=2)


@pytest.mark.parametrize("bits,m", [(3, 4), (3, 1), (2, 3), (4, 8)])
def test_exl3_experts(bits, m):
    run_case(256, 32, 4, 128, 256, szlib.TYPE_EXL3(bits), szlib.TYPE_EXL3(bits), m, seed=3)


@pytest.mark.parametrize("bits,ff,m", [(3, 512, 4), (3, 256, 1), (3, 128, 8), (2, 512, 3), (4, 512, 4), (4, 256, 5), (2, 128, 2)])
def test_exl3_streaming_kernels(bits, ff, m):
    # hidden a multiple of 512 and FF in {128, 256, 512} take the TMA-staged tensor-core kernels; the shared expert rides along
    run_case(512, 32, 4, ff, ff, szlib.TYPE_EXL3(bits), szlib.TYPE_EXL3(bits), m, seed=20 + bits)


def test_exl3_streaming_kernels_with_a_different_shared_expert():
    run_case(1024, 32, 6, 256, 512, szlib.TYPE_EXL3(3), szlib.TYPE_EXL3(3), 4, seed=31)   # other width: generic kernels for it
    run_case(512, 32, 6, 256, 256, szlib.TYPE_EXL3(3), szlib.TYPE_Q8_0, 4, seed=32)        # other type
    run_case(512, 32, 6, 256, 0, szlib.TYPE_EXL3(3), szlib.TYPE_EXL3(3), 7, seed=33)       # none


def test_exl3_streaming_kernels_all_rows_one_group():
    L = synth.make_moe_layer(512, 16, 4, 256, 256, szlib.TYPE_EXL3(3), szlib.TYPE_EXL3(3), seed=34)
    layer = moe.MoeLayer(L, "cuda:0")
    x = torch.randn(1, 512, generator=torch.Generator().manual_seed(1)).repeat(8, 1).contiguous()
    y = layer.moe_batch(x.cuda())
    torch.cuda.synchronize()
    want, _, _, _ = ob.moe(synth.to_numpy_layer(L), x[0].numpy())
    assert all(torch.equal(y[0], y[j]) for j in range(8))
    assert np.abs(y[0].cpu().numpy() - want).max() / np.abs(want).max() < REL_TOL


def test_mixed_types_exl3_experts_q8_shared():
    run_case(256, 16, 4, 128, 256, szlib.TYPE_EXL3(3), szlib.TYPE_Q8_0, 4, seed=4)


def test_no_shared_expert():
    run_case(256, 16, 2, 128, 0, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, 3, seed=5)


def test_every_row_picks_the_same_experts():
    # identical rows: every group holds all m rows (the grouped path's widest case)
    L = synth.make_moe_layer(256, 16, 4, 256, 256, szlib.TYPE_IQ3_S, szlib.TYPE_IQ3_S, seed=6)
    layer = moe.MoeLayer(L, "cuda:0")
    x = torch.randn(1, 256, generator=torch.Generator().manual_seed(1)).repeat(8, 1).contiguous()
    y, ridx, _ = layer.moe_batch(x.cuda(), want_routing=True)
    torch.cuda.synchronize()
    want, idx, _, _ = ob.moe(synth.to_numpy_layer(L), x[0].numpy())
    assert all(np.array_equal(ridx[j].cpu().numpy(), idx) for j in range(8))
    assert all(torch.equal(y[0], y[j]) for j in range(8))
    assert np.abs(y[0].cpu().numpy() - want).max() / np.abs(want).max() < REL_TOL


def test_router_ties_go_to_the_lower_index():
    # duplicate router rows give exactly equal logits: the lower expert index wins, as route_into orders them
    L = synth.make_moe_layer(256, 16, 4, 128, 0, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=8)
    L["router"][5] = L["router"][2]
    L["router"][9] = L["router"][2]
    L["router"][2] *= 0
    L["router"][5] *= 0
    L["router"][9] *= 0   # three zero logits, tied; make the others negative for the test row
    layer = moe.MoeLayer(L, "cuda:0")
    x = torch.randn(2, 256, generator=torch.Generator().manual_seed(2))
    _, ridx, rw = layer.moe_batch(x.cuda(), want_routing=True)
    torch.cuda.synchronize()
    Ln = synth.to_numpy_layer(L)
    for j in range(2):
        _, idx, w, _ = ob.moe(Ln, x[j].numpy())
        assert np.array_equal(idx, ridx[j].cpu().numpy())
        got = list(ridx[j].cpu().numpy())
        tied = [e for e in got if e in (2, 5, 9)]
        assert tied == sorted(tied)


@pytest.mark.parametrize("ety", [szlib.TYPE_IQ3_S, szlib.TYPE_EXL3(3)])
def test_repeated_calls_are_deterministic_and_scratch_is_reusable(ety):
    # bit-identical from call to call: the streaming kernels add partial sums with integer atomics, whose order does not matter
    layer, x, y0 = run_case(512, 64, 6, 256, 256, ety, ety, 4, seed=9)
    xd = x.cuda()
    for _ in range(5):
        y = layer.moe_batch(xd)
        torch.cuda.synchronize()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), y0.view(np.uint32))


def test_host_buffer_entry_point_matches_the_device_one():
    layer, x, y0 = run_case(256, 16, 4, 128, 256, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, 4, seed=10)
    xh = x.clone().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    xd, yd = torch.empty_like(x, device="cuda"), torch.empty_like(x, device="cuda")
    layer.moe_batch_host(xh, yh, xd, yd)
    assert np.array_equal(yh.numpy().view(np.uint32), y0.view(np.uint32))


def test_microbench_shapes_iq3_s_and_exl3():
    # benchmark config 2 shapes (hidden 2048, 512 experts top-10, FF 512 + shared 512) with a reduced expert pool so the
    # CPU oracle finishes in seconds: the router only sees the first 64 experts' rows.
    for ety in (szlib.TYPE_IQ3_S, szlib.TYPE_EXL3(3)):
        run_case(2048, 64, 10, 512, 512, ety, ety, 4, seed=12)


@pytest.mark.parametrize("bits,H,ne,k,FF,SF,m", [(3, 2048, 64, 10, 512, 512, 4), (3, 512, 32, 6, 256, 256, 8), (2, 1024, 32, 4, 128, 128, 1),
                                                  (4, 512, 16, 4, 512, 512, 3), (3, 1024, 64, 8, 256, 0, 5)])
def test_warp_specialised_exl3_kernels_give_the_bits_of_the_block_synchronous_ones(bits, H, ne, k, FF, SF, m):
    # two implementations of the streaming EXL3 expert kernels (SZ_X3_CLASSIC=1 selects the block-synchronous one): the same units,
    # the same decode, partial sums added as integers - the outputs must agree bit for bit, run after run
    import os
    ety = szlib.TYPE_EXL3(bits)
    L = synth.make_moe_layer(H, ne, k, FF, SF, ety, ety, seed=21)
    layer = moe.MoeLayer(L, "cuda:0")
    x = torch.randn(m, H, generator=torch.Generator().manual_seed(4)).cuda()
    outs = {}
    for classic in ("1", "0", "0"):
        os.environ["SZ_X3_CLASSIC"] = classic
        try:
            y = layer.moe_batch(x)
            torch.cuda.synchronize()
        finally:
            del os.environ["SZ_X3_CLASSIC"]
        outs.setdefault(classic, []).append(y.cpu().numpy().copy())
    assert np.array_equal(outs["1"][0].view(np.uint32), outs["0"][0].view(np.uint32))
    assert np.array_equal(outs["0"][0].view(np.uint32), outs["0"][1].view(np.uint32))
    Ln = synth.to_numpy_layer(L)
    for j in range(m):
        want = ob.moe(Ln, x[j].cpu().numpy(), threads=4)[0]
        assert np.abs(outs["0"][0][j] - want).max() / max(np.abs(want).max(), 1e-9) < REL_TOL
