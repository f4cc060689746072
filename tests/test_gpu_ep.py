"""Expert parallelism on the GPU.  One card emulates a group the way the reference tests its two-stage split on one card
(crates/shadowzero/tests/two_stage.rs:1-4): G sharded copies of a layer, each producing its fixed-point share, summed as
integers.  The sum must be bit-identical for every G; with two or more cards the same runs over NCCL."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, synth, moe, ep, model = pkg.lib, pkg.synth, pkg.moe, pkg.ep, pkg.model
REL_TOL = 2e-4


def emulate(L, x, G):
    total = None
    for r in range(G):
        layer = moe.MoeLayer(L, "cuda:0", shard=ep.shard_spec(r, G, L["n_expert"]))
        part = layer.moe_partial(x)
        torch.cuda.synchronize()
        total = part.clone() if total is None else total + part
    return total, layer


@pytest.mark.parametrize("ety,H,ne,k,FF,SF", [
    ("q8", 512, 32, 4, 256, 512),      # generic kernels
    ("iq3", 512, 64, 6, 256, 256),
    ("x3", 512, 32, 4, 256, 256),      # streaming EXL3 kernels, shared expert fused
    ("x3", 1024, 32, 6, 256, 512),     # shared expert on the generic kernels
    ("x3", 512, 32, 6, 128, 0),        # no shared expert
    ("x3", 2048, 512, 10, 512, 512),   # the benchmark's layer shape (configs 2 and 3)
])
def test_group_sizes_agree_bitwise(ety, H, ne, k, FF, SF):
    ty = {"q8": szlib.TYPE_Q8_0, "iq3": szlib.TYPE_IQ3_S, "x3": szlib.TYPE_EXL3(3)}[ety]
    L = synth.make_moe_layer(H, ne, k, FF, SF, ty, ty, seed=41)
    m = 4
    x = torch.randn(m, H, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(torch.float32).cuda()
    ref, layer = emulate(L, x, 1)
    for G in (2, 4, 8):
        got, layer = emulate(L, x, G)
        assert torch.equal(got, ref), G
    y = layer.finish(ref).cpu().numpy()
    whole = moe.MoeLayer(L, "cuda:0").moe_batch(x).cpu().numpy()
    Ln = synth.to_numpy_layer(L)
    for j in range(m):
        want = ob.moe(Ln, x[j].cpu().numpy(), threads=4)[0]
        scale = max(np.abs(want).max(), 1e-9)
        assert np.abs(y[j] - want).max() / scale < REL_TOL
        assert np.abs(y[j] - whole[j]).max() / scale < 1e-6     # the fixed-point path against the f64 accumulation


def test_sharded_layer_needs_the_communicator():
    L = synth.make_moe_layer(256, 16, 4, 128, 128, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=42)
    layer = moe.MoeLayer(L, "cuda:0", shard=(0, 8, True))
    x = torch.randn(2, 256).cuda()
    lib = szlib.load()
    lib.sz_ep_destroy()
    with pytest.raises(szlib.SzError):
        layer.moe_batch(x)
    # a group of one needs no NCCL: the whole layer as one shard gives the emulated bits
    szlib.check(lib.sz_ep_init(0, 1, None))
    try:
        full = moe.MoeLayer(L, "cuda:0", shard=(0, 16, True))
        y = full.moe_batch(x)
        ref, _ = emulate(L, x, 2)
        assert torch.equal(y, full.finish(ref))
    finally:
        lib.sz_ep_destroy()


@pytest.mark.parametrize("ety,H,FF,SF", [("q8", 512, 256, 512), ("x3", 512, 256, 256)])
def test_peer_exchange_emulated_on_one_gpu(ety, H, FF, SF):
    """The exchange over peer memory with every rank's buffer on this GPU: all ranks push, then all ranks add up.  Every rank must
    end with the bits of the integer sum of the shares."""
    ty = {"q8": szlib.TYPE_Q8_0, "x3": szlib.TYPE_EXL3(3)}[ety]
    L = synth.make_moe_layer(H, 32, 4, FF, SF, ty, ty, seed=43)
    x = torch.randn(3, H, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).to(torch.float32).cuda()
    ref, any_layer = emulate(L, x, 1)
    want = any_layer.finish(ref)
    for G in (2, 4):
        ex = ep.PeerExchange(H, local_world=G)
        try:
            layers = [moe.MoeLayer(L, "cuda:0", shard=ep.shard_spec(r, G, 32)) for r in range(G)]
            for rounds in range(3):                      # several exchanges: the slots alternate, the counters accumulate
                for r in range(G):
                    ex.use(r)
                    layers[r].push_partial(x)
                ys = []
                for r in range(G):
                    ex.use(r)
                    ys.append(layers[r].finish_exchange(3))
                torch.cuda.synchronize()
                for r in range(G):
                    assert torch.equal(ys[r], want), (G, rounds, r)
            for r in range(G):
                ex.use(r)
                assert ex.status() == 0
        finally:
            ex.close()


def test_peer_exchange_wait_runs_out_without_hanging():
    """A peer that never sends: the finish kernel gives up after its poll budget, raises the error word, and the context stays
    usable.  (The failure is a flag that nothing sets - no fault, no trap.)"""
    L = synth.make_moe_layer(256, 16, 4, 128, 128, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=44)
    x = torch.randn(2, 256).cuda()
    os.environ["SZ_EP_WAIT_POLLS"] = "50000"          # a short budget: this wait is meant to run out
    try:
        ex = ep.PeerExchange(256, local_world=2)
    finally:
        del os.environ["SZ_EP_WAIT_POLLS"]
    try:
        layer = moe.MoeLayer(L, "cuda:0", shard=ep.shard_spec(0, 2, 16))
        ex.use(0)
        layer.moe_batch(x)                               # rank 1 never pushes
        torch.cuda.synchronize()
        assert ex.status() == 1
        layer.moe_batch(x)                               # later waits return at once
        torch.cuda.synchronize()
        assert torch.isfinite(torch.ones(4, device="cuda").sum()).item()
    finally:
        ex.close()


def test_exchange_cannot_be_taken_apart_under_a_session_that_recorded_passes():
    """A recorded pass (CUDA graph) carries the exchange buffers' addresses in its kernel arguments: detaching, re-attaching, unmapping
    or freeing them while the session lives is refused with an error code (a replay would otherwise write into freed memory).  A
    group of one rank on this GPU; the stale graph is never replayed."""
    lib = szlib.load()
    M = model.make_model(dict(model.TINY, vocab=2048, n_layer=2, attn_interval=2), seed=6)
    ex = ep.PeerExchange(model.TINY["hidden"], local_world=1)
    closed = False
    try:
        dm = model.DeviceModel(M, "cuda:0", ep=(0, 1))
        s = model.Session(dm, 64)
        outs = []
        for i in range(3):                       # the first pass runs eagerly and is recorded, the others replay it
            s.verify([5, 6, 7]); outs.append(s.result(logits=True)[2]); s.commit(0)
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
        assert ex.status() == 0
        assert lib.sz_ep_p2p_detach() == szlib.E_ARG
        assert lib.sz_ep_p2p_free(ex.own[0]) == szlib.E_ARG
        with pytest.raises(szlib.SzError):
            ex.use(0)                            # a re-attach is a change of the attachment too
        with pytest.raises(szlib.SzError):
            ex.close()
        del s
        ex.close()
        closed = True
        # a session made while nothing is attached records its passes afresh
        s = model.Session(model.DeviceModel(M, "cuda:0"), 64)
        s.verify([5, 6, 7]); again = s.result(logits=True)[2]; s.commit(0)
        assert np.abs(again - outs[0]).max() <= 1e-5 * np.abs(outs[0]).max()
    finally:
        if not closed:
            ex.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out_dir):
    import threading
    import torch.distributed as dist
    dog = threading.Timer(150, lambda: os._exit(3))     # a rank that waits for a peer that died ends by itself
    dog.daemon = True
    dog.start()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ep.init_from_process_group()
        dev = "cuda:%d" % rank
        L = synth.make_moe_layer(512, 32, 4, 256, 256, szlib.TYPE_EXL3(3), szlib.TYPE_EXL3(3), seed=41)
        x = torch.randn(4, 512, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(torch.float32).to(dev)
        layer = moe.MoeLayer(L, dev, shard=ep.shard_spec(rank, world, 32))
        y = layer.moe_batch(x)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, "y%d.npy" % rank), y.cpu().numpy())
        # the same layer over peer memory instead of NCCL, several exchanges in a row
        ex = ep.PeerExchange(512)
        try:
            for it in range(4):
                yp = layer.moe_batch(x)
                torch.cuda.synchronize()
                assert torch.equal(yp, y), it
            assert ex.status() == 0
            M2 = model.make_model(model.TINY, seed=1, cycle_alpha=0.24)
            _, cyc2 = model.token_cycles(model.TINY["vocab"], 1)
            dm2 = model.DeviceModel(M2, dev, ep=(rank, world))
            s2 = model.Session(dm2, 512)
            toks2, _, _ = s2.generate(model.make_prompt(128, model.TINY["vocab"], seed=1, cycles=cyc2), 48, spec_k=3)
            np.save(os.path.join(out_dir, "p%d.npy" % rank), np.asarray(toks2, dtype=np.int64))
            assert ex.status() == 0
            assert szlib.load().sz_ep_p2p_detach() != 0     # s2's recorded passes hold the mapped addresses: refused
            del s2
            dist.barrier()
        finally:
            ex.close()
        # a whole model: every rank must generate the same tokens
        M = model.make_model(model.TINY, seed=1, cycle_alpha=0.24)
        _, cyc = model.token_cycles(model.TINY["vocab"], 1)
        dm = model.DeviceModel(M, dev, ep=(rank, world))
        s = model.Session(dm, 512)
        toks, _, st = s.generate(model.make_prompt(128, model.TINY["vocab"], seed=1, cycles=cyc), 48, spec_k=3)
        assert st.accepted > 0
        np.save(os.path.join(out_dir, "t%d.npy" % rank), np.asarray(toks, dtype=np.int64))
        dist.barrier()
        lib = szlib.load()
        assert lib.sz_ep_destroy() != 0          # the session's recorded passes hold the communicator: refused, not a hang
        del s
        szlib.check(lib.sz_ep_destroy())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_over_nccl(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    y0, y1 = np.load(tmp_path / "y0.npy"), np.load(tmp_path / "y1.npy")
    assert np.array_equal(y0, y1)
    L = synth.make_moe_layer(512, 32, 4, 256, 256, szlib.TYPE_EXL3(3), szlib.TYPE_EXL3(3), seed=41)
    x = torch.randn(4, 512, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(torch.float32).cuda()
    ref, layer = emulate(L, x, 1)
    assert np.array_equal(layer.finish(ref).cpu().numpy(), y0)          # two cards == one card, bit for bit
    t0, t1 = np.load(tmp_path / "t0.npy"), np.load(tmp_path / "t1.npy")
    assert np.array_equal(t0, t1)
    assert np.array_equal(np.load(tmp_path / "p0.npy"), t0) and np.array_equal(np.load(tmp_path / "p1.npy"), t0)
    lib = szlib.load()
    szlib.check(lib.sz_ep_init(0, 1, None))
    try:
        M = model.make_model(model.TINY, seed=1, cycle_alpha=0.24)
        _, cyc = model.token_cycles(model.TINY["vocab"], 1)
        s = model.Session(model.DeviceModel(M, "cuda:0", ep=(0, 1)), 512)
        toks, _, _ = s.generate(model.make_prompt(128, model.TINY["vocab"], seed=1, cycles=cyc), 48, spec_k=3)
        assert np.array_equal(np.asarray(toks, dtype=np.int64), t0)
    finally:
        lib.sz_ep_destroy()
