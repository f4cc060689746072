"""Expert parallelism, host side, on CPU: shard arithmetic, the unique-id hand-off over a process group, and the exactness of
the fixed-point exchange - two gloo ranks each sum the experts they hold (outputs from the CPU oracle), all-reduce the int64
terms, and must land on the same bits as one rank holding everything."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import binding as ob
from tests.util import pkg

szlib, synth, ep = pkg.lib, pkg.synth, pkg.ep


def test_shard_ranges_partition_the_experts():
    for ne in (8, 32, 60, 512):
        for world in (1, 2, 3, 4, 8):
            nxt = 0
            for r in range(world):
                first, count = ep.shard_range(r, world, ne)
                assert first == nxt and count in (ne // world, ne // world + 1)
                nxt = first + count
                for e in (first, first + count - 1):
                    assert ep.owner(e, world, ne) == r
            assert nxt == ne
    with pytest.raises(ValueError):
        ep.shard_range(2, 2, 8)
    assert [ep.shard_spec(r, 4, 512) for r in range(4)] == [(0, 128, True), (128, 128, False), (256, 128, False), (384, 128, False)]


def test_fixed_point_is_exact_for_sums_of_terms():
    rng = np.random.default_rng(3)
    v = rng.standard_normal((11, 300)) * 0.3
    f = ep.to_fixed(v)
    for perm in (np.arange(11), rng.permutation(11), rng.permutation(11)):
        assert np.array_equal(f[perm].sum(0), f.sum(0))            # any order, any grouping
    assert np.abs(ep.from_fixed(f.sum(0)) - v.sum(0)).max() < 1e-6


def _expert_terms(Ln, u):
    """(route idx, [k][H] weighted expert outputs, [H] shared term) of one token, each matvec by the oracle."""
    H, FF, SF = Ln["hidden"], Ln["expert_ff"], Ln["shared_ff"]
    _, idx, w, _ = ob.moe(Ln, u)

    def ffn(ty, g, up, dn, ff):
        a = ob.matvec(ty, g, ff, H, u)
        b = ob.matvec(ty, up, ff, H, u)
        act = (a / (1.0 + np.exp(-a.astype(np.float64)))).astype(np.float32) * b
        return ob.matvec(ty, dn, H, ff, act)

    terms = np.stack([w[t] * ffn(Ln["expert_type"], Ln["gate"][e], Ln["up"][e], Ln["down"][e], FF).astype(np.float64)
                      for t, e in enumerate(idx)])
    sgl = float(np.dot(Ln["shared_router"].astype(np.float64).ravel(), u.astype(np.float64)))
    sh = ffn(Ln["shared_type"], Ln["sh_gate"], Ln["sh_up"], Ln["sh_down"], SF).astype(np.float64) / (1.0 + np.exp(-sgl))
    return idx, terms, sh


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 1. the id hand-off: rank 0 draws it, all ranks join with the same bytes
        seen = {}
        r, w = ep.init_from_process_group(get_id=lambda: bytes(range(128)), init=lambda r, w, i: seen.update(rank=r, world=w, id=i))
        assert (r, w) == (rank, world) and seen == dict(rank=rank, world=world, id=bytes(range(128)))
        # 2. the exchange: every rank routes the same token, sums only the experts it holds, all-reduces integers
        L = synth.make_moe_layer(128, 16, 4, 64, 64, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=5)
        Ln = synth.to_numpy_layer(L)
        u = torch.randn(128, generator=torch.Generator().manual_seed(9)).numpy()
        idx, terms, sh = _expert_terms(Ln, u)
        first, count, with_shared = ep.shard_spec(rank, world, 16)
        mine = np.zeros(128, dtype=np.int64)
        for t, e in enumerate(idx):
            if first <= e < first + count:
                mine += ep.to_fixed(terms[t])
        if with_shared:
            mine += ep.to_fixed(sh)
        total = torch.from_numpy(mine.copy())
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        np.save(os.path.join(out_dir, "r%d.npy" % rank), total.numpy())
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reduce_to_the_single_rank_bits(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "r0.npy"), np.load(tmp_path / "r1.npy")
    assert np.array_equal(a, b)
    L = synth.make_moe_layer(128, 16, 4, 64, 64, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=5)
    Ln = synth.to_numpy_layer(L)
    u = torch.randn(128, generator=torch.Generator().manual_seed(9)).numpy()
    idx, terms, sh = _expert_terms(Ln, u)
    one = ep.to_fixed(terms).sum(0) + ep.to_fixed(sh)
    assert np.array_equal(a, one)
    want, _, _, _ = ob.moe(Ln, u)
    assert np.abs(ep.from_fixed(a) - want).max() <= 1e-6 * max(1.0, np.abs(want).max())
