"""The sparse indexer in the CPU restatement (forward.rs:930-976): what it attends to, and that it changes nothing below its budget."""
import numpy as np

from oracle import binding as ob
from tests.util import pkg

md = pkg.model

# a small hybrid with an indexer: 4 heads of 32, blocks of 4 positions, a budget of 32 positions (8 blocks)
IDX = dict(md.TINY, n_layer=4, hidden=256, hc_rank=32, vocab=512, n_head=4, n_kv_head=2, head_dim=64, n_expert=8, n_expert_used=2, expert_ff=128,
           shared_ff=128, ssm_k_heads=2, ssm_v_heads=2, ssm_head_dim=64, idx_heads=4, idx_dim=32, idx_budget=32, idx_ratio=4)


def test_everything_is_attended_to_below_the_budget_and_the_best_blocks_plus_the_tail_above():
    M = md.make_model(IDX, seed=5)
    hm = md.HostModel(M)
    s = ob.Session(hm, kv_q8=False, threads=4)
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 61)]
    keep, ratio = IDX["idx_budget"] // IDX["idx_ratio"], IDX["idx_ratio"]
    for i, t in enumerate(toks):
        s.step(t)
        n = i + 1
        sel = s.selected(3)
        nb = n // ratio
        if nb <= keep:
            assert list(sel) == list(range(n)) and s.idx_scores(3).size == 0
            continue
        sc = s.idx_scores(3)
        assert sc.size == nb and np.all(sc >= 0.0)
        order = sorted(range(nb), key=lambda b: (-sc[b], b))[:keep]           # score descending, block ascending among equals
        want = sorted(p for b in order for p in range(b * ratio, (b + 1) * ratio)) + list(range(nb * ratio, n))
        assert list(sel) == want
        assert len(sel) == IDX["idx_budget"] + n % ratio


def test_a_huge_budget_is_the_model_without_an_indexer():
    cfg = dict(IDX, idx_budget=1 << 20)
    M = md.make_model(cfg, seed=5)
    plain = dict(M, cfg={k: v for k, v in cfg.items() if not k.startswith("idx_")})
    a, b = ob.Session(md.HostModel(M), kv_q8=True, threads=4), ob.Session(md.HostModel(plain), kv_q8=True, threads=4)
    rng = np.random.default_rng(4)
    for t in rng.integers(0, cfg["vocab"], 40):
        la, lb = a.step(int(t)), b.step(int(t))
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))


def test_a_restored_session_selects_as_one_that_never_went_ahead():
    M = md.make_model(IDX, seed=6)
    hm = md.HostModel(M)
    rng = np.random.default_rng(8)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 50)]
    a, b = ob.Session(hm, kv_q8=True, threads=4), ob.Session(hm, kv_q8=True, threads=4)
    for t in toks[:44]:
        a.step(t); b.step(t)
    snap = a.clone()
    for t in (1, 2, 3, 4, 5):                          # a rejected draft: completes a block, then is thrown away
        a.step(t)
    a.assign(snap)
    for t in toks[44:]:
        la, lb = a.step(t), b.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        assert np.array_equal(a.selected(3), b.selected(3))
