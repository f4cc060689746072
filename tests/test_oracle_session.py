"""The oracle's session helpers that the GPU parity tests lean on (CPU only): the synthetic history and the state accessors."""
import numpy as np

from oracle import binding as ob
from tests.util import pkg

md = pkg.model
SMALL = dict(md.TINY, vocab=512, n_expert=8, expert_ff=128, shared_ff=128)


def test_synthetic_history_and_state_pieces():
    M = md.make_model(SMALL, seed=3)
    hm = md.HostModel(M)
    for q8 in (True, False):
        s = ob.Session(hm, kv_q8=q8, threads=2)
        s.fill_synthetic(37, seed=5)
        assert len(s) == 37
        hb = 80 if q8 else 256
        k, v = s.state(2, 3), s.state(3, 3)
        assert k.size == v.size == 37 * SMALL["n_kv_head"] * hb and not np.array_equal(k, v)
        if q8:
            heads = k.reshape(37, SMALL["n_kv_head"], hb)
            codes = heads[..., :64].view(np.int8)
            assert codes.min() >= -127 and codes.max() <= 127 and len(np.unique(codes)) > 200
            assert (heads[..., 64:68].copy().view(np.uint16) == 0x2000).all() and not heads[..., 68:].any()
        else:
            assert np.abs(k.view(np.float32)).max() <= 1.0
        assert not s.state(0, 0).any() and not s.state(1, 0).any()
        # the same seed fills the same bytes; a step on top of the history works and moves the recurrent state
        t = ob.Session(hm, kv_q8=q8, threads=2)
        t.fill_synthetic(37, seed=5)
        assert np.array_equal(t.state(2, 3), k)
        lg = s.step(7)
        assert np.isfinite(lg).all() and len(s) == 38 and s.state(0, 0).any()
        assert s.state(0, 0).size == SMALL["ssm_v_heads"] * 64 * 64 and s.state(1, 0).size == 3 * 3 * 4 * 64


def test_tree_pass_of_the_oracle_is_the_paths_read_one_by_one():
    M = md.make_model(SMALL, seed=3)
    hm = md.HostModel(M)
    prefix = [5, 9, 200, 31]
    ids = [7, 40, 41, 42, 43, 44, 45, 46]
    parents = [-1, 0, 0, 1, 1, 2, 3, 5]         # two children under the root, each branching again
    s = ob.Session(hm, kv_q8=True, threads=2)
    for t in prefix:
        s.step(t)
    lg = s.tree(ids, parents)
    assert len(s) == len(prefix)                 # left as it was
    for j in range(len(ids)):                    # row j = the sequence prefix, root .. j read one token at a time
        path = []
        a = j
        while a >= 0:
            path.append(a); a = parents[a]
        t = ob.Session(hm, kv_q8=True, threads=2)
        for tok in prefix + [ids[a] for a in reversed(path)]:
            want = t.step(tok)
        assert np.array_equal(lg[j].view(np.uint32), want.view(np.uint32)), j
    # keeping a path makes the session the one that read it
    s.tree(ids, parents, keep_path=[0, 2, 5, 7])
    t = ob.Session(hm, kv_q8=True, threads=2)
    for tok in prefix + [ids[0], ids[2], ids[5], ids[7]]:
        t.step(tok)
    assert len(s) == len(t) and np.array_equal(s.step(3).view(np.uint32), t.step(3).view(np.uint32))
    # greedy acceptance: drafts made of the model's own best tokens along one branch are kept, a wrong sibling is not
    base = ob.Session(hm, kv_q8=True, threads=2)
    for tok in prefix:
        base.step(tok)
    chain = [7]
    probe = ob.Session(hm, kv_q8=True, threads=2)
    for tok in prefix:
        probe.step(tok)
    for _ in range(3):
        chain.append(int(np.argmax(probe.step(chain[-1]))))
    wrong = (chain[1] + 1) % SMALL["vocab"]
    ids2 = [chain[0], wrong, chain[1], chain[2], wrong, chain[3]]
    par2 = [-1, 0, 0, 2, 2, 3]
    lg2 = base.tree(ids2, par2)
    path, nxt = ob.tree_accept_greedy(lg2, ids2, par2)
    assert path == [0, 2, 3, 5] and nxt == int(np.argmax(lg2[5]))
    assert ob.tree_accept_greedy(lg2, ids2, par2, eog=chain[2])[0] == [0, 2]     # a drafted end-of-generation token is never kept
