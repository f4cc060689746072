"""Tree verification on the GPU (benchmark config 4's mechanism; no counterpart in the reference, so parity is against this
repository's own CPU restatement: every row of a tree pass is its root-to-row path read one token at a time on a copy of the oracle's
session).  Checked: every row's logits (the benchmark's 1e-2 bound; routing as for chains), greedy acceptance on the device against
the oracle's walk, and - the part a tree adds to a chain - that after keeping a path the session continues exactly as one that read
that path as a chain: recurrent state replayed along the path, keys and values moved from the rows' slots to the depths' positions."""
import numpy as np
import pytest

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, md = pkg.lib, pkg.model
SMALL = dict(md.TINY, vocab=4096, n_expert=16, expert_ff=128, shared_ff=128)
C3_SLICE = dict(n_layer=4, hidden=2048, streams=4, hc_rank=256, vocab=4096, n_head=16, n_kv_head=2, head_dim=256, rope_dims=64,
                n_expert=512, n_expert_used=10, expert_ff=512, shared_ff=512, ssm_k_heads=16, ssm_v_heads=32, ssm_head_dim=128,
                conv_k=4, attn_interval=4, eps=1e-6, rope_theta=1e7)
TREES = {
    "two_branches": [-1, 0, 0, 1, 1, 2, 3, 5],
    "wide": [-1, 0, 0, 0, 0, 1, 2, 3],          # branching 4 at the root
    "deep_then_back": [-1, 0, 1, 2, 0, 4, 5, 1],
    "chain": [-1, 0, 1, 2, 3],
}


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-9))


def models(kind):
    if kind == "tiny":
        M = md.make_model(SMALL, seed=3)
        return SMALL, md.HostModel(M), md.DeviceModel(M), 4
    M = md.make_model(C3_SLICE, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=5)
    return C3_SLICE, md.HostModel(M), md.DeviceModel(M), 16


@pytest.fixture(scope="module", params=["tiny", "c3"])
def setup(request):
    return models(request.param)


@pytest.mark.parametrize("tree", list(TREES))
def test_tree_rows_match_their_paths_and_a_kept_path_continues_exactly(setup, tree):
    cfg, hm, dm, threads = setup
    parents = TREES[tree]
    m = len(parents)
    rng = np.random.default_rng(17)
    prefix = [int(t) for t in rng.integers(0, cfg["vocab"], 11)]      # a pass of 8 and one of 3: the conv window reaches into both
    ids = [int(t) for t in rng.integers(0, cfg["vocab"], m)]
    cpu = ob.Session(hm, kv_q8=True, threads=threads)
    for t in prefix:
        cpu.step(t)
    sess = md.Session(dm, 64, kv_q8=True)
    sess.verify(prefix[:8]); sess.result(); sess.commit(8)
    sess.verify(prefix[8:]); sess.result(); sess.commit(3)
    # the deepest leaf's path is kept
    depth = [0] * m
    for j in range(1, m):
        depth[j] = depth[parents[j]] + 1
    leaf = max(range(m), key=lambda j: (depth[j], -j))
    path = []
    a = leaf
    while a >= 0:
        path.append(a); a = parents[a]
    path.reverse()
    want = cpu.tree(ids, parents, keep_path=path)
    sess.verify_tree(ids, parents)
    _, top, got = sess.result(logits=True)
    for j in range(m):
        assert rel_err(got[j], want[j]) < 1e-2, (tree, j, rel_err(got[j], want[j]))
        assert int(np.argmax(got[j])) == int(np.argmax(want[j]))
        v, i = ob.top64(got[j])
        assert np.array_equal(top[j, 64:], i)
    assert max(rel_err(got[j], want[j]) for j in range(m)) < 2e-3
    sess.commit_path(path)
    assert len(sess) == len(prefix) + len(path) == len(cpu)
    # a session that read the kept path as a chain: the tree session must now be that session, bit for bit
    chain = md.Session(dm, 64, kv_q8=True)
    chain.verify(prefix[:8]); chain.result(); chain.commit(8)
    chain.verify(prefix[8:]); chain.result(); chain.commit(3)
    chain.verify([ids[a] for a in path]); chain_lg = chain.result(logits=True)[2]; chain.commit(len(path))
    for d, a in enumerate(path):                                   # and a tree row IS its chain row
        assert np.array_equal(got[a].view(np.uint32), chain_lg[d].view(np.uint32)), (tree, a)
    for l in range(cfg["n_layer"]):
        if md.is_attention(cfg, l):
            assert np.array_equal(sess.export(szlib.STATE_KV_K, l), chain.export(szlib.STATE_KV_K, l))
            assert np.array_equal(sess.export(szlib.STATE_KV_V, l), chain.export(szlib.STATE_KV_V, l))
        else:
            assert np.array_equal(sess.export(szlib.STATE_DELTA_S, l).view(np.uint32), chain.export(szlib.STATE_DELTA_S, l).view(np.uint32))
            assert np.array_equal(sess.export(szlib.STATE_DELTA_CONV, l).view(np.uint32), chain.export(szlib.STATE_DELTA_CONV, l).view(np.uint32))
    nxt = [int(t) for t in rng.integers(0, cfg["vocab"], 4)]
    sess.verify(nxt); a1 = sess.result(logits=True)[2]; sess.commit(4)
    chain.verify(nxt); a2 = chain.result(logits=True)[2]; chain.commit(4)
    assert np.array_equal(a1.view(np.uint32), a2.view(np.uint32))
    wantn = np.stack([cpu.step(t) for t in nxt])
    assert max(rel_err(a1[j], wantn[j]) for j in range(4)) < 2e-3


def test_greedy_acceptance_down_the_tree_on_the_device(setup):
    cfg, hm, dm, threads = setup
    rng = np.random.default_rng(23)
    prefix = [int(t) for t in rng.integers(0, cfg["vocab"], 6)]
    cpu = ob.Session(hm, kv_q8=True, threads=threads)
    for t in prefix:
        lg = cpu.step(t)
    # the model's own continuation (from the oracle), planted as one branch of the tree among wrong siblings
    root = int(np.argmax(lg))
    probe = ob.Session(hm, kv_q8=True, threads=threads)
    for t in prefix:
        probe.step(t)
    good = [root]
    for _ in range(3):
        good.append(int(np.argmax(probe.step(good[-1]))))
    bad = [(g + 1) % cfg["vocab"] for g in good]
    ids = [good[0], bad[1], good[1], bad[2], good[2], good[3], bad[3], bad[1]]
    parents = [-1, 0, 0, 2, 2, 4, 4, 1]
    want = cpu.tree(ids, parents)
    want_path, want_next = ob.tree_accept_greedy(want, ids, parents)
    assert want_path == [0, 2, 4, 5]
    sess = md.Session(dm, 64, kv_q8=True)
    sess.verify(prefix); sess.result(); sess.commit(len(prefix))
    sess.verify_tree(ids, parents, accept=1)
    (keep, nxt), top, _ = sess.result()
    assert sess.tree_path() == want_path and keep == len(want_path) and nxt == want_next
    with pytest.raises(szlib.SzError):
        sess.commit(keep - 1)                          # the device decided: the host's count must be the device's
    sess.commit(keep)
    assert len(sess) == len(prefix) + keep
    # and the session goes on as the chain would
    chain = md.Session(dm, 64, kv_q8=True)
    chain.verify(prefix); chain.result(); chain.commit(len(prefix))
    chain.verify([ids[a] for a in want_path]); chain.result(); chain.commit(len(want_path))
    sess.verify([nxt]); a1 = sess.result(logits=True)[2]; sess.commit(1)
    chain.verify([nxt]); a2 = chain.result(logits=True)[2]; chain.commit(1)
    assert np.array_equal(a1.view(np.uint32), a2.view(np.uint32))
    # a drafted end-of-generation token is never kept
    s3 = md.Session(dm, 64, kv_q8=True)
    s3.verify(prefix); s3.result(); s3.commit(len(prefix))
    s3.verify_tree(ids, parents, accept=1, eog=good[2])
    (keep, nxt), _, _ = s3.result()
    assert s3.tree_path() == [0, 2] and keep == 2
    s3.commit(keep)
    # nor one of the session's stop ids
    s5 = md.Session(dm, 64, kv_q8=True)
    s5.set_stops([bad[0], good[2]])
    s5.verify(prefix); s5.result(); s5.commit(len(prefix))
    s5.verify_tree(ids, parents, accept=1)
    (keep, nxt), _, _ = s5.result()
    assert s5.tree_path() == [0, 2] and keep == 2
    # misuse
    s4 = md.Session(dm, 64, kv_q8=True)
    with pytest.raises(szlib.SzError):
        s4.verify_tree([1, 2, 3], [-1, 1, 0])          # a parent that comes later
    with pytest.raises(szlib.SzError):
        s4.verify_tree([1, 2, 3], [0, 0, 1])           # no root
    s4.verify_tree([1, 2, 3], [-1, 0, 0])
    s4.result()
    with pytest.raises(szlib.SzError):
        s4.commit(2)                                   # a tree pass the caller decides is closed by its path
    with pytest.raises(szlib.SzError):
        s4.commit_path([0, 1, 2])                      # row 2 is not a child of row 1
    s4.commit_path([0, 2])
    assert len(s4) == 2


def test_tree_passes_replay_through_their_graph(setup):
    cfg, hm, dm, threads = setup
    rng = np.random.default_rng(29)
    parents = TREES["two_branches"]
    outs = []
    for rounds in range(2):
        s = md.Session(dm, 96, kv_q8=True)
        got = []
        for i in range(3):                    # the first tree pass is eager, the next two replay its graph with other tokens
            ids = [int(t) for t in np.random.default_rng(100 + i).integers(0, cfg["vocab"], 8)]
            s.verify_tree(ids, parents)
            got.append(s.result(logits=True)[2])
            s.commit_path([0, 2, 5, 7])
        outs.append(np.concatenate(got))
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
