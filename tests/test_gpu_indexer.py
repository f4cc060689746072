"""The sparse indexer on the GPU against the CPU restatement (forward.rs:930-976): what every row attends to, the logits, and the
bit-stability the reference's own tests ask of it (tests/reference.rs:85-100, 258-290: the attended positions are the reference's;
a batched step equals one token at a time past the indexer's threshold; a rolled-back pass continues exactly)."""
import numpy as np
import pytest

from oracle import binding as ob
from tests.util import pkg

szlib, md = pkg.lib, pkg.model

pytestmark = pytest.mark.gpu

# 4 layers D D D A; the indexer: 4 heads of 32, blocks of 4 positions, a budget of 32 positions (8 blocks)
IDX = dict(md.TINY, n_layer=4, hidden=256, hc_rank=32, vocab=512, n_head=4, n_kv_head=2, head_dim=64, n_expert=8, n_expert_used=2, expert_ff=128,
           shared_ff=128, ssm_k_heads=2, ssm_v_heads=2, ssm_head_dim=64, idx_heads=4, idx_dim=32, idx_budget=32, idx_ratio=4)
LAYER = 3


@pytest.fixture(scope="module")
def model():
    M = md.make_model(IDX, seed=5)
    return M, md.HostModel(M), md.DeviceModel(M)


def block_set(words, nb):
    return {b for b in range(nb) if (int(words[b >> 5]) >> (b & 31)) & 1}


def check_rows(sess, cpu, ids, start):
    """Feeds `ids` as one pass to the GPU session and one by one to the CPU session; compares every row."""
    sess.verify(ids)
    _, _, lg = sess.result(logits=True)
    sess.commit(len(ids))
    sel = sess.export(szlib.STATE_IDX_SELECTED, LAYER)
    ratio, keep = IDX["idx_ratio"], IDX["idx_budget"] // IDX["idx_ratio"]
    worst = 0.0
    for j, t in enumerate(ids):
        want = cpu.step(int(t))
        n = start + j + 1
        nb = n // ratio
        got = block_set(sel[j], nb)
        pos = cpu.selected(LAYER)
        ref = {int(p) // ratio for p in pos if int(p) // ratio < nb}
        if nb <= keep:
            assert got == set(range(nb)) == ref
        else:
            assert len(got) == keep
            sc = cpu.idx_scores(LAYER)
            thr = sorted(sc, reverse=True)[keep - 1]
            for b in got ^ ref:                        # only blocks tied with the last one kept (to rounding) may differ
                assert abs(sc[b] - thr) <= 1e-5 * max(1.0, abs(thr)), "row %d: block %d (score %g, threshold %g)" % (j, b, sc[b], thr)
        if got == ref:
            err = float(np.max(np.abs(lg[j] - want)) / max(1e-9, float(np.max(np.abs(want)))))
            worst = max(worst, err)
            assert err < 1e-2 and int(np.argmax(lg[j])) == int(np.argmax(want))
    return worst


def test_rows_attend_to_what_the_reference_attends_to(model):
    M, hm, dm = model
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 90)]
    cpu = ob.Session(hm, kv_q8=True, threads=4)
    sess = md.Session(dm, 128, kv_q8=True)
    at, worst = 0, 0.0
    for m in (8, 8, 8, 8, 1, 4, 3, 8, 2, 1, 1, 4, 8, 8, 5, 4, 1):   # crosses the threshold (8 complete blocks = 32 positions) inside a pass
        worst = max(worst, check_rows(sess, cpu, toks[at:at + m], at))
        at += m
    assert at > 2 * IDX["idx_budget"]
    print("largest relative logit distance with the indexer selecting: %.3g" % worst)


def test_a_pass_of_rows_equals_one_row_at_a_time(model):
    M, hm, dm = model
    rng = np.random.default_rng(9)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 72)]
    one, many = md.Session(dm, 128, kv_q8=True), md.Session(dm, 128, kv_q8=True)
    many.prefill(toks[:64]); many.result(); many.commit(8)
    for t in toks[:64]:
        one.verify([t]); one.result(); one.commit(1)
    many.verify(toks[64:72]); _, _, a = many.result(logits=True); many.commit(8)
    sa = many.export(szlib.STATE_IDX_SELECTED, LAYER)
    for j, t in enumerate(toks[64:72]):
        one.verify([t]); _, _, b = one.result(logits=True); one.commit(1)
        sb = one.export(szlib.STATE_IDX_SELECTED, LAYER)
        assert np.array_equal(sa[j], sb[0])
        assert np.array_equal(a[j].view(np.uint32), b[0].view(np.uint32)), "row %d" % j


def test_a_rejected_pass_leaves_nothing_behind(model):
    M, hm, dm = model
    rng = np.random.default_rng(12)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 60)]
    a, b = md.Session(dm, 128, kv_q8=True), md.Session(dm, 128, kv_q8=True)
    for s in (a, b):
        s.prefill(toks[:42]); s.result(); s.commit((42 - 1) % 8 + 1)
    a.verify([toks[42], 7, 8, 9]); a.result(); a.commit(1)          # three drafts rejected: they completed block 10 with other keys
    b.verify([toks[42]]); b.result(); b.commit(1)
    for t in toks[43:]:
        a.verify([t]); _, _, la = a.result(logits=True); a.commit(1)
        b.verify([t]); _, _, lb = b.result(logits=True); b.commit(1)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        assert np.array_equal(a.export(szlib.STATE_IDX_SELECTED, LAYER)[0], b.export(szlib.STATE_IDX_SELECTED, LAYER)[0])


def test_what_the_indexer_does_not_run_on_is_refused(model):
    M, hm, dm = model
    with pytest.raises(szlib.SzError):
        md.Session(dm, 128, kv_q8=False)                # the packed cache only
    s = md.Session(dm, 128, kv_q8=True)
    with pytest.raises(szlib.SzError):
        s.verify_tree([1, 2, 3], [-1, 0, 0])


@pytest.mark.parametrize("with_indexer", [True, False])
def test_a_checkpoint_restored_into_another_session_continues_exactly(model, with_indexer):
    """GpuSession::snapshot / restore (session.rs:3339-3541): every piece of the committed state out to the host and back into a
    fresh session - recurrent states, carried conv rows, K and V rows, the indexer's raw keys (pooled keys are rebuilt) - after
    which both sessions give the same bits, pass after pass, and select the same blocks."""
    if with_indexer:
        M, hm, dm = model
    else:
        cfg = {k: v for k, v in IDX.items() if not k.startswith("idx_")}
        dm = md.DeviceModel(md.make_model(cfg, seed=5))
    rng = np.random.default_rng(21)
    toks = [int(t) for t in rng.integers(0, IDX["vocab"], 70)]
    a = md.Session(dm, 128, kv_q8=True)
    a.prefill(toks[:53]); a.result(); a.commit((53 - 1) % 8 + 1)
    a.verify([toks[53], 3, 4]); a.result(); a.commit(1)            # the state to save follows a rejected pass
    ck = a.checkpoint()
    assert ck["positions"] == 54
    b = md.Session(dm, 128, kv_q8=True)
    b.verify([1, 2, 3]); b.result(); b.commit(3)                   # something of its own first: the restore must clear it
    b.restore(ck)
    assert len(b) == 54
    for ids in (toks[54:58], toks[58:59], toks[59:67]):
        a.verify(ids); _, _, la = a.result(logits=True); a.commit(len(ids))
        b.verify(ids); _, _, lb = b.result(logits=True); b.commit(len(ids))
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        if with_indexer:
            assert np.array_equal(a.export(szlib.STATE_IDX_SELECTED, LAYER)[:len(ids)], b.export(szlib.STATE_IDX_SELECTED, LAYER)[:len(ids)])
    with pytest.raises(szlib.SzError):
        b.lib.sz_session_import and szlib.check(b.lib.sz_session_import(b.h, szlib.STATE_IDX_SELECTED, LAYER, ck["pieces"][0][2].ctypes.data, 4, 0, b.stream))
