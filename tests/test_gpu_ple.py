"""The per-layer embedding (hashed n-gram memory of one layer, forward.rs:1036-1074, 1177-1198) on the GPU against the CPU restatement:
logits of every row, rows in a pass equal to rows one at a time, a rejected pass leaves no trace in the conv history or the token
tail, a checkpoint carries both."""
import numpy as np
import pytest

from oracle import binding as ob
from tests.test_oracle_ple import PLE
from tests.util import pkg

szlib, md = pkg.lib, pkg.model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    M = md.make_model(PLE, seed=2)
    return M, md.HostModel(M), md.DeviceModel(M)


def tokens(n, seed, eos_at=()):
    t = [int(x) for x in np.random.default_rng(seed).integers(0, PLE["vocab"], n)]
    for i in eos_at:
        t[i] = PLE["ple_eos"]
    return t


def test_rows_match_the_cpu_steps_across_passes_and_an_end_of_text(model):
    M, hm, dm = model
    toks = tokens(60, 3, eos_at=(5, 6, 30))
    cpu = ob.Session(hm, kv_q8=True, threads=4)
    sess = md.Session(dm, 128, kv_q8=True)
    at, worst = 0, 0.0
    for m in (1, 1, 4, 8, 2, 8, 3, 1, 8, 8, 4, 5, 7):
        ids = toks[at:at + m]
        sess.verify(ids)
        _, _, lg = sess.result(logits=True)
        sess.commit(m)
        for j, t in enumerate(ids):
            want = cpu.step(t)
            err = float(np.max(np.abs(lg[j] - want)) / max(1e-9, float(np.max(np.abs(want)))))
            worst = max(worst, err)
            assert err < 1e-2 and int(np.argmax(lg[j])) == int(np.argmax(want)), "position %d" % (at + j)
        at += m
    print("largest relative logit distance with the per-layer embedding: %.3g" % worst)
    # the carried history is the oracle's, to rounding
    hist = sess.export(szlib.STATE_PLE_HIST, 0)
    assert hist.shape == (9, 4 * PLE["hidden"]) and np.all(np.isfinite(hist)) and float(np.abs(hist).max()) > 0.0
    assert list(sess.export(szlib.STATE_PLE_TAIL, 0)[:3]) == toks[at - 1:at - 4:-1]


def test_a_pass_of_rows_equals_one_row_at_a_time_and_a_rejected_pass_leaves_nothing(model):
    M, hm, dm = model
    toks = tokens(40, 9, eos_at=(17,))
    one, many = md.Session(dm, 128, kv_q8=True), md.Session(dm, 128, kv_q8=True)
    for t in toks[:13]:
        one.verify([t]); one.result(); one.commit(1)
    many.prefill(toks[:13]); many.result(); many.commit((13 - 1) % 8 + 1)
    many.verify([toks[13], 3, PLE["ple_eos"], 4]); many.result(); many.commit(1)      # three drafts rejected, an end-of-text among them
    one.verify([toks[13]]); one.result(); one.commit(1)
    at = 14
    for m in (8, 4, 1, 5, 8):
        ids = toks[at:at + m]
        many.verify(ids); _, _, a = many.result(logits=True); many.commit(m)
        for j, t in enumerate(ids):
            one.verify([t]); _, _, b = one.result(logits=True); one.commit(1)
            assert np.array_equal(a[j].view(np.uint32), b[0].view(np.uint32)), "position %d" % (at + j)
        at += m
    assert np.array_equal(one.export(szlib.STATE_PLE_HIST, 0), many.export(szlib.STATE_PLE_HIST, 0))
    assert np.array_equal(one.export(szlib.STATE_PLE_TAIL, 0), many.export(szlib.STATE_PLE_TAIL, 0))


def test_a_checkpoint_carries_the_history_and_the_tail(model):
    M, hm, dm = model
    toks = tokens(40, 11)
    a = md.Session(dm, 128, kv_q8=True)
    a.prefill(toks[:21]); a.result(); a.commit((21 - 1) % 8 + 1)
    ck = a.checkpoint()
    b = md.Session(dm, 128, kv_q8=True)
    b.verify([9, 8, 7]); b.result(); b.commit(3)
    b.restore(ck)
    for ids in (toks[21:25], toks[25:26], toks[26:34]):
        a.verify(ids); _, _, la = a.result(logits=True); a.commit(len(ids))
        b.verify(ids); _, _, lb = b.result(logits=True); b.commit(len(ids))
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))


def test_greedy_generation_with_speculation_matches_the_cpu_loop(model):
    M, hm, dm = model
    prompt = md.make_prompt(48, PLE["vocab"], seed=4)
    want_toks, want_log, _ = ob.Session(hm, kv_q8=True, threads=4).generate(prompt, 40, spec_k=3)
    toks, log, _ = md.Session(dm, 256, kv_q8=True).generate(prompt, 40, spec_k=3)
    assert toks == want_toks and log == want_log


def test_tree_passes_are_refused(model):
    M, hm, dm = model
    s = md.Session(dm, 64, kv_q8=True)
    with pytest.raises(szlib.SzError):
        s.verify_tree([1, 2, 3], [-1, 0, 0])


def test_a_model_with_every_optional_branch_from_its_file_on_the_device(tmp_path):
    """Per-layer embedding and sparse indexer together, written as a GGUF, loaded onto the device by the library: speculative
    generation equals the CPU loop on the same file (tokens and the accepted count of every pass), past the indexer's threshold."""
    gio = pkg.gguf_io
    cfg = dict(PLE, idx_heads=2, idx_dim=32, idx_budget=16, idx_ratio=4)
    M = md.make_model(cfg, seed=6, cycle_alpha=0.9)
    path = str(tmp_path / "all.gguf")
    gio.write_gguf(path, M)
    host, dev = gio.LoadedModel(path), gio.LoadedModel(path, device="cuda:0")
    prompt = md.make_prompt(64, cfg["vocab"], seed=8)
    want_toks, want_log, want_st = ob.Session(host, kv_q8=True, threads=4).generate(prompt, 48, spec_k=3)
    toks, log, st = md.Session(dev, 256, kv_q8=True).generate(prompt, 48, spec_k=3)
    assert toks == want_toks and log == want_log
    assert st.accepted == want_st.accepted and st.passes > 0
