"""The whole verify step on the GPU against the CPU oracle's Session::step (forward.rs:751-794) on seeded tiny models:
routing indices identical, logits within 1e-2 relative (the benchmark's bound; the reference's own yardstick is rel < 5e-3 with
identical routing, crates/shadowzero/tests/reference.rs:57-66), emitted greedy tokens and accepted counts identical, and the
reference's structural tests: batched == one at a time, a rolled-back pass continues exactly (reference.rs:226-255, 291-319)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, md = pkg.lib, pkg.model

LOGIT_REL = 1e-2   # the benchmark's target: logits within 1e-2 relative error
SMALL = dict(md.TINY, vocab=4096, n_expert=16, expert_ff=128, shared_ff=128)


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-9))


@pytest.fixture(scope="module")
def small():
    M = md.make_model(SMALL, seed=3)
    return M, md.HostModel(M), md.DeviceModel(M)


def cpu_rows(hm, tokens, kv_q8):
    s = ob.Session(hm, kv_q8=kv_q8, threads=4)
    rows, routes = [], []
    for t in tokens:
        rows.append(s.step(t))
        routes.append(s.routes()[0])
    return np.stack(rows), np.stack(routes)


@pytest.mark.parametrize("kv_q8", [False, True])
def test_verify_rows_match_the_cpu_steps(small, kv_q8):
    M, hm, dm = small
    toks = [int(t) for t in np.random.default_rng(1).integers(0, SMALL["vocab"], 19)]
    want, want_routes = cpu_rows(hm, toks, kv_q8)
    sess = md.Session(dm, 64, kv_q8=kv_q8)
    sess.trace_routes(True)
    got, routes = [], []
    for lo in range(0, len(toks), 8):   # passes of 8, 8 and 3 rows
        chunk = toks[lo:lo + 8]
        sess.verify(chunk)
        _, top, lg = sess.result(logits=True)
        idx, _ = sess.routes()
        got.append(lg); routes.append(idx)
        for j in range(len(chunk)):     # the device's top-64 is the oracle's order on the device's own logits
            v, i = ob.top64(lg[j])
            assert np.array_equal(top[j, 64:], i) and np.array_equal(top[j, :64], v.view(np.uint32))
        sess.commit(len(chunk))
    got = np.concatenate(got)
    routes = np.concatenate(routes, axis=1)  # [layer, row, k]
    assert len(sess) == len(toks)
    for j in range(len(toks)):
        assert np.array_equal(routes[:, j, :], want_routes[j]), "routing differs at row %d" % j
        assert rel_err(got[j], want[j]) < LOGIT_REL, (j, rel_err(got[j], want[j]))
        assert int(np.argmax(got[j])) == int(np.argmax(want[j]))
    assert max(rel_err(got[j], want[j]) for j in range(len(toks))) < 1e-3  # where the f32 kernels actually land


def test_batched_equals_one_at_a_time_and_rollback_continues_exactly(small):
    M, hm, dm = small
    toks = [int(t) for t in np.random.default_rng(2).integers(0, SMALL["vocab"], 12)]
    a = md.Session(dm, 64, kv_q8=True)
    single = []
    for t in toks:
        a.verify([t]); single.append(a.result(logits=True)[2][0]); a.commit(1)
    b = md.Session(dm, 64, kv_q8=True)
    b.verify(toks[:5]); first = b.result(logits=True)[2]; b.commit(5)
    for j in range(5):
        assert rel_err(first[j], single[j]) < 1e-5
    # a pass of 5 rows of which only 2 are kept (3 rejected drafts), then the rest: as if the rejected rows never ran
    wrong = [toks[5], toks[6], 7, 8, 9]
    b.verify(wrong); b.result(); b.commit(2)
    assert len(b) == 7
    b.verify(toks[7:12]); rest = b.result(logits=True)[2]; b.commit(5)
    for j in range(5):
        assert rel_err(rest[j], single[7 + j]) < 1e-5, j
    # and bit-identical to a session that never saw the rejected rows
    c = md.Session(dm, 64, kv_q8=True)
    c.verify(toks[:5]); c.result(); c.commit(5)
    c.verify(toks[5:7]); c.result(); c.commit(2)
    c.verify(toks[7:12]); rest_c = c.result(logits=True)[2]; c.commit(5)
    assert np.array_equal(rest.view(np.uint32), rest_c.view(np.uint32))
    # commit(0) keeps nothing
    c.verify([1, 2, 3]); c.result(); c.commit(0)
    assert len(c) == 12


def test_session_refuses_misuse(small):
    M, hm, dm = small
    s = md.Session(dm, 16, kv_q8=True)
    with pytest.raises(szlib.SzError):
        s.verify(list(range(9)))
    s.verify([1, 2])
    with pytest.raises(szlib.SzError):
        s.verify([3])          # previous pass not committed
    with pytest.raises(szlib.SzError):
        s.commit(3)            # more rows than the pass had
    s.commit(2)
    with pytest.raises(szlib.SzError):
        s.commit(1)            # nothing pending
    s.verify(list(range(8))); s.commit(8)
    with pytest.raises(szlib.SzError):
        s.verify(list(range(8)))   # 10 + 8 > 16


@pytest.fixture(scope="module")
def tiny_cycle():
    M = md.make_model(md.TINY, seed=1, cycle_alpha=0.24)
    _, cyc = md.token_cycles(md.TINY["vocab"], 1)
    return M, md.HostModel(M), md.DeviceModel(M), md.make_prompt(256, md.TINY["vocab"], seed=1, cycles=cyc)


def test_config1_greedy_spec3_tokens_and_accepted_counts(tiny_cycle):
    # benchmark config 1: 256-token prompt, 128 new tokens, greedy, --spec 3 with the suffix drafter; CPU scalar path vs GPU
    M, hm, dm, prompt = tiny_cycle
    want_toks, want_log, want_st = ob.Session(hm, kv_q8=True, threads=8).generate(prompt, 128, spec_k=3)
    sess = md.Session(dm, 512, kv_q8=True)
    toks, log, st = sess.generate(prompt, 128, spec_k=3, device_accept=True)
    assert toks == want_toks
    assert log == want_log
    assert (st.passes, st.drafted, st.accepted, st.lookup_passes) == (want_st.passes, want_st.drafted, want_st.accepted, want_st.lookup_passes)
    assert list(st.pos_tried) == list(want_st.pos_tried) and list(st.pos_right) == list(want_st.pos_right)
    assert st.passes > 0 and st.accepted > 0
    # speculation does not change what is generated
    sess2 = md.Session(dm, 512, kv_q8=True)
    plain, _, st2 = sess2.generate(prompt, 128, spec_k=0)
    assert plain == toks and st2.passes == 0


def test_stop_ids_end_the_loop_and_are_never_accepted_as_drafts(tiny_cycle):
    # engine.rs:2381-2390: a pick that is a stop token ends the request, a drafted one is left for the loop's top to see.  The stop
    # list rides to the device with the pass, so deciding on the device and on the host give the same tokens and counts.
    M, hm, dm, prompt = tiny_cycle
    plain, plain_log, _ = md.Session(dm, 512, kv_q8=True).generate(prompt, 64, spec_k=3)
    for j in range(6, 60, 3):                          # every third token of the plain run in turn becomes the stop id
        stop = plain[j]
        cut = plain.index(stop)
        outs = []
        for device_accept in (True, False):
            sess = md.Session(dm, 512, kv_q8=True)
            sess.set_stops([M["cfg"]["vocab"] - 1, stop])
            toks, log, st = sess.generate(prompt, 64, spec_k=3, device_accept=device_accept)
            assert toks == plain[:cut]
            outs.append((toks, log, (st.passes, st.drafted, st.accepted)))
        assert outs[0] == outs[1]
    # the same through the pass itself: the kept count stops before the stop id
    tail = (len(prompt) - 1) % szlib.MAX_VERIFY + 1
    free, sess = md.Session(dm, 512, kv_q8=True), md.Session(dm, 512, kv_q8=True)
    for x in (free, sess):
        x.prefill(prompt); x.result(); x.commit(tail)
    assert plain[2] not in plain[:2]
    free.verify(plain[:4], accept=1); (k0, _), _, _ = free.result()
    sess.set_stops([plain[2]])
    sess.verify(plain[:4], accept=1); (k1, _), _, _ = sess.result()
    assert k0 == 4 and k1 == 2
    with pytest.raises(szlib.SzError):
        sess.set_stops(list(range(8)))                 # seven at most


def test_config1_sampled_spec3(tiny_cycle):
    # sampled acceptance: the token the target would have drawn at that position (sampler.rs:3-9); T = 0.7, top-p 0.9
    M, hm, dm, prompt = tiny_cycle
    want_toks, want_log, want_st = ob.Session(hm, kv_q8=True, threads=8).generate(prompt, 96, spec_k=3, greedy=False,
                                                                                  sampler=ob.SamplerC(0.7, 20, 0.9, 0.0, 11))
    sess = md.Session(dm, 512, kv_q8=True)
    toks, log, st = sess.generate(prompt, 96, spec_k=3, greedy=False, sampler=md.Sampler(0.7, 20, 0.9, 0.0, 11))   # acceptance on the device
    assert toks == want_toks and log == want_log
    host = md.Session(dm, 512, kv_q8=True)
    toks_h, log_h, _ = host.generate(prompt, 96, spec_k=3, greedy=False, sampler=md.Sampler(0.7, 20, 0.9, 0.0, 11), device_accept=False)
    assert toks_h == want_toks and log_h == want_log


def test_sampled_acceptance_on_the_device_is_the_host_draw(small):
    # every row's draw on the device against sz_sample_top on the same top-64 table, over several samplers and positions
    M, hm, dm = small
    L = szlib.load()
    toks = [int(t) for t in np.random.default_rng(9).integers(0, SMALL["vocab"], 8)]
    fresh = md.Session(dm, 64, kv_q8=True)
    with pytest.raises(szlib.SzError):
        fresh.verify_sampled(toks, 0)            # no sampler yet
    for sp in (md.Sampler(0.7, 20, 0.9, 0.0, 11), md.Sampler(1.3, 64, 1.0, 0.05, 5), md.Sampler(0.2, 1, 0.5, 0.0, 3), md.Sampler(2.0, 40, 0.95, 0.1, 77)):
        sess = md.Session(dm, 64, kv_q8=True)
        sess.set_sampler(sp)

        def host_picks(top, pos, n):
            return [int(L.sz_sample_top(C.byref(sp), top[j].ctypes.data_as(C.POINTER(C.c_uint32)), pos + j)) for j in range(n)]

        for pos in (0, 1000003):
            sess.verify_sampled(toks, pos)
            (keep, nxt), top, _ = sess.result()
            picks = host_picks(top, pos, len(toks))
            want_keep = 1
            while want_keep < len(toks) and picks[want_keep - 1] == toks[want_keep]:
                want_keep += 1
            assert keep == want_keep and nxt == picks[keep - 1], (sp.temperature, pos)
            sess.commit(keep)
            assert len(sess) == keep
            sess.reset()
        # drafts that ARE the sampler's draws are all kept: draw row 0, draft it, draw again, ...
        chain = [toks[0]]
        for step in range(3):
            sess.verify_sampled(chain, 40)
            (keep, nxt), top, _ = sess.result()
            assert keep == len(chain) and nxt == host_picks(top, 40, len(chain))[-1]
            sess.commit(keep)
            sess.reset()
            chain.append(nxt)


def test_graph_replay_equals_eager_launches(small):
    # the second pass with the same (rows, head, acceptance) replays a recorded CUDA graph: same bytes as the eager first pass
    M, hm, dm = small
    toks = [int(t) for t in np.random.default_rng(4).integers(0, SMALL["vocab"], 16)]
    outs = []
    for rounds in range(2):
        s = md.Session(dm, 64, kv_q8=True)
        got = []
        for lo in (0, 4, 8, 12):           # four passes of 4 rows: the first is eager, the rest are graph launches
            s.verify(toks[lo:lo + 4]); got.append(s.result(logits=True)[2]); s.commit(4)
        outs.append(np.concatenate(got))
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    want, _ = cpu_rows(hm, toks, True)
    assert max(rel_err(outs[0][j], want[j]) for j in range(16)) < 1e-3


def test_fused_hyper_connection_read_gives_the_bits_of_the_two_launches(small):
    # SZ_HC_FUSED=1: down half, grid-wide barrier (bounded), up half in one launch - the second implementation of the same arithmetic
    import os
    M, hm, dm = small
    toks = [int(t) for t in np.random.default_rng(6).integers(0, SMALL["vocab"], 12)]
    outs = []
    for fused in ("0", "1"):
        os.environ["SZ_HC_FUSED"] = fused
        try:
            s = md.Session(dm, 64, kv_q8=True)
            got = []
            for lo in (0, 4, 8):            # the first pass is eager, the others replay its graph
                s.verify(toks[lo:lo + 4]); got.append(s.result(logits=True)[2]); s.commit(4)
            outs.append(np.concatenate(got))
            del s
        finally:
            del os.environ["SZ_HC_FUSED"]
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


def test_synthetic_history_gives_a_long_context(small):
    M, hm, dm = small
    s = md.Session(dm, 4096, kv_q8=True)
    s.fill_synthetic(3000, seed=7)
    assert len(s) == 3000
    s.verify([5, 6, 7, 8]); (_, _), top, lg = s.result(logits=True); s.commit(4)
    assert len(s) == 3004 and np.isfinite(lg).all()
    # deterministic: the same seed gives the same logits, another seed does not
    t = md.Session(dm, 4096, kv_q8=True)
    t.fill_synthetic(3000, seed=7)
    t.verify([5, 6, 7, 8]); lg2 = t.result(logits=True)[2]; t.commit(4)
    assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32))
    t.fill_synthetic(3000, seed=8)
    t.verify([5, 6, 7, 8]); lg3 = t.result(logits=True)[2]; t.commit(4)
    assert not np.array_equal(lg, lg3)
