"""The verify pass at the benchmark's layer shapes (config 3: hidden 2048, 16 q / 2 kv heads of 256, DeltaNet 16 key / 32 value heads
of 128, 512 experts top-10 of FFN 512 + a shared expert, EXL3 3-bit experts, Q8_0 dense matrices, hyper-connections of 4 streams and
rank 256, Q8_KV cache) against the CPU oracle's Session::step, on a 4-layer slice (one period D D D A) with the vocabulary cut to
4096 so that the CPU side finishes in seconds.  These shapes pick other kernel instantiations than the tiny models do: the DeltaNet
scan with the state split over two thread groups and value heads tiled over half as many key heads (forward.rs:862-864), grouped
attention with 256-wide heads, 8 queries a KV head and many splits, the 512-expert router inside a session.

Yardstick (crates/shadowzero/tests/reference.rs:57-66, 226-255, 291-319): identical routing on every layer, logits within 1e-2
relative (the benchmark's bound), the greedy token equal; batched rows == one at a time; a rolled-back pass continues exactly."""
import numpy as np
import pytest

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, md = pkg.lib, pkg.model

LOGIT_REL = 1e-2
C3_SLICE = dict(n_layer=4, hidden=2048, streams=4, hc_rank=256, vocab=4096, n_head=16, n_kv_head=2, head_dim=256, rope_dims=64,
                n_expert=512, n_expert_used=10, expert_ff=512, shared_ff=512, ssm_k_heads=16, ssm_v_heads=32, ssm_head_dim=128,
                conv_k=4, attn_interval=4, eps=1e-6, rope_theta=1e7)
THREADS = 16


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-9))


@pytest.fixture(scope="module")
def c3():
    M = md.make_model(C3_SLICE, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=5)
    return M, md.HostModel(M), md.DeviceModel(M)


def cpu_steps(cpu, tokens):
    rows, routes = [], []
    for t in tokens:
        rows.append(cpu.step(t))
        routes.append(cpu.routes())
    return np.stack(rows), routes


def same_routing(got, want_idx, want_w):
    """Routing indices equal - except where the reference itself cannot tell two experts apart: their routing weights agree to
    within 1e-5 relative, i.e. their logits differ by less than the last bits of the f32 activations they were computed from, and
    the two sides (f64 dot products over f32 activations that differ in those bits) may rank such a pair either way.  The chosen
    SET must still be the same, and any rank that differs must belong to such a near-tie."""
    if np.array_equal(got, want_idx):
        return True
    for l in range(want_idx.shape[0]):
        if np.array_equal(got[l], want_idx[l]):
            continue
        if sorted(got[l]) != sorted(want_idx[l]):
            return False
        for r in np.nonzero(got[l] != want_idx[l])[0]:
            other = int(np.nonzero(want_idx[l] == got[l][r])[0][0])       # where the oracle ranks the expert the device put at rank r
            if abs(want_w[l][r] - want_w[l][other]) > 1e-5 * want_w[l][r] or abs(other - r) != 1:
                return False
    return True


def check_rows(got, routes, want, want_routes, what):
    worst = 0.0
    for j in range(len(want)):
        assert same_routing(routes[:, j, :], want_routes[j][0], want_routes[j][1]), "%s: routing differs at row %d" % (what, j)
        e = rel_err(got[j], want[j])
        worst = max(worst, e)
        assert e < LOGIT_REL, "%s: row %d logits off by %g" % (what, j, e)
        assert int(np.argmax(got[j])) == int(np.argmax(want[j])), "%s: greedy token differs at row %d" % (what, j)
    return worst


def test_passes_of_1_4_8_rows_with_a_rejected_pass_match_the_cpu_steps(c3):
    M, hm, dm = c3
    toks = [int(t) for t in np.random.default_rng(11).integers(0, C3_SLICE["vocab"], 19)]
    cpu = ob.Session(hm, kv_q8=True, threads=THREADS)
    sess = md.Session(dm, 64, kv_q8=True)
    sess.trace_routes(True)

    def gpu_pass(ids, keep):
        sess.verify(ids)
        _, top, lg = sess.result(logits=True)
        idx, _ = sess.routes()
        for j in range(len(ids)):      # the device's top-64 is the oracle's order on the device's own logits
            v, i = ob.top64(lg[j])
            assert np.array_equal(top[j, 64:], i) and np.array_equal(top[j, :64], v.view(np.uint32))
        sess.commit(keep)
        return lg, idx

    worst = 0.0
    # 1 row, 4 rows, 8 rows: all kept
    at = 0
    for m in (1, 4, 8):
        ids = toks[at:at + m]
        lg, idx = gpu_pass(ids, m)
        want, want_routes = cpu_steps(cpu, ids)
        worst = max(worst, check_rows(lg, idx, want, want_routes, "pass of %d" % m))
        at += m
    # a pass of 4 rows of which 2 are kept (two rejected drafts): the replay of the kept rows rebuilds the recurrent state
    ids = [toks[at], toks[at + 1], 7, 9]
    lg, idx = gpu_pass(ids, 2)
    want, want_routes = cpu_steps(cpu, ids[:2])
    worst = max(worst, check_rows(lg[:2], idx[:, :2], want, want_routes, "rejected pass"))
    at += 2
    assert len(sess) == len(cpu) == at
    # the passes after the rollback continue as if the rejected rows never ran
    ids = toks[at:at + 4]
    lg, idx = gpu_pass(ids, 4)
    want, want_routes = cpu_steps(cpu, ids)
    worst = max(worst, check_rows(lg, idx, want, want_routes, "after the rollback"))
    at += 4
    print("largest relative logit error at config-3 layer shapes: %.3g" % worst)
    assert worst < 2e-3   # where the f32 kernels actually land

    # the committed state, piece by piece, against the oracle's: recurrent state and conv rows of every DeltaNet layer ...
    for l in range(C3_SLICE["n_layer"]):
        if md.is_attention(C3_SLICE, l):
            continue
        S = sess.export(szlib.STATE_DELTA_S, l).reshape(-1)
        S_want = cpu.state(0, l)
        assert np.abs(S - S_want).max() <= 2e-4 * max(np.abs(S_want).max(), 1e-9), "recurrent state of layer %d" % l
        conv = sess.export(szlib.STATE_DELTA_CONV, l).reshape(-1)
        conv_want = cpu.state(1, l)
        assert np.abs(conv - conv_want).max() <= 2e-4 * max(np.abs(conv_want).max(), 1e-9), "conv rows of layer %d" % l
    # ... and the packed Q8_KV cache of the attention layer (272-byte heads: 256 int8 codes, 8 f16 scales, zero padding).  The
    # inputs of the quantiser differ in their last bits between the two sides, so a code may land on the other side of a rounding
    # boundary: codes equal or one apart (rarely), scales equal or one f16 step apart, padding identical
    l = C3_SLICE["n_layer"] - 1
    hd = C3_SLICE["head_dim"]
    for what in (szlib.STATE_KV_K, szlib.STATE_KV_V):
        got = sess.export(what, l)
        want_b = cpu.state(what, l).reshape(got.shape)
        assert got.shape == (at, C3_SLICE["n_kv_head"], 272)
        dq = got[..., :hd].view(np.int8).astype(np.int32) - want_b[..., :hd].view(np.int8).astype(np.int32)
        assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 0.01, (np.abs(dq).max(), (dq != 0).mean())
        sc = got[..., hd:hd + 16].copy().view(np.uint16).astype(np.int32) - want_b[..., hd:hd + 16].copy().view(np.uint16).astype(np.int32)
        assert np.abs(sc).max() <= 1 and (sc != 0).mean() < 0.05
        assert np.array_equal(got[..., hd + 16:], want_b[..., hd + 16:]) and not got[..., hd + 16:].any()


def test_batched_rows_equal_one_at_a_time(c3):
    M, hm, dm = c3
    toks = [int(t) for t in np.random.default_rng(12).integers(0, C3_SLICE["vocab"], 8)]
    a = md.Session(dm, 32, kv_q8=True)
    single = []
    for t in toks:
        a.verify([t]); single.append(a.result(logits=True)[2][0]); a.commit(1)
    b = md.Session(dm, 32, kv_q8=True)
    b.verify(toks[:3]); first = b.result(logits=True)[2]; b.commit(3)
    b.verify([toks[3], toks[4], 5, 6, 7]); b.result(); b.commit(2)      # three rejected drafts
    b.verify(toks[5:8]); rest = b.result(logits=True)[2]; b.commit(3)
    for j in range(3):
        assert rel_err(first[j], single[j]) < 1e-5 and rel_err(rest[j], single[5 + j]) < 1e-5
    # bit-identical to a session that never saw the rejected rows
    c = md.Session(dm, 32, kv_q8=True)
    c.verify(toks[:3]); c.result(); c.commit(3)
    c.verify(toks[3:5]); c.result(); c.commit(2)
    c.verify(toks[5:8]); rest_c = c.result(logits=True)[2]; c.commit(3)
    assert np.array_equal(rest.view(np.uint32), rest_c.view(np.uint32))


def test_a_batched_step_at_the_benchmark_shapes_equals_the_sequences_own_passes(c3, monkeypatch):
    """Five sequences of ragged row counts through sz_batch_verify at config 3's layer shapes (projections of 2,048 and 4,096
    columns through the many-row form of the Q8_0 kernel, reads and MoE over all rows): bit for bit each sequence's own pass;
    and the same with the projections 8 rows a launch."""
    M, hm, dm = c3
    rng = np.random.default_rng(21)
    seqs = [[int(t) for t in rng.integers(0, C3_SLICE["vocab"], 16)] for _ in range(5)]
    alone = [md.Session(dm, 32, kv_q8=True) for _ in range(5)]
    want = []
    plan = [(4, 1, 8, 3, 2), (1, 4, 2, 8, 4)]
    at = [0] * 5
    for ms in plan:
        for b in range(5):
            alone[b].verify(seqs[b][at[b]:at[b] + ms[b]]); want.append(alone[b].result(logits=True)[2].view(np.uint32).copy()); alone[b].commit(ms[b])
            at[b] += ms[b]
    for flag in ("1", "0"):
        monkeypatch.setenv("SZ_BATCH_DENSE_ROWS", flag)
        batch = md.Batch(dm, 5, 32)
        at = [0] * 5
        k = 0
        for ms in plan:
            batch.verify([seqs[b][at[b]:at[b] + ms[b]] for b in range(5)])
            for b in range(5):
                got = batch.sessions[b].result(logits=True)[2].view(np.uint32)
                batch.sessions[b].commit(ms[b])
                assert np.array_equal(got, want[k]), "rows form %s, sequence %d" % (flag, b)
                k += 1
                at[b] += ms[b]


def test_a_batched_step_of_a_hundred_rows_at_the_benchmark_shapes(c3):
    """Twenty-four sequences of 3..6 rows: 512 experts over several windows, projections over three row blocks."""
    M, hm, dm = c3
    n = 24
    rng = np.random.default_rng(23)
    seqs = [[int(t) for t in rng.integers(0, C3_SLICE["vocab"], 6)] for _ in range(n)]
    ms = [3 + b % 4 for b in range(n)]
    batch = md.Batch(dm, n, 16)
    batch.verify([seqs[b][:ms[b]] for b in range(n)])
    for b in range(n):
        got = batch.sessions[b].result(logits=True)[2].view(np.uint32)
        s = md.Session(dm, 16, kv_q8=True)
        s.verify(seqs[b][:ms[b]])
        assert np.array_equal(got, s.result(logits=True)[2].view(np.uint32)), "sequence %d" % b


@pytest.mark.parametrize("length", [700, 5000])
def test_long_context_pass_matches_the_cpu_steps(c3, length):
    """Attention over thousands of cached positions: both sides start from the same seeded cache (the library's synthetic history,
    restated value for value in the oracle), then a 4-row pass and a 1-row pass.  At 5000 positions in a session of 8192 the grouped
    kernel cuts the cache into 32 position ranges a KV head whose partial softmaxes are merged; at 700 the ranges are short."""
    M, hm, dm = c3
    cpu = ob.Session(hm, kv_q8=True, threads=THREADS)
    cpu.fill_synthetic(length, seed=7)
    sess = md.Session(dm, 8192, kv_q8=True)
    sess.fill_synthetic(length, seed=7)
    l = C3_SLICE["n_layer"] - 1
    assert np.array_equal(sess.export(szlib.STATE_KV_K, l), cpu.state(2, l).reshape(length, 2, 272))   # the two fills agree byte for byte
    assert np.array_equal(sess.export(szlib.STATE_KV_V, l), cpu.state(3, l).reshape(length, 2, 272))
    sess.trace_routes(True)
    toks = [int(t) for t in np.random.default_rng(13).integers(0, C3_SLICE["vocab"], 5)]
    worst = 0.0
    for ids in (toks[:4], toks[4:]):
        sess.verify(ids)
        _, top, lg = sess.result(logits=True)
        idx, _ = sess.routes()
        sess.commit(len(ids))
        want, want_routes = cpu_steps(cpu, ids)
        worst = max(worst, check_rows(lg, idx, want, want_routes, "context %d" % length))
    assert len(sess) == length + 5
    print("largest relative logit error at context %d: %.3g" % (length, worst))


def test_the_sparse_indexer_at_the_benchmark_shapes_and_a_long_context():
    """The reference's indexer shape (4 heads of 128, blocks of 4 positions, a budget of 2,048 positions: docs/ARCH.md:142-157) on the
    4-layer slice, past its threshold: 5,000 cached positions = 1,250 complete blocks of which every row keeps 512 and the tail.
    Both sides start from the same seeded caches (attention K / V and the indexer's raw keys)."""
    cfg = dict(C3_SLICE, idx_heads=4, idx_dim=128, idx_budget=2048, idx_ratio=4)
    M = md.make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3), seed=5)
    hm, dm = md.HostModel(M), md.DeviceModel(M)
    length, l = 5000, cfg["n_layer"] - 1
    cpu = ob.Session(hm, kv_q8=True, threads=THREADS)
    cpu.fill_synthetic(length, seed=7)
    sess = md.Session(dm, 8192, kv_q8=True)
    sess.fill_synthetic(length, seed=7)
    toks = [int(t) for t in np.random.default_rng(17).integers(0, cfg["vocab"], 5)]
    worst, at = 0.0, length
    for ids in (toks[:4], toks[4:]):
        sess.verify(ids)
        _, top, lg = sess.result(logits=True)
        sess.commit(len(ids))
        sel = sess.export(szlib.STATE_IDX_SELECTED, l)
        for j, t in enumerate(ids):
            want = cpu.step(t)
            n = at + j + 1
            nb = n // 4
            got = {b for b in range(nb) if (int(sel[j][b >> 5]) >> (b & 31)) & 1}
            ref = {int(p) // 4 for p in cpu.selected(l) if int(p) // 4 < nb}
            assert len(got) == 512 and len(cpu.selected(l)) == 2048 + n % 4
            sc = cpu.idx_scores(l)
            thr = sorted(sc, reverse=True)[511]
            for b in got ^ ref:                        # only blocks tied with the last one kept (to rounding) may differ
                assert abs(sc[b] - thr) <= 1e-5 * max(1.0, abs(thr)), "row %d: block %d (score %g, threshold %g)" % (j, b, sc[b], thr)
            if got == ref:
                e = rel_err(lg[j], want)
                worst = max(worst, e)
                assert e < LOGIT_REL and int(np.argmax(lg[j])) == int(np.argmax(want))
        at += len(ids)
    print("largest relative logit error with the indexer selecting 2,048 of %d positions: %.3g" % (length, worst))
