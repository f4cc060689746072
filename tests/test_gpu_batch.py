"""Several sequences in one step (`sz_batch_verify`, `sz_batch_gen_run`): every sequence's logits, acceptance and tokens are bit for
bit those of a session stepping alone - the sequences share the MoE sublayers' work, not their numbers."""
import numpy as np
import pytest

from tests.util import pkg

szlib, md = pkg.lib, pkg.model

pytestmark = pytest.mark.gpu

CFG = dict(md.TINY, vocab=2048, n_expert=16, n_expert_used=4, shared_ff=256)   # a shared expert as wide as the routed ones: the streaming kernels take it


@pytest.fixture(scope="module")
def dm():
    M = md.make_model(CFG, expert_type=szlib.TYPE_EXL3(3), seed=4, cycle_alpha=0.9, cycle_beta=0.5)
    return md.DeviceModel(M)


def test_a_step_of_several_sequences_equals_their_own_passes(dm):
    rng = np.random.default_rng(2)
    seqs = [[int(t) for t in rng.integers(0, CFG["vocab"], 30)] for _ in range(5)]
    batch = md.Batch(dm, 5, 64)
    alone = [md.Session(dm, 64, kv_q8=True) for _ in range(5)]
    at = [0] * 5
    for step, ms in enumerate([(8, 1, 4, 3, 8), (1, 1, 1, 1, 1), (4, 8, 2, 1, 5), (3, 3, 3, 3, 3)]):
        rows = [seqs[b][at[b]:at[b] + ms[b]] for b in range(5)]
        batch.verify(rows)
        for b in range(5):
            _, top, lg = batch.sessions[b].result(logits=True)
            batch.sessions[b].commit(ms[b])
            alone[b].verify(rows[b]); _, top2, lg2 = alone[b].result(logits=True); alone[b].commit(ms[b])
            assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)), "step %d sequence %d" % (step, b)
            assert np.array_equal(top, top2)
            at[b] += ms[b]
    # a step of some of the sequences only, with acceptance on the device and a rejected draft
    rows = [seqs[0][at[0]:at[0] + 1] + [5, 6], seqs[3][at[3]:at[3] + 2]]
    batch.verify(rows, accept=1, which=[0, 3])
    for b, r in zip((0, 3), rows):
        (keep, nxt), _, _ = batch.sessions[b].result()
        alone[b].verify(r, accept=1); (keep2, nxt2), _, _ = alone[b].result()
        assert (keep, nxt) == (keep2, nxt2)
        batch.sessions[b].commit(keep); alone[b].commit(keep2)
    with pytest.raises(szlib.SzError):
        batch.verify([[1], [2]], which=[1, 1])         # a session twice
    # after the steps the sessions are their own again: a pass alone on one of them is the pass of the session that always was
    for b in (1, 4):
        r = seqs[b][at[b]:at[b] + 3]
        batch.sessions[b].verify(r); _, top, lg = batch.sessions[b].result(logits=True)
        alone[b].verify(r); _, top2, lg2 = alone[b].result(logits=True)
        assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)) and np.array_equal(top, top2)


def test_a_step_of_forty_sequences_and_two_hundred_rows(dm):
    """Many sequences: the reads, projections and experts then run over several row blocks and windows; every sequence still gets
    the bits of its own pass, step after step."""
    n = 40
    rng = np.random.default_rng(31)
    seqs = [[int(t) for t in rng.integers(0, CFG["vocab"], 24)] for _ in range(n)]
    batch = md.Batch(dm, n, 48)
    alone = [md.Session(dm, 48, kv_q8=True) for _ in range(n)]
    at = [0] * n
    for step in range(3):
        ms = [1 + (3 * b + 5 * step) % 8 for b in range(n)]          # 1..8 rows, about 180 a step
        rows = [seqs[b][at[b]:at[b] + ms[b]] for b in range(n)]
        batch.verify(rows, accept=2)                                  # every row accepted on the device
        for b in range(n):
            (keep, _), top, lg = batch.sessions[b].result(logits=True)
            alone[b].verify(rows[b], accept=2); (keep2, _), top2, lg2 = alone[b].result(logits=True)
            assert keep == keep2 == ms[b]
            assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)), "step %d sequence %d" % (step, b)
            assert np.array_equal(top, top2)
            batch.sessions[b].commit(keep); alone[b].commit(keep2)
            at[b] += ms[b]


@pytest.mark.parametrize("rows_max", [None, 16])
def test_prompts_fed_in_lockstep_equal_prompts_fed_alone(dm, rows_max):
    """sz_batch_prefill: prompts of ragged lengths (one token, whole passes, a tail), more sequences than a step holds when the
    scratch is small: the last pass's logits, and a pass after the commit, are bit for bit those of sz_session_prefill."""
    lens = [1, 8, 9, 30, 16, 23]
    prompts = [md.make_prompt(n, CFG["vocab"], seed=40 + i) for i, n in enumerate(lens)]
    batch = md.Batch(dm, len(lens), 64, rows_max=rows_max)
    batch.prefill(prompts)
    for b, p in enumerate(prompts):
        tail = (len(p) - 1) % 8 + 1
        a = md.Session(dm, 64, kv_q8=True)
        a.prefill(p)
        _, top2, lg2 = a.result(logits=True); a.commit(tail)
        s = batch.sessions[b]
        _, top, lg = s.result(logits=True); s.commit(tail)
        assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)) and np.array_equal(top, top2), "prompt %d" % b
        s.verify([5, 6, 7]); a.verify([5, 6, 7])
        assert np.array_equal(s.result(logits=True)[2].view(np.uint32), a.result(logits=True)[2].view(np.uint32)), "after prompt %d" % b
        s.commit(3); a.commit(3)


def test_generation_from_prompts_fed_in_lockstep(dm):
    prompts = [md.make_prompt(40 + 8 * b, CFG["vocab"], seed=10 + b) for b in range(4)]
    toks_b, st_b, _ = md.Batch(dm, 4, 256).generate(prompts, 32, feed="batch")
    toks_a, st_a, _ = md.Batch(dm, 4, 256).generate(prompts, 32, feed="alone")
    assert toks_b == toks_a
    assert [(s.passes, s.drafted, s.accepted) for s in st_b] == [(s.passes, s.drafted, s.accepted) for s in st_a]
    for b, p in enumerate(prompts):
        want, _, _ = md.Session(dm, 256, kv_q8=True).generate(p, 32, spec_k=3)
        assert toks_b[b] == want


def lockstep(dm, vocab, n_seq, n_new, ctx=256):
    """n_seq sequences alone and then in lockstep: tokens and the books of every sequence."""
    import ctypes as C
    prompts = [md.make_prompt(40 + 8 * b, vocab, seed=10 + b) for b in range(n_seq)]
    want = []
    for p in prompts:
        toks, _, st = md.Session(dm, ctx, kv_q8=True).generate(p, n_new + len(want), spec_k=3)
        want.append((toks, st.passes, st.drafted, st.accepted))
    batch = md.Batch(dm, n_seq, ctx)
    gens = [md.Generator(s, p, n_new + b, spec_k=3) for b, (s, p) in enumerate(zip(batch.sessions, prompts))]
    n = n_seq
    gh = (C.c_void_p * n)(*[g.h for g in gens])
    outs = (C.c_void_p * n)(*[C.cast(g.out, C.c_void_p) for g in gens])
    sts = (C.c_void_p * n)(*[C.cast(C.pointer(g.stats), C.c_void_p) for g in gens])
    dev = C.c_double(0.0)
    szlib.check(batch.lib.sz_batch_gen_run(gh, n, 0, outs, sts, batch.rows_max, batch.scratch, batch.scratch_bytes, C.byref(dev), batch.stream))
    for b, g in enumerate(gens):
        assert (g.tokens(), g.stats.passes, g.stats.drafted, g.stats.accepted) == want[b], "sequence %d" % b
    assert dev.value > 0.0


def test_sequences_decoding_in_lockstep_emit_their_own_tokens(dm):
    lockstep(dm, CFG["vocab"], 4, 32)


@pytest.mark.parametrize("ple_layer", [0, 1])
def test_lockstep_on_a_model_with_the_per_layer_embedding_and_the_indexer(ple_layer):
    """The per-layer embedding (first layer: before anything shared has run; a later one: after a shared MoE) and the sparse indexer
    keep their state per sequence while the reads and projections around them run over all rows."""
    from tests.test_oracle_ple import PLE
    cfg = dict(PLE, hidden=512, hc_rank=64, ple_head_dim=128, ple_layer=ple_layer, idx_heads=2, idx_dim=32, idx_budget=16, idx_ratio=4)   # (the streaming expert kernels take a hidden size that is a multiple of 512)
    M = md.make_model(cfg, expert_type=szlib.TYPE_EXL3(3), seed=6, cycle_alpha=0.9)
    lockstep(md.DeviceModel(M), cfg["vocab"], 3, 40)


def test_the_shared_reads_and_projections_change_no_bit(dm, monkeypatch):
    """SZ_BATCH_SHARED=0 shares only the MoE sublayers (every sequence reads and projects its own rows): the same logits."""
    rng = np.random.default_rng(5)
    rows = [[int(t) for t in rng.integers(0, CFG["vocab"], m)] for m in (3, 8, 1, 4, 2, 7)]
    got = []
    # (SZ_BATCH_DENSE_ROWS=0: the projections 8 rows a launch; SZ_BATCH_HC_SPLIT=0: the reads' first half by the pass's own kernel)
    # SZ_BATCH_SCAN_SEQS=0: a scan launch a sequence instead of one a layer
    for shared, rows_form, split, scans in (("1", "1", "1", "1"), ("0", "1", "1", "1"), ("1", "0", "1", "1"), ("1", "1", "0", "1"), ("1", "1", "1", "0")):
        monkeypatch.setenv("SZ_BATCH_SHARED", shared)
        monkeypatch.setenv("SZ_BATCH_DENSE_ROWS", rows_form)
        monkeypatch.setenv("SZ_BATCH_HC_SPLIT", split)
        monkeypatch.setenv("SZ_BATCH_SCAN_SEQS", scans)
        batch = md.Batch(dm, 6, 64)
        batch.verify(rows)
        got.append([batch.sessions[b].result(logits=True)[2].view(np.uint32).copy() for b in range(6)])
    for other in got[1:]:
        for a, b in zip(got[0], other):
            assert np.array_equal(a, b)
