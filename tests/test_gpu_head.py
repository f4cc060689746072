"""The lm_head over an EXL3 output.weight through the C ABI: every stage of the screened (2-bit proxy) form against the CPU
restatement bit for bit, the logits against the exact EXL3 matvec, and the properties the reference's own test asserts
(crates/shadowzero-cuda/tests/head_proxy.rs:84-236): sparse logits identical to the dense ones, top-64 exact over the kept blocks,
the best token's block kept."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib, synth, Head = pkg.lib, pkg.synth, pkg.head.Head


def make(rows, cols, bits, seed=3, sigma=0.02):
    return synth.random_exl3_blobs(1, cols, rows, bits, sigma, seed, "output.weight")[0].numpy()


def rows_of(m, cols, seed=5):
    return np.random.default_rng(seed).normal(size=(m, cols)).astype(np.float32)


def sort_top64(vals, ids):
    """(value descending, id ascending) over the given candidates: the order of kernels/forward.cu:3565-3625."""
    order = np.lexsort((ids, -vals.astype(np.float64)))[:64]
    return vals[order], ids[order]


def check_top(top_row, vals, ids):
    v, i = sort_top64(vals, ids)
    assert np.array_equal(top_row[64:], i.astype(np.uint32))
    assert np.array_equal(top_row[:64], v.view(np.uint32))


@pytest.mark.parametrize("bits,m", [(4, 4), (3, 1), (5, 8), (4, 3)])
def test_every_stage_matches_the_cpu_restatement(bits, m):
    rows, cols, k_blk = 8192, 512, 16
    blob = make(rows, cols, bits)
    x = rows_of(m, cols)
    h = Head(blob, rows, cols, bits, k_blk=k_blk)
    q2, sc = ob.head_proxy_build(rows, cols, bits, blob)
    assert np.array_equal(h.w_q2.cpu().numpy(), q2)
    assert np.array_equal(h.w_sc.cpu().numpy().view(np.uint16), sc)
    top, logits = h.top(torch.from_numpy(x).cuda())
    assert h.stage(szlib.HEAD_ERR, np.uint32)[0] == 0
    xr = ob.head_rotate(blob, x)
    assert np.array_equal(h.stage(szlib.HEAD_XR, np.float32).reshape(8, cols)[:m].view(np.uint32), xr.view(np.uint32))
    xq, x_sc, x_corr = ob.proxy_quant_x(xr)
    assert np.array_equal(h.stage(szlib.HEAD_XQ, np.int8).reshape(8, cols)[:m], xq)
    assert np.array_equal(h.stage(szlib.HEAD_XSC, np.float32).reshape(8, -1)[:m].view(np.uint32), x_sc.view(np.uint32))
    assert np.array_equal(h.stage(szlib.HEAD_XCORR, np.float32).reshape(8, -1)[:m].view(np.uint32), x_corr.view(np.uint32))
    bmax = ob.proxy_bmax(rows, cols, q2, sc, xq, x_sc, x_corr)
    assert np.array_equal(h.stage(szlib.HEAD_BMAX, np.float32).reshape(8, -1)[:m].view(np.uint32), bmax.view(np.uint32))
    k_use, max_sel, ls = h.plan(m)
    assert k_use == ob.head_k_use(k_blk, 64) and max_sel == min(m * k_use, rows // 128) and ls == max_sel * 128
    want_sel = ob.proxy_pick(bmax, k_use, max_sel)
    sel = h.stage(szlib.HEAD_SEL, np.uint32)
    assert sel[0] == want_sel.size and np.array_equal(sel[1:1 + sel[0]], want_sel)
    # the logits of the kept blocks against the exact matvec (f64 sums of the dequantised rows)
    lg = logits.cpu().numpy()
    for j in range(m):
        dense = ob.matvec(ob.EXL3_BASE + bits, blob, rows, cols, x[j], threads=4)
        scale = float(np.abs(dense).max())
        ids = (want_sel[:, None].astype(np.int64) * 128 + np.arange(128)[None, :]).reshape(-1)
        got = lg[j, :ids.size]
        assert np.abs(got - dense[ids]).max() <= 1e-4 * scale
        check_top(top[j], got, ids)
        assert int(np.argmax(dense)) // 128 in want_sel            # head_proxy.rs:232
        assert int(top[j][64]) == int(np.argmax(dense))


@pytest.mark.parametrize("bits", [2, 4, 6, 8])
def test_dense_head_matches_the_exact_matvec_and_the_sparse_logits_are_the_dense_ones(bits):
    rows, cols, m = 2048, 256, 4
    blob = make(rows, cols, bits, seed=9)
    x = rows_of(m, cols, seed=2)
    xd = torch.from_numpy(x).cuda()
    dense_h = Head(blob, rows, cols, bits, k_blk=0)
    top_d, lg_d = dense_h.top(xd)
    lg_d = lg_d.cpu().numpy()
    assert lg_d.shape == (m, rows)
    for j in range(m):
        want = ob.matvec(ob.EXL3_BASE + bits, blob, rows, cols, x[j], threads=4)
        assert np.abs(lg_d[j] - want).max() <= 1e-4 * float(np.abs(want).max())
        check_top(top_d[j], lg_d[j], np.arange(rows))
    sparse_h = Head(blob, rows, cols, bits, k_blk=16)               # 16 blocks = all of them here: clamped to rows / 128
    top_s, lg_s = sparse_h.top(xd)
    sel = sparse_h.stage(szlib.HEAD_SEL, np.uint32)
    lg_s = lg_s.cpu().numpy()
    for s in range(int(sel[0])):                                    # head_proxy.rs:203-211: bit-identical
        ob_ = int(sel[1 + s])
        assert np.array_equal(lg_s[:, s * 128:(s + 1) * 128].view(np.uint32), lg_d[:, ob_ * 128:(ob_ + 1) * 128].view(np.uint32))
    assert int(sel[0]) == rows // 128 and np.array_equal(top_s, top_d)


def test_full_vocabulary_properties():
    """Config 3's head (151936 x 2048 at 4 bits, 128 blocks a row): no CPU pass at this size, the properties instead."""
    rows, cols, bits, m = 151936, 2048, 4, 4
    blob = synth.random_exl3_blobs(1, cols, rows, bits, 0.02, 1, "output.weight", device="cuda")[0]
    x = torch.from_numpy(rows_of(m, cols, seed=11)).cuda()
    h = Head(blob, rows, cols, bits, k_blk=128)
    top, lg = h.top(x)
    assert h.stage(szlib.HEAD_ERR, np.uint32)[0] == 0
    sel = h.stage(szlib.HEAD_SEL, np.uint32)
    n_sel = int(sel[0])
    blocks = sel[1:1 + n_sel].astype(np.int64)
    assert 128 <= n_sel <= 512 and np.all(np.diff(blocks) > 0) and blocks[-1] < rows // 128
    d = Head(blob, rows, cols, bits, k_blk=0)
    top_d, lg_d = d.top(x)
    lg, lg_d = lg.cpu().numpy(), lg_d.cpu().numpy()
    ids = (blocks[:, None] * 128 + np.arange(128)[None, :]).reshape(-1)
    assert np.array_equal(lg[:, :ids.size].view(np.uint32), lg_d[:, ids].view(np.uint32))
    bmax = h.stage(szlib.HEAD_BMAX, np.float32).reshape(8, -1)[:m]
    true_max = lg_d.reshape(m, -1, 128).max(axis=2)
    for j in range(m):
        check_top(top[j], lg[j, :ids.size], ids)
        check_top(top_d[j], lg_d[j], np.arange(rows))
        assert int(top_d[j][64]) // 128 in blocks                   # the screen keeps the best token's block
        assert int(top[j][64]) == int(top_d[j][64])
        g, w = bmax[j].astype(np.float64), true_max[j].astype(np.float64)
        assert float(g @ w / (np.sqrt(g @ g) * np.sqrt(w @ w))) > 0.85   # head_proxy.rs:193
        # each row's own k best blocks by proxy score are in the list
        own = np.argsort(-bmax[j], kind="stable")[:128]
        assert np.isin(own, blocks).all()


# ---- inside a session ---------------------------------------------------------------------------------------------------------------

md = pkg.model
SMALL = dict(md.TINY, vocab=4096, n_expert=16, expert_ff=128, shared_ff=128)


@pytest.fixture(scope="module")
def exl3_head_model():
    M = md.make_model(SMALL, seed=4, head_type=szlib.TYPE_EXL3(4))
    return M, md.HostModel(M), md.DeviceModel(M)


def test_session_with_an_exl3_head_matches_the_cpu_steps(exl3_head_model):
    M, hm, dm = exl3_head_model
    toks = [int(t) for t in np.random.default_rng(1).integers(0, SMALL["vocab"], 11)]
    cpu = ob.Session(hm, kv_q8=True, threads=4)
    want = np.stack([cpu.step(t) for t in toks])
    sess = md.Session(dm, 64, kv_q8=True)
    got = []
    for lo in range(0, len(toks), 8):
        chunk = toks[lo:lo + 8]
        sess.verify(chunk)
        _, top, lg = sess.result(logits=True)
        got.append(lg)
        for j in range(len(chunk)):
            v, i = ob.top64(lg[j])
            assert np.array_equal(top[j, 64:], i) and np.array_equal(top[j, :64], v.view(np.uint32))
        sess.commit(len(chunk))
    got = np.concatenate(got)
    for j in range(len(toks)):
        err = float(np.abs(got[j] - want[j]).max() / np.abs(want[j]).max())
        assert err < 1e-2 and int(np.argmax(got[j])) == int(np.argmax(want[j])), (j, err)


def test_screened_head_in_a_session_agrees_with_the_exact_head_on_the_best_tokens(exl3_head_model):
    M, hm, dm = exl3_head_model
    toks = [int(t) for t in np.random.default_rng(3).integers(0, SMALL["vocab"], 8)]
    exact = md.Session(dm, 64, kv_q8=True)
    exact.verify(toks)
    _, top_e, lg_e = exact.result(logits=True)
    import os
    os.environ["SZ_HEAD_KBLK"] = "16"          # 16 of the 32 blocks a row
    try:
        screened = md.Session(dm, 64, kv_q8=True, head_proxy=True)
    finally:
        del os.environ["SZ_HEAD_KBLK"]
    screened.verify(toks)
    _, top_s, _ = screened.result()
    with pytest.raises(szlib.SzError):
        screened.result(logits=True)             # only the kept blocks have logits
    for j in range(len(toks)):
        assert top_s[j, 64] == top_e[j, 64] and top_s[j, 0] == top_e[j, 0]   # same best token, same logit bits
        # every token the screened head lists carries the exact head's logit
        ids = top_s[j, 64:].astype(np.int64)
        assert np.array_equal(top_s[j, :64], lg_e[j][ids].view(np.uint32))
    # greedy acceptance on the device reads the same table
    screened.commit(8)
    screened.verify([toks[0], int(top_s[0, 64])], accept=1)
    kn, _, _ = screened.result()
    assert kn[0] >= 1


def test_synthetic_reconstruction_is_the_oracle_matrix():
    bits, n_in, n_out = 3, 256, 384
    blob = synth.random_exl3_blobs(1, n_in, n_out, bits, 0.02, 7, "t", device="cuda")[0]
    w = synth.exl3_reconstruct(blob, n_in, n_out, bits).cpu().numpy()
    want = ob.exl3_reconstruct(n_in, n_out, bits, blob.cpu().numpy())
    assert np.abs(w - want).max() <= 1e-5 * np.abs(want).max()


def test_speculation_with_an_exl3_head_emits_the_cpu_tokens():
    """Config 1's run (greedy, --spec 3, suffix drafter) on a model whose head is EXL3 and whose embedding follows the head's
    token cycles: tokens and accepted counts of the CPU scalar path, with the exact head and (same tokens) the screened one."""
    cfg = dict(md.TINY, vocab=4096, n_expert=16, expert_ff=128, shared_ff=128)
    M = md.make_model(cfg, seed=2, head_type=szlib.TYPE_EXL3(4), cycle_alpha=0.5, device="cuda")
    hm, dm = md.HostModel(M), md.DeviceModel(M)
    _, cycles = md.token_cycles(cfg["vocab"], 2)
    prompt = md.make_prompt(96, cfg["vocab"], seed=1, cycles=cycles)
    want_toks, want_log, want_st = ob.Session(hm, kv_q8=True, threads=8).generate(prompt, 64, spec_k=3)
    toks, log, st = md.Session(dm, 256, kv_q8=True).generate(prompt, 64, spec_k=3)
    assert toks == want_toks and log == want_log
    assert st.accepted > 0
    toks_p, log_p, _ = md.Session(dm, 256, kv_q8=True, head_proxy=True).generate(prompt, 64, spec_k=3)
    assert toks_p == want_toks and log_p == want_log
