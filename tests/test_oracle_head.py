"""The oracle's lm_head proxy stage against the assertions of the reference's own test of it
(crates/shadowzero-cuda/tests/head_proxy.rs:84-236), on the blob and inputs its xorshift generator builds from the same seed."""
import numpy as np

from oracle import binding as ob
from tests.test_oracle_exl3 import XorShift


def f16_bits(v):
    return int(np.array([v], dtype=np.float32).astype(np.float16).view(np.uint16)[0])


class RefRng(XorShift):
    def unit(self):  # head_proxy.rs:15-17
        return np.float32(np.float32(self.next() % 20001) / np.float32(10000.0) - np.float32(1.0))


def ref_blob(rng, rows, cols, bits):
    """make_exl3_k5_blob (head_proxy.rs:58-82), no hot rows: suh and svh in 0.8 .. 1.2, marker 0, random trellis words."""
    nt, kt = rows // 16, cols // 16
    tr_words = nt * kt * 8 * bits
    hdr = 2 * cols + 2 * rows + 4
    out = np.zeros(hdr + tr_words * 4, dtype=np.uint8)
    sc = np.array([np.float32(0.8) + np.float32(0.4) * abs(rng.unit()) for _ in range(cols + rows)], dtype=np.float32)
    out[:2 * (cols + rows)] = sc.astype(np.float16).view(np.uint8)
    words = np.array([rng.next() & 0xffffffff for _ in range(tr_words)], dtype=np.uint32)
    out[hdr:] = words.view(np.uint8)
    return out


def proxy_stage(rows, cols, bits, blob, x, k_use):
    m = x.shape[0]
    q2, sc = ob.head_proxy_build(rows, cols, bits, blob)
    xr = ob.head_rotate(blob, x)
    xq, x_sc, x_corr = ob.proxy_quant_x(xr)
    bmax = ob.proxy_bmax(rows, cols, q2, sc, xq, x_sc, x_corr)
    sel = ob.proxy_pick(bmax, k_use, min(m * k_use, rows // 128))
    return q2, sc, xr, (xq, x_sc, x_corr), bmax, sel


def test_reference_test_assertions_hold_for_the_oracle():
    rows, cols, m, k_blk, bits = 4096, 2560, 4, 12, 5   # head_proxy.rs:91
    rng = RefRng(0xabcdef0123456789)
    blob = ref_blob(rng, rows, cols, bits)
    x = np.array([rng.unit() for _ in range(m * cols)], dtype=np.float32).reshape(m, cols)
    n_ob = rows // 128
    q2, sc, xr, (xq, x_sc, x_corr), bmax, sel = proxy_stage(rows, cols, bits, blob, x, k_blk)
    assert k_blk <= sel.size <= min(m * k_blk, n_ob)            # head_proxy.rs:175
    assert np.all(np.diff(sel.astype(np.int64)) > 0)
    dense = np.stack([ob.matvec(ob.EXL3_BASE + bits, blob, rows, cols, x[j], threads=4) for j in range(m)])
    want = dense.reshape(m, n_ob, 128).max(axis=2)
    for j in range(m):
        g, w = bmax[j].astype(np.float64), want[j].astype(np.float64)
        cos = float(g @ w / max(np.sqrt(g @ g) * np.sqrt(w @ w), 1e-24))
        assert cos > 0.85, (j, cos)                              # head_proxy.rs:193
        assert int(np.argmax(dense[j])) // 128 in sel            # head_proxy.rs:232: the screen keeps the best row's block
    # the codes are the four levels, and the proxy reproduces the rotated weights to 2-bit accuracy
    assert q2.size == rows * cols // 4 and sc.size == rows * cols // 128
    codes = np.stack([(q2 >> s) & 3 for s in (0, 2, 4, 6)])
    assert 0.15 < float((codes == 0).mean()) < 0.35 and 0.15 < float((codes == 3).mean()) < 0.35


def test_quantised_inputs_follow_the_kernel_arithmetic():
    rng = np.random.default_rng(5)
    xr = rng.normal(size=(3, 256)).astype(np.float32)
    xr[1, 128:] = 0.0                                             # an all-zero block: scale 0, codes 0
    xq, sc, corr = ob.proxy_quant_x(xr)
    for j in range(3):
        for b in range(2):
            blk = xr[j, b * 128:(b + 1) * 128]
            amax = np.float32(np.abs(blk).max())
            s = np.float32(amax / np.float32(127.0)) if amax > 0 else np.float32(0)
            assert sc[j, b] == s
            inv = np.float32(1.0) / s if s > 0 else np.float32(0)
            q = np.rint(np.clip(blk * inv, -127, 127)).astype(np.int32)
            assert np.array_equal(xq[j, b * 128:(b + 1) * 128].astype(np.int32), q)
            assert corr[j, b] == np.float32(np.float32(-3.0) * np.float32(q.sum())) * s
    assert sc[1, 1] == 0 and not xq[1, 128:].any()


def test_pick_is_the_k_best_by_value_then_index():
    bmax = np.array([[1.0, 5.0, 5.0, np.nan, 2.0, -1.0, 5.0, 0.0],
                     [9.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 8.0]], dtype=np.float32)
    assert ob.proxy_pick(bmax[:1], 2, 8).tolist() == [1, 2]       # ties to the lower index
    assert ob.proxy_pick(bmax[:1], 4, 8).tolist() == [1, 2, 4, 6]
    assert ob.proxy_pick(bmax, 2, 8).tolist() == [0, 1, 2, 7]     # the union over the rows of the pass, ascending
    assert ob.proxy_pick(bmax, 2, 3).tolist() == [0, 1, 2]        # cut at max_sel
    assert ob.proxy_pick(bmax[:1], 20, 8).tolist() == list(range(8))
    assert ob.head_k_use(128, 64) == 128 and ob.head_k_use(128, 16) == 96 and ob.head_k_use(64, 16) == 64 and ob.head_k_use(16, 1) == 16
