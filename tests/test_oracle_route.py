"""The oracle's router against a full sort, with the reference's seed and tie-heavy recipe (forward.rs:1272-1303)."""
import math

import numpy as np

from oracle import binding as ob
from tests.test_oracle_exl3 import XorShift


def full_sort_route(logits, k):
    """softmax over all experts in f64 (libm exp, sum in index order), the k best by (ex desc, index asc),
    weights renormalised over the chosen ones: the definition `route` is tested against in the reference."""
    mx = np.float32(logits.max())
    ex = [math.exp(float(np.float32(v) - mx)) for v in logits]
    z = 0.0
    for e in ex:
        z += e
    order = sorted(range(len(ex)), key=lambda i: (-ex[i], i))[:k]
    tz = 0.0
    for e in order:
        tz += ex[e] / z
    return order, [(ex[e] / z) / tz for e in order]


def test_route_matches_a_full_sort():
    rng = XorShift(0x2545f4914f6cdd1d)
    for trial in range(500):
        raw = [rng.next() for _ in range(512)]
        if trial % 2 == 0:  # coarse values, so ties are common
            logits = np.array([(s % 16) for s in raw], dtype=np.float32) * np.float32(0.5)
        else:
            logits = np.array([(s % 100000) for s in raw], dtype=np.float32) / np.float32(7919.0) - np.float32(6.0)
        want_idx, want_w = full_sort_route(logits, 10)
        idx, w = ob.route(logits, 10)
        assert list(idx) == want_idx, trial
        assert np.array_equal(np.array(want_w).view(np.uint64), w.view(np.uint64)), trial


def test_route_small_and_edge_cases():
    idx, w = ob.route(np.array([0.0, 1.0, 1.0, -1.0], dtype=np.float32), 2)
    assert list(idx) == [1, 2] and abs(w.sum() - 1.0) < 1e-15 and w[0] == w[1]
    idx, w = ob.route(np.array([3.0, 1.0], dtype=np.float32), 4)  # k > n: all of them
    assert list(idx) == [0, 1]
    idx, w = ob.route(np.zeros(0, dtype=np.float32), 4)
    assert len(idx) == 0
    # n > 512 takes the reference's general branch; the same order
    lg = np.random.default_rng(3).standard_normal(700).astype(np.float32)
    idx, w = ob.route(lg, 12)
    want_idx, want_w = full_sort_route(lg, 12)
    assert list(idx) == want_idx
    assert np.array_equal(np.array(want_w).view(np.uint64), w.view(np.uint64))
