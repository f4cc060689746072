"""Sampled acceptance down a draft tree (host code, no GPU): the library's C++ and the oracle's C statement of the same rule agree
decision for decision, and the rule has the property that makes it a sampler at all - whatever the drafter proposes, the token that
comes out at a position is distributed as the target's own distribution there."""
import ctypes as C

import numpy as np

from oracle import binding as ob
from tests.util import pkg

szlib, md = pkg.lib, pkg.model


def top_rows(rng, m, spread=3.0):
    """m rows of a top-64 table: values descending, distinct ids."""
    tv = -np.sort(-rng.normal(0.0, spread, (m, 64)).astype(np.float32), axis=1)
    ti = np.stack([rng.permutation(1000)[:64].astype(np.uint32) for _ in range(m)])
    top = np.concatenate([tv.view(np.uint32), ti], axis=1)
    return tv, ti, np.ascontiguousarray(top)


def lib_accept(sp, top, ids, parents, q, pos, eog=-1):
    L = szlib.load()
    m = len(ids)
    a, p, qq = np.array(ids, dtype=np.uint32), np.array(parents, dtype=np.int32), np.array(q, dtype=np.float32)
    path = np.zeros(m, dtype=np.int32)
    nxt = C.c_uint32()
    n = L.sz_tree_accept_sampled(C.byref(sp), top.ctypes.data, a.ctypes.data, p.ctypes.data, m, qq.ctypes.data, pos, eog, path.ctypes.data, C.byref(nxt))
    return [int(t) for t in path[:n]], int(nxt.value)


def test_library_and_oracle_decide_alike():
    rng = np.random.default_rng(5)
    parents = [-1, 0, 0, 1, 1, 2, 3, 5]
    kept = 0
    for trial in range(300):
        tv, ti, top = top_rows(rng, 8)
        # drafts: often one of the row's likely tokens, sometimes anything
        ids = [int(ti[0, 0])] + [int(ti[parents[j], rng.integers(0, 4)]) if rng.random() < 0.8 else int(rng.integers(0, 1000)) for j in range(1, 8)]
        q = [1.0] + [float(rng.uniform(0.05, 1.0)) for _ in range(7)]
        sp_l = md.Sampler(0.7, 20, 0.9, 0.0, 11 + trial)
        sp_o = ob.SamplerC(0.7, 20, 0.9, 0.0, 11 + trial)
        eog = int(ids[3]) if trial % 7 == 0 else -1
        got = lib_accept(sp_l, top, ids, parents, q, 40 + trial, eog)
        want = ob.tree_accept_sampled(sp_o, tv, ti, ids, parents, q, 40 + trial, eog)
        assert got == want, trial
        path = got[0]
        assert path[0] == 0 and all(parents[path[i]] == path[i - 1] for i in range(1, len(path)))
        assert eog < 0 or all(ids[a] != eog for a in path[1:])
        kept += len(path) - 1
    assert kept > 100                                            # the rule does accept


def test_the_emitted_token_is_distributed_as_the_target_under_a_deterministic_drafter():
    # A drafter that proposes fixed tokens (probability 1 each - a lookup or suffix drafter): a child with token x is kept with
    # probability p(x), a refusal removes x from p, and what is not kept is drawn from the rest - so the token that comes out after
    # the root, a kept child's or the residual draw, must follow the target's p exactly.  One level, p over 6 candidates, three
    # drafted children; many seeds; compared with a plain draw from the same candidates (sz_sample_top) as the yardstick of noise.
    tv = np.full((4, 64), -1e9, dtype=np.float32)
    tv[:, :6] = np.array([2.0, 1.5, 1.0, 0.2, -0.3, -1.0], dtype=np.float32)
    ti = np.tile(np.arange(64, dtype=np.uint32) + 100, (4, 1))
    top = np.ascontiguousarray(np.concatenate([tv.view(np.uint32), ti], axis=1))
    sp_kw = (1.0, 64, 1.0, 0.0)
    p = np.exp(tv[0, :6].astype(np.float64) - 2.0)
    p /= p.sum()
    N = 30000
    counts, plain = np.zeros(6), np.zeros(6)
    kept = 0
    L = szlib.load()
    ids = [100, 103, 100, 105]                                  # children: tokens 3, 0 and 5 of the candidates, in that order
    for seed in range(N):
        sp = md.Sampler(*sp_kw, seed)
        path, nxt = lib_accept(sp, top, ids, [-1, 0, 0, 0], [1.0, 1.0, 1.0, 1.0], 7)
        tok = ids[path[1]] if len(path) > 1 else nxt
        kept += len(path) - 1
        counts[tok - 100] += 1
        plain[int(L.sz_sample_top(C.byref(sp), top[0].ctypes.data_as(C.POINTER(C.c_uint32)), 7)) - 100] += 1
    err = np.abs(counts / N - p).max()
    noise = np.abs(plain / N - p).max()
    assert noise < 0.01 and err < 0.01, (err, noise, counts / N, p)
    assert abs(kept / N - (p[3] + p[0] + p[5])) < 0.01          # a child is kept exactly as often as the target would have said its token
    # a child whose draft probability equals the target's is always kept
    rng = np.random.default_rng(9)
    keptn = 0
    for seed in range(2000):
        d = int(rng.choice(6, p=p))
        path, _ = lib_accept(md.Sampler(*sp_kw, seed), top, [100, 100 + d], [-1, 0], [1.0, float(p[d])], 3)
        keptn += len(path) - 1
    assert keptn == 2000
