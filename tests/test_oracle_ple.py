"""The per-layer embedding (hashed n-gram memory, forward.rs:1036-1074, 1177-1198) in the CPU restatement."""
import ctypes as C

import numpy as np

from oracle import binding as ob
from tests.util import pkg

md = pkg.model

# one PLE layer (layer 1), n-grams of 2 and 3 tokens, 2 heads each: 4 table rows of 64 weights make the embedding of a 256-wide model
PLE = dict(md.TINY, n_layer=4, hidden=256, hc_rank=32, vocab=512, n_head=4, n_kv_head=2, head_dim=64, n_expert=8, n_expert_used=2, expert_ff=128,
           shared_ff=128, ssm_k_heads=2, ssm_v_heads=2, ssm_head_dim=64,
           ple_layer=1, ple_ngram=3, ple_heads_per_ngram=2, ple_head_dim=64, ple_conv_k=4, ple_eos=7,
           ple_multipliers=[-7046029254386353131, 1442695040888963407, 6364136223846793005],
           ple_vocab=[1009, 1013, 1019, 1021], ple_offsets=[0, 1009, 2022, 3041])


def rows_py(cfg, tokens):
    """forward.rs:1177-1198 in plain Python integers (64-bit wrapping by masking)."""
    M = (1 << 64) - 1
    n, eos = len(tokens), cfg["ple_eos"]
    last = max((i for i, t in enumerate(tokens) if t == eos), default=None)

    def hist(s):
        i = n - 1 - s
        return tokens[i] if i >= 0 and (last is None or i >= last) else eos

    def signed(v):
        return v - (1 << 64) if v >> 63 else v

    out = []
    for order in range(2, cfg["ple_ngram"] + 1):
        mixed = (hist(0) * cfg["ple_multipliers"][0]) & M
        for s in range(1, order):
            mixed ^= (hist(s) * cfg["ple_multipliers"][s]) & M
        for j in range(cfg["ple_heads_per_ngram"]):
            i = (order - 2) * cfg["ple_heads_per_ngram"] + j
            out.append(signed(mixed) % cfg["ple_vocab"][i] + cfg["ple_offsets"][i])   # Python's % is the non-negative remainder
    return out


def test_the_table_rows_of_a_history_with_an_end_of_text_in_it():
    hm = md.HostModel(md.make_model(PLE, seed=2))
    L = ob.lib()
    L.szo_ple_rows.restype = C.c_int
    L.szo_ple_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    rng = np.random.default_rng(1)
    for trial in range(200):
        n = int(rng.integers(1, 9))
        toks = [int(t) for t in rng.integers(0, 512, n)]
        if trial % 3 == 0:
            toks[int(rng.integers(0, n))] = PLE["ple_eos"]
        a = np.array(toks, dtype=np.uint32)
        rows = np.zeros(32, dtype=np.int64)
        nr = L.szo_ple_rows(C.byref(hm.model.ple), a.ctypes.data, n, rows.ctypes.data)
        assert list(rows[:nr]) == rows_py(PLE, toks)


def test_the_memory_changes_the_stream_and_a_restored_session_carries_its_history():
    M = md.make_model(PLE, seed=2)
    hm = md.HostModel(M)
    plain = md.HostModel(dict(M, cfg={k: v for k, v in PLE.items() if not k.startswith("ple_")}))
    rng = np.random.default_rng(5)
    toks = [int(t) for t in rng.integers(0, 512, 24)]
    toks[9] = PLE["ple_eos"]
    a, b, c = ob.Session(hm, kv_q8=True, threads=4), ob.Session(hm, kv_q8=True, threads=4), ob.Session(plain, kv_q8=True, threads=4)
    differs = 0
    for i, t in enumerate(toks[:16]):
        la, lb, lc = a.step(t), b.step(t), c.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and np.all(np.isfinite(la))
        differs += int(not np.array_equal(la, lc))
    assert differs == 16                                # the layer is not a no-op
    snap = a.clone()
    for t in (3, 7, 5, 9, 11):                         # a rejected stretch: ten rows of conv history, an end-of-text among them
        a.step(t)
    a.assign(snap)
    for t in toks[16:]:
        la, lb = a.step(t), b.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
