"""Writes tests/golden/session_bits.json: SHA-256 of the logits and top-64 of fixed verify passes (1..8 rows) on three seeded models,
as THIS library computes them on a B200.  Not a parity fixture (the oracle comparisons are the parity tests): a guard for changes
that are meant to keep every bit - index arithmetic, another order of the same additions, a kernel split in two.  Run on a GPU
after a change that is MEANT to move bits:  python tests/golden/make_session_bits.py"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

C3_SLICE = dict(n_layer=4, hidden=2048, streams=4, hc_rank=256, vocab=4096, n_head=16, n_kv_head=2, head_dim=256, rope_dims=64,
                n_expert=512, n_expert_used=10, expert_ff=512, shared_ff=512, ssm_k_heads=16, ssm_v_heads=32, ssm_head_dim=128,
                conv_k=4, attn_interval=4, eps=1e-6, rope_theta=1e7)


def session_bits():
    from tests.util import pkg
    from tests.test_oracle_ple import PLE
    szlib, md = pkg.lib, pkg.model
    out = {}
    cases = (("tiny", dict(md.TINY, vocab=2048), {}),
             ("c3", C3_SLICE, dict(dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_EXL3(3))),
             ("ple32", PLE, {}))
    for name, cfg, kw in cases:
        dm = md.DeviceModel(md.make_model(cfg, seed=5, **kw))
        s = md.Session(dm, 64, kv_q8=True)
        rng = np.random.default_rng(3)
        h = hashlib.sha256()
        for m in (1, 2, 3, 4, 5, 6, 7, 8):
            s.verify([int(t) for t in rng.integers(0, cfg["vocab"], m)])
            _, top, lg = s.result(logits=True)
            h.update(lg.tobytes())
            h.update(top.tobytes())
            s.commit(m)
        out[name] = h.hexdigest()
    return out


if __name__ == "__main__":
    bits = session_bits()
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "session_bits.json"), "w") as f:
        json.dump(bits, f, indent=1)
    print(bits)
