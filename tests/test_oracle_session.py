"""The oracle's session helpers that the GPU parity tests lean on (CPU only): the synthetic history and the state accessors."""
import numpy as np

from oracle import binding as ob
from tests.util import pkg

md = pkg.model
SMALL = dict(md.TINY, vocab=512, n_expert=8, expert_ff=128, shared_ff=128)


def test_synthetic_history_and_state_pieces():
    M = md.make_model(SMALL, seed=3)
    hm = md.HostModel(M)
    for q8 in (True, False):
        s = ob.Session(hm, kv_q8=q8, threads=2)
        s.fill_synthetic(37, seed=5)
        assert len(s) == 37
        hb = 80 if q8 else 256
        k, v = s.state(2, 3), s.state(3, 3)
        assert k.size == v.size == 37 * SMALL["n_kv_head"] * hb and not np.array_equal(k, v)
        if q8:
            heads = k.reshape(37, SMALL["n_kv_head"], hb)
            codes = heads[..., :64].view(np.int8)
            assert codes.min() >= -127 and codes.max() <= 127 and len(np.unique(codes)) > 200
            assert (heads[..., 64:68].copy().view(np.uint16) == 0x2000).all() and not heads[..., 68:].any()
        else:
            assert np.abs(k.view(np.float32)).max() <= 1.0
        assert not s.state(0, 0).any() and not s.state(1, 0).any()
        # the same seed fills the same bytes; a step on top of the history works and moves the recurrent state
        t = ob.Session(hm, kv_q8=q8, threads=2)
        t.fill_synthetic(37, seed=5)
        assert np.array_equal(t.state(2, 3), k)
        lg = s.step(7)
        assert np.isfinite(lg).all() and len(s) == 38 and s.state(0, 0).any()
        assert s.state(0, 0).size == SMALL["ssm_v_heads"] * 64 * 64 and s.state(1, 0).size == 3 * 3 * 4 * 64
