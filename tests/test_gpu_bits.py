"""A guard for changes that are meant to keep every bit (index arithmetic, the same additions in another place): the logits and
top-64 of fixed passes of 1..8 rows on three seeded models hash to what tests/golden/session_bits.json recorded on a B200.  The
comparisons with the CPU restatement are elsewhere; a change that is MEANT to move bits regenerates the file
(tests/golden/make_session_bits.py)."""
import importlib.util
import json
import os

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_fixed_passes_hash_to_the_recorded_bits():
    spec = importlib.util.spec_from_file_location("_make_session_bits", os.path.join(HERE, "golden", "make_session_bits.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    want = json.load(open(os.path.join(HERE, "golden", "session_bits.json")))
    assert mod.session_bits() == want
