"""The C-ABI library loads, exports every symbol the header declares, and refuses bad arguments before touching a GPU."""
import ctypes as C
import os
import re

import pytest

from tests.util import ROOT, pkg

szlib = pkg.lib


def _declared():
    text = open(os.path.join(ROOT, "include", "shadowzero_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sz_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    L = szlib.load()
    names = _declared()
    assert len(names) >= 9
    for n in names:
        assert hasattr(L, n), n
        assert n in szlib.SYMBOLS, "no ctypes signature for %s" % n
    assert sorted(szlib.SYMBOLS) == names
    assert b"sm_100a" in L.sz_version()


def _layer(**kw):
    c = szlib.MoeLayerC()
    d = dict(hidden=256, n_expert=16, top_k=4, expert_ff=256, shared_ff=0, expert_type=szlib.TYPE_Q8_0,
             shared_type=szlib.TYPE_Q8_0, router=4096, gate=4096, up=4096, down=4096, gate_stride=4096, up_stride=4096,
             down_stride=4096)
    d.update(kw)
    for k, v in d.items():
        setattr(c, k, v)
    return c


def test_scratch_query_is_pure_and_checks_arguments():
    L = szlib.load()
    n = C.c_int64()
    assert L.sz_moe_scratch_bytes(C.byref(_layer()), 4, C.byref(n)) == szlib.OK and n.value > 0
    small = n.value
    assert L.sz_moe_scratch_bytes(C.byref(_layer()), 8, C.byref(n)) == szlib.OK and n.value > small
    for bad, code in ((dict(top_k=17), szlib.E_ARG), (dict(hidden=100), szlib.E_ARG), (dict(expert_type=12), szlib.E_TYPE),
                      (dict(n_expert=2000), szlib.E_ARG), (dict(gate=4100), szlib.E_ARG), (dict(up_stride=40), szlib.E_ARG),
                      (dict(expert_type=szlib.TYPE_IQ3_S, expert_ff=128), szlib.E_ARG),
                      (dict(expert_type=szlib.TYPE_EXL3(3)), szlib.E_ARG)):  # EXL3: the trellis, not the blob, is aligned
        assert L.sz_moe_scratch_bytes(C.byref(_layer(**bad)), 4, C.byref(n)) == code, bad
        assert len(L.sz_last_error()) > 0
    assert L.sz_moe_scratch_bytes(C.byref(_layer()), 0, C.byref(n)) == szlib.E_ARG
    assert L.sz_moe_scratch_bytes(C.byref(_layer()), 9, C.byref(n)) == szlib.E_ARG
    ok = _layer(expert_type=szlib.TYPE_EXL3(3), gate=4096 + 12, up=4096 + 12, down=4096 + 12)
    assert L.sz_moe_scratch_bytes(C.byref(ok), 4, C.byref(n)) == szlib.OK


def test_compute_calls_refuse_bad_arguments_without_launching():
    L = szlib.load()
    assert L.sz_dequant(szlib.TYPE_Q8_0, 4096, 35, 8192, 32, 0) == szlib.E_ARG
    assert L.sz_dequant(12, 4096, 144, 8192, 256, 0) == szlib.E_TYPE
    assert L.sz_exl3_reconstruct_inner(9, 4096, 128, 128, 8192, 0) == szlib.E_TYPE
    assert L.sz_exl3_reconstruct_inner(3, 4096, 100, 128, 8192, 0) == szlib.E_ARG
    assert L.sz_moe_verify(C.byref(_layer()), 0, 4, 4096, 0, 0, 4096, 1 << 20, 0) == szlib.E_ARG
    assert L.sz_moe_verify(C.byref(_layer()), 4096, 4, 4096, 0, 0, 4096, 16, 0) == szlib.E_SCRATCH
    with pytest.raises(szlib.SzError):
        szlib.check(L.sz_moe_verify(C.byref(_layer()), 4096, 4, 4096, 0, 0, 4097, 1 << 20, 0))


def test_head_calls_check_their_arguments_without_launching():
    L = szlib.load()
    n = C.c_int64()
    assert L.sz_head_work_bytes(4096, 512, 16, C.byref(n)) == szlib.OK and n.value > 0
    assert L.sz_head_work_bytes(4000, 512, 16, C.byref(n)) == szlib.E_ARG
    assert L.sz_head_work_bytes(4096, 8192, 16, C.byref(n)) == szlib.E_ARG
    h = szlib.HeadC(rows=4096, cols=512, bits=7, k_blk=0, weight=4096 + 12, work=4096, work_bytes=1 << 30)
    assert L.sz_head_top(C.byref(h), 4096, 512, 4, 64, 4096, 4096, 0) == szlib.E_TYPE
    h.bits = 4
    h.weight = 4096
    assert L.sz_head_top(C.byref(h), 4096, 512, 4, 64, 4096, 4096, 0) == szlib.E_ARG
    h.weight = 4096 + 12
    assert L.sz_head_top(C.byref(h), 4096, 512, 9, 64, 4096, 4096, 0) == szlib.E_ARG
    h.work_bytes = 16
    assert L.sz_head_top(C.byref(h), 4096, 512, 4, 64, 4096, 4096, 0) == szlib.E_SCRATCH
    h.work_bytes = 1 << 30
    ku, ms, ls = C.c_int32(), C.c_int32(), C.c_int64()
    h.k_blk = 128                                                   # clamped to the 32 blocks there are
    h.w_q2, h.w_sc = 4096, 4096
    assert L.sz_head_plan(C.byref(h), 4, 64, C.byref(ku), C.byref(ms), C.byref(ls)) == szlib.OK
    assert (ku.value, ms.value, ls.value) == (32, 32, 4096)
    h.rows, h.k_blk = 151936, 128
    assert L.sz_head_plan(C.byref(h), 4, 64, C.byref(ku), C.byref(ms), C.byref(ls)) == szlib.OK
    assert (ku.value, ms.value, ls.value) == (128, 512, 65536)
    assert L.sz_head_plan(C.byref(h), 1, 16, C.byref(ku), C.byref(ms), C.byref(ls)) == szlib.OK and ku.value == 96   # session.rs:5964
    h.k_blk = 0
    assert L.sz_head_plan(C.byref(h), 8, 64, C.byref(ku), C.byref(ms), C.byref(ls)) == szlib.OK and ls.value == 151936
    q2, sc = C.c_int64(), C.c_int64()
    assert L.sz_head_proxy_bytes(151936, 2048, C.byref(q2), C.byref(sc)) == szlib.OK
    assert q2.value + sc.value == 82_653_184                        # the 82.7 MB of the reference's proxy at this shape
