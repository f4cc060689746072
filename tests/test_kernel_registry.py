"""The kernel-launch seam: the registry of entry points against the CUDA sources, both ways (the reference's tests/drift.rs), the
refusals of a launch that does not fit (crates/shadowzero-cuda/tests/gpu.rs), and on a GPU a launch by name that does the kernel's work."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from tests.util import ROOT, pkg

szlib = pkg.lib
CSRC = os.path.join(ROOT, "shadow-engine_b200", "csrc")
FILES = ("sz_session_kernels.cuh", "sz_topk.cuh", "sz_session.cu")   # the translation unit the registry lives in
SCALARS = {"int": szlib.P_I32, "int32_t": szlib.P_I32, "u32": szlib.P_U32, "uint32_t": szlib.P_U32, "unsigned int": szlib.P_U32, "float": szlib.P_F32,
           "u64": szlib.P_U64, "uint64_t": szlib.P_U64, "int64_t": szlib.P_U64, "size_t": szlib.P_U64, "unsigned long long": szlib.P_U64}


def parse_entries(text):
    """Non-template __global__ functions of a source file -> {name: [parameter types]} (None: a type outside the registry's six)."""
    out = {}
    text = re.sub(r"//[^\n]*", "", text)
    pat = r"(template\s*<[^>]*>\s*)?(?:static\s+)?__global__\s+void(?:\s+__launch_bounds__\([^)]*(?:\([^)]*\))?[^)]*\))?\s+(\w+)\s*\(([^)]*)\)"
    for m in re.finditer(pat, text):
        if m.group(1):
            continue
        types = []
        for p in m.group(3).split(","):
            p = p.replace("__restrict__", " ").strip()
            if not p:
                continue
            if "*" in p:
                types.append(szlib.P_CONST_PTR if p.startswith("const ") else szlib.P_PTR)
            else:
                types.append(SCALARS.get(" ".join(p.split()[:-1]).replace("const ", "")))
        out[m.group(2)] = types
    return out


def registry():
    L = szlib.load()
    out = {}
    for i in range(L.sz_kernel_count()):
        name = L.sz_kernel_name(i)
        buf = (C.c_int32 * 24)()
        n = L.sz_kernel_params(name, buf, 24)
        out[name.decode()] = list(buf[:n])
    return out


def test_signatures_match_both_ways():
    reg = registry()
    assert len(reg) >= 10
    on_disk = {}
    for f in FILES:
        on_disk.update(parse_entries(open(os.path.join(CSRC, f)).read()))
    plain = {k: v for k, v in on_disk.items() if None not in v}
    for name, params in plain.items():
        assert name in reg, "entry point %s is not in the registry" % name
        assert reg[name] == params, "%s's parameters differ from the registry" % name
    for name in reg:
        assert name in plain, "registered %s is not in the sources" % name
    assert szlib.load().sz_kernel_params(b"no_such_kernel", None, 0) == -1


def _args(*pairs):
    a = (szlib.KArg * len(pairs))()
    for i, (ty, v) in enumerate(pairs):
        a[i].type = ty
        a[i].bits = struct.unpack("<I", struct.pack("<f", v))[0] if ty == szlib.P_F32 else int(v) & 0xFFFFFFFFFFFFFFFF
    return a


def test_launches_that_do_not_fit_are_refused_before_the_driver():
    L = szlib.load()
    g, b = (C.c_uint32 * 3)(1, 1, 1), (C.c_uint32 * 3)(32, 1, 1)
    assert L.sz_kernel_launch(b"sz_nothing", g, b, 0, 0, None, 0) == szlib.E_ARG and b"no entry point" in L.sz_last_error()
    a = _args((szlib.P_PTR, 4096), (szlib.P_PTR, 4096), (szlib.P_I32, 1))
    assert L.sz_kernel_launch(b"sz_state_update_kernel", g, b, 0, 0, a, 3) == szlib.E_ARG and b"takes 2 arguments, 3 given" in L.sz_last_error()
    a = _args((szlib.P_PTR, 4096), (szlib.P_U32, 7))
    assert L.sz_kernel_launch(b"sz_state_update_kernel", g, b, 0, 0, a, 2) == szlib.E_ARG and b"does not fit" in L.sz_last_error()
    a = _args((szlib.P_CONST_PTR, 4096), (szlib.P_PTR, 4096))      # a const pointer is not a writable one
    assert L.sz_kernel_launch(b"sz_state_update_kernel", g, b, 0, 0, a, 2) == szlib.E_ARG
    a = _args((szlib.P_PTR, 4096), (szlib.P_PTR, 4096))
    big = (C.c_uint32 * 3)(2048, 1, 1)
    assert L.sz_kernel_launch(b"sz_state_update_kernel", g, big, 0, 0, a, 2) == szlib.E_ARG


@pytest.mark.gpu
def test_a_launch_by_name_does_the_kernels_work():
    import torch
    L = szlib.load()
    # sz_state_update_kernel: positions += kept rows, buffers swap;  sz_hc_mix_kernel: u = mean over streams of mix * rn
    state = torch.tensor([40, 0, 0, 0], dtype=torch.int32, device="cuda")
    res = torch.tensor([3, 99], dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    g, b = (C.c_uint32 * 3)(1, 1, 1), (C.c_uint32 * 3)(32, 1, 1)
    szlib.check(L.sz_kernel_launch(b"sz_state_update_kernel", g, b, 0, st, _args((szlib.P_PTR, state.data_ptr()), (szlib.P_PTR, res.data_ptr())), 2))
    torch.cuda.synchronize()
    assert state.tolist()[:2] == [43, 1]
    H, Cs, m = 512, 4, 3
    mix = torch.rand(m, Cs, H, device="cuda")
    rn = torch.randn(m, Cs, H, device="cuda")
    u = torch.empty(m, H, device="cuda")
    g, b = (C.c_uint32 * 3)((H + 255) // 256, m, 1), (C.c_uint32 * 3)(256, 1, 1)
    szlib.check(L.sz_kernel_launch(b"sz_hc_mix_kernel", g, b, 0, st, _args((szlib.P_PTR, mix.data_ptr()), (szlib.P_PTR, rn.data_ptr()), (szlib.P_I32, H),
                                                                          (szlib.P_I32, Cs), (szlib.P_PTR, u.data_ptr())), 5))
    torch.cuda.synchronize()
    want = torch.zeros(m, H, device="cuda", dtype=torch.float64)
    for s in range(Cs):                                   # stream order, then the division (forward.rs:805-811)
        want = want + mix[:, s].double() * rn[:, s].double()
    assert torch.allclose(u, (want / Cs).float(), rtol=1e-6, atol=1e-7)   # (the kernel's f32 multiply-adds round once a term)
