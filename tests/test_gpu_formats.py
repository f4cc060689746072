"""GPU decoders against the oracle, bit for bit (the reference's crates/shadowzero-cuda/tests/dequant.rs:40-70,
convert.rs:41-93 and exl3.rs:64-77 restated through the C ABI)."""
import os

import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.util import pkg

pytestmark = pytest.mark.gpu
szlib = pkg.lib


def _dequant_gpu(ty, data, n):
    L = szlib.load()
    src = torch.from_numpy(np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)).cuda()
    dst = torch.empty(n, dtype=torch.float32, device="cuda")
    szlib.check(L.sz_dequant(ty, src.data_ptr(), src.numel(), dst.data_ptr(), n, 0))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


def test_every_f16_and_bf16_pattern_converts_exactly():
    allh = np.arange(65536, dtype=np.uint16)
    for ty, oty in ((szlib.TYPE_F16, ob.F16), (szlib.TYPE_BF16, ob.BF16)):
        got = _dequant_gpu(ty, allh.view(np.uint8), 65536)
        want = ob.dequant(oty, allh.view(np.uint8))
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got), nan)
        assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


@pytest.mark.parametrize("name,ty,oty,be", [("q8_0", szlib.TYPE_Q8_0, ob.Q8_0, 32), ("iq3_s", szlib.TYPE_IQ3_S, ob.IQ3_S, 256)])
def test_golden_blocks_decode_bit_for_bit(golden_dir, name, ty, oty, be):
    z = np.load(os.path.join(golden_dir, "gguf_dequant.npz"))
    data = z[name + "_bytes"]
    got = _dequant_gpu(ty, data, data.shape[0] * be)
    assert np.array_equal(got.view(np.uint32), z[name + "_f32"].reshape(-1))
    assert np.array_equal(got.view(np.uint32), ob.dequant(oty, data).view(np.uint32))


def test_reference_iq3_s_known_answers(golden_dir):
    lines = [l for l in open(os.path.join(golden_dir, "dequant_ref.txt")).read().splitlines() if l and not l.startswith("#")]
    n = 0
    for i in range(0, len(lines), 3):
        if lines[i].split()[0] != "IQ3_S":
            continue
        data = np.frombuffer(bytes.fromhex(lines[i + 1]), dtype=np.uint8)
        want = np.frombuffer(bytes.fromhex(lines[i + 2]), dtype=">u4").astype(np.uint32)
        assert np.array_equal(_dequant_gpu(szlib.TYPE_IQ3_S, data, 256).view(np.uint32), want)
        n += 1
    assert n == 8


def test_synthetic_blocks_decode_bit_for_bit():
    synth = pkg.synth
    w = synth.normal((64, 1024), 0.02, 11, "w")
    for ty, oty, q in ((szlib.TYPE_Q8_0, ob.Q8_0, synth.quantize_q8_0(w)), (szlib.TYPE_IQ3_S, ob.IQ3_S, synth.quantize_iq3_s(w))):
        got = _dequant_gpu(ty, q.numpy(), w.numel())
        assert np.array_equal(got.view(np.uint32), ob.dequant(oty, q.numpy()).view(np.uint32))


def test_exl3_codebook_all_states():
    L = szlib.load()
    dst = torch.empty(65536, dtype=torch.float32, device="cuda")
    szlib.check(L.sz_exl3_codebook(dst.data_ptr(), 0))
    torch.cuda.synchronize()
    want = np.array([ob.lib().szo_exl3_cb(2, s) for s in range(65536)], dtype=np.float32)
    assert np.array_equal(dst.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_exl3_tile_decode_every_rate(bits):
    # W_hat of a random blob equals the oracle's tile-by-tile decode (reference: tests/exl3.rs random blobs at K = 1..8)
    L = szlib.load()
    n_in, n_out = 256, 384
    blob = pkg.synth.random_exl3_blobs(1, n_in, n_out, bits, 0.02, 40 + bits, "t")[0]
    buf, addr, _ = pkg.moe.place(blob.reshape(1, -1), "cuda", 0)
    dst = torch.empty((n_in, n_out), dtype=torch.float32, device="cuda")
    szlib.check(L.sz_exl3_reconstruct_inner(bits, addr, n_in, n_out, dst.data_ptr(), 0))
    torch.cuda.synchronize()
    tr = blob.numpy()[2 * n_in + 2 * n_out + 4:].view(np.uint16).reshape(n_in // 16, n_out // 16, 16 * bits)
    want = np.empty((n_in, n_out), dtype=np.float32)
    import ctypes as C
    pos = []
    for p in range(256):
        r, c = C.c_int(), C.c_int()
        ob.lib().szo_exl3_tile_pos(p, C.byref(r), C.byref(c))
        pos.append((r.value, c.value))
    for k in range(n_in // 16):
        for n in range(n_out // 16):
            vals = ob.exl3_decode_tile(tr[k, n], bits)
            for p, (r, c) in enumerate(pos):
                want[k * 16 + r, n * 16 + c] = vals[p]
    assert np.array_equal(dst.cpu().numpy().view(np.uint32), want.view(np.uint32))
