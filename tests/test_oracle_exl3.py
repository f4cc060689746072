"""The oracle's EXL3 decoder: the reference's unit tests restated (exl3.rs:601-715) plus a real-tensor slice."""
import os

import numpy as np

from oracle import binding as ob


class XorShift:
    """The xorshift64 the reference's tests seed their data with (exl3.rs:624-631)."""

    def __init__(self, seed):
        self.s = seed

    def next(self):
        m = (1 << 64) - 1
        s = self.s
        s ^= (s << 13) & m
        s ^= s >> 7
        s ^= (s << 17) & m
        self.s = s
        return s


def test_fast_tile_decode_equals_the_bit_loop():
    # exl3.rs:622-641
    rng = XorShift(0x9e3779b97f4a7c15)
    for cb in range(3):
        for bits in range(1, 9):
            tile = np.array([rng.next() & 0xffff for _ in range(16 * bits)], dtype=np.uint16)
            a = ob.exl3_decode_tile(tile, bits, cb)
            b = ob.exl3_decode_tile(tile, bits, cb, fast=True)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (cb, bits)
    for bits in (1, 2, 3):  # K + 0.5, codebook mul1 only
        tile = np.array([rng.next() & 0xffff for _ in range(16 * bits + 8)], dtype=np.uint16)
        a = ob.exl3_decode_tile(tile, bits, 2, half=1)
        b = ob.exl3_decode_tile(tile, bits, 2, half=1, fast=True)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), bits


def _random_linear(rng, inf, outf, bits):
    trellis = np.array([rng.next() & 0xffff for _ in range(inf // 16 * outf // 16 * 16 * bits)], dtype=np.uint16)
    suh = np.array([1.0 if rng.next() & 1 == 0 else -1.0 for _ in range(inf)], dtype=np.float16)
    svh = np.array([(rng.next() % 100) / 50.0 - 1.0 for _ in range(outf)], dtype=np.float32).astype(np.float16)
    blob = np.frombuffer(suh.tobytes() + svh.tobytes() + (1).to_bytes(4, "little") + trellis.tobytes(), dtype=np.uint8)
    return blob


def test_rotated_basis_matvec_equals_reconstructed_matrix_times_x():
    # exl3.rs:643-672: same seed, shapes, data recipe and tolerance (2e-4 of the largest output)
    rng = XorShift(0x2545f4914f6cdd1d)
    for inf, outf, bits in ((256, 128, 2), (128, 256, 3), (384, 256, 4)):
        blob = _random_linear(rng, inf, outf, bits)
        assert blob.size == ob.exl3_blob_len(inf, outf, bits)
        x = np.array([(rng.next() % 2000) / 1000.0 - 1.0 for _ in range(inf)], dtype=np.float32)
        w = ob.exl3_reconstruct(inf, outf, bits, blob)
        want = x.astype(np.float64) @ w.astype(np.float64)
        scale = max(np.abs(want).max(), 1e-9)
        for threads in (1, 3):
            got = ob.matvec(ob.EXL3_BASE + bits, blob, outf, inf, x, threads)
            assert np.abs(got - want).max() < 2e-4 * scale, (inf, outf, bits, threads)


def test_tile_positions_are_a_bijection():
    # exl3.rs:674-682
    import ctypes as C
    seen = set()
    for p in range(256):
        r, c = C.c_int(), C.c_int()
        ob.lib().szo_exl3_tile_pos(p, C.byref(r), C.byref(c))
        assert 0 <= r.value < 16 and 0 <= c.value < 16
        seen.add((r.value, c.value))
    assert len(seen) == 256


def test_hadamard_is_its_own_inverse():
    # exl3.rs:684-696
    v = np.array([(i * 37 % 11) - 5.0 for i in range(128)], dtype=np.float32)
    assert np.abs(ob.wht128(ob.wht128(v)) - v).max() < 1e-4
    # and it is the Sylvester matrix: row i, column j has sign (-1)^popcount(i & j)
    e = np.zeros(128, dtype=np.float32)
    e[5] = 1.0
    want = np.array([(-1.0) ** bin(5 & j).count("1") for j in range(128)]) / np.sqrt(128.0)
    assert np.abs(ob.wht128(e) - want).max() < 1e-6


def test_codebooks_look_like_a_unit_gaussian():
    # exl3.rs:698-714
    L = ob.lib()
    for cb in range(3):
        v = np.array([L.szo_exl3_cb(cb, s) for s in range(65536)], dtype=np.float64)
        assert np.isfinite(v).all()
        assert abs(v.mean()) < 0.1 and 0.7 < v.std() < 1.3
        assert np.array_equal(v.astype(np.float16).astype(np.float64), v), "codebook values are exact f16"


def test_mul1_codebook_from_its_definition():
    # codebook 2 independently in numpy float16 arithmetic: an fma in f16 = one rounding of the exact product-sum
    s = np.arange(65536, dtype=np.uint64)
    x = (s * 0x83DCD12D) & 0xffffffff
    total = 0x6400 + (x & 0xff) + ((x >> 8) & 0xff) + ((x >> 16) & 0xff) + (x >> 24)
    h = total.astype(np.uint16).view(np.float16).astype(np.float64)
    kinv = float(np.uint16(0x1eee).view(np.float16))
    kbias = float(np.uint16(0xc931).view(np.float16))
    want = (h * kinv + kbias).astype(np.float16).astype(np.float32)  # exact in f64, rounded once
    L = ob.lib()
    got = np.array([L.szo_exl3_cb(2, int(i)) for i in range(65536)], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_real_tensor_slices(golden_dir):
    # a real EXL3 projection's corner (K = 2): blob matvec against the reconstructed matrix (tests/exl3.rs:405-430)
    z = np.load(os.path.join(golden_dir, "exl3_real_slice.npz"))
    rng = np.random.default_rng(7)
    for tag in ("k2",):
        inf, outf, bits = (int(v) for v in z[tag + "_shape"])
        blob = z[tag + "_blob"]
        x = rng.uniform(-1, 1, inf).astype(np.float32)
        w = ob.exl3_reconstruct(inf, outf, bits, blob)
        assert np.isfinite(w).all() and 1e-4 < w.std() < 1.0
        want = x.astype(np.float64) @ w.astype(np.float64)
        got = ob.matvec(ob.EXL3_BASE + bits, blob, outf, inf, x, 2)
        assert np.abs(got - want).max() < 2e-4 * np.abs(want).max()
