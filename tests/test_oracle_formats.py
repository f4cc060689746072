"""The oracle's number formats and dequantisers against the reference's own known answers and gguf-py."""
import os

import numpy as np
import pytest

from oracle import binding as ob


def test_f16_known_values_and_round_trip():
    # half.rs:74-90 (known_values) and 93-104 (every_f16_round_trips)
    L = ob.lib()
    assert L.szo_f16_to_f32(0x3c00) == 1.0 and L.szo_f16_to_f32(0xc000) == -2.0
    assert L.szo_f16_to_f32(0x7bff) == 65504.0
    assert L.szo_f16_to_f32(0x0001) == 2.0 ** -24 and L.szo_f16_to_f32(0x03ff) == 1023.0 * 2.0 ** -24
    assert L.szo_f16_to_f32(0x7c00) == float("inf") and np.isnan(L.szo_f16_to_f32(0x7e00))
    assert L.szo_f32_to_f16(1.0) == 0x3c00 and L.szo_f32_to_f16(65520.0) == 0x7c00
    assert L.szo_f32_to_f16(2.0 ** -25) == 0 and L.szo_f32_to_f16(3.0 * 2.0 ** -25) == 2
    assert L.szo_bf16_to_f32(0x3f80) == 1.0 and L.szo_f32_to_bf16(1.0) == 0x3f80
    tie = np.array([0x3f808000, 0x3f818000], dtype=np.uint32).view(np.float32)
    assert L.szo_f32_to_bf16(float(tie[0])) == 0x3f80 and L.szo_f32_to_bf16(float(tie[1])) == 0x3f82
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    for h in range(0, 65536):
        f = L.szo_f16_to_f32(h)
        if np.isnan(ref[h]):
            assert np.isnan(f)
        else:
            assert f == ref[h], hex(h)
            assert L.szo_f32_to_f16(f) == h, hex(h)


def test_f64_to_f16_rounding_table():
    # exl3.rs:606-619
    L = ob.lib()
    f = L.szo_f64_to_f16_bits
    assert f(1.0) == 0x3c00 and f(-2.0) == 0xc000 and f(65504.0) == 0x7bff and f(65520.0) == 0x7c00
    assert f(6.103515625e-5) == 0x0400 and f(5.960464477539063e-8) == 0x0001
    assert f(1.0 + 2.0 ** -11) == 0x3c00 and f(1.0 + 3.0 * 2.0 ** -11) == 0x3c02
    for bits in range(0, 0x7c00):
        assert f(float(np.uint16(bits).view(np.float16))) == bits


def _records(path):
    lines = [l for l in open(path).read().splitlines() if l and not l.startswith("#")]
    assert len(lines) % 3 == 0
    for i in range(0, len(lines), 3):
        ty, tensor, block = lines[i].split()
        yield ty, tensor, block, bytes.fromhex(lines[i + 1]), np.frombuffer(bytes.fromhex(lines[i + 2]), dtype=">u4")


def test_reference_known_answer_blocks_bit_for_bit(golden_dir):
    # the reference's own fixture records (checker: crates/shadowzero-model/tests/dequant.rs:32-57)
    ids = {"F32": ob.F32, "F16": ob.F16, "BF16": ob.BF16, "IQ3_S": ob.IQ3_S}
    seen = {}
    for ty, tensor, block, data, want in _records(os.path.join(golden_dir, "dequant_ref.txt")):
        got = ob.dequant(ids[ty], np.frombuffer(data, dtype=np.uint8)).view(np.uint32)
        assert np.array_equal(got, want.astype(np.uint32)), (ty, tensor, block)
        seen[ty] = seen.get(ty, 0) + 1
    assert seen == {"F32": 8, "F16": 4, "BF16": 8, "IQ3_S": 8}


@pytest.mark.parametrize("name,ty", [("q8_0", ob.Q8_0), ("iq3_s", ob.IQ3_S)])
def test_gguf_py_agrees_bit_for_bit(golden_dir, name, ty):
    z = np.load(os.path.join(golden_dir, "gguf_dequant.npz"))
    got = ob.dequant(ty, z[name + "_bytes"]).view(np.uint32)
    assert np.array_equal(got, z[name + "_f32"].reshape(-1))


def test_q8_0_by_hand():
    blk = np.zeros(34, dtype=np.uint8)
    blk[:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
    blk[2:] = np.arange(-16, 16, dtype=np.int8).view(np.uint8)
    assert np.array_equal(ob.dequant(ob.Q8_0, blk), 0.5 * np.arange(-16, 16, dtype=np.float32))


def test_dequant_refuses_bad_sizes():
    with pytest.raises(ValueError):
        ob.dequant(ob.Q8_0, np.zeros(35, dtype=np.uint8))
