"""Builds the committed golden fixtures.  Run once in the build container, where the reference tree is mounted:

    python tests/golden/make_golden.py [/root/reference]

Writes, beside this script:

  dequant_ref.txt       the IQ3_S, F16, BF16 and F32 known-answer records of the reference's own fixture
                        eval/fixtures/dequant.txt (block bytes -> expected f32 bit patterns, made by the reference's
                        tools/gen_dequant_fixtures.py from ggml's dequantiser); the checker they pin is
                        crates/shadowzero-model/tests/dequant.rs:32-57.
  exl3_real_slice.npz   a 256-input x 128-output corner of the first real EXL3 projection in
                        eval/fixtures/exl3_sample.safetensors (expert 0 gate_proj, K = 2, codebook "mul1"), as a blob
                        in the reference's blob layout (crates/shadowzero-model/src/exl3.rs:388-398).  No expected
                        outputs exist for it; it is an input for the reconstruct() . x == matvec(x) identity
                        (exl3.rs:643-672) with a real checkpoint's suh / svh scales.  The mounted copy of that file is
                        12 bytes short (its second codebook marker sits 5 bytes early: a line-ending conversion ate
                        bytes of the binary), so the second projection (K = 4) is unreadable and is left out, and the
                        trellis words of the first may be shifted against the original checkpoint; every bit string
                        is a valid trellis, so the identity holds regardless.
  gguf_dequant.npz      random Q8_0 and IQ3_S blocks with the f32 values gguf-py 0.19.0 (gguf.quants.dequantize)
                        decodes them to: the second, independent pin of the two ggml formats.
"""
import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def dequant_records(ref):
    keep = {"IQ3_S", "F16", "BF16", "F32"}
    lines = [l for l in open(os.path.join(ref, "eval/fixtures/dequant.txt")).read().splitlines()
             if l and not l.startswith("#")]
    assert len(lines) % 3 == 0
    out = ["# TYPE TENSOR BLOCK / block bytes (hex) / expected f32 bit patterns (hex, big-endian words)",
           "# extracted by tests/golden/make_golden.py from the reference's eval/fixtures/dequant.txt"]
    n = 0
    for i in range(0, len(lines), 3):
        if lines[i].split()[0] in keep:
            out += lines[i:i + 3]
            n += 1
    open(os.path.join(HERE, "dequant_ref.txt"), "w").write("\n".join(out) + "\n")
    return n


def exl3_slices(ref):
    path = os.path.join(ref, "eval/fixtures/exl3_sample.safetensors")
    f = open(path, "rb")
    n = struct.unpack("<Q", f.read(8))[0]
    head = json.loads(f.read(n))
    base = 8 + n
    raw = open(path, "rb").read()

    def tensor(name, dt):
        t = head[name]
        a, b = t["data_offsets"]
        buf = raw[base + a:base + b]
        buf += bytes(b - a - len(buf))  # the fixture file ends 12 bytes short of its last tensor; the slice taken is not near it
        return np.frombuffer(buf, dtype=dt).reshape(t["shape"])

    out = {}
    for tag, prefix in (("k2", "model.language_model.layers.0.mlp.experts.0.gate_proj"),):
        tr = tensor(prefix + ".trellis", np.uint16)       # [in/16, out/16, 16 K]
        suh = tensor(prefix + ".suh", np.uint16)           # f16 bits
        svh = tensor(prefix + ".svh", np.uint16)
        kin, kout = 256, 128                               # two input blocks, one output block of 128
        sl = np.ascontiguousarray(tr[:kin // 16, :kout // 16, :])
        blob = suh[:kin].tobytes() + svh[:kout].tobytes() + struct.pack("<i", 1) + sl.tobytes()
        out[tag + "_blob"] = np.frombuffer(blob, dtype=np.uint8)
        out[tag + "_shape"] = np.array([kin, kout, tr.shape[2] // 16], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "exl3_real_slice.npz"), **out)


def gguf_vectors():
    from gguf import quants, GGMLQuantizationType as T
    rng = np.random.default_rng(0x5a17)
    out = {}
    # Q8_0: random int8 codes, scales over a wide range of f16 values (including subnormals and zero)
    nb = 256
    blk = rng.integers(0, 256, size=(nb, 34), dtype=np.uint8)
    d = rng.standard_normal(nb).astype(np.float32) * np.float32(0.01)
    d[:4] = [0.0, 6e-8, -1.5e-5, 1.0]
    blk[:, :2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
    out["q8_0_bytes"] = blk
    out["q8_0_f32"] = quants.dequantize(blk.reshape(-1), T.Q8_0).astype(np.float32).view(np.uint32)
    # IQ3_S: fully random payload (every bit pattern is a valid block), sane f16 scale
    nb = 96
    blk = rng.integers(0, 256, size=(nb, 110), dtype=np.uint8)
    d = (rng.standard_normal(nb).astype(np.float32) * np.float32(2e-4))
    blk[:, :2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
    out["iq3_s_bytes"] = blk
    out["iq3_s_f32"] = quants.dequantize(blk.reshape(-1), T.IQ3_S).astype(np.float32).view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "gguf_dequant.npz"), **out)


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print("dequant records:", dequant_records(ref))
    exl3_slices(ref)
    gguf_vectors()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
