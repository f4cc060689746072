"""Model files: the library's GGUF reader against the reference's own hand-written file (crates/shadowzero-model/src/gguf.rs:545-615,
restated byte for byte), against gguf-py as an independent reader of the files this repository writes, and - the point of a loader -
a model written to a file, read back and stepped must give the bits of the model it was written from."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from oracle import binding as ob
from tests.util import pkg

szlib, md, gio = pkg.lib, pkg.model, pkg.gguf_io
SMALL = dict(md.TINY, vocab=512, n_expert=8, expert_ff=128, shared_ff=256, n_layer=4)


def put_str(s):
    return struct.pack("<Q", len(s)) + s.encode()


def reference_toy_file(path):
    """The two-tensor file of the reference's reader test (gguf.rs:545-583): 3 key-values (a string, a u32, an array of 2 strings),
    blk.0.w = 32 x 2 F32 at offset 0, blk.1.q = 256 IQ3_S weights (110 bytes) at offset 256, data = 366 bytes of 7."""
    b = b"GGUF" + struct.pack("<IQQ", 3, 2, 3)
    b += put_str("general.architecture") + struct.pack("<I", 8) + put_str("toy")
    b += put_str("toy.block_count") + struct.pack("<II", 4, 2)
    b += put_str("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 2) + put_str("a") + put_str("bc")
    b += put_str("blk.0.w") + struct.pack("<IQQIQ", 2, 32, 2, 0, 0)
    b += put_str("blk.1.q") + struct.pack("<IQIQ", 1, 256, 21, 256)
    b += b"\0" * ((-len(b)) % 32)
    b += bytes([7]) * (256 + 110)
    open(path, "wb").write(b)
    return b


def test_reads_the_reference_hand_written_file(tmp_path):
    L = szlib.load()
    p = str(tmp_path / "toy.gguf")
    full = reference_toy_file(p)
    h = C.c_void_p()
    szlib.check(L.sz_gguf_open(p.encode(), C.byref(h)))
    try:
        assert L.sz_weights_model(h) is None and L.sz_weights_tensor_count(h) == 2
        v = C.c_uint64()
        szlib.check(L.sz_weights_key_u64(h, b"toy.block_count", C.byref(v)))
        assert v.value == 2
        szlib.check(L.sz_weights_key_u64(h, b"tokenizer.ggml.tokens", C.byref(v)))
        assert v.value == 2                                   # an array: its length
        ty, dims, n = C.c_int32(), (C.c_int64 * 4)(), C.c_int64()
        szlib.check(L.sz_weights_tensor_info(h, b"blk.0.w", C.byref(ty), dims, C.byref(n)))
        assert (ty.value, list(dims)[:2], n.value) == (0, [32, 2], 256)
        szlib.check(L.sz_weights_tensor_info(h, b"blk.1.q", C.byref(ty), dims, C.byref(n)))
        assert (ty.value, dims[0], n.value) == (21, 256, 110)
        assert L.sz_weights_tensor_info(h, b"blk.2.x", C.byref(ty), dims, C.byref(n)) == szlib.E_ARG
    finally:
        L.sz_weights_free(h)
    # a tensor that runs past the end of the file must be refused (gguf.rs:617-627)
    cut = str(tmp_path / "cut.gguf")
    open(cut, "wb").write(full[:-200])
    assert L.sz_gguf_open(cut.encode(), C.byref(h)) == szlib.E_ARG
    open(cut, "wb").write(b"GGUX" + full[4:])
    assert L.sz_gguf_open(cut.encode(), C.byref(h)) == szlib.E_ARG and b"magic" in L.sz_last_error()
    assert L.sz_gguf_open(str(tmp_path / "none.gguf").encode(), C.byref(h)) == szlib.E_ARG


@pytest.fixture(scope="module")
def small_file(tmp_path_factory):
    M = md.make_model(SMALL, seed=4)
    path = str(tmp_path_factory.mktemp("gguf") / "small.gguf")
    gio.write_gguf(path, M)
    return M, path


def test_the_written_file_is_a_gguf_other_readers_understand(small_file):
    import gguf
    M, path = small_file
    r = gguf.GGUFReader(path)
    names = {t.name: t for t in r.tensors}
    assert len(names) == len(M["tensors"]) + sum(8 if Ld["shared_ff"] else 4 for Ld in M["moe"])
    t = names["blk.0.attn_qkv.weight"]
    ty, rows, cols, b = M["tensors"]["blk.0.attn_qkv.weight"]
    assert int(t.tensor_type) == ty and [int(d) for d in t.shape] == [cols, rows]
    assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), b.numpy().reshape(-1).view(np.uint8))
    e = names["blk.1.ffn_down_exps.weight"]
    assert [int(d) for d in e.shape] == [SMALL["expert_ff"], SMALL["hidden"], SMALL["n_expert"]]
    assert np.array_equal(np.asarray(e.data).reshape(-1).view(np.uint8), M["moe"][1]["down"].numpy().reshape(-1))
    f = r.get_field("qwen4exp.full_attention_interval")
    assert int(f.parts[-1][0]) == SMALL["attn_interval"]


def test_a_model_read_back_from_its_file_steps_to_the_same_bits(small_file):
    M, path = small_file
    lm = gio.LoadedModel(path)                                # host placement: tensors point into the mapped file
    for k, v in SMALL.items():
        assert lm.cfg[k] == pytest.approx(v), k
    assert lm.tensor_info("blk.3.attn_q.weight")[1][:2] == [SMALL["hidden"], 2 * SMALL["n_head"] * SMALL["head_dim"]]
    a = ob.Session(md.HostModel(M), kv_q8=True, threads=2)
    b = ob.Session(lm, kv_q8=True, threads=2)
    for t in (3, 500, 17, 17, 256):
        la, lb = a.step(t), b.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        assert np.array_equal(a.routes()[0], b.routes()[0])
    del b
    lm.close()


def test_a_file_with_a_sparse_indexer_reads_back_to_the_same_bits(tmp_path):
    cfg = dict(SMALL, idx_heads=2, idx_dim=32, idx_budget=8, idx_ratio=2)
    M = md.make_model(cfg, seed=4)
    path = str(tmp_path / "idx.gguf")
    gio.write_gguf(path, M)
    lm = gio.LoadedModel(path)
    assert (lm.cfg["idx_heads"], lm.cfg["idx_dim"], lm.cfg["idx_budget"]) == (2, 32, 8)
    assert lm.tensor_info("blk.3.indexer.q_proj.weight")[1][:2] == [SMALL["hidden"], 64]
    a = ob.Session(md.HostModel(M), kv_q8=True, threads=2)
    b = ob.Session(lm, kv_q8=True, threads=2)
    for t in (3, 500, 17, 17, 256, 9, 9, 41, 77, 5, 6, 7, 8, 1):    # past the budget of 8 positions: the indexer selects
        la, lb = a.step(t), b.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        assert np.array_equal(a.selected(3), b.selected(3))
    assert len(a.selected(3)) == 8 + len(a) % 2
    del b
    lm.close()


def test_a_file_with_a_per_layer_embedding_reads_back_to_the_same_bits(tmp_path):
    from tests.test_oracle_ple import PLE
    M = md.make_model(PLE, seed=2)
    path = str(tmp_path / "ple.gguf")
    gio.write_gguf(path, M)
    lm = gio.LoadedModel(path)
    for k in ("ple_layer", "ple_ngram", "ple_heads_per_ngram", "ple_head_dim", "ple_conv_k", "ple_eos", "ple_multipliers", "ple_vocab", "ple_offsets"):
        assert lm.cfg[k] == PLE[k], k
    a = ob.Session(md.HostModel(M), kv_q8=True, threads=2)
    b = ob.Session(lm, kv_q8=True, threads=2)
    for t in (3, 500, 17, 7, 256, 9, 9, 41):
        la, lb = a.step(t), b.step(t)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    del b
    lm.close()


def test_files_whose_keys_do_not_fit_are_refused(small_file, tmp_path):
    M, path = small_file
    L = szlib.load()
    raw = open(path, "rb").read()
    key = b"qwen4exp.ple.layers"
    at = raw.index(key) + len(key)                             # value: type u32 (9), element type u32 (11), count u64, then the i64 items
    assert struct.unpack_from("<IIQq", raw, at) == (9, 11, 1, SMALL["n_layer"])
    bad = str(tmp_path / "ple.gguf")
    open(bad, "wb").write(raw[:at + 16] + struct.pack("<q", 1) + raw[at + 24:])
    h = C.c_void_p()
    assert L.sz_model_load_gguf(bad.encode(), szlib.PLACE_HOST, 0, C.byref(h)) == szlib.E_ARG   # a layer is named, the rest of its keys say "none"
    assert b"per-layer embedding" in L.sz_last_error()
    # a missing shape key: the reader says which (forward.rs:78)
    key = b"qwen4exp.ssm.conv_kernel"
    at = raw.index(key)
    open(bad, "wb").write(raw[:at] + b"qwen4exp.ssm.conv_kernex" + raw[at + len(key):])
    assert L.sz_model_load_gguf(bad.encode(), szlib.PLACE_HOST, 0, C.byref(h)) == szlib.E_ARG
    assert b"ssm.conv_kernel" in L.sz_last_error()


@pytest.mark.gpu
@pytest.mark.parametrize("experts", ["q8", "exl3"])
def test_a_model_loaded_onto_the_device_steps_to_the_same_bits(tmp_path, experts):
    import torch  # noqa: F401
    cfg = dict(SMALL, hidden=512, expert_ff=256, shared_ff=256)
    ety = szlib.TYPE_Q8_0 if experts == "q8" else szlib.TYPE_EXL3(3)
    M = md.make_model(cfg, expert_type=ety, seed=9)
    path = str(tmp_path / "m.gguf")
    gio.write_gguf(path, M)
    lm = gio.LoadedModel(path, device="cuda:0")
    a = md.Session(md.DeviceModel(M), 64, kv_q8=True)
    b = md.Session(lm, 64, kv_q8=True)
    for ids in ([5, 6, 7, 8], [9], [10, 11, 12]):
        a.verify(ids); la = a.result(logits=True)[2]; a.commit(len(ids))
        b.verify(ids); lb = b.result(logits=True)[2]; b.commit(len(ids))
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    # and the host placement of the same file under the CPU oracle agrees with the device within the usual bound
    host = gio.LoadedModel(path)
    cpu = ob.Session(host, kv_q8=True, threads=4)
    want = np.stack([cpu.step(t) for t in (5, 6, 7, 8)])
    c = md.Session(lm, 64, kv_q8=True)
    c.verify([5, 6, 7, 8]); got = c.result(logits=True)[2]; c.commit(4)
    assert max(float(np.abs(got[j] - want[j]).max() / np.abs(want[j]).max()) for j in range(4)) < 1e-3
    del a, b, c, cpu
    host.close()
    lm.close()
