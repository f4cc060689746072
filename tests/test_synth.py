"""The seeded weight generators make valid blocks: the oracle decodes them back to what was quantised."""
import numpy as np
import torch

from oracle import binding as ob
from tests.util import pkg

synth = pkg.synth
szlib = pkg.lib


def test_q8_0_quantiser_round_trips_and_matches_gguf():
    from gguf import quants, GGMLQuantizationType as T
    w = synth.normal((8, 256), 0.02, 1, "t")
    q = synth.quantize_q8_0(w).numpy()
    assert q.shape == (8, 256 // 32 * 34)
    want = quants.quantize(w.numpy(), T.Q8_0)
    assert np.array_equal(q, want)
    back = ob.dequant(ob.Q8_0, q).reshape(8, 256)
    assert np.abs(back - w.numpy()).max() <= 0.5 * np.abs(w.numpy()).max() / 127 * 1.01


def test_iq3_s_quantiser_makes_blocks_close_to_the_input():
    w = synth.normal((16, 512), 0.02, 2, "t")
    q = synth.quantize_iq3_s(w).numpy()
    assert q.shape == (16, 2 * 110)
    back = ob.dequant(ob.IQ3_S, q).reshape(16, 512)
    rel = np.linalg.norm(back - w.numpy()) / np.linalg.norm(w.numpy())
    assert rel < 0.25, rel  # ~3.4 bits a weight
    assert np.all(np.sign(back[np.abs(back) > 0]) == np.sign(w.numpy()[np.abs(back) > 0]))
    # gguf-py decodes the same bytes to the same values
    from gguf import quants, GGMLQuantizationType as T
    assert np.array_equal(quants.dequantize(q.reshape(-1), T.IQ3_S).astype(np.float32).view(np.uint32),
                          back.reshape(-1).view(np.uint32))


def test_exl3_blobs_have_the_reference_layout_and_scale():
    blobs = synth.random_exl3_blobs(2, 256, 128, 3, 0.02, 5, "t")
    assert blobs.shape == (2, ob.exl3_blob_len(256, 128, 3)) == (2, synth.exl3_blob_len(256, 128, 3))
    w = ob.exl3_reconstruct(256, 128, 3, blobs[1].numpy())
    assert 0.012 < w.std() < 0.03
    assert not np.array_equal(blobs[0].numpy(), blobs[1].numpy())


def test_generators_are_deterministic():
    a = synth.make_moe_layer(128, 4, 2, 128, 128, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=7)
    b = synth.make_moe_layer(128, 4, 2, 128, 128, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=7)
    c = synth.make_moe_layer(128, 4, 2, 128, 128, szlib.TYPE_Q8_0, szlib.TYPE_Q8_0, seed=8)
    assert torch.equal(a["gate"], b["gate"]) and torch.equal(a["router"], b["router"])
    assert not torch.equal(a["gate"], c["gate"])
