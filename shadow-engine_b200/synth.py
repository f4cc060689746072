"""Seeded synthetic weights in the three expert formats, for tests and benchmarks (no checkpoint is available offline).

- Q8_0: N(0, sigma) quantised with ggml's reference rule (d = amax / 127, q = round(w / d)).
- IQ3_S: N(0, sigma) quantised by a plain nearest-codebook encoder (valid blocks, not ggml's optimised search: gguf-py has
  no IQ3_S quantiser).
- EXL3: random trellis words with suh = +-1 and svh scaled to sigma, which is how the reference's own tests build blobs
  (crates/shadowzero-model/src/exl3.rs:652-658); a trellis quantiser (ExLlamaV3's Viterbi search) is not available.
All generators are deterministic functions of (seed, tensor name) and work on CPU or CUDA torch tensors.
"""
import zlib

import numpy as np
import torch

from . import lib as szlib

_GRID = None


def iq3s_grid():
    """[512, 4] float32 magnitudes of the IQ3_S codebook, read from the library's generated table."""
    global _GRID
    if _GRID is None:
        import os
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "iq3s_grid.inc")
        words = []
        for line in open(path):
            line = line.strip()
            if line.startswith("0x"):
                words += [int(t.strip().rstrip("u"), 16) for t in line.rstrip(",").split(",")]
        w = np.array(words, dtype=np.uint32)
        assert w.size == 512
        _GRID = np.stack([(w >> (8 * j)) & 0xff for j in range(4)], axis=1).astype(np.float32)
    return _GRID


def _gen(seed, name, device):
    g = torch.Generator(device=device)
    g.manual_seed((seed * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7fffffffffffffff)
    return g


def normal(shape, sigma, seed, name, device="cpu"):
    return torch.randn(shape, generator=_gen(seed, name, device), device=device, dtype=torch.float32) * sigma


def quantize_q8_0(w):
    """w: float32 [..., cols] (cols % 32 == 0) -> uint8 [..., cols / 32 * 34]."""
    shp = w.shape
    b = w.reshape(-1, 32)
    amax = b.abs().amax(dim=1, keepdim=True)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(b * inv).clamp(-127, 127).to(torch.int8)
    out = torch.empty((b.shape[0], 34), dtype=torch.uint8, device=w.device)
    out[:, :2] = d.to(torch.float16).view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(*shp[:-1], shp[-1] // 32 * 34)


def quantize_iq3_s(w, chunk=1 << 14):
    """w: float32 [..., cols] (cols % 256 == 0) -> uint8 [..., cols / 256 * 110].  Nearest-codebook encoder."""
    dev = w.device
    shp = w.shape
    grid = torch.from_numpy(iq3s_grid()).to(dev)                     # [512, 4]
    g2 = (grid * grid).sum(dim=1)                                     # [512]
    blocks = w.reshape(-1, 256)
    nb = blocks.shape[0]
    out = torch.zeros((nb, 110), dtype=torch.uint8, device=dev)
    for s0 in range(0, nb, chunk):
        b = blocks[s0:s0 + chunk]
        n = b.shape[0]
        sub = b.reshape(n, 8, 32)
        amax = sub.abs().amax(dim=2)                                  # [n, 8]
        # sub-block scale db = d (1 + 2 s), s in 0..15; the largest magnitude of the codebook is 15
        want = amax / 13.0
        d = (want.amax(dim=1, keepdim=True) / 31.0).clamp_min(1e-12)
        d = d.to(torch.float16).to(torch.float32).clamp_min(6e-8)
        s = torch.round((want / d - 1.0) / 2.0).clamp(0, 15)
        db = d * (1.0 + 2.0 * s)                                      # [n, 8]
        t = (sub.abs() / db.unsqueeze(2)).reshape(n * 64, 4)          # magnitudes in codebook units
        # argmin_i |t - grid_i|^2 = argmin_i (|grid_i|^2 - 2 t . grid_i)
        idx = (g2.unsqueeze(0) - 2.0 * (t @ grid.t())).argmin(dim=1).reshape(n, 64)
        neg = (sub < 0).reshape(n, 32, 8).to(torch.int32)
        signs = (neg << torch.arange(8, device=dev, dtype=torch.int32)).sum(dim=2).to(torch.uint8)
        qh = (((idx >> 8) & 1).reshape(n, 8, 8).to(torch.int32) << torch.arange(8, device=dev, dtype=torch.int32)).sum(dim=2)
        si = s.to(torch.int32)
        o = out[s0:s0 + n]
        o[:, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(n, 2)
        o[:, 2:66] = (idx & 0xff).to(torch.uint8)
        o[:, 66:74] = qh.to(torch.uint8)
        o[:, 74:106] = signs
        o[:, 106:110] = (si[:, 0::2] | (si[:, 1::2] << 4)).to(torch.uint8)
    return out.reshape(*shp[:-1], shp[-1] // 256 * 110)


def exl3_blob_len(n_in, n_out, bits):
    return 2 * n_in + 2 * n_out + 4 + n_in * n_out * bits // 8


def random_exl3_blobs(count, n_in, n_out, bits, sigma, seed, name, device="cpu", even=False):
    """`count` EXL3 blobs (reference layout: f16 suh | f16 svh | marker | trellis) as uint8 [count, blob_len].
    even: every output scale has the magnitude sigma (all rows of the matrix equally strong) instead of sigma * (0.5 .. 1.5)."""
    g = _gen(seed, name, device)
    n = exl3_blob_len(n_in, n_out, bits)
    out = torch.empty((count, n), dtype=torch.uint8, device=device)
    suh = (torch.randint(0, 2, (count, n_in), generator=g, device=device).to(torch.float32) * 2 - 1).to(torch.float16)
    mag = sigma * (0.5 + torch.rand((count, n_out), generator=g, device=device))
    if even:
        mag = torch.full_like(mag, sigma)
    sgn = torch.randint(0, 2, (count, n_out), generator=g, device=device).to(torch.float32) * 2 - 1
    svh = (mag * sgn).to(torch.float16)
    out[:, :2 * n_in] = suh.view(torch.uint8).reshape(count, -1)
    out[:, 2 * n_in:2 * n_in + 2 * n_out] = svh.view(torch.uint8).reshape(count, -1)
    out[:, 2 * n_in + 2 * n_out:2 * n_in + 2 * n_out + 4] = torch.tensor([1, 0, 0, 0], dtype=torch.uint8, device=device)
    ntr = n - (2 * n_in + 2 * n_out + 4)
    step = max(1, (1 << 28) // max(ntr, 1))
    for c0 in range(0, count, step):
        c1 = min(count, c0 + step)
        out[c0:c1, 2 * n_in + 2 * n_out + 4:] = torch.randint(0, 256, (c1 - c0, ntr), generator=g, device=device, dtype=torch.uint8)
    return out


def exl3_reconstruct(blob, n_in, n_out, bits):
    """W [n_in, n_out] float32 = diag(suh) H W_hat H diag(svh) of one EXL3 blob (a uint8 CUDA tensor), H = Hadamard(128) / sqrt(128)
    on every 128-block of both axes (crates/shadowzero-model/src/exl3.rs:246-286).  The trellis is decoded by the library
    (sz_exl3_reconstruct_inner); the rotations are two matrix products here.  For building synthetic models, not for parity."""
    if blob.device.type != "cuda":
        raise ValueError("exl3_reconstruct needs the blob on a CUDA device")
    L = szlib.load()
    blob = blob.contiguous()
    w = torch.empty((n_in, n_out), dtype=torch.float32, device=blob.device)
    szlib.check(L.sz_exl3_reconstruct_inner(bits, blob.data_ptr(), n_in, n_out, w.data_ptr(), torch.cuda.current_stream(blob.device).cuda_stream))
    h = torch.ones((1, 1), dtype=torch.float32, device=blob.device)
    while h.shape[0] < 128:
        h = torch.cat([torch.cat([h, h], dim=1), torch.cat([h, -h], dim=1)], dim=0)
    h = h / 128 ** 0.5
    suh = blob[:2 * n_in].view(torch.float16).to(torch.float32)
    svh = blob[2 * n_in:2 * n_in + 2 * n_out].view(torch.float16).to(torch.float32)
    w = (w.reshape(n_in, n_out // 128, 128) @ h).reshape(n_in, n_out)                 # output side
    w = (h @ w.reshape(n_in // 128, 128, n_out)).reshape(n_in, n_out)                 # input side (H is symmetric)
    return w * suh[:, None] * svh[None, :]


def matrix_bytes(ty, n_in, n_out):
    if ty == szlib.TYPE_Q8_0:
        return n_out * (n_in // 32) * 34
    if ty == szlib.TYPE_IQ3_S:
        return n_out * (n_in // 256) * 110
    if 1020 < ty <= 1028:
        return exl3_blob_len(n_in, n_out, ty - 1020)
    raise ValueError(ty)


def make_matrices(ty, count, n_in, n_out, sigma, seed, name, device="cpu"):
    """`count` matrices [n_in -> n_out] of type `ty` as uint8 [count, matrix_bytes]."""
    if 1020 < ty <= 1028:
        return random_exl3_blobs(count, n_in, n_out, ty - 1020, sigma, seed, name, device)
    out = torch.empty((count, matrix_bytes(ty, n_in, n_out)), dtype=torch.uint8, device=device)
    step = max(1, (1 << 26) // (n_in * n_out))
    for c0 in range(0, count, step):
        c1 = min(count, c0 + step)
        w = normal((c1 - c0, n_out, n_in), sigma, seed, "%s.%d" % (name, c0), device)
        q = quantize_q8_0(w) if ty == szlib.TYPE_Q8_0 else quantize_iq3_s(w)
        out[c0:c1] = q.reshape(c1 - c0, -1)
    return out


def make_moe_layer(hidden, n_expert, top_k, expert_ff, shared_ff, expert_type, shared_type, seed=1, sigma=0.02,
                   router_sigma=None, device="cpu", name="blk.0"):
    """One MoE layer's tensors (torch uint8 / float32) plus its shape: the host-side description both the oracle binding
    and `moe.MoeLayer` accept.  Router rows are N(0, router_sigma) (default 1 / sqrt(hidden): logits ~ N(0, 1) for unit
    inputs)."""
    rs = router_sigma if router_sigma is not None else hidden ** -0.5
    L = dict(hidden=hidden, n_expert=n_expert, top_k=top_k, expert_ff=expert_ff, shared_ff=shared_ff,
             expert_type=expert_type, shared_type=shared_type)
    L["router"] = normal((n_expert, hidden), rs, seed, name + ".ffn_gate_inp", device)
    L["shared_router"] = normal((hidden,), rs, seed, name + ".ffn_gate_inp_shexp", device)
    L["gate"] = make_matrices(expert_type, n_expert, hidden, expert_ff, sigma, seed, name + ".ffn_gate_exps", device)
    L["up"] = make_matrices(expert_type, n_expert, hidden, expert_ff, sigma, seed, name + ".ffn_up_exps", device)
    L["down"] = make_matrices(expert_type, n_expert, expert_ff, hidden, sigma, seed, name + ".ffn_down_exps", device)
    if shared_ff > 0:
        L["sh_gate"] = make_matrices(shared_type, 1, hidden, shared_ff, sigma, seed, name + ".ffn_gate_shexp", device)[0]
        L["sh_up"] = make_matrices(shared_type, 1, hidden, shared_ff, sigma, seed, name + ".ffn_up_shexp", device)[0]
        L["sh_down"] = make_matrices(shared_type, 1, shared_ff, hidden, sigma, seed, name + ".ffn_down_shexp", device)[0]
    return L


def to_numpy_layer(L):
    """The same layer as numpy arrays (what `oracle.binding.moe` takes)."""
    out = {}
    for k, v in L.items():
        out[k] = v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v
    if L["shared_ff"] == 0:
        z = np.zeros(16, dtype=np.uint8)
        out.update(sh_gate=z, sh_up=z, sh_down=z)
    return out
