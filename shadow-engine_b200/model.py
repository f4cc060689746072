"""The model description (struct sz_model) from Python: ctypes mirrors of the header's structs, seeded synthetic models with the
reference's tensor names (crates/shadowzero-model/src/exl3_model.rs:223-243), and the two placements of one model - host memory
for the CPU oracle, HBM for the library."""
import ctypes as C

import numpy as np
import torch

from . import lib as szlib
from . import ep as szep
from . import moe as szmoe
from . import synth


class Tensor(C.Structure):
    _fields_ = [("type", C.c_int32), ("reserved", C.c_int32), ("data", C.c_uint64), ("rows", C.c_int64), ("cols", C.c_int64)]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "hidden", "streams", "hc_rank", "vocab", "n_head", "n_kv_head", "head_dim", "rope_dims",
                                         "n_expert", "n_expert_used", "expert_ff", "shared_ff", "ssm_k_heads", "ssm_v_heads", "ssm_head_dim",
                                         "conv_k", "attn_interval")] + [("eps", C.c_float), ("reserved", C.c_float), ("rope_theta", C.c_double)] + \
               [(n, C.c_int32) for n in ("idx_heads", "idx_dim", "idx_budget", "idx_reserved")]


class Hc(C.Structure):
    _fields_ = [("norm", Tensor), ("down", Tensor), ("up", Tensor), ("inject", Tensor)]


class Layer(C.Structure):
    _fields_ = [("hc_attn", Hc), ("hc_ffn", Hc)] + \
               [(n, Tensor) for n in ("attn_qkv", "attn_gate", "ssm_beta", "ssm_alpha", "ssm_conv1d", "ssm_a", "ssm_dt_bias", "ssm_norm", "ssm_out",
                                      "attn_q", "attn_k", "attn_v", "attn_q_norm", "attn_k_norm", "attn_output",
                                      "idx_q", "idx_k", "idx_q_norm", "idx_k_norm")] + \
               [("idx_ratio", C.c_int32), ("idx_reserved", C.c_int32), ("moe", szlib.MoeLayerC)]


class Ple(C.Structure):
    """struct sz_ple"""
    _fields_ = [(n, C.c_int32) for n in ("layer", "ngram", "heads_per_ngram", "head_dim", "conv_k", "eos")] + \
               [("multipliers", C.c_int64 * 8), ("vocab", C.c_int64 * 32), ("offsets", C.c_int64 * 32)] + \
               [(n, Tensor) for n in ("table", "key", "value", "norm_key", "norm_query", "norm_conv", "conv1d")]


class Model(C.Structure):
    _fields_ = [("cfg", ModelConfig), ("token_embd", Tensor), ("output", Tensor), ("output_hc", Hc), ("layers", C.POINTER(Layer)), ("ple", Ple)]


class Sampler(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("min_p", C.c_float), ("seed", C.c_uint64)]


class GenParams(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("spec_k", "max_new", "lookup_min", "greedy", "eog_token", "device_accept")] + [("sampler", Sampler)] + \
               [("max_rounds", C.c_int32), ("reserved", C.c_int32)]


class GenStats(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_tokens", "passes", "drafted", "accepted", "lookup_passes", "rounds")] + \
               [("pos_tried", C.c_int32 * 8), ("pos_right", C.c_int32 * 8), ("draft_ms", C.c_double), ("verify_ms", C.c_double), ("commit_ms", C.c_double),
                ("device_ms", C.c_double)]


# benchmark config 1: the CPU-runnable tiny hybrid MoE (4 layers D D D A; hidden 512; 8 q / 2 kv heads of 64; DeltaNet 4 heads of 64;
# 32 experts top-4 of FFN 256 + a shared expert of FFN 512; vocab 32000), with the reference's hyper-connections as block glue
# (4 streams, rank = streams * hidden / 32 as in its checkpoints, docs/ARCH.md:79-80).
TINY = dict(n_layer=4, hidden=512, streams=4, hc_rank=64, vocab=32000, n_head=8, n_kv_head=2, head_dim=64, rope_dims=32, n_expert=32,
            n_expert_used=4, expert_ff=256, shared_ff=512, ssm_k_heads=4, ssm_v_heads=4, ssm_head_dim=64, conv_k=4, attn_interval=4,
            eps=1e-6, rope_theta=1e7)


def is_attention(cfg, l):
    return l % cfg["attn_interval"] == cfg["attn_interval"] - 1


def token_cycles(vocab, seed, cycle=16):
    """A seeded permutation of the vocabulary made of cycles of `cycle` tokens: successor[t] is the token after t in its cycle."""
    g = torch.Generator().manual_seed(seed * 7919 + 13)
    order = torch.randperm(vocab, generator=g)
    n = vocab // cycle * cycle
    succ = torch.arange(vocab)
    grp = order[:n].reshape(-1, cycle)
    succ[grp.reshape(-1)] = torch.roll(grp, -1, dims=1).reshape(-1)
    return succ, grp


def make_model(cfg, dense_type=szlib.TYPE_Q8_0, expert_type=szlib.TYPE_Q8_0, shared_type=None, hc_type=szlib.TYPE_BF16, seed=1,
               sigma=0.02, device="cpu", cycle=16, cycle_alpha=0.0, head_type=None, cycle_beta=0.0):
    """Seeded synthetic weights: name -> (ggml type, rows, cols, torch tensor of the stored bytes).  Matrices are N(0, sigma)
    quantised to their type, norm weights are 1, ssm_a is negative, MoE layers come from synth.make_moe_layer.

    A random-init model never repeats itself, so a suffix drafter would have nothing to draft.  With cycle_alpha > 0 the output
    matrix is correlated with the embedding through a seeded permutation of the vocabulary made of `cycle`-token cycles
    (row successor[t] of output.weight = alpha * embedding[t] + sqrt(1 - alpha^2) * noise: still N(0, sigma) entries): the model
    leans towards continuing the cycle of its last token, while the layers' contribution makes it leave the cycle now and then -
    repeated n-grams with occasional surprises, which is what speculation is measured on.

    With cycle_beta > 0 a token also leans, less strongly, towards the token TWO places on in its cycle: when the layers'
    contribution tips the balance the model skips a token but stays inside its cycle, so a drafter that looks the context up in the
    history keeps finding it and is right at a position only some of the time - partial acceptance, position by position, as on
    real text (the reference reports 75 / 75 / 83 % at draft positions 1 / 2 / 3, docs/SPECULATION.md:95-98).

    head_type = TYPE_EXL3(k) stores output.weight as an EXL3 blob (random trellis words: no trellis quantiser is available, so
    the head cannot be made from a wanted matrix).  The correlation then runs the other way: the embedding of token t is made
    from the decoded row successor[t] of the head (CUDA device only: the decode is the library's)."""
    shared_type = expert_type if shared_type is None else shared_type
    head_type = dense_type if head_type is None else head_type
    head_exl3 = 1020 < head_type <= 1028
    H, Cs = cfg["hidden"], cfg["streams"]
    CH = Cs * H
    kd, vd = cfg["ssm_k_heads"] * cfg["ssm_head_dim"], cfg["ssm_v_heads"] * cfg["ssm_head_dim"]
    ch = 2 * kd + vd
    qd, kvd = cfg["n_head"] * cfg["head_dim"], cfg["n_kv_head"] * cfg["head_dim"]
    T = {}

    def mat(name, rows, cols, ty):
        w = synth.normal((rows, cols), sigma, seed, name, device)
        if ty == szlib.TYPE_F32:
            b = w
        elif ty == szlib.TYPE_BF16:
            b = w.to(torch.bfloat16)
        elif ty == szlib.TYPE_F16:
            b = w.to(torch.float16)
        elif ty == szlib.TYPE_Q8_0:
            b = synth.quantize_q8_0(w)
        elif ty == szlib.TYPE_IQ3_S:
            b = synth.quantize_iq3_s(w)
        else:
            raise ValueError(ty)
        T[name] = (ty, rows, cols, b.contiguous())

    def vec(name, values):
        T[name] = (szlib.TYPE_F32, 1, values.numel(), values.to(torch.float32).contiguous())

    def hc(prefix, inject):
        vec(prefix + "_norm.weight", torch.ones(CH, device=device))
        mat(prefix + "_down.weight", cfg["hc_rank"], CH, hc_type)
        mat(prefix + "_up.weight", CH, cfg["hc_rank"], hc_type)
        if inject:
            mat(prefix + "_inject.weight", Cs, CH, hc_type)

    if head_exl3:
        bits = head_type - 1020
        # (every token's row equally strong, as in a Gaussian head: a few loud rows would win every argmax)
        blob = synth.random_exl3_blobs(1, H, cfg["vocab"], bits, sigma, seed, "output.weight", device, even=True)[0]
        T["output.weight"] = (head_type, cfg["vocab"], H, blob.contiguous())
        if cycle_alpha > 0.0:
            rows = synth.exl3_reconstruct(blob, H, cfg["vocab"], bits).t()          # [vocab, H]: row v = the head's weights of token v
            rows = rows * (sigma / rows.std(dim=1, keepdim=True).clamp_min(1e-12))
            succ, _ = token_cycles(cfg["vocab"], seed, cycle)
            noise = synth.normal((cfg["vocab"], H), sigma, seed, "token_embd.weight", device)
            succ = succ.to(rows.device)
            emb = cycle_alpha * rows[succ] + (1.0 - cycle_alpha ** 2) ** 0.5 * noise
            if cycle_beta > 0.0:
                emb += cycle_beta * rows[succ[succ]]
            emb *= 15.0
            del rows, noise
            T["token_embd.weight"] = (dense_type, cfg["vocab"], H, (synth.quantize_q8_0(emb) if dense_type == szlib.TYPE_Q8_0 else emb).contiguous())
        else:
            mat("token_embd.weight", cfg["vocab"], H, dense_type)
    elif cycle_alpha > 0.0:
        # embedding rows 15x larger than the matrices' sigma, so that the token's identity is not drowned by the sublayers' outputs
        emb = synth.normal((cfg["vocab"], H), 15.0 * sigma, seed, "token_embd.weight", device)
        T["token_embd.weight"] = (dense_type, cfg["vocab"], H, (synth.quantize_q8_0(emb) if dense_type == szlib.TYPE_Q8_0 else emb).contiguous())
        noise = synth.normal((cfg["vocab"], H), sigma, seed, "output.weight", device)
        succ, _ = token_cycles(cfg["vocab"], seed, cycle)
        w = torch.empty_like(emb)
        succ = succ.to(emb.device)
        w[succ] = cycle_alpha * (emb / 15.0) + (1.0 - cycle_alpha ** 2) ** 0.5 * noise
        if cycle_beta > 0.0:
            w[succ[succ]] += cycle_beta * (emb / 15.0)
        if dense_type == szlib.TYPE_Q8_0:
            T["output.weight"] = (dense_type, cfg["vocab"], H, synth.quantize_q8_0(w).contiguous())
        elif dense_type == szlib.TYPE_F32:
            T["output.weight"] = (dense_type, cfg["vocab"], H, w.contiguous())
        else:
            raise ValueError("cycle_alpha needs a Q8_0 or F32 head")
    else:
        mat("token_embd.weight", cfg["vocab"], H, dense_type)
        mat("output.weight", cfg["vocab"], H, dense_type)
    hc("output_hc", False)
    if cfg.get("ple_ngram", 0) >= 2:
        # the hashed n-gram memory of one layer: (ngram - 1) * heads_per_ngram table rows of ple_head_dim weights make up one embedding
        pl, nh_ = cfg["ple_layer"], (cfg["ple_ngram"] - 1) * cfg["ple_heads_per_ngram"]
        assert nh_ * cfg["ple_head_dim"] == H and len(cfg["ple_vocab"]) == nh_ and len(cfg["ple_offsets"]) == nh_
        pp = "blk.%d." % pl
        mat("per_layer_token_embd.weight", cfg["ple_offsets"][-1] + cfg["ple_vocab"][-1], cfg["ple_head_dim"], cfg.get("ple_table_type", szlib.TYPE_Q8_0))
        mat(pp + "ple_key.weight", CH, H, hc_type)
        mat(pp + "ple_value.weight", H, H, hc_type)
        for n_ in ("ple_norm_key", "ple_norm_query", "ple_norm_conv"):
            vec(pp + n_ + ".weight", 1.0 + synth.normal((CH,), 0.1, seed, pp + n_, device))
        vec(pp + "ple_conv1d.weight", synth.normal((CH, cfg["ple_conv_k"]), 0.3, seed, pp + "ple_conv1d", device).reshape(-1))
    moe_layers = []
    for l in range(cfg["n_layer"]):
        p = "blk.%d." % l
        hc(p + "hc_attn", True)
        hc(p + "hc_ffn", True)
        if is_attention(cfg, l):
            mat(p + "attn_q.weight", 2 * qd, H, dense_type)
            mat(p + "attn_k.weight", kvd, H, dense_type)
            mat(p + "attn_v.weight", kvd, H, dense_type)
            mat(p + "attn_output.weight", H, qd, dense_type)
            vec(p + "attn_q_norm.weight", torch.ones(cfg["head_dim"], device=device))
            vec(p + "attn_k_norm.weight", torch.ones(cfg["head_dim"], device=device))
            if cfg.get("idx_heads", 0) > 0:
                mat(p + "indexer.q_proj.weight", cfg["idx_heads"] * cfg["idx_dim"], H, dense_type)
                mat(p + "indexer.k_proj.weight", cfg["idx_dim"], H, dense_type)
                # (norm weights away from 1, so that a test notices a forgotten weight)
                vec(p + "indexer.q_norm.weight", 1.0 + synth.normal((cfg["idx_dim"],), 0.1, seed, p + "indexer.q_norm", device))
                vec(p + "indexer.k_norm.weight", 1.0 + synth.normal((cfg["idx_dim"],), 0.1, seed, p + "indexer.k_norm", device))
        else:
            mat(p + "attn_qkv.weight", ch, H, dense_type)
            mat(p + "attn_gate.weight", vd, H, dense_type)
            mat(p + "ssm_beta.weight", cfg["ssm_v_heads"], H, dense_type)
            mat(p + "ssm_alpha.weight", cfg["ssm_v_heads"], H, dense_type)
            mat(p + "ssm_out.weight", H, vd, dense_type)
            vec(p + "ssm_conv1d.weight", synth.normal((ch, cfg["conv_k"]), 0.3, seed, p + "ssm_conv1d", device).reshape(-1))
            vec(p + "ssm_a", -(0.5 + torch.rand(cfg["ssm_v_heads"], generator=synth._gen(seed, p + "ssm_a", device), device=device)))
            vec(p + "ssm_dt.bias", synth.normal((cfg["ssm_v_heads"],), 0.1, seed, p + "ssm_dt", device))
            vec(p + "ssm_norm.weight", torch.ones(cfg["ssm_head_dim"], device=device))
        moe_layers.append(synth.make_moe_layer(H, cfg["n_expert"], cfg["n_expert_used"], cfg["expert_ff"], cfg["shared_ff"], expert_type,
                                               shared_type, seed=seed + 1000 * (l + 1), sigma=sigma, router_sigma=sigma, device=device,
                                               name=p.rstrip(".")))
    return dict(cfg=dict(cfg), tensors=T, moe=moe_layers)


def _fill_config(c, cfg):
    names = {n for n, _ in ModelConfig._fields_}
    for k, v in cfg.items():
        if k in names:
            setattr(c, k, v)


class _Placed:
    """Common part of the two placements: builds struct sz_model from a `put(tensor) -> address` callback."""

    def _build(self, M, put, put_moe):
        cfg = M["cfg"]
        self.cfg = cfg
        self.model = Model()
        _fill_config(self.model.cfg, cfg)
        T = M["tensors"]

        def tens(name):
            ty, rows, cols, b = T[name]
            t = Tensor()
            t.type, t.rows, t.cols, t.data = ty, rows, cols, put(b, 12 if 1020 < ty <= 1028 else 0)  # an EXL3 blob: trellis on a 16-byte boundary
            return t

        def hc(prefix, inject):
            h = Hc()
            h.norm, h.down, h.up = tens(prefix + "_norm.weight"), tens(prefix + "_down.weight"), tens(prefix + "_up.weight")
            if inject:
                h.inject = tens(prefix + "_inject.weight")
            return h

        self.model.token_embd, self.model.output, self.model.output_hc = tens("token_embd.weight"), tens("output.weight"), hc("output_hc", False)
        if cfg.get("ple_ngram", 0) >= 2:
            P, pp = self.model.ple, "blk.%d." % cfg["ple_layer"]
            for k in ("layer", "ngram", "heads_per_ngram", "head_dim", "conv_k", "eos"):
                setattr(P, k, int(cfg["ple_" + k]))
            for i, v in enumerate(cfg["ple_multipliers"]):
                P.multipliers[i] = int(v)
            for i, (v, o) in enumerate(zip(cfg["ple_vocab"], cfg["ple_offsets"])):
                P.vocab[i], P.offsets[i] = int(v), int(o)
            P.table, P.key, P.value = tens("per_layer_token_embd.weight"), tens(pp + "ple_key.weight"), tens(pp + "ple_value.weight")
            P.norm_key, P.norm_query, P.norm_conv = tens(pp + "ple_norm_key.weight"), tens(pp + "ple_norm_query.weight"), tens(pp + "ple_norm_conv.weight")
            P.conv1d = tens(pp + "ple_conv1d.weight")
        self.layers = (Layer * cfg["n_layer"])()
        for l in range(cfg["n_layer"]):
            p = "blk.%d." % l
            L = self.layers[l]
            L.hc_attn, L.hc_ffn = hc(p + "hc_attn", True), hc(p + "hc_ffn", True)
            if is_attention(cfg, l):
                for n in ("attn_q", "attn_k", "attn_v", "attn_output", "attn_q_norm", "attn_k_norm"):
                    setattr(L, n, tens(p + n + ".weight"))
                if cfg.get("idx_heads", 0) > 0:
                    L.idx_q, L.idx_k = tens(p + "indexer.q_proj.weight"), tens(p + "indexer.k_proj.weight")
                    L.idx_q_norm, L.idx_k_norm = tens(p + "indexer.q_norm.weight"), tens(p + "indexer.k_norm.weight")
                    L.idx_ratio = int(cfg.get("idx_ratio", 4))
            else:
                for n in ("attn_qkv", "attn_gate", "ssm_beta", "ssm_alpha", "ssm_out", "ssm_conv1d", "ssm_norm"):
                    setattr(L, n, tens(p + n + ".weight"))
                L.ssm_a, L.ssm_dt_bias = tens(p + "ssm_a"), tens(p + "ssm_dt.bias")
            L.moe = put_moe(M["moe"][l])
        self.model.layers = C.cast(self.layers, C.POINTER(Layer))


class HostModel(_Placed):
    """The model in host memory: what `oracle.binding` sessions take."""

    def __init__(self, M):
        self._keep = []

        def put(b, lead=0):
            a = np.ascontiguousarray(b.detach().cpu().view(torch.uint8).numpy() if b.dtype == torch.bfloat16 else b.detach().cpu().numpy())
            self._keep.append(a)
            return a.ctypes.data

        def put_moe(Ld):
            Ln = synth.to_numpy_layer(Ld)
            self._keep.append(Ln)
            c = szlib.MoeLayerC()
            for k in ("hidden", "n_expert", "top_k", "expert_ff", "shared_ff", "expert_type", "shared_type"):
                setattr(c, k, Ln[k])
            c.router, c.shared_router = Ln["router"].ctypes.data, Ln["shared_router"].ctypes.data
            for k in ("gate", "up", "down"):
                setattr(c, k, Ln[k].ctypes.data)
                setattr(c, k + "_stride", Ln[k].strides[0])
            for k in ("sh_gate", "sh_up", "sh_down"):
                setattr(c, k, Ln[k].ctypes.data)
            return c

        self._build(M, put, put_moe)


class DeviceModel(_Placed):
    """The model resident in HBM: what `Session` takes."""

    def __init__(self, M, device="cuda:0", ep=None):
        """`ep` = (rank, world): hold only this rank's experts of every MoE layer (see `ep.shard_spec`); the library's
        communicator must be up (`ep.init_from_process_group`) before a session of such a model runs a pass."""
        self.device = torch.device(device)
        self._keep = []
        self.ep = ep

        def put(b, lead=0):
            buf, addr, _ = szmoe.place(b.reshape(1, -1), self.device, lead)
            self._keep.append(buf)
            return addr

        def put_moe(Ld):
            shard = szep.shard_spec(ep[0], ep[1], Ld["n_expert"]) if ep else None
            ml = szmoe.MoeLayer(Ld, self.device, shard=shard)
            self._keep.append(ml)
            return ml.c

        self._build(M, put, put_moe)


class Session:
    """A verify session on the GPU (struct sz_session): owns the one device block the library asks for."""

    def __init__(self, dm, ctx, kv_q8=True, stream=None, head_proxy=False):
        """head_proxy: screen an EXL3 output.weight with its 2-bit proxy (SZ_HEAD_PROXY); the proxy is built here."""
        self.lib = szlib.load()
        self.dm = dm
        self.flags = (1 if kv_q8 else 0) | (2 if head_proxy else 0)
        n = C.c_int64()
        szlib.check(self.lib.sz_session_bytes(C.byref(dm.model), ctx, self.flags, C.byref(n)))
        self.mem = torch.empty(n.value + 256, dtype=torch.uint8, device=dm.device)
        addr = self.mem.data_ptr() + (-self.mem.data_ptr()) % 256
        # a stream of its own: the default stream cannot record CUDA graphs, which the session uses for its passes
        torch.cuda.synchronize(dm.device)
        self._stream = stream or torch.cuda.Stream(dm.device)
        self.stream = self._stream.cuda_stream
        self.h = C.c_void_p()
        szlib.check(self.lib.sz_session_create(C.byref(dm.model), ctx, self.flags, addr, n.value, self.stream, C.byref(self.h)))
        self.vocab = dm.cfg["vocab"]

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.sz_session_destroy(self.h)
            self.h = None

    def __len__(self):
        return self.lib.sz_session_len(self.h)

    def reset(self):
        szlib.check(self.lib.sz_session_reset(self.h, self.stream))

    def fill_synthetic(self, length, seed=1):
        szlib.check(self.lib.sz_session_fill_synthetic(self.h, length, seed, self.stream))

    def trace_routes(self, on=True):
        szlib.check(self.lib.sz_session_trace_routes(self.h, 1 if on else 0))

    def verify(self, ids, accept=0, eog=-1, head=True):
        a = (C.c_int32 * len(ids))(*[int(t) for t in ids])
        szlib.check(self.lib.sz_session_verify(self.h, a, len(ids), accept, eog, 1 if head else 0, self.stream))
        self._m = len(ids)

    def verify_tree(self, ids, parents, accept=0, eog=-1):
        """A pass over a draft tree: ids[0] the root, ids[j] a drafted token under row parents[j] (parents[0] = -1)."""
        a = (C.c_int32 * len(ids))(*[int(t) for t in ids])
        p = (C.c_int32 * len(ids))(*[int(t) for t in parents])
        szlib.check(self.lib.sz_session_verify_tree(self.h, a, p, len(ids), accept, eog, self.stream))
        self._m = len(ids)

    def tree_path(self):
        path, n = (C.c_int32 * szlib.MAX_VERIFY)(), C.c_int()
        szlib.check(self.lib.sz_session_tree_path(self.h, path, C.byref(n), self.stream))
        return list(path[:n.value])

    def commit_path(self, path):
        a = (C.c_int32 * len(path))(*[int(t) for t in path])
        szlib.check(self.lib.sz_session_commit_path(self.h, a, len(path), self.stream))

    def set_stops(self, ids):
        """Up to 7 more ids that end generation: device acceptance never keeps a drafted one, and the loop ends at one."""
        a = (C.c_int32 * max(len(ids), 1))(*[int(t) for t in ids])
        szlib.check(self.lib.sz_session_set_stops(self.h, a, len(ids), self.stream))

    def set_sampler(self, sampler):
        szlib.check(self.lib.sz_session_set_sampler(self.h, C.byref(sampler)))

    def verify_sampled(self, ids, pos, eog=-1):
        """A pass whose acceptance is sampled on the device: row i's token is the sampler's draw at output position pos + i."""
        a = (C.c_int32 * len(ids))(*[int(t) for t in ids])
        szlib.check(self.lib.sz_session_verify_sampled(self.h, a, len(ids), pos, eog, self.stream))
        self._m = len(ids)

    def prefill(self, ids):
        a = (C.c_int32 * len(ids))(*[int(t) for t in ids])
        szlib.check(self.lib.sz_session_prefill(self.h, a, len(ids), self.stream))
        self._m = (len(ids) - 1) % szlib.MAX_VERIFY + 1

    def result(self, logits=False):
        """(keep, next), top [m, 128] uint32, logits [m, vocab] float32 or None of the pending pass."""
        m = self._m
        kn = (C.c_int32 * 2)()
        top = np.empty((m, 128), dtype=np.uint32)
        lg = np.empty((m, self.vocab), dtype=np.float32) if logits else None
        szlib.check(self.lib.sz_session_result(self.h, kn, top.ctypes.data_as(C.c_void_p), lg.ctypes.data_as(C.c_void_p) if logits else None, self.stream))
        return (kn[0], kn[1]), top, lg

    def routes(self):
        n = self.dm.cfg["n_layer"]
        idx = np.empty((n, szlib.MAX_VERIFY, szlib.MAX_TOPK), dtype=np.int32)
        w = np.empty((n, szlib.MAX_VERIFY, szlib.MAX_TOPK), dtype=np.float64)
        szlib.check(self.lib.sz_session_routes(self.h, idx.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p), self.stream))
        k = self.dm.cfg["n_expert_used"]
        return idx.reshape(n, -1)[:, :self._m * k].reshape(n, self._m, k), w.reshape(n, -1)[:, :self._m * k].reshape(n, self._m, k)

    def commit(self, keep):
        szlib.check(self.lib.sz_session_commit(self.h, keep, self.stream))

    def export(self, what, layer):
        """One piece of the committed state (sz_session_export): the recurrent state [v heads, d, d] or the carried conv rows
        [conv_k - 1, channels] of a DeltaNet layer as float32, or the K / V cache of an attention layer as bytes
        [positions, kv heads, head bytes]."""
        c = self.dm.cfg
        if what == szlib.STATE_DELTA_S:
            a = np.empty((c["ssm_v_heads"], c["ssm_head_dim"], c["ssm_head_dim"]), dtype=np.float32)
        elif what == szlib.STATE_DELTA_CONV:
            a = np.empty((c["conv_k"] - 1, (2 * c["ssm_k_heads"] + c["ssm_v_heads"]) * c["ssm_head_dim"]), dtype=np.float32)
        elif what == szlib.STATE_PLE_HIST:
            a = np.empty(((c["ple_conv_k"] - 1) * c["ple_ngram"], c["streams"] * c["hidden"]), dtype=np.float32)
        elif what == szlib.STATE_PLE_TAIL:
            a = np.empty(8, dtype=np.int32)
        elif what == szlib.STATE_IDX_RAW:
            a = np.empty((len(self), c["idx_dim"]), dtype=np.float32)
        elif what == szlib.STATE_IDX_SELECTED:
            a = np.empty((szlib.MAX_VERIFY, self.lib.sz_session_idx_words(self.h)), dtype=np.uint32)
        elif what == szlib.STATE_IDX_SCORES:
            a = np.empty((szlib.MAX_VERIFY, 32 * self.lib.sz_session_idx_words(self.h)), dtype=np.float32)
        else:
            hb = c["head_dim"] + ((c["head_dim"] // 32 * 2 + 15) & ~15) if self.flags & 1 else 4 * c["head_dim"]
            a = np.empty((len(self), c["n_kv_head"], hb), dtype=np.uint8)
        szlib.check(self.lib.sz_session_export(self.h, what, layer, a.ctypes.data_as(C.c_void_p), a.nbytes, self.stream))
        return a

    def checkpoint(self):
        """Every piece of the committed state, in host memory (GpuSession::snapshot with the cache): what `restore` takes."""
        c = self.dm.cfg
        pieces = []
        for l in range(c["n_layer"]):
            if is_attention(c, l):
                kinds = [szlib.STATE_KV_K, szlib.STATE_KV_V] + ([szlib.STATE_IDX_RAW] if c.get("idx_heads", 0) else [])
            else:
                kinds = [szlib.STATE_DELTA_S, szlib.STATE_DELTA_CONV]
            pieces += [(k, l, self.export(k, l)) for k in kinds]
        if c.get("ple_ngram", 0) >= 2:
            pieces += [(k, 0, self.export(k, 0)) for k in (szlib.STATE_PLE_HIST, szlib.STATE_PLE_TAIL)]
        return dict(positions=len(self), pieces=pieces)

    def restore(self, ck):
        """Become the session the checkpoint was taken from (GpuSession::restore): reset, every piece back, the length."""
        szlib.check(self.lib.sz_session_reset(self.h, self.stream))
        for what, layer, a in ck["pieces"]:
            a = np.ascontiguousarray(a)
            szlib.check(self.lib.sz_session_import(self.h, what, layer, a.ctypes.data_as(C.c_void_p), a.nbytes, ck["positions"], self.stream))
        szlib.check(self.lib.sz_session_set_len(self.h, ck["positions"], self.stream))

    def generate(self, prompt, max_new, spec_k=3, greedy=True, sampler=None, lookup_min=4, eog=-1, device_accept=True, max_rounds=0):
        p = GenParams(spec_k, max_new, lookup_min, 1 if greedy else 0, eog, 1 if device_accept else 0,
                      sampler or Sampler(1.0, 20, 0.95, 0.0, 1), max_rounds, 0)
        pr = (C.c_uint32 * len(prompt))(*[int(t) for t in prompt])
        out = (C.c_uint32 * max_new)()
        log = (C.c_int32 * (2 * max_new))()
        st = GenStats()
        szlib.check(self.lib.sz_generate(self.h, pr, len(prompt), C.byref(p), out, log, max_new, C.byref(st), self.stream))
        n = st.n_tokens
        return list(out[:n]), [(log[2 * i], log[2 * i + 1]) for i in range(st.passes)], st


class Generator:
    """The loop in pieces (sz_gen_begin / sz_gen_run): feed the prompt, then run rounds and look at the statistics in between."""

    def __init__(self, sess, prompt, max_new, spec_k=3, greedy=True, sampler=None, lookup_min=4, eog=-1, device_accept=True, handle=None):
        """handle: a generator that already exists (sz_batch_gen_begin made it with these parameters): the prompt is not fed again."""
        self.sess, self.lib = sess, sess.lib
        self.p = GenParams(spec_k, max_new, lookup_min, 1 if greedy else 0, eog, 1 if device_accept else 0,
                           sampler or Sampler(1.0, 20, 0.95, 0.0, 1), 0, 0)
        if handle is not None:
            self.h = C.c_void_p(handle)
        else:
            pr = (C.c_uint32 * len(prompt))(*[int(t) for t in prompt])
            self.h = C.c_void_p()
            szlib.check(self.lib.sz_gen_begin(sess.h, pr, len(prompt), C.byref(self.p), sess.stream, C.byref(self.h)))
        self.out = (C.c_uint32 * max_new)()
        self.log = (C.c_int32 * (2 * max_new))()
        self.max_new = max_new
        self.stats = GenStats()

    def run(self, rounds=0):
        szlib.check(self.lib.sz_gen_run(self.h, rounds, self.out, self.log, self.max_new, C.byref(self.stats), self.sess.stream))
        return self.stats

    def tokens(self):
        return list(self.out[:self.stats.n_tokens])

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.sz_gen_free(self.h)
            self.h = None


class Batch:
    """Several sequences stepped together (`sz_batch_verify`, `sz_batch_prefill`, `sz_batch_gen_begin`, `sz_batch_gen_run`): sessions
    of one model on one stream; what reads weights takes the rows of all of them at once."""

    def __init__(self, dm, n, ctx, rows_max=None, kv_q8=True, head_proxy=False):
        self.lib = szlib.load()
        self.dm = dm
        self._stream = torch.cuda.Stream(dm.device)
        self.stream = self._stream.cuda_stream
        self.sessions = [Session(dm, ctx, kv_q8=kv_q8, stream=self._stream, head_proxy=head_proxy) for _ in range(n)]
        self.rows_max = rows_max or min(256, (n * szlib.MAX_VERIFY + 7) // 8 * 8)
        nb = C.c_int64()
        szlib.check(self.lib.sz_batch_scratch_bytes(C.byref(dm.model), self.rows_max, C.byref(nb)))
        self.mem = torch.empty(nb.value + 256, dtype=torch.uint8, device=dm.device)
        self.scratch = self.mem.data_ptr() + (-self.mem.data_ptr()) % 256
        self.scratch_bytes = nb.value
        szlib.check(self.lib.sz_batch_scratch_init(C.byref(dm.model), self.rows_max, self.scratch, self.stream))

    def verify(self, rows, accept=0, eog=-1, which=None):
        """rows: one list of token ids per sequence (`which`: the sessions that take part, default all).  Afterwards every one of
        them holds a pending pass: `result()` and `commit()` on the session."""
        ss = [self.sessions[i] for i in (which if which is not None else range(len(self.sessions)))]
        assert len(ss) == len(rows)
        hs = (C.c_void_p * len(ss))(*[s.h for s in ss])
        flat = [int(t) for r in rows for t in r]
        ids = (C.c_int32 * len(flat))(*flat)
        ms = (C.c_int32 * len(rows))(*[len(r) for r in rows])
        szlib.check(self.lib.sz_batch_verify(hs, len(ss), ids, ms, accept, eog, self.rows_max, self.scratch, self.scratch_bytes, self.stream))
        for s, r in zip(ss, rows):
            s._m = len(r)

    def prefill(self, prompts, which=None):
        """The prompts of the sessions fed in lockstep (`sz_batch_prefill`); every session is left with its last pass pending."""
        ss = [self.sessions[i] for i in (which if which is not None else range(len(self.sessions)))]
        assert len(ss) == len(prompts)
        n = len(ss)
        keep = [(C.c_int32 * len(p))(*[int(t) for t in p]) for p in prompts]
        hs = (C.c_void_p * n)(*[s.h for s in ss])
        ids = (C.c_void_p * n)(*[C.cast(k, C.c_void_p) for k in keep])
        lens = (C.c_int32 * n)(*[len(p) for p in prompts])
        szlib.check(self.lib.sz_batch_prefill(hs, n, ids, lens, self.rows_max, self.scratch, self.scratch_bytes, self.stream))
        for s, p in zip(ss, prompts):
            s._m = (len(p) - 1) % szlib.MAX_VERIFY + 1

    def begin(self, prompts, max_new, spec_k=3, eog=-1):
        """A generator per session, the prompts fed in lockstep (`sz_batch_gen_begin`)."""
        n = len(prompts)
        assert n == len(self.sessions)
        par = GenParams(spec_k, max_new, 4, 1, eog, 1, Sampler(1.0, 20, 0.95, 0.0, 1), 0, 0)
        keep = [(C.c_uint32 * len(p))(*[int(t) for t in p]) for p in prompts]
        hs = (C.c_void_p * n)(*[s.h for s in self.sessions])
        pr = (C.c_void_p * n)(*[C.cast(k, C.c_void_p) for k in keep])
        lens = (C.c_int32 * n)(*[len(p) for p in prompts])
        out = (C.c_void_p * n)()
        szlib.check(self.lib.sz_batch_gen_begin(hs, n, pr, lens, C.byref(par), self.rows_max, self.scratch, self.scratch_bytes, self.stream, out))
        return [Generator(s, p, max_new, spec_k=spec_k, eog=eog, handle=out[b]) for b, (s, p) in enumerate(zip(self.sessions, prompts))]

    def generate(self, prompts, max_new, spec_k=3, eog=-1, rounds=0, feed="batch"):
        """The prompts through the sessions (feed="batch": in lockstep; "alone": one session at a time), then the sequences decode
        in lockstep.  Returns the tokens of every sequence, their statistics and the device time of the steps in ms."""
        if feed == "batch":
            gens = self.begin(prompts, max_new, spec_k=spec_k, eog=eog)
        else:
            gens = [Generator(s, p, max_new, spec_k=spec_k, eog=eog) for s, p in zip(self.sessions, prompts)]
        n = len(gens)
        gh = (C.c_void_p * n)(*[g.h for g in gens])
        outs = (C.c_void_p * n)(*[C.cast(g.out, C.c_void_p) for g in gens])
        sts = (C.c_void_p * n)(*[C.cast(C.pointer(g.stats), C.c_void_p) for g in gens])
        dev = C.c_double(0.0)
        szlib.check(self.lib.sz_batch_gen_run(gh, n, rounds, outs, sts, self.rows_max, self.scratch, self.scratch_bytes, C.byref(dev), self.stream))
        return [g.tokens() for g in gens], [g.stats for g in gens], dev.value


def make_prompt(n_tokens, vocab, seed=1, block=16, substitute=0.1, cycles=None):
    """benchmark config 1's prompt: a block of `block` tokens repeated, with a fraction of random substitutions, so a suffix drafter
    finds repeats.  With `cycles` (token_cycles(...)[1]) the block is one of the model's own token cycles."""
    rng = np.random.default_rng(seed)
    base = rng.integers(0, vocab, block) if cycles is None else cycles[int(rng.integers(0, cycles.shape[0]))].numpy()[:block]
    ids = np.tile(base, (n_tokens + block - 1) // block)[:n_tokens].copy()
    sub = rng.random(n_tokens) < substitute
    ids[sub] = rng.integers(0, vocab, int(sub.sum()))
    return [int(t) for t in ids]
