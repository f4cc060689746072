"""Model files: a GGUF writer for the synthetic models of `model.make_model`, and the library's reader (`sz_model_load_gguf`) as
model placements that `model.Session` and the CPU oracle take.

The writer emits the format the reference reads (crates/shadowzero-model/src/gguf.rs:330-420): magic, version 3, counts, key-values,
tensor table (name, dimensions in ggml order - row length first -, type id, offset), the data section at the next multiple of
general.alignment (32).  Keys are the ones Config::from_gguf reads (crates/shadowzero-model/src/forward.rs:72-142), tensor names and
dimension order those of crates/shadowzero-model/src/exl3_model.rs:223-243.  EXL3 tensors carry the reference's own type ids
(1020 + bits, gguf.rs:141-143) and are sized by their span, as there.  The keys of the two branches this build does not have are
written so that they describe "none": ple.layers names a layer past the last one, every compress ratio is 0."""
import ctypes as C
import struct

import numpy as np
import torch

from . import lib as szlib

ALIGN = 32
T_U32, T_F32, T_STR, T_ARR, T_U64, T_I64, T_F64 = 4, 6, 8, 9, 10, 11, 12


def _s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _kv(key, ty, val):
    out = _s(key) + struct.pack("<I", ty)
    if ty == T_U32:
        return out + struct.pack("<I", val)
    if ty == T_U64:
        return out + struct.pack("<Q", val)
    if ty == T_F32:
        return out + struct.pack("<f", val)
    if ty == T_F64:
        return out + struct.pack("<d", val)
    if ty == T_STR:
        return out + _s(val)
    if ty == T_ARR:   # arrays of i64
        return out + struct.pack("<IQ", T_I64, len(val)) + b"".join(struct.pack("<q", v) for v in val)
    raise ValueError(ty)


def _bytes(t):
    t = t.detach().cpu().contiguous()
    return (t.view(torch.uint8) if t.dtype != torch.uint8 else t).numpy().reshape(-1)


def write_gguf(path, M, arch="qwen4exp"):
    """Writes the model `M` (the dict `model.make_model` returns) as one GGUF file."""
    cfg = M["cfg"]
    n_layer = cfg["n_layer"]
    kvs = [
        _kv("general.architecture", T_STR, arch), _kv("general.alignment", T_U32, ALIGN), _kv("general.name", T_STR, "seeded synthetic hybrid MoE"),
        _kv(arch + ".block_count", T_U32, n_layer), _kv(arch + ".embedding_length", T_U32, cfg["hidden"]),
        _kv(arch + ".attention.key_length", T_U32, cfg["head_dim"]), _kv(arch + ".attention.head_count", T_U32, cfg["n_head"]),
        _kv(arch + ".attention.head_count_kv", T_U32, cfg["n_kv_head"]), _kv(arch + ".attention.layer_norm_rms_epsilon", T_F32, cfg["eps"]),
        _kv(arch + ".rope.dimension_count", T_U32, cfg["rope_dims"]), _kv(arch + ".rope.freq_base", T_F32, cfg["rope_theta"]),
        _kv(arch + ".expert_count", T_U32, cfg["n_expert"]), _kv(arch + ".expert_used_count", T_U32, cfg["n_expert_used"]),
        _kv(arch + ".expert_feed_forward_length", T_U32, cfg["expert_ff"]), _kv(arch + ".ssm.group_count", T_U32, cfg["ssm_k_heads"]),
        _kv(arch + ".ssm.time_step_rank", T_U32, cfg["ssm_v_heads"]), _kv(arch + ".ssm.inner_size", T_U32, cfg["ssm_v_heads"] * cfg["ssm_head_dim"]),
        _kv(arch + ".ssm.conv_kernel", T_U32, cfg["conv_k"]), _kv(arch + ".full_attention_interval", T_U32, cfg["attn_interval"]),
        _kv(arch + ".hyper_connection.count", T_U32, cfg["streams"]), _kv(arch + ".hyper_connection.low_rank", T_U32, cfg["hc_rank"]),
    ]
    if cfg.get("ple_ngram", 0) >= 2:  # the per-layer embedding of one layer (forward.rs:93-136)
        kvs += [_kv(arch + ".ple.layers", T_ARR, [cfg["ple_layer"]]), _kv(arch + ".ple.ngram_size", T_U32, cfg["ple_ngram"]),
                _kv(arch + ".ple.heads_per_ngram", T_U32, cfg["ple_heads_per_ngram"]), _kv(arch + ".embedding_length_per_layer_input", T_U32, cfg["ple_head_dim"]),
                _kv(arch + ".ple.conv_kernel", T_U32, cfg["ple_conv_k"]), _kv(arch + ".ple.eos_token_id", T_U32, cfg["ple_eos"]),
                _kv(arch + ".ple.layer_multipliers", T_ARR, list(cfg["ple_multipliers"])), _kv(arch + ".ple.head_vocab_sizes", T_ARR, list(cfg["ple_vocab"])),
                _kv(arch + ".ple.head_offsets", T_ARR, list(cfg["ple_offsets"]))]
    else:                             # none: the keys are there for the reference's Config::from_gguf, naming a layer past the last
        kvs += [_kv(arch + ".ple.layers", T_ARR, [n_layer]), _kv(arch + ".ple.ngram_size", T_U32, 1), _kv(arch + ".ple.heads_per_ngram", T_U32, 1),
                _kv(arch + ".embedding_length_per_layer_input", T_U32, 0), _kv(arch + ".ple.conv_kernel", T_U32, 1), _kv(arch + ".ple.eos_token_id", T_U32, 0),
                _kv(arch + ".ple.layer_multipliers", T_ARR, []), _kv(arch + ".ple.head_vocab_sizes", T_ARR, []), _kv(arch + ".ple.head_offsets", T_ARR, [])]
    if cfg.get("idx_heads", 0) > 0:   # the sparse indexer of the attention layers (forward.rs:137-140)
        ratios = [int(cfg.get("idx_ratio", 4)) if (l % cfg["attn_interval"] == cfg["attn_interval"] - 1) else 0 for l in range(n_layer)]
        kvs += [_kv(arch + ".attention.indexer.head_count", T_U32, cfg["idx_heads"]), _kv(arch + ".attention.indexer.key_length", T_U32, cfg["idx_dim"]),
                _kv(arch + ".attention.indexer.top_k", T_U32, cfg["idx_budget"]), _kv(arch + ".attention.compress_ratios", T_ARR, ratios)]
    else:                             # none: no heads, a budget no context reaches
        kvs += [_kv(arch + ".attention.indexer.head_count", T_U32, 0), _kv(arch + ".attention.indexer.key_length", T_U32, 0),
                _kv(arch + ".attention.indexer.top_k", T_U32, 1 << 30), _kv(arch + ".attention.compress_ratios", T_ARR, [0] * n_layer)]
    tensors = []   # (name, dims in ggml order, type id, uint8 array)

    def add(name, dims, ty, data):
        tensors.append((name, dims, ty, _bytes(data)))

    for name, (ty, rows, cols, b) in M["tensors"].items():
        is_vec = ty == szlib.TYPE_F32 and rows == 1
        add(name, [cols] if is_vec else [cols, rows], ty, b)
    for l, Ld in enumerate(M["moe"]):
        p = "blk.%d." % l
        H, ne, FF, SF = Ld["hidden"], Ld["n_expert"], Ld["expert_ff"], Ld["shared_ff"]
        add(p + "ffn_gate_inp.weight", [H, ne], szlib.TYPE_F32, Ld["router"])
        add(p + "ffn_gate_exps.weight", [H, FF, ne], Ld["expert_type"], Ld["gate"])
        add(p + "ffn_up_exps.weight", [H, FF, ne], Ld["expert_type"], Ld["up"])
        add(p + "ffn_down_exps.weight", [FF, H, ne], Ld["expert_type"], Ld["down"])
        if SF > 0:
            add(p + "ffn_gate_inp_shexp.weight", [H], szlib.TYPE_F32, Ld["shared_router"])
            add(p + "ffn_gate_shexp.weight", [H, SF], Ld["shared_type"], Ld["sh_gate"])
            add(p + "ffn_up_shexp.weight", [H, SF], Ld["shared_type"], Ld["sh_up"])
            add(p + "ffn_down_shexp.weight", [SF, H], Ld["shared_type"], Ld["sh_down"])
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)) + b"".join(kvs)
    infos, off = [], 0
    for name, dims, ty, data in tensors:
        infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off))
        off = (off + data.size + ALIGN - 1) // ALIGN * ALIGN
    head += b"".join(infos)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((-len(head)) % ALIGN))
        for _, _, _, data in tensors:
            f.write(data.tobytes())
            f.write(b"\0" * ((-data.size) % ALIGN))
    return path


class LoadedModel:
    """A GGUF file read by the library (`sz_model_load_gguf`): `.model` is struct sz_model, `.cfg` its shape as a dict.  Placed in
    host memory it is what `oracle.binding.Session` takes, placed on the device what `model.Session` takes."""

    def __init__(self, path, device=None):
        from . import model as md
        self.lib = szlib.load()
        self.h = C.c_void_p()
        self.device = torch.device(device) if device is not None else None
        stream = 0
        if self.device is not None:
            torch.cuda.set_device(self.device)
            stream = torch.cuda.current_stream(self.device).cuda_stream
        szlib.check(self.lib.sz_model_load_gguf(str(path).encode(), szlib.PLACE_HOST if device is None else szlib.PLACE_DEVICE, stream, C.byref(self.h)))
        self.model = md.Model.from_address(self.lib.sz_weights_model(self.h))
        c = self.model.cfg
        self.cfg = {n: getattr(c, n) for n, _ in md.ModelConfig._fields_ if n != "reserved"}
        P = self.model.ple
        if P.ngram >= 2:
            heads = (P.ngram - 1) * P.heads_per_ngram
            self.cfg.update(ple_layer=P.layer, ple_ngram=P.ngram, ple_heads_per_ngram=P.heads_per_ngram, ple_head_dim=P.head_dim, ple_conv_k=P.conv_k,
                            ple_eos=P.eos, ple_multipliers=list(P.multipliers[:P.ngram]), ple_vocab=list(P.vocab[:heads]), ple_offsets=list(P.offsets[:heads]))

    def tensor_info(self, name):
        ty, dims, n = C.c_int32(), (C.c_int64 * 4)(), C.c_int64()
        szlib.check(self.lib.sz_weights_tensor_info(self.h, name.encode(), C.byref(ty), dims, C.byref(n)))
        return ty.value, list(dims), n.value

    def close(self):
        if getattr(self, "h", None):
            self.lib.sz_weights_free(self.h)
            self.h = None

    def __del__(self):
        self.close()
