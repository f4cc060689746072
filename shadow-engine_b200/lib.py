"""ctypes binding of libshadowzero_b200.so: one declaration per entry point of include/shadowzero_b200.h."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libshadowzero_b200.so")

OK, E_ARG, E_TYPE, E_CUDA, E_SCRATCH, E_DEVICE = 0, 1, 2, 3, 4, 5
TYPE_F32, TYPE_F16, TYPE_Q8_0, TYPE_IQ3_S, TYPE_BF16 = 0, 1, 8, 21, 30
MAX_VERIFY, MAX_TOPK = 8, 16


def TYPE_EXL3(k):
    return 1020 + k


class SzError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("shadowzero_b200 error %d: %s" % (code, text))
        self.code = code


class MoeLayerC(C.Structure):
    """struct sz_moe_layer"""
    _fields_ = [("hidden", C.c_int32), ("n_expert", C.c_int32), ("top_k", C.c_int32), ("expert_ff", C.c_int32),
                ("shared_ff", C.c_int32), ("expert_type", C.c_int32), ("shared_type", C.c_int32), ("reserved", C.c_int32),
                ("router", C.c_uint64), ("shared_router", C.c_uint64),
                ("gate", C.c_uint64), ("up", C.c_uint64), ("down", C.c_uint64),
                ("gate_stride", C.c_uint64), ("up_stride", C.c_uint64), ("down_stride", C.c_uint64),
                ("sh_gate", C.c_uint64), ("sh_up", C.c_uint64), ("sh_down", C.c_uint64),
                ("ep_first", C.c_int32), ("ep_count", C.c_int32), ("ep_shared", C.c_int32), ("ep_reserved", C.c_int32)]


class KArg(C.Structure):
    """struct sz_karg"""
    _fields_ = [("type", C.c_int32), ("reserved", C.c_int32), ("bits", C.c_uint64)]


P_PTR, P_CONST_PTR, P_U32, P_I32, P_U64, P_F32 = range(6)


class HeadC(C.Structure):
    """struct sz_head"""
    _fields_ = [("rows", C.c_int32), ("cols", C.c_int32), ("bits", C.c_int32), ("k_blk", C.c_int32),
                ("weight", C.c_uint64), ("w_q2", C.c_uint64), ("w_sc", C.c_uint64), ("work", C.c_uint64), ("work_bytes", C.c_int64)]


PLACE_HOST, PLACE_DEVICE = 0, 1
STATE_DELTA_S, STATE_DELTA_CONV, STATE_KV_K, STATE_KV_V, STATE_IDX_SELECTED, STATE_IDX_SCORES, STATE_IDX_RAW, STATE_PLE_HIST, STATE_PLE_TAIL = range(9)
HEAD_XR, HEAD_XQ, HEAD_XSC, HEAD_XCORR, HEAD_BMAX, HEAD_SEL, HEAD_ERR = range(7)

# name -> (restype, argtypes); every symbol include/shadowzero_b200.h declares
SYMBOLS = {
    "sz_version": (C.c_char_p, []),
    "sz_last_error": (C.c_char_p, []),
    "sz_trace_begin": (C.c_int, [C.POINTER(C.c_uint64), C.c_int, C.c_uint64]),
    "sz_trace_end": (C.c_int, []),
    "sz_trace_name": (C.c_char_p, [C.c_int]),
    "sz_dequant": (C.c_int, [C.c_int, C.c_uint64, C.c_int64, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_exl3_codebook": (C.c_int, [C.c_uint64, C.c_uint64]),
    "sz_exl3_reconstruct_inner": (C.c_int, [C.c_int, C.c_uint64, C.c_int64, C.c_int64, C.c_uint64, C.c_uint64]),
    "sz_moe_scratch_bytes": (C.c_int, [C.POINTER(MoeLayerC), C.c_int, C.POINTER(C.c_int64)]),
    "sz_moe_scratch_init": (C.c_int, [C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_moe_verify": (C.c_int, [C.POINTER(MoeLayerC), C.c_uint64, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                C.c_int64, C.c_uint64]),
    "sz_moe_verify_host": (C.c_int, [C.POINTER(MoeLayerC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_uint64, C.c_uint64, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_moe_launches": (C.c_int, [C.POINTER(MoeLayerC)]),
    "sz_moe_rows_scratch_bytes": (C.c_int, [C.POINTER(MoeLayerC), C.c_int, C.POINTER(C.c_int64)]),
    "sz_moe_rows": (C.c_int, [C.POINTER(MoeLayerC), C.c_uint64, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_moe_rows_status": (C.c_int, [C.POINTER(MoeLayerC), C.c_int, C.c_uint64, C.POINTER(C.c_int), C.c_uint64]),
    "sz_model_load_gguf": (C.c_int, [C.c_char_p, C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]),
    "sz_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "sz_weights_key_u64": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "sz_weights_model": (C.c_void_p, [C.c_void_p]),
    "sz_weights_bytes": (C.c_int64, [C.c_void_p]),
    "sz_weights_tensor_count": (C.c_int, [C.c_void_p]),
    "sz_weights_tensor_info": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "sz_weights_free": (None, [C.c_void_p]),
    # the session (struct pointers are passed with ctypes.byref, so they are declared as void pointers here)
    "sz_session_bytes": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "sz_session_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_uint64, C.c_int64, C.c_uint64, C.POINTER(C.c_void_p)]),
    "sz_session_destroy": (None, [C.c_void_p]),
    "sz_session_reset": (C.c_int, [C.c_void_p, C.c_uint64]),
    "sz_session_len": (C.c_int, [C.c_void_p]),
    "sz_session_capacity": (C.c_int, [C.c_void_p]),
    "sz_session_pending": (C.c_int, [C.c_void_p]),
    "sz_session_prefill": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_uint64]),
    "sz_session_verify": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64]),
    "sz_session_set_sampler": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sz_session_idx_words": (C.c_int, [C.c_void_p]),
    "sz_session_import": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_uint64]),
    "sz_session_set_len": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64]),
    "sz_session_set_stops": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_uint64]),
    "sz_session_stops": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    "sz_session_verify_sampled": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_uint64, C.c_int, C.c_uint64]),
    "sz_session_verify_tree": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_uint64]),
    "sz_session_tree_path": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int), C.c_uint64]),
    "sz_session_commit_path": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_uint64]),
    "sz_session_result": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p, C.c_void_p, C.c_uint64]),
    "sz_session_commit": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64]),
    "sz_session_fill_synthetic": (C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_uint64]),
    "sz_session_export": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_uint64]),
    "sz_session_trace_routes": (C.c_int, [C.c_void_p, C.c_int]),
    "sz_session_routes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64]),
    "sz_kernel_count": (C.c_int, []),
    "sz_kernel_name": (C.c_char_p, [C.c_int]),
    "sz_kernel_params": (C.c_int, [C.c_char_p, C.POINTER(C.c_int32), C.c_int]),
    "sz_kernel_launch": (C.c_int, [C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_uint32, C.c_uint64, C.c_void_p, C.c_int]),
    # host side of speculation
    "sz_lookup": (C.c_int, [C.POINTER(C.c_uint32), C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_uint32)]),
    "sz_drafter_new": (C.c_void_p, [C.c_int, C.c_int, C.c_int]),
    "sz_drafter_free": (None, [C.c_void_p]),
    "sz_drafter_push": (None, [C.c_void_p, C.c_uint32]),
    "sz_drafter_extend": (None, [C.c_void_p, C.POINTER(C.c_uint32), C.c_int]),
    "sz_drafter_len": (C.c_int, [C.c_void_p]),
    "sz_drafter_propose": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]),
    "sz_drafter_propose_with_min": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]),
    "sz_drafter_propose_after": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]),
    "sz_policy_new": (C.c_void_p, [C.c_int, C.c_int, C.c_double]),
    "sz_policy_free": (None, [C.c_void_p]),
    "sz_policy_accept_ema": (C.c_double, [C.c_void_p]),
    "sz_policy_neural_k": (C.c_int, [C.c_void_p, C.c_int]),
    "sz_policy_choose": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "sz_policy_chain": (C.c_int, [C.c_void_p, C.c_int, C.c_double, C.c_int, C.c_int]),
    "sz_policy_observe": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double]),
    "sz_policy_observe_chain": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double]),
    "sz_uniform": (C.c_double, [C.c_uint64, C.c_uint64]),
    "sz_sample_top": (C.c_uint32, [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint64]),
    "sz_tree_accept_sampled": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_int, C.c_void_p,
                                         C.POINTER(C.c_uint32)]),
    "sz_generate": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.c_int,
                              C.c_void_p, C.c_uint64]),
    "sz_gen_begin": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]),
    "sz_gen_run": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.c_int, C.c_void_p, C.c_uint64]),
    "sz_gen_set_stops": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.c_uint64]),
    "sz_gen_free": (None, [C.c_void_p]),
    "sz_batch_scratch_bytes": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int64)]),
    "sz_batch_scratch_init": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64, C.c_uint64]),
    "sz_batch_verify": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_uint64,
                                  C.c_int64, C.c_uint64]),
    "sz_batch_prefill": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_batch_gen_begin": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_void_p, C.c_int, C.c_uint64, C.c_int64,
                                     C.c_uint64, C.POINTER(C.c_void_p)]),
    "sz_batch_gen_run": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_uint64, C.c_int64,
                                   C.POINTER(C.c_double), C.c_uint64]),
    "sz_mma_cols_scratch_bytes": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "sz_mma_cols": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int64, C.c_uint64, C.c_int64, C.c_int, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_mma_cols_status": (C.c_int, [C.c_uint64, C.c_int, C.POINTER(C.c_int), C.c_uint64]),
    "sz_ep_unique_id": (C.c_int, [C.c_void_p]),
    "sz_ep_init": (C.c_int, [C.c_int, C.c_int, C.c_void_p]),
    "sz_ep_world": (C.c_int, []),
    "sz_ep_destroy": (C.c_int, []),
    "sz_moe_verify_partial": (C.c_int, [C.POINTER(MoeLayerC), C.c_uint64, C.c_int, C.c_uint64, C.c_uint64, C.c_int64, C.c_uint64]),
    "sz_moe_finish": (C.c_int, [C.c_uint64, C.c_int, C.c_int, C.c_uint64, C.c_uint64]),
    "sz_ep_p2p_bytes": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "sz_ep_p2p_alloc": (C.c_int, [C.c_int64, C.POINTER(C.c_uint64)]),
    "sz_ep_p2p_free": (C.c_int, [C.c_uint64]),
    "sz_ep_ipc_export": (C.c_int, [C.c_uint64, C.c_void_p]),
    "sz_ep_ipc_import": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "sz_ep_ipc_close": (C.c_int, [C.c_uint64]),
    "sz_ep_p2p_attach": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_uint64)]),
    "sz_ep_p2p_detach": (C.c_int, []),
    "sz_ep_p2p_world": (C.c_int, []),
    "sz_ep_p2p_status": (C.c_int, [C.POINTER(C.c_int)]),
    "sz_moe_finish_exchange": (C.c_int, [C.POINTER(MoeLayerC), C.c_int, C.c_uint64, C.c_uint64]),
    "sz_moe_static_scratch_max": (C.c_int, [C.POINTER(C.c_int64)]),
    "sz_moe_static_status": (C.c_int, [C.POINTER(C.c_int), C.c_uint64]),
    "sz_moe_static_reset": (C.c_int, []),
    "sz_head_proxy_bytes": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "sz_head_work_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "sz_head_work_init": (C.c_int, [C.POINTER(HeadC), C.c_uint64]),
    "sz_head_proxy_build": (C.c_int, [C.POINTER(HeadC), C.c_uint64]),
    "sz_head_plan": (C.c_int, [C.POINTER(HeadC), C.c_int, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "sz_head_top": (C.c_int, [C.POINTER(HeadC), C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64]),
    "sz_head_stage": (C.c_int, [C.POINTER(HeadC), C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_int64)]),
    "sz_moe_verify_static": (C.c_int, [C.POINTER(MoeLayerC), C.c_uint64, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
}

_lib = None


def load():
    """Loads the library; raises if it has not been built (no fallback of any kind)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python -c 'import __graft_entry__ as g; g.build()'`" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != OK:
        raise SzError(rc, load().sz_last_error().decode("utf-8", "replace"))


def version():
    return load().sz_version().decode()
