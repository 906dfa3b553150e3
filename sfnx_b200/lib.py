"""ctypes binding of libsfnx_b200.so, the C ABI declared in include/sfnx_b200.h.

Pointers are plain integers (torch `tensor.data_ptr()`), streams are `torch.cuda.Stream.cuda_stream` values.  A call
that returns non-zero raises FnxError with fnx_last_error()'s text, as the reference's launch wrappers throw
std::runtime_error.  There is no CPU fallback: without the built library, loading raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsfnx_b200.so")

MAXT = 16
TOPK_N = 64
HS = 128
Q4_K, Q6_K, Q8_0 = 12, 14, 8


class FnxError(RuntimeError):
    pass


class Job(C.Structure):
    _fields_ = [("w", C.c_int), ("n", C.c_int), ("y", C.c_int * MAXT), ("out", C.c_int * MAXT)]


class Q8S(C.Structure):
    _fields_ = [("q", C.c_void_p), ("d", C.c_void_p)]


class Experts(C.Structure):
    _fields_ = [("type", C.c_int), ("nrows", C.c_int), ("ncols", C.c_int), ("a", C.c_void_p), ("b", C.c_void_p),
                ("c", C.c_void_p), ("d", C.c_void_p), ("stride", C.c_size_t), ("stride_b", C.c_size_t)]


class GdnLanes(C.Structure):
    _fields_ = [("S", C.c_void_p), ("hist", C.c_void_p), ("ctl", C.c_void_p), ("row0", C.c_void_p), ("snap", C.c_void_p), ("hsnap", C.c_void_p)]


class LaneRows(C.Structure):
    _fields_ = [("pos", C.c_void_p), ("pt", C.c_void_p)]


class KvPages(C.Structure):
    _fields_ = [("pt", C.c_void_p), ("page", C.c_size_t), ("rows", C.c_int), ("cap", C.c_int), ("q8", C.c_int)]


class Rope(C.Structure):
    _fields_ = [("base", C.c_float), ("nrot", C.c_int)]


class StackCfg(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("n", "nexp", "topk", "ff", "nk", "nv", "nq", "nkv", "hd", "nrot", "vocab0", "vocab_rows",
                                        "nlayers", "ncard", "card")] + [("eps", C.c_float), ("rope_base", C.c_float), ("hc", C.c_int),
                                                                        ("hc_lr", C.c_int), ("r_preset", C.c_int), ("qsa_top", C.c_int),
                                                                        ("qsa_ring_rows", C.c_int), ("qsa_max_pools", C.c_int)]


class HcW(C.Structure):
    _fields_ = [("norm", C.c_void_p), ("down", Q8S), ("up", Q8S), ("inj", C.c_void_p)]


class QsaW(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ("wq", "wk", "qn", "kn", "ring", "pooled")] + [("page", C.c_size_t)]


class Layer(C.Structure):
    _fields_ = [("kind", C.c_int), ("norm1", C.c_void_p), ("norm2", C.c_void_p),
                ("qkvz", Q8S), ("ab", C.c_void_p), ("conv", C.c_void_p), ("dt", C.c_void_p), ("a", C.c_void_p),
                ("ssm_norm", C.c_void_p), ("ssm_out", Q8S), ("vmap", C.c_void_p),
                ("S", C.c_void_p), ("hist", C.c_void_p), ("snap", C.c_void_p), ("hsnap", C.c_void_p),
                ("wq", Q8S), ("wk", Q8S), ("wv", Q8S), ("wo", Q8S), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("kc", C.c_void_p), ("vc", C.c_void_p), ("pages", KvPages),
                ("router", C.c_void_p), ("gate_up", Experts), ("down", Experts), ("sh_gate_up", Q8S), ("sh_down", Q8S), ("gdn_log", C.c_void_p),
                ("hcw", HcW * 2), ("idx", QsaW)]


class WindowLanes(C.Structure):
    _fields_ = [("nseg", C.c_int), ("rows", C.c_int), ("ctl", C.c_void_p), ("row0", C.c_void_p), ("row_pos", C.c_void_p), ("row_pt", C.c_void_p),
                ("ctl_host", C.c_void_p), ("pt_host", C.c_void_p), ("S", C.c_void_p), ("hist", C.c_void_p), ("S_host", C.c_void_p),
                ("hist_host", C.c_void_p), ("idx_ring_host", C.c_void_p)]


class Draft(C.Structure):
    _fields_ = [("norm_emb", C.c_void_p), ("norm_hid", C.c_void_p), ("fc_emb", Q8S), ("fc_hid", Q8S)]


class Head(C.Structure):
    _fields_ = [("norm", C.c_void_p), ("out", Q8S), ("mix", HcW)]


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("top_k", C.c_int)]


RING_MAX = 8


class Ring(C.Structure):
    _fields_ = [("nrank", C.c_int), ("rank", C.c_int), ("slot", (C.c_void_p * RING_MAX) * 2), ("pad", C.c_void_p * RING_MAX),
                ("state", C.c_void_p), ("spin_limit", C.c_uint), ("ll", (C.c_void_p * RING_MAX) * 2), ("ll_count", C.c_size_t)]


class MoeRows(C.Structure):
    _fields_ = [("part", C.c_void_p), ("topw", C.c_void_p), ("sh", C.c_void_p), ("logits", C.c_void_p), ("nexp", C.c_int), ("topk", C.c_int)]


class GdnReplay(C.Structure):
    _fields_ = [("S", C.c_void_p), ("log", C.c_void_p), ("vmap", C.c_void_p), ("nk", C.c_int), ("nv", C.c_int), ("row0", C.c_int), ("n", C.c_int)]


class CopyJob(C.Structure):
    _fields_ = [("dst", C.c_void_p), ("src", C.c_void_p), ("bytes", C.c_size_t)]


_p, _i, _f, _z, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_ulonglong

# name -> argument types; every function returns int status unless listed in _OTHER
_SIGS = {
    "fnx_quantize_q8_1": [_p, _p, _i, _i, _p],
    "fnx_rms_norm_rows": [_p, _p, _p, _p, _p, _i, _i, _f, _p],
    "fnx_q8s_gemv": [Q8S, _i, _i, _p, _p, _i, _i, _p],
    "fnx_q8s_gemv_segs": [_p, _p, _p, _p, _i, _i, _p, _i, _p],
    "fnx_q8s_gemv_blocks": [Q8S, _i, _i, _p, _p, _i, _i, _p],
    "fnx_gemv_f32": [_p, _p, _p, _i, _i, _i, _p],
    "fnx_router_route": [_p, _p, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p],
    "fnx_moe_gate_up": [C.POINTER(Experts), _p, _p, _i, _p, _p, _p],
    "fnx_moe_down": [C.POINTER(Experts), _p, _p, _i, _p, _i, _p, _p, _p],
    "fnx_mmvq": [C.POINTER(Experts), _p, _p, _i, _p, _p, _i, _p],
    "fnx_q8s_gemv_f32": [Q8S, _i, _i, _p, _p, _p, _p, _p, _i, _i, _p],
    "fnx_moe_gate_up_mma": [C.POINTER(Experts), _p, _p, _i, _p, _p, _p],
    "fnx_swiglu_h16": [_p, _i, _i, _p, _p],
    "fnx_moe_down_mma": [C.POINTER(Experts), _p, _p, _i, _p, _p, _p],
    "fnx_moe_down_noalloc": [C.POINTER(Experts), _p, _p, _i, _p, _i, _p, _p],
    "fnx_shared_expert": [Q8S, Q8S, _p, _i, _i, _i, _p, _p, _p, _p],
    "fnx_moe_combine": [_p, _p, _p, _p, _i, _p, _i, _i, _i, _p],
    "fnx_gdn_core": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _i, _f, _p, _p],
    "fnx_gdn_core_segs": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, C.POINTER(GdnLanes), _i, _i, _f, _p],
    "fnx_gdn_core_lanes": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, C.POINTER(GdnLanes), _i, _f, _p],
    "fnx_copy_many": [_p, _i, _p],
    "fnx_l2_prefetch": [_p, _z, _p],
    "fnx_gdn_core_log": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _i, _f, _p],
    "fnx_gdn_replay": [_p, _i, _i, _p],
    "fnx_ring_gather": [_p, _i, _p, _i, _p, _p, _p, _p, _p],
    "fnx_attn_finish_ring": [_p, _p, _p, _p, _p, _i, _i, _i, _p, _p],
    "fnx_hc_expand": [_p, _p, _i, _i, _i, _p],
    "fnx_hc_add_streams": [_p, _p, _p, _i, _i, _i, _p],
    "fnx_draft_begin": [_p, _p, _p, _p, _p, _i, _p],
    "fnx_hc_write": [_p, _p, _p, _i, _i, _i, _p],
    "fnx_hc_read": [_p, _p, _p, _p, Q8S, Q8S, _p, _f, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "fnx_attn_prep_append": [_p, _p, _p, _p, _p, _p, _p, KvPages, _i, _i, _i, _p, _f, Rope, _i, _i, _i, _p],
    "fnx_attn_partial": [_p, _p, _p, KvPages, _p, _i, _i, _i, _p, _i, _i, _i, _p, _p],
    "fnx_attn_partial_exact": [_p, _p, _p, KvPages, _p, _i, _i, _i, _p, _i, _i, _i, _p, _p],
    "fnx_attn_part_lanes": [_p, _p, _p, KvPages, LaneRows, _p, _i, _i, _i, _i, _i, _i, _p, _p],
    "fnx_attn_partial_cells": [_p, _p, _p, KvPages, LaneRows, _p, _i, _i, _i, _p, _i, _i, _i, _p, _p, _p, _i, _p],
    "fnx_attn_finish": [_p, _i, _i, _p, _p, _i, _i, _i, _i, _i, _p],
    "fnx_qsa_rows": [],
    "fnx_qsa_maxsel": [_i],
    "fnx_qsa_proj": [_p, _p, _p, _p, _i, _i, _p],
    "fnx_qsa_index": [_p, _p, _p, _p, _i, _p, KvPages, _i, _p, _p, _i, _f, Rope, _p],
    "fnx_qsa_select": [_p, _p, KvPages, LaneRows, _p, _p, _p, _i, _p, _i, _i, _i, _i, _p],
    "fnx_qsa": [_p, _p, _p, _i, _p, _p, _p, _p, _i, _p, KvPages, _p, _p, _p, _p, _i, _p, _i, _f, Rope, _i, _i, _i, _p],
    "fnx_argmax": [_p, _i, _i, _i, _p, _p, _p, _p, _p],
    "fnx_penalize_row": [_p, _i, _p, _p, _p],
    "fnx_top_tokens": [_p, _i, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p],
    "fnx_repack_q8_0_split": [_p, _p, _p, _z, _z, _p],
    "fnx_repack_q6k_units": [_p, _z, _z, _z, _z, _p, _p, _p, _p, _p],
    "fnx_synth_normal": [_p, _z, _f, _u64, _p],
    "fnx_synth_quant": [_i, _p, _z, _f, _u64, _p],
    "fnx_math_probe": [_i, _p, _p, _z, _p],
    "fnx_embed_rows": [_p, _p, _p, _i, _i, _p],
    "fnx_window_init": [_p, _p, _p],
    "fnx_window_side_stream": [_p, _p, _p],
    "fnx_window_ring": [_p],
    "fnx_window_stage": [_p, _p, _p, _p, _i, _i, _p],
    "fnx_window_commit": [_p, _p, _p, _i, _i, _i, _p, _p],
    "fnx_window_stage_lanes": [_p, _p, _p, _p, C.POINTER(WindowLanes), _i, _p],
    "fnx_window_commit_lanes": [_p, _p, _p, C.POINTER(WindowLanes), _p, _p, _p, _p],
    "fnx_top_merge": [_p, _p, _i, _i, _p, _p],
    "fnx_ring_sum": [_p, _i, _i, C.POINTER(Ring), _p, _p],
    "fnx_boundary_rows": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p, _p],
}
_OTHER = {
    "fnx_last_error": (C.c_char_p, []),
    "fnx_built_arch": (_i, []),
    "fnx_device_fault": (C.c_uint, []),
    "fnx_router_scratch_bytes": (_z, []),
    "fnx_moe_h_bytes": (_z, [_i, _i]),
    "fnx_gdn_scratch_floats": (_z, [_i]),
    "fnx_gdn_log_floats": (_z, [_i, _i]),
    "fnx_attn_scratch_floats": (_z, [_i, _i, _i]),
    "fnx_kvq_halves": (_z, [_i, _i, _i]),
    "fnx_hc_scratch_floats": (_z, [_i, _i, _i, _i]),
    "fnx_kv_rows_per_card": (_i, [_i, _i]),
    "fnx_attn_splits": (_i, [_i]),
    "fnx_window_workspace_bytes": (_z, [_p]),
    "fnx_window_plan": (_i, [_p, _p, _p, _i]),
    "fnx_window_buf": (_p, [_p, _p, _i]),
    "fnx_accept_greedy": (_i, [_p, _p, _i]),
    "fnx_lookup_drafts": (_i, [_p, _i, _i, _i, _i, _p]),
    "fnx_trace_begin": (_i, []),
    "fnx_trace_end": (_i, [_p, _p, _p, _i]),
    "fnx_window_kernel_count": (C.c_long, [_i]),
    "fnx_rng_new": (_p, [_u64]),
    "fnx_rng_free": (None, [_p]),
    "fnx_accept_sampled": (_i, [_p, _i, _p, _p, _p, _p, _p]),
    "fnx_ff_lo": (_i, [_i, _i, _i]),
    "fnx_vhead_card": (_i, [_i, _i, _i, _i]),
    "fnx_khead_first": (_i, [_i, _i, _i, _i]),
    "fnx_khead_count": (_i, [_i, _i, _i, _i]),
}

_lib = None


def declared_symbols():
    """Every entry point include/sfnx_b200.h declares."""
    return sorted(list(_SIGS) + list(_OTHER))


def load():
    """The loaded library (raises if it has not been built: there is no other implementation to fall back to)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FnxError("libsfnx_b200.so is not built: run `python -m sfnx_b200.build` (nvcc, sm_100a)")
        lib = C.CDLL(LIB_PATH)
        for name, args in _SIGS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i
        for name, (res, args) in _OTHER.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res
        _lib = lib
    return _lib


def call(name, *args):
    """Calls a status-returning entry point; raises FnxError with the library's text on failure."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise FnxError(lib.fnx_last_error().decode())
    return 0


def ptr(t):
    """Device (or host) address of a torch tensor, None -> NULL."""
    return None if t is None else t.data_ptr()


def stream():
    import torch

    return torch.cuda.current_stream().cuda_stream
