"""ctypes binding of libqdecode.so (the C ABI declared in include/qdecode.h).

The library is the only compute path: if it cannot be loaded the import fails
loudly; there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

PAGE_TOKENS = 64
HEAD_DIM = 128
MAX_ROWS = 64
ERR_DEVICE = -4      # q_status Q_ERR_DEVICE: a device status word reported a wait that ran out


class GemmPlan(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("chunks_per_group", C.c_int32), ("groups", C.c_int32),
        ("units_per_worker", C.c_int32), ("workers", C.c_int32),
        ("slots", C.c_int32), ("grid", C.c_int32), ("block", C.c_int32),
        ("group_rows", C.c_int32),
    ]


class KVLayout(C.Structure):
    _fields_ = [
        ("d_kpool", C.c_void_p), ("d_vpool", C.c_void_p), ("d_block_table", C.c_void_p),
        ("pages_per_seq", C.c_int32), ("n_kv_heads", C.c_int32),
    ]


class Config(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("inter", C.c_int32), ("n_layers", C.c_int32),
        ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("vocab", C.c_int32),
        ("vocab_offset", C.c_int32), ("full_vocab", C.c_int32), ("tp_size", C.c_int32),
        ("max_rows", C.c_int32), ("rms_eps", C.c_float), ("attn_scale", C.c_float),
    ]


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "wqkv", "wo", "wgu", "wdown", "ln_in", "ln_post", "q_gain", "k_gain", "kpool", "vpool",
        "wqkv_tc", "wo_tc", "wgu_tc", "wdown_tc")]


MAX_PEERS = 8


class Peers(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("partials", C.c_void_p * MAX_PEERS),
                ("flags", C.c_void_p * MAX_PEERS), ("epoch", C.c_void_p)]


class State(C.Structure):
    _fields_ = [
        ("embed", C.c_void_p), ("lm_head", C.c_void_p), ("ln_final", C.c_void_p),
        ("cos", C.c_void_p), ("sin", C.c_void_p), ("tokens", C.c_void_p), ("pos", C.c_void_p),
        ("block_table", C.c_void_p), ("pages_per_seq", C.c_int32), ("batch", C.c_int32),
        ("attn_splits", C.c_int32), ("q_tokens", C.c_int32),
        ("x", C.c_void_p), ("normed", C.c_void_p), ("q", C.c_void_p), ("attended", C.c_void_p),
        ("act", C.c_void_p), ("partials", C.c_void_p), ("reduced", C.c_void_p),
        ("attn_o", C.c_void_p), ("attn_ml", C.c_void_p), ("attn_tickets", C.c_void_p),
        ("logits", C.c_void_p),
        ("arg_val", C.c_void_p), ("arg_idx", C.c_void_p), ("arg_scratch", C.c_void_p),
        ("lm_head_tc", C.c_void_p), ("status_out", C.c_void_p),
    ]


_P = C.c_void_p
_I = C.c_int
_F = C.c_float
_PLAN = C.POINTER(GemmPlan)
_KV = C.POINTER(KVLayout)

# name -> (restype, argtypes); exactly the symbols include/qdecode.h declares.
SIGNATURES = {
    "q_last_error": (C.c_char_p, []),
    "q_version": (_I, []),
    "q_set_pdl": (_I, [_I]),
    "q_set_option": (_I, [C.c_char_p, _I]),
    "q_debug_timeline": (_I, [_P, _I]),
    "q_debug_timeline_kinds": (_I, [_P, _I]),
    "q_debug_attn_trace": (_I, [_P]),
    "q_debug_gemm_trace": (_I, [C.POINTER(C.c_uint64), _I]),
    "q_debug_tc_trace": (_I, [C.POINTER(C.c_uint64), _I]),
    "q_gemm_plan": (_I, [_I, _I, _I, _PLAN]),
    "q_packed_weight_bytes": (C.c_int64, [_I, _I]),
    "q_pack_weight": (_I, [_P, _P, _I, _I, _P]),
    "q_unpack_weight": (_I, [_P, _P, _I, _I, _P]),
    "q_gemm_splitk": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q_gemm_splitk_addnorm": (_I, [_P, _P, _PLAN, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "q_gemm_swiglu": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q_gemm_swiglu_addnorm": (_I, [_P, _P, _PLAN, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "q_reduce_partials": (_I, [_P, _PLAN, _P, _P]),
    "q_packed_weight_bytes_tc": (C.c_int64, [_I, _I]),
    "q_pack_weight_tc": (_I, [_P, _P, _I, _I, _P]),
    "q_unpack_weight_tc": (_I, [_P, _P, _I, _I, _P]),
    "q_gemm_tc_plan": (_I, [_I, _I, _I, _PLAN]),
    "q_gemm_tc": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q_peer_flag_bytes": (C.c_int64, []),
    "q_argmax_merge_peers": (_I, [_P, _P, C.POINTER(Peers), _I, _P, _P, _I, _P]),
    "q_step_merge": (_I, [_P, _P, _P, _P]),
    "q_verify_step": (_I, [_P, _P]),
    "q_clear_status": (_I, []),
    "q_add_rmsnorm_peers": (_I, [_P, C.POINTER(Peers), _P, _PLAN, _P, _P, _P, _I, _I, _F, _P]),
    "q_gemm_push": (_I, [_P, _P, _PLAN, C.POINTER(Peers), _P]),
    "q_gemm_splitk_addnorm_peers": (_I, [_P, C.POINTER(Peers), _PLAN, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "q_gemm_swiglu_addnorm_peers": (_I, [_P, C.POINTER(Peers), _PLAN, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "q_engine_peer_floats": (C.c_int64, [_P, _I]),
    "q_bind_peers": (_I, [_P, C.POINTER(Peers)]),
    "q_decode_step_peers": (_I, [_P, _P]),
    "q_static_scratch_floats": (C.c_int64, []),
    "q_linear_f32_static": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "q_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "q_embed_rmsnorm": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "q_add_rmsnorm": (_I, [_P, _P, _PLAN, _P, _P, _P, _I, _I, _F, _P]),
    "q_swiglu": (_I, [_P, _PLAN, _P, _I, _I, _P]),
    "q_swiglu_interleaved": (_I, [_P, _PLAN, _P, _I, _I, _P]),
    "q_qkv_norm_rope_cache": (_I, [_P, _PLAN, _P, _P, _P, _P, _P, _P, _KV, _I, _I, _I, _F, _P]),
    "q_kv_scatter": (_I, [_P, _P, _KV, _I, _I, _I, _P]),
    "q_attention_splits": (_I, [_I, _I, _I]),
    "q_attention": (_I, [_P, _KV, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P]),
    "q_attention_prefill": (_I, [_P, _KV, _P, _P, _I, _I, _I, _F, _P]),
    "q_attention_decode": (_I, [_P, _PLAN, _P, _P, _P, _P, _P, _KV, _P, _P, _P, _P, _I, _I, _I, _F, _F, _P]),
    "q_argmax_scratch_bytes": (C.c_int64, [_I, _I]),
    "q_logits_argmax": (_I, [_P, _PLAN, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _P]),
    "q_argmax_merge": (_I, [_P, _P, _I, _I, _P, _P, _I, _P]),
    "q_create": (_I, [C.POINTER(Config), C.POINTER(_P)]),
    "q_bind_layer": (_I, [_P, _I, C.POINTER(LayerWeights)]),
    "q_bind_state": (_I, [_P, C.POINTER(State)]),
    "q_engine_partial_floats": (C.c_int64, [_P, _I]),
    "q_destroy": (None, [_P]),
    "q_decode_step": (_I, [_P, _P]),
    "q_step_begin": (_I, [_P, _P]),
    "q_step_attn": (_I, [_P, _I, _P]),
    "q_step_post_attn": (_I, [_P, _I, _P]),
    "q_step_post_mlp": (_I, [_P, _I, _P]),
    "q_step_head": (_I, [_P, _P]),
    "q_device_status": (_I, [C.POINTER(C.c_int32 * 4)]),
}


class QDecodeError(RuntimeError):
    """A C-ABI call returned a non-zero status that is not an argument error."""


def _load() -> C.CDLL:
    path: Path = _build.LIB
    if not path.exists():
        # Building is allowed (nvcc cross-compiles without a GPU); falling back is not.
        _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int) -> None:
    """Raises ValueError for argument errors (like the reference's wrappers do
    before any launch) and QDecodeError for everything else."""
    if rc == 0:
        return
    msg = (lib.q_last_error() or b"").decode("utf-8", "replace")
    if rc == -1:
        raise ValueError(msg)
    raise QDecodeError(f"qdecode status {rc}: {msg}")


def plan(M: int, N: int, K: int, tc: bool = False) -> GemmPlan:
    """Split-K plan of the stream-K kernel, or (tc) of the tcgen05 kernel."""
    p = GemmPlan()
    check((lib.q_gemm_tc_plan if tc else lib.q_gemm_plan)(M, N, K, C.byref(p)))
    return p
