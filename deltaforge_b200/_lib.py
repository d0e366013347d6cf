"""ctypes binding of ``libdfb200.so`` (declarations in ``include/dfb200.h``).

There is no fallback: if the library cannot be loaded, or a call returns non-zero, this raises.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

c_i32, c_i64, c_f32, c_vp, c_sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t


class GemvDesc(C.Structure):
    _fields_ = [
        ("x", c_vp), ("x_stride", c_i64), ("rows", c_i32),
        ("packed", c_vp), ("scale", c_vp), ("scale_is_bf16", c_i32),
        ("K", c_i32), ("N", c_i32), ("group", c_i32),
        ("prologue", c_i32), ("norm_w", c_vp), ("eps", c_f32), ("up", c_vp), ("up_stride", c_i64),
        ("epilogue", c_i32), ("out", c_vp), ("out_stride", c_i64), ("residual", c_vp), ("residual_stride", c_i64),
        ("conv_state", c_vp), ("conv_w", c_vp), ("conv_dim", c_i32),
        ("scratch", c_vp), ("scratch_bytes", c_sz), ("math", c_i32), ("force_tiled", c_i32),
        ("packed_k8", c_vp), ("packed_mma", c_vp),
    ]  # fmt: skip


class DeltaNetDesc(C.Structure):
    _fields_ = [
        ("batch", c_i32), ("num_k_heads", c_i32), ("num_v_heads", c_i32), ("dk", c_i32), ("dv", c_i32),
        ("q", c_vp), ("k", c_vp), ("v", c_vp), ("z", c_vp), ("b", c_vp), ("a", c_vp), ("row_stride", c_i64),
        ("a_log", c_vp), ("dt_bias", c_vp), ("norm_w", c_vp), ("norm_w_is_bf16", c_i32), ("eps", c_f32),
        ("state", c_vp), ("out", c_vp), ("out_stride", c_i64),
    ]  # fmt: skip


class AttnDesc(C.Structure):
    _fields_ = [
        ("batch", c_i32), ("hq", c_i32), ("hkv", c_i32), ("d", c_i32),
        ("q", c_vp), ("q_stride", c_i64), ("qh_stride", c_i64),
        ("kcache", c_vp), ("vcache", c_vp), ("kv_batch_stride", c_i64), ("kv_head_stride", c_i64),
        ("key_len", c_i32), ("pos", c_vp), ("scale", c_f32), ("splits", c_i32),
        ("scratch", c_vp), ("scratch_bytes", c_sz),
        ("gate", c_vp), ("gate_stride", c_i64), ("gateh_stride", c_i64), ("gate_is_swish", c_i32),
        ("out", c_vp), ("out_stride", c_i64),
    ]  # fmt: skip


class AttnPrepDesc(C.Structure):
    _fields_ = [
        ("batch", c_i32), ("hq", c_i32), ("hkv", c_i32), ("d", c_i32), ("rotary_dim", c_i32),
        ("proj", c_vp), ("proj_stride", c_i64), ("q_norm_w", c_vp), ("k_norm_w", c_vp), ("eps", c_f32),
        ("inv_freq", c_vp), ("pos", c_vp), ("q_out", c_vp), ("kcache", c_vp), ("vcache", c_vp),
        ("kv_batch_stride", c_i64), ("kv_head_stride", c_i64), ("attn_output_gate", c_i32), ("max_seq", c_i32),
    ]  # fmt: skip


class AttnStepDesc(C.Structure):
    _fields_ = [
        ("batch", c_i32), ("hq", c_i32), ("hkv", c_i32), ("d", c_i32), ("rotary_dim", c_i32),
        ("proj", c_vp), ("proj_stride", c_i64), ("q_norm_w", c_vp), ("k_norm_w", c_vp), ("eps", c_f32),
        ("inv_freq", c_vp), ("pos", c_vp), ("kcache", c_vp), ("vcache", c_vp),
        ("kv_batch_stride", c_i64), ("kv_head_stride", c_i64), ("max_seq", c_i32),
        ("attn_output_gate", c_i32), ("gate_is_swish", c_i32), ("scale", c_f32), ("splits", c_i32), ("cluster_size", c_i32),
        ("scratch", c_vp), ("scratch_bytes", c_sz), ("out", c_vp), ("out_stride", c_i64), ("status", c_vp),
    ]  # fmt: skip


class Linear(C.Structure):
    _fields_ = [
        ("packed", c_vp), ("scale", c_vp), ("scale_is_bf16", c_i32), ("K", c_i32), ("N", c_i32), ("group", c_i32),
        ("packed_k8", c_vp), ("packed_mma", c_vp), ("mma_pair", c_i32),
    ]  # fmt: skip


class LayerDesc(C.Structure):
    _fields_ = [
        ("kind", c_i32), ("input_norm_w", c_vp), ("post_norm_w", c_vp),
        ("in_proj", Linear), ("out_proj", Linear), ("gate_up", Linear), ("down", Linear),
        ("conv_w", c_vp), ("a_log", c_vp), ("dt_bias", c_vp), ("gnorm_w", c_vp), ("gnorm_w_is_bf16", c_i32),
        ("conv_state", c_vp), ("recurrent", c_vp),
        ("q_norm_w", c_vp), ("k_norm_w", c_vp), ("kcache", c_vp), ("vcache", c_vp),
    ]  # fmt: skip


class ModelDesc(C.Structure):
    _fields_ = [
        ("hidden", c_i32), ("intermediate", c_i32), ("vocab", c_i32), ("num_layers", c_i32), ("batch", c_i32), ("max_seq", c_i32),
        ("hq", c_i32), ("hkv", c_i32), ("head_dim", c_i32), ("rotary_dim", c_i32), ("attn_output_gate", c_i32), ("gate_is_swish", c_i32),
        ("lin_k_heads", c_i32), ("lin_v_heads", c_i32), ("lin_dk", c_i32), ("lin_dv", c_i32),
        ("eps", c_f32), ("inv_freq", c_vp), ("embed", c_vp), ("final_norm_w", c_vp), ("head", Linear),
        ("layers_host", C.POINTER(LayerDesc)),
        ("tokens", c_vp), ("history", c_vp), ("pos", c_vp), ("logits", c_vp),
        ("workspace", c_vp), ("workspace_bytes", c_sz), ("attn_splits", c_i32), ("math", c_i32),
        ("tp_size", c_i32), ("tp_rank", c_i32), ("tp_peer_slots", C.POINTER(c_vp)),
    ]  # fmt: skip


# name -> (restype, argtypes); every exported symbol of include/dfb200.h
SIGNATURES = {
    "dfb_last_error": (C.c_char_p, []),
    "dfb_abi_version": (C.c_int, []),
    "dfb_int4_group_size": (C.c_int, [C.c_int]),
    "dfb_int4_quantise_k_major": (C.c_int, [c_vp, C.c_int, C.c_int, C.c_int, c_vp, c_vp, c_vp]),
    "dfb_int4_unpack": (C.c_int, [c_vp, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_int4_dequant": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_int4_repack_k8": (C.c_int, [c_vp, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_int4_repack_mma_bytes": (c_sz, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "dfb_int4_repack_mma": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_int4_gemv_scratch_bytes": (c_sz, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "dfb_int4_gemv": (C.c_int, [C.POINTER(GemvDesc), c_vp]),
    "dfb_int4_gemv_static_max_partials_bytes": (c_sz, []),
    "dfb_int4_gemv_static": (C.c_int, [C.POINTER(GemvDesc), c_vp]),
    "dfb_rms_norm": (C.c_int, [c_vp, c_vp, c_f32, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_add_rms_norm": (C.c_int, [c_vp, c_vp, c_vp, c_f32, C.c_int, C.c_int, c_vp, c_vp, c_vp]),
    "dfb_silu_mul": (C.c_int, [c_vp, c_vp, c_i64, c_vp, c_vp]),
    "dfb_partial_rope": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_causal_conv_step": (C.c_int, [c_vp, c_vp, c_vp, C.c_int, C.c_int, c_vp, c_vp]),
    "dfb_delta_rule_step": (C.c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, C.c_int, C.c_int, C.c_int, C.c_int, c_vp, c_vp, c_vp]),
    "dfb_deltanet_step": (C.c_int, [C.POINTER(DeltaNetDesc), c_vp]),
    "dfb_attn_scratch_bytes": (c_sz, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "dfb_attn_decode": (C.c_int, [C.POINTER(AttnDesc), c_vp]),
    "dfb_attn_prep": (C.c_int, [C.POINTER(AttnPrepDesc), c_vp]),
    "dfb_attn_step": (C.c_int, [C.POINTER(AttnStepDesc), c_vp]),
    "dfb_engine_workspace_bytes": (c_sz, [C.POINTER(ModelDesc)]),
    "dfb_engine_num_segments": (C.c_int, [c_vp]),
    "dfb_engine_step_segment": (C.c_int, [c_vp, C.c_int, c_vp]),
    "dfb_engine_partial_buffer": (c_vp, [c_vp]),
    "dfb_engine_tp_exchange_bytes": (c_sz, [C.c_int, C.c_int, C.c_int]),
    "dfb_engine_create": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(c_vp)]),
    "dfb_engine_destroy": (C.c_int, [c_vp]),
    "dfb_engine_step": (C.c_int, [c_vp, c_vp]),
    "dfb_engine_capture": (C.c_int, [c_vp, c_vp]),
    "dfb_engine_replay": (C.c_int, [c_vp, C.c_int, c_vp]),
    "dfb_engine_decode_host": (C.c_int, [c_vp, c_vp, C.c_int, c_vp, c_vp]),
    "dfb_engine_status": (C.c_int, [c_vp, C.POINTER(C.c_int), c_vp]),
    "dfb_engine_launches_per_step": (C.c_int, [c_vp]),
    "dfb_engine_set_prefetch_distance": (C.c_int, [c_vp, C.c_int]),
    "dfb_engine_set_trace": (C.c_int, [c_vp, c_vp, C.c_int, C.c_int]),
}

_lib: C.CDLL | None = None


class Dfb200Error(RuntimeError):
    """A C entry point returned a non-zero code."""


def library_path() -> Path:
    return _build.LIB


def load() -> C.CDLL:
    """Load the shared library (building it first if the in-tree copy is missing or stale)."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.build()
    except Exception as exc:  # no nvcc, or a compile error: there is nothing to fall back to
        if not _build.LIB.exists():
            raise RuntimeError(
                f"libdfb200.so is not built and cannot be built here ({exc}). This package has no "
                "CPU or PyTorch fallback; run `python -m deltaforge_b200.build` on a machine with nvcc."
            ) from exc
        # An older library is there but the sources changed and the rebuild failed: its struct layouts may no
        # longer match the ctypes declarations above, so loading it is an explicit choice, never a default.
        if not _build.is_current() and os.environ.get("DFB200_ALLOW_STALE_LIBRARY") != "1":
            raise RuntimeError(
                f"libdfb200.so is older than its sources and rebuilding it failed ({exc}); refusing to load it "
                "(set DFB200_ALLOW_STALE_LIBRARY=1 to load the stale library anyway)"
            ) from exc
        path = _build.LIB
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library and the header disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = load().dfb_last_error().decode(errors="replace")
    if rc == 2:
        raise ValueError(f"{what}: {msg}")
    raise Dfb200Error(f"{what} failed (code {rc}): {msg}")
