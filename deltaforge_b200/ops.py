"""``torch.library`` ops backed by the CUDA kernels in ``libdfb200.so``.

Every op of the reference's kernel package that sits on the decode path has a twin here with the same
argument list and the same error behaviour, registered under the ``dfb200::`` namespace:

====================================  ===========================================================
this package                          reference op (file:line of its definition)
====================================  ===========================================================
``dfb200::tiled_gemv_int4``           ``deltaforge::tiled_gemv_int4`` kernels/tiled_gemv.py:915
``dfb200::delta_rule_step``           ``deltaforge::delta_rule_step`` kernels/gated_delta_step.py:109
``dfb200::fused_causal_conv_step``    ``deltaforge::fused_causal_conv_step`` kernels/fused_causal_conv.py:136
``dfb200::gqa_decode_attention``      ``deltaforge::gqa_decode_attention`` kernels/gqa_decode.py:138
``dfb200::split_kv_decode_attention`` ``deltaforge::split_kv_decode_attention`` kernels/flash_decode_splitkv.py:177
``dfb200::add_rms_norm``              ``deltaforge::add_rms_norm`` kernels/fused_rmsnorm_residual.py:164
``dfb200::rms_norm``                  ``deltaforge::rms_norm`` kernels/fused_rmsnorm_residual.py:201
``dfb200::partial_rope``              ``deltaforge::partial_rope`` kernels/fused_rope.py:97
``dfb200::silu_mul``                  ``deltaforge::silu_mul`` kernels/fused_swiglu.py:51
====================================  ===========================================================

plus the fused forms the decode step is built from (``rmsnorm_int4_gemv``, ``int4_gemv_residual``,
``silu_mul_int4_gemv_residual``, ``deltanet_step``, ``attn_prep``, ``attn_decode_gated``) and the two
bit-exactness probes ``int4_unpack`` / ``int4_dequant``.

Conventions kept from the reference: shape and dtype errors are ``ValueError`` and are raised before
the device check, so they surface on any machine; a CPU tensor raises ``RuntimeError`` because there is
no PyTorch fallback (kernels/_triton.py:56-69); outputs are allocated on the input's device; layouts
are coerced with ``.contiguous()``, shapes are not.
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _lib
from ._lib import AttnDesc, AttnPrepDesc, DeltaNetDesc, GemvDesc

MATH_FAST, MATH_EXACT, MATH_FAST_HALF2 = 0, 1, 2
PRO_NONE, PRO_RMSNORM, PRO_SILU_MUL = 0, 1, 2
EPI_STORE, EPI_RESIDUAL, EPI_CONV = 0, 1, 2

BF16 = torch.bfloat16

#: Arithmetic used by the int4 GEMV ops. FAST is the production setting; EXACT rounds each dequantised
#: weight to bf16 like the reference's expression (slower, for cross-checks).
default_math = MATH_FAST


def require_cuda(tensor: Tensor, op: str) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(
            f"dfb200::{op} requires a CUDA tensor and has no PyTorch fallback, on purpose: falling back "
            "would run a different implementation than the one being measured."
        )


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_scratch: dict[tuple, Tensor] = {}


def _zeroed_scratch(device: torch.device, key: tuple, nbytes: int) -> Tensor | None:
    """A per-(device, problem) scratch buffer, zeroed once; the kernels leave their counters at zero."""
    if nbytes == 0:
        return None
    k = (device.index, *key)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _scratch[k] = buf
    return buf


# --------------------------------------------------------------------------------------
# int4 GEMV family
# --------------------------------------------------------------------------------------


def _check_int4(x: Tensor, packed: Tensor, scale: Tensor, group_size: int, op: str) -> tuple[int, int]:
    if packed.dim() != 2 or packed.dtype != torch.uint8:
        raise ValueError(f"{op}: packed must be a 2-D uint8 tensor [K/2, N], got {tuple(packed.shape)} {packed.dtype}")
    half, n = packed.shape
    k = half * 2
    if x.shape[-1] != k:
        raise ValueError(f"{op}: activation has {x.shape[-1]} features, packed weight expects K={k}")
    if group_size <= 0 or half % group_size:
        raise ValueError(f"{op}: group size {group_size} does not divide K/2 = {half}")
    if tuple(scale.shape) != (k // group_size, n):
        raise ValueError(f"{op}: scale must be [K/group, N] = {(k // group_size, n)}, got {tuple(scale.shape)}")
    if scale.dtype not in (torch.float32, BF16):
        raise ValueError(f"{op}: scale must be float32 or bfloat16, got {scale.dtype}")
    if x.dtype != BF16:
        raise ValueError(f"{op}: activations must be bfloat16, got {x.dtype}")
    return k, n


def int4_gemv_fused(
    x: Tensor,
    packed: Tensor,
    scale: Tensor,
    group_size: int,
    *,
    prologue: int = PRO_NONE,
    norm_weight: Tensor | None = None,
    eps: float = 1e-6,
    up: Tensor | None = None,
    epilogue: int = EPI_STORE,
    residual: Tensor | None = None,
    conv_cache: Tensor | None = None,
    conv_weight: Tensor | None = None,
    math: int | None = None,
    force_tiled: bool = False,
    packed_k8: Tensor | None = None,
    packed_mma: Tensor | None = None,
    op: str = "int4_gemv",
) -> Tensor:
    """The general form behind every int4 linear op of this module. Returns ``[..., N]`` bf16.

    ``packed_k8`` is the optional re-packed copy of the weight (``int4_repack_k8``); with it, one
    activation row and the FAST arithmetic the streaming kernel runs instead of the register-tiled one.
    ``packed_mma`` is the optional copy of weight and scales made by ``int4_repack_mma`` (``pair=False``); with
    it, one activation row and the FAST arithmetic run on the integer tensor-core instruction.
    """
    k, n = _check_int4(x, packed, scale, group_size, op)
    if packed_k8 is not None and (packed_k8.dtype != torch.int32 or tuple(packed_k8.shape) != (k // 8, n)):
        raise ValueError(f"{op}: packed_k8 must be int32 [K/8, N] = {(k // 8, n)}, got {tuple(packed_k8.shape)} {packed_k8.dtype}")
    if prologue == PRO_RMSNORM:
        if norm_weight is None or norm_weight.shape != (k,):
            raise ValueError(f"{op}: RMSNorm weight must have {k} elements")
    if prologue == PRO_SILU_MUL and (up is None or up.shape != x.shape):
        raise ValueError(f"{op}: `up` must match the gate activation's shape {tuple(x.shape)}")
    lead = x.shape[:-1]
    rows = 1
    for s in lead:
        rows *= s
    if epilogue == EPI_RESIDUAL and (residual is None or residual.shape != (*lead, n)):
        raise ValueError(f"{op}: residual must have shape {(*lead, n)}")
    conv_dim = 0
    if epilogue == EPI_CONV:
        if conv_cache is None or conv_weight is None or conv_cache.dim() != 3 or conv_cache.shape[2] != 3:
            raise ValueError(f"{op}: conv epilogue needs a (B, C, 3) history and a (C, 4) weight")
        conv_dim = conv_cache.shape[1]
        if conv_cache.shape[0] != rows or conv_dim > n or conv_weight.numel() != conv_dim * 4:
            raise ValueError(f"{op}: conv history {tuple(conv_cache.shape)} does not match rows={rows}, N={n}")
        if not conv_cache.is_contiguous():
            raise ValueError(f"{op}: the conv history is updated in place and must be contiguous")
    require_cuda(x, op)
    flat = x.reshape(rows, k).contiguous()
    packed = packed.contiguous()
    scale = scale.contiguous()
    out = torch.empty((rows, n), device=x.device, dtype=BF16)
    if rows == 0:
        return out.reshape(*lead, n)
    lib = _lib.load()
    nbytes = lib.dfb_int4_gemv_scratch_bytes(rows, k, n, group_size)
    scratch = _zeroed_scratch(x.device, ("gemv", rows, k, n), nbytes)
    d = GemvDesc()
    d.x, d.x_stride, d.rows = flat.data_ptr(), k, rows
    d.packed, d.scale, d.scale_is_bf16 = packed.data_ptr(), scale.data_ptr(), int(scale.dtype == BF16)
    d.K, d.N, d.group = k, n, group_size
    d.prologue, d.eps = prologue, eps
    keep = [flat, packed, scale, out, scratch]
    if prologue == PRO_RMSNORM:
        nw = norm_weight.to(BF16).contiguous()
        keep.append(nw)
        d.norm_w = nw.data_ptr()
    if prologue == PRO_SILU_MUL:
        upc = up.reshape(rows, k).contiguous()
        keep.append(upc)
        d.up, d.up_stride = upc.data_ptr(), k
    d.epilogue, d.out, d.out_stride = epilogue, out.data_ptr(), n
    if epilogue == EPI_RESIDUAL:
        res = residual.reshape(rows, n).contiguous()
        keep.append(res)
        d.residual, d.residual_stride = res.data_ptr(), n
    if epilogue == EPI_CONV:
        cw = conv_weight.reshape(conv_dim, 4).to(BF16).contiguous()
        keep.append(cw)
        d.conv_state, d.conv_w, d.conv_dim = conv_cache.data_ptr(), cw.data_ptr(), conv_dim
    d.scratch, d.scratch_bytes = _ptr(scratch), nbytes
    d.math = default_math if math is None else math
    d.force_tiled = int(force_tiled)
    if packed_k8 is not None:
        packed_k8 = packed_k8.contiguous()
        keep.append(packed_k8)
        d.packed_k8 = packed_k8.data_ptr()
    if packed_mma is not None:
        want = _lib.load().dfb_int4_repack_mma_bytes(k, n, 0, int(scale.dtype == BF16))
        if packed_mma.dtype != torch.uint8 or packed_mma.numel() != want or not packed_mma.is_contiguous():
            raise ValueError(f"{op}: packed_mma must be the {want} contiguous bytes int4_repack_mma(pair=False) returns for this weight")
        keep.append(packed_mma)
        d.packed_mma = packed_mma.data_ptr()
    _lib.check(lib.dfb_int4_gemv(C.byref(d), _stream(x)), f"dfb200::{op}")
    return out.reshape(*lead, n)


@torch.library.custom_op("dfb200::tiled_gemv_int4", mutates_args=())
def tiled_gemv_int4(x: Tensor, packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """Group-wise int4 GEMV. ``packed`` is ``[K // 2, N]``, ``scale`` ``[K // group, N]``."""
    return int4_gemv_fused(x, packed, scale, group_size, op="tiled_gemv_int4")


@tiled_gemv_int4.register_fake
def _(x, packed, scale, group_size):
    return x.new_empty((*x.shape[:-1], packed.shape[1]))


@torch.library.custom_op("dfb200::rmsnorm_int4_gemv", mutates_args=())
def rmsnorm_int4_gemv(x: Tensor, norm_weight: Tensor, eps: float, packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """``tiled_gemv_int4(rms_norm(x, norm_weight, eps), ...)`` in one kernel."""
    return int4_gemv_fused(x, packed, scale, group_size, prologue=PRO_RMSNORM, norm_weight=norm_weight, eps=eps, op="rmsnorm_int4_gemv")


@rmsnorm_int4_gemv.register_fake
def _(x, norm_weight, eps, packed, scale, group_size):
    return x.new_empty((*x.shape[:-1], packed.shape[1]))


@torch.library.custom_op("dfb200::int4_gemv_residual", mutates_args=())
def int4_gemv_residual(x: Tensor, packed: Tensor, scale: Tensor, group_size: int, residual: Tensor) -> Tensor:
    """``residual + tiled_gemv_int4(x, ...)`` in one kernel (the sum is rounded to bf16 once more)."""
    return int4_gemv_fused(x, packed, scale, group_size, epilogue=EPI_RESIDUAL, residual=residual, op="int4_gemv_residual")


@int4_gemv_residual.register_fake
def _(x, packed, scale, group_size, residual):
    return torch.empty_like(residual)


@torch.library.custom_op("dfb200::silu_mul_int4_gemv_residual", mutates_args=())
def silu_mul_int4_gemv_residual(gate: Tensor, up: Tensor, packed: Tensor, scale: Tensor, group_size: int, residual: Tensor) -> Tensor:
    """``residual + tiled_gemv_int4(silu(gate) * up, ...)``: the MLP's down projection in one kernel."""
    return int4_gemv_fused(
        gate, packed, scale, group_size, prologue=PRO_SILU_MUL, up=up, epilogue=EPI_RESIDUAL, residual=residual,
        op="silu_mul_int4_gemv_residual",
    )  # fmt: skip


@silu_mul_int4_gemv_residual.register_fake
def _(gate, up, packed, scale, group_size, residual):
    return torch.empty_like(residual)


@torch.library.custom_op("dfb200::rmsnorm_int4_gemv_conv", mutates_args=("conv_cache",))
def rmsnorm_int4_gemv_conv(
    x: Tensor, norm_weight: Tensor, eps: float, packed: Tensor, scale: Tensor, group_size: int, conv_cache: Tensor, conv_weight: Tensor
) -> Tensor:
    """DeltaNet input projections: RMSNorm, GEMV over qkv|z|b|a, conv step + SiLU on the first C columns."""
    return int4_gemv_fused(
        x, packed, scale, group_size, prologue=PRO_RMSNORM, norm_weight=norm_weight, eps=eps, epilogue=EPI_CONV,
        conv_cache=conv_cache, conv_weight=conv_weight, op="rmsnorm_int4_gemv_conv",
    )  # fmt: skip


@rmsnorm_int4_gemv_conv.register_fake
def _(x, norm_weight, eps, packed, scale, group_size, conv_cache, conv_weight):
    return x.new_empty((*x.shape[:-1], packed.shape[1]))


@torch.library.custom_op("dfb200::int4_repack_k8", mutates_args=())
def int4_repack_k8(packed: Tensor) -> Tensor:
    """``packed [K/2, N]`` uint8 -> int32 ``[K/8, N]``: word ``(kb, n)`` holds the eight nibbles of column
    ``n`` for rows ``8kb .. 8kb+7`` (nibble ``i`` = row ``8kb + i``). The layout the streaming GEMV reads."""
    if packed.dim() != 2 or packed.dtype != torch.uint8 or (packed.shape[0] * 2) % 8:
        raise ValueError(f"int4_repack_k8: expected uint8 [K/2, N] with K a multiple of 8, got {tuple(packed.shape)} {packed.dtype}")
    require_cuda(packed, "int4_repack_k8")
    packed = packed.contiguous()
    half, n = packed.shape
    out = torch.empty((half // 4, n), dtype=torch.int32, device=packed.device)
    if out.numel():
        _lib.check(_lib.load().dfb_int4_repack_k8(packed.data_ptr(), 2 * half, n, out.data_ptr(), _stream(packed)), "dfb200::int4_repack_k8")
    return out


@int4_repack_k8.register_fake
def _(packed):
    return packed.new_empty((packed.shape[0] // 4, packed.shape[1]), dtype=torch.int32)


def int4_repack_mma(packed: Tensor, scale: Tensor, *, pair: bool = False) -> Tensor:
    """``packed [K/2, N]`` uint8 and ``scale [K/128, N]`` (fp32 or bf16) -> the bytes the integer tensor-core GEMV
    streams (``dfb_int4_repack_mma``): one contiguous unit per (column tile, 128-row group) with the group's words in
    operand-fragment order followed by its scales. ``pair=True`` lays a ``gate_proj|up_proj`` matrix out with each
    tile holding 128 gate columns and the matching up columns. K must be a multiple of 128."""
    if packed.dim() != 2 or packed.dtype != torch.uint8:
        raise ValueError(f"int4_repack_mma: expected uint8 [K/2, N], got {tuple(packed.shape)} {packed.dtype}")
    half, n = packed.shape
    k = 2 * half
    if k % 128 or scale.shape != (k // 128, n) or scale.dtype not in (torch.float32, BF16):
        raise ValueError(f"int4_repack_mma: K = {k} must be a multiple of 128 with scales [K/128, N] in fp32 or bf16, got {tuple(scale.shape)} {scale.dtype}")
    if pair and n % 2:
        raise ValueError("int4_repack_mma: a gate|up pair has an even number of columns")
    require_cuda(packed, "int4_repack_mma")
    packed, scale = packed.contiguous(), scale.contiguous()
    lib = _lib.load()
    is_bf16 = int(scale.dtype == BF16)
    out = torch.empty(lib.dfb_int4_repack_mma_bytes(k, n, int(pair), is_bf16), dtype=torch.uint8, device=packed.device)
    _lib.check(lib.dfb_int4_repack_mma(packed.data_ptr(), scale.data_ptr(), is_bf16, k, n, int(pair), out.data_ptr(), _stream(packed)),
               "dfb200::int4_repack_mma")  # fmt: skip
    return out


@torch.library.custom_op("dfb200::int4_unpack", mutates_args=())
def int4_unpack(packed: Tensor) -> Tensor:
    """``packed [K/2, N]`` -> signed int8 values ``[K, N]`` (low nibbles are rows 0..K/2)."""
    if packed.dim() != 2 or packed.dtype != torch.uint8:
        raise ValueError(f"int4_unpack: expected a 2-D uint8 tensor, got {tuple(packed.shape)} {packed.dtype}")
    require_cuda(packed, "int4_unpack")
    packed = packed.contiguous()
    half, n = packed.shape
    out = torch.empty((2 * half, n), dtype=torch.int8, device=packed.device)
    if out.numel():
        _lib.check(_lib.load().dfb_int4_unpack(packed.data_ptr(), 2 * half, n, out.data_ptr(), _stream(packed)), "dfb200::int4_unpack")
    return out


@int4_unpack.register_fake
def _(packed):
    return packed.new_empty((packed.shape[0] * 2, packed.shape[1]), dtype=torch.int8)


@torch.library.custom_op("dfb200::int4_dequant", mutates_args=())
def int4_dequant(packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """bf16 weight ``[K, N]`` = bf16(value * scale): the tensor the reference's expression multiplies by."""
    if packed.dim() != 2 or packed.dtype != torch.uint8:
        raise ValueError(f"int4_dequant: expected a 2-D uint8 tensor, got {tuple(packed.shape)} {packed.dtype}")
    half, n = packed.shape
    if group_size <= 0 or half % group_size or tuple(scale.shape) != (2 * half // group_size, n):
        raise ValueError(f"int4_dequant: scale {tuple(scale.shape)} does not match K={2 * half}, N={n}, group={group_size}")
    if scale.dtype not in (torch.float32, BF16):
        raise ValueError(f"int4_dequant: scale must be float32 or bfloat16, got {scale.dtype}")
    require_cuda(packed, "int4_dequant")
    packed, scale = packed.contiguous(), scale.contiguous()
    out = torch.empty((2 * half, n), dtype=BF16, device=packed.device)
    if out.numel():
        rc = _lib.load().dfb_int4_dequant(
            packed.data_ptr(), scale.data_ptr(), int(scale.dtype == BF16), 2 * half, n, group_size, out.data_ptr(), _stream(packed)
        )
        _lib.check(rc, "dfb200::int4_dequant")
    return out


@int4_dequant.register_fake
def _(packed, scale, group_size):
    return packed.new_empty((packed.shape[0] * 2, packed.shape[1]), dtype=BF16)


# --------------------------------------------------------------------------------------
# Norms and elementwise
# --------------------------------------------------------------------------------------


def _check_norm(x: Tensor, weight: Tensor, name: str, residual: Tensor | None = None) -> None:
    if weight.dim() != 1 or not weight.is_contiguous():
        raise ValueError("norm weight must be a contiguous 1-D tensor; the kernel indexes it by column")
    if x.shape[-1] != weight.shape[0]:
        raise ValueError(f"weight has {weight.shape[0]} elements, activation row is {x.shape[-1]}")
    if residual is not None:
        if residual.shape != x.shape:
            raise ValueError(f"residual shape {tuple(residual.shape)} != activation shape {tuple(x.shape)}")
        if residual.dtype != x.dtype:
            raise ValueError(f"residual dtype {residual.dtype} != activation dtype {x.dtype}")
    if x.dtype != BF16:
        raise ValueError(f"{name}: activations must be bfloat16, got {x.dtype}")
    require_cuda(x, name)


@torch.library.custom_op("dfb200::rms_norm", mutates_args=())
def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """RMSNorm with the ``1 + weight`` scale."""
    _check_norm(x, weight, "rms_norm")
    x = x.contiguous()
    w = weight.to(BF16)
    n = x.shape[-1]
    out = torch.empty_like(x)
    if x.numel():
        _lib.check(_lib.load().dfb_rms_norm(x.data_ptr(), w.data_ptr(), eps, x.numel() // n, n, out.data_ptr(), _stream(x)), "dfb200::rms_norm")
    return out


@rms_norm.register_fake
def _(x, weight, eps):
    return torch.empty_like(x)


@torch.library.custom_op("dfb200::add_rms_norm", mutates_args=())
def add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """``(residual + x, rms_norm(residual + x))`` in one pass."""
    _check_norm(x, weight, "add_rms_norm", residual=residual)
    x, residual = x.contiguous(), residual.contiguous()
    w = weight.to(BF16)
    n = x.shape[-1]
    resid_out, out = torch.empty_like(x), torch.empty_like(x)
    if x.numel():
        rc = _lib.load().dfb_add_rms_norm(
            x.data_ptr(), residual.data_ptr(), w.data_ptr(), eps, x.numel() // n, n, resid_out.data_ptr(), out.data_ptr(), _stream(x)
        )
        _lib.check(rc, "dfb200::add_rms_norm")
    return resid_out, out


@add_rms_norm.register_fake
def _(x, residual, weight, eps):
    return torch.empty_like(x), torch.empty_like(x)


@torch.library.custom_op("dfb200::silu_mul", mutates_args=())
def silu_mul(gate: Tensor, up: Tensor) -> Tensor:
    """``F.silu(gate) * up`` in one pass."""
    if gate.shape != up.shape:
        raise ValueError(f"gate shape {tuple(gate.shape)} != up shape {tuple(up.shape)}")
    if gate.dtype != up.dtype:
        raise ValueError(f"gate dtype {gate.dtype} != up dtype {up.dtype}")
    if gate.dtype != BF16:
        raise ValueError(f"silu_mul: activations must be bfloat16, got {gate.dtype}")
    require_cuda(gate, "silu_mul")
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(up)
    if out.numel():
        _lib.check(_lib.load().dfb_silu_mul(gate.data_ptr(), up.data_ptr(), out.numel(), out.data_ptr(), _stream(gate)), "dfb200::silu_mul")
    return out


@silu_mul.register_fake
def _(gate, up):
    return torch.empty_like(up)


@torch.library.custom_op("dfb200::partial_rope", mutates_args=())
def partial_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotate the leading ``rotary_dim`` dims of ``x (batch, heads, seq, head_dim)``."""
    if x.dim() != 4:
        raise ValueError(f"expected (batch, heads, seq, head_dim), got {tuple(x.shape)}")
    if cos.shape != sin.shape:
        raise ValueError(f"cos shape {tuple(cos.shape)} != sin shape {tuple(sin.shape)}")
    if cos.dim() != 3:
        raise ValueError(f"expected cos as (batch, seq, rotary_dim), got {tuple(cos.shape)}")
    batch, heads, seq_len, head_dim = x.shape
    rotary_dim = cos.shape[-1]
    if cos.shape[0] != batch or cos.shape[1] != seq_len:
        raise ValueError(f"cos {tuple(cos.shape)} does not match x {tuple(x.shape)} on batch/seq")
    if rotary_dim > head_dim:
        raise ValueError(f"rotary_dim {rotary_dim} exceeds head_dim {head_dim}")
    if rotary_dim % 2:
        raise ValueError(f"rotary_dim must be even to rotate in halves, got {rotary_dim}")
    if x.dtype != BF16:
        raise ValueError(f"partial_rope: activations must be bfloat16, got {x.dtype}")
    require_cuda(x, "partial_rope")
    x = x.contiguous()
    cos, sin = cos.to(BF16).contiguous(), sin.to(BF16).contiguous()
    out = torch.empty_like(x)
    if out.numel():
        rc = _lib.load().dfb_partial_rope(
            x.data_ptr(), cos.data_ptr(), sin.data_ptr(), batch, heads, seq_len, head_dim, rotary_dim, out.data_ptr(), _stream(x)
        )
        _lib.check(rc, "dfb200::partial_rope")
    return out


@partial_rope.register_fake
def _(x, cos, sin):
    return torch.empty_like(x)


@torch.library.custom_op("dfb200::fused_causal_conv_step", mutates_args=("conv_cache",))
def fused_causal_conv_step(x: Tensor, conv_cache: Tensor, weight: Tensor) -> Tensor:
    """``x (B, C, 1)``, ``conv_cache (B, C, 3)`` advanced in place, ``weight (C, 1, 4)`` -> ``(B, C, 1)``."""
    batch, channels, steps = x.shape
    if steps != 1:
        raise ValueError(f"fused_causal_conv_step is the decode step; got seq_len {steps}")
    if conv_cache.shape != (batch, channels, 3):
        raise ValueError(f"expected a (B, C, 3) history, got {tuple(conv_cache.shape)}")
    w = weight.reshape(channels, -1)
    if w.shape[1] != 4:
        raise ValueError(f"this kernel is the four-tap case; got {w.shape[1]} taps")
    if x.dtype != BF16 or conv_cache.dtype != BF16:
        raise ValueError("fused_causal_conv_step: activations and history must be bfloat16")
    if not conv_cache.is_contiguous():
        raise ValueError("the conv history is updated in place and must be contiguous")
    require_cuda(x, "fused_causal_conv_step")
    xc = x.contiguous()
    w = w.to(BF16).contiguous()
    out = torch.empty_like(xc)
    if out.numel():
        rc = _lib.load().dfb_causal_conv_step(xc.data_ptr(), conv_cache.data_ptr(), w.data_ptr(), batch, channels, out.data_ptr(), _stream(x))
        _lib.check(rc, "dfb200::fused_causal_conv_step")
    return out


@fused_causal_conv_step.register_fake
def _(x, conv_cache, weight):
    return torch.empty_like(x)


# --------------------------------------------------------------------------------------
# Gated DeltaNet
# --------------------------------------------------------------------------------------


@torch.library.custom_op("dfb200::delta_rule_step", mutates_args=())
def delta_rule_step(state: Tensor, query: Tensor, key: Tensor, value: Tensor, g: Tensor, beta: Tensor) -> tuple[Tensor, Tensor]:
    """One delta-rule step on pre-normalised q, k. Returns ``(output fp32, new_state)``."""
    if state.dim() != 4:
        raise ValueError(f"expected state (batch, heads, key_dim, value_dim), got {tuple(state.shape)}")
    batch, heads, key_dim, value_dim = state.shape
    for name, t, shape in (
        ("query", query, (batch, heads, key_dim)),
        ("key", key, (batch, heads, key_dim)),
        ("value", value, (batch, heads, value_dim)),
        ("g", g, (batch, heads)),
        ("beta", beta, (batch, heads)),
    ):
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
    if state.dtype != torch.float32:
        raise ValueError(
            f"the recurrent state is fp32 by config (mamba_ssm_dtype), got {state.dtype}. "
            "Running it in bf16 would change the model, not just the kernel."
        )
    require_cuda(state, "delta_rule_step")
    state = state.contiguous()
    q, k, v, gg, bb = (t.float().contiguous() for t in (query, key, value, g, beta))
    out = torch.empty((batch, heads, value_dim), device=state.device, dtype=torch.float32)
    state_out = torch.empty_like(state)
    if state.numel():
        rc = _lib.load().dfb_delta_rule_step(
            state.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), gg.data_ptr(), bb.data_ptr(),
            batch, heads, key_dim, value_dim, out.data_ptr(), state_out.data_ptr(), _stream(state),
        )  # fmt: skip
        _lib.check(rc, "dfb200::delta_rule_step")
    return out, state_out


@delta_rule_step.register_fake
def _(state, query, key, value, g, beta):
    b, h, _, dv = state.shape
    return torch.empty((b, h, dv), device=state.device, dtype=torch.float32), torch.empty_like(state)


@torch.library.custom_op("dfb200::deltanet_step", mutates_args=("state",))
def deltanet_step(
    q: Tensor, k: Tensor, v: Tensor, z: Tensor, b: Tensor, a: Tensor, a_log: Tensor, dt_bias: Tensor, norm_weight: Tensor,
    eps: float, state: Tensor,
) -> Tensor:  # fmt: skip
    """DeltaNet core for one token: ``q,k (B,Hk,dk)``, ``v,z (B,Hv,dv)``, ``b,a (B,Hv)`` post-conv bf16;
    ``state (B,Hv,dk,dv)`` fp32 updated in place. Returns the gated-normed output ``(B, Hv*dv)`` bf16."""
    if state.dim() != 4 or state.dtype != torch.float32:
        raise ValueError(f"state must be fp32 (batch, heads, key_dim, value_dim), got {tuple(state.shape)} {state.dtype}")
    batch, hv, dk, dv = state.shape
    if q.dim() != 3 or q.shape != k.shape or q.shape[0] != batch or q.shape[2] != dk:
        raise ValueError(f"q/k must be (batch, key_heads, {dk}), got {tuple(q.shape)} and {tuple(k.shape)}")
    hk = q.shape[1]
    if hk == 0 or hv % hk:
        raise ValueError(f"{hv} value heads do not divide into {hk} key heads")
    for name, t, shape in (("v", v, (batch, hv, dv)), ("z", z, (batch, hv, dv)), ("b", b, (batch, hv)), ("a", a, (batch, hv))):
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
    if a_log.shape != (hv,) or dt_bias.shape != (hv,) or norm_weight.shape != (dv,):
        raise ValueError("A_log and dt_bias must have one entry per value head, the norm weight one per value dim")
    if not state.is_contiguous():
        raise ValueError("the recurrent state is updated in place and must be contiguous")
    require_cuda(state, "deltanet_step")
    # one row per sequence: [q | k | v | z | b | a]
    row = torch.cat([t.reshape(batch, -1).to(BF16) for t in (q, k, v, z, b, a)], dim=1).contiguous()
    kd, vd = hk * dk, hv * dv
    out = torch.empty((batch, vd), device=state.device, dtype=BF16)
    al, dtb, nw = a_log.float().contiguous(), dt_bias.float().contiguous(), norm_weight.float().contiguous()
    d = DeltaNetDesc()
    d.batch, d.num_k_heads, d.num_v_heads, d.dk, d.dv = batch, hk, hv, dk, dv
    es = row.element_size()
    base = row.data_ptr()
    d.q, d.k, d.v = base, base + kd * es, base + 2 * kd * es
    d.z, d.b, d.a = base + (2 * kd + vd) * es, base + (2 * kd + 2 * vd) * es, base + (2 * kd + 2 * vd + hv) * es
    d.row_stride = row.shape[1]
    d.a_log, d.dt_bias, d.norm_w = al.data_ptr(), dtb.data_ptr(), nw.data_ptr()
    d.norm_w_is_bf16 = int(norm_weight.dtype == BF16)
    d.eps = eps
    d.state, d.out, d.out_stride = state.data_ptr(), out.data_ptr(), vd
    if batch:
        _lib.check(_lib.load().dfb_deltanet_step(C.byref(d), _stream(state)), "dfb200::deltanet_step")
    return out


@deltanet_step.register_fake
def _(q, k, v, z, b, a, a_log, dt_bias, norm_weight, eps, state):
    return state.new_empty((state.shape[0], state.shape[1] * state.shape[3]), dtype=BF16)


# --------------------------------------------------------------------------------------
# Decode attention
# --------------------------------------------------------------------------------------


def _check_attn(query: Tensor, key: Tensor, value: Tensor) -> tuple[int, int, int, int, int]:
    if query.dim() != 3:
        raise ValueError(f"expected query (batch, heads_q, head_dim), got {tuple(query.shape)}")
    if key.dim() != 4 or value.dim() != 4:
        raise ValueError(f"expected key/value (batch, heads_kv, key_len, head_dim), got {tuple(key.shape)} and {tuple(value.shape)}")
    if key.shape != value.shape:
        raise ValueError(f"key {tuple(key.shape)} and value {tuple(value.shape)} must match")
    batch, heads_q, head_dim = query.shape
    kv_batch, heads_kv, key_len, kv_dim = key.shape
    if kv_batch != batch or kv_dim != head_dim:
        raise ValueError(f"key {tuple(key.shape)} does not match query {tuple(query.shape)}")
    if heads_kv == 0 or heads_q % heads_kv:
        raise ValueError(f"{heads_q} query heads do not divide into {heads_kv} KV heads")
    if key_len < 1:
        raise ValueError("cannot attend over an empty KV cache")
    for name, t in (("query", query), ("key", key), ("value", value)):
        if t.stride(-1) != 1:
            raise ValueError(f"{name} must have the head dimension innermost and contiguous")
        if t.dtype != BF16:
            raise ValueError(f"{name} must be bfloat16, got {t.dtype}")
    return batch, heads_q, heads_kv, key_len, head_dim


def _attention(query: Tensor, key: Tensor, value: Tensor, scale: float, splits: int, gate: Tensor | None, swish: bool, op: str) -> Tensor:
    batch, hq, hkv, key_len, d = _check_attn(query, key, value)
    if gate is not None and gate.shape != query.shape:
        raise ValueError(f"gate shape {tuple(gate.shape)} != query shape {tuple(query.shape)}")
    require_cuda(query, op)
    query = query.contiguous()
    # Key and value may be views of a longer cache: rows stay where they are as long as a head's rows
    # are `head_dim` apart; anything else is copied.
    def rows_dense(t: Tensor) -> bool:
        return t.stride(2) == d and t.stride(3) == 1

    if not (rows_dense(key) and rows_dense(value) and key.stride() == value.stride()):
        key, value = key.contiguous(), value.contiguous()
    out = torch.empty((batch, hq * d), device=query.device, dtype=BF16)
    lib = _lib.load()
    nbytes = lib.dfb_attn_scratch_bytes(batch, hq, hkv, d, splits)
    scratch = _zeroed_scratch(query.device, ("attn", batch, hq, hkv, d, splits), nbytes)
    a = AttnDesc()
    a.batch, a.hq, a.hkv, a.d = batch, hq, hkv, d
    a.q, a.q_stride, a.qh_stride = query.data_ptr(), hq * d, d
    a.kcache, a.vcache = key.data_ptr(), value.data_ptr()
    a.kv_batch_stride, a.kv_head_stride = key.stride(0), key.stride(1)
    a.key_len, a.pos, a.scale, a.splits = key_len, None, scale, splits
    a.scratch, a.scratch_bytes = _ptr(scratch), nbytes
    if gate is not None:
        gate = gate.to(BF16).contiguous()
        a.gate, a.gate_stride, a.gateh_stride, a.gate_is_swish = gate.data_ptr(), hq * d, d, int(swish)
    a.out, a.out_stride = out.data_ptr(), hq * d
    _lib.check(lib.dfb_attn_decode(C.byref(a), _stream(query)), f"dfb200::{op}")
    return out.reshape(batch, hq, d)


@torch.library.custom_op("dfb200::gqa_decode_attention", mutates_args=())
def gqa_decode_attention(query: Tensor, key: Tensor, value: Tensor, scale: float) -> Tensor:
    """Single-token GQA attention against an unexpanded KV cache, one pass over the keys."""
    return _attention(query, key, value, scale, 1, None, False, "gqa_decode_attention")


@gqa_decode_attention.register_fake
def _(query, key, value, scale):
    return torch.empty_like(query)


@torch.library.custom_op("dfb200::split_kv_decode_attention", mutates_args=())
def split_kv_decode_attention(query: Tensor, key: Tensor, value: Tensor, scale: float, splits: int) -> Tensor:
    """Same result with the key scan cut into ``splits`` slices merged by log-sum-exp."""
    if splits < 1 or splits & (splits - 1):
        raise ValueError(f"splits must be a power of two so the merge can index it, got {splits}")
    if splits > 128:
        raise ValueError(f"at most 128 splits are supported, got {splits}")
    return _attention(query, key, value, scale, splits, None, False, "split_kv_decode_attention")


@split_kv_decode_attention.register_fake
def _(query, key, value, scale, splits):
    return torch.empty_like(query)


@torch.library.custom_op("dfb200::attn_decode_gated", mutates_args=())
def attn_decode_gated(query: Tensor, key: Tensor, value: Tensor, scale: float, splits: int, gate: Tensor, swish: bool) -> Tensor:
    """Split-KV decode attention times the output gate (sigmoid, or SiLU when ``swish``)."""
    if splits < 1 or splits > 128:
        raise ValueError(f"splits must be in 1..128, got {splits}")
    return _attention(query, key, value, scale, splits, gate, swish, "attn_decode_gated")


@attn_decode_gated.register_fake
def _(query, key, value, scale, splits, gate, swish):
    return torch.empty_like(query)


@torch.library.custom_op("dfb200::attn_prep", mutates_args=("key_cache", "value_cache"))
def attn_prep(
    proj: Tensor, q_norm_weight: Tensor, k_norm_weight: Tensor, eps: float, inv_freq: Tensor, pos: Tensor,
    key_cache: Tensor, value_cache: Tensor, num_heads: int, output_gate: bool,
) -> Tensor:  # fmt: skip
    """q/k RMSNorm, partial RoPE at device position ``pos`` and the KV-cache write, from the fused
    ``q(|gate)|k|v`` projection row ``proj (B, width)``. Returns the rotated query ``(B, Hq, D)``."""
    if key_cache.dim() != 4 or key_cache.shape != value_cache.shape:
        raise ValueError(f"caches must both be (batch, kv_heads, max_seq, head_dim), got {tuple(key_cache.shape)}")
    batch, hkv, max_seq, d = key_cache.shape
    width = num_heads * d * (2 if output_gate else 1) + 2 * hkv * d
    if proj.shape != (batch, width):
        raise ValueError(f"proj must be {(batch, width)}, got {tuple(proj.shape)}")
    if q_norm_weight.shape != (d,) or k_norm_weight.shape != (d,):
        raise ValueError(f"q/k norm weights must have {d} elements")
    rd = 2 * inv_freq.numel()
    if rd > d:
        raise ValueError(f"rotary_dim {rd} exceeds head_dim {d}")
    if pos.dtype != torch.int32 or pos.numel() != 1:
        raise ValueError("pos must be a single int32 on the device")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("the KV caches are written in place and must be contiguous")
    require_cuda(proj, "attn_prep")
    proj = proj.contiguous()
    qw, kw = q_norm_weight.to(BF16).contiguous(), k_norm_weight.to(BF16).contiguous()
    inv = inv_freq.float().contiguous()
    q_out = torch.empty((batch, num_heads, d), device=proj.device, dtype=BF16)
    p = AttnPrepDesc()
    p.batch, p.hq, p.hkv, p.d, p.rotary_dim = batch, num_heads, hkv, d, rd
    p.proj, p.proj_stride = proj.data_ptr(), width
    p.q_norm_w, p.k_norm_w, p.eps = qw.data_ptr(), kw.data_ptr(), eps
    p.inv_freq, p.pos, p.q_out = inv.data_ptr(), pos.data_ptr(), q_out.data_ptr()
    p.kcache, p.vcache = key_cache.data_ptr(), value_cache.data_ptr()
    p.kv_batch_stride, p.kv_head_stride = hkv * max_seq * d, max_seq * d
    p.attn_output_gate, p.max_seq = int(output_gate), max_seq
    _lib.check(_lib.load().dfb_attn_prep(C.byref(p), _stream(proj)), "dfb200::attn_prep")
    return q_out


@attn_prep.register_fake
def _(proj, q_norm_weight, k_norm_weight, eps, inv_freq, pos, key_cache, value_cache, num_heads, output_gate):
    return proj.new_empty((proj.shape[0], num_heads, key_cache.shape[3]))


@torch.library.custom_op("dfb200::attn_step", mutates_args=("key_cache", "value_cache"))
def attn_step(
    proj: Tensor, q_norm_weight: Tensor, k_norm_weight: Tensor, eps: float, inv_freq: Tensor, pos: Tensor,
    key_cache: Tensor, value_cache: Tensor, num_heads: int, output_gate: bool, swish: bool, splits: int, cluster_size: int,
) -> Tensor:  # fmt: skip
    """``attn_prep`` + gated split-KV decode attention in one launch, for one new token per sequence.

    ``proj (B, width)`` is the fused ``q(|gate)|k|v`` projection row, ``pos`` the device-side number of
    cached tokens (the new token becomes row ``pos`` of the caches). Returns ``(B, Hq * D)`` bf16.
    ``splits`` is a power of two with ``ceil(max_seq / splits) <= 160``; ``cluster_size`` 0 picks min(splits, 4).
    """
    if key_cache.dim() != 4 or key_cache.shape != value_cache.shape:
        raise ValueError(f"caches must both be (batch, kv_heads, max_seq, head_dim), got {tuple(key_cache.shape)}")
    batch, hkv, max_seq, d = key_cache.shape
    width = num_heads * d * (2 if output_gate else 1) + 2 * hkv * d
    if proj.shape != (batch, width):
        raise ValueError(f"proj must be {(batch, width)}, got {tuple(proj.shape)}")
    if q_norm_weight.shape != (d,) or k_norm_weight.shape != (d,):
        raise ValueError(f"q/k norm weights must have {d} elements")
    if splits < 1 or splits & (splits - 1):
        raise ValueError(f"splits must be a power of two, got {splits}")
    if -(-max_seq // splits) > 160:
        raise ValueError(f"{splits} slices of a {max_seq}-row cache exceed 160 keys per slice")
    if pos.dtype != torch.int32 or pos.numel() != 1:
        raise ValueError("pos must be a single int32 on the device")
    if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
        raise ValueError("the KV caches are written in place and must be contiguous")
    if proj.dtype != BF16 or key_cache.dtype != BF16:
        raise ValueError("attn_step: activations and caches must be bfloat16")
    require_cuda(proj, "attn_step")
    proj = proj.contiguous()
    qw, kw = q_norm_weight.to(BF16).contiguous(), k_norm_weight.to(BF16).contiguous()
    inv = inv_freq.float().contiguous()
    out = torch.empty((batch, num_heads * d), device=proj.device, dtype=BF16)
    lib = _lib.load()
    nbytes = lib.dfb_attn_scratch_bytes(batch, num_heads, hkv, d, splits)
    scratch = _zeroed_scratch(proj.device, ("attn", batch, num_heads, hkv, d, splits), nbytes)
    a = _lib.AttnStepDesc()
    a.batch, a.hq, a.hkv, a.d, a.rotary_dim = batch, num_heads, hkv, d, 2 * inv.numel()
    a.proj, a.proj_stride = proj.data_ptr(), width
    a.q_norm_w, a.k_norm_w, a.eps = qw.data_ptr(), kw.data_ptr(), eps
    a.inv_freq, a.pos = inv.data_ptr(), pos.data_ptr()
    a.kcache, a.vcache = key_cache.data_ptr(), value_cache.data_ptr()
    a.kv_batch_stride, a.kv_head_stride, a.max_seq = hkv * max_seq * d, max_seq * d, max_seq
    a.attn_output_gate, a.gate_is_swish, a.scale = int(output_gate), int(swish), d**-0.5
    a.splits, a.cluster_size = splits, cluster_size
    a.scratch, a.scratch_bytes = _ptr(scratch), nbytes
    a.out, a.out_stride, a.status = out.data_ptr(), num_heads * d, None
    _lib.check(lib.dfb_attn_step(C.byref(a), _stream(proj)), "dfb200::attn_step")
    return out


@attn_step.register_fake
def _(proj, q_norm_weight, k_norm_weight, eps, inv_freq, pos, key_cache, value_cache, num_heads, output_gate, swish, splits, cluster_size):
    return proj.new_empty((proj.shape[0], num_heads * key_cache.shape[3]))
