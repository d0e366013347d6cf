"""Install-time int4 quantiser in the reference's K-major format.

Same function as ``quantise_int4_k_major`` of the reference (src/deltaforge/kernels/tiled_gemv.py:
242-278, group rule src/deltaforge/kernels/quantised_linear.py:193-207): symmetric per-group scale
``amax / 7`` (1 for an all-zero group), values clamped to [-7, 7] and stored offset by 8, byte
``[j, n]`` = row ``j`` in the low nibble and row ``j + K/2`` in the high nibble, ``packed`` is
``[K/2, N]`` and ``scale`` ``[K/group, N]`` fp32. Weights on a CUDA device are quantised by the library's
kernel (``dfb_int4_quantise_k_major``); this is set-up work, not the decode path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

INT4_MAX = 7
_CHUNK_ELEMENTS = 1 << 24


@dataclass
class QuantisedWeight:
    qweight: Tensor  # [K/2, N] uint8
    scale: Tensor  # [K/group, N]
    bits: int
    group_size: int
    k8: Tensor | None = None  # [K/8, N] int32: the same nibbles re-packed for the streaming GEMV (made on demand)
    mma: Tensor | None = None  # bytes: weight and scales re-packed for the integer tensor-core GEMV (made on demand)
    mma_pair: bool = False  # `mma` pairs gate_proj and up_proj columns (the gate|up projection of a decode engine)

    @property
    def in_features(self) -> int:
        return self.qweight.shape[0] * 2

    @property
    def out_features(self) -> int:
        return self.qweight.shape[1]


def group_size_for(in_features: int) -> int:
    """Group width along K: 128 when both halves of K are whole 128-row groups, else one group per half (which must
    be a power of two). The format's rule, src/deltaforge/kernels/quantised_linear.py:193-207."""
    if in_features % 2:
        raise ValueError(f"int4 packing needs an even K, got {in_features}")
    if in_features % 256 == 0:
        return 128
    group = in_features // 2
    if group & (group - 1):
        raise ValueError(f"int4 group size {group} for K={in_features} is not a power of two")
    return group


def _quantise_on_host(w: Tensor, group: int) -> tuple[Tensor, Tensor]:
    """The format's arithmetic in torch, K-major from the start, a block of columns at a time (set-up work on
    whatever device holds the weight; the CUDA kernel behind ``quantise_int4_k_major`` gives the same bits)."""
    n, k = w.shape
    packed = torch.empty((k // 2, n), dtype=torch.uint8, device=w.device)
    scale = torch.empty((k // group, n), dtype=torch.float32, device=w.device)
    cols = max(1, _CHUNK_ELEMENTS // k)
    for c0 in range(0, n, cols):
        wt = w[c0 : c0 + cols].float().t().reshape(k // group, group, -1)  # [groups, rows of a group, columns]
        step = wt.abs().amax(dim=1) / INT4_MAX
        step = torch.where(step > 0, step, torch.ones_like(step))
        nib = (torch.round(wt / step.unsqueeze(1)).clamp_(-INT4_MAX, INT4_MAX) + 8).to(torch.uint8).reshape(k, -1)
        packed[:, c0 : c0 + cols] = nib[: k // 2] | (nib[k // 2 :] << 4)  # row j low nibble, row j + K/2 high nibble
        scale[:, c0 : c0 + cols] = step
    return packed, scale


@torch.no_grad()
def quantise_int4_k_major(weight: Tensor) -> QuantisedWeight:
    """``weight [N, K]`` (any float dtype) -> packed K-major int4 with fp32 group scales.

    A CUDA weight in bf16 or fp32 goes through ``dfb_int4_quantise_k_major`` (one pass over the weight); anything
    else through the torch form of the same arithmetic. Both are bit-identical to the reference's packer."""
    w = weight.detach()
    if w.dim() != 2:
        raise ValueError(f"expected a 2-D weight [N, K], got {tuple(w.shape)}")
    n, k = w.shape
    group = group_size_for(k)
    if w.is_cuda and w.dtype in (torch.bfloat16, torch.float32):
        from . import _lib

        w = w.contiguous()
        packed = torch.empty((k // 2, n), dtype=torch.uint8, device=w.device)
        scale = torch.empty((k // group, n), dtype=torch.float32, device=w.device)
        stream = torch.cuda.current_stream(w.device).cuda_stream
        with torch.cuda.device(w.device):
            rc = _lib.load().dfb_int4_quantise_k_major(w.data_ptr(), int(w.dtype == torch.bfloat16), n, k, packed.data_ptr(), scale.data_ptr(), stream)
        _lib.check(rc, "dfb_int4_quantise_k_major")
    else:
        packed, scale = _quantise_on_host(w, group)
    return QuantisedWeight(qweight=packed, scale=scale, bits=4, group_size=group)


def concat_along_n(parts: list[QuantisedWeight]) -> QuantisedWeight:
    """Stack projections that share an input (same K and group) into one weight with N = sum of Ns."""
    k = {p.in_features for p in parts}
    g = {p.group_size for p in parts}
    if len(k) != 1 or len(g) != 1:
        raise ValueError("projections fused along N must share K and group size")
    return QuantisedWeight(
        qweight=torch.cat([p.qweight for p in parts], dim=1).contiguous(),
        scale=torch.cat([p.scale for p in parts], dim=1).contiguous(),
        bits=4,
        group_size=parts[0].group_size,
    )
