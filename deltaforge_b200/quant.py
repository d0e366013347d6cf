"""Install-time int4 quantiser in the reference's K-major format.

Same function as ``quantise_int4_k_major`` of the reference (src/deltaforge/kernels/tiled_gemv.py:
242-278, group rule src/deltaforge/kernels/quantised_linear.py:193-207): symmetric per-group scale
``amax / 7`` (1 for an all-zero group), values clamped to [-7, 7] and stored offset by 8, byte
``[j, n]`` = row ``j`` in the low nibble and row ``j + K/2`` in the high nibble, ``packed`` is
``[K/2, N]`` and ``scale`` ``[K/group, N]`` fp32. It runs in torch on whatever device holds the
weight; this is set-up work, not the decode path.
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

    @property
    def in_features(self) -> int:
        return self.qweight.shape[0] * 2

    @property
    def out_features(self) -> int:
        return self.qweight.shape[1]


def group_size_for(in_features: int) -> int:
    if in_features % 2:
        raise ValueError(f"int4 packing needs an even K, got {in_features}")
    group = 128 if in_features % 256 == 0 else in_features // 2
    if group & (group - 1):
        raise ValueError(f"int4 group size {group} for K={in_features} is not a power of two")
    return group


@torch.no_grad()
def quantise_int4_k_major(weight: Tensor) -> QuantisedWeight:
    """``weight [N, K]`` (any float dtype) -> packed K-major int4 with fp32 group scales."""
    w = weight.detach()
    if w.dim() != 2:
        raise ValueError(f"expected a 2-D weight [N, K], got {tuple(w.shape)}")
    n, k = w.shape
    group = group_size_for(k)
    half = k // 2
    packed = torch.empty((half, n), dtype=torch.uint8, device=w.device)
    scale = torch.empty((k // group, n), dtype=torch.float32, device=w.device)
    step = max(1, _CHUNK_ELEMENTS // k)
    for start in range(0, n, step):
        block = w[start : start + step].float().reshape(-1, k // group, group)
        s = block.abs().amax(dim=2) / INT4_MAX
        s = torch.where(s > 0, s, torch.ones_like(s))
        q = torch.round(block / s.unsqueeze(2)).clamp_(-INT4_MAX, INT4_MAX).to(torch.int16).reshape(-1, k)
        low = (q[:, :half] + 8).to(torch.uint8)
        high = (q[:, half:] + 8).to(torch.uint8)
        packed[:, start : start + step] = (low | (high << 4)).t()
        scale[:, start : start + step] = s.t()
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
