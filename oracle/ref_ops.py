"""CPU restatement of the reference's decode-step operations. TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline / ``--impl reference`` legs may import it. Every function restates one
function of LoveManna/deltaforge in plain torch-on-CPU operations, keeps that function's rounding
points, and cites the file:line it follows (paths are relative to the reference project root).

Parity pin: ``tests/golden/*.pt`` were produced by importing the real reference in the build
container (``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks every function
here against those vectors bit for bit.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

INT4_MAX = 7  # src/deltaforge/kernels/quantised_linear.py:101


# --------------------------------------------------------------------------------------
# int4, group-wise, K-major
# --------------------------------------------------------------------------------------


def group_size_for(in_features: int) -> int:
    """Group width along K. src/deltaforge/kernels/quantised_linear.py:193-207.

    128 when both halves of K split into whole groups (K % 256 == 0), otherwise one group per
    half. Odd K and non-power-of-two groups are refused.
    """
    if in_features % 2:
        raise ValueError(f"int4 packing needs an even K, got {in_features}")
    group = 128 if in_features % 256 == 0 else in_features // 2
    if group & (group - 1):
        raise ValueError(f"int4 group size {group} for K={in_features} is not a power of two")
    return group


def quantise_int4_k_major(weight: Tensor) -> tuple[Tensor, Tensor, int]:
    """``W[N,K]`` -> ``(packed[K/2,N] uint8, scale[K/group,N] fp32, group)``.

    src/deltaforge/kernels/tiled_gemv.py:242-278: symmetric, scale = amax(group)/7 (1 where the
    group is all zero), q = clamp(round(w/scale), -7, 7), stored as q+8; byte [j,n] carries row j
    in its low nibble and row j+K/2 in its high nibble.
    """
    w = weight.detach().float()
    n, k = w.shape
    group = group_size_for(k)
    grouped = w.reshape(n, k // group, group)
    scale = grouped.abs().amax(dim=2) / INT4_MAX
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = torch.round(grouped / scale.unsqueeze(2)).clamp_(-INT4_MAX, INT4_MAX).to(torch.int16).reshape(n, k)
    low = (q[:, : k // 2] + 8).to(torch.uint8)
    high = (q[:, k // 2 :] + 8).to(torch.uint8)
    return (low | (high << 4)).t().contiguous(), scale.t().contiguous(), group


def unpack_int4_k_major(packed: Tensor) -> Tensor:
    """``packed[K/2,N]`` -> signed values ``[K,N]`` int16. tiled_gemv.py:284-287 (the integer half)."""
    low = (packed & 0x0F).to(torch.int16) - 8
    high = (packed >> 4).to(torch.int16) - 8
    return torch.cat((low, high), dim=0)


def dequantise_int4_k_major(packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """``[K,N]`` fp32 weight: value times its group's scale, in fp32. tiled_gemv.py:281-288."""
    k = packed.shape[0] * 2
    n = packed.shape[1]
    q = unpack_int4_k_major(packed).float().reshape(k // group_size, group_size, n)
    return (q * scale.float().unsqueeze(1)).reshape(k, n)


def dequant_gemv_int4(x: Tensor, packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """The int4 linear as the reference's champion computes it.

    src/deltaforge/kernels/visible_int4_head.py:187-199: dequantise, round the scaled weight to
    the activation dtype, then ``x.float() @ W.float()`` and round the result to that dtype.
    """
    k = packed.shape[0] * 2
    n = packed.shape[1]
    flat = x.reshape(-1, k)
    dense = dequantise_int4_k_major(packed, scale, group_size).to(x.dtype)
    return (flat.float() @ dense.float()).to(x.dtype).reshape(*x.shape[:-1], n)


def dequant_gemv_int4_fp32(x: Tensor, packed: Tensor, scale: Tensor, group_size: int) -> Tensor:
    """fp32 recompute of the same product with no output rounding: the tolerance yardstick."""
    k = packed.shape[0] * 2
    dense = dequantise_int4_k_major(packed, scale, group_size).to(x.dtype)
    return x.reshape(-1, k).double() @ dense.double()


# --------------------------------------------------------------------------------------
# Norms and elementwise
# --------------------------------------------------------------------------------------


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """fp32 normalise, scale by ``1 + weight``, back to x's dtype. src/deltaforge/reference.py:92-96."""
    y = x.float()
    y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    y = y * (1.0 + weight.float())
    return y.to(x.dtype)


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float) -> Tensor:
    """Normalise, round to x's dtype, times plain ``weight``, times silu(gate) in fp32.

    src/deltaforge/reference.py:115-121. ``weight * normed`` follows torch type promotion, so a
    bf16 weight rounds that product to bf16 and an fp32 weight does not.
    """
    y = x.float()
    y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    y = weight * y.to(x.dtype)
    y = y * F.silu(gate.float())
    return y.to(x.dtype)


def add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """``(residual + x, rms_norm(residual + x))``; the sum is rounded to the activation dtype first.

    src/deltaforge/kernels/fused_rmsnorm_residual.py:164-193 and :76-82 (rounding of the sum).
    """
    summed = residual + x
    return summed, rms_norm(summed, weight, eps)


def silu_mul(gate: Tensor, up: Tensor) -> Tensor:
    """``silu(gate) * up`` with the SiLU rounded to the activation dtype before the multiply.

    src/deltaforge/reference.py:692-693; src/deltaforge/kernels/fused_swiglu.py:18-22.
    """
    return F.silu(gate) * up


def output_gate(gate: Tensor, gate_type: str = "sigmoid") -> Tensor:
    """fp32 nonlinearity of the attention output gate, cast back. src/deltaforge/reference.py:558-568."""
    if gate_type == "sigmoid":
        return torch.sigmoid(gate.float()).to(gate.dtype)
    if gate_type == "swish":
        return F.silu(gate.float()).to(gate.dtype)
    raise ValueError(f"unknown output_gate_type {gate_type!r}")


# --------------------------------------------------------------------------------------
# Rotary embedding
# --------------------------------------------------------------------------------------


def rotate_half(x: Tensor) -> Tensor:
    """``[a, b] -> [-b, a]`` over the last axis. src/deltaforge/reference.py:132-134."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def rope_inv_freq(rotary_dim: int, theta: float) -> Tensor:
    """``theta ** (-2i / rotary_dim)`` in fp32. src/deltaforge/reference.py:170-172."""
    return 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def rope_cos_sin(position_ids: Tensor, inv_freq: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    """cos/sin tables ``(batch, seq, 2 * len(inv_freq))`` for text positions.

    src/deltaforge/reference.py:189-200. ``inv_freq`` is a module buffer there, so casting the model
    to bf16 rounds it to bf16 too and the angles are computed from the rounded frequencies (the
    product is still fp32 by type promotion); pass the buffer as the model holds it. For text all
    three mRoPE rows hold the same position, so the interleave selects equal values and the result
    is standard RoPE (asserted exactly by the reference, reference_test.py:156-192); the interleave
    is therefore not restated.
    """
    freqs = position_ids.float().unsqueeze(-1) * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def partial_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotate the leading ``rotary_dim`` dims of ``x (batch, heads, seq, head_dim)``.

    src/deltaforge/reference.py:137-149; arithmetic stays in x's dtype.
    """
    cos = cos.unsqueeze(1)
    sin = sin.unsqueeze(1)
    rd = cos.shape[-1]
    rot = x[..., :rd]
    return torch.cat(((rot * cos) + (rotate_half(rot) * sin), x[..., rd:]), dim=-1)


# --------------------------------------------------------------------------------------
# Gated DeltaNet pieces
# --------------------------------------------------------------------------------------


def causal_conv_step(x: Tensor, conv_cache: Tensor, weight: Tensor) -> Tensor:
    """One decode step of the 4-tap depthwise causal conv + SiLU; advances ``conv_cache`` in place.

    ``x (B,C,1)``, ``conv_cache (B,C,3)`` oldest first, ``weight (C,1,4)``.
    src/deltaforge/kernels/inline_causal_conv.py:98-129 (bit-identical to the ``F.conv1d`` path of
    src/deltaforge/reference.py:496-510): four fp32 products summed left to right, rounded to the
    activation dtype, then SiLU.
    """
    channels = x.shape[1]
    w = weight.reshape(channels, -1).float()
    h = conv_cache
    xv = x[..., 0]
    acc = h[..., 0].float() * w[:, 0] + h[..., 1].float() * w[:, 1] + h[..., 2].float() * w[:, 2] + xv.float() * w[:, 3]
    out = F.silu(acc.to(x.dtype)).unsqueeze(-1)
    conv_cache.copy_(torch.cat((h[..., 1:], x.to(conv_cache.dtype)), dim=-1))
    return out


def l2norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """``x * rsqrt(sum(x^2) + eps)``. src/deltaforge/reference.py:403-404."""
    return x * torch.rsqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def delta_rule_step(state: Tensor, q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor) -> tuple[Tensor, Tensor]:
    """One token of the gated delta rule on pre-normalised q, k. All fp32.

    ``state (B,H,Dk,Dv)``, ``q,k (B,H,Dk)``, ``v (B,H,Dv)``, ``g,beta (B,H)``.
    Loop body of src/deltaforge/reference.py:450-458 (same contract as the reference's
    ``deltaforge::delta_rule_step`` op, src/deltaforge/kernels/gated_delta_step.py:109-123).
    """
    state = state * g.exp()[..., None, None]
    recalled = (state * k.unsqueeze(-1)).sum(dim=-2)
    delta = (v - recalled) * beta.unsqueeze(-1)
    state = state + k.unsqueeze(-1) * delta.unsqueeze(-2)
    out = (state * q.unsqueeze(-1)).sum(dim=-2)
    return out, state


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, initial_state: Tensor | None):
    """Sequential delta rule over ``(B, T, H, D)`` inputs. src/deltaforge/reference.py:407-461."""
    in_dtype = q.dtype
    q, k, v, beta, g = (t.transpose(1, 2).float().contiguous() for t in (q, k, v, beta, g))
    q = l2norm(q)
    k = l2norm(k)
    q = q / math.sqrt(q.shape[-1])
    b, h, t, dk = k.shape
    dv = v.shape[-1]
    state = torch.zeros((b, h, dk, dv), dtype=torch.float32, device=v.device) if initial_state is None else initial_state.float()
    out = torch.zeros_like(v)
    for i in range(t):
        out[:, :, i], state = delta_rule_step(state, q[:, :, i], k[:, :, i], v[:, :, i], g[:, :, i], beta[:, :, i])
    return out.transpose(1, 2).contiguous().to(in_dtype), state


def delta_gates(a_proj: Tensor, b_proj: Tensor, a_log: Tensor, dt_bias: Tensor) -> tuple[Tensor, Tensor]:
    """``beta = sigmoid(b)`` in b's dtype; ``g = -exp(A_log) * softplus(a + dt_bias)`` in fp32.

    src/deltaforge/reference.py:528-532.
    """
    beta = b_proj.sigmoid()
    g = -a_log.float().exp() * F.softplus(a_proj.float() + dt_bias.float())
    return g, beta


# --------------------------------------------------------------------------------------
# Decode attention
# --------------------------------------------------------------------------------------


def decode_attention(query: Tensor, key: Tensor, value: Tensor, scale: float) -> Tensor:
    """Single-token GQA attention, as the reference's module computes it at seq_len 1.

    ``query (B,Hq,D)``, ``key/value (B,Hkv,L,D)`` -> ``(B,Hq,D)``.
    src/deltaforge/kernels/gqa_decode.py:322-335 (restating src/deltaforge/reference.py:655-672):
    expand KV heads, activation-dtype matmul, scale, fp32 softmax rounded back, matmul.
    """
    groups = query.shape[1] // key.shape[1]
    k = key.repeat_interleave(groups, dim=1)
    v = value.repeat_interleave(groups, dim=1)
    scores = torch.matmul(query.unsqueeze(2), k.transpose(2, 3)) * scale
    weights = F.softmax(scores, dim=-1, dtype=torch.float32).to(query.dtype)
    return torch.matmul(weights, v).squeeze(2)


def decode_attention_fp64(query: Tensor, key: Tensor, value: Tensor, scale: float) -> Tensor:
    """The same attention in fp64 with no intermediate rounding: the tolerance yardstick."""
    groups = query.shape[1] // key.shape[1]
    k = key.double().repeat_interleave(groups, dim=1)
    v = value.double().repeat_interleave(groups, dim=1)
    scores = torch.matmul(query.double().unsqueeze(2), k.transpose(2, 3)) * scale
    return torch.matmul(scores.softmax(dim=-1), v).squeeze(2)
