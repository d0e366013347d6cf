"""Algorithmic bytes of one decode step: what the roofline fraction is computed from.

Counts each byte the step must move through HBM once (SI units, like the reference's byte model,
src/deltaforge/harness/bytes_model.py:11-15): int4 weights and their group scales, the KV cache read,
the recurrent state read and written, the conv history read and written, and the logits written.
Activations between kernels (a few hundred KB, L2-resident) are not counted. The reference's own
model ignores scale bytes (bytes_model.py:262-271); this one includes them.
"""

from __future__ import annotations

from .config import FULL_ATTENTION, LINEAR_ATTENTION


def linear_params(cfg) -> tuple[int, int]:
    """(parameters in the layer projections, parameters in the head)."""
    h, i = cfg.hidden_size, cfg.intermediate_size
    mlp = 3 * h * i
    lin = h * (cfg.linear_conv_dim + cfg.linear_value_dim + 2 * cfg.linear_num_value_heads) + cfg.linear_value_dim * h
    qw = cfg.num_attention_heads * cfg.head_dim * (2 if cfg.attn_output_gate else 1)
    att = h * (qw + 2 * cfg.num_key_value_heads * cfg.head_dim) + cfg.num_attention_heads * cfg.head_dim * h
    layers = sum(mlp + (lin if t == LINEAR_ATTENTION else att) for t in cfg.layer_types)
    return layers, cfg.vocab_size * h


def decode_bytes_per_step(cfg, *, batch: int, context: int, scale_bytes: int = 2, group: int = 128) -> dict[str, int]:
    """Bytes per decode step of ``batch`` sequences with ``context`` tokens already cached."""
    layers, head = linear_params(cfg)
    params = layers + head
    weights = params // 2 + params // group * scale_bytes
    n_att = sum(t == FULL_ATTENTION for t in cfg.layer_types)
    n_lin = sum(t == LINEAR_ATTENTION for t in cfg.layer_types)
    kv = batch * n_att * 2 * cfg.num_key_value_heads * (context + 1) * cfg.head_dim * 2
    state = batch * n_lin * 2 * cfg.linear_num_value_heads * cfg.linear_key_head_dim * cfg.linear_value_head_dim * 4
    conv = batch * n_lin * 2 * cfg.linear_conv_dim * (cfg.linear_conv_kernel_dim - 1) * 2
    logits = batch * cfg.vocab_size * 2
    total = weights + kv + state + conv + logits
    return {"weights": weights, "kv": kv, "state": state, "conv": conv, "logits": logits, "total": total}


def gemv_bytes(k: int, n: int, rows: int = 1, scale_bytes: int = 4, group: int = 128) -> int:
    """Algorithmic bytes of one int4 GEMV launch: packed weights, scales, and the bf16 output."""
    return k * n // 2 + (k // group) * n * scale_bytes + rows * n * 2
