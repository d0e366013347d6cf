"""Test helper: a CPU oracle model that holds exactly the int4 buffers of a ``ModelWeights``.

The full-size parity tests generate the synthetic 4B-shaped model directly in its quantised form
(``deltaforge_b200.synth``) and need the CPU oracle to multiply by the very same nibbles and scales. The
oracle's module tree is built on the meta device (its fp32 ``nn.Linear`` weights would take 17 GB and are
never read: every linear's forward is the int4 torch expression) and only the tensors the forward pass
touches are made real.
"""

from __future__ import annotations

import torch
from torch import nn

from deltaforge_b200.config import LINEAR_ATTENTION
from oracle import ref_model as M
from oracle import ref_ops as R

BF16 = torch.bfloat16


class _MemoInt4Linear(M._Int4Linear):
    """The oracle's int4 linear with its dequantised weight kept between calls.

    ``R.dequant_gemv_int4`` dequantises, rounds the weight to the activation dtype and multiplies in fp32 at every call.
    The rounded weight depends on the buffers only, so a test that runs the oracle for many positions may keep it: the
    same product of the same values, about four times faster per position."""

    def forward(self, x):  # type: ignore[override]
        dense = getattr(self, "_dense", None)
        if dense is None or dense[0] != x.dtype:
            w = R.dequantise_int4_k_major(self.w_k_major, self.qscale, self.qgroup).to(x.dtype)
            dense = (x.dtype, w.float() if _MEMO_FP32 else w)
            self._dense = dense
        k = dense[1].shape[0]
        return (x.reshape(-1, k).float() @ dense[1].float()).to(x.dtype).reshape(*x.shape[:-1], dense[1].shape[1])


def _available_host_gb() -> float:
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable:"):
                return int(line.split()[1]) / 1e6
    except OSError:
        pass
    return 0.0


_MEMO_FP32 = _available_host_gb() > 64.0  # 4 bytes per weight when the host has room, 2 (and a conversion per call) otherwise


def _int4(lin: nn.Linear, packed: torch.Tensor, scale: torch.Tensor, group: int, memo: bool = False) -> None:
    lin.register_buffer("w_k_major", packed.cpu().contiguous(), persistent=False)
    lin.register_buffer("qscale", scale.cpu().contiguous(), persistent=False)
    lin.qgroup = group
    lin.__class__ = _MemoInt4Linear if memo else M._Int4Linear


def _split(qw, sizes):
    """Column slices of a projection fused along N."""
    assert sum(sizes) == qw.out_features
    out, at = [], 0
    for n in sizes:
        out.append((qw.qweight[:, at : at + n], qw.scale[:, at : at + n], qw.group_size))
        at += n
    return out


def _param(t: torch.Tensor) -> nn.Parameter:
    return nn.Parameter(t.detach().cpu().clone(), requires_grad=False)


@torch.no_grad()
def oracle_from_weights(weights, memo: bool = False) -> M.OracleModel:
    """The oracle's int4 model (``install_int4_everywhere`` form) around the buffers of ``weights``. ``memo``: the layer
    projections keep their dequantised weights between calls (for runs over many positions; needs 6-12 GB of host memory
    at full size)."""
    cfg = weights.config
    with torch.device("meta"):
        model = M.OracleModel(cfg)
    model.embed_tokens.weight = _param(weights.embed.to(BF16))
    model.norm.weight = _param(weights.final_norm.to(BF16))
    model.register_buffer("inv_freq", weights.inv_freq.detach().cpu().to(BF16), persistent=False)
    i = cfg.intermediate_size
    for layer, lw in zip(model.layers, weights.layers):
        layer.input_layernorm.weight = _param(lw.input_norm.to(BF16))
        layer.post_attention_layernorm.weight = _param(lw.post_norm.to(BF16))
        (gp, gs, gg), (up, us, ug) = _split(lw.gate_up, [i, i])
        _int4(layer.mlp.gate_proj, gp, gs, gg, memo)
        _int4(layer.mlp.up_proj, up, us, ug, memo)
        _int4(layer.mlp.down_proj, lw.down.qweight, lw.down.scale, lw.down.group_size, memo)
        if lw.kind == LINEAR_ATTENTION:
            m = layer.linear_attn
            hv = cfg.linear_num_value_heads
            parts = _split(lw.in_proj, [cfg.linear_conv_dim, cfg.linear_value_dim, hv, hv])
            for lin, (p, s, g) in zip((m.in_proj_qkv, m.in_proj_z, m.in_proj_b, m.in_proj_a), parts):
                _int4(lin, p, s, g, memo)
            _int4(m.out_proj, lw.out_proj.qweight, lw.out_proj.scale, lw.out_proj.group_size, memo)
            m.conv1d.weight = _param(lw.conv_w.to(BF16).reshape(cfg.linear_conv_dim, 1, -1))
            m.A_log = _param(lw.a_log.to(BF16))
            m.dt_bias = _param(lw.dt_bias.to(BF16))
            m.norm.weight = _param(lw.gnorm_w.to(BF16) if lw.gnorm_w_is_bf16 else lw.gnorm_w.float())
        else:
            m = layer.self_attn
            d = cfg.head_dim
            qn = cfg.num_attention_heads * d * (2 if cfg.attn_output_gate else 1)
            kvn = cfg.num_key_value_heads * d
            parts = _split(lw.in_proj, [qn, kvn, kvn])
            for lin, (p, s, g) in zip((m.q_proj, m.k_proj, m.v_proj), parts):
                _int4(lin, p, s, g, memo)
            _int4(m.o_proj, lw.out_proj.qweight, lw.out_proj.scale, lw.out_proj.group_size, memo)
            m.q_norm.weight = _param(lw.q_norm.to(BF16))
            m.k_norm.weight = _param(lw.k_norm.to(BF16))
    model.register_buffer("head_w_k_major", weights.head.qweight.cpu().contiguous(), persistent=False)
    model.register_buffer("head_qscale", weights.head.scale.cpu().contiguous(), persistent=False)
    model.head_qgroup = weights.head.group_size

    class _Int4Head(type(model)):  # type: ignore[misc]
        def project_logits(self, h):
            if not memo:
                return R.dequant_gemv_int4(h, self.head_w_k_major, self.head_qscale, self.head_qgroup)
            dense = getattr(self, "_head_dense", None)
            if dense is None or dense[0] != h.dtype:
                w = R.dequantise_int4_k_major(self.head_w_k_major, self.head_qscale, self.head_qgroup).to(h.dtype)
                dense = (h.dtype, w.float() if _MEMO_FP32 else w)
                self._head_dense = dense
            k = dense[1].shape[0]
            return (h.reshape(-1, k).float() @ dense[1].float()).to(h.dtype).reshape(*h.shape[:-1], dense[1].shape[1])

    model.__class__ = _Int4Head
    return model.eval()


@torch.no_grad()
def oracle_cache_like(model: M.OracleModel, cache) -> M.OracleCache:
    """A CPU cache with the contents and position of a device cache."""
    oc = M.OracleCache(model.config, cache.batch_size, cache.max_seq_len, device="cpu", dtype=BF16)
    for a, b in zip(oc.state_tensors(), cache.state_tensors()):
        a.copy_(b.cpu())
    oc.seq_len = cache.seq_len
    return oc
