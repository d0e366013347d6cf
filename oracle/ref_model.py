"""CPU restatement of the reference's decode model. TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / ``--impl reference``
legs may import this module. It rebuilds LoveManna/deltaforge's ``ReferenceModel`` (src/deltaforge/
reference.py:738-817) out of the functions in ``oracle.ref_ops``, with the reference's parameter
names, so a ``state_dict`` moves between the two unchanged; ``tests/golden/make_golden.py`` uses
that to pin this restatement against the real reference's logits and cache tensors.

The module tree (``layers[i].linear_attn.in_proj_qkv`` and so on) is also the shape the product's
installers expect of a model, so the GPU tests install the CUDA path onto an instance of this
class exactly as a reference user would onto a ``ReferenceModel``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from . import ref_ops as R

LINEAR_ATTENTION = "linear_attention"
FULL_ATTENTION = "full_attention"


class _Scale(nn.Module):
    """Holder for a norm weight; the arithmetic lives in ref_ops."""

    def __init__(self, dim: int, eps: float, init: float, dtype=None) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.full((dim,), init, dtype=dtype))


class OracleCache:
    """Decode state with the reference's tensor shapes (src/deltaforge/reference.py:241-299).

    KV ``(B, Hkv, max_seq, D)`` per full-attention layer; conv history ``(B, C, 3)`` and fp32
    recurrent state ``(B, Hv, Dk, Dv)`` per DeltaNet layer; ``seq_len`` is write offset and position.
    """

    def __init__(self, config, batch_size: int, max_seq_len: int, device="cpu", dtype=torch.float32) -> None:
        self.config, self.batch_size, self.max_seq_len = config, batch_size, max_seq_len
        self.device, self.dtype, self.seq_len = torch.device(device), dtype, 0
        self.layers: list[dict[str, Tensor]] = []
        for kind in config.layer_types:
            if kind == FULL_ATTENTION:
                shape = (batch_size, config.num_key_value_heads, max_seq_len, config.head_dim)
                self.layers.append(
                    {"keys": torch.zeros(shape, device=device, dtype=dtype), "values": torch.zeros(shape, device=device, dtype=dtype)}
                )
            else:
                self.layers.append(
                    {
                        "conv": torch.zeros(
                            (batch_size, config.linear_conv_dim, config.linear_conv_kernel_dim - 1), device=device, dtype=dtype
                        ),
                        "recurrent": torch.zeros(
                            (batch_size, config.linear_num_value_heads, config.linear_key_head_dim, config.linear_value_head_dim),
                            device=device,
                            dtype=torch.float32,
                        ),
                    }
                )

    def state_tensors(self) -> tuple[Tensor, ...]:
        out: list[Tensor] = []
        for layer in self.layers:
            out.extend(layer[k] for k in (("keys", "values") if "keys" in layer else ("conv", "recurrent")))
        return tuple(out)

    def ensure_capacity(self, n: int) -> None:
        if self.seq_len + n > self.max_seq_len:
            raise ValueError(f"cache overflow: {self.seq_len} + {n} > max_seq_len={self.max_seq_len}")

    def advance(self, n: int) -> None:
        self.ensure_capacity(n)
        self.seq_len += n


class _DeltaNet(nn.Module):
    def __init__(self, c) -> None:
        super().__init__()
        self.c = c
        self.in_proj_qkv = nn.Linear(c.hidden_size, c.linear_conv_dim, bias=False)
        self.in_proj_z = nn.Linear(c.hidden_size, c.linear_value_dim, bias=False)
        self.in_proj_b = nn.Linear(c.hidden_size, c.linear_num_value_heads, bias=False)
        self.in_proj_a = nn.Linear(c.hidden_size, c.linear_num_value_heads, bias=False)
        self.conv1d = nn.Conv1d(c.linear_conv_dim, c.linear_conv_dim, c.linear_conv_kernel_dim, groups=c.linear_conv_dim, bias=False)
        self.dt_bias = nn.Parameter(torch.zeros(c.linear_num_value_heads))
        self.A_log = nn.Parameter(torch.zeros(c.linear_num_value_heads, dtype=torch.float32))
        self.norm = _Scale(c.linear_value_head_dim, c.rms_norm_eps, 1.0, dtype=torch.float32)
        self.out_proj = nn.Linear(c.linear_value_dim, c.hidden_size, bias=False)

    def forward(self, h: Tensor, cache: dict[str, Tensor] | None) -> Tensor:
        """src/deltaforge/reference.py:512-550."""
        c = self.c
        b, t, _ = h.shape
        qkv = self.in_proj_qkv(h).transpose(1, 2)
        if t == 1 and cache is not None:
            qkv = R.causal_conv_step(qkv, cache["conv"], self.conv1d.weight)
        else:  # prefill: the library conv the reference itself calls (reference.py:496-510)
            hist = c.linear_conv_kernel_dim - 1
            prefix = cache["conv"] if cache is not None else qkv.new_zeros((b, qkv.shape[1], hist))
            full = torch.cat((prefix.to(qkv.dtype), qkv), dim=-1)
            out = F.conv1d(full, self.conv1d.weight, groups=self.conv1d.groups)
            if cache is not None:
                cache["conv"].copy_(full[..., -hist:])
            qkv = F.silu(out)
        qkv = qkv.transpose(1, 2)
        q, k, v = torch.split(qkv, [c.linear_key_dim, c.linear_key_dim, c.linear_value_dim], dim=-1)
        q = q.reshape(b, t, c.linear_num_key_heads, c.linear_key_head_dim)
        k = k.reshape(b, t, c.linear_num_key_heads, c.linear_key_head_dim)
        v = v.reshape(b, t, c.linear_num_value_heads, c.linear_value_head_dim)
        z = self.in_proj_z(h).reshape(b, t, c.linear_num_value_heads, c.linear_value_head_dim)
        g, beta = R.delta_gates(self.in_proj_a(h), self.in_proj_b(h), self.A_log, self.dt_bias)
        if c.linear_value_groups > 1:
            q = q.repeat_interleave(c.linear_value_groups, dim=2)
            k = k.repeat_interleave(c.linear_value_groups, dim=2)
        core, state = R.gated_delta_rule(q, k, v, g, beta, cache["recurrent"] if cache is not None else None)
        if cache is not None:
            cache["recurrent"].copy_(state)
        d = c.linear_value_head_dim
        core = R.gated_rms_norm(core.reshape(-1, d), z.reshape(-1, d), self.norm.weight, self.norm.eps)
        return self.out_proj(core.reshape(b, t, c.linear_value_dim))


class _Attention(nn.Module):
    def __init__(self, c) -> None:
        super().__init__()
        self.c = c
        mult = 2 if c.attn_output_gate else 1
        self.q_proj = nn.Linear(c.hidden_size, c.num_attention_heads * c.head_dim * mult, bias=c.attention_bias)
        self.k_proj = nn.Linear(c.hidden_size, c.num_key_value_heads * c.head_dim, bias=c.attention_bias)
        self.v_proj = nn.Linear(c.hidden_size, c.num_key_value_heads * c.head_dim, bias=c.attention_bias)
        self.o_proj = nn.Linear(c.num_attention_heads * c.head_dim, c.hidden_size, bias=c.attention_bias)
        self.q_norm = _Scale(c.head_dim, c.rms_norm_eps, 0.0)
        self.k_norm = _Scale(c.head_dim, c.rms_norm_eps, 0.0)

    def forward(self, h: Tensor, cos: Tensor, sin: Tensor, cache: dict[str, Tensor] | None, offset: int) -> Tensor:
        """src/deltaforge/reference.py:610-677."""
        c = self.c
        b, t, _ = h.shape
        d = c.head_dim
        proj = self.q_proj(h)
        gate = None
        if c.attn_output_gate:
            proj = proj.view(b, t, c.num_attention_heads, 2 * d)
            q, gate = torch.chunk(proj, 2, dim=-1)
            gate = gate.reshape(b, t, -1)
        else:
            q = proj.view(b, t, c.num_attention_heads, d)
        q = R.rms_norm(q, self.q_norm.weight, self.q_norm.eps).transpose(1, 2)
        k = R.rms_norm(self.k_proj(h).view(b, t, c.num_key_value_heads, d), self.k_norm.weight, self.k_norm.eps).transpose(1, 2)
        v = self.v_proj(h).view(b, t, c.num_key_value_heads, d).transpose(1, 2)
        q = R.partial_rope(q, cos, sin)
        k = R.partial_rope(k, cos, sin)
        if cache is not None:
            end = offset + t
            cache["keys"][:, :, offset:end] = k.to(cache["keys"].dtype)
            cache["values"][:, :, offset:end] = v.to(cache["values"].dtype)
            k, v = cache["keys"][:, :, :end], cache["values"][:, :, :end]
        groups = c.num_key_value_groups
        if groups > 1:
            k = k.repeat_interleave(groups, dim=1)
            v = v.repeat_interleave(groups, dim=1)
        scores = torch.matmul(q, k.transpose(2, 3)) * (d**-0.5)
        if t > 1:
            qpos = torch.arange(t, device=scores.device) + offset
            blocked = torch.arange(k.shape[2], device=scores.device).unsqueeze(0) > qpos.unsqueeze(1)
            scores = scores.masked_fill(blocked, torch.finfo(scores.dtype).min)
        w = F.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
        attn = torch.matmul(w, v).transpose(1, 2).reshape(b, t, -1)
        if gate is not None:
            attn = attn * R.output_gate(gate, c.output_gate_type)
        return self.o_proj(attn)


class _MLP(nn.Module):
    def __init__(self, c) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(R.silu_mul(self.gate_proj(x), self.up_proj(x)))


class _Layer(nn.Module):
    def __init__(self, c, idx: int) -> None:
        super().__init__()
        self.layer_idx, self.layer_type = idx, c.layer_types[idx]
        if self.layer_type == LINEAR_ATTENTION:
            self.linear_attn = _DeltaNet(c)
        else:
            self.self_attn = _Attention(c)
        self.mlp = _MLP(c)
        self.input_layernorm = _Scale(c.hidden_size, c.rms_norm_eps, 0.0)
        self.post_attention_layernorm = _Scale(c.hidden_size, c.rms_norm_eps, 0.0)

    def forward(self, h, cos, sin, cache: OracleCache | None, offset: int):
        """src/deltaforge/reference.py:714-735."""
        lc = cache.layers[self.layer_idx] if cache is not None else None
        n = R.rms_norm(h, self.input_layernorm.weight, self.input_layernorm.eps)
        mixed = self.linear_attn(n, lc) if self.layer_type == LINEAR_ATTENTION else self.self_attn(n, cos, sin, lc, offset)
        h = h + mixed
        n = R.rms_norm(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps)
        return h + self.mlp(n)


class OracleModel(nn.Module):
    """``forward(input_ids, cache, num_logits_to_keep=...) -> (logits, cache)``; tied LM head."""

    def __init__(self, config) -> None:
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList(_Layer(config, i) for i in range(config.num_hidden_layers))
        self.norm = _Scale(config.hidden_size, config.rms_norm_eps, 0.0)
        # A buffer, as in the reference (reference.py:173): a dtype cast of the model rounds it too.
        self.register_buffer("inv_freq", R.rope_inv_freq(config.rotary_dim, config.rope_theta), persistent=False)

    def new_cache(self, batch_size: int, max_seq_len: int) -> OracleCache:
        p = self.embed_tokens.weight
        return OracleCache(self.config, batch_size, max_seq_len, device=p.device, dtype=p.dtype)

    def project_logits(self, h: Tensor) -> Tensor:
        """src/deltaforge/reference.py:764-777."""
        return F.linear(h, self.embed_tokens.weight.to(h.dtype))

    @torch.no_grad()
    def forward(self, input_ids: Tensor, cache: OracleCache | None = None, *, num_logits_to_keep: int = 0):
        """src/deltaforge/reference.py:779-817."""
        c = self.config
        b, t = input_ids.shape
        offset = 0
        if cache is not None:
            cache.ensure_capacity(t)
            offset = cache.seq_len
        pos = (torch.arange(t, device=input_ids.device) + offset).unsqueeze(0).expand(b, -1)
        h = self.embed_tokens(input_ids)
        cos, sin = R.rope_cos_sin(pos, self.inv_freq, h.dtype)
        for layer in self.layers:
            h = layer(h, cos, sin, cache, offset)
        h = R.rms_norm(h, self.norm.weight, self.norm.eps)
        if num_logits_to_keep:
            h = h[:, -num_logits_to_keep:]
        logits = self.project_logits(h)
        if cache is not None:
            cache.advance(t)
        return logits, cache


# --------------------------------------------------------------------------------------
# The reference's int4 torch path, installed on every linear and the tied head
# --------------------------------------------------------------------------------------


class _Int4Linear(nn.Linear):
    """``DequantInt4Linear`` of src/deltaforge/kernels/visible_int4_head.py:272-285."""

    def forward(self, x: Tensor) -> Tensor:  # type: ignore[override]
        return R.dequant_gemv_int4(x, self.w_k_major, self.qscale, self.qgroup)


def install_int4_everywhere(model: OracleModel) -> OracleModel:
    """Quantise every ``nn.Linear`` and the tied head to group-wise int4, torch-expression forward.

    Follows ``install_int4_wide_torch_dequant`` (src/deltaforge/kernels/visible_int4_head.py:335-361,
    :504-518) widened to the 32-row gate projections (src/deltaforge/kernels/tiled_gemv.py:1145-1154)
    so that, as the benchmark config states, all linears are int4. Quantised copies are buffers
    named ``w_k_major`` / ``qscale`` plus attribute ``qgroup`` (tiled_gemv.py:1049-1071).
    """
    for module in model.modules():
        if isinstance(module, nn.Linear) and not isinstance(module, _Int4Linear):
            packed, scale, group = R.quantise_int4_k_major(module.weight)
            module.register_buffer("w_k_major", packed, persistent=False)
            module.register_buffer("qscale", scale, persistent=False)
            module.qgroup = group
            module.__class__ = _Int4Linear
    packed, scale, group = R.quantise_int4_k_major(model.embed_tokens.weight)
    model.register_buffer("head_w_k_major", packed, persistent=False)
    model.register_buffer("head_qscale", scale, persistent=False)
    model.head_qgroup = group

    base = type(model)

    class _Int4Head(base):  # type: ignore[misc, valid-type]
        def project_logits(self, h: Tensor) -> Tensor:
            return R.dequant_gemv_int4(h, self.head_w_k_major, self.head_qscale, self.head_qgroup)

    model.__class__ = _Int4Head
    return model


@torch.no_grad()
def greedy_decode(model, input_ids: Tensor, max_new_tokens: int, cache=None) -> Tensor:
    """Greedy loop of src/deltaforge/model.py:108-148 (without the pluggable-loop hook)."""
    if max_new_tokens < 1:
        raise ValueError("max_new_tokens must be at least 1")
    b, t = input_ids.shape
    if cache is None:
        cache = model.new_cache(b, t + max_new_tokens)
    logits, _ = model(input_ids, cache, num_logits_to_keep=1)
    tok = logits[:, -1].argmax(dim=-1, keepdim=True)
    out = [tok]
    for _ in range(max_new_tokens - 1):
        logits, _ = model(tok, cache, num_logits_to_keep=1)
        tok = logits[:, -1].argmax(dim=-1, keepdim=True)
        out.append(tok)
    return torch.cat(out, dim=1)
