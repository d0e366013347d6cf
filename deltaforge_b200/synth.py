"""Seeded synthetic weights and decode state with the benchmark model's shapes and distributions.

No checkpoint exists on the machines this runs on, so the benchmark and the full-size tests use
random-init stand-ins: int4 nibbles uniform in 0..15, group scales |N(0, 0.02)| (fp32 or bf16), norm
weights N(0, 0.1) under the ``1 + w`` convention, conv taps N(0, 0.5), ``A = exp(A_log) ~ U(0, 16)``,
embeddings N(0, 1); caches are filled with N(0, 1) (KV, conv history) and N(0, 0.1) (recurrent state).
Every tensor comes from its own ``torch.Generator`` seeded from one base seed, so a given
``(config, seed)`` names the same model on every machine.
"""

from __future__ import annotations

import torch

from .config import FULL_ATTENTION, LINEAR_ATTENTION
from .engine import BF16, LayerWeights, ModelWeights
from .quant import QuantisedWeight, group_size_for


class _Seeds:
    def __init__(self, base: int, device) -> None:
        self.base, self.n, self.device = base, 0, device

    def next(self) -> torch.Generator:
        self.n += 1
        return torch.Generator(device=self.device).manual_seed(self.base * 1_000_003 + self.n)


def random_int4(k: int, n: int, gen: torch.Generator, device, scale_dtype=torch.float32) -> QuantisedWeight:
    group = group_size_for(k)
    packed = torch.randint(0, 256, (k // 2, n), generator=gen, dtype=torch.uint8, device=device)
    scale = (torch.randn((k // group, n), generator=gen, device=device).abs() * 0.02 + 1e-5).to(scale_dtype)
    return QuantisedWeight(packed, scale, 4, group)


@torch.no_grad()
def random_model_weights(cfg, seed: int = 0, device="cuda", scale_dtype=torch.bfloat16) -> ModelWeights:
    """A random-init int4 model of ``cfg``'s architecture, generated directly in the quantised format."""
    s = _Seeds(seed, device)
    h, i = cfg.hidden_size, cfg.intermediate_size

    def norm_w(n: int) -> torch.Tensor:
        return (torch.randn(n, generator=s.next(), device=device) * 0.1).to(BF16)

    def q(k: int, n: int) -> QuantisedWeight:
        return random_int4(k, n, s.next(), device, scale_dtype)

    embed = torch.randn((cfg.vocab_size, h), generator=s.next(), device=device, dtype=torch.float32).to(BF16)
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.rotary_dim, 2, dtype=torch.float32) / cfg.rotary_dim))
    inv_freq = inv_freq.to(BF16).float().to(device)  # a bf16 model holds this buffer in bf16
    out = ModelWeights(cfg, embed, norm_w(h), q(h, cfg.vocab_size), inv_freq)
    for kind in cfg.layer_types:
        if kind == LINEAR_ATTENTION:
            hv, dv = cfg.linear_num_value_heads, cfg.linear_value_head_dim
            in_n = cfg.linear_conv_dim + cfg.linear_value_dim + 2 * hv
            a = torch.rand(hv, generator=s.next(), device=device) * 16 + 1e-3
            lw = LayerWeights(
                kind=kind, input_norm=norm_w(h), post_norm=norm_w(h),
                in_proj=q(h, in_n), out_proj=q(cfg.linear_value_dim, h), gate_up=q(h, 2 * i), down=q(i, h),
                conv_w=(torch.randn((cfg.linear_conv_dim, 4), generator=s.next(), device=device) * 0.5).to(BF16),
                a_log=a.log().to(BF16).float(),
                dt_bias=(torch.randn(hv, generator=s.next(), device=device) * 0.1).to(BF16).float(),
                gnorm_w=(1.0 + 0.1 * torch.randn(dv, generator=s.next(), device=device)).to(BF16).float(),
                gnorm_w_is_bf16=True,
            )  # fmt: skip
        else:
            d = cfg.head_dim
            in_n = cfg.num_attention_heads * d * (2 if cfg.attn_output_gate else 1) + 2 * cfg.num_key_value_heads * d
            lw = LayerWeights(
                kind=kind, input_norm=norm_w(h), post_norm=norm_w(h),
                in_proj=q(h, in_n), out_proj=q(cfg.num_attention_heads * d, h), gate_up=q(h, 2 * i), down=q(i, h),
                q_norm=norm_w(d), k_norm=norm_w(d),
            )  # fmt: skip
        out.layers.append(lw)
    return out


@torch.no_grad()
def fill_cache(cache, context: int, seed: int = 1) -> None:
    """Prefill a decode cache with seeded noise as if ``context`` tokens had been processed."""
    if context > cache.max_seq_len:
        raise ValueError(f"context {context} exceeds the cache's max_seq_len {cache.max_seq_len}")
    dev = cache.state_tensors()[0].device
    s = _Seeds(seed, dev)
    for layer in cache.layers:
        if "keys" in layer:
            for name in ("keys", "values"):
                t = layer[name]
                t.zero_()
                t[:, :, :context].copy_(torch.randn(t[:, :, :context].shape, generator=s.next(), device=dev, dtype=torch.float32))
        else:
            layer["conv"].copy_(torch.randn(layer["conv"].shape, generator=s.next(), device=dev, dtype=torch.float32))
            layer["recurrent"].copy_(torch.randn(layer["recurrent"].shape, generator=s.next(), device=dev) * 0.1)
    cache.seq_len = context
