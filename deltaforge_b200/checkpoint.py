"""Weights from disk: a Hugging Face checkpoint of the model, or this package's own quantised file.

Two entry points, both producing the ``ModelWeights`` a ``DecodeEngine`` takes:

* ``load_hf_checkpoint(path, config)`` reads the ``.safetensors`` shards of a Qwen3.5 checkpoint tensor by tensor and
  quantises every projection to group-wise int4 on the device as it arrives (``quantise_int4_k_major``: the CUDA packer),
  so the bf16 model is never resident as a whole. Tensor names follow the checkpoint's: the text decoder lives under
  ``model.language_model.``, the vision tower (``model.visual.``) and the multi-token-prediction head (``mtp.``) are
  skipped, exactly the selection of the reference's loader (src/deltaforge/weights.py:43-45, :124-150, :192-270), and a
  tensor inside the text decoder that this code does not know is an error, never silently dropped. The fused layouts the
  engine wants (``in_proj_qkv|z|b|a``, ``q|k|v``, ``gate|up``) are concatenations of the separately quantised
  projections, which is exact because groups run along K.
* ``save_quantised`` / ``load_quantised`` write and read the quantised model itself (packed nibbles, scales, norms, conv
  taps, gates, embedding) as one ``.safetensors`` file plus the configuration in its metadata, so that a 4.2 B-parameter
  model is packed once, not at every start (the reference re-quantises on every install,
  src/deltaforge/kernels/tiled_gemv.py:1049-1071).

No checkpoint of the model exists on the machines this was built on; the tests write small synthetic checkpoints with
the checkpoint's tensor names and shapes rules and read them back.
"""

from __future__ import annotations

import dataclasses
import json
import re
from pathlib import Path

import torch
from torch import Tensor

from .config import FULL_ATTENTION, LINEAR_ATTENTION, ModelConfig
from .engine import BF16, LayerWeights, ModelWeights
from .quant import QuantisedWeight, concat_along_n, quantise_int4_k_major

TEXT_PREFIX = "model.language_model."
SKIPPED_PREFIXES = ("model.visual.", "mtp.")
_LAYER = re.compile(re.escape(TEXT_PREFIX) + r"layers\.(\d+)\.(.+)$")

_DELTANET = ("linear_attn.in_proj_qkv.weight", "linear_attn.in_proj_z.weight", "linear_attn.in_proj_b.weight", "linear_attn.in_proj_a.weight",
             "linear_attn.conv1d.weight", "linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.norm.weight", "linear_attn.out_proj.weight")  # fmt: skip
_ATTENTION = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
              "self_attn.q_norm.weight", "self_attn.k_norm.weight")  # fmt: skip
_COMMON = ("input_layernorm.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")


class CheckpointError(RuntimeError):
    """The checkpoint and the model configuration do not line up."""


def checkpoint_files(path: str | Path) -> list[Path]:
    """The ``.safetensors`` files of a checkpoint: the file itself, the shards its index names, or every shard there."""
    path = Path(path)
    if path.is_file():
        return [path]
    index = path / "model.safetensors.index.json"
    if index.exists():
        return [path / shard for shard in sorted(set(json.loads(index.read_text())["weight_map"].values()))]
    shards = sorted(path.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    return shards


def _is_projection(suffix: str) -> bool:
    return suffix.endswith("_proj.weight") or suffix.startswith("linear_attn.in_proj_")


@torch.no_grad()
def load_hf_checkpoint(path: str | Path, config: ModelConfig, device="cuda", scale_dtype: torch.dtype | None = BF16) -> ModelWeights:
    """Read a checkpoint into int4 ``ModelWeights`` on ``device``, quantising projection by projection."""
    from safetensors import safe_open

    dev = torch.device(device)
    per_layer: list[dict[str, object]] = [{} for _ in range(config.num_hidden_layers)]
    top: dict[str, Tensor] = {}

    def quantised(t: Tensor) -> QuantisedWeight:
        qw = quantise_int4_k_major(t.to(dev))
        if scale_dtype is not None and qw.scale.dtype != scale_dtype:
            qw = QuantisedWeight(qw.qweight, qw.scale.to(scale_dtype), 4, qw.group_size)
        return qw

    for shard in checkpoint_files(path):
        with safe_open(str(shard), framework="pt") as handle:
            for name in handle.keys():  # noqa: SIM118 - safe_open has no __contains__
                if name.startswith(SKIPPED_PREFIXES):
                    continue
                if name in (TEXT_PREFIX + "embed_tokens.weight", TEXT_PREFIX + "norm.weight", "lm_head.weight"):
                    top[name.removeprefix(TEXT_PREFIX)] = handle.get_tensor(name)
                    continue
                m = _LAYER.match(name)
                if m is None:
                    raise CheckpointError(f"unrecognised checkpoint tensor: {name!r}")
                idx, suffix = int(m.group(1)), m.group(2)
                if idx >= config.num_hidden_layers:
                    raise CheckpointError(f"{name!r}: the configuration has {config.num_hidden_layers} layers")
                kind = config.layer_types[idx]
                known = _COMMON + (_DELTANET if kind == LINEAR_ATTENTION else _ATTENTION)
                if suffix not in known:
                    raise CheckpointError(f"unrecognised tensor {name!r} for a {kind} layer")
                t = handle.get_tensor(name)
                per_layer[idx][suffix] = quantised(t) if _is_projection(suffix) else t.to(dev)

    if "embed_tokens.weight" not in top or "norm.weight" not in top:
        raise CheckpointError("the checkpoint lacks the embedding table or the final norm")
    embed = top["embed_tokens.weight"].to(dev, BF16).contiguous()
    if tuple(embed.shape) != (config.vocab_size, config.hidden_size):
        raise CheckpointError(f"embedding table is {tuple(embed.shape)}, the configuration says {(config.vocab_size, config.hidden_size)}")
    head_src = embed if config.tie_word_embeddings else top.get("lm_head.weight")
    if head_src is None:
        raise CheckpointError("untied embeddings need lm_head.weight")
    inv_freq = 1.0 / (config.rope_theta ** (torch.arange(0, config.rotary_dim, 2, dtype=torch.float32) / config.rotary_dim))
    out = ModelWeights(config, embed, top["norm.weight"].to(dev, BF16).contiguous(), quantised(head_src),
                       inv_freq.to(BF16).float().to(dev))  # fmt: skip
    for idx, (kind, got) in enumerate(zip(config.layer_types, per_layer)):
        want = _COMMON + (_DELTANET if kind == LINEAR_ATTENTION else _ATTENTION)
        missing = [s for s in want if s not in got]
        if missing:
            raise CheckpointError(f"layer {idx} ({kind}) lacks {missing}")
        norm = lambda s: got[s].to(BF16).contiguous()  # noqa: E731
        gate_up = concat_along_n([got["mlp.gate_proj.weight"], got["mlp.up_proj.weight"]])
        if kind == LINEAR_ATTENTION:
            taps = got["linear_attn.conv1d.weight"].reshape(config.linear_conv_dim, -1).to(BF16).contiguous()
            if taps.shape[1] != 4:
                raise CheckpointError(f"layer {idx}: the fused conv is the four-tap case; got {taps.shape[1]} taps")
            gnorm = got["linear_attn.norm.weight"]
            lw = LayerWeights(
                kind=kind, input_norm=norm("input_layernorm.weight"), post_norm=norm("post_attention_layernorm.weight"),
                in_proj=concat_along_n([got["linear_attn.in_proj_qkv.weight"], got["linear_attn.in_proj_z.weight"],
                                        got["linear_attn.in_proj_b.weight"], got["linear_attn.in_proj_a.weight"]]),
                out_proj=got["linear_attn.out_proj.weight"], gate_up=gate_up, down=got["mlp.down_proj.weight"], conv_w=taps,
                a_log=got["linear_attn.A_log"].float().contiguous(), dt_bias=got["linear_attn.dt_bias"].float().contiguous(),
                gnorm_w=gnorm.float().contiguous(), gnorm_w_is_bf16=gnorm.dtype == BF16,
            )  # fmt: skip
        elif kind == FULL_ATTENTION:
            lw = LayerWeights(
                kind=kind, input_norm=norm("input_layernorm.weight"), post_norm=norm("post_attention_layernorm.weight"),
                in_proj=concat_along_n([got["self_attn.q_proj.weight"], got["self_attn.k_proj.weight"], got["self_attn.v_proj.weight"]]),
                out_proj=got["self_attn.o_proj.weight"], gate_up=gate_up, down=got["mlp.down_proj.weight"],
                q_norm=norm("self_attn.q_norm.weight"), k_norm=norm("self_attn.k_norm.weight"),
            )  # fmt: skip
        else:
            raise CheckpointError(f"layer {idx} has unknown kind {kind!r}")
        out.layers.append(lw)
    return out


# ---------------------------------------------------------------------------------------------------------------------
# the quantised model as one file
# ---------------------------------------------------------------------------------------------------------------------

_QW_FIELDS = ("in_proj", "out_proj", "gate_up", "down")
_T_FIELDS = ("input_norm", "post_norm", "conv_w", "a_log", "dt_bias", "gnorm_w", "q_norm", "k_norm")


def _config_to_json(config) -> str:
    return json.dumps({k: (list(v) if isinstance(v, tuple) else v) for k, v in dataclasses.asdict(config).items()})


def save_quantised(weights: ModelWeights, path: str | Path) -> None:
    """Write the quantised model to ``path`` (safetensors): every tensor a ``DecodeEngine`` needs, nothing re-derivable."""
    from safetensors.torch import save_file

    tensors: dict[str, Tensor] = {
        "embed": weights.embed, "final_norm": weights.final_norm, "inv_freq": weights.inv_freq,
        "head.qweight": weights.head.qweight, "head.scale": weights.head.scale,
    }  # fmt: skip
    meta = {"format": "dfb200-int4-k-major-v1", "config": _config_to_json(weights.config), "head.group": str(weights.head.group_size)}
    for i, lw in enumerate(weights.layers):
        for f in _QW_FIELDS:
            qw: QuantisedWeight = getattr(lw, f)
            tensors[f"layers.{i}.{f}.qweight"], tensors[f"layers.{i}.{f}.scale"] = qw.qweight, qw.scale
            meta[f"layers.{i}.{f}.group"] = str(qw.group_size)
        for f in _T_FIELDS:
            t = getattr(lw, f)
            if t is not None:
                tensors[f"layers.{i}.{f}"] = t
        meta[f"layers.{i}.kind"] = lw.kind
        meta[f"layers.{i}.gnorm_w_is_bf16"] = str(int(lw.gnorm_w_is_bf16))
    save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, str(path), metadata=meta)


def load_quantised(path: str | Path, device="cuda") -> ModelWeights:
    """Read a file written by ``save_quantised``: bit-identical tensors, no quantisation work."""
    from safetensors import safe_open

    dev = torch.device(device)
    with safe_open(str(path), framework="pt") as handle:
        meta = handle.metadata() or {}
        if meta.get("format") != "dfb200-int4-k-major-v1":
            raise CheckpointError(f"{path} is not a quantised model file of this package (format {meta.get('format')!r})")
        cfg_dict = {k: (tuple(v) if isinstance(v, list) else v) for k, v in json.loads(meta["config"]).items()}
        config = ModelConfig(**cfg_dict)
        get = lambda name: handle.get_tensor(name).to(dev)  # noqa: E731
        names = set(handle.keys())

        def qw(prefix: str) -> QuantisedWeight:
            return QuantisedWeight(get(prefix + ".qweight"), get(prefix + ".scale"), 4, int(meta[prefix + ".group"]))

        out = ModelWeights(config, get("embed"), get("final_norm"), qw("head"), get("inv_freq"))
        for i in range(config.num_hidden_layers):
            opt = {f: (get(f"layers.{i}.{f}") if f"layers.{i}.{f}" in names else None) for f in _T_FIELDS}
            out.layers.append(
                LayerWeights(
                    kind=meta[f"layers.{i}.kind"], in_proj=qw(f"layers.{i}.in_proj"), out_proj=qw(f"layers.{i}.out_proj"),
                    gate_up=qw(f"layers.{i}.gate_up"), down=qw(f"layers.{i}.down"),
                    gnorm_w_is_bf16=bool(int(meta[f"layers.{i}.gnorm_w_is_bf16"])), **opt,
                )  # fmt: skip
            )
    return out
