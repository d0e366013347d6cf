"""Checkpoint reading and the quantised on-disk format, on the CPU with small synthetic checkpoints.

A checkpoint is written with the real checkpoint's tensor naming (text decoder under ``model.language_model.``, plus a
vision-tower and an MTP tensor that must be skipped), in two shards with an index file; what ``load_hf_checkpoint`` makes
of it must equal, bit for bit, what quantising the same model in memory gives.
"""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import save_file

from deltaforge_b200 import checkpoint as CK
from deltaforge_b200 import engine as E
from deltaforge_b200.config import tiny_config
from oracle import ref_model as M


def seeded_model(cfg):
    torch.manual_seed(3)
    model = M.OracleModel(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.copy_(0.1 * torch.randn(p.shape))
            elif name.endswith("A_log"):
                p.copy_(torch.log(torch.rand(p.shape) * 8 + 0.1))
            else:
                p.copy_(torch.randn(p.shape) * 0.05)
    return model.to(torch.bfloat16).eval()


def write_checkpoint(model, directory):
    state = {CK.TEXT_PREFIX + k: v.detach().clone() for k, v in model.state_dict().items()}
    state["model.visual.patch_embed.weight"] = torch.zeros(4, 4)
    state["mtp.layers.0.weight"] = torch.zeros(2, 2)
    names = sorted(state)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fname, keys in shards.items():
        save_file({k: state[k].contiguous() for k in keys}, str(directory / fname))
        weight_map.update({k: fname for k in keys})
    (directory / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    return state


def assert_same_weights(a: E.ModelWeights, b: E.ModelWeights):
    assert torch.equal(a.embed, b.embed) and torch.equal(a.final_norm, b.final_norm) and torch.equal(a.inv_freq, b.inv_freq)
    assert torch.equal(a.head.qweight, b.head.qweight) and torch.equal(a.head.scale, b.head.scale)
    assert len(a.layers) == len(b.layers)
    for la, lb in zip(a.layers, b.layers):
        assert la.kind == lb.kind and la.gnorm_w_is_bf16 == lb.gnorm_w_is_bf16
        for f in ("in_proj", "out_proj", "gate_up", "down"):
            qa, qb = getattr(la, f), getattr(lb, f)
            assert qa.group_size == qb.group_size
            assert torch.equal(qa.qweight, qb.qweight) and torch.equal(qa.scale, qb.scale), f
        for f in ("input_norm", "post_norm", "conv_w", "a_log", "dt_bias", "gnorm_w", "q_norm", "k_norm"):
            ta, tb = getattr(la, f), getattr(lb, f)
            assert (ta is None) == (tb is None), f
            if ta is not None:
                assert ta.dtype == tb.dtype and torch.equal(ta, tb), f


def test_checkpoint_reads_as_the_in_memory_quantisation(tmp_path):
    cfg = tiny_config()
    model = seeded_model(cfg)
    write_checkpoint(model, tmp_path)
    got = CK.load_hf_checkpoint(tmp_path, cfg, device="cpu", scale_dtype=None)
    want = E.weights_from_model(M.install_int4_everywhere(seeded_model(cfg)), device="cpu")
    assert_same_weights(got, want)
    assert len(CK.checkpoint_files(tmp_path)) == 2


def test_quantised_file_round_trip(tmp_path):
    cfg = tiny_config()
    write_checkpoint(seeded_model(cfg), tmp_path)
    weights = CK.load_hf_checkpoint(tmp_path, cfg, device="cpu")
    path = tmp_path / "model.int4.safetensors"
    CK.save_quantised(weights, path)
    back = CK.load_quantised(path, device="cpu")
    assert back.config == cfg
    assert_same_weights(back, weights)
    assert back.weight_bytes() == weights.weight_bytes()


def test_unknown_and_missing_tensors_are_errors(tmp_path):
    cfg = tiny_config()
    model = seeded_model(cfg)
    state = write_checkpoint(model, tmp_path)
    extra = tmp_path / "extra"
    extra.mkdir()
    bad = dict(state)
    bad[CK.TEXT_PREFIX + "layers.0.linear_attn.mystery.weight"] = torch.zeros(2, 2)
    save_file({k: v.contiguous() for k, v in bad.items()}, str(extra / "model.safetensors"))
    with pytest.raises(CK.CheckpointError, match="unrecognised"):
        CK.load_hf_checkpoint(extra, cfg, device="cpu")
    fewer = tmp_path / "fewer"
    fewer.mkdir()
    short = {k: v for k, v in state.items() if not k.endswith("layers.1.mlp.down_proj.weight")}
    save_file({k: v.contiguous() for k, v in short.items()}, str(fewer / "model.safetensors"))
    with pytest.raises(CK.CheckpointError, match="lacks"):
        CK.load_hf_checkpoint(fewer, cfg, device="cpu")
    with pytest.raises(CK.CheckpointError, match="not a quantised model file"):
        CK.load_quantised(extra / "model.safetensors", device="cpu")
