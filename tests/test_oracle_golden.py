"""The CPU oracle against vectors produced by the real reference (tests/golden/make_golden.py).

Everything here is bit-exact: the oracle restates the reference's torch expressions, so on the same
inputs it must return the same bits. One thread, as when the vectors were made, so that reductions
run in the same order.
"""

from __future__ import annotations

import pytest
import torch

from deltaforge_b200.config import tiny_config
from oracle import ref_model as M
from oracle import ref_ops as R

torch.set_num_threads(1)


def same(a: torch.Tensor, b: torch.Tensor) -> None:
    assert a.dtype == b.dtype and a.shape == b.shape
    assert torch.equal(a, b), f"max abs diff {(a.float() - b.float()).abs().max().item()}"


def test_group_size_for(golden):
    for k, group in golden("int4")["group_size_for"].items():
        assert R.group_size_for(k) == group
    with pytest.raises(ValueError):
        R.group_size_for(7)
    with pytest.raises(ValueError):
        R.group_size_for(6 * 2 * 5)  # half is not a power of two


def test_quantise_pack_dequant_gemv(golden):
    for case in golden("int4")["cases"]:
        packed, scale, group = R.quantise_int4_k_major(case["weight"])
        assert group == case["group"]
        same(packed, case["packed"])
        same(scale, case["scale"])
        same(R.dequantise_int4_k_major(packed, scale, group), case["dense_fp32"])
        same(R.dequant_gemv_int4(case["x"], packed, scale, group), case["y"])


def test_raw_nibbles_cover_all_sixteen_values(golden):
    raw = golden("int4")["raw"]
    q = R.unpack_int4_k_major(raw["packed"])
    assert q.min().item() == -8 and q.max().item() == 7
    same(R.dequantise_int4_k_major(raw["packed"], raw["scale"], raw["group"]), raw["dense_fp32"])
    same(R.dequant_gemv_int4(raw["x"], raw["packed"], raw["scale"], raw["group"]), raw["y"])


def test_pack_identities():
    # Known answers in the reference's own tests (tiled_gemv_test.py:424-463): byte = low | high << 4,
    # low nibble is row j, high nibble is row j + K/2, values offset by 8.
    w = torch.zeros((1, 4))
    w[0] = torch.tensor([7.0, -7.0, 1.0, 0.0])
    packed, scale, group = R.quantise_int4_k_major(w)
    assert group == 2 and packed.shape == (2, 1) and scale.shape == (2, 1)
    assert packed[0, 0].item() == (7 + 8) | ((7 + 8) << 4)  # second group rescales 1.0 to 7
    assert packed[1, 0].item() == (-7 + 8) | ((0 + 8) << 4)
    assert torch.equal(R.unpack_int4_k_major(packed)[:, 0], torch.tensor([7, -7, 7, 0], dtype=torch.int16))
    zero = R.quantise_int4_k_major(torch.zeros((3, 8)))
    assert torch.all(zero[1] == 1.0) and torch.all(zero[0] == 0x88)


def test_elementwise(golden):
    g = golden("elementwise")
    same(R.rms_norm(g["rms"]["x"], g["rms"]["w"], g["rms"]["eps"]), g["rms"]["y"])
    gd = g["gated"]
    same(R.gated_rms_norm(gd["x"], gd["z"], gd["w_fp32"], gd["eps"]), gd["y_fp32w"])
    same(R.gated_rms_norm(gd["x"], gd["z"], gd["w_fp32"].to(torch.bfloat16), gd["eps"]), gd["y_bf16w"])
    rp = g["rope"]
    cos, sin = R.rope_cos_sin(rp["pos"], R.rope_inv_freq(rp["rotary_dim"], rp["theta"]), torch.bfloat16)
    same(cos, rp["cos"])
    same(sin, rp["sin"])
    same(R.partial_rope(rp["x"], cos, sin), rp["y"])
    same(R.rotate_half(g["rotate_half"]["x"]), g["rotate_half"]["y"])
    assert g["rotate_half"]["y"].tolist() == [-3.0, -4.0, 1.0, 2.0]
    same(R.silu_mul(g["swiglu"]["gate"], g["swiglu"]["up"]), g["swiglu"]["y"])
    same(R.output_gate(g["outgate"]["gate"], "sigmoid"), g["outgate"]["sigmoid"])
    same(R.output_gate(g["outgate"]["gate"], "swish"), g["outgate"]["swish"])
    summed, _ = R.add_rms_norm(g["residual"]["b"], g["residual"]["a"], g["rms"]["w"], 1e-6)
    same(summed, g["residual"]["sum"])


def test_rope_position_zero_is_identity():
    cos, sin = R.rope_cos_sin(torch.zeros((1, 1), dtype=torch.long), R.rope_inv_freq(8, 1e4), torch.float32)
    x = torch.randn((1, 2, 1, 32))
    assert torch.equal(R.partial_rope(x, cos, sin), x)


def test_rms_norm_weight_is_zero_centred():
    x = torch.randn((2, 16))
    base = R.rms_norm(x, torch.zeros(16), 1e-6)
    assert torch.allclose(R.rms_norm(x, torch.ones(16), 1e-6), 2 * base)


def test_conv_step(golden):
    c = golden("deltanet")["conv"]
    cache = c["cache"].clone()
    same(R.causal_conv_step(c["x"], cache, c["w"]), c["y"])
    same(cache, c["cache_after"])
    hist = torch.tensor([[[1.0, 2.0, 3.0]]])
    R.causal_conv_step(torch.tensor([[[4.0]]]), hist, torch.zeros((1, 1, 4)))
    assert hist.tolist() == [[[2.0, 3.0, 4.0]]]


def test_delta_rule(golden):
    d = golden("deltanet")
    r = d["rule"]
    out, state = R.gated_delta_rule(r["q"], r["k"], r["v"], r["g"], r["beta"], r["state"])
    same(out, r["out"])
    same(state, r["state_after"])
    gt = d["gates"]
    g, beta = R.delta_gates(gt["a"], gt["b"], gt["A_log"], gt["dt_bias"])
    same(g, gt["g"])
    same(beta, gt["beta"])


def test_delta_rule_beta_zero_only_decays():
    s = torch.randn((1, 2, 4, 4))
    q = R.l2norm(torch.randn((1, 2, 4)))
    k = R.l2norm(torch.randn((1, 2, 4)))
    g = -torch.rand((1, 2))
    _, s1 = R.delta_rule_step(s, q, k, torch.randn((1, 2, 4)), g, torch.zeros((1, 2)))
    assert torch.equal(s1, s * g.exp()[..., None, None])
    assert s1.dtype == torch.float32


def test_attention(golden):
    for case in golden("attention")["cases"]:
        same(R.decode_attention(case["q"], case["k"], case["v"], case["scale"]), case["y"])


def _oracle_from_golden(g):
    model = M.OracleModel(tiny_config())
    missing = model.load_state_dict(g["state_dict"], strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    return model.to(torch.bfloat16).eval()


def _run(model, prompt, steps=4):
    cache = model.new_cache(prompt.shape[0], 16)
    logits, _ = model(prompt, cache, num_logits_to_keep=1)
    all_logits = [logits]
    tok = logits[:, -1].argmax(dim=-1, keepdim=True)
    toks = [tok]
    for _ in range(steps):
        logits, _ = model(tok, cache, num_logits_to_keep=1)
        all_logits.append(logits)
        tok = logits[:, -1].argmax(dim=-1, keepdim=True)
        toks.append(tok)
    return torch.stack(all_logits), torch.cat(toks, dim=1), cache


def test_model_bf16_matches_reference(golden):
    g = golden("tiny_model")
    logits, toks, cache = _run(_oracle_from_golden(g), g["prompt"])
    same(logits, g["bf16"]["logits"])
    same(toks, g["bf16"]["tokens"])
    assert cache.seq_len == g["bf16"]["seq_len"]
    for mine, theirs in zip(cache.state_tensors(), g["bf16"]["cache"]):
        same(mine, theirs)


def test_model_int4_matches_reference(golden):
    g = golden("tiny_model")
    model = M.install_int4_everywhere(_oracle_from_golden(g))
    logits, toks, cache = _run(model, g["prompt"])
    same(logits, g["int4"]["logits"])
    same(toks, g["int4"]["tokens"])
    for mine, theirs in zip(cache.state_tensors(), g["int4"]["cache"]):
        same(mine, theirs)
    model2 = M.install_int4_everywhere(_oracle_from_golden(g))
    same(M.greedy_decode(model2, g["prompt"], 6), g["int4_greedy"])


def test_cache_overflow_raises():
    model = M.OracleModel(tiny_config())
    cache = model.new_cache(1, 2)
    with pytest.raises(ValueError):
        model(torch.zeros((1, 3), dtype=torch.long), cache)
