"""Parity at the sizes the benchmark configurations name, against the CPU oracle on identical int4 buffers.

* The tied LM head at its full size: 248320 x 2560, bf16 group scales, final RMSNorm fused as the prologue,
  every one of the 248320 logits compared with ``dequant_gemv_int4(rms_norm(x))`` and its fp64 recompute.
* The whole 32-layer 4B-shaped decode step with a 4096-token cache: the CUDA step in both arithmetic modes
  (FAST, the one the benchmark times, and EXACT) against the oracle, teacher-forced on the oracle's own
  continuation for 32 positions. What is measured is what the reference's distribution check measures
  (src/deltaforge/harness/correctness.py:383-464): mean KL(P_oracle || P_cuda) in nats and top-1 agreement,
  plus max / rms logit error in units of the logit scale.

The weights are the synthetic stand-ins of ``deltaforge_b200.synth`` (uniform nibbles, |N(0, 0.02)| scales),
generated once in the quantised form; ``tests/oracle_build.py`` wraps the same buffers in the oracle's module
tree. Set ``DFB200_PARITY_REPORT`` to a file name to get the measured figures as JSON lines.
"""

from __future__ import annotations

import json
import os

import pytest
import torch

from deltaforge_b200 import engine as E
from deltaforge_b200 import ops, qwen3_5_4b_config, synth
from oracle import ref_ops as R
from oracle_build import oracle_cache_like, oracle_from_weights

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def report(record: dict) -> None:
    print("PARITY " + json.dumps(record))
    path = os.environ.get("DFB200_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(record) + "\n")


def kl_and_agreement(ref_logits: torch.Tensor, cand_logits: torch.Tensor) -> tuple[float, float]:
    lr = torch.log_softmax(ref_logits.float().reshape(-1, ref_logits.shape[-1]), dim=-1)
    lc = torch.log_softmax(cand_logits.float().reshape(-1, cand_logits.shape[-1]), dim=-1)
    kl = (lr.exp() * (lr - lc)).sum(-1).mean().item()
    agree = (lr.argmax(-1) == lc.argmax(-1)).float().mean().item()
    return kl, agree


def test_lm_head_at_full_size_against_the_oracle():
    """The LM-head configuration: all 248320 columns, bf16 scales, RMSNorm prologue, through the streaming kernel."""
    k, n = 2560, 248320
    g = torch.Generator().manual_seed(2024)
    packed = torch.randint(0, 256, (k // 2, n), generator=g, dtype=torch.uint8)
    scale = (torch.randn((k // 128, n), generator=g).abs() * 0.02).clamp_min(1e-5).to(BF16)
    x = torch.randn((1, k), generator=g).to(BF16)
    gamma = (torch.randn(k, generator=g) * 0.1).to(BF16)
    xn = R.rms_norm(x, gamma, 1e-6)
    want = R.dequant_gemv_int4(xn, packed, scale, 128)  # the oracle's bf16 logits
    pd = packed.to(DEV)
    k8 = ops.int4_repack_k8(pd)
    got = ops.int4_gemv_fused(
        x.to(DEV), pd, scale.to(DEV), 128, prologue=ops.PRO_RMSNORM, norm_weight=gamma.to(DEV), eps=1e-6, packed_k8=k8
    ).cpu()
    assert got.shape == want.shape and got.dtype == BF16
    # the fp64 recompute, in column chunks (the dequantised matrix is 5 GB in fp64)
    truth = torch.empty((1, n), dtype=torch.float64)
    for c0 in range(0, n, 31040):
        c1 = min(n, c0 + 31040)
        dense = R.dequantise_int4_k_major(packed[:, c0:c1], scale[:, c0:c1], 128).to(BF16).double()
        truth[:, c0:c1] = xn.double() @ dense
    rms = truth.pow(2).mean().sqrt().item()
    err = (got.double() - truth).abs()
    # north-star bar: rtol 2e-2 against the fp32 recompute (atol 2e-2 of the mean magnitude for values near zero)
    bound = 2e-2 * truth.abs() + 2e-2 * truth.abs().mean()
    assert bool((err <= bound).all()), f"worst excess {(err - bound).max().item():.4g}"
    err_o = (got.double() - want.double()).abs()
    assert bool((err_o <= 2e-2 * want.double().abs() + 2e-2 * truth.abs().mean()).all())
    rel_rms = (err.pow(2).mean().sqrt() / rms).item()
    oracle_rms = ((want.double() - truth).pow(2).mean().sqrt() / rms).item()
    differ = (got != want).float().mean().item()
    report({"case": "lm_head_248320x2560", "rms_err_over_rms": rel_rms, "oracle_rms_err_over_rms": oracle_rms,
            "max_err_over_rms": (err.max() / rms).item(), "fraction_of_logits_differing_from_oracle": differ,
            "argmax_equal": bool(got.float().argmax() == want.float().argmax())})  # fmt: skip
    assert rel_rms < 3e-3  # bf16 output rounding alone is 1.7e-3
    assert got.float().argmax() == want.float().argmax() or (want.float().topk(2).values.diff().abs().item() < 2e-2 * rms)


@pytest.fixture(scope="module")
def full_model():
    cfg = qwen3_5_4b_config()
    weights = synth.random_model_weights(cfg, seed=4321, device=DEV, scale_dtype=BF16)
    # uniform nibbles with |N(0, 0.02)| scales give logits of standard deviation 4.6; a quarter of that (an exact
    # scaling of the bf16 group scales) puts them at the order-one scale of a trained model's, so that KL reads
    # as it would there
    weights.head.scale.mul_(0.25)
    return cfg, weights


def test_32_layer_step_with_a_4096_token_cache_against_the_oracle(full_model):
    """The benchmarked configuration, teacher-forced for 32 positions, FAST and EXACT arithmetic."""
    cfg, weights = full_model
    context, positions = 4096, 32
    max_seq = context + positions + 8
    caches = {m: E.DecodeCache(cfg, 1, max_seq, device=DEV) for m in ("fast", "exact")}
    synth.fill_cache(caches["fast"], context, seed=99)
    caches["exact"].load_from(caches["fast"])
    oracle = oracle_from_weights(weights, memo=True)  # 32 positions: the dequantised weights are kept between them
    ocache = oracle_cache_like(oracle, caches["fast"])
    engines = {
        "fast": E.DecodeEngine(weights, caches["fast"], math=E.MATH_FAST),
        "exact": E.DecodeEngine(weights, caches["exact"], math=E.MATH_EXACT),
    }
    tok = torch.tensor([[1000]])
    ref, got = [], {m: [] for m in engines}
    for _ in range(positions):
        lr, _ = oracle(tok, ocache, num_logits_to_keep=1)
        for m, eng in engines.items():
            got[m].append(eng.step(tok.reshape(-1).to(DEV)).float().cpu().clone())
        ref.append(lr[:, -1].float())
        tok = lr[:, -1].argmax(-1, keepdim=True)  # every arm continues on the oracle's token
    ref_t = torch.stack(ref)
    scale = ref_t.std().item()
    figures = {}
    for m, eng in engines.items():
        eng.check_status()
        g = torch.stack(got[m])
        diff = (ref_t - g).abs()
        kl, agree = kl_and_agreement(ref_t, g)
        top2 = ref_t.topk(2, dim=-1).values
        gap = (top2[..., 0] - top2[..., 1]).reshape(-1)
        figures[m] = {"max_err_over_scale": diff.max().item() / scale, "rms_err_over_scale": diff.pow(2).mean().sqrt().item() / scale,
                      "kl_nats": kl, "top1_agreement": agree, "logit_scale": scale, "positions": positions,
                      "smallest_oracle_top2_gap_over_scale": gap.min().item() / scale}  # fmt: skip
        report({"case": "32_layers_ctx4096", "math": m, **figures[m]})
        # cache contents after 32 steps: the new KV rows and the recurrent state
        for a, b in zip(ocache.state_tensors(), eng.cache.state_tensors()):
            a, b = a.float(), b.float().cpu()
            assert (a - b).abs().max().item() <= (2e-2 if m == "exact" else 2e-1) + 5e-2 * a.abs().max().item()
    # Bars: EXACT reproduces the oracle's products up to fp32 summation order; FAST leaves out one bf16 rounding
    # per weight. Both stay far below the reference's own int4-vs-bf16 KL of 1.7e-2 to 9e-2 nats.
    assert figures["exact"]["kl_nats"] < 1e-3 and figures["exact"]["rms_err_over_scale"] < 3e-2
    assert figures["fast"]["kl_nats"] < 5e-3 and figures["fast"]["rms_err_over_scale"] < 6e-2
    # greedy tokens agree wherever the oracle's top-2 gap is larger than the arm's own worst logit error
    for m, eng in engines.items():
        g = torch.stack(got[m])
        top2 = ref_t.topk(2, dim=-1).values
        decisive = (top2[..., 0] - top2[..., 1]) > 2 * (ref_t - g).abs().amax(-1)
        assert bool((ref_t.argmax(-1) == g.argmax(-1))[decisive].all())


def test_batch_32_with_a_16k_token_cache_against_the_oracle():
    """The many-sequence configuration on a 4-layer cut (one full-attention layer): 32 sequences, 16384 cached tokens each, so
    the engine takes the tensor-core projections and the tensor-core split-KV decode kernel."""
    from deltaforge_b200.config import ModelConfig, hybrid_layer_types

    cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096,
                      layer_types=hybrid_layer_types(4), name="qwen3.5-4b-width-4l")  # fmt: skip
    batch, context, steps = 32, 16384, 2
    weights = synth.random_model_weights(cfg, seed=77, device=DEV, scale_dtype=BF16)
    cache = E.DecodeCache(cfg, batch, context + steps + 6, device=DEV)
    synth.fill_cache(cache, context, seed=5)
    oracle = oracle_from_weights(weights)
    ocache = oracle_cache_like(oracle, cache)
    eng = E.DecodeEngine(weights, cache, attn_splits=16)  # the configuration names 16 to 64 key slices
    tok = torch.randint(0, cfg.vocab_size, (batch, 1), generator=torch.Generator().manual_seed(3))
    ref, got = [], []
    for _ in range(steps):
        lr, _ = oracle(tok, ocache, num_logits_to_keep=1)
        got.append(eng.step(tok.reshape(-1).to(DEV)).float().cpu().clone())
        ref.append(lr[:, -1].float())
        tok = lr[:, -1].argmax(-1, keepdim=True)
    eng.check_status()
    ref_t, g = torch.stack(ref), torch.stack(got)
    scale = ref_t.std().item()
    diff = (ref_t - g).abs()
    kl, agree = kl_and_agreement(ref_t, g)
    report({"case": "4_layers_batch32_ctx16384", "max_err_over_scale": diff.max().item() / scale,
            "rms_err_over_scale": diff.pow(2).mean().sqrt().item() / scale, "kl_nats": kl, "top1_agreement": agree,
            "attn_splits": eng.attn_splits})  # fmt: skip
    assert diff.max().item() < 8e-2 * scale and diff.pow(2).mean().sqrt().item() < 1.5e-2 * scale
    assert kl < 2e-4
    for a, b in zip(ocache.state_tensors(), cache.state_tensors()):
        a, b = a.float(), b.float().cpu()
        assert (a - b).abs().max().item() <= 2e-2 + 2e-2 * a.abs().max().item()
