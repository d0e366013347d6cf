"""The test helper that builds a CPU oracle around a ``ModelWeights``: its memoising linears (dequantise once,
multiply many times) must give exactly what the oracle's own int4 linears give."""

from __future__ import annotations

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from oracle_build import oracle_cache_like, oracle_from_weights  # noqa: E402

from deltaforge_b200 import engine as E  # noqa: E402
from deltaforge_b200 import synth  # noqa: E402
from deltaforge_b200.config import tiny_config  # noqa: E402


def test_memoised_oracle_linears_are_bit_identical():
    cfg = tiny_config()
    weights = synth.random_model_weights(cfg, seed=11, device="cpu", scale_dtype=torch.bfloat16)
    plain, memo = oracle_from_weights(weights), oracle_from_weights(weights, memo=True)
    cache = E.DecodeCache(cfg, 1, 16, device="cpu")
    synth.fill_cache(cache, 5, seed=3)
    ca, cb = oracle_cache_like(plain, cache), oracle_cache_like(memo, cache)
    tok = torch.tensor([[7]])
    for _ in range(3):
        la, _ = plain(tok, ca, num_logits_to_keep=1)
        lb, _ = memo(tok, cb, num_logits_to_keep=1)
        assert torch.equal(la, lb)
        tok = la[:, -1].argmax(-1, keepdim=True)
    for a, b in zip(ca.state_tensors(), cb.state_tensors()):
        assert torch.equal(a, b)
