"""The bounds build (``-DDFB_BOUNDS``): the ragged-shape tests and a small decode engine run once more on the library
variant whose kernels check every store and tile index, in a child process (``DFB200_BOUNDS_BUILD=1`` selects the
variant at import), and no kernel may have recorded a violation (status 60 and up)."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

ENGINE_CHECK = """
import torch
from deltaforge_b200 import _lib, engine as E, synth
from deltaforge_b200.config import ModelConfig, hybrid_layer_types
assert _lib.library_path().name == "libdfb200_bounds.so"
cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
w = synth.random_model_weights(cfg, seed=3, device="cuda", scale_dtype=torch.bfloat16)
for ctx, max_seq in ((5, 64), (300, 512), (4096, 4200)):
    cache = E.DecodeCache(cfg, 1, max_seq, device="cuda")
    synth.fill_cache(cache, ctx, seed=5)
    eng = E.DecodeEngine(w, cache)
    eng.decode(torch.tensor([17], device="cuda"), 3)
    eng.check_status()  # raises on any recorded code, the bounds codes included
    assert bool(torch.isfinite(eng.logits.float()).all())
print("bounds engine ok")
"""


def _run(args: list[str]) -> subprocess.CompletedProcess:
    env = dict(os.environ, DFB200_BOUNDS_BUILD="1", PYTHONPATH=str(ROOT))
    return subprocess.run([sys.executable, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)


def test_ragged_launches_pass_on_the_bounds_build():
    proc = _run(["-m", "pytest", "tests/test_canaries_gpu.py", "tests/test_gemv_mma_gpu.py", "-m", "gpu", "-x", "-q"])
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]


def test_decode_engine_records_no_violation_on_the_bounds_build():
    proc = _run(["-c", ENGINE_CHECK])
    assert proc.returncode == 0 and "bounds engine ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-2000:]
