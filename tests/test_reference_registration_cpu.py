"""``register_with_reference`` against the real reference package, where that package is importable.

The reference is a separate project: these tests run where ``deltaforge`` can be imported (``PYTHONPATH`` or the
directory named by ``DELTAFORGE_REFERENCE_SRC``) and are skipped elsewhere. No GPU is needed: registration only
fills tables and registers per-device kernels on op objects.
"""

from __future__ import annotations

import importlib
import os
import sys

import pytest
import torch

src = os.environ.get("DELTAFORGE_REFERENCE_SRC")
if src and src not in sys.path:
    sys.path.insert(0, src)
try:
    kernels = importlib.import_module("deltaforge.kernels")
    ref_model = importlib.import_module("deltaforge.model")
except ImportError:  # the reference does not travel with this repository
    pytest.skip("the reference package `deltaforge` is not importable here", allow_module_level=True)

from deltaforge_b200 import installers  # noqa: E402

NAMES = ["b200_decode_step", "b200_int4_linears", *installers.PER_OP_KERNELS]


def test_registration_fills_the_references_three_tables_and_is_idempotent():
    first = installers.register_with_reference()
    for name in NAMES:
        assert name in kernels.REGISTRY  # KernelRegistry.__contains__, not its private table
        assert name in ref_model.INSTALLERS
        assert name in kernels.CHECK_BUILDERS  # reported as checked, not "unchecked"
        assert name in first
    kernels.REGISTRY.check_invariants()
    before = len(kernels.REGISTRY)
    second = installers.register_with_reference()
    assert len(kernels.REGISTRY) == before and sorted(second) == sorted(first)
    # every registration replaces an operation the reference allows to be replaced, and none is a champion
    for entry in kernels.REGISTRY:
        if entry.name in NAMES:
            assert entry.replaces in kernels.REPLACEABLE_OPS
            assert str(getattr(entry.status, "value", entry.status)) == "candidate"


def test_every_reference_op_object_gets_a_cuda_kernel():
    installers.register_with_reference()
    for op_name, (module_name, attr, ours) in installers.DROP_IN_OPS.items():
        their_op = getattr(importlib.import_module(module_name), attr)
        # torch.library.CustomOpDef keeps per-device implementations in _backend_fns
        assert "cuda" in their_op._backend_fns, op_name
        assert f"deltaforge::{op_name}" in installers.register_with_reference()
        # same argument list on both sides: the redirect forwards positionally
        ours_schema = str(ours._opoverload._schema).split("(", 1)[1]
        theirs_schema = str(their_op._opoverload._schema).split("(", 1)[1]
        assert ours_schema == theirs_schema, (op_name, ours_schema, theirs_schema)


def test_a_cpu_tensor_still_has_no_fallback_after_the_redirect():
    installers.register_with_reference()
    gemv = importlib.import_module("deltaforge.kernels.tiled_gemv").tiled_gemv_int4
    x = torch.zeros((1, 1, 256), dtype=torch.bfloat16)
    packed = torch.zeros((128, 8), dtype=torch.uint8)
    scale = torch.ones((2, 8))
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        gemv(x, packed, scale, 128)
