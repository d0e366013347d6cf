"""dfb_int4_gemv_static: the split-K GEMV on the library's built-in device scratch.

Collected last (the file name sorts after the others) so that it also runs after every other GPU test has
used the device, and it must pass when run alone. Each case calls the existing entry point (caller
scratch) and the static one on the same inputs, the static one twice in a row, and wants identical bits:
both run the same kernel with the same fixed-order reduction.
"""

from __future__ import annotations

import ctypes as C

import pytest
import torch

from deltaforge_b200 import _lib
from deltaforge_b200._lib import GemvDesc
from deltaforge_b200.quant import quantise_int4_k_major

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16
PRO_RMSNORM, EPI_RESIDUAL, MATH_FAST, MATH_EXACT = 1, 1, 0, 1


def _problem(rows, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    qw = quantise_int4_k_major(torch.randn((n, k), generator=g) * 0.05)
    dev = torch.device("cuda", 0)
    return {
        "x": torch.randn((rows, k), generator=g).to(BF16).to(dev),
        "packed": qw.qweight.to(dev),
        "scale": qw.scale.to(dev),
        "norm_w": (torch.randn((k,), generator=g) * 0.1).to(BF16).to(dev),
        "residual": torch.randn((rows, n), generator=g).to(BF16).to(dev),
        "group": qw.group_size,
    }


def _desc(p, rows, k, n, out, math, fused):
    d = GemvDesc()
    d.x, d.x_stride, d.rows = p["x"].data_ptr(), k, rows
    d.packed, d.scale, d.scale_is_bf16 = p["packed"].data_ptr(), p["scale"].data_ptr(), 0
    d.K, d.N, d.group = k, n, p["group"]
    d.eps = 1e-6
    d.out, d.out_stride = out.data_ptr(), n
    d.math = math
    if fused:
        d.prologue, d.norm_w = PRO_RMSNORM, p["norm_w"].data_ptr()
        d.epilogue, d.residual, d.residual_stride = EPI_RESIDUAL, p["residual"].data_ptr(), n
    return d


def _run_existing(lib, p, rows, k, n, math, fused):
    out = torch.empty((rows, n), device="cuda:0", dtype=BF16)
    nbytes = lib.dfb_int4_gemv_scratch_bytes(rows, k, n, p["group"])
    scratch = torch.zeros(max(nbytes, 1), device="cuda:0", dtype=torch.uint8)
    d = _desc(p, rows, k, n, out, math, fused)
    d.scratch, d.scratch_bytes, d.force_tiled = scratch.data_ptr(), nbytes, 1
    _lib.check(lib.dfb_int4_gemv(C.byref(d), None), "dfb_int4_gemv")
    torch.cuda.synchronize()
    return out


def _run_static(lib, p, rows, k, n, math, fused):
    out = torch.full((rows, n), float("nan"), device="cuda:0", dtype=BF16)
    d = _desc(p, rows, k, n, out, math, fused)
    _lib.check(lib.dfb_int4_gemv_static(C.byref(d), None), "dfb_int4_gemv_static")
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize(
    "rows,k,n",
    [
        (1, 2560, 2048),   # one row, ten K slabs
        (1, 9216, 2560),   # the MLP down projection: 36 K slabs
        (1, 2560, 18432),  # the fused gate|up projection, the largest layer matrix (720 KiB of partials)
        (3, 2560, 520),    # ragged last column tile, two row blocks
        (8, 512, 264),     # four rows per CTA
        (1, 256, 512),     # a single K slab: no partial sums at all
    ],
)
@pytest.mark.parametrize("math", [MATH_FAST, MATH_EXACT])
@pytest.mark.parametrize("fused", [False, True])
def test_static_scratch_gemv_matches_caller_scratch_gemv(rows, k, n, math, fused):
    lib = _lib.load()
    p = _problem(rows, k, n, 1000 + rows + k + n)
    want = _run_existing(lib, p, rows, k, n, math, fused)
    first = _run_static(lib, p, rows, k, n, math, fused)
    second = _run_static(lib, p, rows, k, n, math, fused)
    assert not torch.isnan(first.float()).any()
    assert torch.equal(first, want)
    assert torch.equal(second, want)
    # and against the CPU oracle's expression for the same problem (rtol 2e-2 of the value, atol 2e-2 of the mean magnitude)
    from oracle import ref_ops as R

    x = p["x"].cpu()
    xin = R.rms_norm(x, p["norm_w"].cpu(), 1e-6) if fused else x
    ref = R.dequant_gemv_int4(xin, p["packed"].cpu(), p["scale"].cpu(), p["group"])
    if fused:
        ref = p["residual"].cpu() + ref
    err = (first.float().cpu() - ref.float()).abs()
    assert bool((err <= 2e-2 * ref.float().abs() + 2e-2 * ref.float().abs().mean()).all())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second CUDA device in this process")
def test_static_scratch_gemv_on_a_second_device_of_the_process():
    """Kernel attributes are per device: the first call on device 1 must set them there too (four rows per CTA
    take more dynamic shared memory than a kernel gets without the opt-in)."""
    lib = _lib.load()
    rows, k, n = 8, 2560, 1024
    p0 = _problem(rows, k, n, 77)
    want = _run_static(lib, p0, rows, k, n, MATH_FAST, False).cpu()
    dev1 = torch.device("cuda", 1)
    p1 = {key: (v.to(dev1) if torch.is_tensor(v) else v) for key, v in p0.items()}
    with torch.cuda.device(dev1):
        out = torch.full((rows, n), float("nan"), device=dev1, dtype=BF16)
        d = _desc(p1, rows, k, n, out, MATH_FAST, False)
        _lib.check(lib.dfb_int4_gemv_static(C.byref(d), None), "dfb_int4_gemv_static")
        torch.cuda.synchronize(dev1)
    assert torch.equal(out.cpu(), want)


def test_static_scratch_gemv_alternating_sizes():
    """Back-to-back calls of different shapes share the one array: each clears what it needs."""
    lib = _lib.load()
    shapes = [(1, 9216, 2560), (3, 2560, 520), (1, 2560, 18432), (1, 9216, 2560)]
    for i, (rows, k, n) in enumerate(shapes):
        p = _problem(rows, k, n, 2000 + i)
        want = _run_existing(lib, p, rows, k, n, MATH_FAST, True)
        assert torch.equal(_run_static(lib, p, rows, k, n, MATH_FAST, True), want)


def test_static_scratch_gemv_refuses_what_does_not_fit():
    lib = _lib.load()
    limit = lib.dfb_int4_gemv_static_max_partials_bytes()
    assert limit == 2 << 20
    # the LM head at one row needs 10 * 248320 * 4 bytes of partial sums
    rows, k, n = 1, 2560, 248320
    assert rows * (k // 256) * n * 4 > limit
    out = torch.empty((rows, 8), device="cuda:0", dtype=BF16)  # never written: the call is refused
    dummy = torch.zeros(16, device="cuda:0", dtype=torch.uint8)
    d = GemvDesc()
    d.x, d.x_stride, d.rows = dummy.data_ptr(), k, rows
    d.packed, d.scale = dummy.data_ptr(), dummy.data_ptr()
    d.K, d.N, d.group = k, n, 128
    d.out, d.out_stride = out.data_ptr(), n
    rc = lib.dfb_int4_gemv_static(C.byref(d), None)
    assert rc == 2
    msg = lib.dfb_last_error().decode()
    assert "built-in" in msg and str(limit) in msg
    # outside the group-128 layout there is no split-K scratch to replace
    d.K, d.N, d.group = 128, 96, 64
    assert lib.dfb_int4_gemv_static(C.byref(d), None) == 2
    assert "group-128" in lib.dfb_last_error().decode()
    torch.cuda.synchronize()
