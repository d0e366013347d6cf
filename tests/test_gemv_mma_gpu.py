"""The one-row int4 GEMV on the integer tensor-core instruction (``mma.sync m16n8k32``), through the C ABI.

Same checks as the other GEMV kernels get: against the CPU oracle's expression and the fp64 product at every
projection shape of the 4B model (ragged last tile, shards of a tensor-parallel rank included), both scale dtypes,
every fused prologue and epilogue, and bit-stable from run to run. The activation is held as 15-bit block integers
here (16-bit in the dp4a kernels), so the two kernel families agree to within last-bit flips of the bf16 output.
"""

from __future__ import annotations

import pytest
import torch

from deltaforge_b200 import ops
from oracle import ref_ops as R

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def problem(k, n, seed, scale_dtype):
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(seed), dtype=torch.uint8)
    scale = (torch.randn((k // 128, n), generator=gen(seed + 1)).abs() * 0.02 + 1e-4).to(scale_dtype)
    x = torch.randn((1, k), generator=gen(seed + 2)).to(BF16)
    return packed, scale, x


SHAPES = [(2560, 12352), (2560, 10240), (2560, 18432), (4096, 2560), (9216, 2560), (512, 2560), (2560, 1544), (256, 264)]


@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("scale_dtype", [torch.float32, BF16])
def test_mma_gemv_against_oracle_and_fp64(k, n, scale_dtype):
    packed, scale, x = problem(k, n, 7 * k + n, scale_dtype)
    pd, sd, xd = packed.to(DEV), scale.to(DEV), x.to(DEV)
    pm = ops.int4_repack_mma(pd, sd)
    got = ops.int4_gemv_fused(xd, pd, sd, 128, packed_mma=pm).cpu()
    want = R.dequant_gemv_int4(x, packed, scale, 128)
    q = R.unpack_int4_k_major(packed).double().reshape(k // 128, 128, n) * scale.double().unsqueeze(1)
    truth = x.double() @ q.reshape(k, n)
    rms = truth.pow(2).mean().sqrt().item()
    err = (got.double() - truth).abs()
    assert bool((err <= 2e-2 * truth.abs() + 2e-2 * truth.abs().mean()).all())
    assert bool(((got.float() - want.float()).abs() <= 2e-2 * want.float().abs() + 2e-2 * truth.abs().mean().item()).all())
    assert (err.pow(2).mean().sqrt() / rms).item() < 2.4e-3  # bf16 output rounding alone is 1.7e-3
    # the dp4a kernel on the k8 copy computes the same exact group sums from a 16-bit activation
    other = ops.int4_gemv_fused(xd, pd, sd, 128, packed_k8=ops.int4_repack_k8(pd)).cpu()
    assert (got.float() - other.float()).abs().max().item() <= 2**-7 * other.float().abs().max().item()
    assert (got != other).float().mean().item() < 0.1
    for key, buf in ops._scratch.items():  # the status word at the end of the scratch stays zero
        if key[1] == "gemv":
            assert int(buf[-256:-252].view(torch.int32).item()) == 0


def test_mma_gemv_prologues_and_epilogues():
    k, n = 2560, 2560
    packed, scale, _ = problem(k, n, 11, torch.float32)
    x = torch.randn((1, 1, k), generator=gen(3)).to(BF16)
    w = (torch.randn(k, generator=gen(4)) * 0.1).to(BF16)
    res = torch.randn((1, 1, n), generator=gen(5)).to(BF16)
    up = torch.randn((1, 1, k), generator=gen(6)).to(BF16)
    cache = torch.randn((1, 1024, 3), generator=gen(7)).to(BF16)
    taps = (torch.randn((1024, 4), generator=gen(8)) * 0.5).to(BF16).to(DEV)
    pd, sd = packed.to(DEV), scale.to(DEV)
    pm = ops.int4_repack_mma(pd, sd)
    for kw in (
        dict(prologue=ops.PRO_RMSNORM, norm_weight=w.to(DEV)),
        dict(epilogue=ops.EPI_RESIDUAL, residual=res.to(DEV)),
        dict(prologue=ops.PRO_SILU_MUL, up=up.to(DEV), epilogue=ops.EPI_RESIDUAL, residual=res.to(DEV)),
        dict(prologue=ops.PRO_RMSNORM, norm_weight=w.to(DEV), epilogue=ops.EPI_CONV, conv_weight=taps),
    ):
        ca, cb = cache.clone().to(DEV), cache.clone().to(DEV)
        extra_a = dict(conv_cache=ca) if kw.get("epilogue") == ops.EPI_CONV else {}
        extra_b = dict(conv_cache=cb) if kw.get("epilogue") == ops.EPI_CONV else {}
        a = ops.int4_gemv_fused(x.to(DEV), pd, sd, 128, force_tiled=True, **kw, **extra_a).float()
        b = ops.int4_gemv_fused(x.to(DEV), pd, sd, 128, packed_mma=pm, **kw, **extra_b).float()
        assert (a - b).abs().max().item() <= 2**-6 * a.abs().max().item()
        assert (a != b).float().mean().item() < 0.1
        if extra_a:
            assert torch.equal(ca[:, :, :2], cb[:, :, :2])  # the two older taps are copies; the newest is the GEMV's own output
            assert (ca[:, :, 2].float() - cb[:, :, 2].float()).abs().max().item() <= 2**-6 * ca[:, :, 2].float().abs().max().item()


def test_mma_gemv_wide_dynamic_range_and_determinism():
    k, n = 9216, 2560
    packed, scale, _ = problem(k, n, 21, BF16)
    x = torch.randn((1, k), generator=gen(3))
    x[0, ::97] *= 300.0  # outlier channels next to ordinary ones
    x[0, 5::61] *= 1e-3
    x = x.to(BF16)
    q = R.unpack_int4_k_major(packed).double().reshape(k // 128, 128, n) * scale.double().unsqueeze(1)
    truth = x.double() @ q.reshape(k, n)
    pd, sd, xd = packed.to(DEV), scale.to(DEV), x.to(DEV)
    pm = ops.int4_repack_mma(pd, sd)
    first = ops.int4_gemv_fused(xd, pd, sd, 128, packed_mma=pm)
    rms = truth.pow(2).mean().sqrt()
    assert ((first.double().cpu() - truth).pow(2).mean().sqrt() / rms).item() < 2.4e-3
    for _ in range(10):
        assert torch.equal(ops.int4_gemv_fused(xd, pd, sd, 128, packed_mma=pm), first)


def test_repack_rejects_what_the_layout_cannot_hold():
    packed = torch.zeros((32, 8), dtype=torch.uint8)
    with pytest.raises(ValueError):
        ops.int4_repack_mma(packed, torch.ones((1, 8)))  # K = 64 is not whole 128-row groups
    packed = torch.zeros((64, 8), dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        ops.int4_repack_mma(packed, torch.ones((1, 8)))  # CPU tensors
