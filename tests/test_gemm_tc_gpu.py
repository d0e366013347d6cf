"""int4 x bf16 product for 8..128 activation rows on the tensor cores (tcgen05 + TMEM) against the oracle.

The kernel dequantises to exactly the bf16 weights of the reference expression, so the only difference
from the oracle is the order of the fp32 accumulation: outputs agree to the last bf16 step except for
rare ties.
"""

from __future__ import annotations

import pytest
import torch

from deltaforge_b200 import ops
from oracle import ref_ops as R

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def problem(rows, k, n, seed, scale_dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((n, k), generator=g) * 0.05
    packed, scale, group = R.quantise_int4_k_major(w)
    x = torch.randn((rows, k), generator=g).to(BF16)
    return x, packed, scale.to(scale_dtype), group


SHAPES = [
    # rows, K, N: one column tile, ragged last tile, split-K (few tiles), the wide MLP matrix, padded rows
    (8, 256, 128),
    (16, 512, 264),
    (32, 2560, 2048),
    (32, 4096, 2560),
    (32, 9216, 2560),
    (33, 2560, 12352),
    (64, 2560, 2560),
    (128, 1024, 520),
    (100, 2560, 18432),
]


@pytest.mark.parametrize("rows,k,n", SHAPES)
@pytest.mark.parametrize("scale_dtype", [torch.float32, BF16])
def test_tensor_core_product_matches_oracle(rows, k, n, scale_dtype):
    x, packed, scale, group = problem(rows, k, n, 500 + rows + k + n, scale_dtype)
    assert group == 128
    want = R.dequant_gemv_int4(x.unsqueeze(1), packed, scale.float(), group).reshape(rows, n)
    truth = R.dequant_gemv_int4_fp32(x.unsqueeze(1), packed, scale.float(), group).reshape(rows, n)
    pk = packed.to(DEV)
    k8 = ops.int4_repack_k8(pk)
    got = ops.int4_gemv_fused(x.to(DEV), pk, scale.to(DEV), group, packed_k8=k8).cpu()
    assert got.shape == (rows, n) and got.dtype == BF16
    assert torch.isfinite(got.float()).all()
    rms = truth.pow(2).mean().sqrt().item()
    err = (got.double() - truth).abs()
    # the oracle's own bf16 output rounding is 1.7e-3 rms / 1.5e-2 max in these units
    assert (err.max() / rms).item() < 2.5e-2
    assert (err.pow(2).mean().sqrt() / rms).item() < 2.2e-3
    # same bf16 weights, same fp32 products, another summation order: all but a few outputs are the oracle's
    assert (got != want).float().mean().item() < 0.01


def test_tensor_core_product_with_residual_and_repeat():
    rows, k, n = 32, 4096, 2560
    x, packed, scale, group = problem(rows, k, n, 77)
    res = torch.randn((rows, n), generator=torch.Generator().manual_seed(3)).to(BF16)
    y = R.dequant_gemv_int4(x.unsqueeze(1), packed, scale, group).reshape(rows, n)
    want = (res.float() + y.float()).to(BF16)
    pk = packed.to(DEV)
    k8 = ops.int4_repack_k8(pk)
    outs = [
        ops.int4_gemv_fused(x.to(DEV), pk, scale.to(DEV), group, epilogue=ops.EPI_RESIDUAL, residual=res.to(DEV), packed_k8=k8).cpu()
        for _ in range(3)
    ]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])  # fixed split order: repeatable
    assert (outs[0] != want).float().mean().item() < 0.01
    assert (outs[0].float() - want.float()).abs().max().item() < 0.05 * want.float().abs().max().item()
