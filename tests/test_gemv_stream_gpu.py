"""The streaming (TMA ring, persistent CTAs, integer dot products) int4 GEMV against the register-tiled
kernel and the oracle, and the bit-exactness of the re-packed weight layout it reads.

Both kernels compute the FAST arithmetic (per-group sums of x * value, fp32 scale applied once per
group; the dequantised weight is not rounded to bf16). The streaming kernel additionally holds the
activation as 16-bit integers with one exponent per 128-row group, which is exact for every element
within 2^-7 of the group's largest. Shapes cover every projection of the benchmark model, ragged
tiles and both unit heights.
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


SHAPES = [
    (2560, 12352),  # DeltaNet in_proj qkv|z|b|a (ragged last tile)
    (2560, 10240),  # attention q|k|v
    (2560, 18432),  # gate|up
    (9216, 2560),  # down
    (4096, 2560),  # out_proj / o_proj
    (2560, 248320),  # LM head
    (256, 16),  # one group, one sliver of a tile
    (512, 144),
    (2560, 36),
]


@pytest.mark.parametrize("k,n", [(256, 16), (512, 144), (2560, 1000), (9216, 264)])
def test_repack_keeps_every_nibble(k, n):
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(k + n), dtype=torch.uint8)
    words = ops.int4_repack_k8(packed.to(DEV)).cpu()
    assert words.shape == (k // 8, n) and words.dtype == torch.int32
    want = R.unpack_int4_k_major(packed).to(torch.int64) + 8  # [K, N] nibbles 0..15
    w = words.to(torch.int64) & 0xFFFFFFFF
    for i in range(8):
        assert torch.equal((w >> (4 * i)) & 15, want[i::8])


@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("scale_dtype", [torch.float32, BF16])
def test_stream_matches_tiled_and_oracle(k, n, scale_dtype):
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(k + n), dtype=torch.uint8)
    scale = (torch.randn((k // 128, n), generator=gen(k + n + 1)).abs() * 0.02 + 1e-4).to(scale_dtype)
    x = torch.randn((1, k), generator=gen(5)).to(BF16)
    xd, pd, sd = x.to(DEV), packed.to(DEV), scale.to(DEV)
    k8 = ops.int4_repack_k8(pd)
    tiled = ops.int4_gemv_fused(xd, pd, sd, 128, force_tiled=True).float().cpu()
    stream = ops.int4_gemv_fused(xd, pd, sd, 128, packed_k8=k8).float().cpu()
    rms = tiled.pow(2).mean().sqrt().item()
    # same sums up to fp32 rounding and the 2^-16 tail of the integer activations: last-bit flips only
    assert (tiled - stream).abs().max().item() <= 2**-7 * tiled.abs().max().item()
    assert ((tiled != stream).float().mean().item()) < 0.1
    if 1000 <= n <= 20000:  # enough outputs for an rms statistic, small enough for the CPU product
        q = R.unpack_int4_k_major(packed).double().reshape(k // 128, 128, n) * scale.double().unsqueeze(1)
        truth = x.double() @ q.reshape(k, n)
        err = (stream.double() - truth).abs()
        assert (err.pow(2).mean().sqrt() / max(rms, 1e-9)).item() < 2.4e-3  # bf16 output rounding alone is 1.7e-3
    for key, buf in ops._scratch.items():  # the status word at the end of the scratch stays zero
        if key[1] == "gemv":
            assert int(buf[-256:-252].view(torch.int32).item()) == 0


def test_stream_handles_wide_dynamic_range_inside_a_group():
    k, n = 2560, 2048
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(1), dtype=torch.uint8)
    scale = torch.randn((k // 128, n), generator=gen(2)).abs() * 0.02 + 1e-4
    x = torch.randn((1, k), generator=gen(3))
    x[0, ::97] *= 300.0  # outlier channels next to ordinary ones
    x[0, 5::61] *= 1e-3
    x = x.to(BF16)
    q = R.unpack_int4_k_major(packed).double().reshape(k // 128, 128, n) * scale.double().unsqueeze(1)
    truth = x.double() @ q.reshape(k, n)
    pd = packed.to(DEV)
    got = ops.int4_gemv_fused(x.to(DEV), pd, scale.to(DEV), 128, packed_k8=ops.int4_repack_k8(pd)).double().cpu()
    rms = truth.pow(2).mean().sqrt()
    assert ((got - truth).pow(2).mean().sqrt() / rms).item() < 2.4e-3


def test_stream_with_prologues_and_epilogues():
    k, n = 2560, 2560
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(1), dtype=torch.uint8)
    scale = torch.randn((k // 128, n), generator=gen(2)).abs() * 0.02 + 1e-4
    x = torch.randn((1, 1, k), generator=gen(3)).to(BF16)
    w = (torch.randn(k, generator=gen(4)) * 0.1).to(BF16)
    res = torch.randn((1, 1, n), generator=gen(5)).to(BF16)
    up = torch.randn((1, 1, k), generator=gen(6)).to(BF16)
    pd = packed.to(DEV)
    args = (pd, scale.to(DEV), 128)
    k8 = ops.int4_repack_k8(pd)
    cache = torch.randn((1, 1024, 3), generator=gen(7)).to(BF16)
    taps = (torch.randn((1024, 4), generator=gen(8)) * 0.5).to(BF16).to(DEV)
    for kw in (
        dict(prologue=ops.PRO_RMSNORM, norm_weight=w.to(DEV)),
        dict(epilogue=ops.EPI_RESIDUAL, residual=res.to(DEV)),
        dict(prologue=ops.PRO_SILU_MUL, up=up.to(DEV), epilogue=ops.EPI_RESIDUAL, residual=res.to(DEV)),
        dict(prologue=ops.PRO_RMSNORM, norm_weight=w.to(DEV), epilogue=ops.EPI_CONV, conv_weight=taps),
    ):
        ca, cb = cache.clone().to(DEV), cache.clone().to(DEV)
        extra_a = dict(conv_cache=ca) if kw.get("epilogue") == ops.EPI_CONV else {}
        extra_b = dict(conv_cache=cb) if kw.get("epilogue") == ops.EPI_CONV else {}
        a = ops.int4_gemv_fused(x.to(DEV), *args, force_tiled=True, **kw, **extra_a).float()
        b = ops.int4_gemv_fused(x.to(DEV), *args, packed_k8=k8, **kw, **extra_b).float()
        assert (a - b).abs().max().item() <= 2**-6 * a.abs().max().item()
        assert (a != b).float().mean().item() < 0.1


def test_stream_is_deterministic():
    k, n = 9216, 2560
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(7), dtype=torch.uint8).to(DEV)
    scale = (torch.randn((k // 128, n), generator=gen(8)).abs() * 0.02 + 1e-4).to(DEV)
    x = torch.randn((1, k), generator=gen(9)).to(BF16).to(DEV)
    k8 = ops.int4_repack_k8(packed)
    first = ops.int4_gemv_fused(x, packed, scale, 128, packed_k8=k8)
    for _ in range(10):
        assert torch.equal(ops.int4_gemv_fused(x, packed, scale, 128, packed_k8=k8), first)
