"""Per-op parity of the CUDA kernels (through the C ABI) against the CPU oracle and the golden vectors.

Bars: int4 unpack and dequantised weights bit-exact; bf16 outputs of floating-point ops within
rtol 2e-2 / atol 2e-2 of the oracle (the reference's own layer-1 bar is 1e-2, the benchmark's north star asks 2e-2 against
an fp32 recompute) and, where stated, much tighter against an fp64 recompute.
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


def close(got: torch.Tensor, want: torch.Tensor, rtol=2e-2, atol=2e-2):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    assert bool((err <= bound).all()), f"max abs err {err.max().item():.4g}, worst excess {(err - bound).max().item():.4g}"


def rel_to_scale(got: torch.Tensor, truth: torch.Tensor) -> float:
    """max |got - truth| over the rms of truth: error in units of the output's own scale."""
    truth = truth.double().cpu()
    return ((got.double().cpu() - truth).abs().max() / truth.pow(2).mean().sqrt()).item()


def random_int4(k: int, n: int, seed: int, scale_dtype=torch.float32):
    packed = torch.randint(0, 256, (k // 2, n), generator=gen(seed), dtype=torch.uint8)
    group = R.group_size_for(k)
    scale = (torch.randn((k // group, n), generator=gen(seed + 1)).abs() * 0.02 + 1e-4).to(scale_dtype)
    return packed, scale, group


# ---------------------------------------------------------------- int4 unpack / dequant: bit-exact


@pytest.mark.parametrize("k,n", [(256, 48), (512, 1000), (64, 40), (2560, 2048), (9216, 264)])
def test_unpack_and_dequant_bit_exact(k, n):
    packed, scale, group = random_int4(k, n, 10 + k + n)
    assert torch.equal(ops.int4_unpack(packed.to(DEV)).cpu().to(torch.int16), R.unpack_int4_k_major(packed))
    want = R.dequantise_int4_k_major(packed, scale, group).to(BF16)
    assert torch.equal(ops.int4_dequant(packed.to(DEV), scale.to(DEV), group).cpu(), want)
    sb = scale.to(BF16)
    want_b = R.dequantise_int4_k_major(packed, sb, group).to(BF16)
    assert torch.equal(ops.int4_dequant(packed.to(DEV), sb.to(DEV), group).cpu(), want_b)


def test_dequant_matches_reference_golden(golden):
    g = golden("int4")
    for case in g["cases"] + [g["raw"]]:
        got = ops.int4_dequant(case["packed"].to(DEV), case["scale"].to(DEV), case["group"]).cpu()
        assert torch.equal(got, case["dense_fp32"].to(BF16))


def test_quantiser_roundtrip_on_device_matches_oracle():
    w = (torch.randn((96, 512), generator=gen(3)) * 0.02).to(BF16)
    packed, scale, group = R.quantise_int4_k_major(w)
    deq = ops.int4_dequant(packed.to(DEV), scale.to(DEV), group).cpu().float()
    # symmetric int4: every weight is within half a step of its dequantised value
    step = scale.repeat_interleave(group, dim=0)
    # (plus the bf16 rounding of the dequantised value itself, 2^-8 relative)
    assert bool(((deq - w.float().t()).abs() <= 0.5 * step * (1 + 1e-3) + deq.abs() * 2**-8).all())


@pytest.mark.parametrize("n,k", [(96, 512), (1000, 2560), (33, 9216), (40, 64), (8, 128), (520, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, BF16])
def test_cuda_quantiser_is_bit_identical_to_the_oracle(n, k, dtype):
    """``dfb_int4_quantise_k_major`` (behind ``quant.quantise_int4_k_major`` for CUDA weights) against the oracle's
    packer: bytes, scales and group size equal, including all-zero groups, ties at .5 and values beyond the clamp."""
    from deltaforge_b200.quant import quantise_int4_k_major

    w = torch.randn((n, k), generator=gen(n + k)) * 0.05
    w[0, : min(k, 128)] = 0.0  # a group that is all zero: scale 1
    w[1, :8] = torch.tensor([3.5, -3.5, 2.5, -2.5, 0.5, -0.5, 7.0, -7.0]) * (w[1].abs().max() / 7.0)  # ties of round-half-even
    w = w.to(dtype)
    packed, scale, group = R.quantise_int4_k_major(w)
    got = quantise_int4_k_major(w.to(DEV))
    assert got.group_size == group
    assert torch.equal(got.scale.cpu(), scale)
    assert torch.equal(got.qweight.cpu(), packed)
    host = quantise_int4_k_major(w)  # the torch form of the same arithmetic, on the CPU
    assert torch.equal(host.qweight, packed) and torch.equal(host.scale, scale)


def test_cuda_quantiser_matches_reference_golden(golden):
    from deltaforge_b200.quant import quantise_int4_k_major

    g = golden("int4")
    for case in g["cases"]:
        got = quantise_int4_k_major(case["weight"].to(DEV))
        assert torch.equal(got.qweight.cpu(), case["packed"]) and torch.equal(got.scale.cpu(), case["scale"])


# ---------------------------------------------------------------- int4 GEMV


GEMV_SHAPES = [
    # (rows, K, N) — fast path (group 128) and generic path (toy widths), ragged N, multi-row
    (1, 2560, 2048),
    (1, 2560, 12352),
    (1, 4096, 2560),
    (1, 9216, 2560),
    (1, 256, 8),
    (1, 512, 1000),
    (3, 2560, 520),
    (32, 512, 264),
    (1, 128, 96),
    (2, 64, 40),
    (5, 768, 33),
]


@pytest.mark.parametrize("rows", [1, 4])
@pytest.mark.parametrize("math", [ops.MATH_FAST, ops.MATH_FAST_HALF2])
def test_gemv_with_activations_beyond_the_fp16_range(rows, math):
    """Activations of a few 1e5 (the SwiGLU output of a real checkpoint has such channels): the kernels that hold the
    activation as fp16 scale a group down by a power of two first, so the result stays finite and as close to the
    exact product as with ordinary activations; a group of ordinary size next to it is untouched."""
    k, n = 2560, 1024
    packed, scale, group = random_int4(k, n, 4242)
    x = torch.randn((rows, 1, k), generator=gen(5))
    x[..., 256:384] *= 2.0e5  # one scale group far beyond 65504
    x[..., 1300] = -9.0e4     # and a single channel in another
    x = x.to(BF16)
    truth = R.dequant_gemv_int4_fp32(x, packed, scale, group).reshape(rows, 1, n)
    got = ops.int4_gemv_fused(x.to(DEV), packed.to(DEV), scale.to(DEV), group, math=math)
    assert bool(torch.isfinite(got.float()).all())
    err = (got.double().cpu() - truth).abs()
    rms = truth.pow(2).mean().sqrt()
    # (one group dominates every output, so outputs of four or five times the rms occur: the bf16 rounding of the result
    # alone is half a step of 2^-8 of those)
    assert (err.max() / rms).item() < 4e-2
    assert (err.pow(2).mean().sqrt() / rms).item() < 4e-3


@pytest.mark.parametrize("rows,k,n", GEMV_SHAPES)
@pytest.mark.parametrize("math", [ops.MATH_FAST, ops.MATH_EXACT, ops.MATH_FAST_HALF2])
def test_gemv_against_oracle(rows, k, n, math):
    packed, scale, group = random_int4(k, n, 100 + rows + k + n)
    x = torch.randn((rows, 1, k), generator=gen(7 + k)).to(BF16)
    want = R.dequant_gemv_int4(x, packed, scale, group)
    truth = R.dequant_gemv_int4_fp32(x, packed, scale, group).reshape(rows, 1, n)
    got = ops.int4_gemv_fused(x.to(DEV), packed.to(DEV), scale.to(DEV), group, math=math)
    assert got.shape == want.shape and got.dtype == BF16
    sc = truth.abs().mean().item()
    close(got, truth, rtol=2e-2, atol=2e-2 * sc)
    close(got, want, rtol=2e-2, atol=2e-2 * sc)
    # In units of the output's rms. The oracle's own bf16 output rounding sits at about 1.7e-3 rms
    # error and 1.5e-2 max; FAST skips the bf16 rounding of the weights, which moves it to 2.4e-3.
    err = (got.double().cpu() - truth).abs()
    rms = truth.pow(2).mean().sqrt()
    assert (err.max() / rms).item() < 2.5e-2
    # (a handful of outputs is too small a sample for the rms figure: twice the bar there)
    few = 2.0 if rows * n < 1000 else 1.0
    assert (err.pow(2).mean().sqrt() / rms).item() < few * (2.2e-3 if math == ops.MATH_EXACT else 3e-3)
    if math == ops.MATH_EXACT:
        # same products, fp32 accumulation in another order: the bf16 results are the oracle's
        assert (got.cpu() != want).sum().item() <= max(1, int(0.005 * rows * n))
    elif k % 256 == 0 and n % 8 == 0 and rows * n >= 1000:
        # (shapes outside the group-128 fast path run the generic kernel, which always rounds weights)
        # against the exact product with unrounded weights FAST is as accurate as the oracle is
        # against its own definition
        q = R.unpack_int4_k_major(packed).double().reshape(k // group, group, n) * scale.double().unsqueeze(1)
        truth_unrounded = (x.reshape(rows, k).double() @ q.reshape(k, n)).reshape(rows, 1, n)
        err_u = (got.double().cpu() - truth_unrounded).abs()
        assert (err_u.pow(2).mean().sqrt() / rms).item() < 2.4e-3


def test_gemv_exact_mode_matches_reference_golden(golden):
    g = golden("int4")
    for case in g["cases"] + [g["raw"]]:
        x = case["x"]
        got = ops.int4_gemv_fused(x.to(DEV), case["packed"].to(DEV), case["scale"].to(DEV), case["group"], math=ops.MATH_EXACT)
        close(got, case["y"].reshape(got.shape), rtol=1e-2, atol=1e-2 * case["y"].float().abs().mean().item())


def test_gemv_bf16_scales():
    packed, scale, group = random_int4(2560, 1024, 55, scale_dtype=BF16)
    x = torch.randn((1, 2560), generator=gen(56)).to(BF16)
    truth = R.dequant_gemv_int4_fp32(x, packed, scale, group)
    got = ops.tiled_gemv_int4(x.to(DEV), packed.to(DEV), scale.to(DEV), group)
    assert rel_to_scale(got, truth) < 2.5e-2


def test_gemv_is_deterministic_and_scratch_is_reusable():
    packed, scale, group = random_int4(4096, 2560, 77)
    x = torch.randn((1, 4096), generator=gen(78)).to(BF16).to(DEV)
    p, s = packed.to(DEV), scale.to(DEV)
    first = ops.tiled_gemv_int4(x, p, s, group)
    for _ in range(5):
        assert torch.equal(ops.tiled_gemv_int4(x, p, s, group), first)


def test_rmsnorm_prologue_and_residual_epilogue():
    k, n = 2560, 2560
    packed, scale, group = random_int4(k, n, 200)
    x = torch.randn((2, 1, k), generator=gen(201)).to(BF16)
    w = (torch.randn(k, generator=gen(202)) * 0.1).to(BF16)
    res = torch.randn((2, 1, n), generator=gen(203)).to(BF16)
    normed = R.rms_norm(x, w, 1e-6)
    want = R.dequant_gemv_int4(normed, packed, scale, group)
    got = ops.rmsnorm_int4_gemv(x.to(DEV), w.to(DEV), 1e-6, packed.to(DEV), scale.to(DEV), group)
    sc = want.float().abs().mean().item()
    close(got, want, rtol=2e-2, atol=2e-2 * sc)
    want_r = res + R.dequant_gemv_int4(x, packed, scale, group)
    got_r = ops.int4_gemv_residual(x.to(DEV), packed.to(DEV), scale.to(DEV), group, res.to(DEV))
    close(got_r, want_r, rtol=2e-2, atol=2e-2 * sc)


def test_silu_mul_prologue():
    k, n = 9216, 2560
    packed, scale, group = random_int4(k, n, 210)
    gate = torch.randn((1, 1, k), generator=gen(211)).to(BF16)
    up = torch.randn((1, 1, k), generator=gen(212)).to(BF16)
    res = torch.randn((1, 1, n), generator=gen(213)).to(BF16)
    want = res + R.dequant_gemv_int4(R.silu_mul(gate, up), packed, scale, group)
    got = ops.silu_mul_int4_gemv_residual(gate.to(DEV), up.to(DEV), packed.to(DEV), scale.to(DEV), group, res.to(DEV))
    close(got, want, rtol=2e-2, atol=2e-2 * want.float().abs().mean().item())


def test_conv_epilogue_matches_conv_step():
    k, n, c = 2560, 1024 + 64, 1024
    packed, scale, group = random_int4(k, n, 220)
    x = torch.randn((2, 1, k), generator=gen(221)).to(BF16)
    w = (torch.randn(k, generator=gen(222)) * 0.1).to(BF16)
    cache = torch.randn((2, c, 3), generator=gen(223)).to(BF16)
    taps = (torch.randn((c, 1, 4), generator=gen(224)) * 0.5).to(BF16)
    dev_cache = cache.clone().to(DEV)
    got = ops.rmsnorm_int4_gemv_conv(x.to(DEV), w.to(DEV), 1e-6, packed.to(DEV), scale.to(DEV), group, dev_cache, taps.to(DEV))
    # feed the oracle's conv with the kernel's own projection so only the conv arithmetic is compared
    plain = ops.rmsnorm_int4_gemv(x.to(DEV), w.to(DEV), 1e-6, packed.to(DEV), scale.to(DEV), group).cpu()
    ref_cache = cache.clone()
    want_conv = R.causal_conv_step(plain[:, 0, :c].unsqueeze(-1), ref_cache, taps)[..., 0]
    close(got[:, 0, :c], want_conv, rtol=1e-2, atol=1e-2)
    assert torch.equal(got[:, 0, c:].cpu(), plain[:, 0, c:])
    assert torch.equal(dev_cache.cpu(), ref_cache)


def test_gemv_errors_come_before_the_device_check():
    packed, scale, group = random_int4(256, 16, 1)
    x = torch.zeros((1, 128), dtype=BF16)
    with pytest.raises(ValueError):
        ops.tiled_gemv_int4(x, packed, scale, group)  # wrong K, CPU tensors: shape error wins
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        ops.tiled_gemv_int4(torch.zeros((1, 256), dtype=BF16), packed, scale, group)
    assert ops.tiled_gemv_int4(torch.zeros((0, 256), dtype=BF16, device=DEV), packed.to(DEV), scale.to(DEV), group).shape == (0, 16)


# ---------------------------------------------------------------- elementwise


def test_elementwise_against_golden(golden):
    g = golden("elementwise")
    r = g["rms"]
    close(ops.rms_norm(r["x"].to(DEV), r["w"].to(DEV), r["eps"]), r["y"], rtol=1e-2, atol=1e-2)
    rp = g["rope"]
    assert torch.equal(ops.partial_rope(rp["x"].to(DEV), rp["cos"].to(DEV), rp["sin"].to(DEV)).cpu(), rp["y"])
    s = g["swiglu"]
    close(ops.silu_mul(s["gate"].to(DEV), s["up"].to(DEV)), s["y"], rtol=1e-2, atol=1e-2)
    rs = g["residual"]
    summed, normed = ops.add_rms_norm(rs["b"].to(DEV), rs["a"].to(DEV), r["w"].to(DEV), 1e-6)
    assert torch.equal(summed.cpu(), rs["sum"])
    close(normed, R.rms_norm(rs["sum"], r["w"], 1e-6), rtol=1e-2, atol=1e-2)


def test_rms_norm_wide_row_is_nearly_exact():
    x = torch.randn((4, 2560), generator=gen(300)).to(BF16)
    w = (torch.randn(2560, generator=gen(301)) * 0.1).to(BF16)
    got = ops.rms_norm(x.to(DEV), w.to(DEV), 1e-6).cpu()
    want = R.rms_norm(x, w, 1e-6)
    assert (got != want).float().mean().item() < 2e-3  # only reduction-order flips of the last bf16 bit


def test_conv_step_bit_exact(golden):
    c = golden("deltanet")["conv"]
    cache = c["cache"].clone().to(DEV)
    got = ops.fused_causal_conv_step(c["x"].to(DEV), cache, c["w"].to(DEV))
    assert torch.equal(cache.cpu(), c["cache_after"])
    close(got, c["y"], rtol=1e-2, atol=1e-2)
    assert (got.cpu() != c["y"]).float().mean().item() < 0.02
    with pytest.raises(ValueError):
        ops.fused_causal_conv_step(torch.zeros((1, 4, 2), dtype=BF16), torch.zeros((1, 4, 3), dtype=BF16), torch.zeros((4, 1, 4), dtype=BF16))


# ---------------------------------------------------------------- DeltaNet


@pytest.mark.parametrize("batch,heads,dk,dv", [(1, 32, 128, 128), (2, 4, 16, 16), (3, 8, 128, 64), (1, 2, 64, 200)])
def test_delta_rule_step(batch, heads, dk, dv):
    s0 = torch.randn((batch, heads, dk, dv), generator=gen(400)) * 0.1
    q = R.l2norm(torch.randn((batch, heads, dk), generator=gen(401))) / dk**0.5
    k = R.l2norm(torch.randn((batch, heads, dk), generator=gen(402)))
    v = torch.randn((batch, heads, dv), generator=gen(403))
    g = -torch.rand((batch, heads), generator=gen(404))
    beta = torch.rand((batch, heads), generator=gen(405))
    want_o, want_s = R.delta_rule_step(s0, q, k, v, g, beta)
    got_o, got_s = ops.delta_rule_step(*(t.to(DEV) for t in (s0, q, k, v, g, beta)))
    assert got_s.dtype == torch.float32
    assert (got_o.cpu() - want_o).abs().max().item() < 2e-5
    assert (got_s.cpu() - want_s).abs().max().item() < 2e-5


def test_delta_rule_golden_sequence(golden):
    r = golden("deltanet")["rule"]
    q, k, v, beta, g = (t.transpose(1, 2).float().contiguous() for t in (r["q"], r["k"], r["v"], r["beta"], r["g"]))
    q = R.l2norm(q) / q.shape[-1] ** 0.5
    k = R.l2norm(k)
    state = r["state"].to(DEV)
    outs = []
    for t in range(q.shape[2]):
        o, state = ops.delta_rule_step(state, q[:, :, t].to(DEV), k[:, :, t].to(DEV), v[:, :, t].to(DEV), g[:, :, t].to(DEV), beta[:, :, t].to(DEV))
        outs.append(o.cpu())
    assert (state.cpu() - r["state_after"]).abs().max().item() < 1e-5
    got = torch.stack(outs, dim=1)  # (B, T, H, dv)
    close(got, r["out"].float(), rtol=1e-2, atol=1e-2)


def test_delta_rule_rejects_bf16_state():
    z = torch.zeros
    with pytest.raises(ValueError, match="fp32"):
        ops.delta_rule_step(z((1, 1, 4, 4), dtype=BF16), z((1, 1, 4)), z((1, 1, 4)), z((1, 1, 4)), z((1, 1)), z((1, 1)))


@pytest.mark.parametrize(
    "batch,hk,hv,dk,dv,wdtype",
    [
        (1, 16, 32, 128, 128, BF16), (2, 2, 4, 16, 16, BF16), (1, 16, 32, 128, 128, torch.float32),
        # four sequences and more: the one-CTA-per-head kernel
        (4, 16, 32, 128, 128, BF16), (5, 2, 4, 16, 16, BF16), (4, 4, 8, 64, 96, torch.float32),
    ],
)  # fmt: skip
def test_deltanet_step_against_oracle(batch, hk, hv, dk, dv, wdtype):
    q = torch.randn((batch, hk, dk), generator=gen(500)).to(BF16)
    k = torch.randn((batch, hk, dk), generator=gen(501)).to(BF16)
    v = torch.randn((batch, hv, dv), generator=gen(502)).to(BF16)
    z = torch.randn((batch, hv, dv), generator=gen(503)).to(BF16)
    b = torch.randn((batch, hv), generator=gen(504)).to(BF16)
    a = torch.randn((batch, hv), generator=gen(505)).to(BF16)
    a_log = torch.log(torch.rand(hv, generator=gen(506)) * 16 + 1e-3).to(BF16)
    dt_bias = (torch.randn(hv, generator=gen(507)) * 0.1).to(BF16)
    nw = (1.0 + 0.1 * torch.randn(dv, generator=gen(508))).to(wdtype)
    s0 = torch.randn((batch, hv, dk, dv), generator=gen(509)) * 0.1
    # oracle: the reference's sequence of calls (reference.py:528-549) at seq_len 1
    g, beta = R.delta_gates(a.unsqueeze(1), b.unsqueeze(1), a_log, dt_bias)
    rep = hv // hk
    core, s1 = R.gated_delta_rule(
        q.unsqueeze(1).repeat_interleave(rep, dim=2), k.unsqueeze(1).repeat_interleave(rep, dim=2), v.unsqueeze(1), g, beta, s0
    )
    want = R.gated_rms_norm(core.reshape(-1, dv), z.reshape(-1, dv), nw, 1e-6).reshape(batch, hv * dv)
    state = s0.clone().to(DEV)
    got = ops.deltanet_step(*(t.to(DEV) for t in (q, k, v, z, b, a, a_log, dt_bias, nw)), 1e-6, state)
    assert (state.cpu() - s1).abs().max().item() < 5e-5
    close(got, want, rtol=2e-2, atol=2e-2)
    assert (got.cpu().float() - want.float()).abs().mean().item() < 2e-3


# ---------------------------------------------------------------- attention


ATTN_CASES = [(1, 16, 4, 2048, 256), (2, 16, 4, 33, 256), (1, 16, 4, 1, 256), (1, 16, 4, 3, 256), (1, 4, 1, 130, 256), (2, 4, 1, 33, 32), (1, 8, 2, 5, 64)]


@pytest.mark.parametrize("batch,hq,hkv,length,d", ATTN_CASES)
@pytest.mark.parametrize("splits", [1, 8, 64])
def test_attention_against_oracle(batch, hq, hkv, length, d, splits):
    q = torch.randn((batch, hq, d), generator=gen(600)).to(BF16)
    k = torch.randn((batch, hkv, length, d), generator=gen(601)).to(BF16)
    v = torch.randn((batch, hkv, length, d), generator=gen(602)).to(BF16)
    scale = d**-0.5
    truth = R.decode_attention_fp64(q, k, v, scale)
    want = R.decode_attention(q, k, v, scale)
    if splits == 1:
        got = ops.gqa_decode_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale)
    else:
        got = ops.split_kv_decode_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, splits)
    assert (got.cpu().double() - truth).abs().max().item() < 8e-3  # bf16 output rounding of O(1) values
    close(got, want, rtol=2e-2, atol=2e-2)


# many sequences or a long cache: the tensor-core kernel (16-key tiles through a ring, mma.sync)
ATTN_MMA_CASES = [
    (2, 16, 4, 1100, 1), (2, 16, 4, 1100, 8), (3, 8, 2, 4099, 8), (1, 16, 4, 20000, 64), (2, 8, 1, 700, 1),
    (2, 4, 4, 300, 1), (2, 4, 2, 515, 2), (4, 16, 4, 129, 1),
]  # fmt: skip


@pytest.mark.parametrize("batch,hq,hkv,length,splits", ATTN_MMA_CASES)
def test_attention_tensor_core_path_against_oracle(batch, hq, hkv, length, splits):
    d = 256
    q = torch.randn((batch, hq, d), generator=gen(610)).to(BF16)
    k = torch.randn((batch, hkv, length, d), generator=gen(611)).to(BF16)
    v = torch.randn((batch, hkv, length, d), generator=gen(612)).to(BF16)
    scale = d**-0.5
    truth = R.decode_attention_fp64(q, k, v, scale)
    want = R.decode_attention(q, k, v, scale)
    if splits == 1:
        got = ops.gqa_decode_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale)
    else:
        got = ops.split_kv_decode_attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, splits)
    assert torch.isfinite(got.float()).all()
    assert (got.cpu().double() - truth).abs().max().item() < 8e-3
    close(got, want, rtol=2e-2, atol=2e-2)


def test_attention_golden(golden):
    for case in golden("attention")["cases"]:
        got = ops.split_kv_decode_attention(case["q"].to(DEV), case["k"].to(DEV), case["v"].to(DEV), case["scale"], 8)
        close(got, case["y"], rtol=2e-2, atol=2e-2)


def test_attention_on_a_cache_view_and_with_gate():
    b, hq, hkv, d, max_seq, length = 2, 16, 4, 256, 300, 77
    kc = torch.randn((b, hkv, max_seq, d), generator=gen(610)).to(BF16).to(DEV)
    vc = torch.randn((b, hkv, max_seq, d), generator=gen(611)).to(BF16).to(DEV)
    q = torch.randn((b, hq, d), generator=gen(612)).to(BF16)
    gate = torch.randn((b, hq, d), generator=gen(613)).to(BF16)
    got = ops.attn_decode_gated(q.to(DEV), kc[:, :, :length], vc[:, :, :length], d**-0.5, 16, gate.to(DEV), False)
    want = R.decode_attention(q, kc[:, :, :length].cpu(), vc[:, :, :length].cpu(), d**-0.5) * R.output_gate(gate)
    close(got, want, rtol=2e-2, atol=2e-2)


def test_attention_errors():
    q = torch.zeros((1, 16, 256), dtype=BF16)
    kv = torch.zeros((1, 4, 8, 256), dtype=BF16)
    with pytest.raises(ValueError, match="power of two"):
        ops.split_kv_decode_attention(q, kv, kv, 1.0, 3)
    with pytest.raises(ValueError, match="empty"):
        ops.gqa_decode_attention(q, kv[:, :, :0], kv[:, :, :0], 1.0)
    with pytest.raises(ValueError, match="divide"):
        ops.gqa_decode_attention(torch.zeros((1, 6, 256), dtype=BF16), kv, kv, 1.0)
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        ops.gqa_decode_attention(q, kv, kv, 1.0)


def test_attn_prep_against_oracle():
    b, hq, hkv, d, rd, max_seq, position = 2, 16, 4, 256, 64, 64, 37
    width = hq * 2 * d + 2 * hkv * d
    proj = torch.randn((b, width), generator=gen(700)).to(BF16)
    qw = (torch.randn(d, generator=gen(701)) * 0.1).to(BF16)
    kw = (torch.randn(d, generator=gen(702)) * 0.1).to(BF16)
    inv_freq = R.rope_inv_freq(rd, 1e7).to(BF16).float()  # as a bf16 model holds it
    kc = torch.zeros((b, hkv, max_seq, d), dtype=BF16, device=DEV)
    vc = torch.zeros_like(kc)
    pos = torch.tensor([position], dtype=torch.int32, device=DEV)
    q_out = ops.attn_prep(proj.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, inv_freq.to(DEV), pos, kc, vc, hq, True)
    # oracle, following reference.py:621-650
    pq = proj[:, : hq * 2 * d].view(b, 1, hq, 2 * d)
    query = pq[..., :d]
    key = proj[:, hq * 2 * d : hq * 2 * d + hkv * d].view(b, 1, hkv, d)
    value = proj[:, hq * 2 * d + hkv * d :].view(b, 1, hkv, d)
    cos, sin = R.rope_cos_sin(torch.full((b, 1), position), inv_freq, BF16)
    want_q = R.partial_rope(R.rms_norm(query, qw, 1e-6).transpose(1, 2), cos, sin)[:, :, 0]
    want_k = R.partial_rope(R.rms_norm(key, kw, 1e-6).transpose(1, 2), cos, sin)[:, :, 0]
    close(q_out, want_q, rtol=1e-2, atol=1e-2)
    close(kc[:, :, position], want_k, rtol=1e-2, atol=1e-2)
    assert torch.equal(vc[:, :, position].cpu(), value[:, 0])
    assert (q_out.cpu() != want_q).float().mean().item() < 0.01
    untouched = torch.ones(max_seq, dtype=torch.bool)
    untouched[position] = False
    assert not kc[:, :, untouched].any() and not vc[:, :, untouched].any()
