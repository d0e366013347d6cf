"""Generate the golden vectors that pin ``oracle/`` to the real reference.

Run in a container that has the reference checked out:

    DELTAFORGE_REFERENCE_SRC=/path/to/deltaforge/src python tests/golden/make_golden.py

It imports LoveManna/deltaforge itself, feeds seeded inputs to the reference's own functions and
stores inputs and outputs as small ``.pt`` files beside this script. The reference cannot travel to
the GPU machines, these files can: the CPU suite checks ``oracle/`` against them bit for bit, the
GPU suite checks the CUDA path against them and against ``oracle/`` on fresh inputs.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REF_SRC = os.environ.get("DELTAFORGE_REFERENCE_SRC")
if not REF_SRC:
    raise SystemExit("set DELTAFORGE_REFERENCE_SRC to the `src` directory of a LoveManna/deltaforge checkout")
sys.path.insert(0, REF_SRC)

from deltaforge import reference as ref  # noqa: E402
from deltaforge.config import tiny_config  # noqa: E402
from deltaforge.kernels import gqa_decode, inline_causal_conv, tiled_gemv, visible_int4_head  # noqa: E402
from deltaforge.kernels.quantised_linear import group_size_for  # noqa: E402
from deltaforge.model import greedy_decode  # noqa: E402

BF16 = torch.bfloat16


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def save(name: str, payload: dict) -> None:
    torch.save(payload, HERE / f"{name}.pt")
    size = (HERE / f"{name}.pt").stat().st_size
    print(f"{name}.pt  {size / 1024:.1f} KiB")


def int4_vectors() -> None:
    cases = []
    for seed, (n, k, rows) in enumerate([(96, 512, 1), (40, 256, 3), (64, 64, 2), (8, 768, 1)]):
        w = (torch.randn((n, k), generator=gen(100 + seed)) * 0.02).to(BF16)
        qw = tiled_gemv.quantise_int4_k_major(w)
        dense = tiled_gemv.dequantise_int4_k_major(qw.qweight, qw.scale, group_size=qw.group_size)
        x = torch.randn((rows, 1, k), generator=gen(200 + seed)).to(BF16)
        y = visible_int4_head.torch_dequant_gemv_int4(x, qw.qweight, qw.scale, qw.group_size)
        cases.append(
            {"weight": w, "packed": qw.qweight, "scale": qw.scale, "group": qw.group_size, "dense_fp32": dense, "x": x, "y": y}
        )
    # Raw nibbles over the whole 0..15 range (the quantiser never emits 0, the dequantiser accepts it).
    packed = torch.randint(0, 256, (128, 48), generator=gen(300), dtype=torch.uint8)
    scale = torch.randn((2, 48), generator=gen(301)).abs() * 0.02
    dense = tiled_gemv.dequantise_int4_k_major(packed, scale, group_size=128)
    x = torch.randn((1, 256), generator=gen(302)).to(BF16)
    y = visible_int4_head.torch_dequant_gemv_int4(x, packed, scale, 128)
    raw = {"packed": packed, "scale": scale, "group": 128, "dense_fp32": dense, "x": x, "y": y}
    groups = {k: group_size_for(k) for k in (64, 256, 512, 2560, 4096, 9216, 128, 32)}
    save("int4", {"cases": cases, "raw": raw, "group_size_for": groups})


def elementwise_vectors() -> None:
    x = torch.randn((3, 1, 160), generator=gen(400)).to(BF16)
    w = (torch.randn(160, generator=gen(401)) * 0.1).to(BF16)
    norm = ref.RMSNorm(160)
    norm.weight.data = w.clone()
    rms = norm(x)
    gn = ref.GatedRMSNorm(32)
    gx = torch.randn((12, 32), generator=gen(402)).to(BF16)
    gz = torch.randn((12, 32), generator=gen(403)).to(BF16)
    gw32 = 1.0 + 0.1 * torch.randn(32, generator=gen(404))
    gn.weight.data = gw32.clone()
    gated_fp32w = gn(gx, gz)
    gn.weight.data = gw32.to(BF16)
    gated_bf16w = gn(gx, gz)
    pos = torch.tensor([[0, 1, 7, 4095, 100000]])
    cfg = tiny_config()
    rot = ref.RotaryEmbedding(cfg)
    cos, sin = rot(pos, BF16)
    xr = torch.randn((1, 2, 5, cfg.head_dim), generator=gen(405)).to(BF16)
    roped = ref.apply_partial_rope(xr, cos, sin)
    g = torch.randn((2, 1, 96), generator=gen(406)).to(BF16) * 3
    u = torch.randn((2, 1, 96), generator=gen(407)).to(BF16)
    swi = torch.nn.functional.silu(g) * u
    gate = torch.randn((2, 1, 64), generator=gen(408)).to(BF16) * 4
    save(
        "elementwise",
        {
            "rms": {"x": x, "w": w, "eps": 1e-6, "y": rms},
            "gated": {"x": gx, "z": gz, "w_fp32": gw32, "eps": 1e-6, "y_fp32w": gated_fp32w, "y_bf16w": gated_bf16w},
            "rope": {"pos": pos, "rotary_dim": cfg.rotary_dim, "theta": cfg.rope_theta, "cos": cos, "sin": sin, "x": xr, "y": roped},
            "rotate_half": {"x": torch.tensor([1.0, 2.0, 3.0, 4.0]), "y": ref.rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0]))},
            "swiglu": {"gate": g, "up": u, "y": swi},
            "outgate": {"gate": gate, "sigmoid": ref.apply_output_gate(gate, "sigmoid"), "swish": ref.apply_output_gate(gate, "swish")},
            "residual": {"a": x, "b": (x * 0.37).to(BF16), "sum": x + (x * 0.37).to(BF16)},
        },
    )


def deltanet_vectors() -> None:
    b, c = 2, 96
    x = torch.randn((b, c, 1), generator=gen(500)).to(BF16)
    cache = torch.randn((b, c, 3), generator=gen(501)).to(BF16)
    w = (torch.randn((c, 1, 4), generator=gen(502)) * 0.5).to(BF16)
    cache_after = cache.clone()
    y = inline_causal_conv.inline_causal_conv_step(x, cache_after, w)
    conv = {"x": x, "cache": cache, "w": w, "y": y, "cache_after": cache_after}

    heads, dk, dv, t = 4, 16, 16, 3
    q = torch.randn((b, t, heads, dk), generator=gen(510)).to(BF16)
    k = torch.randn((b, t, heads, dk), generator=gen(511)).to(BF16)
    v = torch.randn((b, t, heads, dv), generator=gen(512)).to(BF16)
    g = -torch.rand((b, t, heads), generator=gen(513))
    beta = torch.rand((b, t, heads), generator=gen(514)).to(BF16)
    s0 = torch.randn((b, heads, dk, dv), generator=gen(515)) * 0.1
    out, s1 = ref.recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=s0)
    rule = {"q": q, "k": k, "v": v, "g": g, "beta": beta, "state": s0, "out": out, "state_after": s1}

    a = torch.randn((b, 1, heads), generator=gen(520)).to(BF16)
    bb = torch.randn((b, 1, heads), generator=gen(521)).to(BF16)
    a_log = torch.log(torch.rand(heads, generator=gen(522)) * 16 + 1e-3)
    dt_bias = (torch.randn(heads, generator=gen(523)) * 0.1).to(BF16)
    gg = -a_log.float().exp() * torch.nn.functional.softplus(a.float() + dt_bias.float())
    gates = {"a": a, "b": bb, "A_log": a_log, "dt_bias": dt_bias, "g": gg, "beta": bb.sigmoid()}
    save("deltanet", {"conv": conv, "rule": rule, "gates": gates})


def attention_vectors() -> None:
    cases = []
    for i, (b, hq, hkv, length, d) in enumerate([(1, 4, 1, 33, 32), (2, 8, 2, 1, 64), (1, 16, 4, 130, 256)]):
        q = torch.randn((b, hq, d), generator=gen(600 + i)).to(BF16)
        k = torch.randn((b, hkv, length, d), generator=gen(610 + i)).to(BF16)
        v = torch.randn((b, hkv, length, d), generator=gen(620 + i)).to(BF16)
        scale = d**-0.5
        y = gqa_decode._reference_decode_attention(q, k, v, scale)
        cases.append({"q": q, "k": k, "v": v, "scale": scale, "y": y})
    save("attention", {"cases": cases})


def model_vectors() -> None:
    cfg = tiny_config()
    torch.manual_seed(7)
    model = ref.ReferenceModel(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("A_log"):
                p.copy_(torch.log(torch.rand(p.shape) * 8 + 0.1))
            elif name.endswith("dt_bias"):
                p.copy_(torch.randn(p.shape) * 0.1)
            elif "norm" in name and name.endswith("linear_attn.norm.weight"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape))
            elif "norm" in name:
                p.copy_(0.1 * torch.randn(p.shape))
            elif "conv1d" in name:
                p.copy_(0.5 * torch.randn(p.shape))
            elif "embed_tokens" in name:
                p.copy_(torch.randn(p.shape))
            else:
                p.copy_(torch.randn(p.shape) * (p.shape[-1] ** -0.5))
    model = model.to(dtype=BF16).eval()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    prompt = torch.randint(0, cfg.vocab_size, (2, 5), generator=gen(700))

    def run(m):
        cache = m.new_cache(2, 16)
        with torch.no_grad():
            logits0, _ = m(prompt, cache, num_logits_to_keep=1)
            steps = [logits0]
            tok = logits0[:, -1].argmax(dim=-1, keepdim=True)
            toks = [tok]
            for _ in range(4):
                lg, _ = m(tok, cache, num_logits_to_keep=1)
                steps.append(lg)
                tok = lg[:, -1].argmax(dim=-1, keepdim=True)
                toks.append(tok)
        return {
            "logits": torch.stack(steps),
            "tokens": torch.cat(toks, dim=1),
            "cache": [t.clone() for t in cache.state_tensors()],
            "seq_len": cache.seq_len,
        }

    bf16_run = run(model)

    # int4 on every linear and the head, through the reference's own torch-expression installers.
    visible_int4_head.install_int4_wide_torch_dequant(model)
    visible_int4_head._install_dequant_linears(tiled_gemv._gate_linears(model), visible_int4_head.DequantInt4Linear)
    kinds = sorted({type(m).__name__ for m in model.modules() if isinstance(m, torch.nn.Linear)})
    assert kinds == ["DequantInt4Linear"], kinds
    int4_run = run(model)
    with torch.no_grad():
        greedy = greedy_decode(model, prompt, 6)
    save(
        "tiny_model",
        {"state_dict": state, "prompt": prompt, "bf16": bf16_run, "int4": int4_run, "int4_greedy": greedy},
    )


if __name__ == "__main__":
    torch.set_num_threads(1)  # one thread: reductions take one fixed order, so vectors regenerate identically
    int4_vectors()
    elementwise_vectors()
    deltanet_vectors()
    attention_vectors()
    model_vectors()
