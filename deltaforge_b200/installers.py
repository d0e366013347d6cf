"""Installers: put the CUDA decode step under a reference-structured model, the reference's way.

Conventions kept from the reference's installers (src/deltaforge/model.py:46-80 and the per-kernel
modules): an installer has the signature ``installer(model, entry=None)``; it installs by class swap
(``obj.__class__ = Subclass``, never by assigning a bound method; kernels/fused_rmsnorm_residual.py:
252-257), subclassing ``type(obj)`` so installs compose (kernels/tiled_gemv.py:1085-1104); it is
idempotent through a ``_deltaforge_*`` flag (kernels/tiled_gemv.py:1224-1229); quantised copies are
non-persistent buffers named ``w_k_major`` / ``qscale`` plus the attribute ``qgroup``, never parameters
(kernels/tiled_gemv.py:1049-1071); prefill (``seq_len > 1``) keeps the model's own path, decode does not
fall back (kernels/fused_causal_conv.py:187-196).

Two granularities:

* ``install_b200_decode_step`` replaces the whole single-token forward with the captured CUDA graph
  (registry operation ``decode_step``).
* ``install_b200_int4_linears`` swaps every ``nn.Linear`` (and the tied head) for the int4 GEMV op and
  leaves the rest of the model alone (the reference's ``install_int4_wide_torch_dequant`` shape,
  kernels/visible_int4_head.py:335-361).

``register_with_reference()`` adds both, and one kernel per reference operation, to the reference's
``REGISTRY`` / ``INSTALLERS`` / ``CHECK_BUILDERS`` tables when that package is importable, and points the
reference's own ``deltaforge::`` ops at these kernels.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from . import ops
from .engine import MATH_FAST, DecodeEngine, weights_from_model
from .quant import quantise_int4_k_major

FLAG_STEP = "_deltaforge_b200_decode_step"
FLAG_LINEARS = "_deltaforge_b200_int4_linears"


# --------------------------------------------------------------------------------------
# int4 linears as module swaps
# --------------------------------------------------------------------------------------


class B200Int4Linear(nn.Linear):
    """``nn.Linear`` whose forward is the int4 GEMV kernel on its ``w_k_major`` / ``qscale`` buffers."""

    def forward(self, x: Tensor) -> Tensor:  # type: ignore[override]
        if x.numel() // x.shape[-1] > 64:  # prefill-sized input: dequantise once, dense product
            dense = ops.int4_dequant(self.w_k_major, self.qscale, self.qgroup)
            out = (x.float() @ dense.float()).to(x.dtype)
        else:
            out = ops.tiled_gemv_int4(x, self.w_k_major, self.qscale, self.qgroup)
        return out if self.bias is None else out + self.bias


class B200Int4LMHead(nn.Module):
    def __init__(self, packed: Tensor, scale: Tensor, group_size: int) -> None:
        super().__init__()
        self.register_buffer("w_k_major", packed, persistent=False)
        self.register_buffer("qscale", scale, persistent=False)
        self.kind = "int4"
        self.qgroup = group_size

    def forward(self, hidden_states: Tensor) -> Tensor:
        return ops.tiled_gemv_int4(hidden_states, self.w_k_major, self.qscale, self.qgroup)


def _attach_int4(linear: nn.Linear) -> None:
    if getattr(linear, "w_k_major", None) is None:
        qw = quantise_int4_k_major(linear.weight)
        linear.register_buffer("w_k_major", qw.qweight, persistent=False)
        linear.register_buffer("qscale", qw.scale, persistent=False)
        linear.qgroup = qw.group_size


def install_b200_int4_linears(model, entry=None) -> None:
    """Every ``nn.Linear`` -> ``B200Int4Linear``; the tied head -> ``B200Int4LMHead`` via ``project_logits``."""
    if getattr(model, FLAG_LINEARS, False):
        return
    for module in list(model.modules()):
        if isinstance(module, nn.Linear) and not isinstance(module, B200Int4Linear):
            _attach_int4(module)
            module.__class__ = B200Int4Linear
    qw = quantise_int4_k_major(model.embed_tokens.weight if model.config.tie_word_embeddings else model.lm_head.weight)
    model.tiled_lm_head = B200Int4LMHead(qw.qweight, qw.scale, qw.group_size)
    base = type(model)

    class B200HeadModel(base):  # type: ignore[misc, valid-type]
        def project_logits(self, hidden_states: Tensor) -> Tensor:
            return self.tiled_lm_head(hidden_states)

    B200HeadModel.__name__ = f"B200Head{base.__name__}"
    model.__class__ = B200HeadModel
    setattr(model, FLAG_LINEARS, True)


# --------------------------------------------------------------------------------------
# whole decode step
# --------------------------------------------------------------------------------------


def _engine_for(model, cache) -> DecodeEngine:
    engines = model.__dict__.setdefault("_dfb200_engines", {})
    key = id(cache)
    eng = engines.get(key)
    if eng is None or eng.cache is not cache:
        if model.__dict__.get("_dfb200_weights") is None:
            model.__dict__["_dfb200_weights"] = weights_from_model(
                model, device=next(model.parameters()).device, scale_dtype=model.__dict__.get("_dfb200_scale_dtype")
            )
        eng = DecodeEngine(
            model.__dict__["_dfb200_weights"], cache, attn_splits=model.__dict__.get("_dfb200_attn_splits"),
            math=model.__dict__.get("_dfb200_math", MATH_FAST),
        )  # fmt: skip
        engines[key] = eng
    return eng


def install_b200_decode_step(
    model, entry=None, *, attn_splits: int | None = None, math: int = MATH_FAST, scale_dtype=None
) -> None:
    """Replace the single-token forward of ``model`` with the captured CUDA decode step.

    All linears and the head run as group-128 int4 (quantised here unless the model already carries
    int4 buffers). Calls with ``seq_len > 1``, no cache, or explicit ``position_ids`` keep the model's
    own forward, which fills the same cache tensors the kernels then update in place.
    """
    if getattr(model, FLAG_STEP, False):
        return
    if not next(model.parameters()).is_cuda:
        raise RuntimeError("install_b200_decode_step requires the model on a CUDA device and has no PyTorch fallback")
    base = type(model)

    class B200DecodeStepModel(base):  # type: ignore[misc, valid-type]
        def decode_engine(self, cache) -> DecodeEngine:
            return _engine_for(self, cache)

        @torch.no_grad()
        def forward(self, input_ids, cache=None, *, position_ids=None, num_logits_to_keep: int = 0):
            batch, seq_len = input_ids.shape
            if seq_len != 1 or cache is None or position_ids is not None:
                extra = {} if position_ids is None else {"position_ids": position_ids}
                return super().forward(input_ids, cache, num_logits_to_keep=num_logits_to_keep, **extra)
            ops.require_cuda(input_ids, "decode_step")
            logits = _engine_for(self, cache).step(input_ids[:, 0])
            return logits.clone().view(batch, 1, -1), cache

        def decode_loop(self, model, input_ids, max_new_tokens: int, cache):
            """Greedy loop hook of ``greedy_decode`` (src/deltaforge/model.py:129-138): the prompt goes
            through the model's prefill path, the new tokens through replays of the captured graph."""
            prompt_len = input_ids.shape[1]
            if prompt_len > 1:
                super().forward(input_ids[:, :-1], cache, num_logits_to_keep=1)
            return _engine_for(self, cache).decode(input_ids[:, -1], max_new_tokens)

    B200DecodeStepModel.__name__ = f"B200DecodeStep{base.__name__}"
    model.__class__ = B200DecodeStepModel
    model.__dict__["_dfb200_attn_splits"] = attn_splits
    model.__dict__["_dfb200_math"] = math
    model.__dict__["_dfb200_scale_dtype"] = scale_dtype
    setattr(model, FLAG_STEP, True)


def is_installed(model) -> bool:
    return bool(getattr(model, FLAG_STEP, False) or getattr(model, FLAG_LINEARS, False))


# --------------------------------------------------------------------------------------
# hooking into the reference package when it is importable
# --------------------------------------------------------------------------------------

#: reference op name -> the op of this package with the same argument list
DROP_IN_OPS = {
    "tiled_gemv_int4": ("deltaforge.kernels.tiled_gemv", "tiled_gemv_int4", ops.tiled_gemv_int4),
    "delta_rule_step": ("deltaforge.kernels.gated_delta_step", "delta_rule_step", ops.delta_rule_step),
    "fused_causal_conv_step": ("deltaforge.kernels.fused_causal_conv", "fused_causal_conv_step", ops.fused_causal_conv_step),
    "gqa_decode_attention": ("deltaforge.kernels.gqa_decode", "gqa_decode_attention", ops.gqa_decode_attention),
    "split_kv_decode_attention": ("deltaforge.kernels.flash_decode_splitkv", "split_kv_decode_attention", ops.split_kv_decode_attention),
    "add_rms_norm": ("deltaforge.kernels.fused_rmsnorm_residual", "add_rms_norm", ops.add_rms_norm),
    "rms_norm": ("deltaforge.kernels.fused_rmsnorm_residual", "rms_norm", ops.rms_norm),
    "partial_rope": ("deltaforge.kernels.fused_rope", "apply_partial_rope", ops.partial_rope),
    "silu_mul": ("deltaforge.kernels.fused_swiglu", "silu_mul", ops.silu_mul),
}


def _forward_to(op):
    def kernel(*args):
        return op(*args)

    return kernel


#: kernel name here -> (operation it replaces, the reference's own kernel whose installer performs the module swap and
#: whose layer-1 checks probe the op, the reference ops that installer's modules call). The per-op kernels are the
#: reference's module swaps with their ``deltaforge::`` ops answered by ``libdfb200.so``: nothing of the reference's
#: module code is restated here.
PER_OP_KERNELS = {
    "b200_deltanet_step": ("gated_delta_rule", "gated_delta_step", ("delta_rule_step",)),
    "b200_causal_conv": ("causal_conv", "fused_causal_conv", ("fused_causal_conv_step",)),
    "b200_attn_decode": ("gqa_attention", "flash_decode_splitkv", ("split_kv_decode_attention", "gqa_decode_attention")),
    "b200_rmsnorm_residual": ("rms_norm_residual", "fused_rmsnorm_residual", ("add_rms_norm", "rms_norm")),
    "b200_rope": ("qkv_projection_rope", "fused_rope", ("partial_rope",)),
    "b200_swiglu": ("swiglu_mlp", "fused_swiglu", ("silu_mul",)),
}

_redirected: set[str] = set()


def redirect_reference_op(op_name: str) -> None:
    """Register this package's CUDA kernel on the reference's ``deltaforge::<op_name>`` op object (once)."""
    import importlib

    if op_name in _redirected:
        return
    module_name, attr, ours = DROP_IN_OPS[op_name]
    their_op = getattr(importlib.import_module(module_name), attr)
    their_op.register_kernel("cuda")(_forward_to(ours))
    _redirected.add(op_name)


def _per_op_installer(ref_kernel: str, op_names: tuple[str, ...]):
    def installer(model, entry=None) -> None:
        import importlib

        for op_name in op_names:
            redirect_reference_op(op_name)
        importlib.import_module("deltaforge.model").INSTALLERS[ref_kernel](model, entry)

    installer.__name__ = f"install_b200_via_{ref_kernel}"
    return installer


def _per_op_checks(ref_kernel: str, op_names: tuple[str, ...]):
    def builder(model, **kwargs):
        import importlib

        for op_name in op_names:
            redirect_reference_op(op_name)
        return importlib.import_module("deltaforge.kernels").CHECK_BUILDERS[ref_kernel](model, **kwargs)

    return builder


def int4_gemv_checks(model, *, device="cuda", dtype=None, seed: int = 0, replaces: str = "decode_step"):
    """Layer-1 probes of the int4 GEMV, in the reference's form (src/deltaforge/kernels/quantised_linear.py:737-741,
    src/deltaforge/harness/correctness.py:136-200): for the narrowest and the widest layer projection, the K = 9216
    one and the tied head, activations of shape ``(1, 1, K)`` and ``(32, 1, K)``, this package's op against the
    reference's torch expression on the same packed weight."""
    import importlib

    check_kernel = importlib.import_module("deltaforge.harness.correctness").check_kernel
    ref_gemv = importlib.import_module("deltaforge.kernels.visible_int4_head").torch_dequant_gemv_int4
    ref_quant = importlib.import_module("deltaforge.kernels.tiled_gemv").quantise_int4_k_major
    linears = [m for m in model.modules() if isinstance(m, nn.Linear)]
    by_shape = {}
    for lin in linears:
        by_shape.setdefault((lin.out_features, lin.in_features), lin)
    shapes = sorted(by_shape)
    picks = {shapes[0], shapes[-1], max(shapes, key=lambda nk: nk[1])}
    probes = [(by_shape[nk].weight, f"N={nk[0]} K={nk[1]}") for nk in sorted(picks)]
    head = model.embed_tokens.weight if model.config.tie_word_embeddings else model.lm_head.weight
    probes.append((head, f"N={head.shape[0]} K={head.shape[1]} (lm head)"))
    gen = torch.Generator(device=device).manual_seed(seed)
    checks = []
    for weight, label in probes:
        qw = ref_quant(weight.detach().to(device))
        packed, scale, group = qw.qweight, qw.scale, int(qw.group_size)
        k = weight.shape[1]
        for shape, note in (((1, 1, k), "batch 1, one token"), ((32, 1, k), "batch 32, one token")):
            x = torch.randn(shape, device=device, dtype=weight.dtype, generator=gen)
            checks.append(
                check_kernel(
                    f"b200.int4_gemv[{label}]",
                    lambda a, q, sc, g=group: ref_gemv(a, q, sc, g),
                    lambda a, q, sc, g=group: ops.tiled_gemv_int4(a, q, sc, g),
                    args=(x, packed, scale),
                    replaces=replaces,
                    note=note,
                )
            )
    return tuple(checks)


def register_with_reference(*, redirect_ops: bool = True) -> dict[str, object]:
    """Register this package's kernels with an importable ``deltaforge`` package.

    Adds to ``deltaforge.kernels.REGISTRY`` (as candidates), ``deltaforge.model.INSTALLERS`` and
    ``deltaforge.kernels.CHECK_BUILDERS``: ``b200_decode_step`` (replaces ``decode_step``), ``b200_int4_linears``
    (replaces ``swiglu_mlp``, the operation the reference's wide int4 installer is filed under) and one kernel per
    reference operation (``PER_OP_KERNELS``). With ``redirect_ops`` it also registers a CUDA kernel on each of the
    reference's own ``deltaforge::`` op objects, so its existing module classes dispatch to ``libdfb200.so`` with no
    model change. Idempotent. Returns what was registered. Raises ``ImportError`` if the reference is not importable.
    """
    import importlib

    kernels = importlib.import_module("deltaforge.kernels")
    ref_model = importlib.import_module("deltaforge.model")
    done: dict[str, object] = {}
    table = [
        ("b200_decode_step", "decode_step", install_b200_decode_step, lambda model, **kw: int4_gemv_checks(model, replaces="decode_step", **kw)),
        ("b200_int4_linears", "swiglu_mlp", install_b200_int4_linears, lambda model, **kw: int4_gemv_checks(model, replaces="swiglu_mlp", **kw)),
    ]  # fmt: skip
    for name, (replaces, ref_kernel, op_names) in PER_OP_KERNELS.items():
        table.append((name, replaces, _per_op_installer(ref_kernel, op_names), _per_op_checks(ref_kernel, op_names)))
    for name, replaces, installer, checks in table:
        if name not in kernels.REGISTRY:
            kernels.REGISTRY.register(name, installer, replaces=replaces, status="candidate", notes="sm_100a CUDA, libdfb200.so")
        if name not in ref_model.INSTALLERS:
            ref_model.register_installer(name, installer)
        if name not in kernels.CHECK_BUILDERS:
            kernels.register_checks(name, checks)
        done[name] = installer
    if redirect_ops:
        for op_name, (_, _, ours) in DROP_IN_OPS.items():
            redirect_reference_op(op_name)
            done[f"deltaforge::{op_name}"] = ours
    return done
