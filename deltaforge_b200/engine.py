"""Whole-step decode engine: weights, decode state and the captured CUDA graph.

``DecodeEngine`` is the host side of ``dfb_engine_*`` (include/dfb200.h). It holds the int4 weights of
one model replica, binds to a decode cache that has the reference's tensor layout
(``DecodeCache``, src/deltaforge/reference.py:241-299: KV ``(B, Hkv, max_seq, D)`` bf16, conv history
``(B, C, 3)`` bf16, recurrent state ``(B, Hv, dk, dv)`` fp32) and runs ``ReferenceModel.forward`` for
``seq_len == 1`` (reference.py:779-817) plus the greedy argmax (src/deltaforge/model.py:141-147) as one
CUDA graph. The kernels update the cache tensors in place, so ``snapshot`` / ``restore`` / ``rewind`` of
the cache keep working and prefill can be done by any code that fills those tensors.

torch is used for device memory and streams only; every kernel on the path is in ``libdfb200.so``.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch
from torch import Tensor

from . import _lib
from ._lib import LayerDesc, Linear, ModelDesc
from .config import FULL_ATTENTION, LINEAR_ATTENTION
from .quant import QuantisedWeight, concat_along_n, quantise_int4_k_major

BF16 = torch.bfloat16
MATH_FAST, MATH_EXACT = 0, 1


@dataclass
class LayerWeights:
    kind: str
    input_norm: Tensor
    post_norm: Tensor
    in_proj: QuantisedWeight  # DeltaNet: qkv|z|b|a ; attention: q|k|v
    out_proj: QuantisedWeight
    gate_up: QuantisedWeight
    down: QuantisedWeight
    conv_w: Tensor | None = None  # (C, 4) bf16
    a_log: Tensor | None = None  # fp32 copies of what the model holds
    dt_bias: Tensor | None = None
    gnorm_w: Tensor | None = None
    gnorm_w_is_bf16: bool = True
    q_norm: Tensor | None = None
    k_norm: Tensor | None = None


@dataclass
class ModelWeights:
    config: object
    embed: Tensor  # (V, H) bf16, the lookup table
    final_norm: Tensor
    head: QuantisedWeight
    inv_freq: Tensor  # fp32 values as the model holds them (bf16-rounded in a bf16 model)
    layers: list[LayerWeights] = field(default_factory=list)

    def weight_bytes(self) -> int:
        """Bytes of int4 weights and scales one decode step streams (the embedding row is not counted)."""
        total = 0
        for qw in [self.head] + [q for L in self.layers for q in (L.in_proj, L.out_proj, L.gate_up, L.down)]:
            total += qw.qweight.numel() + qw.scale.numel() * qw.scale.element_size()
        return total


def _quantised(linear, device, scale_dtype) -> QuantisedWeight:
    """The int4 form of an ``nn.Linear``: its installed buffers if it has them, else quantise its weight."""
    if getattr(linear, "bias", None) is not None:
        raise ValueError("projections with a bias are not supported by the fused decode step")
    packed = getattr(linear, "w_k_major", None)
    if packed is not None and packed.dtype == torch.uint8:
        qw = QuantisedWeight(packed.to(device), linear.qscale.to(device), 4, int(linear.qgroup))
    else:
        qw = quantise_int4_k_major(linear.weight.to(device))
    if scale_dtype is not None and qw.scale.dtype != scale_dtype:
        qw = QuantisedWeight(qw.qweight, qw.scale.to(scale_dtype), 4, qw.group_size)
    return qw


@torch.no_grad()
def weights_from_model(model, device="cuda", scale_dtype: torch.dtype | None = None) -> ModelWeights:
    """Collect (and where needed quantise) the decode weights of a reference-structured model.

    ``model`` has the module tree of ``ReferenceModel`` (src/deltaforge/reference.py:738-752). Linears
    that already carry ``w_k_major`` / ``qscale`` / ``qgroup`` buffers (the reference's int4 installers,
    src/deltaforge/kernels/tiled_gemv.py:1049-1071) contribute those exact buffers; the tied head uses
    ``tiled_lm_head`` / ``head_w_k_major`` buffers when present, else the embedding matrix is quantised.
    """
    cfg = model.config
    dev = torch.device(device)

    def norm(w: Tensor) -> Tensor:
        return w.detach().to(dev, BF16).contiguous()

    embed = model.embed_tokens.weight.detach().to(dev, BF16).contiguous()
    head_src = model.embed_tokens if cfg.tie_word_embeddings else model.lm_head
    tiled = getattr(model, "tiled_lm_head", None)
    if tiled is not None and getattr(tiled, "w_k_major", None) is not None:
        head = QuantisedWeight(tiled.w_k_major.to(dev), tiled.qscale.to(dev), 4, int(tiled.qgroup))
    elif getattr(model, "head_w_k_major", None) is not None:
        head = QuantisedWeight(model.head_w_k_major.to(dev), model.head_qscale.to(dev), 4, int(model.head_qgroup))
    else:
        head = quantise_int4_k_major(head_src.weight.to(dev))
    if scale_dtype is not None:
        head = QuantisedWeight(head.qweight, head.scale.to(scale_dtype), 4, head.group_size)
    inv_freq = getattr(model, "inv_freq", None)
    if inv_freq is None:
        inv_freq = model.rotary_emb.inv_freq
    out = ModelWeights(cfg, embed, norm(model.norm.weight), head, inv_freq.detach().float().to(dev).contiguous())
    for layer in model.layers:
        q = lambda lin: _quantised(lin, dev, scale_dtype)  # noqa: E731
        gate_up = concat_along_n([q(layer.mlp.gate_proj), q(layer.mlp.up_proj)])
        down = q(layer.mlp.down_proj)
        if layer.layer_type == LINEAR_ATTENTION:
            m = layer.linear_attn
            lw = LayerWeights(
                kind=LINEAR_ATTENTION,
                input_norm=norm(layer.input_layernorm.weight),
                post_norm=norm(layer.post_attention_layernorm.weight),
                in_proj=concat_along_n([q(m.in_proj_qkv), q(m.in_proj_z), q(m.in_proj_b), q(m.in_proj_a)]),
                out_proj=q(m.out_proj),
                gate_up=gate_up,
                down=down,
                conv_w=m.conv1d.weight.detach().reshape(cfg.linear_conv_dim, -1).to(dev, BF16).contiguous(),
                a_log=m.A_log.detach().float().to(dev).contiguous(),
                dt_bias=m.dt_bias.detach().float().to(dev).contiguous(),
                gnorm_w=m.norm.weight.detach().float().to(dev).contiguous(),
                gnorm_w_is_bf16=m.norm.weight.dtype == BF16,
            )
            if lw.conv_w.shape[1] != 4:
                raise ValueError(f"the fused conv is the four-tap case; got {lw.conv_w.shape[1]} taps")
        else:
            m = layer.self_attn
            lw = LayerWeights(
                kind=FULL_ATTENTION,
                input_norm=norm(layer.input_layernorm.weight),
                post_norm=norm(layer.post_attention_layernorm.weight),
                in_proj=concat_along_n([q(m.q_proj), q(m.k_proj), q(m.v_proj)]),
                out_proj=q(m.o_proj),
                gate_up=gate_up,
                down=down,
                q_norm=norm(m.q_norm.weight),
                k_norm=norm(m.k_norm.weight),
            )
        out.layers.append(lw)
    return out


def cache_layer_tensors(layer) -> dict[str, Tensor]:
    """Tensors of one cache layer, for the reference's dataclasses and for plain dicts alike."""
    if isinstance(layer, dict):
        return layer
    if hasattr(layer, "conv"):
        return {"conv": layer.conv, "recurrent": layer.recurrent}
    return {"keys": layer.keys, "values": layer.values}


class DecodeCache:
    """Decode state in the reference's layout, with its ``DecodeCache`` interface (reference.py:241-395)."""

    def __init__(self, config, batch_size: int, max_seq_len: int, device="cuda", dtype=BF16) -> None:
        self.config, self.batch_size, self.max_seq_len = config, batch_size, max_seq_len
        self.device, self.dtype, self.seq_len = torch.device(device), dtype, 0
        self.layers: list[dict[str, Tensor]] = []
        for kind in config.layer_types:
            if kind == FULL_ATTENTION:
                shape = (batch_size, config.num_key_value_heads, max_seq_len, config.head_dim)
                self.layers.append({"keys": torch.zeros(shape, device=device, dtype=dtype), "values": torch.zeros(shape, device=device, dtype=dtype)})
            else:
                self.layers.append(
                    {
                        "conv": torch.zeros((batch_size, config.linear_conv_dim, config.linear_conv_kernel_dim - 1), device=device, dtype=dtype),
                        "recurrent": torch.zeros(
                            (batch_size, config.linear_num_value_heads, config.linear_key_head_dim, config.linear_value_head_dim),
                            device=device, dtype=torch.float32,
                        ),
                    }
                )  # fmt: skip

    def state_tensors(self) -> tuple[Tensor, ...]:
        out: list[Tensor] = []
        for layer in self.layers:
            out.extend(layer[k] for k in (("keys", "values") if "keys" in layer else ("conv", "recurrent")))
        return tuple(out)

    def reset(self) -> None:
        self.seq_len = 0
        for t in self.state_tensors():
            t.zero_()

    def snapshot(self):
        return (self.seq_len, tuple(t.clone() for t in self.state_tensors()))

    def restore(self, snapshot) -> None:
        seq_len, tensors = snapshot
        live = self.state_tensors()
        if len(live) != len(tensors) or any(a.shape != b.shape or a.dtype != b.dtype for a, b in zip(live, tensors)):
            raise ValueError("snapshot came from a different cache")
        for t, saved in zip(live, tensors):
            t.copy_(saved)  # in place: the captured graph holds these addresses
        self.seq_len = seq_len

    def load_from(self, other) -> None:
        """Copy the state of another cache with the same layout (e.g. one filled by a CPU prefill)."""
        theirs = other.state_tensors()
        mine = self.state_tensors()
        if len(mine) != len(theirs):
            raise ValueError("caches have different layer structure")
        for a, b in zip(mine, theirs):
            if a.shape[-2:] != b.shape[-2:] and a.dim() == 4 and a.shape[2] != b.shape[2]:  # KV with another max_seq
                n = min(a.shape[2], b.shape[2])
                a[:, :, :n].copy_(b[:, :, :n])
            else:
                a.copy_(b)
        self.seq_len = other.seq_len

    def ensure_capacity(self, num_tokens: int) -> None:
        if self.seq_len + num_tokens > self.max_seq_len:
            raise ValueError(f"cache overflow: {self.seq_len} + {num_tokens} > max_seq_len={self.max_seq_len}")

    def advance(self, num_tokens: int) -> None:
        self.ensure_capacity(num_tokens)
        self.seq_len += num_tokens

    def rewind(self, to_seq_len: int) -> None:
        if to_seq_len < 0:
            raise ValueError(f"cannot rewind past 0, got {to_seq_len}")
        if to_seq_len > self.seq_len:
            raise ValueError(f"can only rewind backwards: asked for {to_seq_len} from {self.seq_len}")
        self.seq_len = to_seq_len


def default_attn_splits(max_seq_len: int, batch: int, kv_heads: int, sm_count: int = 148) -> int:
    """Enough key slices that batch * kv_heads * splits CTAs cover the SMs about twice, with at least
    64 keys per slice; a power of two between 1 and 64."""
    # The fused attention kernel stages a slice of at most 160 keys in shared memory, one CTA per SM,
    # and its cost grows with the number of CTAs: take the fewest slices that fit (up to 128).
    splits = 1
    while splits < 128 and -(-max_seq_len // splits) > 160:
        splits *= 2
    if batch <= 2 and -(-max_seq_len // splits) <= 160:
        # Short caches: still use the SMs. (More, shorter slices than one CTA per SM were measured at 4K tokens: 256 CTAs
        # of 105 KB cannot sit beside the projection before them, start in waves only when it has left, and the kernel
        # takes 20 us instead of 12.)
        while splits * 2 * batch * kv_heads <= sm_count and max_seq_len // (splits * 2) >= 64:
            splits *= 2
        return splits
    # longer caches take the two-kernel path, which has no slice limit: about eight waves of CTAs, slices of
    # at least 256 keys (the tensor-core kernel streams 16-key tiles through a ring and wants a long slice)
    want = max(1, (8 * sm_count) // max(1, batch * kv_heads))
    splits = 1
    while splits * 2 <= min(want, 128) and max_seq_len // (splits * 2) >= 256:
        splits *= 2
    return splits


class DecodeEngine:
    """One model replica's decode step on one GPU, bound to one cache."""

    def __init__(
        self,
        weights: ModelWeights,
        cache,
        *,
        attn_splits: int | None = None,
        math: int = MATH_FAST,
        tp_size: int = 1,
        tp_rank: int = 0,
        tp_peer_slots: list[int] | None = None,
        prefetch_distance: int | None = None,
        tensor_core_gemv: bool = True,
    ) -> None:
        """``prefetch_distance``: how many projections ahead the kernels of a batch-1 step ask the L2 cache for
        weights (``dfb_engine_set_prefetch_distance``; ``None`` keeps the library's default, 0 switches it off).
        ``tensor_core_gemv``: batch 1 runs the layer projections on the integer tensor-core instruction, from one more
        re-packed copy of each weight (off: the dp4a kernels on the ``k8`` copy)."""
        cfg = weights.config
        self.config, self.weights, self.cache = cfg, weights, cache
        self.batch, self.max_seq = cache.batch_size, cache.max_seq_len
        dev = weights.embed.device
        if dev.type != "cuda":
            raise RuntimeError("DecodeEngine requires CUDA tensors and has no PyTorch fallback")
        self.device = dev
        self.lib = _lib.load()
        self.attn_splits = attn_splits or default_attn_splits(self.max_seq, self.batch, cfg.num_key_value_heads)
        self.tokens = torch.zeros(self.batch, dtype=torch.int64, device=dev)
        self.history = torch.zeros((self.max_seq, self.batch), dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.logits = torch.empty((self.batch, cfg.vocab_size), dtype=BF16, device=dev)
        self._pos_host = 0
        self._keep: list = []
        self._captured = False

        def lin(qw: QuantisedWeight, pair: bool = False, layer_sized: bool = True) -> Linear:
            if not (qw.qweight.is_contiguous() and qw.scale.is_contiguous()):
                raise ValueError("quantised weights must be contiguous")
            k, n = qw.in_features, qw.out_features
            # the re-packed copy serves the batch-1 streaming kernels and the tensor-core product (8 rows and more)
            wants_k8 = k % 128 == 0 and (self.batch == 1 or self.batch >= 8)
            if qw.k8 is None and wants_k8 and qw.group_size == 128 and n % 4 == 0:
                from . import ops  # the re-packed copy the streaming GEMV reads; made once per weight

                qw.k8 = ops.int4_repack_k8(qw.qweight)
            k8 = qw.k8.data_ptr() if qw.k8 is not None else None
            wants_mma = tensor_core_gemv and layer_sized and self.batch == 1 and math == MATH_FAST
            if wants_mma and qw.group_size == 128 and k % 128 == 0 and (qw.mma is None or qw.mma_pair != pair):
                from . import ops

                qw.mma, qw.mma_pair = ops.int4_repack_mma(qw.qweight, qw.scale, pair=pair), pair
            mma = qw.mma.data_ptr() if (wants_mma and qw.mma is not None and qw.mma_pair == pair) else None
            return Linear(qw.qweight.data_ptr(), qw.scale.data_ptr(), int(qw.scale.dtype == BF16), k, n, qw.group_size, k8, mma, int(pair))

        layers = (LayerDesc * len(weights.layers))()
        for i, (lw, cl) in enumerate(zip(weights.layers, cache.layers)):
            ct = cache_layer_tensors(cl)
            d = layers[i]
            d.kind = 0 if lw.kind == LINEAR_ATTENTION else 1
            d.input_norm_w, d.post_norm_w = lw.input_norm.data_ptr(), lw.post_norm.data_ptr()
            d.in_proj, d.out_proj, d.gate_up, d.down = lin(lw.in_proj), lin(lw.out_proj), lin(lw.gate_up, pair=True), lin(lw.down)
            for t in ct.values():
                if not (t.is_cuda and t.is_contiguous()):
                    raise ValueError("the decode cache must live on the GPU in contiguous tensors")
            if lw.kind == LINEAR_ATTENTION:
                if ct["conv"].dtype != BF16 or ct["recurrent"].dtype != torch.float32:
                    raise ValueError("conv history must be bfloat16 and the recurrent state float32")
                d.conv_w, d.a_log, d.dt_bias = lw.conv_w.data_ptr(), lw.a_log.data_ptr(), lw.dt_bias.data_ptr()
                d.gnorm_w, d.gnorm_w_is_bf16 = lw.gnorm_w.data_ptr(), int(lw.gnorm_w_is_bf16)
                d.conv_state, d.recurrent = ct["conv"].data_ptr(), ct["recurrent"].data_ptr()
            else:
                if ct["keys"].dtype != BF16:
                    raise ValueError("the KV cache must be bfloat16")
                d.q_norm_w, d.k_norm_w = lw.q_norm.data_ptr(), lw.k_norm.data_ptr()
                d.kcache, d.vcache = ct["keys"].data_ptr(), ct["values"].data_ptr()
        m = ModelDesc()
        m.hidden, m.intermediate, m.vocab = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        m.num_layers, m.batch, m.max_seq = len(weights.layers), self.batch, self.max_seq
        m.hq, m.hkv, m.head_dim, m.rotary_dim = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rotary_dim
        m.attn_output_gate, m.gate_is_swish = int(cfg.attn_output_gate), int(cfg.output_gate_type == "swish")
        m.lin_k_heads, m.lin_v_heads = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        m.lin_dk, m.lin_dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        m.eps = cfg.rms_norm_eps
        m.inv_freq, m.embed, m.final_norm_w = weights.inv_freq.data_ptr(), weights.embed.data_ptr(), weights.final_norm.data_ptr()
        m.head = lin(weights.head, layer_sized=False)
        m.layers_host = layers
        m.tokens, m.history, m.pos, m.logits = self.tokens.data_ptr(), self.history.data_ptr(), self.pos.data_ptr(), self.logits.data_ptr()
        m.attn_splits, m.math = self.attn_splits, math
        m.workspace, m.workspace_bytes = None, 0
        m.tp_size, m.tp_rank = int(tp_size), int(tp_rank)
        if tp_peer_slots is not None:
            self._peer_array = (C.c_void_p * len(tp_peer_slots))(*tp_peer_slots)
            m.tp_peer_slots = C.cast(self._peer_array, C.POINTER(C.c_void_p))
        nbytes = self.lib.dfb_engine_workspace_bytes(C.byref(m))
        self.workspace = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=dev)
        m.workspace, m.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        self._desc, self._layers = m, layers
        handle = C.c_void_p()
        _lib.check(self.lib.dfb_engine_create(C.byref(m), C.byref(handle)), "dfb_engine_create")
        self._handle = handle
        if prefetch_distance is not None:
            _lib.check(self.lib.dfb_engine_set_prefetch_distance(handle, int(prefetch_distance)), "dfb_engine_set_prefetch_distance")

    def set_trace(self, max_ctas: int = 320) -> Tensor | None:
        """Profiling: record per-CTA device timestamps of every launch of the steps captured or enqueued from now
        on. Returns the int64 tensor ``(launches, max_ctas, 8)`` the kernels write (see ``dfb_engine_set_trace``
        for the marks); ``max_ctas=0`` switches tracing off. Call before ``capture()``."""
        if max_ctas <= 0:
            _lib.check(self.lib.dfb_engine_set_trace(self._handle, None, 0, 0), "dfb_engine_set_trace")
            self._trace = None
            return None
        launches = 16 + 8 * len(self.weights.layers)
        self._trace = torch.zeros((launches, max_ctas, 8), dtype=torch.int64, device=self.device)
        _lib.check(self.lib.dfb_engine_set_trace(self._handle, self._trace.data_ptr(), launches, max_ctas), "dfb_engine_set_trace")
        self._captured = False
        return self._trace

    # -- lifecycle -------------------------------------------------------------------------

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self.lib.dfb_engine_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    @property
    def launches_per_step(self) -> int:
        return self.lib.dfb_engine_launches_per_step(self._handle)

    def check_status(self) -> None:
        """Synchronise and raise if a kernel gave up on one of its bounded waits."""
        code = C.c_int(0)
        _lib.check(self.lib.dfb_engine_status(self._handle, C.byref(code), self._stream()), "dfb_engine_status")
        if code.value:
            raise _lib.Dfb200Error(
                f"a decode kernel reported status {code.value}: a bounded wait ran out "
                "(50: a tensor-parallel peer's partial sums never arrived; 60 and up: an index check of the bounds build; "
                "other codes: an asynchronous copy)"
            )

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _sync_position(self) -> None:
        """Make the device-side position equal the cache's ``seq_len`` (it differs after a prefill,
        restore or rewind done outside the engine)."""
        if self._pos_host != self.cache.seq_len:
            self.pos.fill_(self.cache.seq_len)
            self._pos_host = self.cache.seq_len

    def capture(self) -> None:
        """Capture one step into a CUDA graph. The step is not executed."""
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            _lib.check(self.lib.dfb_engine_capture(self._handle, stream.cuda_stream), "dfb_engine_capture")
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self._captured = True

    # -- decode -----------------------------------------------------------------------------

    def _set_tokens(self, tokens: Tensor) -> None:
        tokens = tokens.reshape(-1)
        if tokens.numel() != self.batch:
            raise ValueError(f"expected {self.batch} tokens (one per sequence), got {tokens.numel()}")
        self.tokens.copy_(tokens.to(torch.int64), non_blocking=True)

    def step(self, tokens: Tensor, *, graph: bool = True) -> Tensor:
        """One decode step for ``tokens (B,)``: returns the logits ``(B, V)`` (a view of the engine's
        buffer, overwritten by the next step); the greedy next token is left in ``self.tokens``."""
        self.cache.ensure_capacity(1)
        self._sync_position()
        self._set_tokens(tokens)
        if graph:
            if not self._captured:
                self.capture()
            _lib.check(self.lib.dfb_engine_replay(self._handle, 1, self._stream()), "dfb_engine_replay")
        else:
            _lib.check(self.lib.dfb_engine_step(self._handle, self._stream()), "dfb_engine_step")
        self.cache.advance(1)
        self._pos_host += 1
        return self.logits

    def decode(self, tokens: Tensor, steps: int) -> Tensor:
        """Greedy-decode ``steps`` tokens after ``tokens (B,)`` entirely on the device: the graph is
        replayed ``steps`` times, each replay reading the token the previous one chose. Returns ``(B, steps)``."""
        if steps < 1:
            raise ValueError("steps must be at least 1")
        self.cache.ensure_capacity(steps)
        self._sync_position()
        self._set_tokens(tokens)
        if not self._captured:
            self.capture()
        start = self.cache.seq_len
        _lib.check(self.lib.dfb_engine_replay(self._handle, steps, self._stream()), "dfb_engine_replay")
        self.cache.advance(steps)
        self._pos_host += steps
        return self.history[start : start + steps].t().contiguous()

    def decode_host(self, tokens_host: Tensor, steps: int, out_host: Tensor | None = None) -> Tensor:
        """The serving-style loop through the C ABI with host buffers: per step the input token is copied
        host->device, the graph runs, and the chosen token is copied device->host and waited for.
        ``tokens_host`` is a CPU int64 tensor ``(B,)`` (pinned for asynchronous copies). Returns ``(steps, B)``."""
        if tokens_host.is_cuda or tokens_host.dtype != torch.int64 or tokens_host.numel() != self.batch:
            raise ValueError("tokens_host must be a CPU int64 tensor with one token per sequence")
        if steps < 1:
            raise ValueError("steps must be at least 1")
        self.cache.ensure_capacity(steps)
        self._sync_position()
        if not self._captured:
            self.capture()
        if out_host is None:
            out_host = torch.empty((steps, self.batch), dtype=torch.int64).pin_memory()
        rc = self.lib.dfb_engine_decode_host(self._handle, tokens_host.data_ptr(), steps, out_host.data_ptr(), self._stream())
        _lib.check(rc, "dfb_engine_decode_host")
        self.cache.advance(steps)
        self._pos_host += steps
        return out_host
