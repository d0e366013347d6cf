"""Tensor parallelism for the decode step: one process per GPU, every rank a shard of every layer.

Sharding (the reference has no multi-GPU path; this follows its tensor shapes, src/deltaforge/reference.py:
477-494, 592-605, 688-690): attention by query / KV head, DeltaNet by key / value head (value head ``h``
uses key head ``h // (Hv / Hk)``, so a rank that owns a contiguous block of value heads owns the matching
block of key heads), the MLP by intermediate channel, the tied head by vocabulary slice. Projections that
produce per-head or per-channel outputs are sliced along N, which in the K-major int4 layout is a plain
column slice of ``packed`` and ``scale``. The projections back to the hidden size (``out_proj`` / ``o_proj``,
``down_proj``) are sliced along K on scale-group boundaries and re-packed, so every rank holds bit-identical
int4 values and scales of its rows; each rank's product is a partial sum over its rows, the partial sums are
added across ranks in fp32 (two all-reduces per layer), and the sum is rounded to bf16 and added to the
residual stream exactly where the unsharded projection would have been. Norm weights, the embedding table
and the residual stream are replicated. Greedy sampling compares each rank's best logit.

Two forms of the exchange. ``exchange="nccl"``: the partial sums are added by ``torch.distributed.all_reduce``
on the engine's stream between segments; kernels and collectives can be recorded into one CUDA graph per
token (``graph=True``). ``exchange="peer"``: the K-sharded projection's epilogue stores every partial sum,
tagged with an epoch, into a buffer of every rank (symmetric memory), and the next kernel polls its own
buffer (bounded) and adds the ranks' values in rank order; the token pick exchanges (logit, index) the same
way. No collective call remains and the token is one CUDA graph of this library's kernels. The peer form
needs one GPU per rank, because the ranks' kernels wait on one another.
"""

from __future__ import annotations

import dataclasses

import torch
from torch import Tensor

from . import _lib
from .config import LINEAR_ATTENTION
from .engine import DecodeCache, DecodeEngine, LayerWeights, ModelWeights
from .quant import QuantisedWeight

BF16 = torch.bfloat16


# --------------------------------------------------------------------------------------
# sharding of shapes and weights (pure tensor code: runs on any device)
# --------------------------------------------------------------------------------------


def kv_heads_per_rank(cfg, tp: int) -> int:
    """KV heads a rank holds: its share, or one replicated head when there are more ranks than KV heads."""
    hkv = cfg.num_key_value_heads
    if hkv % tp == 0:
        return hkv // tp
    if tp % hkv == 0 and (cfg.num_attention_heads // hkv) % (cfg.num_attention_heads // tp) == 0:
        return 1  # tp / hkv consecutive ranks share one KV head; each takes some of its query heads
    raise ValueError(f"num_key_value_heads = {hkv} neither divides over nor is replicated evenly across {tp} ranks")


def shard_config(cfg, tp: int):
    """The model configuration one of ``tp`` ranks sees: its share of heads, MLP channels and vocabulary.

    With more ranks than KV heads (eight ranks, four KV heads) every KV head lives on ``tp / hkv`` consecutive
    ranks: each of them projects, caches and reads that head's keys and values and owns a disjoint part of
    the head's query heads, so the rank still sees whole GQA groups and nothing crosses ranks before ``o_proj``."""
    for name in ("num_attention_heads", "linear_num_key_heads", "linear_num_value_heads", "intermediate_size", "vocab_size"):
        if getattr(cfg, name) % tp:
            raise ValueError(f"{name} = {getattr(cfg, name)} does not divide over {tp} ranks")
    if (cfg.intermediate_size // tp) % 128 or (cfg.linear_num_value_heads // tp * cfg.linear_value_head_dim) % 128:
        raise ValueError("K-sharded projections must keep whole 128-row scale groups on every rank")
    return dataclasses.replace(
        cfg,
        num_attention_heads=cfg.num_attention_heads // tp,
        num_key_value_heads=kv_heads_per_rank(cfg, tp),
        linear_num_key_heads=cfg.linear_num_key_heads // tp,
        linear_num_value_heads=cfg.linear_num_value_heads // tp,
        intermediate_size=cfg.intermediate_size // tp,
        vocab_size=cfg.vocab_size // tp,
    )


def unpack_k_major(packed: Tensor) -> Tensor:
    """``packed [K/2, N]`` -> the stored nibbles ``[K, N]`` (still value + 8), uint8."""
    return torch.cat([packed & 0xF, packed >> 4], dim=0)


def pack_k_major(nibbles: Tensor) -> Tensor:
    """Stored nibbles ``[K, N]`` -> ``packed [K/2, N]``: row ``j`` low, row ``j + K/2`` high."""
    half = nibbles.shape[0] // 2
    return (nibbles[:half] | (nibbles[half:] << 4)).contiguous()


def slice_columns(qw: QuantisedWeight, cols: Tensor | slice) -> QuantisedWeight:
    return QuantisedWeight(qw.qweight[:, cols].contiguous(), qw.scale[:, cols].contiguous(), qw.bits, qw.group_size)


def slice_rows(qw: QuantisedWeight, k0: int, k1: int) -> QuantisedWeight:
    """Rows ``[k0, k1)`` of the weight (whole scale groups), re-packed K-major: same nibbles, same scales.

    The shard keeps the parent's group size even where the reference's own packer would not pick it for a
    matrix of that depth (``down_proj`` over eight ranks is 1152 rows = nine groups, an odd count, which
    ``group_size_for`` refuses): a shard never goes through that packer, its groups are the parent's."""
    g = qw.group_size
    if k0 % g or k1 % g:
        raise ValueError(f"row slice [{k0}, {k1}) does not fall on {g}-row scale groups")
    if (k1 - k0) % 2:
        raise ValueError(f"a {k1 - k0}-row shard cannot be packed two rows to a byte")
    nib = unpack_k_major(qw.qweight)[k0:k1]
    return QuantisedWeight(pack_k_major(nib), qw.scale[k0 // g : k1 // g].contiguous(), qw.bits, g)


def _cat(parts: list[Tensor], device) -> Tensor:
    return torch.cat([p.to(device) for p in parts])


def shard_layer(lw: LayerWeights, cfg, rank: int, tp: int) -> LayerWeights:
    dev = lw.in_proj.qweight.device
    ar = lambda a, b: torch.arange(a, b, device=dev)  # noqa: E731
    inter = cfg.intermediate_size
    i0, i1 = rank * inter // tp, (rank + 1) * inter // tp
    gate_up = slice_columns(lw.gate_up, _cat([ar(i0, i1), ar(inter + i0, inter + i1)], dev))
    down = slice_rows(lw.down, i0, i1)
    if lw.kind == LINEAR_ATTENTION:
        hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        k0, k1 = rank * hk // tp, (rank + 1) * hk // tp
        v0, v1 = rank * hv // tp, (rank + 1) * hv // tp
        kd, vd = hk * dk, hv * dv
        qkv = [ar(k0 * dk, k1 * dk), ar(kd + k0 * dk, kd + k1 * dk), ar(2 * kd + v0 * dv, 2 * kd + v1 * dv)]
        cols = _cat(qkv + [ar(2 * kd + vd + v0 * dv, 2 * kd + vd + v1 * dv), ar(2 * kd + 2 * vd + v0, 2 * kd + 2 * vd + v1),
                           ar(2 * kd + 2 * vd + hv + v0, 2 * kd + 2 * vd + hv + v1)], dev)  # fmt: skip
        return LayerWeights(
            kind=lw.kind, input_norm=lw.input_norm, post_norm=lw.post_norm,
            in_proj=slice_columns(lw.in_proj, cols), out_proj=slice_rows(lw.out_proj, v0 * dv, v1 * dv), gate_up=gate_up, down=down,
            conv_w=lw.conv_w[_cat(qkv, dev)].contiguous(), a_log=lw.a_log[v0:v1].contiguous(), dt_bias=lw.dt_bias[v0:v1].contiguous(),
            gnorm_w=lw.gnorm_w, gnorm_w_is_bf16=lw.gnorm_w_is_bf16,
        )  # fmt: skip
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qw = 2 * d if cfg.attn_output_gate else d
    q0, q1 = rank * hq // tp, (rank + 1) * hq // tp
    g0, g1 = kv_head_range(cfg, rank, tp)  # with more ranks than KV heads: the one head all its query heads belong to
    cols = _cat([ar(q0 * qw, q1 * qw), ar(hq * qw + g0 * d, hq * qw + g1 * d), ar(hq * qw + hkv * d + g0 * d, hq * qw + hkv * d + g1 * d)], dev)
    return LayerWeights(
        kind=lw.kind, input_norm=lw.input_norm, post_norm=lw.post_norm,
        in_proj=slice_columns(lw.in_proj, cols), out_proj=slice_rows(lw.out_proj, q0 * d, q1 * d), gate_up=gate_up, down=down,
        q_norm=lw.q_norm, k_norm=lw.k_norm,
    )  # fmt: skip


def shard_weights(weights: ModelWeights, rank: int, tp: int) -> ModelWeights:
    """Rank ``rank``'s shard of the model (``weights`` is the whole model, on any device)."""
    cfg = weights.config
    local = shard_config(cfg, tp)
    v0, v1 = rank * cfg.vocab_size // tp, (rank + 1) * cfg.vocab_size // tp
    out = ModelWeights(local, weights.embed, weights.final_norm, slice_columns(weights.head, slice(v0, v1)), weights.inv_freq)
    out.layers = [shard_layer(lw, cfg, rank, tp) for lw in weights.layers]
    return out


def kv_head_range(cfg, rank: int, tp: int) -> tuple[int, int]:
    """The KV heads ``[g0, g1)`` of the unsharded model that rank ``rank`` holds."""
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    if hkv % tp == 0:
        return rank * hkv // tp, (rank + 1) * hkv // tp
    kv_heads_per_rank(cfg, tp)  # raises if the replicated layout does not apply
    g0 = (rank * hq // tp) // (hq // hkv)
    return g0, g0 + 1


@torch.no_grad()
def load_cache_shard(local_cache, whole_cache, cfg, rank: int, tp: int) -> None:
    """Fill rank ``rank``'s cache (built for ``shard_config(cfg, tp)``) from an unsharded cache of ``cfg``: its KV
    heads, its conv channels (the q, k and v blocks of its key / value heads) and its value heads' state."""
    from .engine import cache_layer_tensors

    hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    g0, g1 = kv_head_range(cfg, rank, tp)
    k0, k1, v0, v1 = rank * hk // tp, (rank + 1) * hk // tp, rank * hv // tp, (rank + 1) * hv // tp
    kd = hk * dk
    for wl, ll in zip(whole_cache.layers, local_cache.layers):
        wt, lt = cache_layer_tensors(wl), cache_layer_tensors(ll)
        if "keys" in wt:
            n = min(lt["keys"].shape[2], wt["keys"].shape[2])
            lt["keys"][:, :, :n].copy_(wt["keys"][:, g0:g1, :n])
            lt["values"][:, :, :n].copy_(wt["values"][:, g0:g1, :n])
        else:
            dev = wt["conv"].device
            rows = torch.cat([torch.arange(k0 * dk, k1 * dk), torch.arange(kd + k0 * dk, kd + k1 * dk),
                              torch.arange(2 * kd + v0 * dv, 2 * kd + v1 * dv)]).to(dev)  # fmt: skip
            lt["conv"].copy_(wt["conv"][:, rows])
            lt["recurrent"].copy_(wt["recurrent"][:, v0:v1])
    local_cache.seq_len = whole_cache.seq_len


def weights_to(weights: ModelWeights, device) -> ModelWeights:
    """Move a (sharded) weight set to ``device``."""

    def q(w: QuantisedWeight) -> QuantisedWeight:
        return QuantisedWeight(w.qweight.to(device), w.scale.to(device), w.bits, w.group_size)

    def t(x):
        return None if x is None else x.to(device)

    out = ModelWeights(weights.config, weights.embed.to(device), weights.final_norm.to(device), q(weights.head), weights.inv_freq.to(device))
    for lw in weights.layers:
        out.layers.append(
            LayerWeights(
                kind=lw.kind, input_norm=t(lw.input_norm), post_norm=t(lw.post_norm), in_proj=q(lw.in_proj), out_proj=q(lw.out_proj),
                gate_up=q(lw.gate_up), down=q(lw.down), conv_w=t(lw.conv_w), a_log=t(lw.a_log), dt_bias=t(lw.dt_bias),
                gnorm_w=t(lw.gnorm_w), gnorm_w_is_bf16=lw.gnorm_w_is_bf16, q_norm=t(lw.q_norm), k_norm=t(lw.k_norm),
            )  # fmt: skip
        )
    return out


# --------------------------------------------------------------------------------------
# the engine of one rank
# --------------------------------------------------------------------------------------


class TensorParallelEngine:
    """One rank of a tensor-parallel decode step (batch 1..N, greedy).

    ``local_weights`` / ``cache`` hold this rank's shard (``shard_weights``, ``DecodeCache(shard_config(cfg, tp), ...)``);
    ``group`` is a ``torch.distributed`` process group whose backend can reduce CUDA tensors (NCCL).
    """

    def __init__(self, local_weights: ModelWeights, cache: DecodeCache, *, rank: int, tp: int, group=None, exchange: str = "nccl",
                 peer_slots: list[int] | None = None) -> None:  # fmt: skip
        """``exchange``: ``"nccl"`` adds the partial sums with ``torch.distributed.all_reduce`` between segments;
        ``"peer"`` gives every rank a symmetric exchange buffer (``torch.distributed._symmetric_memory``) and lets
        the kernels store into their peers' buffers and wait for one another: no collective call remains and the
        whole token is one CUDA graph of this library's kernels. ``"peer"`` needs one GPU per rank. ``peer_slots``:
        for callers that map the ranks' exchange buffers themselves, the ``tp`` device pointers (entry ``rank`` is
        this rank's own zeroed buffer of ``dfb_engine_tp_exchange_bytes``); without it symmetric memory is used."""
        import torch.distributed as dist

        if exchange not in ("nccl", "peer"):
            raise ValueError(f"exchange must be 'nccl' or 'peer', got {exchange!r}")
        self.dist, self.group, self.rank, self.tp, self.exchange = dist, group, rank, tp, exchange
        self.cache = cache
        self.vocab_local = local_weights.config.vocab_size
        hidden = local_weights.config.hidden_size
        peer_ptrs = None
        if exchange == "peer" and peer_slots is not None:
            if len(peer_slots) != tp:
                raise ValueError(f"peer_slots must hold {tp} device pointers, got {len(peer_slots)}")
            peer_ptrs = [int(p) for p in peer_slots]
        elif exchange == "peer":
            import torch.distributed._symmetric_memory as symm_mem

            lib = _lib.load()
            dev = local_weights.embed.device
            nbytes = lib.dfb_engine_tp_exchange_bytes(cache.batch_size, hidden, tp)
            self.exchange_buffer = symm_mem.empty(nbytes // 8, dtype=torch.int64, device=dev)
            self.exchange_buffer.zero_()
            torch.cuda.synchronize(dev)
            handle = symm_mem.rendezvous(self.exchange_buffer, group if group is not None else dist.group.WORLD)
            peer_ptrs = [int(p) for p in handle.buffer_ptrs]
            self._symm_handle = handle
            dist.barrier(group=group)  # every rank's buffer is zeroed and mapped before anyone stores into it
        self.engine = DecodeEngine(local_weights, cache, tp_size=tp, tp_rank=rank, tp_peer_slots=peer_ptrs)
        self.lib = self.engine.lib
        dev = self.engine.device
        if exchange == "nccl":
            ptr = self.lib.dfb_engine_partial_buffer(self.engine._handle)
            off = ptr - self.engine.workspace.data_ptr()
            n = self.engine.batch * hidden
            self.partial = self.engine.workspace[off : off + 4 * n].view(torch.float32)  # the fp32 partial sums, in place
        self.segments = self.lib.dfb_engine_num_segments(self.engine._handle)
        self.best = torch.zeros((self.engine.batch, 2), dtype=torch.float32, device=dev)
        self.gathered = torch.zeros((tp, self.engine.batch, 2), dtype=torch.float32, device=dev)
        self._graph = None
        self._warm = False
        self._lined_up = False
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def _line_up(self) -> None:
        """Peer exchange: the ranks' kernels wait on one another with a limit of about two seconds, so the hosts
        must not start a step further apart than that. Everything slow and rank-local (graph capture) is done
        first, then the ranks meet at a barrier; called at the start of every ``decode`` and of the first ``step``."""
        eng = self.engine
        if not eng._captured:
            eng.capture()
        torch.cuda.synchronize(eng.device)
        self.dist.barrier(group=self.group)
        self._lined_up = True

    def check_status(self) -> None:
        """Synchronise, combine the ranks' status words (maximum) and raise on every rank if any rank's kernels
        gave up a wait: a rank that timed out has skipped a residual add, and what it stored for its peers
        afterwards is wrong although their own status words stay zero."""
        code = _lib.C.c_int(0)
        _lib.check(self.lib.dfb_engine_status(self.engine._handle, _lib.C.byref(code), self.engine._stream()), "dfb_engine_status")
        self._flag.fill_(code.value)
        self.dist.all_reduce(self._flag, op=self.dist.ReduceOp.MAX, group=self.group)
        worst = int(self._flag.item())
        if worst:
            raise _lib.Dfb200Error(
                f"tensor-parallel step failed: a rank's kernels reported status {worst} (50: a peer's partial sums did not "
                f"arrive within the wait limit; this rank's own status is {code.value}). Tokens, caches and recurrent state "
                "after that point are not valid."
            )

    def _run(self) -> None:
        stream = torch.cuda.current_stream(self.engine.device).cuda_stream
        for seg in range(self.segments):
            _lib.check(self.lib.dfb_engine_step_segment(self.engine._handle, seg, stream), "dfb_engine_step_segment")
            if seg + 1 < self.segments:
                self.dist.all_reduce(self.partial, group=self.group)
        # greedy pick across the vocabulary shards: the largest logit wins, the lowest global index on ties
        val, idx = self.engine.logits.float().max(dim=-1)
        self.best[:, 0] = val
        self.best[:, 1] = (idx + self.rank * self.vocab_local).float()  # exact: vocabulary sizes are far below 2^24
        self.dist.all_gather_into_tensor(self.gathered.view(-1), self.best.view(-1), group=self.group)
        vals, ids = self.gathered[..., 0], self.gathered[..., 1]
        top = vals.max(dim=0, keepdim=True).values
        masked = torch.where(vals == top, ids, torch.full_like(ids, float("inf")))
        self.engine.tokens.copy_(masked.min(dim=0).values.long())

    def step(self, tokens: Tensor, *, graph: bool = False, check: bool = False) -> Tensor:
        """One token for every sequence; returns this rank's slice of the logits ``[batch, vocab / tp]``.
        ``check`` (peer exchange): wait for the step and raise if any rank's kernels gave up a wait.

        By default the segments and the collectives between them are launched directly. With ``graph=True`` the
        first call still runs directly (that also sets NCCL's channels up) and from the second call on one CUDA
        graph per token, collectives included, is replayed."""
        eng = self.engine
        if self.exchange == "peer":  # the engine's own step: kernels only
            if not self._lined_up:
                self._line_up()
            out = eng.step(tokens, graph=True)
            if check:
                self.check_status()
            return out
        self.cache.ensure_capacity(1)
        eng._sync_position()
        eng._set_tokens(tokens)
        if graph and self._warm:
            if self._graph is None:
                # Recording collectives into a CUDA graph is something only NCCL can do: any other backend moves the data
                # through the host and synchronises the stream, which a capturing stream refuses, and the rank that gets
                # that error leaves its peers waiting inside their next collective.
                if self.dist.get_backend(self.group) != "nccl":
                    raise ValueError("graph=True records the all-reduces into a CUDA graph and needs the NCCL backend")
                # Every rank enters the capture together, with nothing of the warm step still queued, and the capture is
                # thread-local: NCCL's watchdog thread polls CUDA events, which under the default (global) mode
                # invalidates a capture in progress on one rank only, again leaving the others waiting.
                torch.cuda.synchronize(eng.device)
                self.dist.barrier(group=self.group)
                self._graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self._graph, capture_error_mode="thread_local"):  # recorded, not executed
                    self._run()
            self._graph.replay()
        else:
            self._run()
            self._warm = True
        self.cache.advance(1)
        eng._pos_host += 1
        return eng.logits

    def decode(self, tokens: Tensor, steps: int, *, graph: bool = False, check: bool = True) -> Tensor:
        """Greedy loop on the device: returns the chosen tokens ``[batch, steps]`` (identical on every rank).
        With the peer exchange the ranks line up at a barrier first and, unless ``check`` is off, the call waits for
        the tokens and raises on every rank if any rank's kernels gave up a wait."""
        if self.exchange == "peer":
            self._line_up()
            out = self.engine.decode(tokens, steps)
            if check:
                self.check_status()
            return out
        out = []
        t = tokens
        for _ in range(steps):
            self.step(t, graph=graph)
            t = self.engine.tokens.clone()
            out.append(t)
        return torch.stack(out, dim=1)
