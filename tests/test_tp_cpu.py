"""Tensor-parallel sharding on the CPU: every rank's shard holds bit-identical int4 values and scales, the
N-sharded projections concatenate to the whole, and the K-sharded partial sums add up to the whole product.
The two-rank part runs as gloo processes."""

from __future__ import annotations

import dataclasses

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deltaforge_b200 import tp as TP
from deltaforge_b200.config import ModelConfig, hybrid_layer_types
from deltaforge_b200.quant import quantise_int4_k_major
from oracle import ref_ops as R


def test_row_and_column_slices_keep_every_dequantised_weight():
    qw = quantise_int4_k_major(torch.randn(520, 1024, generator=torch.Generator().manual_seed(1)) * 0.05)
    full = R.dequantise_int4_k_major(qw.qweight, qw.scale, qw.group_size)
    for tp in (2, 4):
        rows = [TP.slice_rows(qw, r * 1024 // tp, (r + 1) * 1024 // tp) for r in range(tp)]
        assert all(s.group_size == 128 for s in rows)
        got = torch.cat([R.dequantise_int4_k_major(s.qweight, s.scale, s.group_size) for s in rows], dim=0)
        assert torch.equal(got, full)
    cols = TP.slice_columns(qw, slice(8, 264))
    assert torch.equal(R.dequantise_int4_k_major(cols.qweight, cols.scale, cols.group_size), full[:, 8:264])
    with pytest.raises(ValueError):
        TP.slice_rows(qw, 64, 576)  # not on a scale-group boundary


def test_shard_config_divides_heads_channels_and_vocabulary():
    cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
    loc = TP.shard_config(cfg, 4)
    assert (loc.num_attention_heads, loc.num_key_value_heads) == (cfg.num_attention_heads // 4, cfg.num_key_value_heads // 4)
    assert (loc.linear_num_key_heads, loc.linear_num_value_heads) == (cfg.linear_num_key_heads // 4, cfg.linear_num_value_heads // 4)
    assert loc.intermediate_size == 2304 and loc.vocab_size == 1024 and loc.hidden_size == cfg.hidden_size
    loc8 = TP.shard_config(cfg, 8)  # four KV heads over eight ranks: every head lives on two of them
    assert (loc8.num_attention_heads, loc8.num_key_value_heads, loc8.intermediate_size) == (2, 1, 1152)
    with pytest.raises(ValueError):
        TP.shard_config(cfg, 16)  # 9216 / 16 = 576 rows are not whole 128-row groups
    with pytest.raises(ValueError):
        TP.shard_config(dataclasses.replace(cfg, vocab_size=4098), 4)


def _rank_main(rank: int, world: int, port: int, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)  # the same weights on every rank
        down = quantise_int4_k_major(torch.randn(256, 1024, generator=g) * 0.05)
        x = torch.randn(1, 1024, generator=g).to(torch.bfloat16)
        k0, k1 = rank * 1024 // world, (rank + 1) * 1024 // world
        shard = TP.slice_rows(down, k0, k1)
        dense = R.dequantise_int4_k_major(shard.qweight, shard.scale, shard.group_size).to(torch.bfloat16).float()
        partial = x[:, k0:k1].float() @ dense  # this rank's fp32 partial sum
        dist.all_reduce(partial)
        whole = R.dequant_gemv_int4_fp32(x.unsqueeze(1), down.qweight, down.scale, down.group_size).reshape(1, -1)
        # greedy pick across vocabulary shards: largest value wins, lowest global index on ties
        logits = torch.tensor([[1.0, 5.0, 5.0, 2.0]]) if rank == 0 else torch.tensor([[5.0, 0.0, 7.0, 7.0]])
        val, idx = logits.max(dim=-1)
        best = torch.stack([val, (idx + rank * 4).float()], dim=-1)
        gathered = [torch.zeros_like(best) for _ in range(world)]
        dist.all_gather(gathered, best)
        stacked = torch.stack(gathered)
        vals, ids = stacked[..., 0], stacked[..., 1]
        top = vals.max(dim=0, keepdim=True).values
        pick = torch.where(vals == top, ids, torch.full_like(ids, float("inf"))).min(dim=0).values.long()
        if rank == 0:
            results.put((float((partial - whole.float()).abs().max()), float(whole.abs().max()), int(pick[0])))
    finally:
        dist.destroy_process_group()


def test_two_ranks_partial_sums_and_token_pick():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29600 + (torch.randint(0, 300, (1,)).item())
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, scale, pick = results.get(timeout=10)
    assert err <= 1e-5 * max(scale, 1.0)
    assert pick == 6  # 7.0 at global index 6 (rank 1, local index 2), not the equal value at 7


def test_eight_ranks_replicate_kv_heads_and_split_down_proj_into_nine_groups():
    """Eight ranks over four KV heads and 72 scale groups of ``down_proj``: every rank holds whole groups with the
    parent's values and scales (bit-identical dequantised rows), ranks 2j and 2j+1 hold KV head j and its query
    heads 4j..4j+1 / 4j+2..4j+3, and the vocabulary splits into equal column blocks."""
    from deltaforge_b200 import synth

    cfg = ModelConfig(hidden_size=512, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
    loc = TP.shard_config(cfg, 8)
    assert (loc.num_attention_heads, loc.num_key_value_heads) == (2, 1)
    assert (loc.linear_num_key_heads, loc.linear_num_value_heads) == (2, 4)
    assert loc.intermediate_size == 1152 and loc.vocab_size == 512
    assert [TP.kv_head_range(cfg, r, 8) for r in range(8)] == [(0, 1), (0, 1), (1, 2), (1, 2), (2, 3), (2, 3), (3, 4), (3, 4)]
    full = synth.random_model_weights(cfg, seed=9, device="cpu", scale_dtype=torch.float32)
    shards = [TP.shard_weights(full, r, 8) for r in range(8)]
    for li, lw in enumerate(full.layers):
        # K-sharded projections: the shards' rows, stacked, are the parent's rows
        for name in ("down", "out_proj"):
            parent = getattr(lw, name)
            want = R.dequantise_int4_k_major(parent.qweight, parent.scale, parent.group_size)
            got = torch.cat([R.dequantise_int4_k_major(getattr(s.layers[li], name).qweight, getattr(s.layers[li], name).scale, 128) for s in shards])
            assert torch.equal(got, want)
        assert all(s.layers[li].down.in_features == 1152 and s.layers[li].down.group_size == 128 for s in shards)
        # gate|up: rank r's columns are its 1152 gate channels then its 1152 up channels
        gu = R.dequantise_int4_k_major(lw.gate_up.qweight, lw.gate_up.scale, 128)
        for r, s in enumerate(shards):
            mine = R.dequantise_int4_k_major(s.layers[li].gate_up.qweight, s.layers[li].gate_up.scale, 128)
            assert torch.equal(mine[:, :1152], gu[:, r * 1152 : (r + 1) * 1152])
            assert torch.equal(mine[:, 1152:], gu[:, 9216 + r * 1152 : 9216 + (r + 1) * 1152])
        if lw.kind != "linear_attention":
            d, hq = cfg.head_dim, cfg.num_attention_heads
            w = R.dequantise_int4_k_major(lw.in_proj.qweight, lw.in_proj.scale, 128)
            for r, s in enumerate(shards):
                mine = R.dequantise_int4_k_major(s.layers[li].in_proj.qweight, s.layers[li].in_proj.scale, 128)
                assert mine.shape[1] == 2 * 2 * d + 2 * d
                assert torch.equal(mine[:, : 4 * d], w[:, r * 4 * d : (r + 1) * 4 * d])  # two query heads with their gates
                kv = r // 2
                assert torch.equal(mine[:, 4 * d : 5 * d], w[:, hq * 2 * d + kv * d : hq * 2 * d + (kv + 1) * d])
                assert torch.equal(mine[:, 5 * d :], w[:, hq * 2 * d + 4 * d + kv * d : hq * 2 * d + 4 * d + (kv + 1) * d])
    head = R.dequantise_int4_k_major(full.head.qweight, full.head.scale, full.head.group_size)
    got = torch.cat([R.dequantise_int4_k_major(s.head.qweight, s.head.scale, s.head.group_size) for s in shards], dim=1)
    assert torch.equal(got, head)
    with pytest.raises(ValueError):
        TP.shard_config(cfg, 16)  # 9216 / 16 = 576 rows are not whole 128-row groups
