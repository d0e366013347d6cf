"""Tensor-parallel decode on two GPUs against the single-GPU engine on the same weights.

Both ranks build the same seeded model; rank 0 also runs the unsharded engine; the tensor-parallel logits
(gathered over the vocabulary shards) must match it within the noise of a different summation order, and
the greedy tokens must agree on every rank. With two CUDA devices the ranks sit on one GPU each and reduce
over NCCL; with a single device both ranks share it and reduce over gloo (through the host). The segments
are launched directly in both cases: the kernels never wait on one another across ranks, the host does.
"""

from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rank_main(rank: int, world: int, port: int, results, two_devices: bool, exchange: str = "nccl"):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank if two_devices else 0)
    torch.cuda.set_device(dev)
    if two_devices:
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    else:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        from deltaforge_b200 import engine as E
        from deltaforge_b200 import synth
        from deltaforge_b200 import tp as TP
        from deltaforge_b200.config import ModelConfig, hybrid_layer_types

        cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
        full = synth.random_model_weights(cfg, seed=3, device=dev, scale_dtype=torch.bfloat16)
        ctx_len, steps = 8192, 4  # the context the tensor-parallel benchmark configuration names
        # the whole model's cache, filled with seeded contents, and this rank's slice of it
        whole_cache = E.DecodeCache(cfg, 1, ctx_len + 64, device=dev)
        synth.fill_cache(whole_cache, ctx_len, seed=5)
        local_cfg = TP.shard_config(cfg, world)
        cache = E.DecodeCache(local_cfg, 1, ctx_len + 64, device=dev)
        TP.load_cache_shard(cache, whole_cache, cfg, rank, world)
        eng = TP.TensorParallelEngine(TP.shard_weights(full, rank, world), cache, rank=rank, tp=world, exchange=exchange)
        tok = torch.tensor([17], device=dev)
        tp_logits, tp_tokens = [], []
        t = tok
        for i in range(steps):
            # collectives: launched directly; peer exchange: the first step directly, the rest as one graph replay
            local = eng.step(t, graph=(exchange == "peer" and i > 0)).clone()
            gathered = [torch.zeros_like(local) for _ in range(world)]
            dist.all_gather(gathered, local)
            tp_logits.append(torch.cat(gathered, dim=-1))
            t = eng.engine.tokens.clone()
            tp_tokens.append(t)
        ok = True
        msg = ""
        if rank == 0:
            ref = E.DecodeEngine(full, whole_cache)
            t = tok
            for i in range(steps):
                want = ref.step(t).clone()
                scale = want.float().std().item()
                err = (want.float() - tp_logits[i].float()).abs().max().item()
                if not err < 6e-2 * scale:
                    ok, msg = False, f"step {i}: max logit error {err:.4g} at scale {scale:.4g}"
                t = tp_tokens[i]  # teacher-forced on the tensor-parallel continuation
                if ok and int(want.argmax(-1)) != int(t) and (want.float().topk(2).values.diff().abs().item() > 2 * err):
                    ok, msg = False, f"step {i}: token {int(t)} vs {int(want.argmax(-1))}"
            ref.check_status()
        eng.engine.check_status()
        all_tok = [torch.zeros_like(tp_tokens[-1]) for _ in range(world)]
        dist.all_gather(all_tok, tp_tokens[-1])
        if rank == 0:
            same = all(int(a) == int(all_tok[0]) for a in all_tok)
            results.put((ok and same, msg or ("" if same else "ranks disagree on the token")))
    finally:
        dist.destroy_process_group()


def _run_two_ranks(exchange: str):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29700 + int(torch.randint(0, 200, (1,)).item())
    two = torch.cuda.device_count() >= 2
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results, two, exchange)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:  # a rank that never finished: end exactly the processes this test started
        p.kill()
        p.join(10)
    assert not hung, "a rank did not finish within 150 s"
    assert all(p.exitcode == 0 for p in procs)
    ok, msg = results.get(timeout=10)
    assert ok, msg


def test_tensor_parallel_two_ranks_match_single_gpu():
    _run_two_ranks("nccl")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="kernels of different ranks wait on one another: one GPU per rank")
def test_tensor_parallel_peer_exchange_matches_single_gpu():
    """The ranks add their partial sums and pick the token by peer stores inside the kernels (no collective call)."""
    _run_two_ranks("peer")


def test_peer_exchange_wait_runs_out_and_reports_status():
    """A rank whose peer never shows up: the wait for the peer's partial sums is bounded (about two seconds for
    the first kernel that waits; once the status word is set every later wait gives up at once), the kernels
    return, the engine's status word says 50 and the CUDA context stays usable. The 'peer' here is a second
    local buffer that nothing fills, so no kernel waits for another kernel."""
    from deltaforge_b200 import _lib
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import synth
    from deltaforge_b200 import tp as TP
    from deltaforge_b200.config import ModelConfig, hybrid_layer_types

    dev = torch.device("cuda", 0)
    cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
    full = synth.random_model_weights(cfg, seed=3, device=dev, scale_dtype=torch.bfloat16)
    cache = E.DecodeCache(TP.shard_config(cfg, 2), 1, 64, device=dev)
    nbytes = _lib.load().dfb_engine_tp_exchange_bytes(1, cfg.hidden_size, 2)
    mine = torch.zeros(nbytes // 8, dtype=torch.int64, device=dev)
    absent = torch.zeros_like(mine)  # where rank 1's buffer would be mapped; rank 1's slots of `mine` stay empty
    eng = E.DecodeEngine(TP.shard_weights(full, 0, 2), cache, tp_size=2, tp_rank=0, tp_peer_slots=[mine.data_ptr(), absent.data_ptr()])
    eng.step(torch.tensor([17], device=dev), graph=False)
    with pytest.raises(_lib.Dfb200Error, match="status 50"):
        eng.check_status()
    assert int(absent.ne(0).sum()) > 0  # rank 0 did store its partial sums into the peer's buffer
    assert float(torch.ones(8, device=dev).sum()) == 8.0  # the context still works


def test_tensor_parallel_decode_raises_when_a_peer_never_arrives():
    """The same absent peer through ``TensorParallelEngine.decode``: the call must raise, not hand back tokens
    computed from a residual stream that missed an add. One process stands in for the job (a one-rank gloo
    group carries the barrier and the status reduction); rank 1's buffer is local memory nothing fills."""
    import torch.distributed as dist

    from deltaforge_b200 import _lib
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import synth
    from deltaforge_b200 import tp as TP
    from deltaforge_b200.config import ModelConfig, hybrid_layer_types

    dev = torch.device("cuda", 0)
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29917", rank=0, world_size=1)
    try:
        cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
        full = synth.random_model_weights(cfg, seed=3, device=dev, scale_dtype=torch.bfloat16)
        cache = E.DecodeCache(TP.shard_config(cfg, 2), 1, 64, device=dev)
        nbytes = _lib.load().dfb_engine_tp_exchange_bytes(1, cfg.hidden_size, 2)
        mine = torch.zeros(nbytes // 8, dtype=torch.int64, device=dev)
        absent = torch.zeros_like(mine)
        eng = TP.TensorParallelEngine(TP.shard_weights(full, 0, 2), cache, rank=0, tp=2, exchange="peer",
                                      peer_slots=[mine.data_ptr(), absent.data_ptr()])  # fmt: skip
        with pytest.raises(_lib.Dfb200Error, match="status 50"):
            eng.decode(torch.tensor([17], device=dev), 2)
        assert int(eng.engine.tokens[0]) == -1  # the pick that could not complete left the mark, not a token
        assert float(torch.ones(8, device=dev).sum()) == 8.0  # the context still works
    finally:
        if own_group:
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [4, 8])
def test_sharded_step_emulated_on_one_gpu_matches_the_unsharded_engine(world):
    """All ranks' shards on ONE GPU, driven segment by segment from the host, the fp32 partial sums added in
    rank order between segments (what the all-reduce does): no kernel waits on another, so the eight-rank
    sharding (each KV head on two ranks, nine-group ``down_proj`` shards, 31040... here 512 vocabulary columns per
    rank) is checked against the unsharded engine wherever one GPU is all there is."""
    import ctypes as C

    from deltaforge_b200 import _lib
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import synth
    from deltaforge_b200 import tp as TP
    from deltaforge_b200.config import ModelConfig, hybrid_layer_types

    dev = torch.device("cuda", 0)
    lib = _lib.load()
    cfg = ModelConfig(hidden_size=2560, intermediate_size=9216, num_hidden_layers=4, vocab_size=4096, layer_types=hybrid_layer_types(4))
    full = synth.random_model_weights(cfg, seed=3, device=dev, scale_dtype=torch.bfloat16)
    ctx_len, steps = 1000, 3
    whole_cache = E.DecodeCache(cfg, 1, ctx_len + 16, device=dev)
    synth.fill_cache(whole_cache, ctx_len, seed=5)
    local_cfg = TP.shard_config(cfg, world)
    engines, partials = [], []
    for r in range(world):
        cache = E.DecodeCache(local_cfg, 1, ctx_len + 16, device=dev)
        TP.load_cache_shard(cache, whole_cache, cfg, r, world)
        eng = E.DecodeEngine(TP.shard_weights(full, r, world), cache, tp_size=world, tp_rank=r)
        off = lib.dfb_engine_partial_buffer(eng._handle) - eng.workspace.data_ptr()
        partials.append(eng.workspace[off : off + 4 * cfg.hidden_size].view(torch.float32))
        engines.append(eng)
    ref = E.DecodeEngine(full, whole_cache)
    segments = lib.dfb_engine_num_segments(engines[0]._handle)
    assert segments == 2 * cfg.num_hidden_layers + 1
    stream = torch.cuda.current_stream(dev).cuda_stream
    tok = torch.tensor([17], device=dev)
    for _ in range(steps):
        for eng in engines:
            eng.cache.ensure_capacity(1)
            eng._sync_position()
            eng._set_tokens(tok)
        for seg in range(segments):
            for eng in engines:
                _lib.check(lib.dfb_engine_step_segment(eng._handle, seg, C.c_void_p(stream)), "dfb_engine_step_segment")
            if seg + 1 < segments:
                total = partials[0].clone()
                for p in partials[1:]:
                    total += p  # rank order, fp32
                for p in partials:
                    p.copy_(total)
        for eng in engines:
            eng.cache.advance(1)
            eng._pos_host += 1
        logits = torch.cat([eng.logits for eng in engines], dim=-1)
        want = ref.step(tok).clone()
        scale = want.float().std().item()
        err = (want.float() - logits.float()).abs().max().item()
        assert err < 6e-2 * scale, f"max logit error {err:.4g} at scale {scale:.4g}"
        if want.float().topk(2).values.diff().abs().item() > 2 * err:
            assert int(logits.float().argmax(-1)) == int(want.argmax(-1))
        tok = want.argmax(-1).reshape(1)
    for eng in engines + [ref]:
        eng.check_status()
    # the KV rows written during the steps: a head that lives on two ranks holds the same rows on both
    if world == 8:
        a = E.cache_layer_tensors(engines[0].cache.layers[3])["keys"]
        b = E.cache_layer_tensors(engines[1].cache.layers[3])["keys"]
        assert torch.equal(a, b)
