"""Benchmark of the int4 decode step: one JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): the full Qwen3.5-4B-shaped int4 decode step at batch 1 with a
4096-token context, synthetic random-init weights and caches
(``deltaforge_b200.synth``). A "step" is one decode step = one token per sequence, run as one replay of
the captured CUDA graph. With N > 1 GPUs every rank decodes its own independent sequence (no
collectives on the data path, weak scaling); the timed region is bracketed by a barrier and a device
synchronise, timed with CUDA events on the launching stream, and the maximum over ranks is reported.

Keys beyond the common contract:
  e2e            the same metric through ``dfb_engine_decode_host``: per step the input token is
                 copied from pinned host memory, the graph runs, the chosen token is copied back and
                 waited for.
  roofline       the int4 GEMV kernel on its largest launch of the step (the LM head, 328 MB), timed
                 alone with CUDA events in this process.
  roofline_step  the whole step: algorithmic bytes per token / device time per token.
  cpu_baseline   the CPU port of the reference's PyTorch path (``oracle/``) timed on this machine's host
                 cores on a bounded sample of the same step.

``--impl reference`` times that CPU port as the measured arm; it runs on rank 0 only.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

CONTEXT = 4096
BATCH = 1
WORKLOAD = "qwen3.5-4b int4 decode step, batch 1, ctx 4096: 32 layers [3 Gated DeltaNet : 1 gated attention], hidden 2560, vocab 248320"
METRIC = "decode tokens/s (bs1, 4K ctx)"


# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of these kernels on these matrices (records of
# those captures, not re-measured by a bench run). Head: mean of two captured launches. Layer projections: 24 DeltaNet
# layers at 16.733 + 5.469 + 24.390 + 12.238 MB and 8 attention layers at 13.576 + 5.602 + 24.390 + 12.238 MB, over the
# 128 launches of one token; these kernels write nothing to DRAM (their output rows stay in the L2).
HEAD_GEMV_DRAM_BYTES_PER_LAUNCH = 327_891_968 + 4_020_096
LAYER_GEMV_DRAM_BYTES_PER_LAUNCH = 14_518_700


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# CPU port of the reference (reported baseline, and the --impl reference arm)
# --------------------------------------------------------------------------------------


def cpu_sample_model(head_fraction: int):
    """A 2-layer (one DeltaNet, one full-attention) model at the benchmark widths with a 1/head_fraction
    slice of the vocabulary, int4 on every linear through the oracle's torch-expression installer."""
    from deltaforge_b200.config import FULL_ATTENTION, LINEAR_ATTENTION, ModelConfig
    from oracle import ref_model as M

    cfg = ModelConfig(
        hidden_size=2560, intermediate_size=9216, num_hidden_layers=2, vocab_size=248320 // head_fraction,
        layer_types=(LINEAR_ATTENTION, FULL_ATTENTION), name="cpu-sample",
    )  # fmt: skip
    torch.manual_seed(0)
    model = M.OracleModel(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name or name.endswith("dt_bias") or name.endswith("A_log"):
                continue
            p.copy_(torch.randn(p.shape) * (p.shape[-1] ** -0.5))
    model = M.install_int4_everywhere(model.to(torch.bfloat16).eval())
    cache = model.new_cache(BATCH, CONTEXT + 64)
    for t in cache.state_tensors():
        t.copy_(torch.randn(t.shape) * 0.1)
    cache.seq_len = CONTEXT
    return model, cache, cfg


def cpu_step_seconds(model, cache, head_fraction: int, repeats: int, whole: bool) -> list[float]:
    """Seconds for one token, measured ``repeats`` times on the sample model.

    ``whole``: a token's worth of work is actually executed, the DeltaNet sample layer 24 times, the attention sample
    layer (ctx 4096) 8 times and the 1/head_fraction slice of the LM head head_fraction times, and timed as one
    region. Otherwise one pass over each is timed and scaled (24x, 8x, head_fraction x): an extrapolation."""
    from oracle import ref_ops as R

    tok = torch.zeros((BATCH, 1), dtype=torch.long)
    out = []
    for _ in range(repeats):
        cache.seq_len = CONTEXT
        h = model.embed_tokens(tok)
        pos = torch.full((BATCH, 1), CONTEXT)
        cos, sin = R.rope_cos_sin(pos, model.inv_freq, h.dtype)
        if whole:
            t0 = time.perf_counter()
            for _ in range(24):
                h = model.layers[0](h, cos, sin, cache, CONTEXT)
            for _ in range(8):
                h = model.layers[1](h, cos, sin, cache, CONTEXT)
            hn = R.rms_norm(h, model.norm.weight, model.norm.eps)
            for _ in range(head_fraction):
                model.project_logits(hn)
            out.append(time.perf_counter() - t0)
            continue
        t0 = time.perf_counter()
        h1 = model.layers[0](h, cos, sin, cache, CONTEXT)
        t1 = time.perf_counter()
        h2 = model.layers[1](h1, cos, sin, cache, CONTEXT)
        t2 = time.perf_counter()
        model.project_logits(R.rms_norm(h2, model.norm.weight, model.norm.eps))
        t3 = time.perf_counter()
        out.append(24 * (t1 - t0) + 8 * (t2 - t1) + head_fraction * (t3 - t2))
    return out


def usable_host_cores() -> int:
    """Cores this process may use: its affinity mask, capped by the cgroup CPU quota when there is one."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        quota, period = Path("/sys/fs/cgroup/cpu.max").read_text().split()[:2]
        if quota != "max":
            n = min(n, max(1, int(quota) // int(period)))
    except (OSError, ValueError):
        pass
    return max(1, n)


def run_cpu_port(steps: int, warmup: int, budget_s: float) -> dict:
    """Time the CPU port for ``steps`` steps after ``warmup``. Whole tokens are executed when that fits ``budget_s``;
    otherwise one pass over the sample is timed per step and scaled, and the result says ``extrapolated``."""
    # torchrun pins OMP_NUM_THREADS to 1; this arm runs on one rank alone and takes every host core
    torch.set_num_threads(max(torch.get_num_threads(), usable_host_cores()))
    threads = torch.get_num_threads()
    head_fraction = 8
    model, cache, _ = cpu_sample_model(head_fraction)
    region_t0 = time.perf_counter()
    with torch.no_grad():
        first = cpu_step_seconds(model, cache, head_fraction, 1, whole=False)[0]  # also first-touches the temporaries
        estimate = cpu_step_seconds(model, cache, head_fraction, 1, whole=False)[0]
        whole = estimate * (steps + warmup) <= budget_s
        cpu_step_seconds(model, cache, head_fraction, max(0, warmup - (0 if whole else 1)), whole)
        times = cpu_step_seconds(model, cache, head_fraction, steps, whole)
    sec = sum(times) / len(times)
    work = "the DeltaNet sample layer 24 times, the attention sample layer (ctx %d) 8 times, the LM head in %d column slices" % (CONTEXT, head_fraction)
    return {
        "value": BATCH / sec,
        "unit": "tokens/s",
        "cores": threads,
        "kind": "port",
        "extrapolated": not whole,
        "sample": (
            (f"per step one token's worth of work is executed and timed as a whole: {work}" if whole else
             f"per step ONE pass over a DeltaNet layer, an attention layer (ctx {CONTEXT}) and 1/{head_fraction} of the LM head is timed "
             f"and scaled to 24 + 8 layers + the whole head")
            + f"; a two-layer model at the benchmark's widths through oracle/ (torch CPU, {threads} threads); {steps} timed steps"
        ),
        "seconds_per_token": sec,
        "timed_seconds": time.perf_counter() - region_t0,
        "first_pass_seconds": first,
    }


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        # NCCL prints its version banner on stdout at this level; stdout carries the one JSON line only
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, rank, world, local
    return None, 0, 1, 0


def time_head_gemv(weights, iters: int = 30) -> tuple[float, int]:
    """Average device time (ms) of the LM-head GEMV launch, alone, and its algorithmic bytes."""
    from deltaforge_b200 import ops
    from deltaforge_b200.bytes_model import gemv_bytes

    head = weights.head
    k, n = head.in_features, head.out_features
    x = torch.randn((1, k), device=head.qweight.device).to(torch.bfloat16)
    nw = weights.final_norm
    if head.k8 is None:
        head.k8 = ops.int4_repack_k8(head.qweight)

    def call():  # the launch the decode step makes for the head: final RMSNorm fused, streaming kernel
        return ops.int4_gemv_fused(
            x, head.qweight, head.scale, head.group_size, prologue=ops.PRO_RMSNORM, norm_weight=nw, eps=1e-6, packed_k8=head.k8
        )

    for _ in range(5):
        call()
    torch.cuda.synchronize()
    # `iters` launches recorded into one CUDA graph, so that the host's per-call cost is outside the timed region.
    # A one-element torch kernel between them keeps consecutive launches from overlapping through programmatic
    # dependent launch (in the decode step the head runs once per token, after other kernels); its microsecond
    # is counted against the GEMV.
    tick = torch.zeros(1, device=x.device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            call()
            tick.add_(1.0)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 4
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * reps), gemv_bytes(k, n, rows=1, scale_bytes=head.scale.element_size())


def run_ours(args) -> dict | None:
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import qwen3_5_4b_config, synth
    from deltaforge_b200.bytes_model import decode_bytes_per_step

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the decode step has no CPU path")
    dist, rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = qwen3_5_4b_config() if args.layers is None else qwen3_5_4b_config(num_hidden_layers=args.layers)
    steps, warmup = args.steps, max(args.warmup, 3)
    weights = synth.random_model_weights(cfg, seed=1234 + rank, device=dev, scale_dtype=torch.bfloat16)
    cache = E.DecodeCache(cfg, BATCH, CONTEXT + steps + warmup + 8, device=dev)
    synth.fill_cache(cache, CONTEXT, seed=77 + rank)
    snap = cache.snapshot()
    eng = E.DecodeEngine(weights, cache, prefetch_distance=args.prefetch_distance,
                         tensor_core_gemv=not args.no_tensor_core_gemv)
    tok = torch.full((BATCH,), 1000 + rank, dtype=torch.int64, device=dev)
    eng.capture()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up, then the device-timed region: K replays of the graph, each consuming the previous token
    eng.decode(tok, warmup)
    cache.restore(snap)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clocks:
        e0.record()
        generated = eng.decode(tok, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if steps * 0.5 < 400:  # keep the sampler alive for a few hundred ms so it sees clocks under load
            cache.restore(snap)
            eng.decode(tok, min(steps, 256))
            torch.cuda.synchronize()
    barrier()
    eng.check_status()  # a kernel whose bounded wait gave up makes the number meaningless: raise, do not print it
    finite = bool(torch.isfinite(eng.logits.float()).all())

    # end to end through the C ABI with host buffers
    cache.restore(snap)
    host_tok = tok.cpu().pin_memory()
    out_host = torch.empty((steps, BATCH), dtype=torch.int64).pin_memory()
    eng.decode_host(host_tok, min(warmup, 8), torch.empty((min(warmup, 8), BATCH), dtype=torch.int64).pin_memory())
    cache.restore(snap)
    barrier()
    t0 = time.perf_counter()
    eng.decode_host(host_tok, steps, out_host)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    eng.check_status()
    same = bool(torch.equal(out_host.t().to(dev), generated))

    times = torch.tensor([ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = times.tolist()

    head_ms, head_bytes = time_head_gemv(weights) if rank == 0 else (0.0, 0)
    launches_per_step, attn_splits = eng.launches_per_step, eng.attn_splits
    proj_stats = None
    if rank == 0:
        # After every timed region: re-capture the step with the kernels' per-CTA timestamp marks on, run a few tokens, and
        # read the last one launch by launch. A launch's time is its share of the step's critical path: from the last
        # exit of the launch before it to its own last exit.
        from deltaforge_b200 import timeline as TL

        cache.restore(snap)
        trace = eng.set_trace()
        eng.decode(tok, 4)
        torch.cuda.synchronize()
        rows = TL.summarise(trace, TL.launch_names(list(cfg.layer_types), launches_per_step))
        eng.set_trace(0)
        if args.timeline:
            Path(args.timeline).write_text(TL.render(rows) + "\n")
        proj = [r for r in rows if r["name"].split(".")[-1] in ("in_proj", "out_proj", "gate_up", "down") and "chain" in r and "boundary" in r]
        if proj:
            layer_bytes = sum(
                q.qweight.numel() + q.scale.numel() * q.scale.element_size() + 2 * q.out_features
                for L in weights.layers for q in (L.in_proj, L.out_proj, L.gate_up, L.down)
            )  # fmt: skip
            proj_stats = {"launches": len(proj), "us": sum(r["chain"] + r["boundary"] for r in proj),
                          "bytes": layer_bytes * len(proj) / (4 * len(weights.layers))}  # fmt: skip
    tp_line = None
    if dist is not None and not args.no_tp_arm and BATCH == 1:
        # the multi-GPU run also reports the tensor-parallel form of the same model on the same GPUs
        del eng, cache, snap
        torch.cuda.empty_cache()
        try:
            tp_line = tp_arm(dist, rank, world, dev, min(steps, 64), min(warmup, 8), args.layers)
        except Exception as exc:  # the data-parallel line stands on its own
            tp_line = {"n": world, "error": f"{type(exc).__name__}: {exc}"[:400]}
    if rank != 0:
        return None
    peak, peak_kind = measured_peaks()
    bytes_step = decode_bytes_per_step(cfg, batch=BATCH, context=CONTEXT, scale_bytes=2)
    ms_per_step = ms_max / steps
    value = world * BATCH * steps / (ms_max / 1e3)
    head_gbs = head_bytes / (head_ms * 1e-3) / 1e9
    step_gbs = bytes_step["total"] / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate and recurrent state",
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD if args.layers is None else f"{WORKLOAD} CUT TO {args.layers} LAYERS (profiler captures only, not a bench value)",
            "batch_per_gpu": BATCH,
            "context": CONTEXT,
            "sequences": world * BATCH,
            "parallelism": f"independent sequences x{world}, no collectives",
            "l2": "each step streams 2.4 GB of weights, KV and state, 19x the 126 MB L2; no flush needed",
            "engine": "graph",
            "attn_splits": attn_splits,
            "scale_dtype": "bf16",
        },
        "e2e": {
            "value": world * BATCH * steps / (e2e_ms_max / 1e3),
            "unit": "tokens/s",
            "h2d_bytes_per_step": 8 * BATCH,
            "d2h_bytes_per_step": 8 * BATCH,
            "tokens_match_device_loop": same,
        },
        "gpu_launches": steps * launches_per_step,
        "launches_per_step": launches_per_step,
        "clocks": clocks.summary(),
        "roofline": None,
        "roofline_head": {
            "kernel": "gemv_stream_kernel (int4 GEMV, RMSNorm prologue) on the LM head 248320x2560, timed alone with CUDA events",
            "bound": "hbm",
            "achieved": head_gbs,
            "peak": peak,
            "unit": "GB/s",
            "frac": head_gbs / peak,
            "peak_kind": f"of {peak_kind}",
            "bytes_per_launch": head_bytes,
            "us_per_launch": head_ms * 1e3,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this matrix, from an ncu capture of
            # the same launch (a record of that capture, not re-measured by this run)
            "traffic": HEAD_GEMV_DRAM_BYTES_PER_LAUNCH,
        },
        "roofline_step": {
            "bound": "hbm",
            "bytes_per_token": bytes_step["total"],
            "achieved": step_gbs,
            "peak": peak,
            "unit": "GB/s",
            "frac": step_gbs / peak,
            "frac_of_nominal_8tbs": step_gbs / 8000.0,
            "breakdown": bytes_step,
        },
        "finite_logits": finite,
    }
    if proj_stats is not None:
        # the dominant kernel family: the int4 GEMV of the 128 layer projections (4 launches per layer)
        gbs = proj_stats["bytes"] / (proj_stats["us"] * 1e-6) / 1e9
        line["roofline"] = {
            "kernel": "layer-projection int4 GEMV (gemv_mma_kernel / gemv_cluster_kernel), all launches of one token",
            "bound": "hbm",
            "achieved": gbs,
            "peak": peak,
            "unit": "GB/s",
            "frac": gbs / peak,
            "peak_kind": f"of {peak_kind}",
            "launches": proj_stats["launches"],
            "bytes_per_launch": proj_stats["bytes"] / proj_stats["launches"],
            "us_per_launch": proj_stats["us"] / proj_stats["launches"],
            "timed_by": "device timestamps (%globaltimer) recorded by the kernels in a traced replay of the same graph: a launch's "
            "time is its share of the step's critical path, from the previous launch's last exit to its own last exit",
            "traffic": LAYER_GEMV_DRAM_BYTES_PER_LAUNCH,
        }
    else:
        line["roofline"] = line["roofline_head"]
    if tp_line is not None:
        line["tp"] = tp_line
    return line


TP_CONTEXT = 8192


def tp_arm(dist, rank: int, world: int, dev, steps: int, warmup: int, layers: int | None) -> dict | None:
    """After the data-parallel measurement of a multi-GPU run: the same GPUs as ONE tensor-parallel replica
    (batch 1, 8192 tokens of context, peer-store exchange, one CUDA graph per token), and the single-GPU step at the
    same context for the speed-up. Returns the ``tp`` object of the JSON line on rank 0."""
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import qwen3_5_4b_config, synth
    from deltaforge_b200 import timeline as TL
    from deltaforge_b200 import tp as TP

    cfg = qwen3_5_4b_config() if layers is None else qwen3_5_4b_config(num_hidden_layers=layers)
    full = synth.random_model_weights(cfg, seed=1234, device=dev, scale_dtype=torch.bfloat16)  # same seed on every rank
    tok = torch.full((1,), 1000, dtype=torch.int64, device=dev)
    max_seq = TP_CONTEXT + steps + warmup + 16

    def timed(run) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # one GPU, same context (every rank runs it: the maximum is what a single GPU of this box does)
    cache1 = E.DecodeCache(cfg, 1, max_seq, device=dev)
    synth.fill_cache(cache1, TP_CONTEXT, seed=77)
    eng1 = E.DecodeEngine(full, cache1)
    eng1.decode(tok, warmup)
    one_ms = timed(lambda: eng1.decode(tok, steps)) / steps
    del eng1, cache1
    shard = TP.shard_weights(full, rank, world)
    del full
    torch.cuda.empty_cache()
    cache = E.DecodeCache(TP.shard_config(cfg, world), 1, max_seq, device=dev)
    synth.fill_cache(cache, TP_CONTEXT, seed=77)
    eng = TP.TensorParallelEngine(shard, cache, rank=rank, tp=world, exchange="peer")
    eng.decode(tok, warmup)
    tp_ms = timed(lambda: eng.decode(tok, steps, check=False)) / steps
    eng.check_status()
    # per-exchange cost from the kernels' own timestamps: from the last exit of the K-sharded projection to the
    # exit of the kernel that waited for every rank's words and added them
    trace = eng.engine.set_trace()
    eng.decode(tok, 3)
    torch.cuda.synchronize()
    rows = TL.summarise(trace, [f"launch{i}" for i in range(trace.shape[0])])
    eng.engine.set_trace(0)
    gaps, prev_exit = [], None
    for r in rows:
        if r["ctas"] == -(-cfg.hidden_size // 256) and r.get("dots_done") is None and prev_exit is not None and r["exit_last"] is not None:
            gaps.append(r["exit_last"] - prev_exit)
        if r["exit_last"] is not None:
            prev_exit = r["exit_last"]
    dist.barrier()
    if rank != 0:
        return None
    exchanges = 2 * cfg.num_hidden_layers
    return {
        "n": world,
        "context": TP_CONTEXT,
        "ms_per_step": tp_ms,
        "tokens_per_s": 1e3 / tp_ms,
        "one_gpu_ms_per_step": one_ms,
        "speedup_vs_1gpu": one_ms / tp_ms,
        "exchange": "peer stores from the projection's epilogue into every rank's buffer; no collective call; one CUDA graph per token",
        "exchanges_per_token": exchanges,
        "us_per_exchange": (sum(gaps) / len(gaps)) if gaps else None,
        "us_per_exchange_is": "rank 0, last traced token: last exit of the K-sharded projection -> exit of the kernel that polled "
        "every rank's words, added them in rank order and updated the residual stream",
        "steps": steps,
    }


def run_tp(args) -> dict | None:
    """All ranks of the job form ONE tensor-parallel replica decoding one batch."""
    from deltaforge_b200 import engine as E
    from deltaforge_b200 import qwen3_5_4b_config, synth
    from deltaforge_b200 import tp as TP
    from deltaforge_b200.bytes_model import decode_bytes_per_step

    dist, rank, world, local = dist_setup(args.gpus)
    if dist is None:
        raise RuntimeError("--tp needs a multi-rank launch (torchrun)")
    dev = torch.device("cuda", local)
    cfg = qwen3_5_4b_config() if args.layers is None else qwen3_5_4b_config(num_hidden_layers=args.layers)
    steps, warmup = args.steps, max(args.warmup, 3)
    full = synth.random_model_weights(cfg, seed=1234, device=dev, scale_dtype=torch.bfloat16)  # same seed on every rank
    shard = TP.shard_weights(full, rank, world)
    del full
    torch.cuda.empty_cache()
    cache = E.DecodeCache(TP.shard_config(cfg, world), BATCH, CONTEXT + steps + warmup + 8, device=dev)
    synth.fill_cache(cache, CONTEXT, seed=77)
    eng = TP.TensorParallelEngine(shard, cache, rank=rank, tp=world, exchange=args.tp_exchange)
    tok = torch.full((BATCH,), 1000, dtype=torch.int64, device=dev)
    eng.decode(tok, warmup, graph=args.tp_graph)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        e0.record()
        eng.decode(tok, steps, graph=args.tp_graph)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    dist.barrier()
    times = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    eng.engine.check_status()
    if rank != 0:
        return None
    peak, peak_kind = measured_peaks()
    ms_max = times.item()
    bytes_step = decode_bytes_per_step(cfg, batch=BATCH, context=CONTEXT, scale_bytes=2)
    return {
        "metric": METRIC,
        "value": BATCH * steps / (ms_max / 1e3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_max / steps,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate and recurrent state",
        "data": "synthetic",
        "config": {
            "workload": f"qwen3.5-4b int4 decode step, batch {BATCH}, ctx {CONTEXT}, ONE replica tensor-parallel over {world} GPUs",
            "parallelism": f"tp{world}: heads, MLP channels and vocabulary sharded; two fp32 all-reduces per layer",
            "all_reduces_per_token": 2 * cfg.num_hidden_layers,
            "exchange": "peer stores inside the kernels (no collective call)" if args.tp_exchange == "peer" else "NCCL all-reduce",
            "launch": "one CUDA graph per token" if (args.tp_graph or args.tp_exchange == "peer") else "segments and collectives launched directly",
        },
        "clocks": clocks.summary(),
        "roofline_step": {"bytes_per_token": bytes_step["total"], "achieved": bytes_step["total"] / (ms_max / steps * 1e-3) / 1e9,
                          "peak": peak * world, "unit": "GB/s", "peak_kind": f"of {peak_kind}, x{world} GPUs"},
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU port leg of the default run")
    ap.add_argument(
        "--layers",
        type=int,
        default=None,
        help="cut the model to this many layers (a multiple of 4) so that a profiler capture holds little device memory; "
        "the line it prints is marked and is not a bench value",
    )
    ap.add_argument("--no-tp-arm", action="store_true", help="with N > 1 GPUs: skip the tensor-parallel arm after the data-parallel run")
    ap.add_argument("--tp", action="store_true", help="all ranks form one tensor-parallel replica (not the default data-parallel run)")
    ap.add_argument("--tp-exchange", choices=("nccl", "peer"), default="nccl", help="with --tp: how the ranks add their partial sums")
    ap.add_argument("--tp-graph", action="store_true", help="with --tp: record kernels and collectives into one CUDA graph per token")
    ap.add_argument("--no-tensor-core-gemv", action="store_true", help="run the layer projections on the dp4a kernels instead of the integer mma")
    ap.add_argument("--timeline", default=None, help="after the timed runs, write a per-launch timeline of one step to this file")
    ap.add_argument("--prefetch-distance", type=int, default=None,
                    help="projections ahead for which the step's kernels ask the L2 for weights (0: off; default: the library's)")
    ap.add_argument("--batch", type=int, default=None, help="sequences per GPU (default 1: the metric's configuration)")
    ap.add_argument("--context", type=int, default=None, help="tokens already in the cache (default 4096)")
    args = ap.parse_args()
    global BATCH, CONTEXT, WORKLOAD
    if args.batch is not None or args.context is not None:
        BATCH = args.batch or BATCH
        CONTEXT = args.context or CONTEXT
        WORKLOAD = f"qwen3.5-4b int4 decode step, batch {BATCH}, ctx {CONTEXT} (not the metric's configuration)"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        res = run_cpu_port(args.steps, max(args.warmup, 1), budget_s=150.0)
        line = {
            "impl": "reference",
            "metric": METRIC,
            "value": res["value"],
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 1),
            "ms_per_step": res["seconds_per_token"] * 1e3,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "int4 weights dequantised to bf16, fp32 matmul (the reference's torch expression)",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "batch_per_gpu": BATCH,
                "context": CONTEXT,
                "sequences": BATCH,
                "parallelism": "host cores of rank 0 only",
                "l2": "not applicable (CPU arm)",
                "engine": "oracle port on the CPU",
                "attn_splits": None,
                "scale_dtype": "fp32",
            },
            "extrapolated": res["extrapolated"],
            "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return

    line = run_tp(args) if args.tp else run_ours(args)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    if line is None:
        return
    if world == 1 and not args.no_cpu_baseline:
        torch.cuda.empty_cache()
        line["cpu_baseline"] = run_cpu_port(3, 1, budget_s=60.0)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
