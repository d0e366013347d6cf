"""CPU-only checks: the C-ABI library loads and exports what the header declares, host-side logic,
argument errors of the ops (raised before any device work), and the two-rank sharding helpers on gloo."""

from __future__ import annotations

import os
import re
import socket
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

from deltaforge_b200 import _lib, bytes_model, engine, ops, parallel, quant
from deltaforge_b200.config import qwen3_5_4b_config, tiny_config
from oracle import ref_ops as R

ROOT = Path(__file__).resolve().parent.parent
BF16 = torch.bfloat16


def declared_symbols() -> set[str]:
    text = (ROOT / "include" / "dfb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(dfb_[a-z0-9_]+)\s*\(", text))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/dfb200.h but not exported"
    assert names == set(_lib.SIGNATURES), names ^ set(_lib.SIGNATURES)
    assert lib.dfb_abi_version() == 1
    assert lib.dfb_last_error() is not None


def test_header_is_plain_c_and_a_c_program_can_bind_the_library(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and as C++11 on its own, and a C program that includes it
    must link against the library and call an entry point that needs no device."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler here")
    header = ROOT / "include" / "dfb200.h"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c", str(header)], check=True)
    gxx = shutil.which("g++")
    if gxx is not None:
        subprocess.run([gxx, "-std=c++11", "-fsyntax-only", "-x", "c++", str(header)], check=True)
    lib = _lib.library_path()
    _lib.load()  # builds it if it is missing
    src = tmp_path / "bind.c"
    src.write_text(
        '#include <stdio.h>\n#include "dfb200.h"\n'
        "int main(void) {\n"
        "  if (dfb_abi_version() != 1) return 1;\n"
        "  if (dfb_int4_gemv(0, 0) != 2) return 2; /* null descriptor: a bad-argument code, no device touched */\n"
        '  printf("%zu\\n", dfb_int4_gemv_scratch_bytes(4, 2560, 2560, 128));\n'
        "  return 0;\n}\n"
    )
    exe = tmp_path / "bind"
    subprocess.run([gcc, "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe), str(lib), f"-Wl,-rpath,{lib.parent}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    assert int(out.strip()) > 4 * 10 * 2560 * 4


def test_scratch_size_queries_need_no_device():
    lib = _lib.load()
    assert lib.dfb_int4_gemv_scratch_bytes(1, 64, 40, 32) == 0  # generic path: no scratch
    assert lib.dfb_int4_gemv_scratch_bytes(4, 2560, 2560, 128) > 4 * 10 * 2560 * 4
    assert lib.dfb_attn_scratch_bytes(1, 16, 4, 256, 1) == 0
    assert lib.dfb_attn_scratch_bytes(2, 16, 4, 256, 8) >= 2 * 16 * 8 * 256 * 4


def test_c_entry_points_reject_bad_arguments_without_a_device():
    lib = _lib.load()
    assert lib.dfb_int4_unpack(None, 8, 8, None, None) == 2
    assert b"null" in lib.dfb_last_error()
    d = _lib.GemvDesc()
    assert lib.dfb_int4_gemv(None, None) == 2
    d.rows, d.K, d.N, d.group = 1, 7, 8, 1
    d.x = d.packed = d.scale = d.out = 1  # non-null, never dereferenced: the shape check comes first
    assert lib.dfb_int4_gemv(d, None) == 2 and b"even" in lib.dfb_last_error()
    assert lib.dfb_engine_replay(None, 1, None) == 2


def test_ops_check_shapes_before_devices():
    packed = torch.zeros((128, 16), dtype=torch.uint8)
    scale = torch.ones((2, 16))
    with pytest.raises(ValueError, match="expects K=256"):
        ops.tiled_gemv_int4(torch.zeros((1, 64), dtype=BF16), packed, scale, 128)
    with pytest.raises(ValueError, match="scale must be"):
        ops.tiled_gemv_int4(torch.zeros((1, 256), dtype=BF16), packed, torch.ones((3, 16)), 128)
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        ops.tiled_gemv_int4(torch.zeros((1, 256), dtype=BF16), packed, scale, 128)
    with pytest.raises(ValueError, match="fp32"):
        z = torch.zeros
        ops.delta_rule_step(z((1, 1, 4, 4), dtype=BF16), z((1, 1, 4)), z((1, 1, 4)), z((1, 1, 4)), z((1, 1)), z((1, 1)))
    with pytest.raises(ValueError, match="rotary_dim must be even"):
        ops.partial_rope(torch.zeros((1, 1, 1, 8), dtype=BF16), torch.zeros((1, 1, 3)), torch.zeros((1, 1, 3)))
    with pytest.raises(ValueError, match="four-tap"):
        ops.fused_causal_conv_step(torch.zeros((1, 4, 1), dtype=BF16), torch.zeros((1, 4, 3), dtype=BF16), torch.zeros((4, 1, 3), dtype=BF16))
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        ops.silu_mul(torch.zeros(4, dtype=BF16), torch.zeros(4, dtype=BF16))


def test_fake_kernels_give_shapes_for_tracing():
    with torch._subclasses.fake_tensor.FakeTensorMode():
        x = torch.empty((2, 1, 256), dtype=BF16)
        packed = torch.empty((128, 48), dtype=torch.uint8)
        scale = torch.empty((2, 48))
        assert torch.ops.dfb200.tiled_gemv_int4(x, packed, scale, 128).shape == (2, 1, 48)
        state = torch.empty((1, 4, 16, 16))
        out, new_state = torch.ops.dfb200.delta_rule_step(state, torch.empty((1, 4, 16)), torch.empty((1, 4, 16)), torch.empty((1, 4, 16)), torch.empty((1, 4)), torch.empty((1, 4)))
        assert out.shape == (1, 4, 16) and new_state.shape == state.shape


def test_quantiser_is_the_oracles():
    w = (torch.randn((40, 512), generator=torch.Generator().manual_seed(0)) * 0.02).to(BF16)
    qw = quant.quantise_int4_k_major(w)
    packed, scale, group = R.quantise_int4_k_major(w)
    assert qw.group_size == group == 128 and qw.bits == 4
    assert torch.equal(qw.qweight, packed) and torch.equal(qw.scale, scale)
    assert quant.group_size_for(64) == 32
    with pytest.raises(ValueError):
        quant.group_size_for(60)
    both = quant.concat_along_n([qw, qw])
    assert both.qweight.shape == (256, 80) and both.scale.shape == (4, 80)
    with pytest.raises(ValueError):
        quant.concat_along_n([qw, quant.quantise_int4_k_major(torch.zeros((4, 256)))])


def test_byte_model_matches_the_survey_arithmetic():
    cfg = qwen3_5_4b_config()
    assert bytes_model.linear_params(cfg) == (3_569_090_560, 635_699_200)
    b = bytes_model.decode_bytes_per_step(cfg, batch=1, context=4096, scale_bytes=2)
    assert b["weights"] == 2_168_094_720 and b["state"] == 100_663_296
    assert abs(b["total"] - 2_406_900_000) < 2_000_000
    assert bytes_model.gemv_bytes(2560, 248320, scale_bytes=2) == 317_849_600 + 9_932_800 + 496_640


def test_default_attention_slices():
    assert engine.default_attn_splits(4240, 1, 4) == 32  # 133 keys per slice, 128 CTAs
    assert engine.default_attn_splits(8192, 1, 4) == 64
    assert engine.default_attn_splits(16, 2, 1) == 1
    s = engine.default_attn_splits(32768 + 64, 32, 4)
    assert s & (s - 1) == 0 and 1 <= s <= 128


def test_cache_contract():
    cache = engine.DecodeCache(tiny_config(), 2, 8, device="cpu")
    assert [tuple(t.shape) for t in cache.state_tensors()] == [(2, 128, 3), (2, 4, 16, 16), (2, 1, 8, 32), (2, 1, 8, 32)]
    assert cache.state_tensors()[1].dtype == torch.float32
    cache.advance(8)
    with pytest.raises(ValueError, match="cache overflow"):
        cache.ensure_capacity(1)
    with pytest.raises(ValueError):
        cache.rewind(9)
    snap = cache.snapshot()
    ptrs = [t.data_ptr() for t in cache.state_tensors()]
    cache.reset()
    cache.restore(snap)
    assert cache.seq_len == 8 and ptrs == [t.data_ptr() for t in cache.state_tensors()]


def test_engine_refuses_cpu_weights():
    from deltaforge_b200 import synth

    w = synth.random_model_weights(tiny_config(), seed=0, device="cpu", scale_dtype=torch.float32)
    with pytest.raises(RuntimeError, match="no PyTorch fallback"):
        engine.DecodeEngine(w, engine.DecodeCache(tiny_config(), 1, 4, device="cpu"))


def test_shard_range_partitions_exactly():
    for n, world in [(0, 3), (1, 4), (32, 8), (33, 8), (7, 2)]:
        seen = []
        for r in range(world):
            seen.extend(parallel.shard_range(n, r, world))
        assert seen == list(range(n))
        sizes = [len(parallel.shard_range(n, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_range(4, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_rank_worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    r = parallel.init("gloo")
    mine = parallel.shard_range(5, r.rank, r.world)  # 5 sequences over 2 ranks: 3 + 2
    seconds = 2.0 if r.rank == 0 else 4.0  # rank 1 is the slow one
    parallel.barrier()
    total = parallel.aggregate_throughput(len(mine) * 10, seconds)
    slowest = parallel.max_over_ranks(seconds)
    out.put((r.rank, list(mine), total, slowest))
    torch.distributed.destroy_process_group()


def test_two_ranks_on_gloo_aggregate_like_the_bench():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][1] == [0, 1, 2] and got[1][1] == [3, 4]
    for _, _, total, slowest in got:
        assert slowest == 4.0 and total == pytest.approx(50 / 4.0)
