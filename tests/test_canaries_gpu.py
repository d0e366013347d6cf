"""Canary padding around the outputs of the ragged-shape launches (the stand-in for a memory checker).

Every kernel family of the int4 GEMV, the DeltaNet step and the decode attention are called straight through the C ABI
with their output in the middle of a larger buffer filled with a marker pattern: shapes whose last column tile, last
key slice or last row block is partial. A store one element outside the output shows up as a changed marker.
"""

from __future__ import annotations

import ctypes as C

import pytest
import torch

from deltaforge_b200 import _lib, ops
from deltaforge_b200._lib import AttnDesc, DeltaNetDesc, GemvDesc

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"
PAD = 512  # elements of marker on either side
MARK = -1234.0


def padded(numel: int, dtype=BF16):
    buf = torch.full((numel + 2 * PAD,), MARK, dtype=dtype, device=DEV)
    return buf, buf[PAD : PAD + numel]


def assert_padding_intact(buf: torch.Tensor, numel: int):
    torch.cuda.synchronize()
    assert bool((buf[:PAD] == MARK).all()), "a store landed before the output"
    assert bool((buf[PAD + numel :] == MARK).all()), "a store landed after the output"
    assert not bool((buf[PAD : PAD + numel] == MARK).any()), "part of the output was never written"


@pytest.mark.parametrize("k,n", [(2560, 1000), (2560, 12352), (4096, 264), (9216, 2564), (2560, 4100)])
@pytest.mark.parametrize("path", ["tiled", "k8", "mma"])
def test_gemv_kernels_store_nothing_outside_a_ragged_output(k, n, path):
    lib = _lib.load()
    g = torch.Generator().manual_seed(k + n)
    packed = torch.randint(0, 256, (k // 2, n), generator=g, dtype=torch.uint8).to(DEV)
    scale = (torch.randn((k // 128, n), generator=g).abs() * 0.02 + 1e-4).to(DEV)
    x = torch.randn((1, k), generator=g).to(BF16).to(DEV)
    buf, out = padded(n)
    nbytes = lib.dfb_int4_gemv_scratch_bytes(1, k, n, 128)
    sbuf = torch.zeros(nbytes + 2 * PAD, dtype=torch.uint8, device=DEV)
    sbuf[:PAD] = 0xA5
    sbuf[PAD + nbytes :] = 0xA5
    d = GemvDesc()
    d.x, d.x_stride, d.rows = x.data_ptr(), k, 1
    d.packed, d.scale, d.scale_is_bf16 = packed.data_ptr(), scale.data_ptr(), 0
    d.K, d.N, d.group = k, n, 128
    d.eps = 1e-6
    d.out, d.out_stride = out.data_ptr(), n
    d.scratch, d.scratch_bytes = sbuf[PAD:].data_ptr(), nbytes
    keep = []
    if path == "tiled":
        d.force_tiled = 1
    elif path == "k8":
        keep.append(ops.int4_repack_k8(packed))
        d.packed_k8 = keep[-1].data_ptr()
    else:
        keep.append(ops.int4_repack_mma(packed, scale))
        d.packed_mma = keep[-1].data_ptr()
    _lib.check(lib.dfb_int4_gemv(C.byref(d), None), "dfb_int4_gemv")
    assert_padding_intact(buf, n)
    assert bool((sbuf[:PAD] == 0xA5).all()) and bool((sbuf[PAD + nbytes :] == 0xA5).all()), "a store landed outside the scratch"
    want = ops.int4_gemv_fused(x, packed, scale, 128, force_tiled=True)
    assert (out.float() - want.float().reshape(-1)).abs().max().item() <= 2**-6 * want.float().abs().max().item()


@pytest.mark.parametrize("key_len,splits", [(1, 1), (3, 2), (33, 8), (2049, 64)])
def test_attention_decode_stores_nothing_outside_its_output(key_len, splits):
    lib = _lib.load()
    hq, hkv, dh = 16, 4, 256
    g = torch.Generator().manual_seed(key_len)
    q = torch.randn((1, hq, dh), generator=g).to(BF16).to(DEV)
    kc = torch.randn((1, hkv, key_len, dh), generator=g).to(BF16).to(DEV)
    vc = torch.randn((1, hkv, key_len, dh), generator=g).to(BF16).to(DEV)
    buf, out = padded(hq * dh)
    nbytes = lib.dfb_attn_scratch_bytes(1, hq, hkv, dh, splits)
    sbuf = torch.zeros(max(nbytes, 16) + 2 * PAD, dtype=torch.uint8, device=DEV)
    sbuf[:PAD] = 0xA5
    sbuf[PAD + nbytes :] = 0xA5
    d = AttnDesc()
    d.batch, d.hq, d.hkv, d.d = 1, hq, hkv, dh
    d.q, d.q_stride, d.qh_stride = q.data_ptr(), hq * dh, dh
    d.kcache, d.vcache = kc.data_ptr(), vc.data_ptr()
    d.kv_batch_stride, d.kv_head_stride = hkv * key_len * dh, key_len * dh
    d.key_len, d.scale, d.splits = key_len, dh**-0.5, splits
    d.scratch, d.scratch_bytes = sbuf[PAD:].data_ptr(), nbytes
    d.out, d.out_stride = out.data_ptr(), hq * dh
    _lib.check(lib.dfb_attn_decode(C.byref(d), None), "dfb_attn_decode")
    assert_padding_intact(buf, hq * dh)
    assert bool((sbuf[:PAD] == 0xA5).all()) and bool((sbuf[PAD + nbytes :] == 0xA5).all())
    want = ops.split_kv_decode_attention(q, kc, vc, dh**-0.5, splits) if splits > 1 else ops.gqa_decode_attention(q, kc, vc, dh**-0.5)
    assert (out.float() - want.float().reshape(-1)).abs().max().item() <= 2e-2


def test_deltanet_step_stores_nothing_outside_its_output_and_state():
    lib = _lib.load()
    hk, hv, dk, dv = 2, 4, 128, 128
    g = torch.Generator().manual_seed(5)
    row = torch.randn((1, 2 * hk * dk + 2 * hv * dv + 2 * hv), generator=g).to(BF16).to(DEV)
    sbuf, state = padded(hv * dk * dv, torch.float32)
    state.copy_(torch.randn(hv * dk * dv, generator=g) * 0.1)
    obuf, out = padded(hv * dv)
    a_log = torch.zeros(hv, device=DEV)
    dt = torch.zeros(hv, device=DEV)
    nw = torch.ones(dv, device=DEV)
    d = DeltaNetDesc()
    d.batch, d.num_k_heads, d.num_v_heads, d.dk, d.dv = 1, hk, hv, dk, dv
    base = row.data_ptr()
    d.q, d.k, d.v = base, base + 2 * hk * dk, base + 2 * 2 * hk * dk
    d.z = base + 2 * (2 * hk * dk + hv * dv)
    d.b = base + 2 * (2 * hk * dk + 2 * hv * dv)
    d.a = base + 2 * (2 * hk * dk + 2 * hv * dv + hv)
    d.row_stride = row.shape[1]
    d.a_log, d.dt_bias, d.norm_w, d.norm_w_is_bf16, d.eps = a_log.data_ptr(), dt.data_ptr(), nw.data_ptr(), 1, 1e-6
    d.state, d.out, d.out_stride = state.data_ptr(), out.data_ptr(), hv * dv
    _lib.check(lib.dfb_deltanet_step(C.byref(d), None), "dfb_deltanet_step")
    assert_padding_intact(obuf, hv * dv)
    torch.cuda.synchronize()
    assert bool((sbuf[:PAD] == MARK).all()) and bool((sbuf[PAD + hv * dk * dv :] == MARK).all())
