"""Grouped-query / multi-query decode over a strided KV cache (fa_decode_gqa) against the CPU
oracle: per query head one query row, K and V of KV head hq // group, every key visible.
Tolerances: fp16 O 2e-3, LSE 1e-3 (max abs); bf16 O two ulp + 5e-3."""
import numpy as np
import pytest
import torch

from helpers import to_dev

pytestmark = pytest.mark.gpu


def run_gqa(fa, dev, q, k, v, scale, dtype="f16", layout="bhsd", num_splits=0, want_lse=True):
    """q [B,Hq,D], k/v [B,Hkv,S,D] float32 already rounded.  Returns (o [B,Hq,D], lse [B,Hq])."""
    b, hq, d = q.shape
    _, hkv, s, _ = k.shape
    dq = to_dev(q, dtype, dev)
    if layout == "bhsd":
        dk, dv = to_dev(k, dtype, dev), to_dev(v, dtype, dev)
        strides = (0, 0, 0)
    elif layout == "bshd":                                  # [B, S, Hkv, D]
        dk, dv = (to_dev(np.ascontiguousarray(x.transpose(0, 2, 1, 3)), dtype, dev) for x in (k, v))
        strides = (s * hkv * d, d, hkv * d)
    else:                                                   # padded rows: [B, Hkv, S, D + 64]
        pad = 64
        def padded(x):
            t = torch.full((b, hkv, s, d + pad), float("nan"), device=dev, dtype=dq.dtype)
            t[..., :d] = to_dev(x, dtype, dev)
            return t
        dk, dv = padded(k), padded(v)
        strides = (hkv * s * (d + pad), s * (d + pad), d + pad)
    do = torch.full((b, hq, d), float("nan"), device=dev, dtype=dq.dtype)
    dl = torch.full((b, hq), float("nan"), device=dev, dtype=torch.float32) if want_lse else None
    splits = num_splits or fa.decode_gqa_default_splits(b, hkv, s)
    ws_bytes = fa.decode_workspace_bytes(b, hq, d, splits)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    fa.decode_gqa(dq, dk, dv, do, dl, b, hq, hkv, s, d, float(scale), dtype=dtype, num_splits=num_splits,
                  kv_strides=strides, workspace=ws, workspace_bytes=ws_bytes)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    return do.float().cpu().numpy(), (dl.cpu().numpy() if want_lse else None)


def oracle_gqa(oracle, q, k, v, scale):
    b, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    kx = np.repeat(k, g, axis=1).reshape(b * hq, k.shape[2], d)
    vx = np.repeat(v, g, axis=1).reshape(b * hq, k.shape[2], d)
    o, l = oracle.attention(q.reshape(b * hq, 1, d), kx, vx, scale, False)
    return o[:, 0].reshape(b, hq, d), l[:, 0].reshape(b, hq)


def make(oracle, seed, b, hq, hkv, s, d, dtype):
    q = oracle.round_to(oracle.normal_inputs(seed, (b, hq, d), n=1)[0], dtype)
    k, v = (oracle.round_to(x, dtype) for x in oracle.normal_inputs(seed + 1, (b, hkv, s, d), n=2))
    return q, k, v


@pytest.mark.parametrize("b,hq,hkv,s,d", [
    (2, 8, 2, 1000, 128),       # group 4, ragged last tile
    (1, 8, 1, 640, 64),         # multi-query, d 64
    (3, 6, 6, 257, 128),        # group 1 (plain multi-head through the same path)
    (1, 32, 4, 4096, 128),      # group 8, several splits
    (2, 4, 2, 100, 64),         # shorter than one key tile
])
def test_gqa_matches_oracle_fp16(fa, oracle, dev, b, hq, hkv, s, d):
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 40 + s, b, hq, hkv, s, d, "f16")
    o, l = run_gqa(fa, dev, q, k, v, scale)
    o_ref, l_ref = oracle_gqa(oracle, q, k, v, scale)
    assert np.abs(o - o_ref).max() < 2e-3
    assert np.abs(l - l_ref).max() < 1e-3


@pytest.mark.parametrize("layout", ["bshd", "padded"])
def test_gqa_strided_cache_layouts(fa, oracle, dev, layout):
    b, hq, hkv, s, d = 2, 8, 2, 900, 128
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 77, b, hq, hkv, s, d, "f16")
    o, l = run_gqa(fa, dev, q, k, v, scale, layout=layout)
    o_ref, l_ref = oracle_gqa(oracle, q, k, v, scale)
    assert np.abs(o - o_ref).max() < 2e-3
    assert np.abs(l - l_ref).max() < 1e-3


def test_gqa_bf16_and_explicit_splits(fa, oracle, dev):
    b, hq, hkv, s, d = 1, 16, 2, 3000, 128
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 91, b, hq, hkv, s, d, "bf16")
    o_ref, l_ref = oracle_gqa(oracle, q, k, v, scale)
    for splits in (1, 3, 24):
        o, l = run_gqa(fa, dev, q, k, v, scale, dtype="bf16", num_splits=splits)
        assert np.abs(o - o_ref).max() < 2 * 2.0 ** -8 * np.abs(o_ref).max() + 5e-3
        assert np.abs(l - l_ref).max() < 1e-3


def test_gqa_agrees_with_plain_decode_when_group_is_one(fa, oracle, dev):
    """Same inputs through fa_decode (streaming kernel) and fa_decode_gqa (tensor-core kernel)."""
    b, h, s, d = 2, 4, 2048, 128
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 13, b, h, h, s, d, "f16")
    o_g, l_g = run_gqa(fa, dev, q, k, v, scale)
    dq, dk, dv = (to_dev(x, "f16", dev) for x in (q, k, v))
    do = torch.zeros((b, h, d), device=dev, dtype=torch.float16)
    dl = torch.zeros((b, h), device=dev, dtype=torch.float32)
    wsb = fa.decode_workspace_bytes(b, h, d, 8)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode(dq, dk, dv, do, dl, None, b, h, s, d, float(scale), dtype="f16", num_splits=8,
              workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    assert np.abs(do.float().cpu().numpy() - o_g).max() < 2e-3
    assert np.abs(dl.cpu().numpy() - l_g).max() < 1e-3


def test_gqa_argument_errors(fa, dev):
    t = torch.zeros(4096, device=dev, dtype=torch.float16)
    ws = torch.empty(1 << 20, device=dev, dtype=torch.uint8)
    ok = dict(dtype="f16", workspace=ws, workspace_bytes=ws.numel())
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 6, 4, 128, 64, 0.1, **ok) == fa.FA_ERR_INVALID_ARGUMENT   # 6 % 4
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 4, 2, 128, 96, 0.1, **ok) == fa.FA_ERR_UNSUPPORTED        # d_head
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 4, 2, 128, 64, 0.1, kv_strides=(8192, 4100, 64), **ok) == fa.FA_ERR_MISALIGNED
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 4, 2, 128, 64, 0.1, dtype="f16", workspace=ws,
                             workspace_bytes=16) == fa.FA_ERR_WORKSPACE
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 256, 1, 128, 64, 0.1, **ok) == fa.FA_ERR_UNSUPPORTED      # group > 128
