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


def oracle_ragged(oracle, q, k, v, lens, scale):
    """Per sequence its own KV length (0 allowed: O = 0, LSE = -inf)."""
    b, hq, d = q.shape
    o = np.zeros((b, hq, d), np.float32)
    l = np.full((b, hq), -np.inf, np.float32)
    for i in range(b):
        if lens[i] > 0:
            oi, li = oracle_gqa(oracle, q[i:i + 1], k[i:i + 1, :, :lens[i]], v[i:i + 1, :, :lens[i]], scale)
            o[i], l[i] = oi[0], li[0]
    return o, l


@pytest.mark.parametrize("page_size", [16, 64, 128, 256])
def test_gqa_paged_cache_with_sequence_lengths(fa, oracle, dev, page_size):
    """Pages scattered through a pool whose unused parts hold NaN; ragged sequence lengths,
    one of them zero, one ending exactly on a page boundary."""
    b, hq, hkv, d = 4, 8, 2, 128
    lens = [1000, 0, 512, 77]
    smax = 1024
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 300 + page_size, b, hq, hkv, smax, d, "f16")
    o_ref, l_ref = oracle_ragged(oracle, q, k, v, lens, scale)

    pages_per_seq = smax // page_size
    n_pages = b * pages_per_seq + 5
    rng = np.random.default_rng(page_size)
    perm = rng.permutation(n_pages)[: b * pages_per_seq].reshape(b, pages_per_seq)
    # pool layout [page][key in page][KV head][D]
    kp = torch.full((n_pages, page_size, hkv, d), float("nan"), device=dev, dtype=torch.float16)
    vp = torch.full((n_pages, page_size, hkv, d), float("nan"), device=dev, dtype=torch.float16)
    table = np.full((b, pages_per_seq), -1, np.int32)
    dk, dv = to_dev(k, "f16", dev), to_dev(v, "f16", dev)
    for i in range(b):
        for pg in range((lens[i] + page_size - 1) // page_size):
            r0, r1 = pg * page_size, min((pg + 1) * page_size, lens[i])
            table[i, pg] = perm[i, pg]
            kp[perm[i, pg], : r1 - r0] = dk[i, :, r0:r1].permute(1, 0, 2)
            vp[perm[i, pg], : r1 - r0] = dv[i, :, r0:r1].permute(1, 0, 2)
    dtab = torch.from_numpy(table).to(dev)
    dlens = torch.tensor(lens, device=dev, dtype=torch.int32)
    dq = to_dev(q, "f16", dev)
    do = torch.full((b, hq, d), float("nan"), device=dev, dtype=torch.float16)
    dl = torch.full((b, hq), float("nan"), device=dev, dtype=torch.float32)
    splits = fa.decode_gqa_default_splits(b, hkv, smax)
    wsb = fa.decode_workspace_bytes(b, hq, d, splits)
    ws = torch.full((wsb // 4,), float("nan"), device=dev, dtype=torch.float32)
    fa.decode_gqa(dq, kp, vp, do, dl, b, hq, hkv, smax, d, float(scale), dtype="f16",
                  kv_strides=(0, d, hkv * d), block_table=dtab, block_table_stride=pages_per_seq,
                  page_size=page_size, num_pages=n_pages, kv_page_stride=page_size * hkv * d, seq_lens=dlens,
                  workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    o, l = do.float().cpu().numpy(), dl.cpu().numpy()
    assert np.isfinite(o).all()
    assert np.abs(o - o_ref).max() < 2e-3
    assert l[1].tolist() == [-np.inf] * hq
    live = np.isfinite(l_ref)
    assert np.abs(l[live] - l_ref[live]).max() < 1e-3


def test_gqa_sequence_lengths_on_a_dense_cache(fa, oracle, dev):
    """seq_lens with a plain [B, Hkv, Smax, D] cache whose tail rows hold NaN; several splits, so
    some (sequence, split) pairs are empty."""
    b, hq, hkv, d, smax = 3, 4, 1, 64, 4096
    lens = [4096, 130, 2049]
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 501, b, hq, hkv, smax, d, "f16")
    o_ref, l_ref = oracle_ragged(oracle, q, k, v, lens, scale)
    dq, dk, dv = (to_dev(x, "f16", dev) for x in (q, k, v))
    for i in range(b):
        dk[i, :, lens[i]:] = float("nan")
        dv[i, :, lens[i]:] = float("nan")
    dlens = torch.tensor(lens, device=dev, dtype=torch.int32)
    do = torch.full((b, hq, d), float("nan"), device=dev, dtype=torch.float16)
    dl = torch.full((b, hq), float("nan"), device=dev, dtype=torch.float32)
    wsb = fa.decode_workspace_bytes(b, hq, d, 8)
    ws = torch.full((wsb // 4,), float("nan"), device=dev, dtype=torch.float32)
    fa.decode_gqa(dq, dk, dv, do, dl, b, hq, hkv, smax, d, float(scale), dtype="f16", num_splits=8,
                  seq_lens=dlens, workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    assert np.abs(do.float().cpu().numpy() - o_ref).max() < 2e-3
    assert np.abs(dl.cpu().numpy() - l_ref).max() < 1e-3


@pytest.mark.parametrize("paged", [False, True])
def test_gqa_e4m3_cache(fa, oracle, dev, paged):
    """e4m3 query and KV cache with per-(batch, KV head) scales, bf16 output.  The oracle runs in fp32 on
    the dequantised values, so the comparison measures the kernel, not the quantiser; tolerance as for
    the e4m3 prefill: O max-abs 3e-2, LSE 1e-3.  The paged variant also gives the sequences different
    lengths and fills unused cache bytes with 0x7F (an e4m3 NaN code)."""
    b, hq, hkv, d, smax = 2, 8, 2, 128, 1024
    g = hq // hkv
    lens = [1000, 333] if paged else [smax, smax]
    scale = 1.0 / np.sqrt(d)
    k_f, v_f = oracle.normal_inputs(900 + paged, (b * hkv, smax, d), n=2)
    q_f = oracle.normal_inputs(902 + paged, (b * hkv, g, d), n=1)[0]          # the group shares a scale
    (qc, qs, qd), (kc, ks, kd), (vc, vs, vd) = (oracle.quantize_e4m3(x) for x in (q_f, k_f, v_f))
    q_deq = qd.reshape(b, hq, d)
    k_deq, v_deq = kd.reshape(b, hkv, smax, d), vd.reshape(b, hkv, smax, d)
    o_ref, l_ref = oracle_ragged(oracle, q_deq, k_deq, v_deq, lens, scale)

    dq = torch.from_numpy(qc.reshape(b, hq, d)).to(dev)
    sq, sk, sv = (torch.from_numpy(x).to(dev) for x in (qs, ks, vs))
    kc4, vc4 = (torch.from_numpy(x.reshape(b, hkv, smax, d)).to(dev) for x in (kc, vc))
    kw = {}
    if paged:
        ps = 64
        pages_per_seq = smax // ps
        n_pages = b * pages_per_seq + 3
        perm = np.random.default_rng(5).permutation(n_pages)[: b * pages_per_seq].reshape(b, pages_per_seq)
        kp = torch.full((n_pages, ps, hkv, d), 0x7F, device=dev, dtype=torch.uint8)
        vp = torch.full((n_pages, ps, hkv, d), 0x7F, device=dev, dtype=torch.uint8)
        table = np.full((b, pages_per_seq), -1, np.int32)
        for i in range(b):
            for pg in range((lens[i] + ps - 1) // ps):
                r0, r1 = pg * ps, min((pg + 1) * ps, lens[i])
                table[i, pg] = perm[i, pg]
                kp[perm[i, pg], : r1 - r0] = kc4[i, :, r0:r1].permute(1, 0, 2)
                vp[perm[i, pg], : r1 - r0] = vc4[i, :, r0:r1].permute(1, 0, 2)
        kbuf, vbuf = kp, vp
        kw = dict(kv_strides=(0, d, hkv * d), block_table=torch.from_numpy(table).to(dev),
                  block_table_stride=pages_per_seq, page_size=ps, num_pages=n_pages, kv_page_stride=ps * hkv * d,
                  seq_lens=torch.tensor(lens, device=dev, dtype=torch.int32))
    else:
        kbuf, vbuf = kc4, vc4
    do = torch.full((b, hq, d), float("nan"), device=dev, dtype=torch.bfloat16)
    dl = torch.full((b, hq), float("nan"), device=dev, dtype=torch.float32)
    splits = fa.decode_gqa_default_splits(b, hkv, smax)
    wsb = fa.decode_workspace_bytes(b, hq, d, splits)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode_gqa(dq, kbuf, vbuf, do, dl, b, hq, hkv, smax, d, float(scale), dtype="e4m3", q_scale=sq, k_scale=sk,
                  v_scale=sv, workspace=ws, workspace_bytes=wsb, **kw)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    o, l = do.float().cpu().numpy(), dl.cpu().numpy()
    assert np.isfinite(o).all()
    assert np.abs(o - o_ref).max() < 3e-2
    assert np.abs(l - l_ref).max() < 1e-3


@pytest.mark.parametrize("b,hq,hkv,s,d,dtype", [
    (1, 128, 1, 300, 64, "f16"),     # the largest group: every row of the query tile is a head
    (2, 6, 2, 1, 128, "f16"),        # a single key; group of 3
    (1, 33, 1, 257, 128, "bf16"),    # group just past one warp of rows
])
def test_gqa_edge_groups_and_lengths(fa, oracle, dev, b, hq, hkv, s, d, dtype):
    scale = 1.0 / np.sqrt(d)
    q, k, v = make(oracle, 1200 + hq + s, b, hq, hkv, s, d, dtype)
    o, l = run_gqa(fa, dev, q, k, v, scale, dtype=dtype)
    o_ref, l_ref = oracle_gqa(oracle, q, k, v, scale)
    tol = 2e-3 if dtype == "f16" else 2 * 2.0 ** -8 * np.abs(o_ref).max() + 5e-3
    assert np.abs(o - o_ref).max() < tol
    assert np.abs(l - l_ref).max() < 1e-3


def oracle_multi_token(oracle, q, k, v, lens, scale):
    """q [B,T,Hq,D]; token t of sequence b sees keys [0, lens[b] - T + t]."""
    b, t_n, hq, d = q.shape
    o = np.zeros((b, t_n, hq, d), np.float32)
    l = np.full((b, t_n, hq), -np.inf, np.float32)
    for i in range(b):
        for t in range(t_n):
            vis = lens[i] - t_n + t + 1
            if vis > 0:
                oi, li = oracle_gqa(oracle, q[i:i + 1, t], k[i:i + 1, :, :vis], v[i:i + 1, :, :vis], scale)
                o[i, t], l[i, t] = oi[0], li[0]
    return o, l


@pytest.mark.parametrize("b,t_n,hq,hkv,smax,d,lens", [
    (2, 4, 8, 2, 700, 128, None),            # 4 draft tokens, group 4
    (1, 8, 8, 1, 1024, 64, None),            # 8 tokens x 8 heads = 64 rows of the tile
    (3, 3, 4, 4, 512, 128, [512, 130, 2]),   # ragged; the last sequence is shorter than the token count
    (1, 16, 8, 1, 300, 128, None),           # the full tile: 16 x 8 = 128 rows
    (2, 40, 8, 1, 700, 128, None),           # 40 tokens x 8 heads: three query tiles per KV head
    (1, 300, 2, 2, 1000, 64, None),          # a 300-token chunk appended to a 700-key prefix, group 1
    (2, 50, 6, 2, 600, 128, [600, 45]),      # group 3 (42 tokens per tile); second sequence shorter than the chunk
])
def test_multi_token_decode(fa, oracle, dev, b, t_n, hq, hkv, smax, d, lens):
    scale = 1.0 / np.sqrt(d)
    q = oracle.round_to(oracle.normal_inputs(1500 + t_n, (b, t_n, hq, d), n=1)[0], "f16")
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(1501 + t_n, (b, hkv, smax, d), n=2))
    o_ref, l_ref = oracle_multi_token(oracle, q, k, v, lens or [smax] * b, scale)
    dq, dk, dv = (to_dev(x, "f16", dev) for x in (q, k, v))
    kw = {}
    if lens is not None:
        for i in range(b):
            dk[i, :, lens[i]:] = float("nan")
            dv[i, :, lens[i]:] = float("nan")
        kw["seq_lens"] = torch.tensor(lens, device=dev, dtype=torch.int32)
    do = torch.full((b, t_n, hq, d), float("nan"), device=dev, dtype=torch.float16)
    dl = torch.full((b, t_n, hq), float("nan"), device=dev, dtype=torch.float32)
    splits = fa.decode_gqa_default_splits(b, hkv, smax)
    wsb = fa.decode_workspace_bytes(b, t_n * hq, d, splits)
    ws = torch.full((wsb // 4,), float("nan"), device=dev, dtype=torch.float32)
    fa.decode_gqa(dq, dk, dv, do, dl, b, hq, hkv, smax, d, float(scale), dtype="f16", num_q_tokens=t_n,
                  workspace=ws, workspace_bytes=wsb, **kw)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    o, l = do.float().cpu().numpy(), dl.cpu().numpy()
    assert np.isfinite(o).all()
    assert np.abs(o - o_ref).max() < 2e-3
    live = np.isfinite(l_ref)
    assert np.abs(l[live] - l_ref[live]).max() < 1e-3
    assert np.all(np.isneginf(l[~live]))


def test_multi_token_decode_argument_errors(fa, dev):
    t = torch.zeros(1 << 16, device=dev, dtype=torch.float16)
    ws = torch.empty(1 << 22, device=dev, dtype=torch.uint8)
    ok = dict(dtype="f16", workspace=ws, workspace_bytes=ws.numel())
    assert fa.decode_gqa_raw(t, t, t, t, None, 1, 4, 1, 2, 64, 0.1, num_q_tokens=3, **ok) == fa.FA_ERR_INVALID_ARGUMENT # more tokens than keys


def test_whole_sequence_as_chunk_equals_causal_prefill(fa, oracle, dev):
    """With T = Skv and one query head per KV head the chunk path computes causal self-attention:
    it must agree with fa_prefill on the same data (both within tolerance of each other)."""
    b, h, s, d = 2, 3, 700, 64
    scale = 1.0 / np.sqrt(d)
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(1700, (b * h, s, d)))
    dq, dk, dv = (to_dev(x, "f16", dev) for x in (q, k, v))
    o1 = torch.empty_like(dq)
    l1 = torch.empty((b * h, s), device=dev, dtype=torch.float32)
    fa.prefill(dq, dk, dv, o1, l1, b, h, s, d, float(scale), True, dtype="f16")
    # chunk path: q, o as [B, T, Hq, D]; cache [B, Hkv, Skv, D]
    q4 = dq.view(b, h, s, d).permute(0, 2, 1, 3).contiguous()
    o2 = torch.full((b, s, h, d), float("nan"), device=dev, dtype=torch.float16)
    l2 = torch.full((b, s, h), float("nan"), device=dev, dtype=torch.float32)
    n_qt = (s + 127) // 128
    splits = fa.decode_gqa_default_splits(b * n_qt, h, s)
    wsb = fa.decode_workspace_bytes(b, s * h, d, splits)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode_gqa(q4, dk.view(b, h, s, d), dv.view(b, h, s, d), o2, l2, b, h, h, s, d, float(scale), dtype="f16",
                  num_q_tokens=s, workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    o2p = o2.permute(0, 2, 1, 3).reshape(b * h, s, d)
    l2p = l2.permute(0, 2, 1).reshape(b * h, s)
    assert (o2p.float() - o1.float()).abs().max().item() < 2e-3
    assert (l2p - l1).abs().max().item() < 1e-3
