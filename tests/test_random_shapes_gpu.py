"""Seeded random shapes for the three tensor-core paths against their references: many small
problems with awkward sizes (lengths around tile and step boundaries, odd head counts, groups that do
not divide the tile, ragged and paged caches).  Tolerances as in the per-path tests."""
import numpy as np
import pytest
import torch

from helpers import run_prefill, to_dev
from test_backward_gpu import autograd_reference, run_backward, TD, TOL
from test_decode_gqa_gpu import oracle_multi_token

pytestmark = pytest.mark.gpu

LENGTHS = [1, 2, 7, 31, 63, 64, 65, 127, 128, 129, 191, 200, 255, 256, 257, 300, 383, 385, 511, 640, 700]


@pytest.mark.parametrize("case", range(16))
def test_prefill_random(fa, oracle, dev, case):
    rng = np.random.RandomState(1000 + case)
    bh = int(rng.randint(1, 6))
    s = int(rng.choice(LENGTHS))
    d = int(rng.choice([64, 128]))
    causal = bool(rng.randint(2))
    dtype = "f16" if rng.randint(2) else "bf16"
    scale = float(rng.choice([0.05, 1.0 / np.sqrt(d), 0.3]))
    q, k, v = (oracle.round_to(x, dtype) for x in oracle.normal_inputs(2000 + case, (bh, s, d)))
    o, l = run_prefill(fa, dev, q, k, v, scale, causal, dtype)
    o_ref, l_ref = oracle.attention(q, k, v, scale, causal)
    assert fa.device_status() == 0
    # bf16: two output ulps at the largest magnitude plus the rounding of P (see test_prefill_gpu)
    tol = 2e-3 if dtype == "f16" else 2 * 2.0 ** -8 * np.abs(o_ref).max() + 5e-3
    assert np.abs(o - o_ref).max() < tol, (bh, s, d, causal, dtype)
    assert np.abs(l - l_ref).max() < 1e-3


@pytest.mark.parametrize("case", range(12))
def test_backward_random(fa, dev, case):
    rng = np.random.RandomState(3000 + case)
    bh = int(rng.randint(1, 4))
    s = int(rng.choice(LENGTHS))
    d = int(rng.choice([64, 128]))
    causal = bool(rng.randint(2))
    dtype = "f16" if rng.randint(2) else "bf16"
    g = torch.Generator().manual_seed(4000 + case)
    q, k, v, d_o = (torch.randn((bh, s, d), generator=g).to(TD[dtype]) for _ in range(4))
    scale = 1.0 / np.sqrt(d)
    ref = autograd_reference(q, k, v, d_o, scale, causal)
    got = run_backward(fa, dev, q, k, v, d_o, scale, causal, dtype)
    rel, ab = TOL[dtype]
    for name, r, x in zip(("dQ", "dK", "dV"), ref, got):
        assert torch.isfinite(x).all(), (name, bh, s, d, causal, dtype)
        assert (x - r).abs().max().item() < rel * r.abs().max().item() + ab, (name, bh, s, d, causal, dtype)


@pytest.mark.parametrize("case", range(16))
def test_decode_gqa_random(fa, oracle, dev, case):
    rng = np.random.RandomState(5000 + case)
    b = int(rng.randint(1, 4))
    hkv = int(rng.choice([1, 2, 3]))
    group = int(rng.choice([1, 2, 3, 4, 8, 16]))
    hq = hkv * group
    d = int(rng.choice([64, 128]))
    smax = int(rng.choice([64, 128, 192, 320, 512, 1024]))
    t_n = int(rng.choice([1, 1, 2, 5, 40]))
    t_n = min(t_n, smax)
    lens = [int(rng.randint(0, smax + 1)) for _ in range(b)]
    lens[0] = smax                                             # at least one full-length sequence
    paged = bool(rng.randint(2))
    page = int(rng.choice([16, 32, 64, 128]))
    scale = 1.0 / np.sqrt(d)
    q = oracle.round_to(oracle.normal_inputs(6000 + case, (b, t_n, hq, d), n=1)[0], "f16")
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(6100 + case, (b, hkv, smax, d), n=2))
    o_ref, l_ref = oracle_multi_token(oracle, q, k, v, lens, scale)
    dq, dk, dv = (to_dev(x, "f16", dev) for x in (q, k, v))
    kw = dict(seq_lens=torch.tensor(lens, device=dev, dtype=torch.int32))
    if paged and smax % page == 0:
        pps = smax // page
        n_pages = b * pps + 4
        perm = rng.permutation(n_pages)[: b * pps].reshape(b, pps)
        kp = torch.full((n_pages, page, hkv, d), float("nan"), device=dev, dtype=torch.float16)
        vp = torch.full((n_pages, page, hkv, d), float("nan"), device=dev, dtype=torch.float16)
        table = np.full((b, pps), -1, np.int32)
        for i in range(b):
            for pg in range((lens[i] + page - 1) // page):
                r0, r1 = pg * page, min((pg + 1) * page, lens[i])
                table[i, pg] = perm[i, pg]
                kp[perm[i, pg], : r1 - r0] = dk[i, :, r0:r1].permute(1, 0, 2)
                vp[perm[i, pg], : r1 - r0] = dv[i, :, r0:r1].permute(1, 0, 2)
        kbuf, vbuf = kp, vp
        kw.update(kv_strides=(0, d, hkv * d), block_table=torch.from_numpy(table).to(dev), block_table_stride=pps,
                  page_size=page, num_pages=n_pages, kv_page_stride=page * hkv * d)
    else:
        for i in range(b):
            dk[i, :, lens[i]:] = float("nan")
            dv[i, :, lens[i]:] = float("nan")
        kbuf, vbuf = dk, dv
    do = torch.full((b, t_n, hq, d), float("nan"), device=dev, dtype=torch.float16)
    dl = torch.full((b, t_n, hq), float("nan"), device=dev, dtype=torch.float32)
    splits = int(rng.choice([0, 1, 2, 5]))
    tpt = min(t_n, 128 // group)
    eff = splits or fa.decode_gqa_default_splits(b * (-(-t_n // tpt)), hkv, smax)
    wsb = fa.decode_workspace_bytes(b, t_n * hq, d, eff)
    ws = torch.full((max(wsb, 4) // 4,), float("nan"), device=dev, dtype=torch.float32)
    fa.decode_gqa(dq, kbuf, vbuf, do, dl, b, hq, hkv, smax, d, float(scale), dtype="f16", num_splits=eff,
                  num_q_tokens=t_n, workspace=ws, workspace_bytes=wsb, **kw)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    o, l = do.float().cpu().numpy(), dl.cpu().numpy()
    ctx = (b, hq, hkv, d, smax, t_n, lens, paged, page, eff)
    assert np.isfinite(o).all(), ctx
    assert np.abs(o - o_ref).max() < 2e-3, ctx
    live = np.isfinite(l_ref)
    assert np.abs(l[live] - l_ref[live]).max() < 1e-3, ctx
    assert np.all(np.isneginf(l[~live])), ctx
