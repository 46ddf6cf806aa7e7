"""The BASELINE configurations at full size.  The CPU oracle cannot do whole
tensors of this size in seconds, so each case checks (a) a set of query rows of
several heads against the oracle (first rows, rows around tile boundaries, last
rows), and (b) size-independent properties: row 0 of causal attention equals
V[0] with LSE = scale*q0.k0; non-causal LSE is the same for any permutation of the
keys; every output is finite."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROWS = np.concatenate([np.arange(0, 132), np.arange(1020, 1030), np.arange(4090, 4100)]).astype(np.int32)


def _gpu_normal(torch, dev, seed, shape, dtype):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randn(shape, device=dev, dtype=torch.float32, generator=g).to(dtype)


@pytest.mark.parametrize("causal", [True, False])
def test_config3_bf16_b1_h32_s8192_d128(fa, dev, oracle, causal):
    import torch
    bh, s, d = 32, 8192, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    q, k, v = (_gpu_normal(torch, dev, 3000 + i, (bh, s, d), torch.bfloat16) for i in range(3))
    o = torch.full_like(q, float("nan"))
    lse = torch.full((bh, s), float("nan"), device=dev, dtype=torch.float32)
    fa.prefill(q, k, v, o, lse, 1, bh, s, d, scale, causal, dtype="bf16")
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    rows = np.concatenate([ROWS, np.arange(8184, 8192)]).astype(np.int32)
    heads = [0, 13, 31]
    qh, kh, vh = (x[heads].float().cpu().numpy() for x in (q, k, v))
    o_ref, l_ref = oracle.attention(qh, kh, vh, scale, causal, rows=rows)
    og = o[heads].float().cpu().numpy()[:, rows]
    lg = lse[heads].cpu().numpy()[:, rows]
    assert np.abs(lg - l_ref).max() < 1e-3
    assert np.abs(og - o_ref).max() < 1e-2                      # bf16 output rounding floor, see test_prefill_gpu
    if causal:
        assert (o[:, 0].float() - v[:, 0].float()).abs().max().item() < 1e-2
        dot = (q[:, 0].float() * k[:, 0].float()).sum(-1) * scale
        assert (lse[:, 0] - dot).abs().max().item() < 1e-3
    else:
        perm = torch.randperm(s, device=dev)
        o2 = torch.empty_like(o)
        lse2 = torch.empty_like(lse)
        fa.prefill(q, k[:, perm].contiguous(), v[:, perm].contiguous(), o2, lse2, 1, bh, s, d, scale, False,
                   dtype="bf16")
        torch.cuda.synchronize()
        assert (lse2 - lse).abs().max().item() < 1e-3            # key order does not change the LSE
        assert (o2.float() - o.float()).abs().max().item() < 1.6e-2


def test_config5_fp8_b8_h16_s4096_d128(fa, dev, oracle):
    import torch
    bh, s, d = 128, 4096, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    codes, scales, deq_heads = [], [], []
    heads = [0, 77, 127]
    for i in range(3):
        x = _gpu_normal(torch, dev, 5000 + i, (bh, s, d), torch.float32)
        amax = x.abs().amax(dim=(1, 2)).clamp_min(1e-12)
        sc = (amax / 448.0).float()
        q8 = (x / sc[:, None, None]).to(torch.float8_e4m3fn)
        codes.append(q8.view(torch.uint8))
        scales.append(sc)
        deq_heads.append((q8[heads].float() * sc[heads, None, None]).cpu().numpy())
        del x
    o = torch.full((bh, s, d), float("nan"), device=dev, dtype=torch.bfloat16)
    lse = torch.full((bh, s), float("nan"), device=dev, dtype=torch.float32)
    fa.prefill(codes[0], codes[1], codes[2], o, lse, 8, 16, s, d, scale, True, dtype="e4m3",
               q_scale=scales[0], k_scale=scales[1], v_scale=scales[2])
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    rows = ROWS[ROWS < s]
    o_ref, l_ref = oracle.attention(deq_heads[0], deq_heads[1], deq_heads[2], scale, True, rows=rows)
    assert np.abs(o[heads].float().cpu().numpy()[:, rows] - o_ref).max() < 3e-2
    assert np.abs(lse[heads].cpu().numpy()[:, rows] - l_ref).max() < 1e-3


def test_config4_decode_b32_h32_skv16384_d128_every_head(fa, dev, oracle):
    """All 1024 (batch, head) pairs against the oracle, 16 splits + combine."""
    import torch
    b, h, skv, d = 32, 32, 16384, 128
    bh = b * h
    scale = float(1.0 / np.sqrt(np.float32(d)))
    k = torch.empty((bh, skv, d), device=dev, dtype=torch.float16)
    v = torch.empty_like(k)
    for t, seed in ((k, 4100), (v, 4200)):
        for i in range(0, bh, 128):
            t[i:i + 128] = _gpu_normal(torch, dev, seed + i, (128, skv, d), torch.float16)
    q = _gpu_normal(torch, dev, 4300, (bh, d), torch.float16)
    o = torch.full((bh, d), float("nan"), device=dev, dtype=torch.float16)
    lse = torch.full((bh,), float("nan"), device=dev, dtype=torch.float32)
    wsb = fa.decode_workspace_bytes(b, h, d, 16)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode(q, k, v, o, lse, None, b, h, skv, d, scale, dtype="f16", num_splits=16, workspace=ws,
              workspace_bytes=wsb)
    torch.cuda.synchronize()
    og, lg = o.float().cpu().numpy(), lse.cpu().numpy()
    qc = q.float().cpu().numpy().reshape(bh, 1, d)
    worst_o = worst_l = 0.0
    for i in range(0, bh, 128):
        kc, vc = k[i:i + 128].float().cpu().numpy(), v[i:i + 128].float().cpu().numpy()
        o_ref, l_ref = oracle.attention(qc[i:i + 128], kc, vc, scale, False)
        worst_o = max(worst_o, float(np.abs(og[i:i + 128] - o_ref[:, 0]).max()))
        worst_l = max(worst_l, float(np.abs(lg[i:i + 128] - l_ref[:, 0]).max()))
    assert worst_o < 2e-3 and worst_l < 1e-3, (worst_o, worst_l)
