"""Split-KV decode and LSE-combine parity through the C ABI against the CPU oracle."""
import numpy as np
import pytest

from helpers import to_dev

pytestmark = pytest.mark.gpu

TOL_O = 2e-3
TOL_LSE = 1e-3


def _run_decode(fa, dev, q, k, v, scale, dtype, splits, want_f32=False):
    import torch
    bh, skv, d = k.shape
    dq, dk, dv = (to_dev(x, dtype, dev) for x in (q.reshape(bh, d), k, v))
    do = torch.full((bh, d), float("nan"), device=dev, dtype=dq.dtype)
    dl = torch.full((bh,), float("nan"), device=dev, dtype=torch.float32)
    df = torch.full((bh, d), float("nan"), device=dev, dtype=torch.float32) if want_f32 else None
    n = splits if splits else fa.decode_default_splits(1, bh, skv)
    wsb = fa.decode_workspace_bytes(1, bh, d, max(n, 1))
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode(dq, dk, dv, do, dl, df, 1, bh, skv, d, float(scale), dtype=dtype, num_splits=splits,
              workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    return do.float().cpu().numpy(), dl.cpu().numpy(), (df.cpu().numpy() if want_f32 else None)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("skv,splits", [(1, 1), (17, 1), (100, 3), (1000, 4), (1024, 16), (4097, 0), (5000, 7)])
def test_decode_f16(fa, dev, oracle, d, skv, splits):
    bh = 5
    scale = float(1.0 / np.sqrt(np.float32(d)))
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(40 + skv, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(41 + skv, (bh, 1, d), n=1)[0], "f16")
    o, lse, _ = _run_decode(fa, dev, q, k, v, scale, "f16", splits)
    o_ref, l_ref = oracle.attention(q, k, v, scale, False)
    assert np.abs(o - o_ref[:, 0]).max() < TOL_O
    assert np.abs(lse - l_ref[:, 0]).max() < TOL_LSE


def test_decode_bf16(fa, dev, oracle):
    bh, skv, d = 4, 3000, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    k, v = (oracle.round_to(x, "bf16") for x in oracle.normal_inputs(60, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(61, (bh, 1, d), n=1)[0], "bf16")
    o, lse, of = _run_decode(fa, dev, q, k, v, scale, "bf16", 6, want_f32=True)
    o_ref, l_ref = oracle.attention(q, k, v, scale, False)
    assert np.abs(of - o_ref[:, 0]).max() < 1e-4          # fp32 result: no output rounding
    assert np.abs(o - o_ref[:, 0]).max() < TOL_O          # |O| << 1 here, bf16 rounding is small
    assert np.abs(lse - l_ref[:, 0]).max() < TOL_LSE


def test_decode_equals_last_causal_prefill_row(fa, dev, oracle):
    """Decode over a cache == the last row of causal self-attention on the same keys."""
    from helpers import run_prefill
    bh, s, d = 3, 384, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(70, (bh, s, d)))
    o_pre, l_pre = run_prefill(fa, dev, q, k, v, scale, True)
    o_dec, l_dec, _ = _run_decode(fa, dev, q[:, -1:], k, v, scale, "f16", 3)
    assert np.abs(o_dec - o_pre[:, -1]).max() < 2e-3
    assert np.abs(l_dec - l_pre[:, -1]).max() < 1e-3


def test_combine_merges_rank_partials(fa, dev, oracle):
    """The exchange step of KV-sequence-sharded decode, emulated on one GPU: each
    'rank' decodes its slice (fp32 partial + LSE), the partials are stacked the way
    an all-gather lays them out, and fa_combine merges them."""
    import torch
    bh, skv, d, ranks = 8, 4096, 128, 4
    scale = float(1.0 / np.sqrt(np.float32(d)))
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(80, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(81, (bh, 1, d), n=1)[0], "f16")
    per = skv // ranks
    parts_o, parts_l = [], []
    for r in range(ranks):
        _, l, of = _run_decode(fa, dev, q, k[:, r * per:(r + 1) * per], v[:, r * per:(r + 1) * per],
                               scale, "f16", 2, want_f32=True)
        parts_o.append(of); parts_l.append(l)
    go = torch.from_numpy(np.stack(parts_o)).to(dev)          # [ranks, bh, d]
    gl = torch.from_numpy(np.stack(parts_l)).to(dev)          # [ranks, bh]
    do = torch.zeros((bh, d), device=dev, dtype=torch.float16)
    dl = torch.zeros((bh,), device=dev, dtype=torch.float32)
    fa.combine(go, gl, ranks, bh, d, do, dl, dtype="f16")
    torch.cuda.synchronize()
    o_ref, l_ref = oracle.attention(q, k, v, scale, False)
    assert np.abs(do.float().cpu().numpy() - o_ref[:, 0]).max() < TOL_O
    assert np.abs(dl.cpu().numpy() - l_ref[:, 0]).max() < TOL_LSE
    # and against the oracle's own merge of the same partials
    om, lm = oracle.merge(np.stack(parts_o, 1), np.stack(parts_l, 1))
    assert np.abs(do.float().cpu().numpy() - om).max() < 1e-3
    assert np.abs(dl.cpu().numpy() - lm).max() < 1e-5


def test_combine_packed_reads_the_gathered_buffer_in_place(fa, dev, oracle):
    """fa_combine_packed on [ranks, rows, D + 1] blocks (normalised O then LSE per row), the layout one
    all-gather of packed rows produces; an empty rank (LSE = -inf) must carry weight zero."""
    import torch
    bh, skv, d, ranks = 6, 3000, 64, 3
    scale = 0.125
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(90, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(91, (bh, 1, d), n=1)[0], "f16")
    per = skv // ranks
    packed = np.zeros((ranks + 1, bh, d + 1), np.float32)
    for r in range(ranks):
        _, l, of = _run_decode(fa, dev, q, k[:, r * per:(r + 1) * per], v[:, r * per:(r + 1) * per],
                               scale, "f16", 2, want_f32=True)
        packed[r, :, :d] = of
        packed[r, :, d] = l
    packed[ranks, :, :d] = 123.0                              # a rank without keys: must not contribute
    packed[ranks, :, d] = -np.inf
    g = torch.from_numpy(packed).to(dev)
    do = torch.zeros((bh, d), device=dev, dtype=torch.float16)
    dl = torch.zeros((bh,), device=dev, dtype=torch.float32)
    fa.combine_packed(g, ranks + 1, bh, d, do, dl, dtype="f16")
    torch.cuda.synchronize()
    o_ref, l_ref = oracle.attention(q, k, v, scale, False)
    assert np.abs(do.float().cpu().numpy() - o_ref[:, 0]).max() < TOL_O
    assert np.abs(dl.cpu().numpy() - l_ref[:, 0]).max() < TOL_LSE


def test_kv_sharded_entry_on_a_one_rank_communicator(fa, dev, oracle):
    """fa_decode_kv_sharded end to end on one GPU: an NCCL communicator of one rank (created through
    the library's own NCCL binding), the packed partial written in place, the in-place all-gather and
    the packed merge.  With one rank the result must equal plain fa_decode's."""
    import torch
    bh, skv, d = 8, 5000, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(92, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(93, (bh, 1, d), n=1)[0], "f16")
    dq = torch.from_numpy(q.reshape(bh, d)).to(dev, torch.float16)
    dk, dv = (torch.from_numpy(x).to(dev, torch.float16) for x in (k, v))
    comm = fa.nccl_comm_create(1, fa.nccl_unique_id(), 0)
    try:
        splits = 4
        wsb = fa.decode_workspace_bytes(1, bh, d, splits)
        ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
        gb = fa.decode_kv_sharded_gather_bytes(1, bh, d, 1)
        gather = torch.full((gb // 4,), float("nan"), device=dev, dtype=torch.float32)
        do = torch.full((bh, d), float("nan"), device=dev, dtype=torch.float16)
        dl = torch.full((bh,), float("nan"), device=dev, dtype=torch.float32)
        for _ in range(2):                                    # buffers are reused across calls
            rc = fa.decode_kv_sharded_raw(dq, dk, dv, do, dl, 1, bh, skv, d, scale, comm, gather, gb,
                                          num_splits=splits, workspace=ws, workspace_bytes=wsb)
            assert rc == 0, fa.last_cuda_error()
        torch.cuda.synchronize()
        o_ref, l_ref = oracle.attention(q, k, v, scale, False)
        assert np.abs(do.float().cpu().numpy() - o_ref[:, 0]).max() < TOL_O
        assert np.abs(dl.cpu().numpy() - l_ref[:, 0]).max() < TOL_LSE
        o_plain, l_plain, _ = _run_decode(fa, dev, q, k, v, scale, "f16", splits)
        assert np.array_equal(do.float().cpu().numpy(), o_plain) and np.array_equal(dl.cpu().numpy(), l_plain)
        # too small a receive buffer is refused before anything is launched
        assert fa.decode_kv_sharded_raw(dq, dk, dv, do, dl, 1, bh, skv, d, scale, comm, gather, gb - 4,
                                        num_splits=splits, workspace=ws, workspace_bytes=wsb) == fa.FA_ERR_WORKSPACE
    finally:
        fa.nccl_comm_destroy(comm)


def test_decode_many_heads(fa, dev, oracle):
    """batch * heads beyond 65535 (the limit of a grid's second dimension; the kernel's grid is
    one-dimensional)."""
    import torch
    bh, skv, d = 70000, 48, 64
    g = torch.Generator(device=dev).manual_seed(5)
    dq = torch.randn((bh, d), device=dev, generator=g).half()
    dk = torch.randn((bh, skv, d), device=dev, generator=g).half()
    dv = torch.randn((bh, skv, d), device=dev, generator=g).half()
    do = torch.empty((bh, d), device=dev, dtype=torch.float16)
    dl = torch.empty((bh,), device=dev, dtype=torch.float32)
    wsb = fa.decode_workspace_bytes(1, bh, d, 1)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.decode(dq, dk, dv, do, dl, None, 1, bh, skv, d, 0.125, num_splits=1, workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    heads = [0, 65535, 65536, 69999]
    o_ref, l_ref = oracle.attention(dq[heads].float().cpu().numpy()[:, None], dk[heads].float().cpu().numpy(),
                                    dv[heads].float().cpu().numpy(), 0.125, False)
    assert np.abs(do[heads].float().cpu().numpy() - o_ref[:, 0]).max() < TOL_O
    assert np.abs(dl[heads].cpu().numpy() - l_ref[:, 0]).max() < TOL_LSE


def test_decode_rejects_small_workspace(fa, dev):
    import torch
    t = torch.zeros(4096, device=dev, dtype=torch.float16)
    rc = fa.decode_raw(t, t, t, t, None, None, 1, 1, 16, 128, 0.1, num_splits=2, workspace=t,
                       workspace_bytes=16)
    assert rc == fa.FA_ERR_WORKSPACE
