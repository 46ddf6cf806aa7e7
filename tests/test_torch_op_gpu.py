"""torch.ops.fa_b200.* against torch's own scaled_dot_product_attention evaluated in fp32 on the CPU
(fp32 reference of the same op; tolerance: the 16-bit rounding of P and O, 2e-3 abs for fp16)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op(fa):
    import __graft_entry__ as ge
    return ge.load_module("torch_op")


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_matches_sdpa(op, dev, dtype, tol, causal):
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn((2, 3, 200, 64), generator=g).to(dtype) for _ in range(3))
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
    out = op.sdpa(q.to(dev), k.to(dev), v.to(dev), is_causal=causal)
    assert out.dtype == dtype and out.shape == q.shape
    assert (out.float().cpu() - ref).abs().max().item() < tol
    o2, lse = torch.ops.fa_b200.prefill(q.to(dev), k.to(dev), v.to(dev), 0.125, causal)
    s = (q.float() @ k.float().transpose(-1, -2)) * 0.125
    if causal:
        s = s.masked_fill(torch.ones(200, 200, dtype=torch.bool).triu(1), float("-inf"))
    assert (lse.cpu() - torch.logsumexp(s, -1)).abs().max().item() < 1e-3
    assert torch.equal(o2, out)


def test_decode_matches_sdpa(op, dev):
    g = torch.Generator().manual_seed(6)
    q = torch.randn((2, 4, 1, 128), generator=g).half()
    k, v = (torch.randn((2, 4, 3000, 128), generator=g).half() for _ in range(2))
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    out = op.sdpa(q.to(dev), k.to(dev), v.to(dev))
    assert (out.float().cpu() - ref).abs().max().item() < 2e-3


def test_non_contiguous_inputs_and_side_stream(op, dev):
    g = torch.Generator().manual_seed(7)
    base = torch.randn((2, 130, 3, 64), generator=g).half().to(dev)       # [B, S, H, D]
    q = base.permute(0, 2, 1, 3)                                          # [B, H, S, D] view
    ref = torch.nn.functional.scaled_dot_product_attention(q.float().cpu(), q.float().cpu(), q.float().cpu())
    st = torch.cuda.Stream(device=dev)
    st.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(st):
        out = op.sdpa(q, q, q)
    st.synchronize()
    assert (out.float().cpu() - ref).abs().max().item() < 2e-3


def test_autograd_through_sdpa(op, dev):
    """loss.backward() through op.sdpa reaches fa_backward; compared with fp32 autograd on the CPU."""
    g = torch.Generator().manual_seed(8)
    q, k, v, w = (torch.randn((2, 2, 192, 64), generator=g).half() for _ in range(4))
    ref_in = [t.float().requires_grad_(True) for t in (q, k, v)]
    (torch.nn.functional.scaled_dot_product_attention(*ref_in, is_causal=True) * w.float()).sum().backward()
    dev_in = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    (op.sdpa(*dev_in, is_causal=True) * w.to(dev)).sum().backward()
    for r, x in zip(ref_in, dev_in):
        assert x.grad is not None and x.grad.dtype == torch.float16
        err = (x.grad.float().cpu() - r.grad).abs().max().item()
        assert err < 4e-3 * r.grad.abs().max().item() + 2e-3


def test_decode_gqa_op_with_paged_cache(op, dev):
    """torch.ops.fa_b200.decode_gqa on a paged cache against SDPA in fp32 on the CPU, per sequence."""
    g = torch.Generator().manual_seed(9)
    b, t, hq, hkv, d, page, lens = 2, 3, 8, 2, 128, 64, [500, 130]
    pages_per_seq = 8
    q = torch.randn((b, t, hq, d), generator=g).half()
    k = torch.randn((b, pages_per_seq * page, hkv, d), generator=g).half()
    v = torch.randn((b, pages_per_seq * page, hkv, d), generator=g).half()
    n_pages = b * pages_per_seq + 2
    perm = torch.randperm(n_pages, generator=g)[: b * pages_per_seq].view(b, pages_per_seq)
    kp = torch.full((n_pages, page, hkv, d), float("nan"), dtype=torch.float16)
    vp = torch.full((n_pages, page, hkv, d), float("nan"), dtype=torch.float16)
    for i in range(b):
        for pg in range(pages_per_seq):
            r0 = pg * page
            n = max(0, min(page, lens[i] - r0))
            kp[perm[i, pg], :n] = k[i, r0:r0 + n]
            vp[perm[i, pg], :n] = v[i, r0:r0 + n]
    o, lse = torch.ops.fa_b200.decode_gqa(q.to(dev), kp.to(dev), vp.to(dev), d ** -0.5,
                                          torch.tensor(lens, dtype=torch.int32, device=dev), perm.to(torch.int32).to(dev))
    assert o.shape == q.shape and lse.shape == (b, t, hq)
    for i in range(b):
        for tt in range(t):
            vis = lens[i] - t + tt + 1
            kk = k[i, :vis].permute(1, 0, 2).repeat_interleave(hq // hkv, 0).float()      # [Hq, vis, D]
            vv = v[i, :vis].permute(1, 0, 2).repeat_interleave(hq // hkv, 0).float()
            ref = torch.nn.functional.scaled_dot_product_attention(q[i, tt].float()[:, None], kk, vv)[:, 0]
            assert (o[i, tt].float().cpu() - ref).abs().max().item() < 2e-3
