"""fa_backward (dQ, dK, dV) against torch autograd evaluated in fp32 on the CPU on the same rounded
inputs.  The reference project has no backward pass, so there are no golden vectors: the fp32 autograd
of softmax(scale * Q K^T + mask) V is the definition.  O and LSE fed to the backward come from this
library's forward.  Tolerance (max abs, relative to the largest reference entry): P and dS are rounded
to the storage type before the second set of products, so fp16 is held to 4e-3 * max|ref| + 2e-3 and
bf16 to 3e-2 * max|ref| + 1e-2."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {"f16": (4e-3, 2e-3), "bf16": (3e-2, 1e-2)}
TD = {"f16": torch.float16, "bf16": torch.bfloat16}


def autograd_reference(q, k, v, d_o, scale, causal):
    q, k, v = (x.clone().float().requires_grad_(True) for x in (q, k, v))
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        n = q.shape[-2]
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
    o = torch.softmax(s, -1) @ v
    o.backward(d_o.float())
    return q.grad, k.grad, v.grad


def run_backward(fa, dev, q, k, v, d_o, scale, causal, dtype):
    bh, s, d = q.shape
    dq_, dk_, dv_, ddo = (x.to(dev) for x in (q, k, v, d_o))
    o = torch.empty_like(dq_)
    lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
    fa.prefill(dq_, dk_, dv_, o, lse, 1, bh, s, d, float(scale), causal, dtype=dtype)
    gq, gk, gv = (torch.full_like(dq_, float("nan")) for _ in range(3))
    wsb = fa.backward_workspace_bytes(1, bh, s)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    fa.backward(dq_, dk_, dv_, o, ddo, lse, gq, gk, gv, 1, bh, s, d, float(scale), causal, dtype=dtype,
                workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    return gq.float().cpu(), gk.float().cpu(), gv.float().cpu()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,s,d", [(2, 128, 64), (3, 300, 64), (2, 257, 128), (1, 1024, 128), (2, 40, 64)])
def test_backward_matches_autograd(fa, dev, dtype, causal, bh, s, d):
    g = torch.Generator().manual_seed(1000 + s + d)
    q, k, v, d_o = (torch.randn((bh, s, d), generator=g).to(TD[dtype]) for _ in range(4))
    scale = 1.0 / np.sqrt(d)
    ref = autograd_reference(q, k, v, d_o, scale, causal)
    got = run_backward(fa, dev, q, k, v, d_o, scale, causal, dtype)
    rel, ab = TOL[dtype]
    for name, r, x in zip(("dQ", "dK", "dV"), ref, got):
        assert torch.isfinite(x).all(), name
        err = (x - r).abs().max().item()
        assert err < rel * r.abs().max().item() + ab, (name, err, r.abs().max().item())


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,s,d,dtype", [(300, 192, 64, "f16"), (500, 64, 64, "f16"), (450, 320, 64, "bf16"),
                                          (200, 192, 128, "f16"), (330, 100, 128, "bf16")])
def test_backward_many_items_per_cta(fa, dev, causal, bh, s, d, dtype):
    """More (tile, head) work items than SMs, with odd step counts per item: every persistent CTA
    walks several items, so the step parity, the ring positions and the stationary-tile buffers
    carry over from one item to the next, some items give one of the two step parities nothing to
    do, and outputs are staged and stored while the next item runs."""
    g = torch.Generator().manual_seed(4000 + bh + s + d)
    q, k, v, d_o = (torch.randn((bh, s, d), generator=g).to(TD[dtype]) for _ in range(4))
    scale = 1.0 / np.sqrt(d)
    ref = autograd_reference(q, k, v, d_o, scale, causal)
    got = run_backward(fa, dev, q, k, v, d_o, scale, causal, dtype)
    rel, ab = TOL[dtype]
    for name, r, x in zip(("dQ", "dK", "dV"), ref, got):
        assert torch.isfinite(x).all(), name
        # per head, so that one wrong item cannot hide behind the largest entry of another head
        err = (x - r).abs().amax(dim=(1, 2))
        bound = rel * r.abs().amax(dim=(1, 2)) + ab
        bad = torch.nonzero(err > bound).flatten().tolist()
        assert not bad, (name, bad[:8], err.max().item())


def test_backward_argument_errors(fa, dev):
    t = torch.zeros(128 * 64, device=dev, dtype=torch.float16)
    l = torch.zeros(128, device=dev, dtype=torch.float32)
    ws = torch.empty(1024, device=dev, dtype=torch.uint8)
    ok = dict(dtype="f16", workspace=ws, workspace_bytes=ws.numel())
    assert fa.backward_raw(t, t, t, t, t, l, t, t, None, 1, 1, 128, 64, 0.125, False, **ok) == fa.FA_ERR_INVALID_ARGUMENT
    assert fa.backward_raw(t, t, t, t, t, l, t, t, t, 1, 1, 128, 96, 0.125, False, **ok) == fa.FA_ERR_UNSUPPORTED
    assert fa.backward_raw(t, t, t, t, t, l, t, t, t, 1, 1, 128, 64, 0.125, False, dtype="f16", workspace=ws,
                           workspace_bytes=16) == fa.FA_ERR_WORKSPACE
    assert fa.backward_raw(t, t, t, t, t, l, t, t, t, 1, 1, 128, 64, -1.0, False, **ok) == fa.FA_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("s", [1, 63, 65, 129])
def test_backward_edge_lengths(fa, dev, s):
    """Sequences shorter than one step, one row past a step and one row past a tile."""
    g = torch.Generator().manual_seed(77 + s)
    q, k, v, d_o = (torch.randn((2, s, 64), generator=g).half() for _ in range(4))
    for causal in (False, True):
        ref = autograd_reference(q, k, v, d_o, 0.125, causal)
        got = run_backward(fa, dev, q, k, v, d_o, 0.125, causal, "f16")
        for name, r, x in zip(("dQ", "dK", "dV"), ref, got):
            assert torch.isfinite(x).all(), name
            assert (x - r).abs().max().item() < 4e-3 * r.abs().max().item() + 2e-3, (name, causal)


def test_backward_outputs_complete_for_the_next_kernel_on_the_stream(fa, dev):
    """The dQ kernel is launched as a programmatic dependent of the dK/dV kernel; work enqueued after
    fa_backward on the same stream - directly, and as the next node of a captured graph - must still
    see dK and dV complete.  A copy kernel right behind fa_backward (no synchronisation in between)
    has to read exactly what a synchronised run leaves in the buffers."""
    bh, s, d = 48, 2048, 64
    g = torch.Generator().manual_seed(4242)
    q, k, v, d_o = (torch.randn((bh, s, d), generator=g).half().to(dev) for _ in range(4))
    o = torch.empty_like(q)
    lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
    fa.prefill(q, k, v, o, lse, 1, bh, s, d, 0.125, True)
    wsb = fa.backward_workspace_bytes(1, bh, s)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    gq, gk, gv = (torch.empty_like(q) for _ in range(3))
    snap_k, snap_v = torch.empty_like(q), torch.empty_like(q)

    def enqueue(stream):
        fa.backward(q, k, v, o, d_o, lse, gq, gk, gv, 1, bh, s, d, 0.125, True, workspace=ws,
                    workspace_bytes=wsb, stream=stream)
        snap_k.copy_(gk)                                  # same stream, no synchronisation in between
        snap_v.copy_(gv)

    # reference: a synchronised run
    fa.backward(q, k, v, o, d_o, lse, gq, gk, gv, 1, bh, s, d, 0.125, True, workspace=ws, workspace_bytes=wsb)
    torch.cuda.synchronize()
    ref_k, ref_v = gk.clone(), gv.clone()
    assert torch.isfinite(ref_k).all() and torch.isfinite(ref_v).all()

    stream = torch.cuda.Stream()
    for _ in range(3):
        for t in (gk, gv, snap_k, snap_v):
            t.fill_(float("nan"))
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            enqueue(stream)
        stream.synchronize()
        assert torch.equal(snap_k, ref_k) and torch.equal(snap_v, ref_v)

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            enqueue(stream)
    for _ in range(3):
        for t in (gk, gv, snap_k, snap_v):
            t.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(snap_k, ref_k) and torch.equal(snap_v, ref_v)
    assert fa.device_status() == 0
