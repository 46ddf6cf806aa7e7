"""The device-pointer entry points enqueue work only (no allocation, no synchronisation after their
first call on a device), so a sequence of them can be captured into a CUDA graph and replayed on new
contents of the same buffers.  The replayed results must equal direct calls bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefill_decode_backward_in_one_graph(fa, dev):
    bh, s, d = 6, 300, 64
    scale = float(1.0 / np.sqrt(d))
    g = torch.Generator(device=dev)
    g.manual_seed(1)

    def rnd(shape, dtype=torch.float16):
        return torch.randn(shape, device=dev, dtype=torch.float32, generator=g).to(dtype)

    q, k, v, d_o = (rnd((bh, s, d)) for _ in range(4))
    o = torch.empty_like(q)
    lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
    gq, gk, gv = (torch.empty_like(q) for _ in range(3))
    bws = torch.empty(fa.backward_workspace_bytes(1, bh, s), device=dev, dtype=torch.uint8)
    # decode: 2 sequences x 4 query heads over 2 KV heads, cache [B, Hkv, Skv, D]
    qd, kd, vd = rnd((2, 4, d)), rnd((2, 2, 1500, d)), rnd((2, 2, 1500, d))
    od = torch.empty_like(qd)
    ld = torch.empty((2, 4), device=dev, dtype=torch.float32)
    n_splits = fa.decode_gqa_default_splits(2, 2, 1500)
    dws = torch.empty(fa.decode_workspace_bytes(2, 4, d, n_splits), device=dev, dtype=torch.uint8)

    def enqueue(stream):
        fa.prefill(q, k, v, o, lse, 1, bh, s, d, scale, True, dtype="f16", stream=stream)
        fa.backward(q, k, v, o, d_o, lse, gq, gk, gv, 1, bh, s, d, scale, True, dtype="f16", workspace=bws,
                    workspace_bytes=bws.numel(), stream=stream)
        fa.decode_gqa(qd, kd, vd, od, ld, 2, 4, 2, 1500, d, scale, dtype="f16", num_splits=n_splits,
                      workspace=dws, workspace_bytes=dws.numel(), stream=stream)

    outs = (o, lse, gq, gk, gv, od, ld)
    enqueue(torch.cuda.current_stream(dev))               # first calls configure the kernels; not captured
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            enqueue(torch.cuda.current_stream(dev))
    torch.cuda.synchronize()
    for trial in range(2):
        for t in (q, k, v, d_o, qd, kd, vd):               # new contents, same buffers
            t.copy_(rnd(t.shape))
        for t in outs:
            t.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        replayed = [t.clone() for t in outs]
        for t in outs:
            t.fill_(float("nan"))
        enqueue(torch.cuda.current_stream(dev))
        torch.cuda.synchronize()
        assert fa.device_status() == 0
        for a, b in zip(replayed, outs):
            assert torch.isfinite(a.float()).all()
            assert torch.equal(a, b)
