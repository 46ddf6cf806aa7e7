"""FP8 (e4m3, per-(batch*head) absmax scales) prefill through the C ABI.

Q, K, V are drawn iid N(0,1) in fp32, quantised to e4m3 with scale = absmax/448
per head; the oracle runs in fp32 on the DEQUANTISED tensors, so the comparison
measures the kernel, not the quantiser.  Tolerance stated by the task: output
max-abs 3e-2 (bf16 output); LSE is fp32 and held to 1e-3 like the other paths."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_O_FP8 = 3e-2
TOL_LSE = 1e-3


def _run(fa, dev, oracle, seed, bh, s, causal):
    import torch
    d = 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    xs = oracle.normal_inputs(seed, (bh, s, d))
    codes, scales, deq = zip(*(oracle.quantize_e4m3(x) for x in xs))
    dq, dk, dv = (torch.from_numpy(c).to(dev) for c in codes)
    sq, sk, sv = (torch.from_numpy(x).to(dev) for x in scales)
    do = torch.full((bh, s, d), float("nan"), device=dev, dtype=torch.bfloat16)
    dl = torch.full((bh, s), float("nan"), device=dev, dtype=torch.float32)
    fa.prefill(dq, dk, dv, do, dl, 1, bh, s, d, scale, causal, dtype="e4m3",
               q_scale=sq, k_scale=sk, v_scale=sv)
    torch.cuda.synchronize()
    o_ref, l_ref = oracle.attention(deq[0], deq[1], deq[2], scale, causal)
    o = do.float().cpu().numpy()
    lse = dl.cpu().numpy()
    assert np.isfinite(o).all() and np.isfinite(lse).all()
    return np.abs(o - o_ref).max(), np.abs(lse - l_ref).max()


@pytest.mark.parametrize("s", [128, 200, 512, 1000])
@pytest.mark.parametrize("causal", [True, False])
def test_fp8_prefill(fa, dev, oracle, s, causal):
    err_o, err_l = _run(fa, dev, oracle, 600 + s, 3, s, causal)
    assert err_o < TOL_O_FP8, err_o
    assert err_l < TOL_LSE, err_l


def test_fp8_rejects_d64_and_missing_scales(fa, dev):
    import torch
    t = torch.zeros(4096, device=dev, dtype=torch.uint8)
    f = torch.ones(4, device=dev, dtype=torch.float32)
    assert fa.prefill_raw(t, t, t, t, None, 1, 1, 16, 64, 0.1, True, dtype="e4m3",
                          q_scale=f, k_scale=f, v_scale=f) == fa.FA_ERR_UNSUPPORTED
    assert fa.prefill_raw(t, t, t, t, None, 1, 1, 16, 128, 0.1, True, dtype="e4m3") == fa.FA_ERR_INVALID_ARGUMENT


def _device_inputs(dev, bh, s, seed):
    """e4m3 codes and scales made on the device (for sizes the numpy quantiser would take long on)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    xs = [torch.randn((bh, s, 128), device=dev, generator=g) for _ in range(3)]
    scales = [x.abs().amax(dim=(1, 2)) / 448.0 for x in xs]
    codes = [(x / sc[:, None, None]).to(torch.float8_e4m3fn) for x, sc in zip(xs, scales)]
    deq = [c.float() * sc[:, None, None] for c, sc in zip(codes, scales)]
    return [c.view(torch.uint8).contiguous() for c in codes], [sc.float().contiguous() for sc in scales], deq


def test_fp8_prefill_in_chunks_of_heads(fa, dev, oracle):
    """The fp16 copy of V is made in a bounded scratch: with more than 256 MB of it (1 100 heads of
    1 024 keys) the heads are processed in several chunks, each with its own pointers and scales.
    Heads from the first, a middle and the last chunk are checked against the oracle."""
    import torch
    bh, s = 1100, 1024
    scale = float(1.0 / np.sqrt(np.float32(128)))
    (q8, k8, v8), (sq, sk, sv), deq = _device_inputs(dev, bh, s, 77)
    o = torch.full((bh, s, 128), float("nan"), device=dev, dtype=torch.bfloat16)
    lse = torch.full((bh, s), float("nan"), device=dev, dtype=torch.float32)
    fa.prefill(q8, k8, v8, o, lse, 1, bh, s, 128, scale, True, dtype="e4m3", q_scale=sq, k_scale=sk, v_scale=sv)
    torch.cuda.synchronize()
    assert fa.device_status() == 0
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    heads = [0, 1, 511, 512, 1023, 1024, 1099]
    o_ref, l_ref = oracle.attention(*(x[heads].cpu().numpy() for x in deq), scale, True)
    assert np.abs(o[heads].float().cpu().numpy() - o_ref).max() < TOL_O_FP8
    assert np.abs(lse[heads].cpu().numpy() - l_ref).max() < TOL_LSE


def test_fp8_prefill_scratch_is_kept_and_stream_ordered(fa, dev):
    """After the first call the library's pool holds the scratch: later calls, with synchronisations in
    between, leave the free device memory unchanged; calls on two streams give what a single call gives."""
    import torch
    bh, s = 8, 512
    scale = float(1.0 / np.sqrt(np.float32(128)))
    (q8, k8, v8), (sq, sk, sv), _ = _device_inputs(dev, bh, s, 78)
    kw = dict(dtype="e4m3", q_scale=sq, k_scale=sk, v_scale=sv)

    def call(stream=None):
        o = torch.empty((bh, s, 128), device=dev, dtype=torch.bfloat16)
        lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
        fa.prefill(q8, k8, v8, o, lse, 1, bh, s, 128, scale, False, stream=stream, **kw)
        return o, lse

    o0, l0 = call()
    torch.cuda.synchronize()
    outs = None
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        outs = call()
        torch.cuda.synchronize()
    del outs
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0 - (4 << 20), "the e4m3 scratch should be reused, not re-allocated"
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        o1, l1 = call(s1)
    with torch.cuda.stream(s2):
        o2, l2 = call(s2)
    torch.cuda.synchronize()
    assert torch.equal(o1, o0) and torch.equal(o2, o0) and torch.equal(l1, l0) and torch.equal(l2, l0)
