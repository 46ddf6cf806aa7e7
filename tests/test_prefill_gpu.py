"""Prefill parity through the C ABI against the CPU oracle and the golden fixtures.

Tolerances (stated by the task for N(0,1) inputs): fp16 outputs max-abs 2e-3,
LSE max-abs 1e-3.  bf16 outputs cannot meet 2e-3 against an fp32 oracle because
rounding a value in [1,2) to bf16 alone moves it by up to 3.9e-3; they are held
to 1e-2 against the fp32 oracle and to one bf16 ulp + 3e-3 against the oracle
rounded to bf16."""
import ctypes

import numpy as np
import pytest

from helpers import nrmse_and_bad, run_prefill

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("prefill_variant")]

TOL_O_F16 = 2e-3
TOL_LSE = 1e-3
TOL_O_BF16 = 1e-2


def _check(fa, dev, oracle, seed, bh, s, d, causal, dtype="f16"):
    scale = float(1.0 / np.sqrt(np.float32(d)))
    q, k, v = (oracle.round_to(x, dtype) for x in oracle.normal_inputs(seed, (bh, s, d)))
    o, lse = run_prefill(fa, dev, q, k, v, scale, causal, dtype)
    o_ref, l_ref = oracle.attention(q, k, v, scale, causal)
    assert np.isfinite(o).all() and np.isfinite(lse).all()
    err_o, err_l = np.abs(o - o_ref).max(), np.abs(lse - l_ref).max()
    assert err_l < TOL_LSE, (err_l, err_o)
    assert err_o < (TOL_O_F16 if dtype == "f16" else TOL_O_BF16), err_o
    return err_o, err_l


@pytest.mark.parametrize("s", [1, 63, 64, 65, 127, 128, 129, 255, 256, 300, 512])
@pytest.mark.parametrize("causal", [True, False])
def test_ragged_lengths_d64_f16(fa, dev, oracle, s, causal):
    _check(fa, dev, oracle, 100 + s, 3, s, 64, causal)


@pytest.mark.parametrize("s", [1, 100, 128, 200, 257, 640])
@pytest.mark.parametrize("causal", [True, False])
def test_ragged_lengths_d128_f16(fa, dev, oracle, s, causal):
    _check(fa, dev, oracle, 300 + s, 2, s, 128, causal)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
def test_bf16(fa, dev, oracle, d, causal):
    bh, s = 2, 384
    scale = float(1.0 / np.sqrt(np.float32(d)))
    q, k, v = (oracle.round_to(x, "bf16") for x in oracle.normal_inputs(500 + d, (bh, s, d)))
    o, lse = run_prefill(fa, dev, q, k, v, scale, causal, "bf16")
    o_ref, l_ref = oracle.attention(q, k, v, scale, causal)
    assert np.abs(lse - l_ref).max() < TOL_LSE
    assert np.abs(o - o_ref).max() < TOL_O_BF16
    # Where the 1e-2 goes: rounding the fp32 result to bf16 alone moves it by up to half an ulp of
    # bf16 (2^-9 relative: 3.9e-3 for |O| in [1, 2)); the rest is P, which is rounded to bf16 (8
    # significand bits) before P V.  (P in fp16 next to a bf16 V is not an option: tcgen05.mma
    # kind::f16 with different A and B formats is an illegal instruction on this GPU.)  The second
    # bound is against the oracle ROUNDED to bf16: one output ulp for the output rounding itself
    # plus the measured effect of the bf16 P, printed below.
    ulp = np.maximum(np.abs(o_ref), 2.0 ** -126) * 2.0 ** -7
    diff = np.abs(o - oracle.round_to(o_ref, "bf16"))
    print(f"bf16 d={d} causal={causal}: max|o - o_ref| = {np.abs(o - o_ref).max():.3e}, "
          f"max(|o - bf16(o_ref)| - ulp) = {(diff - ulp).max():.3e}")
    assert (diff <= ulp + 3e-3).all()


def test_config1_b1_h12_s512_d64_causal(fa, dev, oracle):
    """The reference-runnable configuration: full comparison, every row."""
    err_o, err_l = _check(fa, dev, oracle, 1001, 12, 512, 64, True)
    print(f"config1 max|dO|={err_o:.3e} max|dLSE|={err_l:.3e}")


def test_golden_normal_small(fa, dev, oracle, golden):
    g = golden["normal_small"]
    for idx in range(4):
        bh, s, d, causal, seed = (int(x) for x in g[f"case{idx}_meta"])
        q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(seed, (bh, s, d)))
        o, lse = run_prefill(fa, dev, q, k, v, float(1.0 / np.sqrt(np.float32(d))), bool(causal))
        assert np.abs(o - g[f"case{idx}_o"]).max() < TOL_O_F16
        assert np.abs(lse - g[f"case{idx}_lse"]).max() < TOL_LSE


def test_golden_demo_dump(fa, dev, oracle, golden):
    """The reference's committed demo vectors (structured, peaky heads): the GPU
    gets fp16-rounded inputs, the golden output was computed from the un-rounded
    fp32 ones, exactly as the reference's demo does (src/demo.cu:256-342), so the
    reference's own pass rule applies: NRMSE < 0.03 and no bad element."""
    g = golden["demo_b1h4s256d64"]
    q, k, v = (oracle.round_to(g[n][0], "f16") for n in "qkv")
    o, lse = run_prefill(fa, dev, q, k, v, 0.125, True)
    nrmse, bad = nrmse_and_bad(g["o_ref"][0], o)
    assert nrmse < 0.03 and bad == 0, (nrmse, bad)
    # against the oracle on the SAME rounded inputs the tight tolerance holds
    o_ref, l_ref = oracle.attention(q, k, v, 0.125, True)
    assert np.abs(o - o_ref).max() < TOL_O_F16
    assert np.abs(lse - l_ref).max() < TOL_LSE


def _gate_inputs(n):
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    libc.rand.restype = ctypes.c_int
    r = np.array([libc.rand() for _ in range(3 * n)], dtype=np.float32)
    vals = (r / np.float32(2147483647) - np.float32(0.5)) * np.float32(0.5)
    return vals[0::3].copy(), vals[1::3].copy(), vals[2::3].copy()


@pytest.mark.parametrize("shape", [(1, 1, 64, 64), (1, 1, 128, 64), (1, 2, 256, 64)])
def test_reference_bench_gate(fa, dev, oracle, golden, shape):
    """The reference's own correctness gate (src/bench.cu:174-305, 385-387)."""
    b, h, s, d = shape
    tag = f"b{b}h{h}s{s}d{d}"
    qf, kf, vf = (x.reshape(b * h, s, d) for x in _gate_inputs(b * h * s * d))
    q, k, v = (oracle.round_to(x, "f16") for x in (qf, kf, vf))
    o, _ = run_prefill(fa, dev, q, k, v, float(1.0 / np.sqrt(np.float32(d))), True)
    o_gold = golden["bench_gate"][tag + "_o"]
    insum = golden["bench_gate"][tag + "_insum"]
    if np.allclose(insum[0], qf.astype(np.float64).sum(), rtol=0, atol=1e-9):
        nrmse, bad = nrmse_and_bad(o_gold, o)
        assert nrmse < 0.03 and bad == 0, (nrmse, bad)
    o_ref, _ = oracle.attention(q, k, v, float(1.0 / np.sqrt(np.float32(d))), True)
    assert np.abs(o - o_ref).max() < TOL_O_F16


def test_lse_optional_and_rows_beyond_s_untouched(fa, dev, oracle):
    """L may be NULL (include/flash_attention.h:56); a ragged last tile must not
    write past the tensor."""
    import torch
    bh, s, d = 2, 130, 64
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(77, (bh, s, d)))
    buf = torch.full((bh * s * d + 4096,), 7.0, device=dev, dtype=torch.float16)
    dq, dk, dv = (torch.from_numpy(x).to(dev, torch.float16) for x in (q, k, v))
    fa.prefill(dq, dk, dv, buf, None, 1, bh, s, d, 0.125, True)
    torch.cuda.synchronize()
    assert (buf[bh * s * d:] == 7.0).all()
    o_ref, _ = oracle.attention(q, k, v, 0.125, True)
    assert np.abs(buf[:bh * s * d].float().cpu().numpy().reshape(bh, s, d) - o_ref).max() < TOL_O_F16


def test_headline_shape_properties(fa, dev, oracle, prefill_variant):
    """B=8,H=12,S=2048,D=64 causal at full size: spot-check heads against the
    oracle, and check properties that hold at any size: row 0 attends only to
    key 0 (O[0] == V[0], LSE[0] == scale*q0.k0), and heads are independent
    (a head's result does not depend on which batch it is computed in)."""
    import torch
    if prefill_variant == "auto":
        # bit-identity across batch sizes holds per kernel; the library's own choice differs
        # between 96 heads and one head, so pin the kernel the 96 heads get
        fa.set_prefill_variant("tile_pair")
    bh, s, d = 96, 2048, 64
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(2002, (bh, s, d)))
    o, lse = run_prefill(fa, dev, q, k, v, 0.125, True)
    assert np.isfinite(o).all() and np.isfinite(lse).all()
    assert np.abs(o[:, 0, :] - v[:, 0, :]).max() < 1e-3
    assert np.abs(lse[:, 0] - 0.125 * (q[:, 0] * k[:, 0]).sum(-1)).max() < TOL_LSE
    heads = [0, 37, 95]
    rows = np.concatenate([np.arange(0, 130), np.arange(1000, 1030), np.arange(2040, 2048)]).astype(np.int32)
    o_ref, l_ref = oracle.attention(q[heads], k[heads], v[heads], 0.125, True, rows=rows)
    assert np.abs(o[heads][:, rows] - o_ref).max() < TOL_O_F16
    assert np.abs(lse[heads][:, rows] - l_ref).max() < TOL_LSE
    o1, l1 = run_prefill(fa, dev, q[37:38], k[37:38], v[37:38], 0.125, True)
    assert np.array_equal(o1[0], o[37]) and np.array_equal(l1[0], lse[37])


def test_cpp_entry_point(fa, dev, oracle):
    """transformer::launch_flash_attention(const FlashAttentionParams&), the
    reference's public function (include/flash_attention.h:67), called by its
    mangled name with the reference's struct layout."""
    import torch

    class Params(ctypes.Structure):
        _fields_ = [("Q", ctypes.c_void_p), ("K", ctypes.c_void_p), ("V", ctypes.c_void_p),
                    ("O", ctypes.c_void_p), ("L", ctypes.c_void_p), ("batch_size", ctypes.c_int),
                    ("num_heads", ctypes.c_int), ("seq_len", ctypes.c_int), ("d_head", ctypes.c_int),
                    ("scale", ctypes.c_float), ("causal", ctypes.c_bool), ("stream", ctypes.c_void_p),
                    ("dtype", ctypes.c_int)]

    bh, s, d = 4, 256, 64
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(88, (bh, s, d)))
    dq, dk, dv = (torch.from_numpy(x).to(dev, torch.float16) for x in (q, k, v))
    do = torch.zeros_like(dq)
    dl = torch.zeros((bh, s), device=dev, dtype=torch.float32)
    p = Params(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), do.data_ptr(), dl.data_ptr(), 2, 2, s, d,
               0.125, True, None, 0)
    fn = getattr(fa.lib(), "_ZN11transformer22launch_flash_attentionERKNS_20FlashAttentionParamsE")
    fn.restype = None
    fn.argtypes = [ctypes.POINTER(Params)]
    fn(ctypes.byref(p))
    torch.cuda.synchronize()
    o_ref, l_ref = oracle.attention(q, k, v, 0.125, True)
    assert np.abs(do.float().cpu().numpy() - o_ref).max() < TOL_O_F16
    assert np.abs(dl.cpu().numpy() - l_ref).max() < TOL_LSE


def test_host_buffer_entry(fa, dev, oracle):
    bh, s, d = 3, 200, 64
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(99, (bh, s, d)))
    hq, hk, hv = (x.astype(np.float16) for x in (q, k, v))
    ho = np.zeros_like(hq)
    hl = np.zeros((bh, s), np.float32)
    rc = fa.prefill_raw(hq.ctypes.data, hk.ctypes.data, hv.ctypes.data, ho.ctypes.data, hl.ctypes.data,
                        1, bh, s, d, 0.125, True, host=True)
    assert rc == 0
    o_ref, l_ref = oracle.attention(q, k, v, 0.125, True)
    assert np.abs(ho.astype(np.float32) - o_ref).max() < TOL_O_F16
    assert np.abs(hl - l_ref).max() < TOL_LSE


def test_host_buffer_entry_pipelined_chunks(fa, dev, oracle):
    """fa_prefill_host cuts large inputs into chunks of heads that flow through several streams;
    the result must be bit-identical to the single-launch device-pointer path."""
    import torch
    bh, s, d = 96, 2048, 64                       # 25 MB per input tensor -> 3 chunks
    q, k, v = (torch.randn((bh, s, d), generator=torch.Generator().manual_seed(7 + i)).to(torch.float16)
               for i in range(3))
    ho = torch.empty_like(q)
    hl = torch.empty((bh, s), dtype=torch.float32)
    rc = fa.prefill_raw(q.data_ptr(), k.data_ptr(), v.data_ptr(), ho.data_ptr(), hl.data_ptr(),
                        8, 12, s, d, 0.125, True, host=True)
    assert rc == 0
    dq, dk, dv = (x.to(dev) for x in (q, k, v))
    do = torch.empty_like(dq)
    dl = torch.empty((bh, s), device=dev, dtype=torch.float32)
    fa.prefill(dq, dk, dv, do, dl, 8, 12, s, d, 0.125, True)
    torch.cuda.synchronize()
    assert torch.equal(ho, do.cpu()) and torch.equal(hl, dl.cpu())
    heads = [0, 50, 95]
    rows = np.array([0, 1, 127, 128, 1000, 2047], np.int32)
    o_ref, l_ref = oracle.attention(q[heads].float().numpy(), k[heads].float().numpy(), v[heads].float().numpy(),
                                    0.125, True, rows=rows)
    assert np.abs(ho[heads].float().numpy()[:, rows] - o_ref).max() < TOL_O_F16
    assert np.abs(hl[heads].numpy()[:, rows] - l_ref).max() < TOL_LSE
