"""fa_decode_static: the decode entry point for callers that are not allowed to
allocate device memory (their runtime owns every byte, or cudaMalloc's implicit
device synchronisation is unacceptable to them).  It keeps the per-split partial
results in an array built into the library instead of a caller workspace.

Checked here, through the C ABI: its output equals fa_decode's on the same
inputs, on two calls in a row of different shape (the second reuses the array
while it still holds the first call's partials), and a problem larger than the
built-in array is refused without launching anything.

This file sorts last on purpose, so a run that stops at the first failure has
already run every other test; it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inputs(oracle, seed, bh, skv, d, dtype, dev):
    import torch
    td = torch.float16 if dtype == "f16" else torch.bfloat16
    k, v = (oracle.round_to(x, dtype) for x in oracle.normal_inputs(seed, (bh, skv, d), n=2))
    q = oracle.round_to(oracle.normal_inputs(seed + 1, (bh, 1, d), n=1)[0], dtype)
    return q, k, v, tuple(torch.from_numpy(x).to(dev, td) for x in (q.reshape(bh, d), k, v))


def _both(fa, dev, dq, dk, dv, bh, skv, d, scale, dtype, splits):
    import torch
    outs = []
    for static in (False, True):
        o = torch.full((bh, d), float("nan"), device=dev, dtype=dq.dtype)
        lse = torch.full((bh,), float("nan"), device=dev, dtype=torch.float32)
        of = torch.full((bh, d), float("nan"), device=dev, dtype=torch.float32)
        if static:
            rc = fa.decode_static_raw(dq, dk, dv, o, lse, of, 1, bh, skv, d, scale, dtype=dtype,
                                      num_splits=splits)
        else:
            wsb = fa.decode_workspace_bytes(1, bh, d, max(splits, fa.decode_default_splits(1, bh, skv)))
            ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
            rc = fa.decode_raw(dq, dk, dv, o, lse, of, 1, bh, skv, d, scale, dtype=dtype,
                               num_splits=splits, workspace=ws, workspace_bytes=wsb)
        assert rc == fa.FA_OK, fa.error_string(rc)
        torch.cuda.synchronize()
        outs.append((o.float().cpu().numpy(), lse.cpu().numpy(), of.cpu().numpy()))
    return outs


def test_static_scratch_decode_matches_workspace_decode_twice(fa, dev, oracle):
    # call 1: many parts; call 2: fewer heads, fewer splits, other d_head and dtype -> the array
    # still holds call 1's partials beyond (and under) what call 2 writes.
    for seed, bh, skv, d, dtype, splits in ((900, 6, 3000, 128, "f16", 8), (910, 3, 1000, 64, "bf16", 3)):
        scale = float(1.0 / np.sqrt(np.float32(d)))
        q, k, v, (dq, dk, dv) = _inputs(oracle, seed, bh, skv, d, dtype, dev)
        (o_ws, l_ws, f_ws), (o_st, l_st, f_st) = _both(fa, dev, dq, dk, dv, bh, skv, d, scale, dtype, splits)
        # same kernels, same split geometry: the two entry points must agree to the last bit,
        # well inside the 2e-3 / 1e-3 tolerances of the other decode tests
        assert np.abs(o_st - o_ws).max() <= 2e-3 and np.abs(l_st - l_ws).max() <= 1e-3
        assert np.array_equal(o_st, o_ws) and np.array_equal(l_st, l_ws) and np.array_equal(f_st, f_ws)
        o_ref, l_ref = oracle.attention(q, k, v, scale, False)
        assert np.abs(f_st - o_ref[:, 0]).max() < 1e-4
        assert np.abs(l_st - l_ref[:, 0]).max() < 1e-3


def test_static_scratch_default_splits(fa, dev, oracle):
    bh, skv, d = 4, 4096, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    q, k, v, (dq, dk, dv) = _inputs(oracle, 920, bh, skv, d, "f16", dev)
    (o_ws, l_ws, _), (o_st, l_st, _) = _both(fa, dev, dq, dk, dv, bh, skv, d, scale, "f16", 0)
    assert np.array_equal(o_st, o_ws) and np.array_equal(l_st, l_ws)


def test_static_scratch_rejects_oversized_problem(fa, dev):
    """16384 heads-x-splits at d_head 128 fit (8.45 MB); 2048 heads x 16 splits (16.9 MB of
    partials) do not, and the call must refuse on the host without launching.  The buffers are
    sized honestly for that problem (16 keys per head), so if the check ever regressed the result
    would be a wrong answer, not an out-of-bounds access."""
    import torch
    bh, skv, d = 2048, 16, 128
    q = torch.zeros((bh, d), device=dev, dtype=torch.float16)
    k = torch.zeros((bh, skv, d), device=dev, dtype=torch.float16)
    v = torch.zeros((bh, skv, d), device=dev, dtype=torch.float16)
    o = torch.full((bh, d), 7.0, device=dev, dtype=torch.float16)
    rc = fa.decode_static_raw(q, k, v, o, None, None, 64, 32, skv, d, 0.1, num_splits=16)
    assert rc == fa.FA_ERR_WORKSPACE
    torch.cuda.synchronize()
    assert (o == 7.0).all()                                   # nothing ran
    assert 2048 * 16 * 129 * 4 > fa.DECODE_STATIC_SCRATCH_BYTES >= 1024 * 16 * 129 * 4


def test_static_scratch_calls_leave_free_device_memory_unchanged(fa, dev, oracle):
    """The reason the entry point exists: after the first call on a device (which resolves the
    built-in array's address, and may be when the driver loads the library's device code), a call
    takes no device memory and gives none back."""
    import torch
    bh, skv, d = 8, 2048, 128
    scale = float(1.0 / np.sqrt(np.float32(d)))
    _, _, _, (dq, dk, dv) = _inputs(oracle, 930, bh, skv, d, "f16", dev)
    o = torch.empty((bh, d), device=dev, dtype=torch.float16)
    lse = torch.empty((bh,), device=dev, dtype=torch.float32)
    assert fa.decode_static_raw(dq, dk, dv, o, lse, None, 1, bh, skv, d, scale, num_splits=4) == fa.FA_OK
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for splits in (4, 8, 2):
        assert fa.decode_static_raw(dq, dk, dv, o, lse, None, 1, bh, skv, d, scale, num_splits=splits) == fa.FA_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
