"""Tensor-core known-answer test through the C ABI (fa_kat): the tcgen05 analogue
of the reference's identity-matrix MMA check (src/bench.cu:51-165)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bits(x, dtype):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    t = t.to(torch.float16 if dtype == "f16" else torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16).copy(), t.float().numpy()


def _round16(x, dtype):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    return t.to(torch.float16 if dtype == "f16" else torch.bfloat16).float().numpy()


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("d", [64, 128])
def test_identity_counting_pattern_exact(fa, dev, dtype, d):
    """Q = stacked identities, K = V = small integer counting patterns: every
    product and sum is exactly representable, so S and O must match exactly."""
    q = np.zeros((128, d), np.float32)
    q[np.arange(128), np.arange(128) % d] = 1.0
    k = ((np.arange(128)[:, None] * 3 + np.arange(d)[None, :]) % 7).astype(np.float32)
    v = ((np.arange(128)[:, None] + 2 * np.arange(d)[None, :]) % 5).astype(np.float32) - 2.0
    (qb, qf), (kb, kf), (vb, vf) = (_bits(x, dtype) for x in (q, k, v))
    s, o = fa.kat(dtype, d, qb, kb, vb, 1.0)
    s_ref = qf @ kf.T                      # S[r][j] = K[j][r % d]
    assert np.array_equal(s, s_ref)
    o_ref = _round16(s_ref, dtype).astype(np.float64) @ vf.astype(np.float64)
    assert np.array_equal(o, o_ref.astype(np.float32))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("d", [64, 128])
def test_random_tile(fa, dev, dtype, d):
    rng = np.random.default_rng(3)
    (qb, qf), (kb, kf), (vb, vf) = (_bits(rng.standard_normal((128, d), dtype=np.float32), dtype)
                                    for _ in range(3))
    p_scale = 0.05
    s, o = fa.kat(dtype, d, qb, kb, vb, p_scale)
    s_ref = qf.astype(np.float64) @ kf.astype(np.float64).T
    assert np.abs(s - s_ref).max() < 1e-3
    p = _round16(s * np.float32(p_scale), dtype).astype(np.float64)
    o_ref = p @ vf.astype(np.float64)
    assert np.abs(o - o_ref).max() < 1e-3
