"""CPU-only: pins the oracle against the reference's golden vectors and checks
the oracle's own extensions (LSE, row subsets, rectangular, merge)."""
import ctypes

import numpy as np
import pytest


def test_demo_fixture_matches_oracle(oracle, golden):
    """scripts/{q,k,v}_data.bin -> output_ref.bin / attention_weights.bin of the
    reference (B=1,H=4,S=256,D=64, causal, scale 1/8)."""
    g = golden["demo_b1h4s256d64"]
    q, k, v = (g[n][0] for n in "qkv")
    o, lse = oracle.attention(q, k, v, 0.125, True)
    assert np.abs(o - g["o_ref"][0]).max() < 2e-6
    for h in range(4):
        _, _, p = oracle.head_rows(q[h], k[h], v[h], 0.125, True, rows=np.arange(0, 256, 8), want_p=True)
        assert np.abs(p - g["p_ref_rows8"][0, h]).max() < 5e-6
    o64, l64 = oracle.attention_f64(q, k, v, 0.125, True)
    assert np.abs(o64 - o).max() < 2e-6
    assert np.abs(l64 - lse).max() < 2e-5


def _gate_inputs(n):
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    libc.rand.restype = ctypes.c_int
    r = np.array([libc.rand() for _ in range(3 * n)], dtype=np.float32)
    vals = (r / np.float32(2147483647) - np.float32(0.5)) * np.float32(0.5)
    return vals[0::3].copy(), vals[1::3].copy(), vals[2::3].copy()


@pytest.mark.parametrize("shape", [(1, 1, 64, 64), (1, 1, 128, 64), (1, 2, 256, 64)])
def test_bench_gate_fixture_matches_oracle(oracle, golden, shape):
    """The reference's correctness-gate shapes and srand(42) generator
    (src/bench.cu:185-190, 385-387); outputs recorded from its cpu_attention."""
    b, h, s, d = shape
    tag = f"b{b}h{h}s{s}d{d}"
    q, k, v = (x.reshape(b * h, s, d) for x in _gate_inputs(b * h * s * d))
    insum = golden["bench_gate"][tag + "_insum"]
    got = np.array([q.astype(np.float64).sum(), k.astype(np.float64).sum(), v.astype(np.float64).sum()])
    if not np.allclose(insum, got, rtol=0, atol=1e-9):
        pytest.skip("libc rand() differs from the one the fixture was made with")
    o, _ = oracle.attention(q, k, v, 1.0 / np.sqrt(np.float32(d)), True)
    assert np.array_equal(o, golden["bench_gate"][tag + "_o"])


def test_normal_small_fixture(oracle, golden):
    g = golden["normal_small"]
    for idx in range(4):
        bh, s, d, causal, seed = (int(x) for x in g[f"case{idx}_meta"])
        q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(seed, (bh, s, d)))
        o, lse = oracle.attention(q, k, v, float(1.0 / np.sqrt(np.float32(d))), bool(causal))
        assert np.array_equal(o, g[f"case{idx}_o"])
        assert np.array_equal(lse, g[f"case{idx}_lse"])


def test_reference_function_bit_exact_when_built(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("reference cpu_attention not built on this machine")
    q, k, v = oracle.normal_inputs(5, (1, 96, 64))
    for causal in (True, False):
        ro, rp = oracle.ref_head(q[0], k[0], v[0], 0.125, causal)
        o, _, p = oracle.head_rows(q[0], k[0], v[0], 0.125, causal, want_p=True)
        assert np.array_equal(ro, o) and np.array_equal(rp, p)


def test_row_subset_and_rectangular(oracle):
    q, k, v = oracle.normal_inputs(6, (1, 80, 64))
    o_all, l_all, _ = oracle.head_rows(q[0], k[0], v[0], 0.125, True)
    rows = np.array([0, 7, 79], np.int32)
    o_sub, l_sub, _ = oracle.head_rows(q[0], k[0], v[0], 0.125, True, rows=rows)
    assert np.array_equal(o_sub, o_all[rows]) and np.array_equal(l_sub, l_all[rows])
    # last causal row == single-row non-causal decode over the whole cache
    o_dec, l_dec, _ = oracle.head_rows(q[0][79:80], k[0], v[0], 0.125, False)
    assert np.array_equal(o_dec[0], o_all[79]) and l_dec[0] == l_all[79]


def test_merge_equals_unsplit(oracle):
    k, v = oracle.normal_inputs(8, (2, 300, 64), n=2)
    q = oracle.normal_inputs(9, (2, 1, 64), n=1)[0]
    o_full, l_full = oracle.attention(q, k, v, 0.125, False)
    parts_o, parts_l = [], []
    for a, b in ((0, 100), (100, 228), (228, 300)):
        o, l = oracle.attention(q, k[:, a:b], v[:, a:b], 0.125, False)
        parts_o.append(o[:, 0]); parts_l.append(l[:, 0])
    o_m, l_m = oracle.merge(np.stack(parts_o, 1), np.stack(parts_l, 1))
    assert np.abs(o_m - o_full[:, 0]).max() < 1e-6
    assert np.abs(l_m - l_full[:, 0]).max() < 1e-5


def test_e4m3_quantiser_roundtrip(oracle):
    x = oracle.normal_inputs(10, (2, 64, 128), n=1)[0]
    codes, scale, deq = oracle.quantize_e4m3(x)
    assert codes.dtype == np.uint8 and scale.shape == (2,)
    assert np.abs(deq - x).max() < 0.07 * np.abs(x).max()
