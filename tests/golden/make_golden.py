"""Regenerates the committed golden fixtures from a checkout of the reference.

Run once where the reference checkout and the built ``oracle/_ref/libref_cpu.so``
exist:  ``python tests/golden/make_golden.py``.  The tests only read the
``.npz`` files this writes; they never need the checkout.

Fixtures
--------
``demo_b1h4s256d64.npz``
    The reference's committed demo dump (scripts/q_data.bin, k_data.bin,
    v_data.bin -> output_ref.bin, attention_weights.bin; format written by
    src/demo.cu:75-93): un-rounded fp32 inputs of the four structured heads,
    the reference CPU output, and every 8th row of the attention weights.
    scripts/output_gpu.bin is a stale run of an older kernel and is left out.
``bench_gate.npz``
    The three correctness-gate shapes of src/bench.cu:385-387 with the
    ``srand(42)`` generator of src/bench.cu:185-190 (glibc ``rand``), pushed
    through the reference's own ``cpu_attention``; stores the outputs and a
    checksum of the inputs (the tests regenerate the inputs with the same libc
    calls and verify the checksum before use).
``normal_small.npz``
    Seeded N(0,1) fp16-rounded inputs at a few small shapes (causal and not,
    D=64 and 128) with output and LSE from the C restatement, after that
    restatement was checked bit-for-bit against ``cpu_attention``.
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402

# the reference checkout: FA_REFERENCE_DIR, else a directory "reference" next to this repository
REFERENCE = os.environ.get("FA_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def read_dump(path: str) -> np.ndarray:
    """int32 ndims, ndims x int32 dims, float32 row-major (src/demo.cu:75-93)."""
    raw = np.fromfile(path, dtype=np.uint8)
    ndims = int(raw[:4].view(np.int32)[0])
    dims = raw[4:4 + 4 * ndims].view(np.int32)
    data = raw[4 + 4 * ndims:].view(np.float32)
    return data.reshape([int(x) for x in dims]).copy()


def bench_gate_inputs(n_elems: int):
    """Q,K,V of src/bench.cu:185-190: srand(42), then per element three rand()
    calls in the order Q,K,V, each mapped to (rand()/RAND_MAX - 0.5) * 0.5."""
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    libc.rand.restype = ctypes.c_int
    r = np.array([libc.rand() for _ in range(3 * n_elems)], dtype=np.float32)
    rand_max = np.float32(2147483647)
    vals = (r / rand_max - np.float32(0.5)) * np.float32(0.5)
    return vals[0::3].copy(), vals[1::3].copy(), vals[2::3].copy()


def main() -> None:
    s = os.path.join(REFERENCE, "scripts")
    q, k, v = (read_dump(os.path.join(s, n + "_data.bin")) for n in "qkv")
    o_ref = read_dump(os.path.join(s, "output_ref.bin"))
    p_ref = read_dump(os.path.join(s, "attention_weights.bin"))
    np.savez_compressed(os.path.join(HERE, "demo_b1h4s256d64.npz"),
                        q=q, k=k, v=v, o_ref=o_ref, p_ref_rows8=p_ref[:, :, ::8, :].copy())

    gate = {}
    for (b, h, sl, d) in ((1, 1, 64, 64), (1, 1, 128, 64), (1, 2, 256, 64)):
        n = b * h * sl * d
        gq, gk, gv = (x.reshape(b * h, sl, d) for x in bench_gate_inputs(n))
        o = oracle.ref_attention(gq, gk, gv, 1.0 / np.sqrt(np.float32(d)), True)
        tag = f"b{b}h{h}s{sl}d{d}"
        gate[tag + "_o"] = o
        gate[tag + "_insum"] = np.array([gq.astype(np.float64).sum(), gk.astype(np.float64).sum(),
                                         gv.astype(np.float64).sum()])
    np.savez_compressed(os.path.join(HERE, "bench_gate.npz"), **gate)

    small = {}
    for idx, (bh, sl, d, causal) in enumerate(((3, 200, 64, 1), (2, 129, 64, 0), (2, 192, 128, 1),
                                               (1, 65, 128, 0))):
        q3, k3, v3 = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(700 + idx, (bh, sl, d)))
        scale = float(1.0 / np.sqrt(np.float32(d)))
        o3, l3 = oracle.attention(q3, k3, v3, scale, bool(causal))
        if causal or True:
            ro, _ = oracle.ref_head(q3[0], k3[0], v3[0], scale, bool(causal))
            assert np.array_equal(ro, o3[0]), "restatement drifted from the reference function"
        tag = f"case{idx}"
        small[tag + "_meta"] = np.array([bh, sl, d, causal, 700 + idx])
        small[tag + "_o"] = o3
        small[tag + "_lse"] = l3
    np.savez_compressed(os.path.join(HERE, "normal_small.npz"), **small)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
