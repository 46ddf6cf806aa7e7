"""ctypes front end of the CPU checker (test infrastructure, never shipped).

Only the tests, the smoke test and the benchmark's CPU-baseline leg import
this module.  It wraps

* ``liboracle.so``            - the C restatement (``attention_oracle.c``) of
  the reference's naive fp32 attention (src/demo.cu:28-70) extended with LSE,
  rectangular problems and row subsets;
* ``_ref/libref_cpu.so``      - the reference's own ``cpu_attention`` compiled
  from the reference checkout (when it was available at build time);

and gives a float64 numpy restatement used to cross-check both on small cases
and to check whole long-sequence heads quickly through BLAS.
"""
from __future__ import annotations

import ctypes
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import build_oracle as _b

_F = ctypes.POINTER(ctypes.c_float)
_I = ctypes.POINTER(ctypes.c_int)
_lib = None
_ref = None


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_F)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_b.HERE, "liboracle.so")
        if not os.path.exists(path):
            _b.build_oracle()
        _lib = ctypes.CDLL(path)
        _lib.fa_oracle_rows.restype = ctypes.c_int
        _lib.fa_oracle_rows.argtypes = [_F, _F, _F, _F, _F, _F, _I, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int]
        _lib.fa_oracle_merge.restype = None
        _lib.fa_oracle_merge.argtypes = [_F, _F, ctypes.c_int, ctypes.c_int, _F, _F]
    return _lib


def ref_lib():
    """The reference's own cpu_attention, or None when it was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(_b.REF_OUT, "libref_cpu.so")
        if not os.path.exists(path):
            if not _b.have_reference():
                return None
            _b.build_ref_cpu()
        _ref = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        fn = getattr(_ref, _b.REF_CPU_SYMBOL)
        fn.restype = None
        fn.argtypes = [_F, _F, _F, _F, _F, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_bool]
    return _ref


def head_rows(q, k, v, scale, causal, rows=None, causal_shift=0, want_p=False):
    """One head through the C restatement.  q [Sq,D], k/v [Skv,D] float32.
    Returns (o [n_rows,D], lse [n_rows], p [n_rows,Skv] or None)."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    n_kv, d = k.shape
    if rows is None:
        n_rows, rows_p = q.shape[0], None
    else:
        rows = np.ascontiguousarray(rows, np.int32)
        n_rows, rows_p = rows.size, rows.ctypes.data_as(_I)
    o = np.empty((n_rows, d), np.float32)
    lse = np.empty((n_rows,), np.float32)
    p = np.empty((n_rows, n_kv), np.float32) if want_p else None
    rc = lib().fa_oracle_rows(_fp(q), _fp(k), _fp(v), _fp(o), _fp(lse),
                              _fp(p) if want_p else None, rows_p, n_rows, n_kv, d,
                              float(scale), int(bool(causal)), int(causal_shift))
    if rc != 0:
        raise MemoryError("oracle scratch allocation failed")
    return o, lse, p


def attention(q, k, v, scale, causal, rows=None, causal_shift=0, threads=None):
    """All heads.  q [BH,Sq,D], k/v [BH,Skv,D] float32 -> (o [BH,n_rows,D], lse [BH,n_rows]).
    Heads run on a thread pool (ctypes releases the GIL)."""
    bh = q.shape[0]
    threads = threads or min(bh, os.cpu_count() or 1)

    def one(i):
        o, lse, _ = head_rows(q[i], k[i], v[i], scale, causal, rows, causal_shift)
        return o, lse

    with ThreadPoolExecutor(max_workers=threads) as ex:
        res = list(ex.map(one, range(bh)))
    return np.stack([r[0] for r in res]), np.stack([r[1] for r in res])


def ref_head(q, k, v, scale, causal):
    """One square head through the reference's own cpu_attention.  Returns (o, p)."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("reference cpu_attention was not built (oracle/_ref missing)")
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    s, d = q.shape
    o = np.empty((s, d), np.float32)
    p = np.empty((s, s), np.float32)
    getattr(r, _b.REF_CPU_SYMBOL)(_fp(q), _fp(k), _fp(v), _fp(o), _fp(p), s, d, float(scale), bool(causal))
    return o, p


def ref_attention(q, k, v, scale, causal, threads=None):
    """All heads through the reference's cpu_attention on a thread pool; o only."""
    bh = q.shape[0]
    threads = threads or min(bh, os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=threads) as ex:
        res = list(ex.map(lambda i: ref_head(q[i], k[i], v[i], scale, causal)[0], range(bh)))
    return np.stack(res)


def merge(o_part, lse_part):
    """LSE merge of partial results.  o_part [..., P, D], lse_part [..., P] ->
    (o [..., D], lse [...]) through the C restatement."""
    o_part = np.ascontiguousarray(o_part, np.float32)
    lse_part = np.ascontiguousarray(lse_part, np.float32)
    lead = lse_part.shape[:-1]
    n_parts, d = o_part.shape[-2:]
    op = o_part.reshape(-1, n_parts, d)
    lp = lse_part.reshape(-1, n_parts)
    o = np.empty((op.shape[0], d), np.float32)
    lse = np.empty((op.shape[0],), np.float32)
    for i in range(op.shape[0]):
        lib().fa_oracle_merge(_fp(op[i]), _fp(lp[i]), n_parts, d, _fp(o[i]),
                              lse[i:i + 1].ctypes.data_as(_F))
    return o.reshape(*lead, d), lse.reshape(lead)


def attention_f64(q, k, v, scale, causal, causal_shift=0):
    """float64 numpy restatement (BLAS matmuls): q [...,Sq,D], k/v [...,Skv,D].
    Same definition as the C oracle, evaluated in double; used to cross-check it
    and to check whole long heads quickly.  Returns (o, lse) float64."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64)
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * float(scale)
    if causal:
        sq, skv = s.shape[-2:]
        i = np.arange(sq)[:, None]
        j = np.arange(skv)[None, :]
        s = np.where(j > i + causal_shift, -np.inf, s)
    m = s.max(axis=-1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(axis=-1, keepdims=True)
    o = np.matmul(p / l, v)
    return o, (m + np.log(l))[..., 0]


# ----------------------------------------------------------------------------
# Synthetic inputs: iid N(0,1) from a seeded generator, rounded to the storage
# type; the oracle always sees the rounded values converted back to float32.
# ----------------------------------------------------------------------------
def normal_inputs(seed: int, shape, n: int = 3):
    rng = np.random.Generator(np.random.Philox(seed))
    return [rng.standard_normal(shape, dtype=np.float32) for _ in range(n)]


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 -> storage dtype -> float32 (what the GPU actually consumes)."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    td = {"f16": torch.float16, "bf16": torch.bfloat16, "e4m3": torch.float8_e4m3fn}[dtype]
    return t.to(td).to(torch.float32).numpy()


def quantize_e4m3(x: np.ndarray):
    """Per-(b,h) absmax quantisation to e4m3: x [BH,S,D] float32 ->
    (codes uint8 [BH,S,D], scale float32 [BH], dequantised float32 [BH,S,D]);
    scale = absmax/448 so that x ~= code_value * scale."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    amax = t.abs().amax(dim=(1, 2)).clamp_min(1e-12)
    scale = (amax / 448.0).to(torch.float32)
    q8 = (t / scale[:, None, None]).to(torch.float8_e4m3fn)
    deq = q8.to(torch.float32) * scale[:, None, None]
    return q8.view(torch.uint8).numpy(), scale.numpy(), deq.numpy()
