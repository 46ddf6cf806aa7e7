"""Helpers shared by the GPU parity tests."""
import numpy as np

TORCH_DT = {"f16": "float16", "bf16": "bfloat16"}


def to_dev(x: np.ndarray, dtype: str, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev, getattr(torch, TORCH_DT[dtype]))


def run_prefill(fa, dev, q, k, v, scale, causal, dtype="f16", want_lse=True):
    """q,k,v float32 [BH,S,D] already rounded to dtype.  Returns (o float32, lse float32)."""
    import torch
    bh, s, d = q.shape
    dq, dk, dv = (to_dev(x, dtype, dev) for x in (q, k, v))
    do = torch.full_like(dq, float("nan"))
    dl = torch.full((bh, s), float("nan"), device=dev, dtype=torch.float32) if want_lse else None
    fa.prefill(dq, dk, dv, do, dl, 1, bh, s, d, float(scale), causal, dtype=dtype)
    torch.cuda.synchronize()
    return do.float().cpu().numpy(), (dl.cpu().numpy() if want_lse else None)


def nrmse_and_bad(ref: np.ndarray, got: np.ndarray):
    """The reference's pass rule (src/bench.cu:282-301): NRMSE and the count of
    elements with abs error > 0.05 and relative error > 0.1."""
    ref = ref.astype(np.float64).ravel()
    got = got.astype(np.float64).ravel()
    err = np.abs(ref - got)
    rel = err / (np.abs(ref) + 1e-6)
    nrmse = np.sqrt((err ** 2).sum() / ((ref ** 2).sum() + 1e-10))
    return float(nrmse), int(((err > 0.05) & (rel > 0.1)).sum())
