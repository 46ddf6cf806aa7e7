"""PyTorch custom operators over the C ABI: ``torch.ops.fa_b200.prefill`` / ``decode`` /
``decode_gqa`` / ``prefill_backward``.

``prefill`` is differentiable with respect to q, k and v (``fa_backward``); the gradient of its LSE
output is not supported.  ``decode`` is forward only.  Tensors use the layout of
``torch.nn.functional.scaled_dot_product_attention``: ``[B, H, S, D]``,
contiguous, fp16 or bf16, on a CUDA device; the kernels see them as the
reference's ``[B*H, S, D]`` (include/flash_attention.h:46-61).  The operators
launch on the current CUDA stream of the tensors' device and allocate their
outputs (and the decode workspace) with torch.

``sdpa()`` is a convenience with the keyword names of
``scaled_dot_product_attention`` for the cases this library covers.

There is no fallback: on a machine without the library or without a B200-class
GPU the operators raise.
"""
from __future__ import annotations

import math

import torch

import fa_b200 as _fa
from fa_b200 import FaError

_DTYPES = {torch.float16: "f16", torch.bfloat16: "bf16"}


def _check(q, k, v):
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("fa_b200: q, k, v must share dtype float16 or bfloat16")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("fa_b200: tensors must be on a CUDA device (there is no CPU path)")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("fa_b200: expected [B, H, S, D] tensors")


@torch.library.custom_op("fa_b200::prefill", mutates_args=())
def prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
            causal: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """Self-attention forward.  Returns (O [B,H,S,D] in the input dtype, LSE [B,H,S] fp32, natural log)."""
    _check(q, k, v)
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("fa_b200::prefill: q, k, v must have the same shape")
    b, h, s, d = q.shape
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((b, h, s), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        _fa.prefill(q, k, v, o, lse, b, h, s, d, float(scale), bool(causal), dtype=_DTYPES[q.dtype],
                    stream=torch.cuda.current_stream(q.device))
    return o, lse


@prefill.register_fake
def _(q, k, v, scale, causal):
    b, h, s, _ = q.shape
    return torch.empty_like(q), q.new_empty((b, h, s), dtype=torch.float32)


@torch.library.custom_op("fa_b200::prefill_backward", mutates_args=())
def prefill_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                     d_o: torch.Tensor, scale: float, causal: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients (dQ, dK, dV) of ``prefill`` for the upstream gradient ``d_o`` of O."""
    _check(q, k, v)
    b, h, s, d = q.shape
    q, k, v, o, d_o, lse = (t.contiguous() for t in (q, k, v, o, d_o.to(q.dtype), lse))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    with torch.cuda.device(q.device):
        wsb = _fa.backward_workspace_bytes(b, h, s)
        ws = torch.empty(wsb, device=q.device, dtype=torch.uint8)
        _fa.backward(q, k, v, o, d_o, lse, dq, dk, dv, b, h, s, d, float(scale), bool(causal),
                     dtype=_DTYPES[q.dtype], workspace=ws, workspace_bytes=wsb,
                     stream=torch.cuda.current_stream(q.device))
    return dq, dk, dv


@prefill_backward.register_fake
def _(q, k, v, o, lse, d_o, scale, causal):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _prefill_setup_context(ctx, inputs, output):
    q, k, v, scale, causal = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.scale, ctx.causal = scale, causal


def _prefill_backward(ctx, d_o, d_lse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = prefill_backward(q, k, v, o, lse, d_o, ctx.scale, ctx.causal)
    return dq, dk, dv, None, None


torch.library.register_autograd("fa_b200::prefill", _prefill_backward, setup_context=_prefill_setup_context)


@torch.library.custom_op("fa_b200::decode", mutates_args=())
def decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
           num_splits: int) -> tuple[torch.Tensor, torch.Tensor]:
    """One query row per head against a KV cache: q [B,H,1,D], k/v [B,H,Skv,D].

    Returns (O [B,H,1,D], LSE [B,H,1]).  ``num_splits`` 0 picks the library default."""
    _check(q, k, v)
    b, h, one, d = q.shape
    if one != 1 or k.shape[:2] != (b, h) or k.shape[3] != d or v.shape != k.shape:
        raise ValueError("fa_b200::decode: expected q [B,H,1,D] and k, v [B,H,Skv,D]")
    skv = k.shape[2]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((b, h, 1), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        splits = num_splits if num_splits > 0 else _fa.decode_default_splits(b, h, skv)
        ws_bytes = _fa.decode_workspace_bytes(b, h, d, splits)
        ws = torch.empty(ws_bytes, device=q.device, dtype=torch.uint8)
        _fa.decode(q, k, v, o, lse, None, b, h, skv, d, float(scale), dtype=_DTYPES[q.dtype],
                   num_splits=splits, workspace=ws, workspace_bytes=ws_bytes,
                   stream=torch.cuda.current_stream(q.device))
    return o, lse


@decode.register_fake
def _(q, k, v, scale, num_splits):
    b, h, _, _ = q.shape
    return torch.empty_like(q), q.new_empty((b, h, 1), dtype=torch.float32)


@torch.library.custom_op("fa_b200::decode_gqa", mutates_args=())
def decode_gqa(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, scale: float,
               seq_lens: torch.Tensor | None = None,
               block_table: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Grouped-query attention of new tokens over a KV cache (``fa_decode_gqa``).

    q ``[B, T, Hq, D]`` (the T tokens are the last T cache entries of each sequence; token t sees keys
    up to its own position).  Cache, not paged: ``[B, Skv, Hkv, D]``; paged (``block_table`` int32
    ``[B, max_pages]``): page pools ``[P, page_size, Hkv, D]``.  ``seq_lens`` int32 ``[B]`` optional.
    Returns (O ``[B, T, Hq, D]``, LSE ``[B, T, Hq]``)."""
    if q.dtype not in _DTYPES or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise TypeError("fa_b200::decode_gqa: q and the cache must share dtype float16 or bfloat16")
    if not (q.is_cuda and k_cache.is_cuda and v_cache.is_cuda):
        raise RuntimeError("fa_b200: tensors must be on a CUDA device (there is no CPU path)")
    if q.dim() != 4 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError("fa_b200::decode_gqa: expected q [B,T,Hq,D] and 4-D caches of equal shape")
    b, t, hq, d = q.shape
    q, k_cache, v_cache = q.contiguous(), k_cache.contiguous(), v_cache.contiguous()
    hkv = k_cache.shape[2]
    kw = {}
    if block_table is None:
        if k_cache.shape[0] != b:
            raise ValueError("fa_b200::decode_gqa: cache batch differs from q")
        skv = k_cache.shape[1]
        kw["kv_strides"] = (skv * hkv * d, d, hkv * d)
    else:
        n_pages, page = k_cache.shape[0], k_cache.shape[1]
        block_table = block_table.to(torch.int32).contiguous()
        skv = block_table.shape[1] * page
        kw.update(kv_strides=(0, d, hkv * d), block_table=block_table, block_table_stride=block_table.shape[1],
                  page_size=page, num_pages=n_pages, kv_page_stride=page * hkv * d)
    if seq_lens is not None:
        kw["seq_lens"] = seq_lens.to(torch.int32).contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((b, t, hq), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        group = hq // hkv
        n_qt = -(-t // max(1, min(t, 128 // group)))
        splits = _fa.decode_gqa_default_splits(b * n_qt, hkv, skv)
        ws_bytes = _fa.decode_workspace_bytes(b, t * hq, d, splits)
        ws = torch.empty(ws_bytes, device=q.device, dtype=torch.uint8)
        _fa.decode_gqa(q, k_cache, v_cache, o, lse, b, hq, hkv, skv, d, float(scale), dtype=_DTYPES[q.dtype],
                       num_splits=splits, num_q_tokens=t, workspace=ws, workspace_bytes=ws_bytes,
                       stream=torch.cuda.current_stream(q.device), **kw)
    return o, lse


@decode_gqa.register_fake
def _(q, k_cache, v_cache, scale, seq_lens=None, block_table=None):
    b, t, hq, _ = q.shape
    return torch.empty_like(q), q.new_empty((b, t, hq), dtype=torch.float32)


def sdpa(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, attn_mask=None,
         dropout_p: float = 0.0, is_causal: bool = False, scale: float | None = None) -> torch.Tensor:
    """``scaled_dot_product_attention`` for the cases the library covers (no mask, no dropout).

    Self-attention (equal sequence lengths) runs the prefill kernel; a single query row against a
    longer cache runs split-KV decode.  Anything else raises: there is no fallback."""
    if attn_mask is not None or dropout_p != 0.0:
        raise NotImplementedError("fa_b200.sdpa: attn_mask and dropout are not supported")
    d = query.shape[-1]
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    if query.shape[-2] == key.shape[-2]:
        return prefill(query, key, value, sc, bool(is_causal))[0]
    if query.shape[-2] == 1 and not is_causal:
        return decode(query, key, value, sc, 0)[0]
    raise NotImplementedError("fa_b200.sdpa: only self-attention and single-row decode are covered")


__all__ = ["prefill", "prefill_backward", "decode", "decode_gqa", "sdpa", "FaError"]
