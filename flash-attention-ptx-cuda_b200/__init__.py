"""Python binding of libfa_b200.so over its C ABI (include/fa_b200.h), via ctypes.

The product is the shared library; this module only marshals pointers so that
tests, the benchmark and Python callers reach the same entry points a C, Go or
Rust binding would.  There is no fallback path: if the library is missing or
the device is not a B200-class GPU, calls raise.

The directory name contains hyphens, so it cannot be imported with a plain
``import`` statement; ``__graft_entry__.load_package()`` loads it under the
module name ``fa_b200``.

Device memory is handled by the caller.  The helpers here accept raw integer
device pointers, or any object with ``data_ptr()`` (torch tensors are used for
allocation and streams only).
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# FA_B200_LIB points the binding at another build of the same library (development only).
LIB_PATH = os.environ.get("FA_B200_LIB") or os.path.join(HERE, "libfa_b200.so")

FA_OK = 0
FA_ERR_INVALID_ARGUMENT = -1
FA_ERR_UNSUPPORTED = -2
FA_ERR_MISALIGNED = -3
FA_ERR_WORKSPACE = -4
FA_ERR_CUDA = -5
FA_ERR_DEVICE_TIMEOUT = -6
FA_ERR_NOT_SM100 = -7
FA_ERR_NCCL = -8
FA_DTYPE_F16, FA_DTYPE_BF16, FA_DTYPE_E4M3 = 0, 1, 2
DTYPES = {"f16": FA_DTYPE_F16, "bf16": FA_DTYPE_BF16, "e4m3": FA_DTYPE_E4M3}

# Every symbol include/fa_b200.h declares; the CPU-only tests check they all resolve.
EXPORTED_SYMBOLS = (
    "fa_prefill", "fa_prefill_host", "fa_decode", "fa_decode_static", "fa_decode_workspace_bytes",
    "fa_decode_default_splits", "fa_decode_gqa", "fa_decode_gqa_default_splits", "fa_backward",
    "fa_backward_workspace_bytes", "fa_combine", "fa_kat",
    "fa_device_status",
    "fa_clear_device_status", "fa_error_string", "fa_last_cuda_error", "fa_version",
    "fa_set_prefill_variant", "fa_combine_packed", "fa_decode_kv_sharded", "fa_decode_kv_sharded_gather_bytes",
    "fa_nccl_unique_id", "fa_nccl_comm_create", "fa_nccl_comm_destroy", "fa_status_word_to_error",
)


class PrefillArgs(ctypes.Structure):
    """Mirror of ``fa_prefill_args`` (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("batch_size", ctypes.c_int), ("num_heads", ctypes.c_int), ("seq_len", ctypes.c_int),
        ("d_head", ctypes.c_int), ("scale", ctypes.c_float), ("causal", ctypes.c_int),
        ("dtype", ctypes.c_int),
        ("q_scale", ctypes.c_void_p), ("k_scale", ctypes.c_void_p), ("v_scale", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
    ]


class DecodeArgs(ctypes.Structure):
    """Mirror of ``fa_decode_args`` (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("o_f32", ctypes.c_void_p),
        ("batch_size", ctypes.c_int), ("num_heads", ctypes.c_int), ("seq_len_kv", ctypes.c_int),
        ("d_head", ctypes.c_int), ("scale", ctypes.c_float), ("dtype", ctypes.c_int),
        ("num_splits", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
    ]


class DecodeGqaArgs(ctypes.Structure):
    """Mirror of ``fa_decode_gqa_args`` (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("batch_size", ctypes.c_int), ("num_q_heads", ctypes.c_int), ("num_kv_heads", ctypes.c_int),
        ("seq_len_kv", ctypes.c_int), ("d_head", ctypes.c_int), ("scale", ctypes.c_float),
        ("dtype", ctypes.c_int), ("num_splits", ctypes.c_int),
        ("kv_batch_stride", ctypes.c_longlong), ("kv_head_stride", ctypes.c_longlong),
        ("kv_row_stride", ctypes.c_longlong),
        ("block_table", ctypes.c_void_p), ("block_table_stride", ctypes.c_int), ("page_size", ctypes.c_int),
        ("num_pages", ctypes.c_int), ("kv_page_stride", ctypes.c_longlong), ("seq_lens", ctypes.c_void_p),
        ("q_scale", ctypes.c_void_p), ("k_scale", ctypes.c_void_p), ("v_scale", ctypes.c_void_p),
        ("num_q_tokens", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
    ]


class BackwardArgs(ctypes.Structure):
    """Mirror of ``fa_backward_args`` (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("batch_size", ctypes.c_int), ("num_heads", ctypes.c_int), ("seq_len", ctypes.c_int),
        ("d_head", ctypes.c_int), ("scale", ctypes.c_float), ("causal", ctypes.c_int), ("dtype", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t), ("stream", ctypes.c_void_p),
    ]


class FaError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {error_string(code)} ({code})"
                         + (f" [{last_cuda_error()}]" if code == FA_ERR_CUDA else ""))
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libfa_b200.so (no fallback: a missing library is an error)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} not built; run `python flash-attention-ptx-cuda_b200/build.py`")
        l = ctypes.CDLL(LIB_PATH)
        l.fa_prefill.restype = ctypes.c_int
        l.fa_prefill.argtypes = [ctypes.POINTER(PrefillArgs)]
        l.fa_prefill_host.restype = ctypes.c_int
        l.fa_prefill_host.argtypes = [ctypes.POINTER(PrefillArgs)]
        l.fa_decode.restype = ctypes.c_int
        l.fa_decode.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.fa_decode_static.restype = ctypes.c_int
        l.fa_decode_static.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.fa_decode_workspace_bytes.restype = ctypes.c_size_t
        l.fa_decode_workspace_bytes.argtypes = [ctypes.c_int] * 4
        l.fa_decode_default_splits.restype = ctypes.c_int
        l.fa_decode_default_splits.argtypes = [ctypes.c_int] * 3
        l.fa_decode_gqa.restype = ctypes.c_int
        l.fa_decode_gqa.argtypes = [ctypes.POINTER(DecodeGqaArgs)]
        l.fa_decode_gqa_default_splits.restype = ctypes.c_int
        l.fa_decode_gqa_default_splits.argtypes = [ctypes.c_int] * 3
        l.fa_backward.restype = ctypes.c_int
        l.fa_backward.argtypes = [ctypes.POINTER(BackwardArgs)]
        l.fa_backward_workspace_bytes.restype = ctypes.c_size_t
        l.fa_backward_workspace_bytes.argtypes = [ctypes.c_int] * 3
        l.fa_combine.restype = ctypes.c_int
        l.fa_combine.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                 ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                 ctypes.c_void_p]
        l.fa_kat.restype = ctypes.c_int
        l.fa_kat.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                             ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
        l.fa_device_status.restype = ctypes.c_int
        l.fa_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
        l.fa_clear_device_status.restype = ctypes.c_int
        l.fa_error_string.restype = ctypes.c_char_p
        l.fa_error_string.argtypes = [ctypes.c_int]
        l.fa_last_cuda_error.restype = ctypes.c_char_p
        l.fa_version.restype = ctypes.c_int
        l.fa_combine_packed.restype = ctypes.c_int
        l.fa_combine_packed.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        l.fa_decode_kv_sharded.restype = ctypes.c_int
        l.fa_decode_kv_sharded.argtypes = [ctypes.POINTER(DecodeArgs), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        l.fa_decode_kv_sharded_gather_bytes.restype = ctypes.c_size_t
        l.fa_decode_kv_sharded_gather_bytes.argtypes = [ctypes.c_int] * 4
        l.fa_nccl_unique_id.restype = ctypes.c_int
        l.fa_nccl_unique_id.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        l.fa_nccl_comm_create.restype = ctypes.c_int
        l.fa_nccl_comm_create.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                          ctypes.c_int]
        l.fa_nccl_comm_destroy.restype = ctypes.c_int
        l.fa_nccl_comm_destroy.argtypes = [ctypes.c_void_p]
        l.fa_status_word_to_error.restype = ctypes.c_int
        l.fa_status_word_to_error.argtypes = [ctypes.c_int]
        l.fa_set_prefill_variant.restype = ctypes.c_int
        l.fa_set_prefill_variant.argtypes = [ctypes.c_int]
        _lib = l
    return _lib


def error_string(code: int) -> str:
    return lib().fa_error_string(code).decode()


def last_cuda_error() -> str:
    return lib().fa_last_cuda_error().decode()


def _ptr(x) -> int | None:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream_handle(stream) -> int | None:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


def prefill_raw(q, k, v, o, lse, batch_size, num_heads, seq_len, d_head, scale, causal,
                dtype="f16", q_scale=None, k_scale=None, v_scale=None, stream=None,
                host=False) -> int:
    """Calls fa_prefill (or fa_prefill_host) and returns its status code unchanged."""
    a = PrefillArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), batch_size, num_heads, seq_len,
                    d_head, scale, int(bool(causal)), DTYPES[dtype] if isinstance(dtype, str) else dtype,
                    _ptr(q_scale), _ptr(k_scale), _ptr(v_scale), _stream_handle(stream))
    fn = lib().fa_prefill_host if host else lib().fa_prefill
    return fn(ctypes.byref(a))


def prefill(q, k, v, o, lse, batch_size, num_heads, seq_len, d_head, scale, causal, **kw) -> None:
    """fa_prefill on device buffers; raises FaError on a non-zero status."""
    rc = prefill_raw(q, k, v, o, lse, batch_size, num_heads, seq_len, d_head, scale, causal, **kw)
    if rc != FA_OK:
        raise FaError(rc, "fa_prefill")


PREFILL_VARIANTS = {"auto": 0, "one_tile": 1, "tile_pair": 2, "cta_pair": 3}


def set_prefill_variant(variant: str) -> None:
    """fa_set_prefill_variant: which 16-bit prefill kernel runs ("auto" picks by problem size)."""
    rc = lib().fa_set_prefill_variant(PREFILL_VARIANTS[variant])
    if rc != FA_OK:
        raise FaError(rc, "fa_set_prefill_variant")


def decode_workspace_bytes(batch_size, num_heads, d_head, num_splits) -> int:
    return lib().fa_decode_workspace_bytes(batch_size, num_heads, d_head, num_splits)


def decode_default_splits(batch_size, num_heads, seq_len_kv) -> int:
    return lib().fa_decode_default_splits(batch_size, num_heads, seq_len_kv)


def decode_raw(q, k, v, o, lse, o_f32, batch_size, num_heads, seq_len_kv, d_head, scale,
               dtype="f16", num_splits=0, workspace=None, workspace_bytes=0, stream=None) -> int:
    a = DecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(o_f32), batch_size, num_heads,
                   seq_len_kv, d_head, scale, DTYPES[dtype] if isinstance(dtype, str) else dtype,
                   num_splits, _ptr(workspace), workspace_bytes, _stream_handle(stream))
    return lib().fa_decode(ctypes.byref(a))


DECODE_STATIC_SCRATCH_BYTES = 8 * 1024 * 1024 + 512 * 1024


def decode_static_raw(q, k, v, o, lse, o_f32, batch_size, num_heads, seq_len_kv, d_head, scale,
                      dtype="f16", num_splits=0, stream=None) -> int:
    """fa_decode_static: decode with the library's built-in scratch array instead of a
    caller workspace (for callers that may not allocate).  Returns the status code."""
    a = DecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(o_f32), batch_size, num_heads,
                   seq_len_kv, d_head, scale, DTYPES[dtype] if isinstance(dtype, str) else dtype,
                   num_splits, None, 0, _stream_handle(stream))
    return lib().fa_decode_static(ctypes.byref(a))


def decode(*args, **kw) -> None:
    rc = decode_raw(*args, **kw)
    if rc != FA_OK:
        raise FaError(rc, "fa_decode")


def decode_gqa_default_splits(batch_size, num_kv_heads, seq_len_kv) -> int:
    return lib().fa_decode_gqa_default_splits(batch_size, num_kv_heads, seq_len_kv)


def decode_gqa_raw(q, k, v, o, lse, batch_size, num_q_heads, num_kv_heads, seq_len_kv, d_head, scale,
                   dtype="f16", num_splits=0, kv_strides=(0, 0, 0), workspace=None, workspace_bytes=0,
                   stream=None, block_table=None, block_table_stride=0, page_size=0, num_pages=0,
                   kv_page_stride=0, seq_lens=None, q_scale=None, k_scale=None, v_scale=None,
                   num_q_tokens=0) -> int:
    """fa_decode_gqa; ``kv_strides`` = (batch, head, row) strides of the cache in elements
    ((0, 0, 0) = dense [B, Hkv, Skv, D]); ``block_table`` (int32, device) selects the paged
    layout; ``seq_lens`` (int32, device) gives per-sequence lengths.  Returns the status code."""
    a = DecodeGqaArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), batch_size, num_q_heads, num_kv_heads,
                      seq_len_kv, d_head, scale, DTYPES[dtype] if isinstance(dtype, str) else dtype,
                      num_splits, kv_strides[0], kv_strides[1], kv_strides[2], _ptr(block_table),
                      block_table_stride, page_size, num_pages, kv_page_stride, _ptr(seq_lens),
                      _ptr(q_scale), _ptr(k_scale), _ptr(v_scale), num_q_tokens,
                      _ptr(workspace), workspace_bytes, _stream_handle(stream))
    return lib().fa_decode_gqa(ctypes.byref(a))


def decode_gqa(*args, **kw) -> None:
    rc = decode_gqa_raw(*args, **kw)
    if rc != FA_OK:
        raise FaError(rc, "fa_decode_gqa")


def backward_workspace_bytes(batch_size, num_heads, seq_len) -> int:
    return lib().fa_backward_workspace_bytes(batch_size, num_heads, seq_len)


def backward_raw(q, k, v, o, d_o, lse, dq, dk, dv, batch_size, num_heads, seq_len, d_head, scale, causal,
                 dtype="f16", workspace=None, workspace_bytes=0, stream=None) -> int:
    """fa_backward on device buffers; returns the status code."""
    a = BackwardArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(d_o), _ptr(lse), _ptr(dq), _ptr(dk), _ptr(dv),
                     batch_size, num_heads, seq_len, d_head, scale, int(bool(causal)),
                     DTYPES[dtype] if isinstance(dtype, str) else dtype, _ptr(workspace), workspace_bytes,
                     _stream_handle(stream))
    return lib().fa_backward(ctypes.byref(a))


def backward(*args, **kw) -> None:
    rc = backward_raw(*args, **kw)
    if rc != FA_OK:
        raise FaError(rc, "fa_backward")


def combine(o_parts, lse_parts, n_parts, rows, d_head, o, lse, dtype="f16", stream=None) -> None:
    rc = lib().fa_combine(_ptr(o_parts), _ptr(lse_parts), n_parts, rows, d_head, _ptr(o), _ptr(lse),
                          DTYPES[dtype] if isinstance(dtype, str) else dtype, _stream_handle(stream))
    if rc != FA_OK:
        raise FaError(rc, "fa_combine")


def combine_packed(packed_parts, n_parts, rows, d_head, o, lse, dtype="f16", stream=None) -> None:
    """fa_combine_packed: LSE merge of [n_parts, rows, d_head + 1] fp32 partials (O then LSE per row)."""
    rc = lib().fa_combine_packed(_ptr(packed_parts), n_parts, rows, d_head, _ptr(o), _ptr(lse),
                                 DTYPES[dtype] if isinstance(dtype, str) else dtype, _stream_handle(stream))
    if rc != FA_OK:
        raise FaError(rc, "fa_combine_packed")


NCCL_UNIQUE_ID_BYTES = 128


def nccl_unique_id() -> bytes:
    """fa_nccl_unique_id: a fresh NCCL id (rank 0 creates it, every rank passes it to nccl_comm_create)."""
    buf = ctypes.create_string_buffer(NCCL_UNIQUE_ID_BYTES)
    rc = lib().fa_nccl_unique_id(buf, NCCL_UNIQUE_ID_BYTES)
    if rc != FA_OK:
        raise FaError(rc, "fa_nccl_unique_id")
    return buf.raw


def nccl_comm_create(n_ranks: int, unique_id: bytes, rank: int) -> int:
    """fa_nccl_comm_create: an ncclComm_t (as an integer handle) for the current device."""
    comm = ctypes.c_void_p()
    buf = ctypes.create_string_buffer(unique_id, NCCL_UNIQUE_ID_BYTES)
    rc = lib().fa_nccl_comm_create(ctypes.byref(comm), n_ranks, buf, NCCL_UNIQUE_ID_BYTES, rank)
    if rc != FA_OK:
        raise FaError(rc, "fa_nccl_comm_create")
    return comm.value


def nccl_comm_destroy(comm: int) -> None:
    rc = lib().fa_nccl_comm_destroy(comm)
    if rc != FA_OK:
        raise FaError(rc, "fa_nccl_comm_destroy")


def decode_kv_sharded_gather_bytes(batch_size, num_heads, d_head, n_ranks) -> int:
    return lib().fa_decode_kv_sharded_gather_bytes(batch_size, num_heads, d_head, n_ranks)


def decode_kv_sharded_raw(q, k, v, o, lse, batch_size, num_heads, local_kv, d_head, scale, comm, gather,
                          gather_bytes, dtype="f16", num_splits=0, workspace=None, workspace_bytes=0,
                          stream=None) -> int:
    """fa_decode_kv_sharded on this rank's key slice; returns the status code."""
    a = DecodeArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), None, batch_size, num_heads, local_kv,
                   d_head, scale, DTYPES[dtype] if isinstance(dtype, str) else dtype, num_splits,
                   _ptr(workspace), workspace_bytes, _stream_handle(stream))
    return lib().fa_decode_kv_sharded(ctypes.byref(a), comm, _ptr(gather), gather_bytes)


def kat(dtype: str, d_head: int, q, k, v, p_scale: float):
    """Tensor-core known-answer test.  q,k,v: numpy uint16 arrays [128,d_head] holding
    fp16/bf16 bit patterns.  Returns (S [128,128], O [128,d_head]) float32."""
    import numpy as np
    s = np.zeros((128, 128), np.float32)
    o = np.zeros((128, d_head), np.float32)
    rc = lib().fa_kat(DTYPES[dtype], d_head, q.ctypes.data, k.ctypes.data, v.ctypes.data,
                      p_scale, s.ctypes.data, o.ctypes.data)
    if rc != FA_OK:
        raise FaError(rc, "fa_kat")
    return s, o


def device_status() -> int:
    """Status word of the current device (0 = clean).  Synchronises."""
    w = ctypes.c_int(0)
    rc = lib().fa_device_status(ctypes.byref(w))
    if rc not in (FA_OK, FA_ERR_DEVICE_TIMEOUT):
        raise FaError(rc, "fa_device_status")
    return w.value


def clear_device_status() -> None:
    rc = lib().fa_clear_device_status()
    if rc != FA_OK:
        raise FaError(rc, "fa_clear_device_status")
