"""CPU-only: the C-ABI library loads, exports every declared symbol, and rejects
bad arguments on the host before touching a device."""
import ctypes
import os
import re


def test_library_exports_every_declared_symbol(fa):
    lib = fa.lib()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "fa_b200.h")).read()
    declared = set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", header))
    declared -= {"fa_prefill_args", "fa_decode_args"}
    assert declared == set(fa.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    # the reference's C++ entry point, by its mangled name
    assert hasattr(lib, "_ZN11transformer22launch_flash_attentionERKNS_20FlashAttentionParamsE")
    assert lib.fa_version() >= 100


def test_error_strings(fa):
    for code in range(0, -8, -1):
        assert fa.error_string(code) != "unknown error"
    assert fa.error_string(-99) == "unknown error"


def test_host_side_validation_needs_no_device(fa):
    lib = fa.lib()
    assert lib.fa_prefill(None) == fa.FA_ERR_INVALID_ARGUMENT
    a = fa.PrefillArgs()
    assert lib.fa_prefill(ctypes.byref(a)) == fa.FA_ERR_INVALID_ARGUMENT
    a = fa.PrefillArgs(q=16, k=16, v=16, o=16, batch_size=1, num_heads=1, seq_len=8, d_head=64,
                       scale=0.0, causal=1, dtype=0)
    assert lib.fa_prefill(ctypes.byref(a)) == fa.FA_ERR_INVALID_ARGUMENT   # scale must be > 0
    a.scale = 0.125
    a.d_head = 96
    assert lib.fa_prefill(ctypes.byref(a)) == fa.FA_ERR_UNSUPPORTED
    a.d_head = 64
    a.dtype = 7
    assert lib.fa_prefill(ctypes.byref(a)) == fa.FA_ERR_UNSUPPORTED
    a.dtype = 0
    a.q = 8                                                               # not 16-byte aligned
    assert lib.fa_prefill(ctypes.byref(a)) == fa.FA_ERR_MISALIGNED
    assert lib.fa_decode(None) == fa.FA_ERR_INVALID_ARGUMENT
    assert fa.decode_workspace_bytes(32, 32, 128, 16) == 32 * 32 * 16 * 129 * 4
    assert fa.decode_workspace_bytes(0, 1, 128, 1) == 0
