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


def test_host_side_validation_of_the_added_entry_points(fa):
    lib = fa.lib()
    assert lib.fa_decode_gqa(None) == fa.FA_ERR_INVALID_ARGUMENT
    assert lib.fa_backward(None) == fa.FA_ERR_INVALID_ARGUMENT
    g = fa.DecodeGqaArgs(q=16, k=16, v=16, o=16, batch_size=1, num_q_heads=6, num_kv_heads=4, seq_len_kv=128,
                         d_head=64, scale=0.125, dtype=0)
    assert lib.fa_decode_gqa(ctypes.byref(g)) == fa.FA_ERR_INVALID_ARGUMENT   # 6 query heads over 4 KV heads
    g.num_q_heads = 8
    g.d_head = 96
    assert lib.fa_decode_gqa(ctypes.byref(g)) == fa.FA_ERR_UNSUPPORTED
    g.d_head = 64
    g.kv_batch_stride, g.kv_head_stride, g.kv_row_stride = 8192, 4100, 64    # head stride not a multiple of 8
    assert lib.fa_decode_gqa(ctypes.byref(g)) == fa.FA_ERR_MISALIGNED
    g.kv_head_stride = 4096
    g.block_table, g.page_size, g.num_pages, g.block_table_stride, g.kv_page_stride = 16, 24, 4, 8, 4096
    assert lib.fa_decode_gqa(ctypes.byref(g)) == fa.FA_ERR_INVALID_ARGUMENT   # page size not a power of two
    b = fa.BackwardArgs(q=16, k=16, v=16, o=16, d_o=16, lse=16, dq=16, dk=16, dv=16, batch_size=1, num_heads=1,
                        seq_len=128, d_head=64, scale=0.125, causal=1, dtype=2)
    assert lib.fa_backward(ctypes.byref(b)) == fa.FA_ERR_UNSUPPORTED          # e4m3 has no backward
    b.dtype = 0
    b.workspace, b.workspace_bytes = 16, 8
    assert lib.fa_backward(ctypes.byref(b)) == fa.FA_ERR_WORKSPACE
    assert fa.backward_workspace_bytes(2, 3, 100) == 2 * 3 * 100 * 4
