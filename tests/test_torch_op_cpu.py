"""The PyTorch operators register and infer shapes without a GPU."""
import torch


def test_ops_registered_and_fake_shapes(fa):
    import __graft_entry__ as ge
    ge.load_module("torch_op")
    assert all(hasattr(torch.ops.fa_b200, n) for n in ("prefill", "decode", "decode_gqa", "prefill_backward"))
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        q = torch.empty((2, 3, 40, 64), dtype=torch.float16)
        o, lse = torch.ops.fa_b200.prefill(q, q, q, 0.125, True)
        assert o.shape == q.shape and o.dtype == torch.float16
        assert lse.shape == (2, 3, 40) and lse.dtype == torch.float32
        q1 = torch.empty((2, 3, 1, 128), dtype=torch.bfloat16)
        kv = torch.empty((2, 3, 77, 128), dtype=torch.bfloat16)
        o1, l1 = torch.ops.fa_b200.decode(q1, kv, kv, 0.1, 0)
        assert o1.shape == q1.shape and l1.shape == (2, 3, 1)


def test_cpu_tensors_are_rejected(fa):
    import __graft_entry__ as ge
    import pytest
    op = ge.load_module("torch_op")
    q = torch.zeros((1, 1, 8, 64), dtype=torch.float16)
    with pytest.raises(RuntimeError):
        op.prefill(q, q, q, 0.125, False)
    with pytest.raises(NotImplementedError):
        op.sdpa(q, q, q, dropout_p=0.1)
