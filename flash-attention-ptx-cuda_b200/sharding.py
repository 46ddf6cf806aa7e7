"""Multi-GPU partitioning of the attention forward path (one process per GPU).

Two ways the path shards, and only these two:

* by (batch x head): every head is independent, so prefill and batched decode
  split the flattened batch*head axis into contiguous ranges, one per rank, and
  need NO collective (``head_shard``);
* by KV sequence, for one long cache: each rank holds a contiguous slice of the
  keys, runs split-KV decode on it and contributes a normalised fp32 partial O
  with its LSE; ONE all-gather of ``[B*H, D+1]`` floats per rank brings all
  partials into local memory, where ``fa_combine`` merges them
  (``kv_shard``, ``gather_partials``, ``sharded_decode``).

The reference is single-GPU (no NCCL/MPI call site exists in it); the exchange
step is defined by the LSE-merge identity its attention satisfies.
"""
from __future__ import annotations


def _split(total: int, rank: int, world: int):
    base, rem = divmod(total, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def head_shard(n_bh: int, rank: int, world: int):
    """(first head, number of heads) of `rank`: contiguous, remainder to the low ranks."""
    return _split(n_bh, rank, world)


def kv_shard(seq_len_kv: int, rank: int, world: int):
    """(first key, number of keys) of `rank`."""
    return _split(seq_len_kv, rank, world)


def gather_partials(o_f32, lse, group=None):
    """All-gathers each rank's partial.  o_f32 [BH, D] fp32, lse [BH] fp32 (torch tensors on
    the backend's device: CUDA for nccl, CPU for gloo).  Returns
    (o_parts [world, BH, D], lse_parts [world, BH]) - the layout fa_combine reads.
    O and LSE travel in one message: [BH, D+1]."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    bh, d = o_f32.shape
    packed = torch.cat([o_f32, lse.reshape(bh, 1)], dim=1).contiguous()
    flat = torch.empty((world * bh, d + 1), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed, group=group)     # rank r lands in rows [r*bh, (r+1)*bh)
    out = flat.view(world, bh, d + 1)
    return out[:, :, :d].contiguous(), out[:, :, d].contiguous()


class ShardedDecode:
    """KV-sequence-sharded decode on this rank's GPU: fa_decode on the local key slice,
    one all-gather, fa_combine.  Buffers are allocated once and reused."""

    def __init__(self, fa, batch_size, num_heads, d_head, local_kv, dtype="f16", num_splits=0, group=None):
        import torch
        import torch.distributed as dist
        self.fa, self.group = fa, group
        self.b, self.h, self.d, self.dtype = batch_size, num_heads, d_head, dtype
        self.bh = batch_size * num_heads
        self.world = dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.splits = num_splits or fa.decode_default_splits(batch_size, num_heads, max(local_kv, 1))
        self.ws_bytes = fa.decode_workspace_bytes(batch_size, num_heads, d_head, self.splits)
        self.ws = torch.empty(self.ws_bytes, device=dev, dtype=torch.uint8)
        self.packed = torch.empty((self.bh, d_head + 1), device=dev, dtype=torch.float32)
        self.o_local = torch.empty((self.bh, d_head), device=dev, dtype=torch.float32)
        self.lse_local = torch.empty((self.bh,), device=dev, dtype=torch.float32)
        self.gathered_flat = torch.empty((self.world * self.bh, d_head + 1), device=dev, dtype=torch.float32)
        self.gathered = self.gathered_flat.view(self.world, self.bh, d_head + 1)
        self.o_parts = torch.empty((self.world, self.bh, d_head), device=dev, dtype=torch.float32)
        self.lse_parts = torch.empty((self.world, self.bh), device=dev, dtype=torch.float32)

    def __call__(self, q, k_local, v_local, o, lse, scale, stream=None):
        """q [BH, D]; k_local, v_local [BH, local_kv, D]; o [BH, D] 16-bit, lse [BH] fp32 (outputs,
        identical on every rank).  Enqueues on the current torch stream."""
        import torch
        import torch.distributed as dist
        stream = stream or torch.cuda.current_stream()
        local_kv = k_local.shape[1]
        self.fa.decode(q, k_local, v_local, None, self.lse_local, self.o_local, self.b, self.h, local_kv,
                       self.d, float(scale), dtype=self.dtype, num_splits=self.splits, workspace=self.ws,
                       workspace_bytes=self.ws_bytes, stream=stream)
        self.packed[:, :self.d].copy_(self.o_local)
        self.packed[:, self.d].copy_(self.lse_local)
        dist.all_gather_into_tensor(self.gathered_flat, self.packed, group=self.group)
        self.o_parts.copy_(self.gathered[:, :, :self.d])
        self.lse_parts.copy_(self.gathered[:, :, self.d])
        self.fa.combine(self.o_parts, self.lse_parts, self.world, self.bh, self.d, o, lse,
                        dtype=self.dtype, stream=stream)
