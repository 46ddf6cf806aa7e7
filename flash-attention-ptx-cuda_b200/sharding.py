"""Multi-GPU partitioning of the attention forward path (one process per GPU).

Two ways the path shards, and only these two:

* by (batch x head): every head is independent, so prefill and batched decode
  split the flattened batch*head axis into contiguous ranges, one per rank, and
  need NO collective (``head_shard``);
* by KV sequence, for one long cache: each rank holds a contiguous slice of the
  keys, runs split-KV decode on it and contributes a normalised fp32 partial O
  with its LSE; ONE all-gather of ``[B*H, D+1]`` floats per rank brings all
  partials into local memory, where the merge kernel reads them in place
  (``kv_shard``, ``ShardedDecode`` over ``fa_decode_kv_sharded``; ``gather_partials``
  is the same exchange through ``torch.distributed`` for host-side tests).

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
    """KV-sequence-sharded decode on this rank's GPU through ``fa_decode_kv_sharded``: split-KV
    decode on the local key slice, whose merge writes the rank's packed ``[BH, D+1]`` block into
    the all-gather's receive buffer; one in-place ``ncclAllGather``; ``fa_combine_packed`` on the
    gathered blocks.  Four launches on one stream, no copies in between.

    The library talks to NCCL itself (its own communicator, one rank per GPU); the id travels
    over the existing ``torch.distributed`` group, which is used for nothing else.  Buffers are
    allocated once and reused.  A rank whose slice is empty (``local_kv == 0``) contributes
    weight zero.  Call ``close()`` (or use as a context manager) to destroy the communicator."""

    def __init__(self, fa, batch_size, num_heads, d_head, local_kv, dtype="f16", num_splits=0, group=None):
        import torch
        import torch.distributed as dist
        self.fa, self.group = fa, group
        self.b, self.h, self.d, self.dtype = batch_size, num_heads, d_head, dtype
        self.bh = batch_size * num_heads
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.splits = num_splits or fa.decode_default_splits(batch_size, num_heads, max(local_kv, 1))
        self.ws_bytes = fa.decode_workspace_bytes(batch_size, num_heads, d_head, self.splits)
        self.ws = torch.empty(self.ws_bytes, device=dev, dtype=torch.uint8)
        self.gather_bytes = fa.decode_kv_sharded_gather_bytes(batch_size, num_heads, d_head, self.world)
        self.gathered = torch.empty((self.world, self.bh, d_head + 1), device=dev, dtype=torch.float32)
        ids = [fa.nccl_unique_id() if self.rank == 0 else None]
        dist.broadcast_object_list(ids, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.comm = fa.nccl_comm_create(self.world, ids[0], self.rank)

    def __call__(self, q, k_local, v_local, o, lse, scale, stream=None):
        """q [BH, D]; k_local, v_local [BH, local_kv, D]; o [BH, D] 16-bit, lse [BH] fp32 (outputs,
        identical on every rank).  Everything is enqueued on ``stream`` (default: the current
        torch stream)."""
        import torch
        stream = stream or torch.cuda.current_stream()
        local_kv = k_local.shape[1]
        rc = self.fa.decode_kv_sharded_raw(q, k_local, v_local, o, lse, self.b, self.h, local_kv, self.d,
                                           float(scale), self.comm, self.gathered, self.gather_bytes,
                                           dtype=self.dtype, num_splits=self.splits if local_kv else 0,
                                           workspace=self.ws, workspace_bytes=self.ws_bytes, stream=stream)
        if rc != self.fa.FA_OK:
            raise self.fa.FaError(rc, "fa_decode_kv_sharded")

    LAUNCHES_PER_STEP = 4          # split partials, their merge, the all-gather, the cross-rank merge

    def close(self):
        if getattr(self, "comm", None):
            import torch
            torch.cuda.synchronize()
            self.fa.nccl_comm_destroy(self.comm)
            self.comm = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
