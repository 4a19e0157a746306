"""Partitioning of the hot path over the GPUs of one box, one process per GPU.

The reference is single-GPU (CudaDevice::new(0), src/main.rs:38); its kernels already address a
head group by column offset with explicit row strides (cuda/attn_fwd_i8.cuh:378-384) and GEMM rows
are independent, so the units of work are independent:

  attention / decode : (sequence, head) units - sequences are split first, so that q and kv of a
                       sequence stay on one GPU; if there are fewer sequences than ranks, the heads
                       of a sequence are split into contiguous column blocks
  GEMM / RMSNorm     : contiguous token-row blocks, rounded to the M tile; weights replicated

No data moves between ranks inside the path. `gather_rows` / `gather_heads` collect outputs on
every rank (torch.distributed all_gather: NCCL on GPUs, gloo in the CPU tests) for a consumer that
wants the whole tensor.
"""
from dataclasses import dataclass


def split_range(n: int, parts: int, index: int, multiple: int = 1):
    """[begin, end) of block `index` when `n` items are cut into `parts` contiguous blocks whose sizes
    are multiples of `multiple` (the last non-empty block takes the remainder)."""
    if parts <= 0 or not (0 <= index < parts):
        raise ValueError(f"bad partition {index} of {parts}")
    chunks = (n + multiple - 1) // multiple
    base, extra = divmod(chunks, parts)
    b = index * base + min(index, extra)
    e = b + base + (1 if index < extra else 0)
    return min(b * multiple, n), min(e * multiple, n)


@dataclass(frozen=True)
class AttnShard:
    seq_begin: int    # sequences [seq_begin, seq_end) of the batch
    seq_end: int
    head_begin: int   # heads [head_begin, head_end) of those sequences
    head_end: int


def attn_shard(batch: int, n_heads: int, world: int, rank: int, heads_multiple: int = 1) -> AttnShard:
    """Sequences first; with fewer sequences than ranks, `world // batch` ranks share one sequence and
    split its heads (world must then be a multiple of batch)."""
    if world <= batch:
        b, e = split_range(batch, world, rank)
        return AttnShard(b, e, 0, n_heads)
    if world % batch != 0:
        raise ValueError(f"world size {world} must be a multiple of the batch {batch} to split heads")
    per_seq = world // batch
    seq = rank // per_seq
    hb, he = split_range(n_heads, per_seq, rank % per_seq, heads_multiple)
    return AttnShard(seq, seq + 1, hb, he)


def row_shard(rows: int, world: int, rank: int, tile: int = 128):
    """Token rows of a GEMM / RMSNorm for this rank, in whole M tiles."""
    return split_range(rows, world, rank, tile)


def gather_rows(local, rows_total: int, world: int, tile: int = 128, group=None):
    """all_gather of row blocks made by `row_shard` into one [rows_total, ...] tensor on every rank."""
    import torch
    import torch.distributed as dist
    sizes = [row_shard(rows_total, world, r, tile) for r in range(world)]
    pad = max(e - b for b, e in sizes)
    buf = torch.zeros((pad,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    buf[: local.shape[0]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([p[: e - b] for p, (b, e) in zip(parts, sizes)], dim=0)


def gather_attn(local, batch: int, n_heads: int, head_dim: int, world: int, group=None):
    """all_gather of attention outputs [seqs, S, heads*D] made by `attn_shard` into [batch, S, H*D].
    Shards of different sizes (a batch or a head count that the ranks do not divide) are padded to the
    largest one for the collective, as `gather_rows` does, so every rank sends the same count."""
    import torch
    import torch.distributed as dist
    shards = [attn_shard(batch, n_heads, world, r) for r in range(world)]
    s_len = local.shape[1]
    seqs = max(sh.seq_end - sh.seq_begin for sh in shards)
    cols = max(sh.head_end - sh.head_begin for sh in shards) * head_dim
    if local.shape[0] > seqs or local.shape[2] > cols:
        raise ValueError(f"local shard {tuple(local.shape)} is larger than any shard of this partition")
    buf = local.contiguous()
    if tuple(local.shape) != (seqs, s_len, cols):
        buf = torch.zeros((seqs, s_len, cols), dtype=local.dtype, device=local.device)
        buf[: local.shape[0], :, : local.shape[2]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    out = torch.empty((batch, s_len, n_heads * head_dim), dtype=local.dtype, device=local.device)
    for p, sh in zip(parts, shards):
        nb, nc = sh.seq_end - sh.seq_begin, (sh.head_end - sh.head_begin) * head_dim
        out[sh.seq_begin:sh.seq_end, :, sh.head_begin * head_dim:sh.head_end * head_dim] = p[:nb, :, :nc]
    return out
