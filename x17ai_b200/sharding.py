"""Partitioning of the hot path over the GPUs of one box, one process per GPU.

The reference is single-GPU (CudaDevice::new(0), src/main.rs:38); its kernels already address a
head group by column offset with explicit row strides (cuda/attn_fwd_i8.cuh:378-384) and GEMM rows
are independent, so the units of work are independent:

  attention / decode : (sequence, head) units - sequences are split first, so that q and kv of a
                       sequence stay on one GPU; if there are fewer sequences than ranks, the heads
                       of a sequence are split into contiguous column blocks
  GEMM / RMSNorm     : contiguous token-row blocks, rounded to the M tile; weights replicated

No data moves between ranks inside the path. `gather_rows` / `gather_attn` collect outputs on
every rank (torch.distributed all_gather: NCCL on GPUs, gloo in the CPU tests) for a consumer that
wants the whole tensor; `PeerOutputs` has the attention kernel's epilogue store every shard into
every GPU's buffer instead (peer stores over NVLink), so that no gather pass follows.
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


class PeerOutputs:
    """Every rank's attention output on every GPU without a gather pass: one buffer per GPU with a slot per rank
    ([world, seqs, S, cols], slots padded to the largest shard), allocated as symmetric memory so that each process
    holds the peers' buffers mapped at addresses of its own. A rank launches its shard with `out` = its slot of its
    own buffer and `peer_outs` = the same slot of every peer's (AttnKernel.launch_head_block): the kernel's epilogue
    writes each 16 bytes to all of them. `barrier()` (a device-side barrier between the ranks on the current torch
    stream) orders every rank's launch before anyone reads; `assemble()` is the [batch, S, H * D] view of it."""

    def __init__(self, batch: int, n_heads: int, head_dim: int, seq_len: int, world: int, rank: int, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        if world > 8:
            raise ValueError("peer outputs are for the GPUs of one box (at most 8)")
        self.batch, self.n_heads, self.head_dim, self.seq_len, self.world, self.rank = batch, n_heads, head_dim, seq_len, world, rank
        self.shards = [attn_shard(batch, n_heads, world, r) for r in range(world)]
        self.seqs = max(sh.seq_end - sh.seq_begin for sh in self.shards)
        self.cols = max(sh.head_end - sh.head_begin for sh in self.shards) * head_dim
        group = group if group is not None else dist.group.WORLD
        self.buf = symm.empty((world, self.seqs, seq_len, self.cols), dtype=torch.int8, device=device)
        self.handle = symm.rendezvous(self.buf, group)
        slot_bytes = self.seqs * seq_len * self.cols
        sh = self.shards[rank]
        # this rank's slot: in its own buffer (the kernel's `out`, row stride `cols`) and in every peer's
        self.out = self.buf[rank, : sh.seq_end - sh.seq_begin]
        self.peer_outs = [int(ptr) + rank * slot_bytes for r, ptr in enumerate(self.handle.buffer_ptrs) if r != rank]

    def barrier(self, timeout_ms: int = 10000):
        """Device-side barrier between the ranks on the current torch stream; it gives up after `timeout_ms`
        (a rank that never arrives must not leave the others' GPUs waiting)."""
        self.handle.barrier(0, int(timeout_ms))

    def assemble(self):
        import torch
        out = torch.empty((self.batch, self.seq_len, self.n_heads * self.head_dim), dtype=torch.int8, device=self.buf.device)
        for r, sh in enumerate(self.shards):
            nb, nc = sh.seq_end - sh.seq_begin, (sh.head_end - sh.head_begin) * self.head_dim
            out[sh.seq_begin:sh.seq_end, :, sh.head_begin * self.head_dim:sh.head_end * self.head_dim] = self.buf[r, :nb, :, :nc]
        return out
