"""Partitioning over ranks, with two gloo ranks on the CPU standing in for two GPUs: every rank
computes its shard (here with the CPU oracle in place of the CUDA kernels), outputs are gathered, and
the result must equal the unsharded computation bit for bit - the units are independent."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_split_range_covers_everything_once():
    from x17ai_b200.sharding import attn_shard, row_shard, split_range
    for n, parts, mult in [(16384, 8, 128), (1000, 3, 128), (5, 8, 1), (0, 2, 1), (131072, 4, 128)]:
        seen = []
        for i in range(parts):
            b, e = split_range(n, parts, i, mult)
            assert 0 <= b <= e <= n and (b % mult == 0 or b == n)
            seen += list(range(b, e))
        assert seen == list(range(n))
    assert row_shard(16384, 8, 3) == (6144, 8192)
    # configs[1]: 8 sequences on 8 GPUs -> one sequence each, all heads local
    assert [attn_shard(8, 32, 8, r) for r in range(8)][5].__dict__ == dict(seq_begin=5, seq_end=6, head_begin=0, head_end=32)
    # configs[4]: 4 sequences on 8 GPUs -> two GPUs per sequence, 16 heads each
    s = attn_shard(4, 32, 8, 5)
    assert (s.seq_begin, s.seq_end, s.head_begin, s.head_end) == (2, 3, 16, 32)
    with pytest.raises(ValueError):
        attn_shard(3, 32, 8, 0)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import attn as o_attn, formats, gemm as o_gemm
        from x17ai_b200 import sharding
        rng = np.random.default_rng(0)          # every rank builds the same inputs
        # ---- GEMM rows: Q projection of 300 token rows, 128-row tiles ----
        x = formats.quantize_fixedi8(rng.standard_normal((300, 128)))
        w = formats.quantize_fixedi8(rng.standard_normal((128, 128)))
        full = o_gemm.attn_q_fwd(x, w)
        b, e = sharding.row_shard(300, world, rank)
        local = torch.from_numpy(o_gemm.attn_q_fwd(x[b:e], w)) if e > b else torch.zeros((0, 128), dtype=torch.int8)
        got = sharding.gather_rows(local, 300, world)
        ok1 = np.array_equal(got.numpy(), full)
        # ---- attention: one sequence, heads split over the two ranks ----
        B, H, D, S, W = 1, 4, 32, 64, 16
        qq = formats.quantize_fixedi8(rng.standard_normal((B, S, H * D)))
        kv = formats.quantize_fixedi8(rng.standard_normal((B, S, 2 * H * D)))
        sk = formats.quantize_fixedi8(rng.standard_normal((H, D)))
        sv = formats.quantize_fixedi8(rng.standard_normal((H, D)))
        temp = np.ones(H, np.float32)
        ref, _ = o_attn.attn_fwd_i8(qq[0], kv[0], sk, sv, temp, W, H, D)
        sh = sharding.attn_shard(B, H, world, rank)
        hs = slice(sh.head_begin, sh.head_end)
        nh = sh.head_end - sh.head_begin
        o, _ = o_attn.attn_fwd_i8(qq[0][:, sh.head_begin * D:sh.head_end * D], kv[0][:, 2 * sh.head_begin * D:2 * sh.head_end * D],
                                  sk[hs], sv[hs], temp[hs], W, nh, D)
        got = sharding.gather_attn(torch.from_numpy(o)[None], B, H, D, world)
        ok2 = np.array_equal(got[0].numpy(), ref)
        # ---- attention: three sequences over two ranks (shards of two and of one sequence) ----
        B3 = 3
        q3 = formats.quantize_fixedi8(rng.standard_normal((B3, S, H * D)))
        kv3 = formats.quantize_fixedi8(rng.standard_normal((B3, S, 2 * H * D)))
        ref3 = np.stack([o_attn.attn_fwd_i8(q3[b], kv3[b], sk, sv, temp, W, H, D)[0] for b in range(B3)])
        sh3 = sharding.attn_shard(B3, H, world, rank)
        loc3 = np.stack([o_attn.attn_fwd_i8(q3[b], kv3[b], sk, sv, temp, W, H, D)[0] for b in range(sh3.seq_begin, sh3.seq_end)])
        got3 = sharding.gather_attn(torch.from_numpy(loc3), B3, H, D, world)
        ok2 = ok2 and np.array_equal(got3.numpy(), ref3)
        q.put((rank, ok1, ok2))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True, True), (1, True, True)]
