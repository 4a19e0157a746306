"""The sharded attention on real GPUs: every rank launches the CUDA kernel on its (sequence, head-block) shard of one
fixed batch (x17ai_b200.sharding.attn_shard; the reference kernel addresses a head group the same way, by column
offset with explicit row strides, cuda/attn_fwd_i8.cuh:378-384) and the assembled or gathered result equals the
single launch over the whole batch byte for byte: the units are independent."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


def _inputs(B, S, H, D, device, seed=5):
    g = torch.Generator(device=device).manual_seed(seed)
    codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=g, device=device) * 8.0), -127, 127).to(torch.int8)
    q, kv, sk, sv = codes(B, S, H * D), codes(B, S, 2 * H * D), codes(H, D), codes(H, D)
    temp = (0.5 + torch.rand(H, generator=g, device=device)).float()
    return q, kv, sk, sv, temp


def _shard_launch(stream, sh, q, kv, sk, sv, temp, D, W):
    """The launch of one rank: its sequences, its head block, outputs of its own."""
    from x17ai_b200 import kernels as K
    H = sk.shape[0]
    nb, nh = sh.seq_end - sh.seq_begin, sh.head_end - sh.head_begin
    S = q.shape[1]
    out = torch.zeros(nb, S, nh * D, dtype=torch.int8, device=q.device)
    l = torch.zeros(nb, nh, S, dtype=torch.float32, device=q.device)
    torch.cuda.synchronize(q.device)
    kern = K.AttnKernel(K.AttnKernelConfig(nh, D, H * D, 2 * H * D, nh * D))
    kern.launch_head_block(stream, q[sh.seq_begin:sh.seq_end], kv[sh.seq_begin:sh.seq_end], sk, sv, temp, out, l, W,
                           sh.head_begin)
    stream.synchronize()
    return out, l


@pytest.mark.parametrize("B,H,D,S,W,world", [(2, 4, 128, 384, 128, 2), (2, 4, 128, 384, 128, 8), (3, 4, 64, 256, 0, 2),
                                             (1, 8, 32, 256, 64, 4)])
def test_shard_launches_reproduce_the_whole_launch(stream, B, H, D, S, W, world):
    from x17ai_b200 import kernels as K, sharding
    dev = torch.device("cuda", 0)
    q, kv, sk, sv, temp = _inputs(B, S, H, D, dev)
    want = torch.zeros(B, S, H * D, dtype=torch.int8, device=dev)
    want_l = torch.zeros(B, H, S, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D)).launch(stream, q, kv, sk, sv, temp, want, want_l, W)
    stream.synchronize()
    got = torch.zeros_like(want)
    got_l = torch.zeros_like(want_l)
    for rank in range(world):
        sh = sharding.attn_shard(B, H, world, rank)
        out, l = _shard_launch(stream, sh, q, kv, sk, sv, temp, D, W)
        got[sh.seq_begin:sh.seq_end, :, sh.head_begin * D:sh.head_end * D] = out
        got_l[sh.seq_begin:sh.seq_end, sh.head_begin:sh.head_end] = l
    assert torch.equal(got, want)
    assert torch.equal(got_l, want_l)


def test_head_block_arguments(stream):
    from x17ai_b200 import X17Error, kernels as K
    dev = torch.device("cuda", 0)
    q, kv, sk, sv, temp = _inputs(1, 128, 4, 64, dev)
    kern = K.AttnKernel(K.AttnKernelConfig(2, 64, 4 * 64, 8 * 64, 2 * 64))
    out = torch.zeros(1, 128, 2 * 64, dtype=torch.int8, device=dev)
    with pytest.raises(X17Error, match="lies outside the 4 heads"):
        kern.launch_head_block(stream, q, kv, sk, sv, temp, out, None, 0, 3)


def _rank(rank, world, port, B, H, D, S, W, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from x17ai_b200 import device, kernels as K, sharding
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        with device.CudaStream(rank) as stream:
            q, kv, sk, sv, temp = _inputs(B, S, H, D, dev)       # the same seed on every rank: the same batch
            sh = sharding.attn_shard(B, H, world, rank)
            out, _ = _shard_launch(stream, sh, q, kv, sk, sv, temp, D, W)
            full = sharding.gather_attn(out, B, H, D, world)
            torch.cuda.synchronize()
            want = torch.zeros(B, S, H * D, dtype=torch.int8, device=dev)
            K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D)).launch(stream, q, kv, sk, sv, temp, want, None, W)
            stream.synchronize()
            ok = bool(torch.equal(full, want)) and stream.read_status() == [0, 0, 0, 0]
        result.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H", [(2, 4), (1, 4), (3, 4)])
def test_two_gpus_gather_the_single_gpu_result(B, H):
    """Two ranks, one GPU each, NCCL all_gather of the shards (whole sequences; head blocks of one sequence; shards
    of different sizes): every rank ends with the bytes of the single launch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29600 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_rank, args=(r, 2, port, B, H, 128, 384, 128, result)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(result.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]


def _rank_peer(rank, world, port, B, H, D, S, W, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    from x17ai_b200 import device, kernels as K, sharding
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        with device.CudaStream(rank) as stream:
            q, kv, sk, sv, temp = _inputs(B, S, H, D, dev)
            peers = sharding.PeerOutputs(B, H, D, S, world, rank, dev)
            peers.buf.zero_()
            torch.cuda.synchronize()
            dist.barrier()                      # nobody's zero-fill may land on a peer's stores
            sh = peers.shards[rank]
            nh = sh.head_end - sh.head_begin
            kern = K.AttnKernel(K.AttnKernelConfig(nh, D, H * D, 2 * H * D, peers.cols))
            kern.launch_head_block(stream, q[sh.seq_begin:sh.seq_end], kv[sh.seq_begin:sh.seq_end], sk, sv, temp, peers.out,
                                   None, W, sh.head_begin, peer_outs=peers.peer_outs)
            with torch.cuda.stream(torch.cuda.ExternalStream(stream.handle)):
                peers.barrier()                 # every rank's launch has completed
            stream.synchronize()
            full = peers.assemble()
            want = torch.zeros(B, S, H * D, dtype=torch.int8, device=dev)
            K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D)).launch(stream, q, kv, sk, sv, temp, want, None, W)
            stream.synchronize()
            torch.cuda.synchronize()
            ok = bool(torch.equal(full, want)) and stream.read_status() == [0, 0, 0, 0]
            dist.barrier()                      # nobody frees a buffer that a peer may still read or write
        result.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H", [(2, 4), (1, 4), (3, 4)])
def test_two_gpus_store_their_outputs_on_each_other(B, H):
    """Two ranks, one GPU each: the kernel's epilogue stores every shard into both GPUs' buffers (peer stores over
    NVLink, no gather pass); after a barrier every rank holds the bytes of the single launch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29700 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_rank_peer, args=(r, 2, port, B, H, 128, 384, 128, result)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(result.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]
