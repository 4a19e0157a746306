"""The decode entry point that allocates nothing (x17ai_b200_attn_decode_i8_noalloc).

It serves hosts that cannot allocate device memory at call time (memory carved up at start-up,
a memory pool that is exhausted or switched off, a no-allocation policy after warm-up): the
split-KV partials live in a 4 MiB array inside the library image.  Checked here through the C
ABI: its output equals the allocating entry point's bit for bit (same kernels, same order of
operations) on two calls in a row that reuse the scratch, and the oracle's within the decode bar;
the driver reports the same free device memory before and after the calls; a request beyond the
built-in scratch is refused with a clear message; where a second GPU is visible the per-device
set-up is exercised there too.  This file sorts last so that a failure here cannot
hide another test's result in a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

from conftest import code_hist
from oracle import attn as o_attn, formats

pytestmark = pytest.mark.gpu


def _case(rng, B, H, D, T):
    q = formats.quantize_fixedi8(rng.standard_normal((B, H * D)))
    kv = formats.quantize_fixedi8(rng.standard_normal((B, T, H * 2 * D)))
    sk = formats.quantize_fixedi8(rng.standard_normal((H, D)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    return (q, kv, sk, sv, temp), [torch.from_numpy(a).cuda() for a in (q, kv, sk, sv, temp)]


def _compare(stream, device):
    from x17ai_b200 import kernels as K
    B, H, D = 2, 4, 128
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    rng = np.random.default_rng(2024)
    # two calls in a row with different shapes and split counts: the second reuses (and must fully
    # overwrite) the slots the first one left behind
    for T, kv_len, W, splits in [(2048, 2048, 0, 8), (1024, 700, 256, 3)]:
        host, dev = _case(rng, B, H, D, T)
        q, kv, sk, sv, temp = [t.to(device) for t in dev]
        ref = torch.zeros((B, H * D), dtype=torch.int8, device=device)
        ref_l = torch.zeros((B, H), dtype=torch.float32, device=device)
        got = torch.full((B, H * D), 77, dtype=torch.int8, device=device)
        got_l = torch.zeros((B, H), dtype=torch.float32, device=device)
        torch.cuda.synchronize(device)
        kern.decode(stream, q, kv, kv_len, sk, sv, temp, ref, ref_l, window_size=W, n_splits=splits)
        stream.synchronize()
        free_before = torch.cuda.mem_get_info(device)[0]
        kern.decode(stream, q, kv, kv_len, sk, sv, temp, got, got_l, window_size=W, n_splits=splits, no_alloc=True)
        stream.synchronize()
        assert torch.cuda.mem_get_info(device)[0] == free_before, "the call changed the device's free memory"
        assert torch.equal(got, ref)
        assert torch.equal(got_l, ref_l)
        o_out, o_l = o_attn.attn_decode_i8(host[0], host[1], kv_len, host[2], host[3], host[4], W, H, D, kv_tile=1 << 20)
        hist = code_hist(got.cpu().numpy(), o_out)
        assert hist[2:].sum() == 0 and hist[1] / o_out.size <= 0.08, hist
        assert np.max(np.abs(got_l.cpu().numpy() - o_l)) <= 1e-3


def test_no_alloc_decode_matches_allocating_entry_point(stream):
    _compare(stream, torch.device("cuda", 0))


def test_no_alloc_decode_on_a_second_device():
    """The scratch array's address is resolved per device (with that device current)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    from x17ai_b200 import device
    with device.CudaStream(1) as stream1:
        _compare(stream1, torch.device("cuda", 1))
        assert stream1.read_status() == [0, 0, 0, 0]


def test_no_alloc_decode_rejects_oversized_request(stream):
    from x17ai_b200 import X17Error, kernels as K
    B, H, D, T = 64, 32, 128, 4096
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    q = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
    kv = torch.zeros((B, 256, 2 * H * D), dtype=torch.int8, device="cuda")   # small cache: the check comes first
    sk = torch.zeros((H, D), dtype=torch.int8, device="cuda")
    temp = torch.ones(H, dtype=torch.float32, device="cuda")
    out = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    with pytest.raises(X17Error, match="exceeds the built-in scratch"):
        kern.decode(stream, q, kv, 256, sk, sk, temp, out, None, n_splits=16, no_alloc=True)
