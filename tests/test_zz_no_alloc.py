"""The decode entry point that allocates nothing (x17ai_b200_attn_decode_i8_noalloc).

It serves hosts that cannot allocate device memory at call time (memory carved up at start-up,
a memory pool that is exhausted or switched off, a no-allocation policy after warm-up): the
split-KV partials live in a 4 MiB array inside the library image.  Checked here through the C
ABI: its output equals the allocating entry point's bit for bit (same kernels, same order of
operations) on two calls in a row that reuse the scratch, and a request beyond the built-in
scratch is refused with a clear message.  This file sorts last so that a failure here cannot
hide another test's result in a run that stops at the first failure.
"""
import numpy as np
import pytest
import torch

from oracle import formats

pytestmark = pytest.mark.gpu


def _case(rng, B, H, D, T):
    q = formats.quantize_fixedi8(rng.standard_normal((B, H * D)))
    kv = formats.quantize_fixedi8(rng.standard_normal((B, T, H * 2 * D)))
    sk = formats.quantize_fixedi8(rng.standard_normal((H, D)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    return [torch.from_numpy(a).cuda() for a in (q, kv, sk, sv, temp)]


def test_no_alloc_decode_matches_allocating_entry_point(stream):
    from x17ai_b200 import kernels as K
    B, H, D = 2, 4, 128
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    rng = np.random.default_rng(2024)
    # two calls in a row with different shapes and split counts: the second reuses (and must fully
    # overwrite) the slots the first one left behind
    for T, kv_len, W, splits in [(2048, 2048, 0, 8), (1024, 700, 256, 3)]:
        q, kv, sk, sv, temp = _case(rng, B, H, D, T)
        ref = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
        ref_l = torch.zeros((B, H), dtype=torch.float32, device="cuda")
        got = torch.full((B, H * D), 77, dtype=torch.int8, device="cuda")
        got_l = torch.zeros((B, H), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        kern.decode(stream, q, kv, kv_len, sk, sv, temp, ref, ref_l, window_size=W, n_splits=splits)
        kern.decode(stream, q, kv, kv_len, sk, sv, temp, got, got_l, window_size=W, n_splits=splits, no_alloc=True)
        stream.synchronize()
        assert torch.equal(got, ref)
        assert torch.equal(got_l, ref_l)


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
