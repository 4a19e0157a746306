"""int8 decode attention through the C ABI against the oracle (row kv_len of the prefill kernel)."""
import numpy as np
import pytest
import torch

from conftest import code_hist
from oracle import attn as o_attn, formats

pytestmark = pytest.mark.gpu


def _case(rng, B, H, D, T):
    q = formats.quantize_fixedi8(rng.standard_normal((B, H * D)))
    k = rng.standard_normal((B, T, H, D))
    k = k / np.sqrt((k ** 2).mean(-1, keepdims=True))
    v = rng.standard_normal((B, T, H, D)) * 1.3
    kv = formats.quantize_fixedi8(np.concatenate((k, v), axis=-1).reshape(B, T, H * 2 * D))
    sk = rng.standard_normal((H, D))
    sk = formats.quantize_fixedi8(sk / np.sqrt((sk ** 2).mean(-1, keepdims=True)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    return q, kv, sk, sv, temp


@pytest.mark.parametrize("B,H,D,T,kv_len,W,splits", [
    (3, 4, 128, 512, 512, 0, 1),
    (3, 4, 128, 512, 300, 128, 1),
    (2, 2, 64, 256, 256, 64, 1),
    (2, 2, 32, 128, 100, 0, 1),
    (1, 2, 128, 2048, 2048, 0, 4),     # split-KV path through scratch memory
    (2, 2, 128, 1024, 777, 512, 3),
    (2, 4, 128, 64, 0, 0, 1),          # empty cache: only the sink token
])
def test_decode_vs_oracle(stream, B, H, D, T, kv_len, W, splits):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(B + H + D + T + kv_len + W)
    q, kv, sk, sv, temp = _case(rng, B, H, D, T)
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(a).cuda()
    out = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
    l = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    tq, tkv = t(q), t(kv)
    torch.cuda.synchronize()
    kern.decode(stream, tq, tkv, kv_len, t(sk), t(sv), t(temp), out, l, window_size=W, n_splits=splits)
    stream.synchronize()
    ref_out, ref_l = o_attn.attn_decode_i8(q, kv, kv_len, sk, sv, temp, W, H, D, kv_tile=1 << 20)
    hist = code_hist(out.cpu().numpy(), ref_out)
    # The kernel rounds P against running maxima per lane group, the oracle against the final
    # maximum: two different roundings of the same probabilities. Neither is off by more than one
    # code; where O / sum lands within ~0.01 of a half-integer the two round apart (a few percent).
    assert hist[2:].sum() == 0 and hist[1] / ref_out.size <= 0.08, hist
    assert np.max(np.abs(l.cpu().numpy() - ref_l)) <= 1e-3


def test_decode_per_sequence_lengths(stream):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(99)
    B, H, D, T = 4, 2, 128, 512
    q, kv, sk, sv, temp = _case(rng, B, H, D, T)
    lens = np.array([512, 17, 0, 256], dtype=np.uint32)
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(a).cuda()
    out = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
    tl = torch.from_numpy(lens.view(np.int32)).cuda()
    tq, tkv = t(q), t(kv)
    torch.cuda.synchronize()
    kern.decode(stream, tq, tkv, T, t(sk), t(sv), t(temp), out, None, window_size=0, kv_lens=tl, n_splits=1)
    stream.synchronize()
    got = out.cpu().numpy()
    for b in range(B):
        ref, _ = o_attn.attn_decode_i8(q[b:b + 1], kv[b:b + 1], int(lens[b]), sk, sv, temp, 0, H, D, kv_tile=1 << 20)
        hist = code_hist(got[b], ref[0])
        assert hist[2:].sum() == 0 and hist[1] / ref.size <= 0.08


def test_decode_per_sequence_lengths_split(stream):
    """Per-sequence lengths through the split-KV path (partials in scratch memory, merge kernel); a length
    above the cache's capacity is clamped to it on the device instead of reading past the cache."""
    from x17ai_b200 import X17Error, kernels as K
    rng = np.random.default_rng(7)
    B, H, D, T = 4, 2, 128, 1024
    q, kv, sk, sv, temp = _case(rng, B, H, D, T)
    lens = np.array([1024, 333, 5000, 640], dtype=np.uint32)    # 5000 > T: treated as T
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(a).cuda()
    tq, tkv, tsk, tsv, tt = t(q), t(kv), t(sk), t(sv), t(temp)
    tl = torch.from_numpy(lens.view(np.int32)).cuda()
    torch.cuda.synchronize()
    for splits, no_alloc in ((3, False), (4, True)):
        out = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
        torch.cuda.synchronize()
        kern.decode(stream, tq, tkv, T, tsk, tsv, tt, out, None, window_size=256, kv_lens=tl, n_splits=splits,
                    no_alloc=no_alloc)
        stream.synchronize()
        got = out.cpu().numpy()
        for b in range(B):
            ref, _ = o_attn.attn_decode_i8(q[b:b + 1], kv[b:b + 1], min(int(lens[b]), T), sk, sv, temp, 256, H, D,
                                           kv_tile=1 << 20)
            hist = code_hist(got[b], ref[0])
            assert hist[2:].sum() == 0 and hist[1] / ref.size <= 0.08, (splits, b, hist)
    out = torch.zeros((B, H * D), dtype=torch.int8, device="cuda")
    with pytest.raises(X17Error, match="kv_lens must be int32"):
        kern.decode(stream, tq, tkv, T, tsk, tsv, tt, out, None, kv_lens=tl.to(torch.int64))
    with pytest.raises(X17Error, match="kv_lens must be int32"):
        kern.decode(stream, tq, tkv, T, tsk, tsv, tt, out, None, kv_lens=tl[:2])
