"""The benchmark's full sizes. The oracle cannot evaluate a whole launch of these sizes in seconds, so each
test runs the full launch on the device and checks
  * sampled units (a (sequence, head) pair, a token row, a sequence of the decode batch) against the oracle
    on exactly the inputs the device used, with the bars of the small-size tests, and
  * properties that hold at any size: a unit's result does not depend on the other units of the launch
    (the same unit launched alone returns the same bytes), and keys outside a query's window cannot
    change its output.
Inputs are seeded synthetic tensors of the benchmark's shapes and distributions.
"""
import numpy as np
import pytest
import torch

from conftest import code_hist
from oracle import attn as o_attn, gemm as o_gemm, rms_norm as o_rms

pytestmark = pytest.mark.gpu
ALL = 1 << 20


def _codes(g, *shape):
    """FixedI8 codes of N(0,1) values, generated on the device."""
    return torch.clamp(torch.round(torch.randn(*shape, generator=g, device="cuda") * 8.0), -127, 127).to(torch.int8)


def test_attention_prefill_full_size(stream):
    """configs[1]: batch 8, 32 heads x 128, 8192 tokens, window 1024 (1.03e12 operations, q + kv + out = 1.07 GB)."""
    from x17ai_b200 import kernels as K
    B, H, D, S, W = 8, 32, 128, 8192, 1024
    g = torch.Generator(device="cuda").manual_seed(0)
    q, kv, sk, sv = _codes(g, B, S, H * D), _codes(g, B, S, 2 * H * D), _codes(g, H, D), _codes(g, H, D)
    temp = (0.5 + torch.rand(H, generator=g, device="cuda")).float()
    out = torch.zeros(B, S, H * D, dtype=torch.int8, device="cuda")
    l = torch.zeros(B, H, S, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    kern.launch(stream, q, kv, sk, sv, temp, out, l, W)
    stream.synchronize()

    # sampled (sequence, head) units against the oracle with the kernel's schedule (one tile)
    for b, h in ((0, 0), (5, 17), (7, 31)):
        qh = q[b, :, h * D:(h + 1) * D].cpu().numpy()
        kvh = kv[b, :, 2 * h * D:2 * (h + 1) * D].cpu().numpy()
        ref_out, ref_l = o_attn.attn_fwd_i8(qh, kvh, sk[h:h + 1].cpu().numpy(), sv[h:h + 1].cpu().numpy(),
                                            temp[h:h + 1].cpu().numpy(), W, 1, D, kv_tile=ALL)
        got = out[b, :, h * D:(h + 1) * D].cpu().numpy()
        hist = code_hist(got, ref_out)
        assert hist[2:].sum() == 0 and hist[1] / got.size <= 5e-3, (b, h, hist[:4])
        assert np.max(np.abs(l[b, h].cpu().numpy() - ref_l[0])) <= 1e-3

    # a sequence launched alone returns the bytes it got inside the batch
    out1 = torch.zeros(1, S, H * D, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    kern.launch(stream, q[3:4], kv[3:4], sk, sv, temp, out1, None, W)
    stream.synchronize()
    assert torch.equal(out1[0], out[3])

    # keys further back than the window cannot matter: new values in the first half of sequence 3 leave
    # every query from 4096 + 1024 on unchanged, and do change earlier ones
    kv2 = kv[3:4].clone()
    kv2[0, :S // 2] = _codes(g, S // 2, 2 * H * D)
    torch.cuda.synchronize()
    kern.launch(stream, q[3:4], kv2, sk, sv, temp, out1, None, W)
    stream.synchronize()
    first_free = S // 2 + W   # query i sees keys i - W .. i - 1
    assert torch.equal(out1[0, first_free:], out[3, first_free:])
    assert not torch.equal(out1[0, :S // 2], out[3, :S // 2])


def test_attention_pv_fp8_full_size(stream):
    """configs[2]: the fp8 P.V variant at batch 8, 32 heads x 128, 8192 tokens, window 1024; sampled (sequence,
    head) units against the oracle of this mode (bf16 output within 1e-2 x RMS), and a sequence launched alone
    returns the bytes it got inside the batch."""
    from oracle import formats
    from x17ai_b200 import kernels as K
    B, H, D, S, W = 8, 32, 128, 8192, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    q, kv, sk = _codes(g, B, S, H * D), _codes(g, B, S, 2 * H * D), _codes(g, H, D)
    kv.view(B, S, H, 2, D)[:, :, :, 1, :] = torch.randn(B, S, H, D, generator=g, device="cuda").to(torch.float8_e4m3fn).view(torch.int8)
    sv8 = torch.randn(H, D, generator=g, device="cuda").to(torch.float8_e4m3fn).view(torch.uint8)
    temp = (0.5 + torch.rand(H, generator=g, device="cuda")).float()
    v_scale = (0.25 + torch.rand(H, generator=g, device="cuda")).float()
    out = torch.zeros(B, S, H * D, dtype=torch.bfloat16, device="cuda")
    l = torch.zeros(B, H, S, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    kern.launch_pv_fp8(stream, q, kv, sk, sv8, temp, v_scale, out, l, W)
    stream.synchronize()
    for b, h in ((0, 3), (6, 30)):
        qh = q[b, :, h * D:(h + 1) * D].cpu().numpy()
        kh = kv[b, :, 2 * h * D:2 * h * D + D].cpu().numpy()
        vh = kv[b, :, 2 * h * D + D:2 * (h + 1) * D].cpu().numpy().view(np.uint8)
        ref, ref_l = o_attn.attn_fwd_pv_fp8(qh, kh, vh, sk[h:h + 1].cpu().numpy(), sv8[h:h + 1].cpu().numpy(),
                                            temp[h:h + 1].cpu().numpy(), v_scale[h:h + 1].cpu().numpy(), W, 1, D)
        got = out[b, :, h * D:(h + 1) * D].float().cpu().numpy()
        rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
        assert np.max(np.abs(got - ref)) <= 1e-2 * rms + 2.0 ** -8 * np.abs(ref).max(), (b, h)
        assert np.max(np.abs(l[b, h].cpu().numpy() - ref_l[0])) <= 1e-3
    out1 = torch.zeros(1, S, H * D, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    kern.launch_pv_fp8(stream, q[5:6], kv[5:6], sk, sv8, temp, v_scale, out1, None, W)
    stream.synchronize()
    assert torch.equal(out1[0], out[5])


def test_attention_per_token_scales_full_size(stream):
    """The per-token-scale mode at configs[1]'s size through two properties that need no oracle at that size: with
    every scale 1/8 it is the FixedI8 kernel (out = code / 8 to half a code and bf16 precision, L equal), and
    doubling every query scale of a sequence while halving its temperature changes nothing."""
    from x17ai_b200 import kernels as K
    B, H, D, S, W = 8, 32, 128, 8192, 1024
    g = torch.Generator(device="cuda").manual_seed(4)
    q, kv, sk, sv = _codes(g, B, S, H * D), _codes(g, B, S, 2 * H * D), _codes(g, H, D), _codes(g, H, D)
    temp = (0.5 + torch.rand(H, generator=g, device="cuda")).float()
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    out_i8 = torch.zeros(B, S, H * D, dtype=torch.int8, device="cuda")
    l_i8 = torch.zeros(B, H, S, dtype=torch.float32, device="cuda")
    eighth = torch.full((B, H, S), 0.125, dtype=torch.float32, device="cuda")
    out = torch.zeros(B, S, H * D, dtype=torch.bfloat16, device="cuda")
    l = torch.zeros(B, H, S, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern.launch(stream, q, kv, sk, sv, temp, out_i8, l_i8, W)
    kern.launch_scaled(stream, q, eighth, kv, eighth, eighth, sk, sv, temp, out, l, W)
    stream.synchronize()
    want = out_i8.float() / 8.0
    diff = (out.float() - want).abs().max().item()
    assert diff <= 0.5 / 8 + 2.0 ** -8 * want.abs().max().item() + 1e-3, diff
    assert (l - l_i8).abs().max().item() <= 1e-3
    # scale invariance: q_scale * 2 with temperature / 2 is the same attention (powers of two: exact in f32)
    out2 = torch.zeros_like(out)
    torch.cuda.synchronize()
    kern.launch_scaled(stream, q, eighth * 2.0, kv, eighth, eighth, sk, sv, temp * 0.5, out2, None, W)
    stream.synchronize()
    assert stream.read_status() == [0, 0, 0, 0]
    assert torch.equal(out2, out)      # the row factor temperature * q_scale is the same float


def test_ffn_full_size(stream):
    """configs[3]: 16384 tokens, d_model 4096, hidden 14336: GeGLU GEMM and the e4m3 x int8 projection with the
    gated residual, sampled token rows against the oracle (rows are independent units)."""
    from x17ai_b200 import kernels as K
    M, Dm, F = 16384, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(1)
    x, wf, wy = _codes(g, M, Dm), _codes(g, 2 * F, Dm), _codes(g, 2 * Dm, F)
    f = torch.zeros(M, F, dtype=torch.uint8, device="cuda")
    y = torch.zeros(M, Dm, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    k_f, k_y = K.GemmKernel(K.ffn_f_fwd_config(Dm, F)), K.GemmKernel(K.ffn_y_fwd_f8_config(F, Dm))
    wy_split = K.split_i8_weights(stream, wy)
    k_f.launch(stream, x, wf, f)
    k_y.launch(stream, f, wy_split, y, residual=x)
    stream.synchronize()
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191, 8192, 12345, 16256, 16383], device="cuda")
    xs, fs, ys = x[rows].cpu().numpy(), f[rows].cpu().numpy(), y[rows].cpu().numpy()
    ref_f = o_gemm.ffn_f_fwd(xs, wf.cpu().numpy())
    assert (fs != ref_f).mean() <= 2e-3
    ref_y = o_gemm.ffn_y_fwd_f8(fs, wy.cpu().numpy(), xs)
    assert (ys != ref_y).mean() <= 2e-3
    # the same rows as a launch of their own (128 rows: one tile) return the same bytes
    xa = x[8192:8320].contiguous()
    fa = torch.zeros(128, F, dtype=torch.uint8, device="cuda")
    ya = torch.zeros(128, Dm, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    k_f.launch(stream, xa, wf, fa)
    k_y.launch(stream, fa, wy_split, ya, residual=xa)
    stream.synchronize()
    assert torch.equal(fa, f[8192:8320]) and torch.equal(ya, y[8192:8320])


def test_decode_full_size(stream):
    """configs[4] decode: 256 sequences, one new token each against an int8 cache of 4096 tokens (8.6 GB),
    sampled sequences against the oracle; a sequence decoded alone agrees within one code."""
    from x17ai_b200 import kernels as K
    B, H, D, T = 256, 32, 128, 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    kv = torch.empty(B, T, 2 * H * D, dtype=torch.int8, device="cuda")
    for b in range(B):   # filled per sequence: the float staging tensor stays small
        kv[b] = _codes(g, T, 2 * H * D)
    q, sk, sv = _codes(g, B, H * D), _codes(g, H, D), _codes(g, H, D)
    temp = (0.5 + torch.rand(H, generator=g, device="cuda")).float()
    out = torch.zeros(B, H * D, dtype=torch.int8, device="cuda")
    l = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    kern.decode(stream, q, kv, T, sk, sv, temp, out, l, window_size=T)
    stream.synchronize()
    pick = [0, 101, 255]
    ref_out, ref_l = o_attn.attn_decode_i8(q[pick].cpu().numpy(), kv[pick].cpu().numpy(), T, sk.cpu().numpy(),
                                           sv.cpu().numpy(), temp.cpu().numpy(), T, H, D, kv_tile=ALL)
    hist = code_hist(out[pick].cpu().numpy(), ref_out)
    assert hist[2:].sum() == 0 and hist[1] / ref_out.size <= 0.08, hist[:4]
    assert np.max(np.abs(l[pick].cpu().numpy() - ref_l)) <= 1e-3
    out1 = torch.zeros(1, H * D, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    kern.decode(stream, q[101:102], kv[101:102], T, sk, sv, temp, out1, None, window_size=T)
    stream.synchronize()
    hist = code_hist(out1.cpu().numpy(), out[101:102].cpu().numpy())
    # alone, the sequence is split over more CTAs than inside the batch: another rounding schedule of the
    # same probabilities, so a code may move by one step, never by more
    assert hist[2:].sum() == 0, hist[:4]


def test_rms_norm_full_size(stream):
    """131072 rows x 4096 (the block's token count at configs[4]): sampled rows against the oracle, and a
    slice of rows normalised alone returns the same bytes."""
    from x17ai_b200 import kernels as K
    M, Dm = 131072, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.empty(M, Dm, dtype=torch.uint8, device="cuda")
    for r0 in range(0, M, 16384):
        x[r0:r0 + 16384] = (torch.randn(16384, Dm, generator=g, device="cuda") * 2.0).to(torch.float8_e4m3fn).view(torch.uint8)
    y = torch.zeros(M, Dm, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    K.rms_norm(stream, K.RMS_E4M3_FIXED, x, y)
    stream.synchronize()
    rows = torch.tensor([0, 1, 4095, 65535, 65536, 100000, 131071], device="cuda")
    ref = o_rms.rms_norm_e4m3_i8(x[rows].cpu().numpy())
    dd = np.abs(y[rows].cpu().numpy().astype(np.int32) - ref.astype(np.int32))
    assert dd.max() <= 1 and (dd > 0).mean() <= 2e-3
    y1 = torch.zeros(256, Dm, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    K.rms_norm(stream, K.RMS_E4M3_FIXED, x[70000:70256].contiguous(), y1)
    stream.synchronize()
    assert torch.equal(y1, y[70000:70256])
