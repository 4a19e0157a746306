"""int8 sliding-window attention through the C ABI against the oracle (cuda/attn_fwd_i8.cuh
restated in oracle/attn.py) and against the reference model's own fixtures.

The CUDA kernel finds the row maximum first and quantises P against it, which is the oracle
evaluated with a single KV tile (`kv_tile >= seq_len`).  Exact parts are checked exactly: the
int32 scores, and the int32 P.V accumulator given the kernel's own P.  P itself and the final
codes may differ from the oracle by one step where ex2.approx and libm exp2 straddle a rounding
boundary; the bars below were chosen from what the reference's own kernel achieves against its
float64 model (expected.txt:65-99).
"""
import numpy as np
import pytest
import torch

from conftest import code_hist, load_golden
from oracle import attn as o_attn, formats

pytestmark = pytest.mark.gpu
ALL = 1 << 20


@pytest.fixture(autouse=True, params=["persistent", "persistent_runs_of_3", "persistent_runs_of_1", "per_tile"])
def attn_schedule(request):
    """Every test of this file runs on both attention kernels; the persistent one also with short runs of
    query tiles per item, so that small shapes cross item boundaries and take the unfused first sweep."""
    from x17ai_b200 import kernels as K
    which, tiles = {"persistent": (K.ATTN_PERSISTENT, 0), "persistent_runs_of_3": (K.ATTN_PERSISTENT, 3),
                    "persistent_runs_of_1": (K.ATTN_PERSISTENT, 1), "per_tile": (K.ATTN_PER_TILE, 0)}[request.param]
    K.set_attn_schedule(which, tiles)
    yield request.param
    K.set_attn_schedule()


def _inputs(rng, B, S, H, D, kv_pad=0, q_pad=0):
    q = formats.quantize_fixedi8(rng.standard_normal((B, S, H * D + q_pad)))
    k = rng.standard_normal((B, S, H, D))
    k = k / np.sqrt((k ** 2).mean(-1, keepdims=True))   # unit RMS, as the KV projection produces
    v = rng.standard_normal((B, S, H, D)) * 1.3
    kv = np.concatenate((k, v), axis=-1).reshape(B, S, H * 2 * D)
    kv = formats.quantize_fixedi8(kv)
    if kv_pad:
        kv = np.concatenate((kv, np.zeros((B, S, kv_pad), np.int8)), axis=-1)
    sk = rng.standard_normal((H, D))
    sk = formats.quantize_fixedi8(sk / np.sqrt((sk ** 2).mean(-1, keepdims=True)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    return q, kv, sk, sv, temp


def _launch(stream, q, kv, sk, sv, temp, H, D, window, debug=False):
    from x17ai_b200 import kernels as K
    B, S = q.shape[0], q.shape[1]
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, q.shape[2], kv.shape[2], H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tq, tkv, tsk, tsv, tt = t(q), t(kv), t(sk), t(sv), t(temp)
    out = torch.zeros((B, S, H * D), dtype=torch.int8, device="cuda")
    l = torch.zeros((B, H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    if debug:
        ds = torch.zeros((B * H, S, S), dtype=torch.int32, device="cuda")
        dp = torch.zeros((B * H, S, S), dtype=torch.uint8, device="cuda")
        do = torch.zeros((B * H, S, D), dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        kern.launch_debug(stream, tq, tkv, tsk, tsv, tt, out, l, window, ds, dp, do)
        stream.synchronize()
        return out.cpu().numpy(), l.cpu().numpy(), ds.cpu().numpy(), dp.cpu().numpy(), do.cpu().numpy()
    kern.launch(stream, tq, tkv, tsk, tsv, tt, out, l, window)
    stream.synchronize()
    return out.cpu().numpy(), l.cpu().numpy()


def _oracle(q, kv, sk, sv, temp, H, D, window, kv_tile=ALL):
    outs, ls = [], []
    for b in range(q.shape[0]):
        o, l = o_attn.attn_fwd_i8(q[b][:, :H * D], kv[b][:, :2 * H * D], sk, sv, temp, window, H, D, kv_tile=kv_tile)
        outs.append(o); ls.append(l)
    return np.stack(outs), np.stack(ls)


def _check(out, l, ref_out, ref_l):
    hist = code_hist(out, ref_out)
    assert hist[2:].sum() == 0, f"codes off by more than one: {hist}"
    assert hist[1] / out.size <= 5e-3, f"too many codes off by one: {hist}"
    assert np.max(np.abs(l - ref_l)) <= 1e-3


@pytest.mark.parametrize("D,S,W", [(128, 256, 0), (128, 384, 128), (64, 256, 64), (32, 256, 48), (128, 512, 160)])
def test_attention_stages_exact(stream, D, S, W):
    """int32 scores and the int32 P.V accumulator are bit-exact; P is within one step of the oracle."""
    rng = np.random.default_rng(D + S + W)
    B, H = 1, 2
    W16 = ((W + 15) // 16) * 16
    q, kv, sk, sv, temp = _inputs(rng, B, S, H, D)
    out, l, ds, dp, do = _launch(stream, q, kv, sk, sv, temp, H, D, W16, debug=True)
    i = np.arange(S)[:, None]; j = np.arange(S)[None, :]
    visible = (j < i) & ((j >= i - W16) if W16 else True)
    for h in range(H):
        qh = q[0][:, h * D:(h + 1) * D].astype(np.int64)
        kh = kv[0][:, 2 * h * D:2 * h * D + D].astype(np.int64)
        vh = kv[0][:, 2 * h * D + D:2 * (h + 1) * D].astype(np.int64)
        s_ref = qh @ kh.T
        assert np.array_equal(ds[h][visible], s_ref[visible].astype(np.int32)), "Q.K^T int32 scores differ"
        assert np.all(dp[h][~visible] == 0), "masked probabilities must be zero"
        o_ref = dp[h].astype(np.int64) @ vh
        assert np.array_equal(do[h], o_ref.astype(np.int32)), "P.V int32 accumulator differs"
    ref_out, ref_l = _oracle(q, kv, sk, sv, temp, H, D, W16)
    _check(out, l, ref_out, ref_l)


@pytest.mark.parametrize("B,H,D,S,W", [
    (1, 4, 64, 256, 64),       # the reference's CPU-runnable case (batch 1, 4 heads, seq 256, window 64)
    (2, 3, 128, 640, 256),
    (1, 2, 128, 1024, 0),
    (1, 2, 64, 200, 32),       # ragged: seq not a multiple of the query tile
    (1, 2, 32, 128, 16),
    (2, 2, 128, 2048, 1024),
])
def test_attention_vs_oracle(stream, B, H, D, S, W):
    rng = np.random.default_rng(B * 7 + H * 5 + D + S + W)
    q, kv, sk, sv, temp = _inputs(rng, B, S, H, D)
    out, l = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    ref_out, ref_l = _oracle(q, kv, sk, sv, temp, H, D, W)
    _check(out, l, ref_out, ref_l)


def test_attention_strided_rows(stream):
    """q_stride / kv_stride larger than the packed width (head-sharded launches address a column
    block of a wider tensor, attn_fwd_i8.cuh:378-384)."""
    rng = np.random.default_rng(11)
    B, H, D, S, W = 1, 2, 128, 256, 64
    q, kv, sk, sv, temp = _inputs(rng, B, S, H, D, kv_pad=256, q_pad=128)
    out, l = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    ref_out, ref_l = _oracle(q, kv, sk, sv, temp, H, D, W)
    _check(out, l, ref_out, ref_l)


def test_attention_negative_temperature(stream):
    rng = np.random.default_rng(12)
    B, H, D, S, W = 1, 2, 64, 256, 0
    q, kv, sk, sv, temp = _inputs(rng, B, S, H, D)
    temp = np.array([-0.7, 0.0], dtype=np.float32)
    out, l = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    ref_out, ref_l = _oracle(q, kv, sk, sv, temp, H, D, W)
    _check(out, l, ref_out, ref_l)


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_attention_against_reference_fixtures(stream, name):
    """Against the reference's float64 model on its own tensors: the reference's kernel differs from
    that model on 34.3 % of codes, by at most 5, and L by at most 0.81 (expected.txt:65-99)."""
    g, c = load_golden(name)
    S, H, D, W = c["S"], c["H"], c["D"], c["W"]
    q = g["q_i8"].reshape(1, S, H * D)
    kv = g["kv_i8"].reshape(1, S, 2 * H * D)
    sk, sv = g["sinks_k_i8"].reshape(H, D), g["sinks_v_i8"].reshape(H, D)
    temp = g["attn_temperature_f32"].reshape(H)
    out, l = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    hist = code_hist(out[0], g["attn_out_i8"].reshape(S, H * D))
    assert hist[1:].sum() / out.size <= 0.40 and hist[6:].sum() == 0
    assert np.max(np.abs(l[0] - g["attn_l_f32"].reshape(H, S))) < 1e-3
    ref_out, ref_l = _oracle(q, kv, sk, sv, temp, H, D, W)
    _check(out, l, ref_out, ref_l)
    # and against the reference kernel's own schedule (16-key running maximum): one step, rarely
    ref16, _ = _oracle(q, kv, sk, sv, temp, H, D, W, kv_tile=16)
    hist = code_hist(out, ref16)
    assert hist[2:].sum() == 0 and hist[1] / out.size <= 0.03


def test_attention_argument_errors(stream):
    from x17ai_b200 import X17Error, kernels as K
    kern = K.AttnKernel(K.AttnKernelConfig(2, 64, 128, 256, 128))
    z = lambda *s, dt=torch.int8: torch.zeros(s, dtype=dt, device="cuda")
    with pytest.raises(X17Error, match="window_size must be zero or divisible by 16"):
        kern.launch(stream, z(128, 128), z(128, 256), z(2, 64), z(2, 64), z(2, dt=torch.float32), z(128, 128), None, 24)
    with pytest.raises(X17Error, match="attention input kv has 64 rows, but should have 128"):
        kern.launch(stream, z(128, 128), z(64, 256), z(2, 64), z(2, 64), z(2, dt=torch.float32), z(128, 128), None, 0)
    with pytest.raises(X17Error, match="has dtype"):
        kern.launch(stream, z(128, 128), z(128, 256), z(2, 64), z(2, 64), z(2, dt=torch.float16), z(128, 128), None, 0)


@pytest.mark.parametrize("B,H,D,S,W", [(1, 2, 128, 384, 128), (2, 2, 64, 256, 0), (1, 4, 32, 200, 48)])
def test_attention_pv_fp8(stream, B, H, D, S, W):
    """fp8 P.V variant: bf16 output within max-abs error 1e-2 x RMS of the oracle's output (the bar the
    benchmark description sets for bf16 outputs); parity for this mode is pinned by the oracle only."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(B + H + D + S + W)
    q, kv, sk, _, temp = _inputs(rng, B, S, H, D)
    v_scale = np.abs(rng.standard_normal(H)).astype(np.float32) + 0.25
    kv4 = kv.reshape(B, S, H, 2, D).copy()
    v_val = rng.standard_normal((B, S, H, D)).astype(np.float32)
    v8 = formats.hw_f32_to_e4m3(v_val)
    kv4[:, :, :, 1, :] = v8.view(np.int8)
    kv = kv4.reshape(B, S, 2 * H * D)
    sv8 = formats.hw_f32_to_e4m3(rng.standard_normal((H, D)).astype(np.float32))
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tq, tkv, tsk, tsv, tt, tvs = t(q), t(kv), t(sk), t(sv8), t(temp), t(v_scale)
    out = torch.zeros((B, S, H * D), dtype=torch.bfloat16, device="cuda")
    l = torch.zeros((B, H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern.launch_pv_fp8(stream, tq, tkv, tsk, tsv, tt, tvs, out, l, W)
    stream.synchronize()
    got = out.float().cpu().numpy()
    for b in range(B):
        k_i8 = kv4[b, :, :, 0, :].reshape(S, H * D)
        ref, ref_l = o_attn.attn_fwd_pv_fp8(q[b], k_i8, v8[b].reshape(S, H * D), sk, sv8, temp, v_scale, W, H, D)
        rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
        assert np.max(np.abs(got[b] - ref)) <= 1e-2 * rms + 2.0 ** -8 * np.abs(ref).max()   # + one bf16 ulp of the largest value
        assert np.max(np.abs(l[b].cpu().numpy() - ref_l)) <= 1e-3


def test_attention_from_host_matches_single_launch(stream):
    """launch_from_host (per-sequence upload -> kernel -> download over three streams) returns
    exactly what one batched launch on device-resident data returns."""
    from x17ai_b200 import device, kernels as K
    B, H, D, S, W = 5, 2, 64, 300, 64
    q, kv, sk, sv, temp = _inputs(np.random.default_rng(11), B, S, H, D)
    want, _ = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    h_q, h_kv = t(q).pin_memory(), t(kv).pin_memory()
    h_out = torch.zeros((B, S, H * D), dtype=torch.int8).pin_memory()
    d_q, d_kv, d_out = torch.zeros_like(h_q, device="cuda"), torch.zeros_like(h_kv, device="cuda"), torch.zeros_like(h_out, device="cuda")
    tsk, tsv, tt = t(sk).cuda(), t(sv).cuda(), t(temp).cuda()
    torch.cuda.synchronize()
    extra = [device.CudaStream(0), device.CudaStream(0)]
    streams = [stream] + extra
    for _ in range(2):   # twice: the second round reuses every staging buffer
        kern.launch_from_host(streams, h_q, h_kv, tsk, tsv, tt, d_q, d_kv, d_out, h_out, None, W)
    for st in streams:
        st.synchronize()
    assert np.array_equal(h_out.numpy(), want)
    with pytest.raises(Exception, match="pinned"):
        kern.launch_from_host(streams, t(q), h_kv, tsk, tsv, tt, d_q, d_kv, d_out, h_out, None, W)
    for st in extra:
        st.close()


@pytest.mark.parametrize("B,H,D,S,W", [(1, 2, 128, 512, 128), (2, 2, 64, 384, 0)])
def test_attention_pv_fp8_against_the_int8_kernel(stream, B, H, D, S, W):
    """The fp8 P.V kernel tied to the int8 kernel, which the reference's own kernel pins: with V drawn from small
    integers (exact as int8 codes and as e4m3 values alike) both kernels normalise the same sum of p * v; they
    differ only in how they quantise p (steps of 1/255 against eight-step e4m3 binades) and in the last rounding
    (int8 code against bf16). So out_fp8 / v_scale stays within one code of the int8 kernel's output everywhere and
    within a fraction of a code on average; a wrong V layout, scale, sink or normaliser would break this at once."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(B + H + D + S + W + 1)
    q, kv, sk, _, temp = _inputs(rng, B, S, H, D)
    v_int = rng.integers(-12, 13, (B, S, H, D)).astype(np.int8)
    sv_int = rng.integers(-12, 13, (H, D)).astype(np.int8)
    kv4 = kv.reshape(B, S, H, 2, D).copy()
    kv4[:, :, :, 1, :] = v_int
    kv_i8 = kv4.reshape(B, S, 2 * H * D)
    out_i8, l_i8 = _launch(stream, q, kv_i8, sk, sv_int, temp, H, D, W)
    # the same values as e4m3 bytes, with a per-head scale that the output must carry
    kv4[:, :, :, 1, :] = formats.hw_f32_to_e4m3(v_int.astype(np.float32)).view(np.int8)
    assert np.array_equal(formats.hw_e4m3_to_f32(kv4[:, :, :, 1, :].view(np.uint8)), v_int.astype(np.float32))
    sv8 = formats.hw_f32_to_e4m3(sv_int.astype(np.float32))
    v_scale = (0.5 + rng.random(H)).astype(np.float32)
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tq, tkv, tsk, tsv, tt, tvs = t(q), t(kv4.reshape(B, S, 2 * H * D)), t(sk), t(sv8), t(temp), t(v_scale)
    out = torch.zeros((B, S, H * D), dtype=torch.bfloat16, device="cuda")
    l = torch.zeros((B, H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern.launch_pv_fp8(stream, tq, tkv, tsk, tsv, tt, tvs, out, l, W)
    stream.synchronize()
    got = out.float().cpu().numpy().reshape(B, S, H, D) / v_scale[None, None, :, None]
    diff = np.abs(got - out_i8.reshape(B, S, H, D).astype(np.float32))
    assert diff.max() <= 1.0 and diff.mean() <= 0.3, (diff.max(), diff.mean())
    # the normaliser: L = log2(scale * sum) + max with scale 256 here and 255 there
    assert np.max(np.abs(l.cpu().numpy() - l_i8 - np.log2(256.0 / 255.0))) <= 1e-3


def _scaled_case(rng, B, S, H, D):
    """N(0,1) q, k, v quantised with per-token-per-head scales (absmax / 127), as the benchmark description draws them."""
    out = []
    for _ in range(3):
        codes, scale = o_attn.quantize_per_token(rng.standard_normal((B, S, H, D)))
        out.append((codes, np.ascontiguousarray(scale.transpose(0, 2, 1))))     # scale [B, H, S]
    sk = formats.quantize_fixedi8(rng.standard_normal((H, D)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    return out, sk, sv, temp


def _launch_scaled(stream, qs, ks, vs, sk, sv, temp, H, D, W):
    from x17ai_b200 import kernels as K
    (qc, qscale), (kc, kscale), (vc, vscale) = qs, ks, vs
    B, S = qc.shape[0], qc.shape[1]
    kv = np.concatenate((kc, vc), axis=-1).reshape(B, S, 2 * H * D)
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    args = [t(qc.reshape(B, S, H * D)), t(qscale), t(kv), t(kscale), t(vscale), t(sk), t(sv), t(temp)]
    out = torch.zeros((B, S, H * D), dtype=torch.bfloat16, device="cuda")
    l = torch.zeros((B, H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern.launch_scaled(stream, *args, out, l, W)
    stream.synchronize()
    return out.float().cpu().numpy().reshape(B, S, H, D), l.cpu().numpy()


@pytest.mark.parametrize("B,H,D,S,W", [
    (1, 4, 64, 256, 64),       # the benchmark description's CPU-runnable case, seed 0
    (2, 2, 128, 640, 256),
    (1, 2, 32, 200, 48),       # ragged
    (1, 2, 128, 512, 0),
])
def test_attention_per_token_scales_bf16_out(stream, B, H, D, S, W):
    """Per-token-per-head scaled int8 inputs, bf16 output: max-abs error <= 1e-2 x RMS (the bar the benchmark description
    sets for bf16 outputs) against the float64 restatement with the kernel's u8 probabilities, and within the
    quantisation noise of those probabilities (a few percent of the RMS at a 48-key window, where every key carries
    weight) of the plain float64 softmax attention of the dequantised inputs. Parity of this mode is pinned by the
    oracle only."""
    rng = np.random.default_rng(0 if (B, H, D, S, W) == (1, 4, 64, 256, 64) else B + H + D + S + W)
    (qs, ks, vs), sk, sv, temp = _scaled_case(rng, B, S, H, D)
    got, l = _launch_scaled(stream, qs, ks, vs, sk, sv, temp, H, D, W)
    for b in range(B):
        args = (qs[0][b], qs[1][b], ks[0][b], ks[1][b], vs[0][b], vs[1][b], sk, sv, temp, W)
        ref_q, ref_l = o_attn.attn_fwd_i8_scaled(*args, quantise_p=True)
        rms = np.sqrt(np.mean(ref_q ** 2))
        assert np.max(np.abs(got[b] - ref_q)) <= 1e-2 * rms + 2.0 ** -8 * np.abs(ref_q).max()    # + one bf16 ulp
        assert np.max(np.abs(l[b] - ref_l)) <= 1e-3
        ref, _ = o_attn.attn_fwd_i8_scaled(*args, quantise_p=False)
        assert np.max(np.abs(got[b] - ref)) <= 6e-2 * rms
        assert np.sqrt(np.mean((got[b] - ref) ** 2)) <= 1e-2 * rms


def test_attention_per_token_scales_reduce_to_fixedi8(stream):
    """With every scale equal to 1/8 the mode is the FixedI8 kernel, which the reference's kernel pins: out = code / 8
    to bf16 and quantisation precision, L equal."""
    rng = np.random.default_rng(77)
    B, H, D, S, W = 1, 2, 128, 384, 128
    q, kv, sk, sv, temp = _inputs(rng, B, S, H, D)
    out_i8, l_i8 = _launch(stream, q, kv, sk, sv, temp, H, D, W)
    kv4 = kv.reshape(B, S, H, 2, D)
    eighth = np.full((B, H, S), 0.125, dtype=np.float32)
    got, l = _launch_scaled(stream, (q.reshape(B, S, H, D), eighth), (kv4[:, :, :, 0], eighth), (kv4[:, :, :, 1], eighth),
                            sk, sv, temp, H, D, W)
    want = out_i8.reshape(B, S, H, D).astype(np.float32) / 8.0
    # the FixedI8 output is rounded to 1/8; the bf16 one carries the unrounded value: half a code plus bf16 precision
    assert np.max(np.abs(got - want)) <= 0.5 / 8 + 2.0 ** -8 * np.abs(want).max() + 1e-3
    assert np.max(np.abs(l - l_i8)) <= 1e-3
