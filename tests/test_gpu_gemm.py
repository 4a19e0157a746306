"""The tcgen05 GEMM and its fused epilogues through the C ABI against the oracle
(cuda/gemm_b8.cuh, cuda/gemm_b16.cuh restated in oracle/gemm.py) and the golden fixtures."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import formats, gemm as o_gemm

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["one_cta", "cta_pair"])
def gemm_tiling(request):
    """Every test runs with both tilings of the GEMM: one CTA per 128 x 256 tile, and clusters of two CTAs on
    256 x 256 tiles (taken for inputs of more than 128 rows whose N is a multiple of 256)."""
    from x17ai_b200 import kernels as K
    K.set_gemm_tiling(K.GEMM_CTA_PAIR if request.param == "cta_pair" else K.GEMM_ONE_CTA)
    yield request.param
    K.set_gemm_tiling()


def _rand_i8(rng, shape, std=1.0):
    return formats.quantize_fixedi8(rng.standard_normal(shape) * std)


def _run(stream, cfg, a, b, c_shape, c_dtype, rrms_shape=None, residual=None):
    from x17ai_b200 import kernels
    k = kernels.GemmKernel(cfg)
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.empty(c_shape, dtype=c_dtype, device="cuda")
    rr = torch.empty(rrms_shape, dtype=torch.float32, device="cuda") if rrms_shape else None
    res = torch.from_numpy(residual).cuda() if residual is not None else None
    torch.cuda.synchronize()  # torch fills/copies run on its own stream
    k.launch(stream, ta, tb, c, rrms=rr, residual=res)
    stream.synchronize()
    return c.cpu().numpy(), (rr.cpu().numpy() if rr is not None else None)


@pytest.mark.parametrize("m,k,n", [(128, 128, 256), (200, 256, 512), (384, 1024, 384), (1024, 512, 1280)])
def test_int32_accumulators_exact(stream, m, k, n):
    """int32 accumulation is bit-exact (raw accumulator output)."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(m + k + n)
    a = rng.integers(-127, 128, (m, k), dtype=np.int8)
    b = rng.integers(-127, 128, (n, k), dtype=np.int8)
    cfg = K.GemmConfig(K.DTYPE_INT8, K.DTYPE_INT8, K.DTYPE_I32_RAW, K.EPI_SCALE, k, n)
    got, _ = _run(stream, cfg, a, b, (m, n), torch.int32)
    assert np.array_equal(got, o_gemm.gemm_i32(a, b))


@pytest.mark.parametrize("m,k,n", [(256, 512, 256), (200, 4096, 512)])
def test_scale_epilogue_exact(stream, m, k, n):
    """attn_q_fwd: f32 multiply of exact integers, bit-reproducible (expected.txt:11 has 0 mismatches)."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(1)
    a, b = _rand_i8(rng, (m, k)), _rand_i8(rng, (n, k))
    got, _ = _run(stream, K.attn_q_fwd_config(k, n), a, b, (m, n), torch.int8)
    assert np.array_equal(got, o_gemm.attn_q_fwd(a, b))


@pytest.mark.parametrize("d", [32, 64, 128])
def test_l2norm_kv_epilogue(stream, d):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(d)
    m, k, heads = 256, 512, 4
    n = heads * 2 * d
    a, b = _rand_i8(rng, (m, k)), _rand_i8(rng, (n, k))
    got, rrms = _run(stream, K.attn_kv_fwd_config(k, n, d), a, b, (m, n), torch.int8, rrms_shape=(m, heads))
    ref, ref_rrms = o_gemm.attn_kv_fwd(a, b, d)
    dd = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert dd.max() <= 1 and (dd > 0).mean() <= 1e-4     # reference: 17 / 67M off by one
    assert np.max(np.abs(rrms - ref_rrms) / ref_rrms) < 1e-6  # reference: <= 3 ULP
    # the V half is exact
    v_cols = np.concatenate([np.arange(h * 2 * d + d, (h + 1) * 2 * d) for h in range(heads)])
    assert np.array_equal(got[:, v_cols], ref[:, v_cols])


def test_geglu_epilogue(stream):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(3)
    m, k, f = 384, 1024, 512
    a, b = _rand_i8(rng, (m, k)), _rand_i8(rng, (2 * f, k))
    got, _ = _run(stream, K.ffn_f_fwd_config(k, f), a, b, (m, f), torch.uint8)
    ref = o_gemm.ffn_f_fwd(a, b)
    diff = got != ref
    assert diff.mean() <= 2e-3  # tanh.approx vs libm tanh; reference vs its model: 5e-5 .. see below
    # differing bytes are neighbouring e4m3 codes
    assert np.all(np.abs(got[diff].astype(np.int32) - ref[diff].astype(np.int32)) <= 1) or \
        np.all(np.abs(formats.e4m3_to_f32(got[diff]) - formats.e4m3_to_f32(ref[diff]))
               <= 0.13 * np.abs(formats.e4m3_to_f32(ref[diff])) + 0.02)


@pytest.mark.parametrize("c_dtype", ["e4m3", "i8"])
def test_residual_epilogue_i8_gemm(stream, c_dtype):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(4)
    m, k, dm = 256, 512, 256
    a, b, x = _rand_i8(rng, (m, k)), _rand_i8(rng, (2 * dm, k)), _rand_i8(rng, (m, dm))
    if c_dtype == "e4m3":
        got, _ = _run(stream, K.attn_y_fwd_config(k, dm), a, b, (m, dm), torch.uint8, residual=x)
        ref = o_gemm.attn_y_fwd(a, b, x)
        assert (got != ref).mean() <= 2e-3
    else:
        got, _ = _run(stream, K.ffn_y_fwd_i8_config(k, dm), a, b, (m, dm), torch.int8, residual=x)
        ref = o_gemm.ffn_y_fwd_i8(a, b, x)
        dd = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        assert dd.max() <= 1 and (dd > 0).mean() <= 2e-3


def test_e4m3_x_i8_split_weights(stream):
    """ffn_y_fwd_f8: e4m3 activations x int8 weights on the fp8 tensor cores via the exact
    weight split w = 16*hi + lo; raw f32 accumulators against the float64 sum."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(5)
    m, k, n = 256, 512, 256
    a = formats.f32_to_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    b = _rand_i8(rng, (n, k))
    tb = torch.from_numpy(b).cuda()
    torch.cuda.synchronize()
    split = K.split_i8_weights(stream, tb)
    stream.synchronize()
    sp = split.cpu().numpy()
    hi = formats.hw_e4m3_to_f32(sp[:, :k]); lo = formats.hw_e4m3_to_f32(sp[:, k:])
    assert np.array_equal(hi + lo, b.astype(np.float32))
    cfg = K.GemmConfig(K.DTYPE_E4M3, K.DTYPE_INT8, K.DTYPE_I32_RAW, K.EPI_SCALE, k, n)
    kern = K.GemmKernel(cfg)
    c = torch.empty((m, n), dtype=torch.int32, device="cuda")
    ta = torch.from_numpy(a).cuda()
    torch.cuda.synchronize()
    kern.launch(stream, ta, split, c)
    stream.synchronize()
    got = c.cpu().numpy().view(np.float32)
    ref = o_gemm.gemm_f32_e4m3_i8(a, b)
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.sqrt(k) * np.abs(ref).max()


def test_e4m3_x_e4m3(stream):
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(6)
    m, k, n = 256, 1024, 512
    a = formats.hw_f32_to_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    b = formats.hw_f32_to_e4m3(rng.standard_normal((n, k)).astype(np.float32))
    cfg = K.GemmConfig(K.DTYPE_E4M3, K.DTYPE_E4M3, K.DTYPE_I32_RAW, K.EPI_SCALE, k, n)
    kern = K.GemmKernel(cfg)
    c = torch.empty((m, n), dtype=torch.int32, device="cuda")
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    torch.cuda.synchronize()
    kern.launch(stream, ta, tb, c)
    stream.synchronize()
    got = c.cpu().numpy().view(np.float32)
    ref = o_gemm.gemm_f32_e4m3_e4m3(a, b)
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.sqrt(k) * np.abs(ref).max()


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_block_gemms_against_reference_fixtures(stream, name):
    """Every GEMM of the reference's block (src/main.rs:387-675) on the reference model's own tensors."""
    from x17ai_b200 import kernels as K
    g, c = load_golden(name)
    S, Dm, D, H, F = c["S"], c["Dm"], c["D"], c["H"], c["F"]
    x = g["x_i8"].reshape(S, Dm)
    q, _ = _run(stream, K.attn_q_fwd_config(Dm, H * D), x, g["attn_q_weights_i8"].reshape(H * D, Dm), (S, H * D), torch.int8)
    assert np.array_equal(q, g["q_i8"].reshape(S, H * D))
    kv, rrms = _run(stream, K.attn_kv_fwd_config(Dm, 2 * H * D, D), x, g["attn_kv_weights_i8"].reshape(2 * H * D, Dm),
                    (S, 2 * H * D), torch.int8, rrms_shape=(S, H))
    dd = np.abs(kv.astype(np.int32) - g["kv_i8"].reshape(kv.shape).astype(np.int32))
    assert dd.max() <= 1 and (dd > 0).mean() <= 1e-4
    assert np.max(np.abs(rrms / g["k_rrms_f32"].reshape(rrms.shape) - 1)) < 1e-6
    f, _ = _run(stream, K.ffn_f_fwd_config(Dm, F), x, g["ffn_f_weights_i8"].reshape(2 * F, Dm), (S, F), torch.uint8)
    assert (f != g["ffn_f_f8"].reshape(S, F)).mean() <= 2e-3
    ay, _ = _run(stream, K.attn_y_fwd_config(H * D, Dm), g["attn_out_i8"].reshape(S, H * D),
                 g["attn_y_weights_i8"].reshape(2 * Dm, H * D), (S, Dm), torch.uint8, residual=x)
    assert (ay != g["attn_y_f8"].reshape(S, Dm)).mean() <= 2e-3
    # ffn_y_fwd_f8: e4m3 activations x int8 weights
    wy = torch.from_numpy(g["ffn_y_weights_i8"].reshape(2 * Dm, F)).cuda()
    torch.cuda.synchronize()
    split = K.split_i8_weights(stream, wy)
    kern = K.GemmKernel(K.ffn_y_fwd_f8_config(F, Dm))
    y = torch.empty((S, Dm), dtype=torch.uint8, device="cuda")
    tf, tx = torch.from_numpy(g["ffn_f_f8"].reshape(S, F)).cuda(), torch.from_numpy(x).cuda()
    torch.cuda.synchronize()
    kern.launch(stream, tf, split, y, residual=tx)
    stream.synchronize()
    assert (y.cpu().numpy() != g["ffn_y_f8"].reshape(S, Dm)).mean() <= 2e-3


@pytest.mark.parametrize("d,heads,gate", [(128, 2, 256), (64, 4, 0), (32, 8, 128)])
def test_fused_qkvg_projection(stream, d, heads, gate):
    """One launch equals the reference's two launches (attn_q_fwd, attn_kv_fwd) plus the raw gate columns."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(d + heads + gate)
    m, k = 300, 512
    hd = heads * d
    x = _rand_i8(rng, (m, k))
    wq, wkv, wg = _rand_i8(rng, (hd, k)), _rand_i8(rng, (2 * hd, k)), _rand_i8(rng, (gate, k))
    w = np.concatenate((wq, wkv, wg), axis=0)
    tx, tw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    q = torch.zeros((m, hd), dtype=torch.int8, device="cuda")
    kv = torch.zeros((m, 2 * hd), dtype=torch.int8, device="cuda")
    rr = torch.zeros((m, heads), dtype=torch.float32, device="cuda")
    g = torch.zeros((m, gate), dtype=torch.int8, device="cuda") if gate else None
    torch.cuda.synchronize()
    K.qkvg_fwd_i8(stream, tx, tw, heads, d, q, kv, rr, g)
    stream.synchronize()
    assert np.array_equal(q.cpu().numpy(), o_gemm.attn_q_fwd(x, wq))
    ref_kv, ref_rr = o_gemm.attn_kv_fwd(x, wkv, d)
    dd = np.abs(kv.cpu().numpy().astype(np.int32) - ref_kv.astype(np.int32))
    assert dd.max() <= 1 and (dd > 0).mean() <= 1e-4
    assert np.max(np.abs(rr.cpu().numpy() - ref_rr) / ref_rr) < 1e-6
    if gate:
        assert np.array_equal(g.cpu().numpy(), o_gemm.attn_q_fwd(x, wg))


def test_gemm_argument_errors(stream):
    from x17ai_b200 import X17Error, kernels as K
    with pytest.raises(X17Error, match="multiple of 128"):
        K.GemmKernel(K.GemmConfig(K.DTYPE_INT8, K.DTYPE_INT8, K.DTYPE_INT8, K.EPI_SCALE, 100, 256))
    k = K.GemmKernel(K.attn_q_fwd_config(256, 256))
    a = torch.zeros((128, 256), dtype=torch.int8, device="cuda")
    b = torch.zeros((256, 128), dtype=torch.int8, device="cuda")
    c = torch.zeros((128, 256), dtype=torch.int8, device="cuda")
    with pytest.raises(X17Error, match="gemm input b has 128 columns, but should have 256"):
        k.launch(stream, a, b, c)


def test_ffn_e4m3_weights_and_activations(stream):
    """The FFN with e4m3 weights and e4m3 activations under per-tensor scales (the benchmark description's second
    FFN run; no reference implementation, so the oracle's restatement is the only pin): both GEMMs on the fp8
    tensor path, GeGLU and gated-residual epilogues as in the int8 run."""
    from x17ai_b200 import kernels as K
    rng = np.random.default_rng(21)
    M, Dm, F = 256, 512, 1024
    xv = rng.standard_normal((M, Dm)).astype(np.float32)
    x8, sx = o_gemm.quantize_e4m3_per_tensor(xv)
    x_i8 = formats.quantize_fixedi8(xv)
    wf8, swf = o_gemm.quantize_e4m3_per_tensor(rng.standard_normal((2 * F, Dm)) * 0.02)
    wy8, swy = o_gemm.quantize_e4m3_per_tensor(rng.standard_normal((2 * Dm, F)) * 0.02)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    f = torch.empty((M, F), dtype=torch.uint8, device="cuda")
    y = torch.empty((M, Dm), dtype=torch.uint8, device="cuda")
    tx8, twf, twy, txi = t(x8), t(wf8), t(wy8), t(x_i8)
    torch.cuda.synchronize()
    K.GemmKernel(K.ffn_f_fwd_e4m3_config(Dm, F, sx, swf)).launch(stream, tx8, twf, f)
    K.GemmKernel(K.ffn_y_fwd_e4m3_config(F, Dm, swy)).launch(stream, f, twy, y, residual=txi)
    stream.synchronize()
    f_ref = o_gemm.ffn_f_fwd_e4m3(x8, sx, wf8, swf)
    got_f = f.cpu().numpy()
    assert (got_f != f_ref).mean() <= 2e-3
    assert np.abs(formats.e4m3_to_f32(got_f)).mean() > 0.01    # the scales put the activations in e4m3's range
    y_ref = o_gemm.ffn_y_fwd_e4m3(got_f, wy8, swy, x_i8)          # on the tensor the device fed the second GEMM
    assert (y.cpu().numpy() != y_ref).mean() <= 2e-3
