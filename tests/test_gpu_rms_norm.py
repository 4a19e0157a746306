"""RMSNorm through the C ABI against the oracle (rms_norm.cu:55-113 restated in oracle/rms_norm.py)."""
import numpy as np
import pytest
import torch

from oracle import formats, rms_norm as o_rms

pytestmark = pytest.mark.gpu


def _legal_e4m3(rng, shape):
    x = rng.standard_normal(shape).astype(np.float32)
    return formats.f32_to_e4m3(x)


@pytest.mark.parametrize("rows,cols", [(1, 512), (37, 2048), (256, 4096), (9, 8192), (5, 16)])
def test_rms_norm_e4m3_fixed(stream, rows, cols):
    from x17ai_b200 import kernels
    rng = np.random.default_rng(rows * 131 + cols)
    x = _legal_e4m3(rng, (rows, cols))
    inp = torch.from_numpy(x).cuda()
    out = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    kernels.rms_norm(stream, kernels.RMS_E4M3_FIXED, inp, out)
    stream.synchronize()
    ref = o_rms.rms_norm_e4m3_i8(x)
    got = out.cpu().numpy()
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    # the GPU sums squares in f32 and uses rsqrt.approx: at most one code off, on rounding ties only
    assert d.max() <= 1 and (d > 0).mean() <= 2e-3


@pytest.mark.parametrize("rows,cols", [(3, 512), (64, 4096)])
def test_rms_norm_bf16_modes(stream, rows, cols):
    from x17ai_b200 import kernels
    rng = np.random.default_rng(7)
    xt = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).to(torch.bfloat16)
    bits = xt.view(torch.int16).numpy().view(np.uint16)
    inp = xt.cuda()
    out = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    kernels.rms_norm(stream, kernels.RMS_BF16_FIXED, inp, out)
    stream.synchronize()
    d = np.abs(out.cpu().numpy().astype(np.int32) - o_rms.rms_norm_bf16_i8_fixed(bits).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() <= 2e-3
    scale = torch.empty((rows,), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kernels.rms_norm(stream, kernels.RMS_BF16_ROWSCALE, inp, out, row_scale=scale)
    stream.synchronize()
    ref_codes, ref_scale = o_rms.rms_norm_bf16_i8_rowscale(bits)
    assert np.allclose(scale.cpu().numpy(), ref_scale, rtol=1e-5)
    d = np.abs(out.cpu().numpy().astype(np.int32) - ref_codes.astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() <= 5e-3
    assert np.abs(out.cpu().numpy()).max() == 127


def test_rms_norm_rejects_bad_width(stream):
    from x17ai_b200 import X17Error, kernels
    inp = torch.zeros((4, 24), dtype=torch.uint8, device="cuda")
    out = torch.empty((4, 24), dtype=torch.int8, device="cuda")
    with pytest.raises(X17Error, match="multiple of 16"):
        kernels.rms_norm(stream, kernels.RMS_E4M3_FIXED, inp, out)
