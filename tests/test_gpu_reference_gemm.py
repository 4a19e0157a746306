"""The reference's own GEMM kernels (cuda/gemm_b8.cuh, cuda/gemm_b16.cuh through templates/basic_gemm,
compiled for sm_100a by oracle/build_ref.py) against this repository's tcgen05 GEMM on the fixture
tensors: the five projections of the block with the constants of src/main.rs:387-675.

The reference kernels are launched through this library's driver shim with the grid and argument
order of gemm.rs:591-641, 690-745. Skipped where oracle/_ref has not been built; the reference's
L2-norm writer only compiles for heads of up to 32 columns, so attn_kv exists for one fixture.
"""
import ctypes
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import load_golden, reference_build_missing
from oracle import gemm as o_gemm

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["one_cta", "cta_pair"])
def gemm_tiling(request):
    """Every test runs with both tilings of the GEMM: one CTA per 128 x 256 tile, and clusters of two CTAs on
    256 x 256 tiles (taken for inputs of more than 128 rows whose N is a multiple of 256)."""
    from x17ai_b200 import kernels as K
    K.set_gemm_tiling(K.GEMM_CTA_PAIR if request.param == "cta_pair" else K.GEMM_ONE_CTA)
    yield request.param
    K.set_gemm_tiling()
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def _run_reference(stream, fixture, kind, a, b, c_shape, c_dtype, rrms_shape=None, residual=None):
    from x17ai_b200.kernel_objects import CubinKernel
    d = REF / f"gemm_{kind}_{fixture}"
    if not (d / "kernel.cubin").exists():
        reference_build_missing(f"{kind} kernel for {fixture}")
    meta = json.loads((d / "meta.json").read_text())
    ta, tb = torch.from_numpy(np.ascontiguousarray(a)).cuda(), torch.from_numpy(np.ascontiguousarray(b)).cuda()
    c = torch.zeros(c_shape, dtype=c_dtype, device="cuda")
    rr = torch.zeros(rrms_shape, dtype=torch.float32, device="cuda") if rrms_shape else None
    res = torch.from_numpy(np.ascontiguousarray(residual)).cuda() if residual is not None else None
    torch.cuda.synchronize()
    assert a.shape[0] % meta["M_PER_BLOCK"] == 0 and b.shape[0] % meta["N_PER_BLOCK"] == 0
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    args = [p(ta), ctypes.c_uint64(a.shape[0]), p(tb), ctypes.c_uint64(b.shape[0]), p(c)]
    if rr is not None:
        args.append(p(rr))
    if res is not None:
        args.append(p(res))
    kern = CubinKernel(stream, d)
    kern.launch(stream, (a.shape[0] // meta["M_PER_BLOCK"], b.shape[0] // meta["N_PER_BLOCK"], 1),
                (meta["THREADS_PER_BLOCK"], 1, 1), meta["SMEM_BYTES"], *args)
    stream.synchronize()
    out = c.cpu().numpy(), (rr.cpu().numpy() if rr is not None else None)
    kern.unload()
    return out


def _run_ours(stream, cfg, a, b, c_shape, c_dtype, rrms_shape=None, residual=None, split=False):
    from x17ai_b200 import kernels as K
    k = K.GemmKernel(cfg)
    ta, tb = torch.from_numpy(np.ascontiguousarray(a)).cuda(), torch.from_numpy(np.ascontiguousarray(b)).cuda()
    c = torch.zeros(c_shape, dtype=c_dtype, device="cuda")
    rr = torch.zeros(rrms_shape, dtype=torch.float32, device="cuda") if rrms_shape else None
    res = torch.from_numpy(np.ascontiguousarray(residual)).cuda() if residual is not None else None
    torch.cuda.synchronize()
    if split:
        tb = K.split_i8_weights(stream, tb)
    k.launch(stream, ta, tb, c, rrms=rr, residual=res)
    stream.synchronize()
    return c.cpu().numpy(), (rr.cpu().numpy() if rr is not None else None)


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_block_gemms_against_reference_kernels(stream, name):
    from x17ai_b200 import kernels as K
    g, c = load_golden(name)
    S, Dm, D, H, F = c["S"], c["Dm"], c["D"], c["H"], c["F"]
    hd = H * D
    x = g["x_i8"].reshape(S, Dm)

    # attn_q: int8 GEMM + scale -> FixedI8: the same codes
    wq = g["attn_q_weights_i8"].reshape(hd, Dm)
    ref, _ = _run_reference(stream, name, "attn_q", x, wq, (S, hd), torch.int8)
    got, _ = _run_ours(stream, K.attn_q_fwd_config(Dm, hd), x, wq, (S, hd), torch.int8)
    assert np.array_equal(got, ref)
    assert np.array_equal(ref, o_gemm.attn_q_fwd(x, wq))   # and the restatement reproduces the reference kernel

    # ffn_f: int8 GEMM + GeGLU -> e4m3
    wf = g["ffn_f_weights_i8"].reshape(2 * F, Dm)
    ref, _ = _run_reference(stream, name, "ffn_f", x, wf, (S, F), torch.uint8)
    got, _ = _run_ours(stream, K.ffn_f_fwd_config(Dm, F), x, wf, (S, F), torch.uint8)
    print(name, "ffn_f: ours vs reference kernel", (got != ref).mean(), "oracle vs reference kernel", (o_gemm.ffn_f_fwd(x, wf) != ref).mean())
    assert np.array_equal(got, ref)   # byte for byte

    # attn_y: int8 GEMM + gated residual -> e4m3, on the fixture's attention output
    ao = g["attn_out_i8"].reshape(S, hd)
    wy = g["attn_y_weights_i8"].reshape(2 * Dm, hd)
    ref, _ = _run_reference(stream, name, "attn_y", ao, wy, (S, Dm), torch.uint8, residual=x)
    got, _ = _run_ours(stream, K.attn_y_fwd_config(hd, Dm), ao, wy, (S, Dm), torch.uint8, residual=x)
    print(name, "attn_y: ours vs reference kernel", (got != ref).mean(), "oracle vs reference kernel", (o_gemm.attn_y_fwd(ao, wy, x) != ref).mean())
    assert np.array_equal(got, ref)   # byte for byte

    # ffn_y: e4m3 activations x int8 weights + gated residual -> e4m3 (the reference converts both to
    # bf16 in registers; here the weights are split into two e4m3 planes)
    ff = g["ffn_f_f8"].reshape(S, F)
    wfy = g["ffn_y_weights_i8"].reshape(2 * Dm, F)
    ref, _ = _run_reference(stream, name, "ffn_y", ff, wfy, (S, Dm), torch.uint8, residual=x)
    got, _ = _run_ours(stream, K.ffn_y_fwd_f8_config(F, Dm), ff, wfy, (S, Dm), torch.uint8, residual=x, split=True)
    print(name, "ffn_y: ours vs reference kernel", (got != ref).mean(), "oracle vs reference kernel", (o_gemm.ffn_y_fwd_f8(ff, wfy, x) != ref).mean())
    assert np.array_equal(got, ref)   # byte for byte

    # attn_kv: int8 GEMM + per-head L2 norm of K, scaled V, rrms side output (head_dim 32 only)
    if (REF / f"gemm_attn_kv_{name}" / "kernel.cubin").exists():
        wkv = g["attn_kv_weights_i8"].reshape(2 * hd, Dm)
        ref, ref_rr = _run_reference(stream, name, "attn_kv", x, wkv, (S, 2 * hd), torch.int8, rrms_shape=(S, H))
        got, rr = _run_ours(stream, K.attn_kv_fwd_config(Dm, 2 * hd, D), x, wkv, (S, 2 * hd), torch.int8, rrms_shape=(S, H))
        dd = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        print(name, "attn_kv: codes differing from the reference kernel", (dd > 0).mean(), "max", dd.max())
        assert dd.max() == 0
        assert np.max(np.abs(rr / ref_rr - 1)) < 1e-6
