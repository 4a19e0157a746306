"""GEMM kernel objects (kernel.cubin + meta.json, x17ai_b200/kernel_objects.py build_gemm): built for the block's
int8 projections on the fixture shapes, loaded through the driver shim and launched exactly as the reference's
host launches its own GEMM cubins (grid (c_rows / M_PER_BLOCK, raw_cols / N_PER_BLOCK, 1), arguments
(a, a_rows, b, b_rows, c[, rrms][, residual]), gemm.rs:591-641, 690-745). The object must return the bytes
of the library's entry point for the same configuration, and the fixtures' tensors where those are exact."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu


def _launch_object(stream, cfg, name, a, b, c, rrms=None, residual=None, grid=None):
    from x17ai_b200 import kernel_objects
    d = kernel_objects.build_gemm(cfg, name)
    kern = kernel_objects.CubinKernel(stream, d)
    m = kern.meta
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    args = [p(a), ctypes.c_uint64(a.shape[0]), p(b), ctypes.c_uint64(b.shape[0]), p(c)]
    if rrms is not None:
        args.append(p(rrms))
    if residual is not None:
        args.append(p(residual))
    if grid is None:
        grid = (max(1, a.shape[0] // m["M_PER_BLOCK"]), max(1, b.shape[0] // m["N_PER_BLOCK"]), 1)
    kern.launch(stream, grid, (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"], *args)
    stream.synchronize()
    kern.unload()


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128"])
def test_gemm_objects_on_fixtures(stream, name):
    from x17ai_b200 import kernels as K
    g, c = load_golden(name)
    S, Dm, D, H, F = c["S"], c["Dm"], c["D"], c["H"], c["F"]
    hd = H * D
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    x = t(g["x_i8"].reshape(S, Dm))
    z = lambda *s, dtype=torch.int8: torch.zeros(*s, dtype=dtype, device="cuda")

    def both(cfg, tag, a, b, c_shape, c_dtype, rrms_shape=None, residual=None):
        c_obj, c_lib = z(*c_shape, dtype=c_dtype), z(*c_shape, dtype=c_dtype)
        r_obj = z(*rrms_shape, dtype=torch.float32) if rrms_shape else None
        r_lib = z(*rrms_shape, dtype=torch.float32) if rrms_shape else None
        torch.cuda.synchronize()
        _launch_object(stream, cfg, f"{tag}_{name}", a, b, c_obj, rrms=r_obj, residual=residual)
        K.GemmKernel(cfg).launch(stream, a, b, c_lib, rrms=r_lib, residual=residual)
        stream.synchronize()
        assert torch.equal(c_obj, c_lib), tag
        if r_obj is not None:
            assert torch.equal(r_obj, r_lib), tag
        return c_obj

    wq = t(g["attn_q_weights_i8"].reshape(hd, Dm))
    q = both(K.attn_q_fwd_config(Dm, hd), "attn_q", x, wq, (S, hd), torch.int8)
    assert np.array_equal(q.cpu().numpy(), g["q_i8"].reshape(S, hd))   # the model's own tensor, exact
    wkv = t(g["attn_kv_weights_i8"].reshape(2 * hd, Dm))
    both(K.attn_kv_fwd_config(Dm, 2 * hd, D), "attn_kv", x, wkv, (S, 2 * hd), torch.int8, rrms_shape=(S, H))
    wf = t(g["ffn_f_weights_i8"].reshape(2 * F, Dm))
    both(K.ffn_f_fwd_config(Dm, F), "ffn_f", x, wf, (S, F), torch.uint8)
    ao = t(g["attn_out_i8"].reshape(S, hd))
    wy = t(g["attn_y_weights_i8"].reshape(2 * Dm, hd))
    both(K.attn_y_fwd_config(hd, Dm), "attn_y", ao, wy, (S, Dm), torch.uint8, residual=x)


def test_gemm_object_any_grid_and_reuse(stream):
    """The object strides over its tiles by the number of CTAs it was launched with: a single CTA, the
    reference's grid and a grid larger than the tile count give the same bytes; a second launch with other
    pointers and another row count uses the same cubin (the maps are patched at every launch)."""
    from x17ai_b200 import kernels as K
    gen = torch.Generator(device="cuda").manual_seed(5)
    codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=gen, device="cuda") * 8.0), -127, 127).to(torch.int8)
    M, Kd, N = 640, 512, 1024
    cfg = K.attn_q_fwd_config(Kd, N)
    a, b = codes(M, Kd), codes(N, Kd)
    want = torch.zeros(M, N, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    K.GemmKernel(cfg).launch(stream, a, b, want)
    stream.synchronize()
    for grid in ((1, 1, 1), None, (7, 5, 1)):
        got = torch.zeros(M, N, dtype=torch.int8, device="cuda")
        torch.cuda.synchronize()
        _launch_object(stream, cfg, "any_grid", a, b, got, grid=grid)
        assert torch.equal(got, want), grid
    a2 = codes(200, Kd)   # ragged row count, other buffers
    want2 = torch.zeros(200, N, dtype=torch.int8, device="cuda")
    got2 = torch.zeros(200, N, dtype=torch.int8, device="cuda")
    torch.cuda.synchronize()
    K.GemmKernel(cfg).launch(stream, a2, b, want2)
    _launch_object(stream, cfg, "any_grid", a2, b, got2, grid=(2, 4, 1))
    stream.synchronize()
    assert torch.equal(got2, want2)
