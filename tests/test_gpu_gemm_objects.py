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
    d = kernel_objects.build_gemm(stream, cfg, name)
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


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_e4m3_x_int8_object_on_fixtures(stream, name):
    """The sixth kernel of the reference's block (ffn_y_fwd_f8, src/main.rs:620-675) as a kernel object: launched
    with the reference's argument list (e4m3 activations, the int8 weights, the FixedI8 residual) after one
    `prepare` launch for those weights, it returns the bytes of the library's entry point, which takes the split
    planes; before `prepare` it computes nothing and says so in its status words."""
    from x17ai_b200 import kernel_objects, kernels as K
    g, c = load_golden(name)
    S, Dm, F = c["S"], c["Dm"], c["F"]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    x, f, wy = t(g["x_i8"].reshape(S, Dm)), t(g["ffn_f_f8"].reshape(S, F)), t(g["ffn_y_weights_i8"].reshape(2 * Dm, F))
    cfg = K.ffn_y_fwd_f8_config(F, Dm)
    want = torch.zeros(S, Dm, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    K.GemmKernel(cfg).launch(stream, f, K.split_i8_weights(stream, wy), want, residual=x)
    stream.synchronize()

    obj = kernel_objects.GemmObject(stream, cfg, f"ffn_y_f8_{name}")
    m = obj.kernel.meta
    p = lambda v: ctypes.c_void_p(v.data_ptr())
    got = torch.full((S, Dm), 7, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    grid = (max(1, S // m["M_PER_BLOCK"]), max(1, 2 * Dm // m["N_PER_BLOCK"]), 1)
    args = (p(f), ctypes.c_uint64(S), p(wy), ctypes.c_uint64(2 * Dm), p(got), p(x))
    # launched cold, as the reference's host would without the set-up launch: refused, nothing written
    obj.kernel.launch(stream, grid, (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"], *args)
    st = obj.kernel.status(stream)
    assert st[0] >> 16 == 15 and st[2] >= 1, st
    assert bool((got == 7).all())
    obj.prepare(stream, wy)
    obj.kernel.launch(stream, grid, (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"], *args)
    assert obj.kernel.status(stream) == [0, 0, 0, 0]
    assert torch.equal(got, want)
    # through the launcher (prepares by itself for a new weight tensor) and again for other weights
    wy2 = t(np.ascontiguousarray(g["ffn_y_weights_i8"].reshape(2 * Dm, F)[::-1]))
    got2, want2 = torch.zeros_like(got), torch.zeros_like(got)
    torch.cuda.synchronize()
    obj.launch(stream, f, wy2, got2, residual=x)
    K.GemmKernel(cfg).launch(stream, f, K.split_i8_weights(stream, wy2), want2, residual=x)
    stream.synchronize()
    assert torch.equal(got2, want2) and obj.kernel.status(stream) == [0, 0, 0, 0]
    obj.kernel.unload()


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


def _launch_attn_object(stream, kern, S, H, tq, tkv, tsk, tsv, tt, out, l, window):
    m = kern.meta
    p = lambda x: ctypes.c_void_p(x.data_ptr() if x is not None else 0)
    heads_per_cta = max(128 // (tq.shape[1] // H), 1)   # attn.rs:438-446
    kern.launch(stream, (S // m["Q_PER_BLOCK"], H // heads_per_cta, 1), (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"],
                ctypes.c_uint64(S), p(tq), p(tkv), p(tsk), p(tsv), p(tt), p(out), p(l), ctypes.c_uint64(window))


@pytest.mark.parametrize("name,S2,W2", [("block_d128_w128", 1024, 256), ("block_d64_w64", 512, 128), ("block_d32_w0", 384, 48)])
def test_attention_object(stream, name, S2, W2):
    """The attention kernel object, launched with the reference's grid and argument list (attn.rs:412-447):
    the bytes of the entry point on the fixture, then again with other buffers, another sequence length and
    window (the maps are patched at every launch), and with a null `l`."""
    from x17ai_b200 import kernel_objects, kernels as K
    g, c = load_golden(name)
    S, D, H, W = c["S"], c["D"], c["H"], c["W"]
    cfg = K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D)
    kern = kernel_objects.CubinKernel(stream, kernel_objects.build_attn(stream, cfg, f"attn_{name}"))
    lib = K.AttnKernel(cfg)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sk, sv, tt = t(g["sinks_k_i8"].reshape(H, D)), t(g["sinks_v_i8"].reshape(H, D)), t(g["attn_temperature_f32"].reshape(H))
    gen = torch.Generator(device="cuda").manual_seed(9)
    codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=gen, device="cuda") * 8.0), -127, 127).to(torch.int8)
    cases = [(S, W, t(g["q_i8"].reshape(S, H * D)), t(g["kv_i8"].reshape(S, 2 * H * D))),
             (S2, W2, codes(S2, H * D), codes(S2, 2 * H * D)),
             (S2, 0, codes(S2, H * D), codes(S2, 2 * H * D))]
    for s_len, win, q, kv in cases:
        out_o = torch.zeros(s_len, H * D, dtype=torch.int8, device="cuda")
        out_l = torch.zeros(s_len, H * D, dtype=torch.int8, device="cuda")
        l_o = torch.zeros(H, s_len, dtype=torch.float32, device="cuda")
        l_l = torch.zeros(H, s_len, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        _launch_attn_object(stream, kern, s_len, H, q, kv, sk, sv, tt, out_o, l_o, win)
        lib.launch(stream, q, kv, sk, sv, tt, out_l, l_l, win)
        stream.synchronize()
        assert torch.equal(out_o, out_l) and torch.equal(l_o, l_l), (s_len, win)
        out_n = torch.zeros_like(out_o)
        torch.cuda.synchronize()
        _launch_attn_object(stream, kern, s_len, H, q, kv, sk, sv, tt, out_n, None, win)
        stream.synchronize()
        assert torch.equal(out_n, out_l)
    kern.unload()


def test_objects_in_the_reference_harness_shape(stream):
    """One sequence of the benchmark's shape through the attention object and the Q projection object with
    the reference's grids: same bytes as the entry points, and the device times next to them."""
    from x17ai_b200 import device, kernel_objects, kernels as K
    H, D, S, W, Dm = 32, 128, 8192, 1024, 4096
    gen = torch.Generator(device="cuda").manual_seed(0)
    codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=gen, device="cuda") * 8.0), -127, 127).to(torch.int8)
    x, wq = codes(S, Dm), codes(H * D, Dm)
    q, kv, sk, sv = codes(S, H * D), codes(S, 2 * H * D), codes(H, D), codes(H, D)
    tt = (0.5 + torch.rand(H, generator=gen, device="cuda")).float()
    acfg = K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D)
    gcfg = K.attn_q_fwd_config(Dm, H * D)
    a_obj = kernel_objects.CubinKernel(stream, kernel_objects.build_attn(stream, acfg, "attn_h32_d128"))
    g_obj = kernel_objects.CubinKernel(stream, kernel_objects.build_gemm(stream, gcfg, "attn_q_4096_4096"))
    a_lib, g_lib = K.AttnKernel(acfg), K.GemmKernel(gcfg)
    out_o, out_l = (torch.zeros(S, H * D, dtype=torch.int8, device="cuda") for _ in range(2))
    q_o, q_l = (torch.zeros(S, H * D, dtype=torch.int8, device="cuda") for _ in range(2))
    torch.cuda.synchronize()
    p = lambda t_: ctypes.c_void_p(t_.data_ptr())
    gm = g_obj.meta

    def run_g_obj():
        g_obj.launch(stream, (S // gm["M_PER_BLOCK"], (H * D) // gm["N_PER_BLOCK"], 1), (gm["THREADS_PER_BLOCK"], 1, 1),
                     gm["SMEM_BYTES"], p(x), ctypes.c_uint64(S), p(wq), ctypes.c_uint64(H * D), p(q_o))

    def timed(fn, n=15):
        """Median device time of single launches (a timer around each, so host pauses between launches do not count)."""
        for _ in range(3):
            fn()
        timers = [device.CudaTimer(stream) for _ in range(n)]
        for tm in timers:
            tm.start()
            fn()
            tm.stop()
        stream.synchronize()
        times = sorted(tm.elapsed_seconds() for tm in timers)
        for tm in timers:
            tm.destroy()
        return times[n // 2]

    t_ao = timed(lambda: _launch_attn_object(stream, a_obj, S, H, q, kv, sk, sv, tt, out_o, None, W))
    t_al = timed(lambda: a_lib.launch(stream, q, kv, sk, sv, tt, out_l, None, W))
    t_go = timed(run_g_obj)
    t_gl = timed(lambda: g_lib.launch(stream, x, wq, q_l))
    print(f"attention: object {t_ao * 1e3:.3f} ms, entry point {t_al * 1e3:.3f} ms; "
          f"Q projection: object {t_go * 1e3:.3f} ms, entry point {t_gl * 1e3:.3f} ms")
    assert torch.equal(out_o, out_l) and torch.equal(q_o, q_l)
    assert t_ao < 1.25 * t_al and t_go < 1.5 * t_gl
    a_obj.unload()
    g_obj.unload()
