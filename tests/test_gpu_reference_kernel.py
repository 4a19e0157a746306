"""The reference's own attention kernel (cuda/attn_fwd_i8.cuh, rendered and compiled for sm_100a by
oracle/build_ref.py into oracle/_ref/) run on the same GPU, on the same inputs:

* it pins the numpy restatement: `oracle.attn` with the reference's 16-key running maximum
  (`kv_tile=16`) must reproduce the reference kernel's codes;
* it is the direct parity check of this repository's kernel against the reference implementation;
* it is launched through this library's own driver shim (`x17ai_cuda_load_module`, `get_kernel`,
  `launch_kernel`) exactly as the reference's Rust host launches it (attn.rs:353-447), which makes
  the shim's drop-in claim concrete.

Skipped where oracle/_ref has not been built (no checkout of the reference at build time).
"""
import ctypes
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import code_hist, load_golden, reference_build_missing
from oracle import attn as o_attn, formats

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def _ref_dir(H, D):
    d = REF / f"attn_h{H}_d{D}"
    if not (d / "kernel.cubin").exists():
        reference_build_missing(f"attention kernel for {H} heads x {D}")
    return d


def _run_reference(stream, q, kv, sk, sv, temp, H, D, window):
    """One sequence through the reference's cubin: grid (seq / Q_PER_BLOCK, head groups), attn.rs:425-447."""
    from x17ai_b200.kernel_objects import CubinKernel
    d = _ref_dir(H, D)
    meta = json.loads((d / "meta.json").read_text())
    S = q.shape[0]
    assert S % meta["Q_PER_BLOCK"] == 0
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tq, tkv, tsk, tsv, tt = t(q), t(kv), t(sk), t(sv), t(temp)
    out = torch.zeros((S, H * D), dtype=torch.int8, device="cuda")
    l = torch.zeros((H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern = CubinKernel(stream, d)
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    kern.launch(stream, (S // meta["Q_PER_BLOCK"], H // meta["heads_per_kernel"], 1), (meta["THREADS_PER_BLOCK"], 1, 1),
                meta["SMEM_BYTES"], ctypes.c_uint64(S), p(tq), p(tkv), p(tsk), p(tsv), p(tt), p(out), p(l),
                ctypes.c_uint64(window))
    stream.synchronize()
    res = out.cpu().numpy(), l.cpu().numpy()
    kern.unload()
    return res


def _run_ours(stream, q, kv, sk, sv, temp, H, D, window):
    from x17ai_b200 import kernels as K
    S = q.shape[0]
    kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tq, tkv, tsk, tsv, tt = t(q), t(kv), t(sk), t(sv), t(temp)
    out = torch.zeros((S, H * D), dtype=torch.int8, device="cuda")
    l = torch.zeros((H, S), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    kern.launch(stream, tq, tkv, tsk, tsv, tt, out, l, window)
    stream.synchronize()
    return out.cpu().numpy(), l.cpu().numpy()


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_reference_kernel_on_fixtures(stream, name):
    g, c = load_golden(name)
    S, H, D, W = c["S"], c["H"], c["D"], c["W"]
    q, kv = g["q_i8"].reshape(S, H * D), g["kv_i8"].reshape(S, 2 * H * D)
    sk, sv = g["sinks_k_i8"].reshape(H, D), g["sinks_v_i8"].reshape(H, D)
    temp = g["attn_temperature_f32"].reshape(H)
    ref_out, ref_l = _run_reference(stream, q, kv, sk, sv, temp, H, D, W)

    # the restatement with the reference's schedule reproduces the reference kernel
    o16, l16 = o_attn.attn_fwd_i8(q, kv, sk, sv, temp, W, H, D, kv_tile=16)
    hist = code_hist(ref_out, o16)
    print(name, "reference kernel vs oracle(kv_tile=16):", hist[:4], "of", ref_out.size)
    assert hist[1:].sum() == 0   # bit for bit
    assert np.max(np.abs(ref_l - l16)) < 1e-3

    # the reference kernel against the reference's float64 model: what expected.txt:65-99 records
    hist = code_hist(ref_out, g["attn_out_i8"].reshape(S, H * D))
    print(name, "reference kernel vs float64 model:", hist[:7] / ref_out.size)
    assert hist[1:].sum() / ref_out.size <= 0.40 and hist[6:].sum() == 0

    # this repository's kernel against the reference kernel
    out, l = _run_ours(stream, q, kv, sk, sv, temp, H, D, W)
    hist = code_hist(out, ref_out)
    print(name, "this kernel vs reference kernel:", hist[:4], "of", out.size)
    mine = code_hist(out, g["attn_out_i8"].reshape(S, H * D))
    print(name, "this kernel vs float64 model:", mine[:7] / out.size)
    # not further from the reference's float64 model than the reference's own kernel is
    theirs = code_hist(ref_out, g["attn_out_i8"].reshape(S, H * D))
    assert mine[2:].sum() <= theirs[2:].sum() * 1.05 + 8
    assert hist[2:].sum() == 0 and hist[1] / out.size <= 0.03
    assert np.max(np.abs(l - ref_l)) < 1e-3


@pytest.mark.parametrize("H,D,S,W", [(4, 64, 512, 128), (2, 128, 1024, 256), (4, 32, 256, 0)])
def test_reference_kernel_on_seeded_inputs(stream, H, D, S, W):
    """Seeded inputs of the benchmark's distribution, longer than the fixtures: the window slides."""
    rng = np.random.default_rng(100 + D)
    q = formats.quantize_fixedi8(rng.standard_normal((S, H * D)))
    k = rng.standard_normal((S, H, D))
    k = k / np.sqrt((k ** 2).mean(-1, keepdims=True))
    v = rng.standard_normal((S, H, D)) * 1.3
    kv = formats.quantize_fixedi8(np.concatenate((k, v), axis=-1).reshape(S, H * 2 * D))
    sk = formats.quantize_fixedi8(rng.standard_normal((H, D)))
    sv = formats.quantize_fixedi8(rng.standard_normal((H, D)) * 1.3)
    temp = (0.5 + rng.random(H)).astype(np.float32)
    ref_out, ref_l = _run_reference(stream, q, kv, sk, sv, temp, H, D, W)
    o16, l16 = o_attn.attn_fwd_i8(q, kv, sk, sv, temp, W, H, D, kv_tile=16)
    hist = code_hist(ref_out, o16)
    print("reference kernel vs oracle(kv_tile=16):", hist[:4], "of", ref_out.size)
    assert hist[2:].sum() == 0 and hist[1] / ref_out.size <= 2e-3
    out, l = _run_ours(stream, q, kv, sk, sv, temp, H, D, W)
    hist = code_hist(out, ref_out)
    assert hist[2:].sum() == 0 and hist[1] / out.size <= 0.03
    assert np.max(np.abs(l - ref_l)) < 1e-3


def test_faster_than_the_reference_kernel(stream):
    """One sequence of the benchmark's shape (32 heads x 128, 8192 tokens, window 1024): this kernel
    must beat the reference's own kernel recompiled for sm_100a, timed the same way on the same data."""
    from x17ai_b200 import device, kernels as K
    from x17ai_b200.kernel_objects import CubinKernel
    H, D, S, W = 32, 128, 8192, 1024
    d = _ref_dir(H, D)
    meta = json.loads((d / "meta.json").read_text())
    g = torch.Generator(device="cuda").manual_seed(0)
    codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=g, device="cuda") * 8.0), -127, 127).to(torch.int8)
    q, kv, sk, sv = codes(S, H * D), codes(S, 2 * H * D), codes(H, D), codes(H, D)
    temp = (0.5 + torch.rand(H, generator=g, device="cuda")).float()
    out_ref = torch.zeros(S, H * D, dtype=torch.int8, device="cuda")
    out = torch.zeros(S, H * D, dtype=torch.int8, device="cuda")
    l = torch.zeros(H, S, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ref = CubinKernel(stream, d)
    ours = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
    p = lambda x: ctypes.c_void_p(x.data_ptr())

    def run_ref():
        ref.launch(stream, (S // meta["Q_PER_BLOCK"], H // meta["heads_per_kernel"], 1), (meta["THREADS_PER_BLOCK"], 1, 1),
                   meta["SMEM_BYTES"], ctypes.c_uint64(S), p(q), p(kv), p(sk), p(sv), p(temp), p(out_ref), p(l),
                   ctypes.c_uint64(W))

    def run_ours():
        ours.launch(stream, q, kv, sk, sv, temp, out, l, W)

    def timed(fn, n=11):
        """Median device time of single launches (a timer around each: host pauses between launches do not count)."""
        for _ in range(3):
            fn()
        timers = [device.CudaTimer(stream) for _ in range(n)]
        for t in timers:
            t.start()
            fn()
            t.stop()
        stream.synchronize()
        times = sorted(t.elapsed_seconds() for t in timers)
        for t in timers:
            t.destroy()
        return times[n // 2]

    t_ref, t_ours = timed(run_ref), timed(run_ours)
    ops = o_attn.attn_ops(1, H, D, S, W)
    print(f"reference kernel {ops / t_ref / 1e12:.1f} TOPS ({t_ref * 1e3:.3f} ms), this kernel {ops / t_ours / 1e12:.1f} TOPS "
          f"({t_ours * 1e3:.3f} ms), ratio {t_ref / t_ours:.2f}")
    hist = code_hist(out.cpu().numpy(), out_ref.cpu().numpy())
    assert hist[2:].sum() == 0 and hist[1] / out.numel() <= 0.03
    assert t_ours < t_ref
    ref.unload()
