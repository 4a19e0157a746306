#!/usr/bin/env python3
"""Benchmark of the quantized block-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (N = 1): the prefill-scale int8 sliding-window attention forward
(batch 8, 32 heads, seq 8192, head_dim 128, window 1024), one launch over the whole batch per
step, synthetic seeded inputs.  With N > 1 (torchrun, one rank per GPU) every rank runs the same
per-GPU workload on its own shard of an N-times larger batch: (batch, head) units are
independent, so there is no data-path collective (weak scaling).

One JSON line on stdout (rank 0).  `value` is measured with inputs resident in HBM; `e2e` goes
through the C ABI with host buffers (pinned), host->device and device->host copies inside the
timed region.  `roofline.achieved` uses the average kernel duration from CUDA events recorded on
the launching stream.  `--impl reference` times the CPU restatement of the reference's algorithm
(oracle/) on the host cores on a bounded sample of the same workload.

Other workloads (`--workload ffn_i8 | ffn_f8 | decode | rms_norm | qkv`) print the same kind of
line for the other kernels of the path.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


# ------------------------------------------------------------------------------------------------
# helpers

def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken between the wall-clock times t_begin and t_end (all if None)."""
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        power = []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if t_begin is not None and not (t_begin - 0.05 <= ts <= t_end + 0.05):
                    continue
                sm.append(float(parts[1])); mx.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def measured_traffic(workload, units):
    """DRAM bytes per launch from the committed ncu summary (profiles/traffic.json): bytes per unit of a
    captured smaller case of the same kernel, scaled to this launch by the units it processes."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.exists():
        return None
    d = json.loads(p.read_text()).get(workload)
    if not d:
        return None
    return d["dram_bytes_per_unit"] * units


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------------
# workloads: each returns an object with .step(), .e2e_step(), .ops, .bytes, .units ...

class AttnPrefill:
    """configs[1]: B8 H32 S8192 D128 W1024, one batched launch per step."""
    name = "int8_sliding_window_attention_prefill"
    bound = "tensor"
    dtype = "s8"

    def __init__(self, stream, device, B=8, H=32, S=8192, D=128, W=1024, seed=0):
        import torch
        from oracle import attn as o_attn
        from x17ai_b200 import kernels as K
        self.torch, self.stream = torch, stream
        self.B, self.H, self.S, self.D, self.W = B, H, S, D, W
        g = torch.Generator(device=device).manual_seed(seed)
        # N(0,1) values -> FixedI8 codes (x8, clamp +-127); K rows unit-RMS by construction of N(0,1)
        def codes(*shape, std=1.0):
            return torch.clamp(torch.round(torch.randn(*shape, generator=g, device=device) * (8.0 * std)), -127, 127).to(torch.int8)
        self.q = codes(B, S, H * D)
        self.kv = codes(B, S, H * 2 * D)
        self.kv.view(B, S, H, 2, D)[:, :, :, 1, :] = codes(B, S, H, D, std=1.3)
        self.sink_k = codes(H, D)
        self.sink_v = codes(H, D, std=1.3)
        self.temp = (0.5 + torch.rand(H, generator=g, device=device)).float()
        self.out = torch.empty(B, S, H * D, dtype=torch.int8, device=device)
        self.l = torch.empty(B, H, S, dtype=torch.float32, device=device)
        self.kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
        self.ops = o_attn.attn_ops(B, H, D, S, W)
        self.ref_ops = self.kern.config.n_ops(S, W) * B
        self.tokens = B * S
        self.units = B * H  # (sequence, head) units of this S, D, W
        self.alg_bytes = self.q.numel() + self.kv.numel() + self.out.numel() + self.l.numel() * 4
        self.launches_per_step = 1
        self.config = {"workload": "configs[1] int8 sliding-window attention prefill", "batch": B, "n_heads": H,
                       "seq_len": S, "head_dim": D, "window": W,
                       "l2": "inputs (q+kv+out = %.0f MB) larger than the 126 MB L2" % (self.alg_bytes / 1e6)}
        torch.cuda.synchronize()

    def step(self):
        self.kern.launch(self.stream, self.q, self.kv, self.sink_k, self.sink_v, self.temp, self.out, self.l, self.W)

    def host_buffers(self):
        t = self.torch
        self.h_q = self.q.cpu().pin_memory(); self.h_kv = self.kv.cpu().pin_memory()
        self.h_out = t.empty_like(self.out, device="cpu").pin_memory()
        self.h2d = self.h_q.numel() + self.h_kv.numel()
        self.d2h = self.h_out.numel()

    def e2e_step(self):
        # sequences are independent: three streams keep the upload of one sequence, the kernel of
        # the previous one and the download of the one before that in flight together
        if not hasattr(self, "e2e_streams"):
            from x17ai_b200 import device
            self.e2e_streams = [self.stream] + [device.CudaStream(self.q.device.index) for _ in range(2)]
        self.kern.launch_from_host(self.e2e_streams, self.h_q, self.h_kv, self.sink_k, self.sink_v, self.temp,
                                   self.q, self.kv, self.out, self.h_out, self.l, self.W)

    def e2e_sync(self):
        for st in getattr(self, "e2e_streams", [self.stream]):
            st.synchronize()

    def cpu_sample(self, seconds_hint=15.0):
        """Oracle on a bounded sample: whole sequences of a few heads."""
        from oracle import attn as o_attn
        S, D, W = self.S, self.D, self.W
        rng = np.random.default_rng(0)
        mk = lambda *s: np.clip(np.rint(rng.standard_normal(s) * 8), -127, 127).astype(np.int8)
        heads, t0, done_ops = 0, time.perf_counter(), 0.0
        while True:
            o_attn.attn_head(mk(S, D), mk(S, D), mk(S, D), mk(D), mk(D), 1.0, W, kv_tile=16)
            heads += 1
            done_ops += o_attn.attn_ops(1, 1, D, S, W)
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        return done_ops / dt, f"{heads} (sequence, head) units of S={S} D={D} W={W}, oracle kv_tile=16, {dt:.1f} s"


class AttnPvFp8(AttnPrefill):
    """configs[2]: the fp8 P.V variant on the prefill shape: int8 Q.K^T, P as e4m3, V as e4m3 with a per-head
    f32 scale, f32 accumulation, bf16 output."""
    name = "attention_pv_fp8_prefill"
    dtype = "s8/e4m3"

    def __init__(self, stream, device, B=8, H=32, S=8192, D=128, W=1024, seed=0):
        super().__init__(stream, device, B, H, S, D, W, seed)
        torch = self.torch
        g = torch.Generator(device=device).manual_seed(seed + 1)
        # V and the sink values as e4m3 bytes of N(0,1) values (OCP e4m3fn, the hardware's format)
        v = torch.randn(B, S, H, D, generator=g, device=device).to(torch.float8_e4m3fn).view(torch.int8)
        self.kv.view(B, S, H, 2, D)[:, :, :, 1, :] = v
        self.sink_v8 = torch.randn(H, D, generator=g, device=device).to(torch.float8_e4m3fn).view(torch.uint8)
        self.v_scale = (0.25 + torch.rand(H, generator=g, device=device)).float()
        self.out = torch.empty(B, S, H * D, dtype=torch.bfloat16, device=device)
        self.alg_bytes = self.q.numel() + self.kv.numel() + 2 * self.out.numel() + self.l.numel() * 4
        self.config = dict(self.config, workload="configs[2] attention with fp8 P.V (e4m3 P and V, bf16 out)")
        torch.cuda.synchronize()

    def step(self):
        self.kern.launch_pv_fp8(self.stream, self.q, self.kv, self.sink_k, self.sink_v8, self.temp, self.v_scale,
                                self.out, self.l, self.W)

    def host_buffers(self):
        t = self.torch
        self.h_q = self.q.cpu().pin_memory(); self.h_kv = self.kv.cpu().pin_memory()
        self.h_out = t.empty_like(self.out, device="cpu").pin_memory()
        self.h2d = self.h_q.numel() + self.h_kv.numel()
        self.d2h = self.h_out.numel() * 2

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_q.data_ptr(), self.q.data_ptr(), 0, self.h_q.numel())
        s.upload(self.h_kv.data_ptr(), self.kv.data_ptr(), 0, self.h_kv.numel())
        self.step()
        s.download(self.out.data_ptr(), self.h_out.data_ptr(), 0, self.h_out.numel() * 2)

    def e2e_sync(self):
        self.stream.synchronize()


class Ffn:
    """configs[3]: gated FFN on 16384 tokens, d_model 4096, hidden 14336 (reference GeGLU form)."""
    bound = "tensor"

    def __init__(self, stream, device, f8=False, M=16384, Dm=4096, F=14336, seed=0):
        import torch
        from x17ai_b200 import kernels as K
        self.torch, self.stream, self.f8 = torch, stream, f8
        self.name = "ffn_fwd_f8" if f8 else "ffn_fwd_i8"
        self.dtype = "e4m3" if f8 else "s8"
        g = torch.Generator(device=device).manual_seed(seed)
        codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=g, device=device) * 8.0), -127, 127).to(torch.int8)
        self.x = codes(M, Dm)
        self.wf = codes(2 * F, Dm)
        self.wy = codes(2 * Dm, F)
        self.f = torch.empty(M, F, dtype=torch.uint8, device=device)
        self.y = torch.empty(M, Dm, dtype=torch.uint8, device=device)
        self.k_f = K.GemmKernel(K.ffn_f_fwd_config(Dm, F))
        torch.cuda.synchronize()
        if f8:   # reference-faithful: e4m3 activations x int8 weights (ffn_y_fwd_f8)
            self.wy_split = K.split_i8_weights(stream, self.wy)
            self.k_y = K.GemmKernel(K.ffn_y_fwd_f8_config(F, Dm))
        else:    # int8 x int8 (ffn_y_fwd_i8): f re-quantised is not part of the reference; use f bytes as i8
            self.k_y = K.GemmKernel(K.ffn_y_fwd_i8_config(F, Dm, c_dtype=K.DTYPE_E4M3))
        stream.synchronize()
        self.M, self.Dm, self.F = M, Dm, F
        self.ops = 2.0 * M * Dm * 2 * F + 2.0 * M * F * 2 * Dm
        self.tokens = M
        self.units = M  # token rows
        self.alg_bytes = M * Dm + 2 * F * Dm + M * F * 2 + 2 * Dm * F + M * Dm * 2
        self.launches_per_step = 2
        self.config = {"workload": "configs[3] gated FFN (GeGLU -> e4m3, gated residual)", "tokens": M, "d_model": Dm,
                       "hidden": F, "ffn_y": "e4m3 x int8 (split weights, kind::f8f6f4)" if f8 else "int8 x int8 (kind::i8)",
                       "l2": "weights + activations (%.0f MB) larger than the 126 MB L2" % (self.alg_bytes / 1e6)}

    def step(self):
        self.k_f.launch(self.stream, self.x, self.wf, self.f)
        if self.f8:
            self.k_y.launch(self.stream, self.f, self.wy_split, self.y, residual=self.x)
        else:
            self.k_y.launch(self.stream, self.f.view(self.torch.int8), self.wy, self.y, residual=self.x)

    def host_buffers(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_y = t.empty_like(self.y, device="cpu").pin_memory()
        self.h2d, self.d2h = self.h_x.numel(), self.h_y.numel()

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_x.data_ptr(), self.x.data_ptr(), 0, self.h_x.numel())
        self.step()
        s.download(self.y.data_ptr(), self.h_y.data_ptr(), 0, self.h_y.numel())

    def cpu_sample(self, seconds_hint=15.0):
        from oracle import gemm as o_gemm
        rng = np.random.default_rng(0)
        rows = 256
        mk = lambda *s: np.clip(np.rint(rng.standard_normal(s) * 8), -127, 127).astype(np.int8)
        x, wf, wy = mk(rows, self.Dm), mk(2 * self.F, self.Dm), mk(2 * self.Dm, self.F)
        t0, n = time.perf_counter(), 0
        while True:
            f = o_gemm.ffn_f_fwd(x, wf)
            o_gemm.ffn_y_fwd_f8(f, wy, x)
            n += 1
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        ops = n * (2.0 * rows * self.Dm * 2 * self.F + 2.0 * rows * self.F * 2 * self.Dm)
        return ops / dt, f"{n} x {rows} token rows of the same FFN, {dt:.1f} s"


class Qkvg:
    """The fused Q / KV projection (one launch for attn_q_fwd + attn_kv_fwd of src/main.rs:387-491) at the
    benchmark's model shape: scale -> FixedI8 for Q and V, per-head L2 norm for K, rrms side output."""
    name = "qkvg_fwd_i8"
    bound = "tensor"
    dtype = "s8"

    def __init__(self, stream, device, M=16384, Dm=4096, H=32, D=128, seed=0):
        import torch
        from x17ai_b200 import kernels as K
        self.torch, self.stream, self.K = torch, stream, K
        g = torch.Generator(device=device).manual_seed(seed)
        codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=g, device=device) * 8.0), -127, 127).to(torch.int8)
        hd = H * D
        self.x, self.w = codes(M, Dm), codes(3 * hd, Dm)
        self.q = torch.empty(M, hd, dtype=torch.int8, device=device)
        self.kv = torch.empty(M, 2 * hd, dtype=torch.int8, device=device)
        self.rrms = torch.empty(M, H, dtype=torch.float32, device=device)
        self.H, self.D, self.M, self.Dm = H, D, M, Dm
        self.ops = 2.0 * M * Dm * 3 * hd
        self.tokens = M
        self.units = M
        self.alg_bytes = M * Dm + 3 * hd * Dm + 3 * M * hd + 4 * M * H
        self.launches_per_step = 1
        self.config = {"workload": "fused Q/KV projection", "tokens": M, "d_model": Dm, "n_heads": H, "head_dim": D,
                       "l2": "x + weights + outputs %.0f MB larger than the 126 MB L2" % (self.alg_bytes / 1e6)}
        torch.cuda.synchronize()

    def step(self):
        self.K.qkvg_fwd_i8(self.stream, self.x, self.w, self.H, self.D, self.q, self.kv, self.rrms)

    def host_buffers(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_q = t.empty_like(self.q, device="cpu").pin_memory()
        self.h_kv = t.empty_like(self.kv, device="cpu").pin_memory()
        self.h2d, self.d2h = self.h_x.numel(), self.h_q.numel() + self.h_kv.numel()

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_x.data_ptr(), self.x.data_ptr(), 0, self.h_x.numel())
        self.step()
        s.download(self.q.data_ptr(), self.h_q.data_ptr(), 0, self.h_q.numel())
        s.download(self.kv.data_ptr(), self.h_kv.data_ptr(), 0, self.h_kv.numel())

    def cpu_sample(self, seconds_hint=10.0):
        from oracle import gemm as o_gemm
        H, D, Dm = self.H, self.D, self.Dm
        rng = np.random.default_rng(0)
        mk = lambda *s: np.clip(np.rint(rng.standard_normal(s) * 8), -127, 127).astype(np.int8)
        x, wq, wkv = mk(512, Dm), mk(H * D, Dm), mk(2 * H * D, Dm)
        t0, n = time.perf_counter(), 0
        while True:
            o_gemm.attn_q_fwd(x, wq)
            o_gemm.attn_kv_fwd(x, wkv, D)
            n += 1
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        return n * 2.0 * 512 * Dm * 3 * H * D / dt, f"{n} x 512 token rows through both projections, {dt:.1f} s"


class Decode:
    """configs[4] tail: batch 256, one new token each, int8 KV cache of 4096 tokens, 32 heads x 128."""
    name = "int8_decode_attention"
    bound = "hbm"
    dtype = "s8"

    def __init__(self, stream, device, B=256, H=32, D=128, T=4096, W=4096, seed=0):
        import torch
        from x17ai_b200 import kernels as K
        self.torch, self.stream = torch, stream
        self.B, self.H, self.D, self.T, self.W = B, H, D, T, W
        g = torch.Generator(device=device).manual_seed(seed)
        self.kv = torch.randint(-40, 41, (B, T, H * 2 * D), generator=g, device=device, dtype=torch.int8)
        self.q = torch.randint(-30, 31, (B, H * D), generator=g, device=device, dtype=torch.int8)
        self.sink_k = torch.randint(-20, 21, (H, D), generator=g, device=device, dtype=torch.int8)
        self.sink_v = torch.randint(-20, 21, (H, D), generator=g, device=device, dtype=torch.int8)
        self.temp = (0.5 + torch.rand(H, generator=g, device=device)).float()
        self.out = torch.empty(B, H * D, dtype=torch.int8, device=device)
        self.kern = K.AttnKernel(K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D))
        self.ops = 4.0 * B * H * D * (T + 1)
        self.tokens = B
        self.units = B * H
        self.alg_bytes = self.kv.numel() + self.q.numel() + self.out.numel()
        self.launches_per_step = 1
        self.config = {"workload": "configs[4] decode: int8 attention of one new token per sequence", "batch": B,
                       "n_heads": H, "head_dim": D, "kv_len": T, "window": W,
                       "l2": "KV cache %.2f GB larger than the 126 MB L2" % (self.kv.numel() / 1e9)}
        torch.cuda.synchronize()

    def step(self):
        self.kern.decode(self.stream, self.q, self.kv, self.T, self.sink_k, self.sink_v, self.temp, self.out, None,
                         window_size=self.W, n_splits=0)

    def host_buffers(self):
        t = self.torch
        self.h_q = self.q.cpu().pin_memory()
        self.h_out = t.empty_like(self.out, device="cpu").pin_memory()
        self.h2d, self.d2h = self.h_q.numel(), self.h_out.numel()

    def e2e_step(self):   # the KV cache lives on the device; a decode step moves q in and out back
        s = self.stream
        s.upload(self.h_q.data_ptr(), self.q.data_ptr(), 0, self.h_q.numel())
        self.step()
        s.download(self.out.data_ptr(), self.h_out.data_ptr(), 0, self.h_out.numel())

    def cpu_sample(self, seconds_hint=10.0):
        from oracle import attn as o_attn
        rng = np.random.default_rng(0)
        H, D, T = 4, self.D, self.T
        q = rng.integers(-30, 31, (1, H * D), dtype=np.int8)
        kv = rng.integers(-40, 41, (1, T, H * 2 * D), dtype=np.int8)
        sk = rng.integers(-20, 21, (H, D), dtype=np.int8)
        t0, n = time.perf_counter(), 0
        while True:
            o_attn.attn_decode_i8(q, kv, T, sk, sk, np.ones(H, np.float32), self.W, H, D, kv_tile=16)
            n += 1
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        return n * H * T * 2 * D / dt, f"{n} x {H} (sequence, head) units of kv_len {T}, {dt:.1f} s"


class RmsNorm:
    """configs[3] front: RMSNorm of [16384, 4096] e4m3 -> FixedI8 (rms_norm.cu form)."""
    name = "rms_norm_e4m3_to_i8"
    bound = "hbm"
    dtype = "f32"

    def __init__(self, stream, device, M=131072, Dm=4096, seed=0):
        import torch
        from x17ai_b200 import kernels as K
        self.torch, self.stream, self.K = torch, stream, K
        g = torch.Generator(device=device).manual_seed(seed)
        self.x = (torch.randint(8, 0x60, (M, Dm), generator=g, device=device, dtype=torch.int16).to(torch.uint8)
                  | (torch.randint(0, 2, (M, Dm), generator=g, device=device, dtype=torch.int16) << 7).to(torch.uint8))
        self.y = torch.empty(M, Dm, dtype=torch.int8, device=device)
        self.ops = 3.0 * M * Dm
        self.tokens = M
        self.units = M
        self.alg_bytes = 2 * M * Dm
        self.launches_per_step = 1
        self.config = {"workload": "RMSNorm e4m3 -> FixedI8", "rows": M, "cols": Dm,
                       "l2": "input + output %.0f MB larger than the 126 MB L2" % (self.alg_bytes / 1e6)}
        torch.cuda.synchronize()

    def step(self):
        self.K.rms_norm(self.stream, self.K.RMS_E4M3_FIXED, self.x, self.y)

    def host_buffers(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_y = t.empty_like(self.y, device="cpu").pin_memory()
        self.h2d, self.d2h = self.h_x.numel(), self.h_y.numel()

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_x.data_ptr(), self.x.data_ptr(), 0, self.h_x.numel())
        self.step()
        s.download(self.y.data_ptr(), self.h_y.data_ptr(), 0, self.h_y.numel())

    def cpu_sample(self, seconds_hint=5.0):
        from oracle import formats, rms_norm as o_rms
        rng = np.random.default_rng(0)
        x = formats.f32_to_e4m3(rng.standard_normal((4096, 4096)).astype(np.float32))
        t0, n = time.perf_counter(), 0
        while True:
            o_rms.rms_norm_e4m3_i8(x)
            n += 1
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        return n * 2 * x.size / dt, f"{n} x [4096, 4096] rows, {dt:.1f} s"


class Block:
    """The reference harness's block forward (src/main.rs:193-255): six kernels per step on one batch of
    sequences at the benchmark's model shape; batch entries go through the block one sequence at a time."""
    name = "block_fwd"
    bound = "tensor"
    dtype = "s8/e4m3"

    def __init__(self, stream, device, B=2, S=8192, Dm=4096, H=32, D=128, F=14336, W=1024, seed=0, fused=True):
        import torch
        from x17ai_b200.block import BlockConfig, BlockForward
        self.torch, self.stream = torch, stream
        g = torch.Generator(device=device).manual_seed(seed)
        codes = lambda *s: torch.clamp(torch.round(torch.randn(*s, generator=g, device=device) * 8.0), -127, 127).to(torch.int8)
        self.x = codes(B, S, Dm)
        self.blk = BlockForward(stream, BlockConfig(Dm, H, D, F, W), codes(H * D, Dm), codes(2 * H * D, Dm),
                                codes(2 * Dm, H * D), codes(2 * F, Dm), codes(2 * Dm, F), codes(H, D), codes(H, D),
                                (0.5 + torch.rand(H, generator=g, device=device)).float(), fused_qkv=fused)
        self.B, self.S = B, S
        self.Dm, self.H, self.D, self.F, self.W = Dm, H, D, F, W
        self.stage_ops = self.blk.n_ops(S)
        self.ops = B * sum(self.stage_ops.values())
        self.tokens = B * S
        self.units = B * S
        self.alg_bytes = 0
        self.launches_per_step = B * (5 if fused else 6)
        self.config = {"workload": "block forward: q/kv projection, int8 attention, attn_y, GeGLU FFN, ffn_y (e4m3 x int8)",
                       "batch": B, "seq_len": S, "d_model": Dm, "n_heads": H, "head_dim": D, "hidden": F, "window": W,
                       "fused_qkv": fused, "l2": "weights 0.42 GB + activations per sequence 0.4 GB, larger than the 126 MB L2"}
        torch.cuda.synchronize()

    def make_sequential(self):
        """--sequential: the eight-launch form (RMSNorm before each sub-block) on an e4m3 hidden state."""
        t = self.torch
        self.sequential = True
        self.h = t.empty((self.B, self.S, self.Dm), dtype=t.uint8, device=self.x.device)
        for b in range(self.B):   # a hidden state of the block's own making
            self.h[b].copy_(self.blk.forward(self.x[b])["ffn_y"])
        t.cuda.synchronize()
        self.launches_per_step += 2 * self.B
        self.config["form"] = "sequential: RMSNorm -> attention sub-block -> RMSNorm -> FFN sub-block"

    def step(self):
        if getattr(self, "sequential", False):
            for b in range(self.B):
                self.blk.forward_layer(self.h[b])
            return
        for b in range(self.B):
            self.blk.forward(self.x[b])

    def host_buffers(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_y = t.empty((self.B, self.S, self.Dm), dtype=t.uint8).pin_memory()
        self.h2d, self.d2h = self.h_x.numel(), self.h_y.numel()

    def e2e_step(self):
        s = self.stream
        for b in range(self.B):
            s.upload(self.h_x[b].data_ptr(), self.x[b].data_ptr(), 0, self.x[b].numel())
            out = self.blk.forward(self.x[b])
            s.download(out["ffn_y"].data_ptr(), self.h_y[b].data_ptr(), 0, out["ffn_y"].numel())

    def cpu_sample(self, seconds_hint=15.0):
        """Oracle on a bounded sample: the six stages on a short sequence of the same model shape."""
        from oracle import attn as o_attn, gemm as o_gemm
        Dm, H, D, F, W = self.Dm, self.H, self.D, self.F, self.W
        S = 256
        rng = np.random.default_rng(0)
        mk = lambda *s: np.clip(np.rint(rng.standard_normal(s) * 8), -127, 127).astype(np.int8)
        x, wq, wkv, way, wf, wy = mk(S, Dm), mk(H * D, Dm), mk(2 * H * D, Dm), mk(2 * Dm, H * D), mk(2 * F, Dm), mk(2 * Dm, F)
        sk, sv, temp = mk(H, D), mk(H, D), np.ones(H, np.float32)
        t0, n = time.perf_counter(), 0
        while True:
            q = o_gemm.attn_q_fwd(x, wq)
            kv, _ = o_gemm.attn_kv_fwd(x, wkv, D)
            ao, _ = o_attn.attn_fwd_i8(q, kv, sk, sv, temp, W, H, D, kv_tile=16)
            o_gemm.attn_y_fwd(ao, way, x)
            f = o_gemm.ffn_f_fwd(x, wf)
            o_gemm.ffn_y_fwd_f8(f, wy, x)
            n += 1
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        ops = (2.0 * S * Dm * (3 * H * D) + 2.0 * S * H * D * 2 * Dm + 2.0 * S * Dm * 2 * F + 2.0 * S * F * 2 * Dm
               + o_attn.attn_ops(1, H, D, S, W))
        return n * ops / dt, f"{n} block forwards of a {S}-token sequence at the same model shape, {dt:.1f} s"


def _shape(args, n):
    if not args.shape:
        return None
    v = [int(x) for x in args.shape.split(",")]
    if len(v) != n:
        raise SystemExit(f"--shape needs {n} comma-separated integers for this workload")
    return v


WORKLOADS = {
    "attn": lambda s, d, a=None: AttnPrefill(s, d, *(_shape(a, 5) or ())),
    "attn_pv_fp8": lambda s, d, a=None: AttnPvFp8(s, d, *(_shape(a, 5) or ())),
    "ffn_i8": lambda s, d, a=None: Ffn(s, d, False, *(_shape(a, 3) or ())),
    "ffn_f8": lambda s, d, a=None: Ffn(s, d, True, *(_shape(a, 3) or ())),
    "qkvg": lambda s, d, a=None: Qkvg(s, d, *(_shape(a, 4) or ())),
    "decode": lambda s, d, a=None: Decode(s, d, *(_shape(a, 5) or ())),
    "rms_norm": lambda s, d, a=None: RmsNorm(s, d, *(_shape(a, 2) or ())),
    "block": lambda s, d, a=None: Block(s, d, *(_shape(a, 7) or ())),
}


# ------------------------------------------------------------------------------------------------

def run_reference(args, rank, world):
    """The reference's CPU path = the CPU restatement (oracle/), all host threads, bounded sample."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    try:  # torchrun pins OMP_NUM_THREADS=1: give the BLAS under numpy every host core back
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    # build the workload description without touching a GPU
    cls = {"attn": AttnPrefill, "attn_pv_fp8": AttnPrefill, "ffn_i8": Ffn, "ffn_f8": Ffn, "decode": Decode,
           "rms_norm": RmsNorm, "block": Block, "qkvg": Qkvg}[args.workload]
    w = cls.__new__(cls)
    if args.workload in ("attn", "attn_pv_fp8"):
        # the fp8 P.V variant has no CPU form of its own: the int8 restatement (same operation count) stands in
        w.S, w.D, w.W, B, H = 8192, 128, 1024, 8, 32
        cfg = {"workload": "configs[1] int8 sliding-window attention prefill", "batch": B, "n_heads": H, "seq_len": 8192,
               "head_dim": 128, "window": 1024}
        unit, metric = "TOPS", "int8 sliding-window attention prefill throughput"
    elif args.workload.startswith("ffn"):
        w.Dm, w.F = 4096, 14336
        cfg = {"workload": "configs[3] gated FFN (GeGLU -> e4m3, gated residual)", "tokens": 16384, "d_model": 4096, "hidden": 14336}
        unit, metric = "TOPS", "gated FFN forward throughput"
    elif args.workload == "decode":
        w.D, w.T, w.W = 128, 4096, 4096
        cfg = {"workload": "configs[4] decode", "batch": 256, "n_heads": 32, "head_dim": 128, "kv_len": 4096}
        unit, metric = "GB/s", "int8 decode attention KV-cache bandwidth"
    elif args.workload == "qkvg":
        w.Dm, w.H, w.D = 4096, 32, 128
        cfg = {"workload": "fused Q/KV projection", "tokens": 16384, "d_model": 4096, "n_heads": 32, "head_dim": 128}
        unit, metric = "TOPS", "fused Q/KV projection throughput"
    elif args.workload == "block":
        w.Dm, w.H, w.D, w.F, w.W = 4096, 32, 128, 14336, 1024
        cfg = {"workload": "block forward: q/kv projection, int8 attention, attn_y, GeGLU FFN, ffn_y (e4m3 x int8)",
               "batch": 2, "seq_len": 8192, "d_model": 4096, "n_heads": 32, "head_dim": 128, "hidden": 14336, "window": 1024}
        unit, metric = "TOPS", "quantized block forward throughput"
    else:
        cfg = {"workload": "RMSNorm e4m3 -> FixedI8", "rows": 131072, "cols": 4096}
        unit, metric = "GB/s", "RMSNorm bandwidth"
    per_step = max(0.3, min(20.0, 120.0 / max(1, args.steps + args.warmup)))  # the whole run: about two minutes
    vals = []
    sample = ""
    for i in range(args.warmup + args.steps):
        rate, sample = w.cpu_sample(per_step)
        if i >= args.warmup:
            vals.append(rate)
    scale = 1e12 if unit == "TOPS" else 1e9
    v = float(np.mean(vals)) / scale
    line = {"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32/int (numpy)", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather", action="store_true", help="N > 1: also time an NCCL all_gather of the step's output "
                    "(reported separately as gather_ms; the path itself needs no collective)")
    ap.add_argument("--sequential", action="store_true", help="block workload: RMSNorm before each sub-block (eight launches)")
    ap.add_argument("--shape", default="", help="override the workload shape (small cases for profiling): attn B,H,S,D,W; "
                    "ffn M,Dm,F; decode B,H,D,T,W; rms_norm M,Dm; block B,S,Dm,H,D,F,W; qkvg M,Dm,H,D")
    ap.add_argument("--attn-schedule", default="per_tile", choices=["persistent", "per_tile"],
                    help="attention kernel: one CTA per 128-query tile (default) or the persistent one")
    ap.add_argument("--attn-item-tiles", type=int, default=0, help="persistent attention: query tiles per item (0 = per launch)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world, local = dist_env()

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from x17ai_b200 import _lib, build, device
    build.build()
    lib = _lib.load()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = device.CudaStream(local)
    from x17ai_b200 import kernels as K
    K.set_attn_schedule(K.ATTN_PER_TILE if args.attn_schedule == "per_tile" else K.ATTN_PERSISTENT, args.attn_item_tiles)
    w = WORKLOADS[args.workload](stream, dev, args)
    if args.sequential:
        if args.workload != "block":
            raise SystemExit("--sequential applies to --workload block")
        w.make_sequential()
        args.no_e2e = True   # the end-to-end leg times the harness form only

    def barrier():
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- device-resident timing ----
    timers = [device.CudaTimer(stream) for _ in range(args.steps)]
    for _ in range(args.warmup):
        w.step()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.5)  # nvidia-smi needs a moment before its first sample
    barrier()
    launches0 = lib.x17ai_b200_launch_count()
    wall0 = time.time()
    t0 = time.perf_counter()
    for i in range(args.steps):
        timers[i].start()
        w.step()
        timers[i].stop()
    stream.synchronize()
    t1 = time.perf_counter()
    wall1 = time.time()
    launches = lib.x17ai_b200_launch_count() - launches0
    time.sleep(0.15)
    clocks = sampler.stop(wall0, wall1)
    dev_times = [t.elapsed_seconds() for t in timers]
    status = stream.read_status()
    if status != [0, 0, 0, 0]:
        raise RuntimeError(f"device status words not clean: {status}")
    # the timed region on the device: first start to last stop = sum of back-to-back steps
    total = torch.tensor([sum(dev_times), t1 - t0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    dev_total, wall_total = float(total[0]), float(total[1])
    kernel_avg = float(np.mean(dev_times))

    # ---- end to end through the C ABI with host buffers ----
    e2e = None
    if not args.no_e2e:
        w.host_buffers()
        e2e_sync = getattr(w, "e2e_sync", stream.synchronize)
        for _ in range(2):
            w.e2e_step()
        e2e_sync()
        barrier()
        n_e2e = max(3, min(args.steps, 10))
        # host clock between two full synchronisations: an end-to-end step may use several
        # streams (copies of one sequence under the kernel of another), which no single
        # stream's events bracket
        tw0 = time.perf_counter()
        for _ in range(n_e2e):
            w.e2e_step()
        e2e_sync()
        tw1 = time.perf_counter()
        e2e_t = torch.tensor([tw1 - tw0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        e2e_time = float(e2e_t[0]) / n_e2e
        e2e = {"h2d_bytes_per_step": int(w.h2d), "d2h_bytes_per_step": int(w.d2h), "ms_per_step": e2e_time * 1e3,
               "steps": n_e2e, "clock": "host, between stream synchronisations",
               "streams": len(getattr(w, "e2e_streams", [stream]))}

    gather_ms = None
    if args.gather and world > 1:
        out_t = getattr(w, "out", None) if hasattr(w, "out") else getattr(w, "y", None)
        parts = [torch.empty_like(out_t) for _ in range(world)]
        for _ in range(2):
            dist.all_gather(parts, out_t)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(5):
            dist.all_gather(parts, out_t)
        ev1.record()
        torch.cuda.synchronize()
        g = torch.tensor([ev0.elapsed_time(ev1) / 5], dtype=torch.float64, device=dev)
        dist.all_reduce(g, op=dist.ReduceOp.MAX)
        gather_ms = float(g[0])

    peaks = measured_peaks()
    if w.bound == "tensor":
        unit, scale = "TOPS", 1e12
        work = w.ops
        # int8 / fp8 dense tensor rate is twice the bf16 rate; the measured denominator is the
        # cuBLAS bf16 figure (sustained: the kernel is timed back to back inside a long step)
        peak = 2.0 * peaks["bf16_sustained"]
        peak_note = f"2 x bf16 sustained of {peaks['source']}"
        r_unit = "TFLOP/s"
    else:
        unit, scale = "GB/s", 1e9
        work = w.alg_bytes
        peak = peaks["hbm_gbs"]
        peak_note = f"copy bandwidth of {peaks['source']}"
        r_unit = "GB/s"
    value = world * work * args.steps / dev_total / scale
    achieved = work / kernel_avg / scale
    line = {
        "metric": {"attn": "int8 sliding-window attention prefill throughput",
                   "attn_pv_fp8": "attention with fp8 P.V prefill throughput", "ffn_i8": "gated FFN forward throughput",
                   "qkvg": "fused Q/KV projection throughput",
                   "ffn_f8": "gated FFN forward throughput", "decode": "int8 decode attention KV-cache bandwidth",
                   "rms_norm": "RMSNorm bandwidth", "block": "quantized block forward throughput"}[args.workload],
        "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic (seeded N(0,1) values quantised to FixedI8 codes)",
        "config": dict(w.config, sharding=f"{world} x per-GPU workload, (batch, head) / token-row units, no collective"),
        "tokens_per_s": world * w.tokens * args.steps / dev_total,
        "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": r_unit, "frac": achieved / peak,
                     "traffic": measured_traffic(args.workload, w.units), "peak_source": peak_note, "kernel_ms": kernel_avg * 1e3,
                     "nominal_frac": achieved / (4500.0 if w.bound == "tensor" else 7700.0)},
        "clocks": clocks,
        "gpu_launches": int(launches),
        "wall_ms_per_step": wall_total / args.steps * 1e3,
    }
    if gather_ms is not None:
        line["gather_ms"] = gather_ms
    if args.workload in ("attn", "attn_pv_fp8"):
        line["reference_count_tops"] = world * w.ref_ops * args.steps / dev_total / 1e12
    if e2e is not None:
        e2e["value"] = world * work / (e2e["ms_per_step"] * 1e-3) / scale
        e2e["unit"] = unit
        line["e2e"] = e2e
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, sample = w.cpu_sample()
        line["cpu_baseline"] = {"value": rate / scale, "unit": unit, "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": sample}
    if rank == 0:
        print(json.dumps(line), flush=True)
    for t in timers:
        t.destroy()
    stream.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
