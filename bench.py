#!/usr/bin/env python3
"""Benchmark of the quantized block-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload: the prefill-scale int8 sliding-window attention forward (configs[1]: batch 8, 32 heads,
seq 8192, head_dim 128, window 1024), synthetic seeded inputs. With N > 1 (torchrun, one rank per GPU) the
FIXED problem is sharded: rank r takes its (sequence, head) units of the one batch (x17ai_b200.sharding.attn_shard),
no data moves inside the path, "scaling": "strong". Beside the compute-only number the line carries the same
step with an NCCL all-gather of the outputs inside it, and with that gather chunked and overlapped.

One JSON line on stdout (rank 0). `value` is measured with inputs resident in HBM; `e2e` goes through the C ABI
with host buffers (pinned), host->device and device->host copies inside the timed region. `roofline.achieved`
uses the average kernel duration from CUDA events recorded on the launching stream. At N = 1 the line also
carries `workloads`: the other kernels of the path (FFN int8 / e4m3, fused projection, decode, RMSNorm, fp8 P.V,
the block), each timed for at least half a second with its own clock record, and `ref_kernel_baseline`: the
reference's own attention kernel compiled for sm_100a on one sequence of the same shape. `--impl reference`
times the reference's CPU path on the host cores on a bounded sample of the same workload.
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


def attn_ops(batch, n_heads, head_dim, seq_len, window):
    """Algorithmic operation count of one attention pass: 4 * B*H*D * sum_i (min(i, W') + 1), W' = window rounded
    up to 16 (0 = unbounded): Q.K^T and P.V of every attended key, the sink included, masked positions excluded."""
    w = None if window == 0 else ((window - 1) // 16 + 1) * 16
    i = np.arange(seq_len, dtype=np.int64)
    n = i if w is None else np.minimum(i, w)
    return 4.0 * batch * n_heads * head_dim * float((n + 1).sum())


def attn_line_config(B, H, S, D, W, world):
    """`config` of the attention line, the same in both arms (`--impl ours`, `--impl reference`): the workload, how it
    is cut over the GPUs, and why L2 does not hold it between steps (rank 0's shard)."""
    from x17ai_b200 import sharding
    sh = sharding.attn_shard(B, H, world, 0)
    nb, nh = sh.seq_end - sh.seq_begin, sh.head_end - sh.head_begin
    alg_bytes = nb * S * nh * D * 4 + nb * nh * S * 4
    return {"workload": "configs[1] int8 sliding-window attention prefill", "batch": B, "n_heads": H, "seq_len": S,
            "head_dim": D, "window": W,
            "l2": "inputs (q+kv+out = %.0f MB per GPU) larger than the 126 MB L2" % (alg_bytes / 1e6),
            "sharding": f"the fixed batch cut into {world} shards of (sequence, head) units, one per GPU, no collective in the path"}


def library_tensor_peaks(torch, dev):
    """cuBLAS int8 (torch._int_mm) and fp8 (torch._scaled_mm) dense rates at 8192^3 on this GPU, best of 10,
    measured outside every timed region: a measured denominator beside the assumed 2 x bf16."""
    out = {}
    n = 8192
    ev = lambda: torch.cuda.Event(enable_timing=True)
    def best(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(10):
            e0, e1 = ev(), ev()
            e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3)
        return 2.0 * n ** 3 / min(ts) / 1e12
    try:
        a = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev).t()
        out["int8_tops"] = best(lambda: torch._int_mm(a, b))
    except Exception as e:   # a torch build without the op: report why, keep going
        out["int8_error"] = str(e)[:80]
    try:
        a8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        out["fp8_tflops"] = best(lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
    except Exception as e:
        out["fp8_error"] = str(e)[:80]
    return out


class ClockSampler:
    """Samples SM clocks, power and throttle reasons during the timed region: through NVML every 5 ms from a
    thread of this process (read-only queries; a timed region of a few milliseconds still gets samples) and,
    beside it, with the nvidia-smi query loop every 100 ms. The summary uses the NVML samples when there are
    any, else nvidia-smi's."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    PERIOD_S = 0.005

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.nvml = []        # (wall time, sm MHz, max MHz, watts, reason bits)
        self._stop = threading.Event()
        self._nvml_thread = None

    def _nvml_loop(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        except Exception:
            return
        while not self._stop.is_set():
            try:
                self.nvml.append((time.time(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), mx,
                                  nv.nvmlDeviceGetPowerUsage(h) / 1000.0, int(reasons(h))))
            except Exception:
                pass
            self._stop.wait(self.PERIOD_S)
        try:
            nv.nvmlShutdown()
        except Exception:
            pass

    def start(self):
        self._nvml_thread = threading.Thread(target=self._nvml_loop, daemon=True)
        self._nvml_thread.start()
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

    # NVML's reason bits (nvml.h: nvmlClocksEventReasons)
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken between the wall-clock times t_begin and t_end (all if None)."""
        import datetime
        self._stop.set()
        if self._nvml_thread is not None:
            self._nvml_thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        all_bits = 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, c, m, w, bits in self.nvml:
            if t_begin is not None and not (t_begin - 0.002 <= ts <= t_end + 0.002):
                continue
            sm.append(float(c)); mx.append(float(m)); power.append(w)
            all_bits |= bits
            for n, b in self.BITS.items():
                if bits & b:
                    reasons.add(n)
        source = "nvml, 5 ms period"
        smi = 0
        smi_rows = []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if t_begin is not None and not (t_begin - 0.05 <= ts <= t_end + 0.05):
                    continue
                smi_rows.append((float(parts[1]), float(parts[2]), float(parts[3]), parts[4:8]))
            except ValueError:
                continue
        smi = len(smi_rows)
        if not sm:
            if self.proc is None and not smi_rows:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml and nvidia-smi unavailable"]}
            source = "nvidia-smi, 100 ms period"
            for c, m, w, flags in smi_rows:
                sm.append(c); mx.append(m); power.append(w)
        for c, m, w, flags in smi_rows:      # reasons seen by either sampler count
            for n, v in zip(names, flags):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_mhz_lowest": min(sm) if sm else None, "sm_mhz_highest": max(sm) if sm else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "samples_nvidia_smi": smi,
                "source": source, "reasons": sorted(reasons), "nvml_reason_bits": hex(all_bits)}


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
    """configs[1]: B8 H32 S8192 D128 W1024. One batched launch per step over this rank's shard of the batch
    (`shard` = x17ai_b200.sharding.AttnShard: whole sequences first, then head blocks of a sequence)."""
    name = "int8_sliding_window_attention_prefill"
    bound = "tensor"
    dtype = "s8"

    def __init__(self, stream, device, B=8, H=32, S=8192, D=128, W=1024, seed=0, shard=None):
        import torch
        from x17ai_b200 import kernels as K, sharding
        self.torch, self.stream, self.K = torch, stream, K
        self.B, self.H, self.S, self.D, self.W = B, H, S, D, W
        self.shard = shard or sharding.AttnShard(0, B, 0, H)
        sh = self.shard
        nb, nh = sh.seq_end - sh.seq_begin, sh.head_end - sh.head_begin
        self.nb, self.nh = nb, nh
        # N(0,1) values -> FixedI8 codes (x8, clamp +-127); every sequence has its own generator, so a rank
        # that holds sequence b of the batch holds the same bytes whatever the number of ranks
        def codes(g, *shape, std=1.0):
            return torch.clamp(torch.round(torch.randn(*shape, generator=g, device=device) * (8.0 * std)), -127, 127).to(torch.int8)
        self.q = torch.empty(nb, S, H * D, dtype=torch.int8, device=device)
        self.kv = torch.empty(nb, S, H * 2 * D, dtype=torch.int8, device=device)
        for i, b in enumerate(range(sh.seq_begin, sh.seq_end)):
            g = torch.Generator(device=device).manual_seed(seed * 1000 + 1 + b)
            self.q[i] = codes(g, S, H * D)
            self.kv[i] = codes(g, S, H * 2 * D)
            self.kv[i].view(S, H, 2, D)[:, :, 1, :] = codes(g, S, H, D, std=1.3)
        g = torch.Generator(device=device).manual_seed(seed)
        self.sink_k = codes(g, H, D)
        self.sink_v = codes(g, H, D, std=1.3)
        self.temp = (0.5 + torch.rand(H, generator=g, device=device)).float()
        self.out = torch.empty(nb, S, nh * D, dtype=torch.int8, device=device)     # this shard's heads only
        self.l = torch.empty(nb, nh, S, dtype=torch.float32, device=device)
        self.kern = K.AttnKernel(K.AttnKernelConfig(nh, D, H * D, 2 * H * D, nh * D))
        self.ops_total = attn_ops(B, H, D, S, W)             # the whole (fixed) problem
        self.ops = attn_ops(nb, nh, D, S, W)                 # this rank's part
        self.ref_ops = K.AttnKernelConfig(H, D, H * D, 2 * H * D, H * D).n_ops(S, W) * B
        self.tokens_total = B * S
        self.tokens = nb * S
        self.units = nb * nh  # (sequence, head) units of this S, D, W
        self.alg_bytes = nb * S * nh * D * 4 + self.l.numel() * 4   # q + k + v + out of the shard's heads, L
        self.launches_per_step = 1
        self.config = {"workload": "configs[1] int8 sliding-window attention prefill", "batch": B, "n_heads": H,
                       "seq_len": S, "head_dim": D, "window": W,
                       "l2": "inputs (q+kv+out = %.0f MB per GPU) larger than the 126 MB L2" % (self.alg_bytes / 1e6)}
        torch.cuda.synchronize()

    def step(self):
        self.kern.launch_head_block(self.stream, self.q, self.kv, self.sink_k, self.sink_v, self.temp, self.out, self.l,
                                    self.W, self.shard.head_begin)

    # ---- the gather of the outputs (a consumer that wants the whole tensor on every GPU) ----
    def gather_setup(self, world, n_chunks=4):
        """Buffers for the two gathered forms: the whole shard after the kernel, and chunk by chunk (sequence x
        head block, each chunk's output contiguous) with chunk i's all-gather under chunk i + 1's kernel."""
        t, K = self.torch, self.K
        self.world = world
        self.ext = t.cuda.ExternalStream(self.stream.handle)
        self.comm = t.cuda.Stream()
        self.gathered = t.empty((world,) + tuple(self.out.shape), dtype=t.int8, device=self.out.device)
        hb_count = max(1, -(-n_chunks // self.nb))           # head blocks per sequence
        while self.nh % hb_count:
            hb_count -= 1
        hb = self.nh // hb_count
        self.chunks = [(i, j * hb) for i in range(self.nb) for j in range(hb_count)]
        self.chunk_kern = K.AttnKernel(K.AttnKernelConfig(hb, self.D, self.H * self.D, 2 * self.H * self.D, hb * self.D))
        self.chunk_out = [t.empty(self.S, hb * self.D, dtype=t.int8, device=self.out.device) for _ in self.chunks]
        self.chunk_l = t.empty(hb, self.S, dtype=t.float32, device=self.out.device)
        self.chunk_gathered = [t.empty((world, self.S, hb * self.D), dtype=t.int8, device=self.out.device) for _ in self.chunks]
        self.chunk_events = [t.cuda.Event() for _ in self.chunks]
        # third form: no gather pass at all, the kernel's epilogue stores each shard on every GPU (peer stores)
        self.peers = None
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings are all this needs
            from x17ai_b200 import sharding
            import torch.distributed as dist
            self.peers = sharding.PeerOutputs(self.B, self.H, self.D, self.S, world, dist.get_rank(), self.out.device)
            self.peer_kern = K.AttnKernel(K.AttnKernelConfig(self.nh, self.D, self.H * self.D, 2 * self.H * self.D, self.peers.cols))
            self.peer_note = "ok"
        except Exception as e:   # symmetric memory unavailable: the line says so and carries the two NCCL forms
            self.peers, self.peer_note = None, f"{type(e).__name__}: {str(e)[:160]}"
        return {"chunks": len(self.chunks), "heads_per_chunk": hb,
                "layout": "gathered[chunk][rank][seq][heads_per_chunk * head_dim]"}

    def step_peer_stores(self):
        """The kernel writes its shard into every GPU's buffer; a device-side barrier between the ranks closes the step
        (when it has passed, every rank's launch of this step has completed and every buffer holds every shard)."""
        self.peer_kern.launch_head_block(self.stream, self.q, self.kv, self.sink_k, self.sink_v, self.temp, self.peers.out,
                                         self.l, self.W, self.shard.head_begin, peer_outs=self.peers.peer_outs)
        with self.torch.cuda.stream(self.ext):
            self.peers.barrier()

    def step_gather(self):
        import torch.distributed as dist
        self.step()
        with self.torch.cuda.stream(self.ext):     # NCCL orders itself after, and the stream after NCCL
            dist.all_gather_into_tensor(self.gathered, self.out)

    def step_gather_overlapped(self):
        import torch.distributed as dist
        t = self.torch
        for c, (i, h0) in enumerate(self.chunks):
            self.chunk_kern.launch_head_block(self.stream, self.q[i], self.kv[i], self.sink_k, self.sink_v, self.temp,
                                              self.chunk_out[c], self.chunk_l, self.W, self.shard.head_begin + h0)
            with t.cuda.stream(self.ext):
                self.chunk_events[c].record()
            with t.cuda.stream(self.comm):
                self.comm.wait_event(self.chunk_events[c])
                dist.all_gather_into_tensor(self.chunk_gathered[c], self.chunk_out[c])
        with t.cuda.stream(self.ext):
            self.ext.wait_stream(self.comm)

    # ---- end to end from pinned host buffers ----
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
        sts = self.e2e_streams
        for i in range(self.nb):
            st = sts[i % len(sts)]
            st.upload(self.h_q[i].data_ptr(), self.q[i].data_ptr(), 0, self.q[i].numel())
            st.upload(self.h_kv[i].data_ptr(), self.kv[i].data_ptr(), 0, self.kv[i].numel())
            self.kern.launch_head_block(st, self.q[i], self.kv[i], self.sink_k, self.sink_v, self.temp, self.out[i],
                                        self.l[i], self.W, self.shard.head_begin)
            st.download(self.out[i].data_ptr(), self.h_out[i].data_ptr(), 0, self.out[i].numel())

    def e2e_sync(self):
        for st in getattr(self, "e2e_streams", [self.stream]):
            st.synchronize()

    # ---- baselines ----
    def ref_kernel_sample(self):
        """The reference's own kernel (cuda/attn_fwd_i8.cuh compiled for sm_100a by oracle/build_ref.py, launched
        through this library's driver shim with the reference's grid, attn.rs:438-446) on one sequence of this
        shape: the same-GPU baseline the new kernel has to beat. None where the cubin was not built."""
        import ctypes
        from x17ai_b200 import device, kernel_objects
        d = ROOT / "oracle" / "_ref" / f"attn_h{self.H}_d{self.D}"
        if not (d / "kernel.cubin").exists() or not (d / "meta.json").exists():
            return None
        t = self.torch
        k = kernel_objects.CubinKernel(self.stream, d)
        m = k.meta
        q, kv = self.q[0], self.kv[0]
        out = t.empty(self.S, self.H * self.D, dtype=t.int8, device=q.device)
        l = t.empty(self.H, self.S, dtype=t.float32, device=q.device)
        t.cuda.synchronize()
        ptr = lambda x: ctypes.c_void_p(x.data_ptr())
        hpk = max(128 // self.D, 1)
        args = (ctypes.c_uint64(self.S), ptr(q), ptr(kv), ptr(self.sink_k), ptr(self.sink_v), ptr(self.temp), ptr(out),
                ptr(l), ctypes.c_uint64(self.W))
        grid = (self.S // m["Q_PER_BLOCK"], self.H // hpk, 1)
        go = lambda: k.launch(self.stream, grid, (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"], *args)
        for _ in range(3):
            go()
        timer = device.CudaTimer(self.stream)
        n = 10
        timer.start()
        for _ in range(n):
            go()
        timer.stop()
        self.stream.synchronize()
        dt = timer.elapsed_seconds() / n
        timer.destroy()
        k.unload()
        ops = attn_ops(1, self.H, self.D, self.S, self.W)
        return {"value": ops / dt / 1e12, "unit": "TOPS", "ms": dt * 1e3,
                "kernel": "the reference's attn_forward (mma.sync, 64 queries per CTA) compiled for sm_100a",
                "sample": f"one sequence of the workload ({self.H} heads x {self.D}, {self.S} tokens, window {self.W}), {n} launches"}

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
            done_ops += attn_ops(1, 1, D, S, W)
            if time.perf_counter() - t0 > seconds_hint:
                break
        dt = time.perf_counter() - t0
        return done_ops / dt, f"{heads} (sequence, head) units of S={S} D={D} W={W}, oracle kv_tile=16, {dt:.1f} s"


def reference_cpu_attention():
    """The reference's own CPU path for this kernel: attn_one_head of its float64 PyTorch model (new_block.py:183-258),
    timed on the case the reference can run on a CPU (batch 1, 4 heads, seq 256, head_dim 64, window 64, seed 0).
    Needs a checkout of the reference (X17AI_REFERENCE); returns None elsewhere."""
    ref = os.environ.get("X17AI_REFERENCE")
    if not ref or not (Path(ref) / "new_block.py").exists():
        return None
    import importlib
    import shutil
    import tempfile
    import torch
    tmp = Path(tempfile.mkdtemp(prefix="x17ref_"))
    try:
        for f in ("new_block.py", "block_utils.py", "jsonc.py"):
            shutil.copy(Path(ref) / f, tmp / f)
        S, H, D, W = 256, 4, 64, 64
        (tmp / "block.config.json").write_text(json.dumps({
            "seq_len": S, "MODEL_DIM": H * D, "HEAD_DIM": D, "N_HEADS": H, "F_WIDTH": 256, "WINDOW_SIZE": W,
            "L2_NORM_EPS": 2.0 ** -70, "V_SCALE_FIX": 1.3}))
        sys.path.insert(0, str(tmp))
        cwd = os.getcwd()
        os.chdir(tmp)
        try:
            nb = importlib.import_module("new_block")
        finally:
            os.chdir(cwd)
        if not hasattr(nb, "attn_one_head"):
            return None
        torch.manual_seed(0)
        q = torch.randn(S, D, dtype=torch.float64); k = torch.randn(S, D, dtype=torch.float64); v = torch.randn(S, D, dtype=torch.float64)
        sk = torch.randn(D, dtype=torch.float64); sv = torch.randn(D, dtype=torch.float64)
        call = (q, k, v, sk, sv, torch.tensor(1.0, dtype=torch.float64))
        nb.attn_one_head(*call)
        best = 1e30
        for _ in range(5):
            t0 = time.perf_counter()
            for _h in range(H):
                nb.attn_one_head(*call)
            best = min(best, time.perf_counter() - t0)
        ops = attn_ops(1, H, D, S, W)
        return {"value": ops / best / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "reference",
                "sample": f"new_block.attn_one_head (float64) on configs[0]: 1 x {H} heads x {S} tokens x {D}, window {W}, "
                          f"best of 5, {best * 1e3:.1f} ms"}
    except Exception:
        return None
    finally:
        if str(tmp) in sys.path:
            sys.path.remove(str(tmp))
        shutil.rmtree(tmp, ignore_errors=True)


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


class AttnScaled(AttnPrefill):
    """The benchmark description's input format on the prefill shape: int8 Q/K/V with one f32 scale per token and
    head (absmax quantisation of N(0,1) values), bf16 output (x17ai_b200_attn_fwd_i8_scaled)."""
    name = "attention_per_token_scales_prefill"
    dtype = "s8 (per-token scales)"

    def __init__(self, stream, device, B=8, H=32, S=8192, D=128, W=1024, seed=0):
        super().__init__(stream, device, B, H, S, D, W, seed)
        torch = self.torch
        g = torch.Generator(device=device).manual_seed(seed + 2)

        def quantise(x):   # [B, S, H, D] -> codes [B, S, H, D] int8, scales [B, H, S] f32
            scale = x.abs().amax(dim=-1).clamp_min(1e-8) / 127.0
            codes = torch.clamp(torch.round(x / scale[..., None]), -127, 127).to(torch.int8)
            return codes, scale.permute(0, 2, 1).contiguous().float()

        qc, self.q_scale = quantise(torch.randn(B, S, H, D, generator=g, device=device))
        self.q.view(B, S, H, D).copy_(qc)
        kc, self.k_scale = quantise(torch.randn(B, S, H, D, generator=g, device=device))
        vc, self.v_scale = quantise(torch.randn(B, S, H, D, generator=g, device=device) * 1.3)
        kv4 = self.kv.view(B, S, H, 2, D)
        kv4[:, :, :, 0, :] = kc
        kv4[:, :, :, 1, :] = vc
        del qc, kc, vc
        self.out = torch.empty(B, S, H * D, dtype=torch.bfloat16, device=device)
        self.alg_bytes = (self.q.numel() + self.kv.numel() + 2 * self.out.numel() + self.l.numel() * 4
                          + 4 * (self.q_scale.numel() + self.k_scale.numel() + self.v_scale.numel()))
        self.config = dict(self.config, workload="configs[1] attention with per-token-per-head scaled int8 inputs, bf16 out")
        torch.cuda.synchronize()

    def step(self):
        self.kern.launch_scaled(self.stream, self.q, self.q_scale, self.kv, self.k_scale, self.v_scale, self.sink_k,
                                self.sink_v, self.temp, self.out, self.l, self.W)

    def host_buffers(self):
        t = self.torch
        self.h_q = self.q.cpu().pin_memory(); self.h_kv = self.kv.cpu().pin_memory()
        self.h_scales = [x.cpu().pin_memory() for x in (self.q_scale, self.k_scale, self.v_scale)]
        self.h_out = t.empty_like(self.out, device="cpu").pin_memory()
        self.h2d = self.h_q.numel() + self.h_kv.numel() + sum(4 * x.numel() for x in self.h_scales)
        self.d2h = self.h_out.numel() * 2

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_q.data_ptr(), self.q.data_ptr(), 0, self.h_q.numel())
        s.upload(self.h_kv.data_ptr(), self.kv.data_ptr(), 0, self.h_kv.numel())
        for h, d in zip(self.h_scales, (self.q_scale, self.k_scale, self.v_scale)):
            s.upload(h.data_ptr(), d.data_ptr(), 0, 4 * h.numel())
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


class FfnE4m3(Ffn):
    """configs[3], second run: the same gated FFN with e4m3 weights and e4m3 activations, one f32 scale per tensor
    (weights N(0, 0.02), scale = absmax / 448). Both GEMMs run as e4m3 x e4m3 on the fp8 tensor path."""

    def __init__(self, stream, device, M=16384, Dm=4096, F=14336, seed=0):
        import torch
        from x17ai_b200 import kernels as K
        self.torch, self.stream, self.f8 = torch, stream, True
        self.name, self.dtype = "ffn_fwd_e4m3", "e4m3"
        g = torch.Generator(device=device).manual_seed(seed)
        def q8(t):   # per-tensor scale, OCP e4m3 bytes
            scale = float(t.abs().max()) / 448.0
            return (t / scale).to(torch.float8_e4m3fn).view(torch.uint8), scale
        xv = torch.randn(M, Dm, generator=g, device=device)
        self.x8, self.sx = q8(xv)
        self.x = torch.clamp(torch.round(xv * 8.0), -127, 127).to(torch.int8)      # the residual stream (FixedI8)
        del xv
        self.wf, self.swf = q8(torch.randn(2 * F, Dm, generator=g, device=device) * 0.02)
        self.wy, self.swy = q8(torch.randn(2 * Dm, F, generator=g, device=device) * 0.02)
        self.f = torch.empty(M, F, dtype=torch.uint8, device=device)
        self.y = torch.empty(M, Dm, dtype=torch.uint8, device=device)
        self.k_f = K.GemmKernel(K.ffn_f_fwd_e4m3_config(Dm, F, self.sx, self.swf))
        self.k_y = K.GemmKernel(K.ffn_y_fwd_e4m3_config(F, Dm, self.swy))
        torch.cuda.synchronize()
        self.M, self.Dm, self.F = M, Dm, F
        self.ops = 2.0 * M * Dm * 2 * F + 2.0 * M * F * 2 * Dm
        self.tokens = M
        self.units = M
        self.alg_bytes = M * Dm + 2 * F * Dm + M * F * 2 + 2 * Dm * F + M * Dm * 2
        self.launches_per_step = 2
        self.config = {"workload": "configs[3] gated FFN, e4m3 weights and activations with per-tensor scales", "tokens": M,
                       "d_model": Dm, "hidden": F, "gemms": "e4m3 x e4m3 (kind::f8f6f4), f32 accumulation",
                       "l2": "weights + activations (%.0f MB) larger than the 126 MB L2" % (self.alg_bytes / 1e6)}

    def step(self):
        self.k_f.launch(self.stream, self.x8, self.wf, self.f)
        self.k_y.launch(self.stream, self.f, self.wy, self.y, residual=self.x)

    def host_buffers(self):
        t = self.torch
        self.h_x = self.x8.cpu().pin_memory()
        self.h_y = t.empty_like(self.y, device="cpu").pin_memory()
        self.h2d, self.d2h = self.h_x.numel(), self.h_y.numel()

    def e2e_step(self):
        s = self.stream
        s.upload(self.h_x.data_ptr(), self.x8.data_ptr(), 0, self.h_x.numel())
        self.step()
        s.download(self.y.data_ptr(), self.h_y.data_ptr(), 0, self.h_y.numel())


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

    def stage_times(self, rounds=5):
        """Per-stage device times of the harness form (src/main.rs:193-255 times every launch): mean over `rounds`
        forwards of one sequence, with the stage's operation count: {stage: {"ms", "tops"}}."""
        acc = {}
        for _ in range(rounds):
            self.blk.forward(self.x[0], timed=True)
            for k, v in self.blk.seconds.items():
                acc[k] = acc.get(k, 0.0) + v / rounds
        ops = dict(self.stage_ops)
        if self.blk.fused_qkv:   # one launch does both projections; the second stage is empty
            ops["attn_q"] = ops["attn_q"] + ops.pop("attn_kv")
        return {k: {"ms": v * 1e3, "tops": (ops[k] / v / 1e12 if k in ops and v > 1e-6 else None)} for k, v in acc.items()}

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
               + attn_ops(1, H, D, S, W))
        return n * ops / dt, f"{n} block forwards of a {S}-token sequence at the same model shape, {dt:.1f} s"


def _shape(args, n):
    if args is None or not args.shape:
        return None
    v = [int(x) for x in args.shape.split(",")]
    if len(v) != n:
        raise SystemExit(f"--shape needs {n} comma-separated integers for this workload")
    return v


WORKLOADS = {
    "attn": lambda s, d, a=None, **kw: AttnPrefill(s, d, *(_shape(a, 5) or ()), **kw),
    "attn_pv_fp8": lambda s, d, a=None: AttnPvFp8(s, d, *(_shape(a, 5) or ())),
    "attn_scaled": lambda s, d, a=None: AttnScaled(s, d, *(_shape(a, 5) or ())),
    "ffn_i8": lambda s, d, a=None: Ffn(s, d, False, *(_shape(a, 3) or ())),
    "ffn_f8": lambda s, d, a=None: Ffn(s, d, True, *(_shape(a, 3) or ())),
    "ffn_e4m3": lambda s, d, a=None: FfnE4m3(s, d, *(_shape(a, 3) or ())),
    "qkvg": lambda s, d, a=None: Qkvg(s, d, *(_shape(a, 4) or ())),
    "decode": lambda s, d, a=None: Decode(s, d, *(_shape(a, 5) or ())),
    "rms_norm": lambda s, d, a=None: RmsNorm(s, d, *(_shape(a, 2) or ())),
    "block": lambda s, d, a=None: Block(s, d, *(_shape(a, 7) or ())),
}
METRICS = {"attn": "int8 sliding-window attention prefill throughput",
           "attn_pv_fp8": "attention with fp8 P.V prefill throughput",
           "attn_scaled": "attention with per-token-per-head scaled int8 inputs prefill throughput",
           "ffn_i8": "gated FFN forward throughput",
           "qkvg": "fused Q/KV projection throughput", "ffn_f8": "gated FFN forward throughput",
           "ffn_e4m3": "gated FFN forward throughput (e4m3 weights and activations)",
           "decode": "int8 decode attention KV-cache bandwidth", "rms_norm": "RMSNorm bandwidth",
           "block": "quantized block forward throughput"}
# the other kernels of the path, reported beside the headline at N = 1 (smaller than the headline's own case
# only where the full one would not fit the few minutes the default run has)
# token-row workloads that --gpus N cuts into one row block per GPU (strong scaling): name -> default --shape
ROW_SHARDED = {"ffn_i8": (16384, 4096, 14336), "ffn_f8": (16384, 4096, 14336), "ffn_e4m3": (16384, 4096, 14336),
               "qkvg": (16384, 4096, 32, 128)}
SIDE_WORKLOADS = ["ffn_i8", "ffn_f8", "ffn_e4m3", "qkvg", "attn_pv_fp8", "attn_scaled", "decode", "rms_norm", "block"]


# ------------------------------------------------------------------------------------------------

def run_reference(args, rank, world):
    """The reference's CPU path, all host threads, bounded sample: its own float64 model where a checkout of the
    reference is at hand (attention only: X17AI_REFERENCE), else the CPU restatement of its kernels (oracle/)."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    try:  # torchrun pins OMP_NUM_THREADS=1: give the BLAS under numpy every host core back
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    # build the workload description without touching a GPU
    cls = {"attn": AttnPrefill, "attn_pv_fp8": AttnPrefill, "attn_scaled": AttnPrefill, "ffn_i8": Ffn, "ffn_f8": Ffn, "ffn_e4m3": Ffn, "decode": Decode,
           "rms_norm": RmsNorm, "block": Block, "qkvg": Qkvg}[args.workload]
    w = cls.__new__(cls)
    if args.workload in ("attn", "attn_pv_fp8", "attn_scaled"):
        # the fp8 P.V and per-token-scale variants: the int8 restatement (same operation count) stands in
        w.S, w.D, w.W, B, H = 8192, 128, 1024, 8, 32
        cfg = attn_line_config(B, H, 8192, 128, 1024, world)
        unit, metric = "TOPS", METRICS["attn"]
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
            "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.workload == "attn" or (args.workload in ROW_SHARDED and world > 1) else "weak",
            "vs_baseline": None, "dtype": "f32/int (numpy)", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.workload == "attn":
        ref = reference_cpu_attention()
        if ref is not None:
            line["cpu_reference_model"] = ref
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa_node(local):
    """Host threads and the pinned buffers they allocate next go to the NUMA node of this rank's GPU (sysfs),
    so that N ranks do not all stage through node 0. Returns a description for the JSON line."""
    try:
        bus = subprocess.run(["nvidia-smi", f"--id={local}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().splitlines()[0].strip()
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:      # NVML pads the domain to eight digits, sysfs uses four
            bus = bus[4:]
        node = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
        if node < 0:
            return {"numa_node": None, "note": "the platform reports no NUMA node for the GPU"}
        cpus = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
        ids = set()
        for part in cpus.split(","):
            a, _, b = part.partition("-")
            ids.update(range(int(a), int(b or a) + 1))
        allowed = ids & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "cpus": len(allowed)}
    except Exception as e:
        return {"numa_node": None, "note": f"not bound: {type(e).__name__}"}


class Runner:
    """Times a workload: per-step CUDA-event timers on the launching stream, clocks sampled over the timed region."""

    def __init__(self, torch, dist, lib, device, stream, local, world, dev):
        self.torch, self.dist, self.lib, self.device = torch, dist, lib, device
        self.stream, self.local, self.world, self.dev = stream, local, world, dev

    def barrier(self):
        self.stream.synchronize()
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()

    def time_steps(self, step, steps, warmup, sync=None):
        """(device seconds of all steps: max over ranks, mean seconds of one step, wall seconds, launches, clocks)"""
        torch = self.torch
        sync = sync or self.stream.synchronize
        timers = [self.device.CudaTimer(self.stream) for _ in range(steps)]
        tw = time.perf_counter()
        for _ in range(warmup):
            step()
        sync()
        per_step = (time.perf_counter() - tw) / max(warmup, 1)
        sampler = ClockSampler(self.local)
        sampler.start()
        # nvidia-smi needs half a second before its first sample. The GPU keeps working through it (more untimed
        # steps): after an idle half second the first timed steps would run while the clocks are still ramping up.
        # Every rank runs the same number of them (a step may hold a collective).
        n_keep = torch.tensor([min(int(PRELOAD_S / max(per_step, 1e-6)) + 1, 200000)], dtype=torch.int64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(n_keep, op=self.dist.ReduceOp.MAX)
        for _ in range(int(n_keep[0])):
            step()
        sync()
        self.barrier()
        launches0 = self.lib.x17ai_b200_launch_count()
        wall0 = time.time()
        t0 = time.perf_counter()
        for i in range(steps):
            timers[i].start()
            step()
            timers[i].stop()
        sync()
        self.stream.synchronize()
        t1 = time.perf_counter()
        wall1 = time.time()
        launches = self.lib.x17ai_b200_launch_count() - launches0
        time.sleep(0.15)
        clocks = sampler.stop(wall0, wall1)
        dev_times = [t.elapsed_seconds() for t in timers]
        for t in timers:
            t.destroy()
        status = self.stream.read_status()
        if status != [0, 0, 0, 0]:
            raise RuntimeError(f"device status words not clean: {status}")
        total = torch.tensor([sum(dev_times), t1 - t0], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(total, op=self.dist.ReduceOp.MAX)
        return float(total[0]), float(np.mean(dev_times)), float(total[1]), int(launches), clocks

    def time_burst(self, step, steps, idle_s=1.0):
        """The same step timed the way a kernel is timed alone: the GPU idles for `idle_s`, three untimed steps bring
        the clocks up, then `steps` steps are timed with device events (N = 1 only). Returns (seconds per step,
        clock record): the burst counterpart of `time_steps`, whose timed region follows half a second of load."""
        self.stream.synchronize()
        time.sleep(idle_s)
        for _ in range(3):
            step()
        self.stream.synchronize()
        sampler = ClockSampler(self.local)
        sampler.start()
        tm = self.device.CudaTimer(self.stream)
        wall0 = time.time()
        tm.start()
        for _ in range(steps):
            step()
        tm.stop()
        self.stream.synchronize()
        wall1 = time.time()
        clocks = sampler.stop(wall0, wall1)
        per = tm.elapsed_seconds() / steps
        tm.destroy()
        return per, clocks

    def steps_for(self, step, seconds, lo=3, hi=100000):
        """How many steps fill `seconds` of device time (measured on three)."""
        tm = self.device.CudaTimer(self.stream)
        step(); self.stream.synchronize()
        tm.start()
        for _ in range(3):
            step()
        tm.stop(); self.stream.synchronize()
        per = max(tm.elapsed_seconds() / 3, 1e-6)
        tm.destroy()
        return int(min(hi, max(lo, np.ceil(seconds / per))))


PRELOAD_S = 0.5   # the step runs back to back for this long right before the timed region (Runner.time_steps)


def roofline(w, achieved, region_s, peaks, lib_peaks, traffic_key, clocks=None):
    """`peak`: the measured denominator of MEASURED_PEAKS.json - for a tensor-bound kernel twice the cuBLAS bf16
    rate (int8 and fp8 run at twice the bf16 rate; no int8 figure is in that file); for an HBM-bound kernel the
    copy bandwidth. That file has a burst figure (a kernel timed alone) and a sustained one (a seconds-long loop
    under the power cap). The timed region here follows half a second of the same step, so the sustained figure
    is the denominator when the load has lasted a second by the end of the region or the clock record shows the
    power cap active; else the burst one. Both fractions are in the line."""
    if w.bound == "tensor":
        capped = bool(clocks) and "sw_power_cap" in (clocks.get("reasons") or [])
        burst = (PRELOAD_S + region_s) < 1.0 and not capped
        peak = 2.0 * (peaks["bf16_burst"] if burst else peaks["bf16_sustained"])
        why = (f"{PRELOAD_S:.1f} s of the same step before a timed region of {region_s:.2f} s"
               + ("; sw_power_cap active in the clock record" if capped else ""))
        r = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
             "traffic": measured_traffic(traffic_key, w.units),
             "peak_source": f"2 x bf16 {'burst' if burst else 'sustained'} of {peaks['source']} ({why})",
             "frac_of_burst": achieved / (2.0 * peaks["bf16_burst"]),
             "frac_of_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
             "nominal_frac": achieved / 4500.0}
        key = "fp8_tflops" if "e4m3" in w.dtype and "s8" not in w.dtype else "int8_tops"
        if lib_peaks.get(key):
            r["peak_library_measured"] = lib_peaks[key]
            r["frac_of_library_measured"] = achieved / lib_peaks[key]
            r["peak_library_source"] = ("torch._scaled_mm e4m3" if key == "fp8_tflops" else "torch._int_mm int8") + " 8192^3, best of 10, this process"
        return r
    peak = peaks["hbm_gbs"]
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": measured_traffic(traffic_key, w.units), "peak_source": f"copy bandwidth of {peaks['source']}",
            "nominal_frac": achieved / 7700.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-side-workloads", action="store_true", help="N = 1, --workload attn: skip the `workloads` object")
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the two gathered forms of the step")
    ap.add_argument("--sequential", action="store_true", help="block workload: RMSNorm before each sub-block (eight launches)")
    ap.add_argument("--shape", default="", help="override the workload shape (small cases for profiling): attn B,H,S,D,W; "
                    "ffn M,Dm,F; decode B,H,D,T,W; rms_norm M,Dm; block B,S,Dm,H,D,F,W; qkvg M,Dm,H,D")
    ap.add_argument("--attn-schedule", default="per_tile", choices=["persistent", "per_tile"],
                    help="attention kernel: one CTA per 128-query tile (default) or the persistent one")
    ap.add_argument("--attn-item-tiles", type=int, default=0, help="persistent attention: query tiles per item (0 = per launch)")
    ap.add_argument("--gemm-tiling", default="cta_pair", choices=["one_cta", "cta_pair"],
                    help="GEMMs: clusters of two CTAs on 256 x 256 tiles (default) or one CTA per 128 x 256 tile")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, world, local = dist_env()

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from x17ai_b200 import _lib, build, device, kernels as K, sharding
    build.build()
    lib = _lib.load()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local)      # before any pinned allocation
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = device.CudaStream(local)
    K.set_attn_schedule(K.ATTN_PER_TILE if args.attn_schedule == "per_tile" else K.ATTN_PERSISTENT, args.attn_item_tiles)
    K.set_gemm_tiling(K.GEMM_CTA_PAIR if args.gemm_tiling == "cta_pair" else K.GEMM_ONE_CTA)
    run = Runner(torch, dist, lib, device, stream, local, world, dev)
    strong = args.workload == "attn"
    row_sharded = args.workload in ROW_SHARDED and world > 1
    if strong:
        B, H = (_shape(args, 5) or (8, 32, 0, 0, 0))[:2]
        shard = sharding.attn_shard(B, H, world, rank)
        w = WORKLOADS["attn"](stream, dev, args, shard=shard)
    elif row_sharded:
        # the fixed token rows of the workload cut into one block per GPU (whole M tiles), weights replicated
        import types
        fields = list(_shape(args, len(ROW_SHARDED[args.workload])) or ROW_SHARDED[args.workload])
        rows_total = fields[0]
        b, e = sharding.row_shard(rows_total, world, rank)
        if e <= b:
            raise SystemExit(f"{args.workload}: {rows_total} token rows are too few for {world} GPUs")
        fields[0] = e - b
        w = WORKLOADS[args.workload](stream, dev, types.SimpleNamespace(shape=",".join(str(v) for v in fields)))
        w.ops_total = w.ops / (e - b) * rows_total
        w.tokens_total = rows_total
        strong = True
    else:
        w = WORKLOADS[args.workload](stream, dev, args)
    if args.sequential:
        if args.workload != "block":
            raise SystemExit("--sequential applies to --workload block")
        w.make_sequential()
        args.no_e2e = True   # the end-to-end leg times the harness form only

    peaks = measured_peaks()
    lib_peaks = library_tensor_peaks(torch, dev) if rank == 0 else {}
    torch.cuda.synchronize()

    # ---- device-resident timing ----
    dev_total, kernel_avg, wall_total, launches, clocks = run.time_steps(w.step, args.steps, args.warmup)
    unit, scale = ("TOPS", 1e12) if w.bound == "tensor" else ("GB/s", 1e9)
    work_rank = w.ops if w.bound == "tensor" else w.alg_bytes
    work_job = (w.ops_total if strong else world * w.ops) if w.bound == "tensor" else world * w.alg_bytes
    tokens_job = w.tokens_total if strong else world * w.tokens
    value = work_job * args.steps / dev_total / scale
    achieved = work_rank / kernel_avg / scale

    # ---- the same step as a burst: after an idle second, without the load in front of the timed region ----
    burst = None
    if world == 1:
        n_burst = max(3, min(args.steps, 20))
        per, bclk = run.time_burst(w.step, n_burst)
        burst = {"value": work_job / per / scale, "unit": unit, "ms_per_step": per * 1e3, "steps": n_burst, "clocks": bclk,
                 "note": "three untimed steps after an idle second, then the timed steps: the condition of the burst peak"}
        if w.bound == "tensor":
            burst["frac_of_burst"] = burst["value"] / (2.0 * peaks["bf16_burst"])

    # ---- the same step with the outputs gathered on every GPU ----
    gather = None
    if args.workload == "attn" and world > 1 and not args.no_gather:
        info = w.gather_setup(world)
        n = max(5, min(args.steps, 50))
        g_total, _, _, _, _ = run.time_steps(w.step_gather, n, 3)
        o_total, _, _, _, _ = run.time_steps(w.step_gather_overlapped, n, 3)
        gather = dict(info, steps=n, gathered_bytes=int(world * w.out.numel()),
                      ms_per_step_gather_in_step=g_total / n * 1e3, value_gather_in_step=work_job * n / g_total / scale,
                      ms_per_step_gather_overlapped=o_total / n * 1e3, value_gather_overlapped=work_job * n / o_total / scale,
                      note="all_gather_into_tensor (NCCL) of the int8 outputs: once after the kernel; and per chunk on a "
                           "second stream under the next chunk's kernel")
        if w.peers is not None:
            p_total, _, _, _, _ = run.time_steps(w.step_peer_stores, n, 3)
            gather.update(ms_per_step_peer_stores=p_total / n * 1e3, value_peer_stores=work_job * n / p_total / scale,
                          peer_stores="the kernel's epilogue stores each shard into every GPU's buffer over NVLink "
                                      "(x17ai_b200_attn_fwd_i8_to_peers), a device-side barrier between the ranks closes "
                                      "the step; no gather pass")
        else:
            gather["peer_stores"] = "not run: " + w.peer_note

    # ---- end to end through the C ABI with host buffers ----
    e2e = None
    if not args.no_e2e:
        w.host_buffers()
        e2e_sync = getattr(w, "e2e_sync", stream.synchronize)
        for _ in range(2):
            w.e2e_step()
        e2e_sync()
        run.barrier()
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
        e2e = {"value": work_job / e2e_time / scale, "unit": unit,
               "h2d_bytes_per_step": int(w.h2d) * world, "d2h_bytes_per_step": int(w.d2h) * world,
               "h2d_bytes_per_rank": int(w.h2d), "h2d_gbs_per_rank": w.h2d / e2e_time / 1e9,
               "ms_per_step": e2e_time * 1e3, "steps": n_e2e, "clock": "host, between stream synchronisations",
               "streams": len(getattr(w, "e2e_streams", [stream])), "host_numa": numa}

    line = {
        "metric": METRICS[args.workload],
        "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_total / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic (seeded N(0,1) values quantised to FixedI8 codes)",
        "config": attn_line_config(w.B, w.H, w.S, w.D, w.W, world) if args.workload == "attn" else dict(w.config, sharding=(
            (f"the fixed {w.tokens_total} token rows cut into {world} blocks of whole M tiles, one per GPU, weights replicated, "
             "no collective in the path" if row_sharded else
             f"the fixed batch cut into {world} shards of (sequence, head) units, one per GPU, no collective in the path")
            if strong else f"{world} x per-GPU workload, token-row units, no collective")),
        "load_before_timed_region": f"{PRELOAD_S} s of the same step after the warm-up steps, back to back",
        "tokens_per_s": tokens_job * args.steps / dev_total,
        "roofline": dict(roofline(w, achieved, dev_total, peaks, lib_peaks, args.workload, clocks), kernel_ms=kernel_avg * 1e3),
        "clocks": clocks,
        "gpu_launches": int(launches),
        "wall_ms_per_step": wall_total / args.steps * 1e3,
        "attn_schedule": args.attn_schedule, "gemm_tiling": args.gemm_tiling,
    }
    if burst is not None:
        line["burst"] = burst
    if args.workload == "block" and world == 1 and not args.sequential:
        line["stages"] = w.stage_times()
    if gather is not None:
        line["gather"] = gather
    if args.workload in ("attn", "attn_pv_fp8", "attn_scaled"):
        line["reference_count_tops"] = (w.ref_ops if strong else world * w.ref_ops) * args.steps / dev_total / 1e12
    if e2e is not None:
        line["e2e"] = e2e

    if rank == 0 and world == 1:
        if args.workload == "attn":
            try:
                rk = w.ref_kernel_sample()
                if rk is not None:
                    line["ref_kernel_baseline"] = rk
            except Exception as e:
                line["ref_kernel_baseline"] = {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
        if not args.no_cpu_baseline:
            rate, sample = w.cpu_sample()
            line["cpu_baseline"] = {"value": rate / scale, "unit": unit, "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": sample}
            if args.workload == "attn":
                ref = reference_cpu_attention()
                if ref is not None:
                    line["cpu_reference_model"] = ref

    # ---- the other kernels of the path (N = 1, default workload) ----
    if rank == 0 and world == 1 and args.workload == "attn" and not args.no_side_workloads and not args.shape:
        del w
        torch.cuda.empty_cache()
        side = {}
        for name in SIDE_WORKLOADS:
            try:
                sw = WORKLOADS[name](stream, dev, None)
                n = run.steps_for(sw.step, 0.7)
                d_total, k_avg, _, n_launch, clk = run.time_steps(sw.step, n, 3)
                u, sc = ("TOPS", 1e12) if sw.bound == "tensor" else ("GB/s", 1e9)
                work = sw.ops if sw.bound == "tensor" else sw.alg_bytes
                side[name] = {"metric": METRICS[name], "value": work * n / d_total / sc, "unit": u, "steps": n,
                              "ms_per_step": d_total / n * 1e3, "tokens_per_s": sw.tokens * n / d_total, "dtype": sw.dtype,
                              "config": sw.config, "gpu_launches": n_launch, "clocks": clk,
                              "roofline": roofline(sw, work / k_avg / sc, d_total, peaks, lib_peaks, name, clk)}
                del sw
            except Exception as e:   # one workload must not cost the headline its line
                side[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
            torch.cuda.empty_cache()
        line["workloads"] = side
        line["library_peaks"] = lib_peaks

    if rank == 0:
        print(json.dumps(line), flush=True)
    stream.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
