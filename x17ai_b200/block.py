"""The reference's block forward as one object: the six launches of src/main.rs:193-255 in its
order, on buffers allocated once.

  q      = attn_q_fwd(x, W_q)                      FixedI8            (main.rs:195-200)
  kv     = attn_kv_fwd(x, W_kv)  + k_rrms          FixedI8, K rows L2-normalised per head (:204-209)
  attn   = attn_fwd_i8(q, kv, sinks, temperature)  FixedI8 + L        (:213-222)
  attn_y = attn_y_fwd(attn, W_attn_y, residual x)  e4m3               (:226-231)
  ffn_f  = ffn_f_fwd(x, W_ffn_f)                   e4m3 (GeGLU)       (:235-240)
  ffn_y  = ffn_y_fwd_f8(ffn_f, W_ffn_y, residual x) e4m3              (:244-249)

Like the reference's harness, both output projections take `x` as the residual and the FFN reads
`x`: the six kernels are the block's kernels, each fed the tensor the reference feeds it.
`fused_qkv=True` replaces the first two launches by the single fused projection.
Every launch goes through the C ABI on the given stream; nothing here computes on the host.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import kernels as K
from .device import CudaGraph, CudaTimer


@dataclass(frozen=True)
class BlockConfig:
    """Shape constants of the reference's harness (src/main.rs:30-47)."""
    model_dim: int
    n_heads: int
    head_dim: int
    ffn_width: int
    window_size: int

    @property
    def attn_width(self) -> int:
        return self.n_heads * self.head_dim


class BlockForward:
    """Weights are int8 device tensors in the reference's layouts ([outputs, inputs], trans = true):
    w_q [H*D, Dm], w_kv [2*H*D, Dm] (per head K then V), w_attn_y [2*Dm, H*D], w_ffn_f [2*F, Dm],
    w_ffn_y [2*Dm, F]; sinks [H, D] int8; temperature [H] f32."""

    STAGES = ("attn_q", "attn_kv", "attn", "attn_y", "ffn_f", "ffn_y")

    def __init__(self, stream, config: BlockConfig, w_q, w_kv, w_attn_y, w_ffn_f, w_ffn_y, sink_k, sink_v,
                 attn_temperature, fused_qkv: bool = False, kernel_objects: bool = False):
        c = self.config = config
        self.stream = stream
        self.fused_qkv = fused_qkv
        hd = c.attn_width
        if fused_qkv and hd % 256 != 0:
            raise K.X17Error(f"fused_qkv needs n_heads * head_dim to be a multiple of 256, got {hd}")
        self.w_q, self.w_kv, self.w_attn_y, self.w_ffn_f, self.w_ffn_y = w_q, w_kv, w_attn_y, w_ffn_f, w_ffn_y
        self.sink_k, self.sink_v, self.attn_temperature = sink_k, sink_v, attn_temperature
        self.k_q = K.GemmKernel(K.attn_q_fwd_config(c.model_dim, hd))
        self.k_kv = K.GemmKernel(K.attn_kv_fwd_config(c.model_dim, 2 * hd, c.head_dim))
        self.k_attn = K.AttnKernel(K.AttnKernelConfig(c.n_heads, c.head_dim, hd, 2 * hd, hd))
        self.k_attn_y = K.GemmKernel(K.attn_y_fwd_config(hd, c.model_dim))
        self.k_ffn_f = K.GemmKernel(K.ffn_f_fwd_config(c.model_dim, c.ffn_width))
        self.k_ffn_y = K.GemmKernel(K.ffn_y_fwd_f8_config(c.ffn_width, c.model_dim))
        if kernel_objects:
            # all six kernels as kernel objects (kernel.cubin + meta.json, launched through the generic
            # load_module / get_kernel / launch_kernel with the reference's grids and arguments) in place of
            # the library's entry points; the e4m3 x int8 projection's object keeps its own e4m3 planes of
            # the int8 weights, made by one set-up launch
            if fused_qkv:
                raise K.X17Error("kernel_objects and fused_qkv exclude each other (the fused projection has no kernel object)")
            from . import kernel_objects as KO
            tag = f"{c.model_dim}_{c.n_heads}x{c.head_dim}_{c.ffn_width}"
            self.k_q = KO.GemmObject(stream, self.k_q.config, f"attn_q_{tag}")
            self.k_kv = KO.GemmObject(stream, self.k_kv.config, f"attn_kv_{tag}")
            self.k_attn_y = KO.GemmObject(stream, self.k_attn_y.config, f"attn_y_{tag}")
            self.k_ffn_f = KO.GemmObject(stream, self.k_ffn_f.config, f"ffn_f_{tag}")
            self.k_attn = KO.AttnObject(stream, self.k_attn.config, f"attn_{tag}")
            self.k_ffn_y = KO.GemmObject(stream, self.k_ffn_y.config, f"ffn_y_f8_{tag}")
        # e4m3 activations x int8 weights run on the fp8 tensor path with the weights split once (the kernel
        # object does that itself from the int8 weights it is given)
        if kernel_objects:
            self.k_ffn_y.prepare(stream, w_ffn_y)
            self.w_ffn_y_split = w_ffn_y
        else:
            self.w_ffn_y_split = K.split_i8_weights(stream, w_ffn_y)
        if fused_qkv:
            self.w_qkv = torch.cat((w_q, w_kv), dim=0).contiguous()
        stream.synchronize()
        self._rows = 0
        self._timers = None
        self._graph = None
        self._graph_x = None

    # file names of the reference's harness (src/main.rs:39-71)
    FILES = {"w_q": "attn_q_weights_i8", "w_kv": "attn_kv_weights_i8", "w_attn_y": "attn_y_weights_i8",
             "w_ffn_f": "ffn_f_weights_i8", "w_ffn_y": "ffn_y_weights_i8", "sink_k": "sinks_k_i8",
             "sink_v": "sinks_v_i8", "attn_temperature": "attn_temperature_f32"}

    @classmethod
    def from_directory(cls, stream, directory, n_heads: int, head_dim: int, window_size: int, fused_qkv: bool = False,
                       kernel_objects: bool = False):
        """Builds the block from the safetensors files the reference's harness reads (one tensor per
        file, `<name>.safetensors`), inferring model_dim and the FFN width from the weight shapes with
        the checks of validate_*_inputs (src/main.rs:257-385). Returns (block, x) with the input
        sequence `x_i8.safetensors` uploaded too when it exists, else x is None."""
        from pathlib import Path
        from . import tensor_io
        d = Path(directory)
        t = {k: tensor_io.load_to_device(d / f"{name}.safetensors", stream) for k, name in cls.FILES.items()}
        hd = n_heads * head_dim
        w_q = t["w_q"]
        if w_q.dim() != 2 or w_q.shape[0] != hd:
            raise K.X17Error(f"attn_q weights must be [{hd}, model_dim], got {list(w_q.shape)}")
        model_dim = w_q.shape[1]
        w_kv = t["w_kv"].reshape(2 * hd, model_dim)          # main.rs:82 flattens the KV weights the same way
        w_attn_y = t["w_attn_y"].reshape(2 * model_dim, hd)
        w_ffn_f = t["w_ffn_f"]
        if w_ffn_f.dim() != 2 or w_ffn_f.shape[1] != model_dim or w_ffn_f.shape[0] % 2 != 0:
            raise K.X17Error(f"ffn_f weights must be [2 * ffn_width, {model_dim}], got {list(w_ffn_f.shape)}")
        ffn_width = w_ffn_f.shape[0] // 2
        w_ffn_y = t["w_ffn_y"].reshape(2 * model_dim, ffn_width)
        blk = cls(stream, BlockConfig(model_dim, n_heads, head_dim, ffn_width, window_size), w_q, w_kv, w_attn_y, w_ffn_f,
                  w_ffn_y, t["sink_k"].reshape(n_heads, head_dim), t["sink_v"].reshape(n_heads, head_dim),
                  t["attn_temperature"].reshape(n_heads), fused_qkv=fused_qkv, kernel_objects=kernel_objects)
        x_path = d / "x_i8.safetensors"
        x = tensor_io.load_to_device(x_path, stream).reshape(-1, model_dim) if x_path.exists() else None
        return blk, x

    # output file names and dtypes' suffixes of the reference's harness (src/main.rs:273-280)
    OUTPUT_FILES = {"q": "q_i8", "kv": "kv_i8", "k_rrms": "k_rrms_f32", "attn_out": "attn_out_i8", "attn_l": "attn_l_f32",
                    "attn_y": "attn_y_f8", "ffn_f": "ffn_f_f8", "ffn_y": "ffn_y_f8"}

    def save_outputs(self, directory, out: dict) -> None:
        """Downloads the tensors forward() returned and writes them as the reference's harness does
        (src/main.rs:255-280): one file per tensor, KV as [rows, heads, 2, head_dim], e4m3 tensors as
        F8_E4M3."""
        from pathlib import Path
        from . import tensor_io
        c = self.config
        for key, name in self.OUTPUT_FILES.items():
            host = tensor_io.download(out[key], self.stream)
            if key == "kv":
                host = host.reshape(-1, c.n_heads, 2, c.head_dim)
            if name.endswith("_f8"):
                host = host.view(torch.float8_e4m3fn)
            tensor_io.write_safetensors_file(Path(directory) / f"{name}.safetensors", host)

    def forward_layer(self, h) -> dict:
        """The sequential form of the layer, eight launches: the hidden state `h` [rows, model_dim] e4m3
        is normalised (Rms_norm::kernel, rms_norm.cu:55-113: e4m3 in, FixedI8 out), goes through the
        attention sub-block with itself as the residual, and the sub-block's e4m3 output is normalised
        again and goes through the FFN sub-block the same way. The reference's harness feeds one x to
        both sub-blocks (src/main.rs:193-255, forward()); this is the order the two formats imply,
        every sub-block reading FixedI8 and writing e4m3. Returns forward()'s tensors plus the two
        normalised inputs; `ffn_y` is the next layer's `h`."""
        c, s = self.config, self.stream
        rows, _ = K.matrix_shape("block", "h", h, (None, c.model_dim), K.DTYPE_E4M3)
        self._buffers(rows, h.device)
        K.rms_norm(s, K.RMS_E4M3_FIXED, h, self.x_attn)
        x = self.x_attn
        if self.fused_qkv:
            K.qkvg_fwd_i8(s, x, self.w_qkv, c.n_heads, c.head_dim, self.q, self.kv, self.k_rrms)
        else:
            self.k_q.launch(s, x, self.w_q, self.q)
            self.k_kv.launch(s, x, self.w_kv, self.kv, rrms=self.k_rrms)
        self.k_attn.launch(s, self.q, self.kv, self.sink_k, self.sink_v, self.attn_temperature, self.attn_out,
                           self.attn_l, c.window_size)
        self.k_attn_y.launch(s, self.attn_out, self.w_attn_y, self.attn_y, residual=x)
        K.rms_norm(s, K.RMS_E4M3_FIXED, self.attn_y, self.x_ffn)
        self.k_ffn_f.launch(s, self.x_ffn, self.w_ffn_f, self.ffn_f)
        self.k_ffn_y.launch(s, self.ffn_f, self.w_ffn_y_split, self.ffn_y, residual=self.x_ffn)
        return {"x_attn": self.x_attn, "q": self.q, "kv": self.kv, "k_rrms": self.k_rrms, "attn_out": self.attn_out,
                "attn_l": self.attn_l, "attn_y": self.attn_y, "x_ffn": self.x_ffn, "ffn_f": self.ffn_f, "ffn_y": self.ffn_y}

    def capture(self, x) -> dict:
        """Records the launches of forward(x) as one graph; replay() then re-runs them on whatever `x`
        and the weights hold at that moment (same buffers, one driver call). Runs forward(x) once
        first so that no kernel is launched for the first time inside the recording."""
        out = self.forward(x)
        self.stream.synchronize()
        if self._graph is not None:
            self._graph.destroy()
        with CudaGraph(self.stream) as g:
            self.forward(x)
        self._graph, self._graph_x = g, x
        return out

    def replay(self) -> None:
        if self._graph is None:
            raise K.X17Error("BlockForward.replay(): capture(x) first")
        self._graph.launch()

    def _buffers(self, rows: int, device):
        if rows == self._rows:
            return
        if self._graph is not None:
            # the recording holds the addresses of the buffers that are about to be replaced
            self._graph.destroy()
            self._graph = None
        c, hd = self.config, self.config.attn_width
        e = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=device)
        self.q = e(rows, hd, dtype=torch.int8)
        self.kv = e(rows, 2 * hd, dtype=torch.int8)
        self.k_rrms = e(rows, c.n_heads, dtype=torch.float32)
        self.attn_out = e(rows, hd, dtype=torch.int8)
        self.attn_l = e(c.n_heads, rows, dtype=torch.float32)
        self.attn_y = e(rows, c.model_dim, dtype=torch.uint8)
        self.ffn_f = e(rows, c.ffn_width, dtype=torch.uint8)
        self.ffn_y = e(rows, c.model_dim, dtype=torch.uint8)
        self.x_attn = e(rows, c.model_dim, dtype=torch.int8)   # forward_layer: RMSNorm of the incoming hidden state
        self.x_ffn = e(rows, c.model_dim, dtype=torch.int8)    # forward_layer: RMSNorm of attn_y
        torch.cuda.synchronize(device)
        self._rows = rows

    def n_ops(self, rows: int) -> dict:
        """Operation counts per stage in the reference's conventions (gemm.rs:445-449, attn.rs:449-471)."""
        c = self.config
        return {
            "attn_q": self.k_q.config.n_ops(rows),
            "attn_kv": self.k_kv.config.n_ops(rows),
            "attn": self.k_attn.config.n_ops(rows, c.window_size),
            "attn_y": self.k_attn_y.config.n_ops(rows),
            "ffn_f": self.k_ffn_f.config.n_ops(rows),
            "ffn_y": self.k_ffn_y.config.n_ops(rows),
        }

    def forward(self, x, timed: bool = False) -> dict:
        """One sequence `x` [rows, model_dim] int8 (FixedI8 codes) through the six kernels. Returns the
        device tensors by the reference's names; with `timed`, `self.seconds` holds per-stage device
        times after the call (the call then synchronises, like the harness)."""
        c, s = self.config, self.stream
        rows, _ = K.matrix_shape("block", "x", x, (None, c.model_dim), K.DTYPE_INT8)
        self._buffers(rows, x.device)
        if timed and self._timers is None:
            self._timers = {name: CudaTimer(s) for name in self.STAGES}
        t = self._timers if timed else None

        def stage(name, fn):
            if t is not None:
                t[name].start()
            fn()
            if t is not None:
                t[name].stop()

        if self.fused_qkv:
            stage("attn_q", lambda: K.qkvg_fwd_i8(s, x, self.w_qkv, c.n_heads, c.head_dim, self.q, self.kv, self.k_rrms))
            stage("attn_kv", lambda: None)
        else:
            stage("attn_q", lambda: self.k_q.launch(s, x, self.w_q, self.q))
            stage("attn_kv", lambda: self.k_kv.launch(s, x, self.w_kv, self.kv, rrms=self.k_rrms))
        stage("attn", lambda: self.k_attn.launch(s, self.q, self.kv, self.sink_k, self.sink_v, self.attn_temperature,
                                                 self.attn_out, self.attn_l, c.window_size))
        stage("attn_y", lambda: self.k_attn_y.launch(s, self.attn_out, self.w_attn_y, self.attn_y, residual=x))
        stage("ffn_f", lambda: self.k_ffn_f.launch(s, x, self.w_ffn_f, self.ffn_f))
        stage("ffn_y", lambda: self.k_ffn_y.launch(s, self.ffn_f, self.w_ffn_y_split, self.ffn_y, residual=x))
        if t is not None:
            s.synchronize()
            self.seconds = {name: t[name].elapsed_seconds() for name in self.STAGES}
        return {"q": self.q, "kv": self.kv, "k_rrms": self.k_rrms, "attn_out": self.attn_out, "attn_l": self.attn_l,
                "attn_y": self.attn_y, "ffn_f": self.ffn_f, "ffn_y": self.ffn_y}
