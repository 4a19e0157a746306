"""The reference's block harness (src/main.rs:37-386) over this library: read the input tensors from
safetensors files, run the six launches with a device timer around each, write the eight output
tensors, and print what was loaded, the dimensions, each kernel's time and rate, and what was stored.

    python -m x17ai_b200.block_main TENSOR_DIR OUTPUT_DIR --heads 64 --head-dim 32 --window 0

The reference compiles N_HEADS, HEAD_DIM and WINDOW_SIZE in (src/main.rs:29-35); here they are
arguments, model_dim and the FFN width come from the weight shapes. The output files carry the
names and layouts the reference's own comparison scripts read (check.sh).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

from . import X17Error
from .block import BlockForward
from .device import CudaStream

# report names of the six stages, in launch order (src/main.rs:355-372)
REPORT_NAMES = {"attn_q": "attn_q_fwd", "attn_kv": "attn_kv_fwd", "attn": "attn_fwd_i8", "attn_y": "attn_y_fwd",
                "ffn_f": "ffn_f_fwd", "ffn_y": "ffn_y_fwd_f8"}


def run(tensor_dir, output_dir, n_heads: int, head_dim: int, window_size: int, fused_qkv: bool = False,
        device_id: int = 0, out=sys.stdout, kernel_objects: bool = False) -> dict:
    """Runs the harness once; returns {stage: seconds}."""
    import torch
    torch.cuda.set_device(device_id)
    with CudaStream(device_id) as stream:
        blk, x = BlockForward.from_directory(stream, tensor_dir, n_heads, head_dim, window_size, fused_qkv=fused_qkv,
                                             kernel_objects=kernel_objects)
        if x is None:
            raise X17Error(f"{Path(tensor_dir) / 'x_i8.safetensors'} not found")
        result = blk.forward(x, timed=True)
        stream.synchronize()
        blk.save_outputs(output_dir, result)
        c, rows = blk.config, x.shape[0]
        p = lambda *a: print(*a, file=out)
        p("loaded:")
        for name, t in (("x", x), ("attn_q_weights", blk.w_q), ("attn_kv_weights", blk.w_kv), ("ffn_f_weights", blk.w_ffn_f),
                        ("ffn_y_weights", blk.w_ffn_y), ("attn_y_weights", blk.w_attn_y), ("sinks_k", blk.sink_k),
                        ("sinks_v", blk.sink_v), ("attn_temperature", blk.attn_temperature)):
            p(f"\t{name}: {list(t.shape)} {t.dtype}, {t.numel() * t.element_size()} bytes")
        p("dimensions:")
        p(f"\tn_inputs={rows}, model_dim={c.model_dim}, n_heads={c.n_heads}, head_dim={c.head_dim}, "
          f"attn_width={c.attn_width}, f_width={c.ffn_width}, window_size={c.window_size}")
        p("launched:")
        ops = blk.n_ops(rows)
        seconds = dict(blk.seconds)
        if blk.fused_qkv:   # one launch wrote Q, KV and the K scales
            ops["attn_q"] += ops.pop("attn_kv")
            seconds.pop("attn_kv")
        for stage, name in REPORT_NAMES.items():
            if stage in seconds:
                name = "qkvg_fwd_i8" if blk.fused_qkv and stage == "attn_q" else name
                p(f"\t{name} in {seconds[stage] * 1e3:.4f} ms, {ops[stage] / seconds[stage] / 1e12:.3f} TOPS")
        p("stored:")
        for name in blk.OUTPUT_FILES.values():
            p(f"\t{Path(output_dir) / (name + '.safetensors')}")
        return seconds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("tensor_dir")
    ap.add_argument("output_dir")
    ap.add_argument("--heads", type=int, required=True)
    ap.add_argument("--head-dim", type=int, required=True)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--fused-qkv", action="store_true")
    ap.add_argument("--kernel-objects", action="store_true",
                    help="launch kernel.cubin + meta.json objects through load_module / get_kernel / launch_kernel, as the "
                         "reference's host does with its own kernels (all stages but the e4m3 x int8 projection)")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)
    try:
        run(a.tensor_dir, a.output_dir, a.heads, a.head_dim, a.window, a.fused_qkv, a.device, kernel_objects=a.kernel_objects)
    except X17Error as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
