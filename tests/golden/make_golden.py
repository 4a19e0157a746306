#!/usr/bin/env python3
"""Generate golden fixtures by running the reference's own float64 PyTorch model.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference reads its shapes from `block.config.json` beside its scripts and writes into
`tmp/block_torch/` beside them, so the three scripts it needs (new_block.py, block_utils.py,
jsonc.py) are copied into a scratch directory together with a small config, executed there
unmodified (`python new_block.py --create-inputs`), and every tensor it stores is collected
into one `.npz` per config next to this file.  Nothing of the reference is kept in the
repository: only the numbers it produced.

Stored per config (names follow the reference's file names, new_block.py:54-81,148-158,296-321):
  inputs   x_i8, sinks_k_i8, sinks_v_i8, attn_temperature_f32, attn_q_weights_i8,
           attn_kv_weights_i8, attn_y_weights_i8, ffn_f_weights_i8, ffn_y_weights_i8
  goldens  q_i8, kv_i8, k_rrms_f32, attn_out_i8, attn_l_f32, attn_out_f32, attn_y_f8,
           attn_y_i8, ffn_f_f8, ffn_y_f8, ffn_y_i8
"""
import json
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

CONFIGS = {
    # name: (seq_len, MODEL_DIM, HEAD_DIM, N_HEADS, F_WIDTH, WINDOW_SIZE)
    "block_d64_w64": (256, 256, 64, 4, 256, 64),
    "block_d128_w128": (384, 256, 128, 2, 256, 128),
    "block_d32_w0": (128, 128, 32, 4, 128, 0),
}

I8 = ["x", "sinks_k", "sinks_v", "attn_q_weights", "attn_kv_weights", "attn_y_weights",
      "ffn_f_weights", "ffn_y_weights", "q", "kv", "attn_out", "attn_y", "ffn_y"]
F32 = ["attn_temperature", "k_rrms", "attn_l", "attn_out"]
F8 = ["ffn_f"]


def run_config(ref: Path, name: str, cfg) -> None:
    seq, dm, hd, nh, fw, win = cfg
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        for f in ("new_block.py", "block_utils.py", "jsonc.py"):
            shutil.copy(ref / f, tmp / f)
        (tmp / "block.config.json").write_text(json.dumps({
            "seq_len": seq, "MODEL_DIM": dm, "HEAD_DIM": hd, "N_HEADS": nh, "F_WIDTH": fw,
            "WINDOW_SIZE": win, "L2_NORM_EPS": 2.0 ** -70, "V_SCALE_FIX": 1.3,
        }))
        subprocess.run([sys.executable, "new_block.py", "--create-inputs"], cwd=tmp, check=True,
                       stdout=subprocess.DEVNULL)
        d = tmp / "tmp" / "block_torch"
        out = {"config": np.array([seq, dm, hd, nh, fw, win], dtype=np.int64)}
        for n in I8:
            out[f"{n}_i8"] = np.fromfile(d / f"{n}_i8.bin", dtype=np.int8)
        for n in F32:
            out[f"{n}_f32"] = np.fromfile(d / f"{n}_f32.bin", dtype=np.float32)
        for n in F8:
            out[f"{n}_f8"] = np.fromfile(d / f"{n}_f8.bin", dtype=np.uint8)
        # the e4m3 forms of the two gated-residual outputs exist only as safetensors
        import torch
        from safetensors.torch import load_file as load_torch
        for n in ("attn_y", "ffn_y"):
            t = next(iter(load_torch(str(d / f"{n}_f8.safetensors")).values()))
            out[f"{n}_f8"] = t.view(torch.uint8).numpy().reshape(-1)
        np.savez_compressed(Path(__file__).parent / f"{name}.npz", **out)
        print(f"wrote {name}.npz")


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>")
    ref = Path(sys.argv[1])
    for name, cfg in CONFIGS.items():
        run_config(ref, name, cfg)


if __name__ == "__main__":
    main()
