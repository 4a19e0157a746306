#!/usr/bin/env python3
"""Builds the reference's OWN int8 attention kernel for sm_100a, as a second checker beside the
numpy restatement. Test infrastructure only: nothing in the product imports, links or runs it.

The reference renders `templates/attn/{common.cuh, kernel.cu, meta.cu}` with the shape constants
and compiles the result against `cuda/attn_fwd_i8.cuh` (src/device/cuda/attn.rs:171-232,
kernel_build.rs:38-134, 200-220). This script does the same from the sources where they lie in a
checkout of the reference: it reads the three template files there, fills in the constants,
points the one relative include at the checkout, and runs nvcc with the reference's own flags
(only the architecture differs: sm_100a instead of sm_86). Everything it writes goes to
`oracle/_ref/attn_h<H>_d<D>/` (git-ignored): the rendered sources, `kernel.cubin`, `meta.json`.
No text of the reference is kept in the repository.

    python oracle/build_ref.py /path/to/reference            # the configurations the tests and bench use
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# (n_heads, head_dim): the three fixture shapes of tests/golden and the benchmark shape
CONFIGS = [(4, 64), (2, 128), (4, 32), (32, 128)]

# kernel_build.rs:200-220, with the architecture replaced and the CUTLASS include paths (unused by
# the attention kernel) left out
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "--ftz=true", "--prec-div=false",
              "--fmad=true", "--use_fast_math", "-DX17_PRECISE_MATH=0", "--expt-relaxed-constexpr",
              "-maxrregcount=255", "-O3"]


def heads_per_kernel(head_dim: int) -> int:
    """attn.rs:56-62."""
    return max(128 // head_dim, 1)


def ref_dir(n_heads: int, head_dim: int) -> Path:
    return OUT / f"attn_h{n_heads}_d{head_dim}"


def build_one(ref: Path, n_heads: int, head_dim: int, force: bool = False) -> Path:
    d = ref_dir(n_heads, head_dim)
    cubin, meta = d / "kernel.cubin", d / "meta.json"
    kernel_header = ref / "cuda" / "attn_fwd_i8.cuh"
    newest = max(p.stat().st_mtime for p in (ref / "cuda").glob("*.cuh"))
    if not force and cubin.exists() and meta.exists() and cubin.stat().st_mtime >= newest:
        return d
    src = d / "src"
    src.mkdir(parents=True, exist_ok=True)
    hd = n_heads * head_dim
    values = {"n_heads": n_heads, "heads_per_kernel": heads_per_kernel(head_dim), "head_dim": head_dim,
              "q_stride": hd, "kv_stride": 2 * hd, "o_stride": hd}
    for name in ("common.cuh", "kernel.cu", "meta.cu"):
        text = (ref / "templates" / "attn" / name).read_text()
        for key, val in values.items():
            text = text.replace("{{" + key + "}}", str(val))
        text = text.replace('"../../../cuda/attn_fwd_i8.cuh"', f'"{kernel_header}"')
        if "{{" in text:
            raise SystemExit(f"{name}: a template constant was left unfilled")
        (src / name).write_text(text)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise SystemExit(f"{' '.join(map(str, cmd))}\n{res.stdout}{res.stderr}")
        return res.stdout

    run([nvcc, *NVCC_FLAGS, "--cubin", "-o", str(cubin), str(src / "kernel.cu")])
    run([nvcc, *NVCC_FLAGS, "-o", str(d / "meta"), str(src / "meta.cu")])
    meta.write_text(json.dumps(dict(json.loads(run([str(d / "meta")])), **values), indent="\t") + "\n")
    return d


def build_all(ref: Path, force: bool = False) -> list:
    return [build_one(ref, h, dd, force) for h, dd in CONFIGS]


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: build_ref.py <checkout of the reference project> [--force]")
    for out in build_all(Path(sys.argv[1]), "--force" in sys.argv):
        print(out)
