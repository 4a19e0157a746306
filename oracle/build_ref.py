#!/usr/bin/env python3
"""Builds the reference's OWN attention and GEMM kernels for sm_100a, as a second checker beside the
numpy restatement. Test infrastructure only: nothing in the product imports, links or runs it.

The reference renders `templates/attn/{common.cuh, kernel.cu, meta.cu}` with the shape constants
and compiles the result against `cuda/attn_fwd_i8.cuh` (src/device/cuda/attn.rs:171-232,
kernel_build.rs:38-134, 200-220). This script does the same from the sources where they lie in a
checkout of the reference: it reads the three template files there, fills in the constants,
points the one relative include at the checkout, and runs nvcc with the reference's own flags
(only the architecture differs: sm_100a instead of sm_86). Everything it writes goes to
`oracle/_ref/attn_h<H>_d<D>/` (git-ignored): the rendered sources, `kernel.cubin`, `meta.json`.
The five GEMMs of the block (`templates/basic_gemm`, constants of src/main.rs:387-675) are built the
same way for the three fixture shapes into `oracle/_ref/gemm_<kernel>_<fixture>/`.
No text of the reference is kept in the repository.

    python oracle/build_ref.py /path/to/reference            # the configurations the tests and bench use
"""
from __future__ import annotations

import json
import math
import os
import re
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


# ---- the reference's GEMM kernels (templates/basic_gemm) ------------------------------------------------

FIXED_I8_SCALE = 8.0                                     # src/main.rs:33
L2_NORM_EPS = 1.0 / (1024.0 ** 7)                        # src/main.rs:35
GELU_VAR_FIX_2 = 1.0 / ((1.0 / 3.0) + (0.5 / math.pi) * (1.0 / math.sqrt(3.0)))  # src/main.rs:650

# (sequence, model_dim, head_dim, n_heads, ffn_width) of the three fixtures in tests/golden
GEMM_SHAPES = {"block_d64_w64": (256, 256, 64, 4, 256), "block_d128_w128": (384, 256, 128, 2, 256),
               "block_d32_w0": (128, 128, 32, 4, 128)}


def cpp_f64(v: float) -> str:
    """format_cpp_f64 (gemm.rs:257-259)."""
    return f"{v:.17e}"


def render(text: str, ctx: dict) -> str:
    """The subset of the template language the reference's GEMM templates use: {{a.b}},
    {% if a.b %} / {% else %} / {% endif %} (nested) and the one {% match b_rows %} block."""
    def lookup(name):
        v = ctx
        for part in name.strip().split("."):
            v = v[part]
        return v
    out, emit = [], [True]
    for tok in re.split(r"({%-?.*?-?%}|{{.*?}})", text, flags=re.S):
        if tok.startswith("{{"):
            if all(emit):
                out.append(str(lookup(tok[2:-2])))
        elif tok.startswith("{%"):
            body = tok.strip("{}%- \t\n")
            if body.startswith("if "):
                emit.append(bool(lookup(body[3:])))
            elif body == "else":
                emit[-1] = not emit[-1]
            elif body in ("endif", "endmatch"):
                emit.pop()
            elif body.startswith("match "):
                emit.append(False)
            elif body.startswith("when Some"):
                emit[-1] = ctx["b_rows"] is not None
                ctx = dict(ctx, rows=ctx["b_rows"])
            elif body.startswith("when None"):
                emit[-1] = ctx["b_rows"] is None
            else:
                raise SystemExit(f"template construct not handled: {tok}")
        elif all(emit):
            out.append(tok)
    return "".join(out)


def gemm_kernels(shape) -> dict:
    """The five GEMMs of the block with the constants of src/main.rs:387-675 and the writer
    descriptions of gemm.rs:84-256."""
    S, Dm, D, H, F = shape
    hd = H * D
    inv_sqrt = lambda x: 1.0 / math.sqrt(float(x))
    blank = dict(use_l2_norm=False, use_geglu=False, use_residual=False, head_dim=0, sep_dim=0, eps_val="",
                 head_scale_val="", head_scale_dscr="", sep_scale_val="", sep_scale_dscr="", inp_scale_val="",
                 inp_scale_dscr="", out_scale_val="", out_scale_dscr="", has_rrms_output=False, has_residual_input=False)
    i8 = ("i8", "I8MatrixLoader")
    e4 = ("b8::E4m3", "E4m3MatrixLoader")
    proj = inv_sqrt(Dm) / (FIXED_I8_SCALE * FIXED_I8_SCALE)
    k = {}
    k["attn_q"] = dict(a=i8, b=i8, a_cols=Dm, b_rows=hd, writer=dict(
        blank, c_type="i8", store_type="b8::I8Store", c_stride_expr="b_rows", inp_scale_val=cpp_f64(proj),
        out_scale_val=cpp_f64(FIXED_I8_SCALE)))
    k["attn_kv"] = dict(a=i8, b=i8, a_cols=Dm, b_rows=2 * hd, writer=dict(
        blank, use_l2_norm=True, c_type="i8", store_type="b8::I8Store", c_stride_expr="b_rows", head_dim=D, sep_dim=D,
        eps_val=cpp_f64(L2_NORM_EPS), head_scale_val=cpp_f64(FIXED_I8_SCALE * math.sqrt(float(D))),
        sep_scale_val=cpp_f64(proj * FIXED_I8_SCALE), has_rrms_output=True))
    k["attn_y"] = dict(a=i8, b=i8, a_cols=hd, b_rows=2 * Dm, writer=dict(
        blank, use_residual=True, c_type="b8::E4m3", store_type="b8::E4m3Store", c_stride_expr="b_rows / 2",
        inp_scale_val=cpp_f64(inv_sqrt(hd) / (FIXED_I8_SCALE * FIXED_I8_SCALE)), out_scale_val=cpp_f64(1.0),
        has_residual_input=True))
    k["ffn_f"] = dict(a=i8, b=i8, a_cols=Dm, b_rows=2 * F, writer=dict(
        blank, use_geglu=True, c_type="b8::E4m3", store_type="b8::E4m3Store", c_stride_expr="b_rows / 2",
        inp_scale_val=cpp_f64(proj), out_scale_val=cpp_f64(1.0)))
    k["ffn_y"] = dict(a=e4, b=i8, a_cols=F, b_rows=2 * Dm, writer=dict(
        blank, use_residual=True, c_type="b8::E4m3", store_type="b8::E4m3Store", c_stride_expr="b_rows / 2",
        inp_scale_val=cpp_f64(math.sqrt(GELU_VAR_FIX_2 / float(F)) / FIXED_I8_SCALE), out_scale_val=cpp_f64(1.0),
        has_residual_input=True))
    return k


def build_gemm(ref: Path, fixture: str, kind: str, cfg: dict, force: bool = False):
    """Returns the directory, or None where the reference's kernel does not compile for the shape (its
    L2-norm writer only takes heads of up to 32 columns)."""
    d = OUT / f"gemm_{kind}_{fixture}"
    cubin, meta = d / "kernel.cubin", d / "meta.json"
    newest = max(p.stat().st_mtime for p in (ref / "cuda").glob("*.cuh"))
    if not force and cubin.exists() and meta.exists() and cubin.stat().st_mtime >= newest:
        return d
    if (d / "unsupported").exists() and not force:
        return None
    src = d / "src"
    src.mkdir(parents=True, exist_ok=True)
    ctx = dict(a_cols=cfg["a_cols"], b_rows=cfg["b_rows"], a_cpp_type=cfg["a"][0], a_loader=cfg["a"][1],
               b_cpp_type=cfg["b"][0], b_loader=cfg["b"][1],
               use_b16_gemm=cfg["a"][0] != "i8" or cfg["b"][0] != "i8", writer=cfg["writer"])
    for name in ("common.cuh", "kernel.cu", "meta.cu"):
        text = render((ref / "templates" / "basic_gemm" / name).read_text(), ctx)
        text = text.replace('"../../../cuda/', f'"{ref / "cuda"}/')
        (src / name).write_text(text)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    res = subprocess.run([nvcc, *NVCC_FLAGS, "--cubin", "-o", str(cubin), str(src / "kernel.cu")], capture_output=True, text=True)
    if res.returncode != 0:
        (d / "unsupported").write_text(res.stderr[-2000:])
        return None
    res = subprocess.run([nvcc, *NVCC_FLAGS, "-o", str(d / "meta"), str(src / "meta.cu")], capture_output=True, text=True)
    if res.returncode != 0:
        raise SystemExit(res.stderr)
    info = json.loads(subprocess.run([str(d / "meta")], capture_output=True, text=True, check=True).stdout)
    info.update(a_cols=cfg["a_cols"], b_rows=cfg["b_rows"], has_rrms_output=cfg["writer"]["has_rrms_output"],
                has_residual_input=cfg["writer"]["has_residual_input"])
    meta.write_text(json.dumps(info, indent="\t") + "\n")
    return d


def build_all(ref: Path, force: bool = False) -> list:
    done = [build_one(ref, h, dd, force) for h, dd in CONFIGS]
    for fixture, shape in GEMM_SHAPES.items():
        for kind, cfg in gemm_kernels(shape).items():
            done.append(build_gemm(ref, fixture, kind, cfg, force))
    return done


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: build_ref.py <checkout of the reference project> [--force]")
    for out in build_all(Path(sys.argv[1]), "--force" in sys.argv):
        print(out)
