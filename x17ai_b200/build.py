"""Builds libx17ai_b200.so in-tree with nvcc for sm_100a (no JIT cache: the built library
travels with the source tree)."""
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libx17ai_b200.so"
SOURCES = [CSRC / "api.cu", CSRC / "shim.cpp"]
HEADERS = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hpp")) + [HERE.parent / "include" / "x17ai_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "--ftz=true", "--fmad=true",
    "-Xcompiler", "-fPIC", "-shared",
    "-Xptxas", "-v",
]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    if os.environ.get("X17AI_B200_LIB"):
        return Path(os.environ["X17AI_B200_LIB"])
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIB), *map(str, SOURCES), "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = res.stdout + res.stderr
    (HERE / "build.log").write_text(" ".join(cmd) + "\n" + log)
    if res.returncode != 0:
        sys.stderr.write(log)
        raise RuntimeError("nvcc failed building libx17ai_b200.so")
    if verbose:
        print(log)
    return LIB


def build_kernel_objects():
    """The cubin + meta.json kernel objects used by the tests (prebuilt so they travel with the tree)."""
    from . import kernel_objects
    for dim in (512, 4096):
        kernel_objects.build_rms_norm(dim)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
