"""Kernel objects in the reference's on-disk form: `cache/kernels/<name>/{kernel.cubin, meta.json}`.

The reference's host renders a template per shape, compiles it with nvcc into a cubin that exports
`extern "C" kernel(...)`, runs a small program that prints launch metadata as JSON, loads the cubin
through the shim and launches it with an array of pointers to the arguments
(src/device/cuda/kernel_build.rs:38-134, cuda_shim.rs:464-489).  This module does the same for the
kernel of this path that needs no host-encoded TMA descriptor (RMSNorm); the tensor-core kernels take
their tensor maps from the host and are reached through their own entry points instead.
"""
import ctypes
import json
import os
import subprocess
from pathlib import Path

from . import _lib
from ._lib import X17Error, check, unwrap

HERE = Path(__file__).resolve().parent
CACHE = HERE / "cache" / "kernels"
SRC = HERE / "csrc" / "kernel_objects"
ROWS_PER_BLOCK = 8
THREADS_PER_BLOCK = 256


def build_rms_norm(model_dim: int, eps: float = 2.0 ** -70, force: bool = False) -> Path:
    """nvcc -> cache/kernels/rms_norm_<dim>/kernel.cubin + meta.json (kernel_build.rs:38-134)."""
    d = CACHE / f"rms_norm_{model_dim}"
    cubin, meta = d / "kernel.cubin", d / "meta.json"
    src = SRC / "rms_norm.cu"
    # the kernel object is rebuilt when its source or any header it includes is newer
    newest = max(f.stat().st_mtime for f in (src, SRC.parent / "rms_norm.cuh", SRC.parent / "ptx.cuh"))
    if not force and cubin.exists() and meta.exists() and cubin.stat().st_mtime >= newest:
        return d
    if model_dim % 16 != 0 or model_dim > 8192:
        raise X17Error(f"rms_norm kernel object requires MODEL_DIM to be a multiple of 16 and at most 8192, got {model_dim}")
    d.mkdir(parents=True, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "--ftz=true", "--fmad=true",
           f"-DMODEL_DIM={model_dim}", f"-DL2_NORM_EPS={eps!r}", "--cubin", "-o", str(cubin), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise X17Error(f"nvcc failed for {src}:\n{res.stderr}")
    meta.write_text(json.dumps({"THREADS_PER_BLOCK": THREADS_PER_BLOCK, "SMEM_BYTES": 0, "ROWS_PER_BLOCK": ROWS_PER_BLOCK},
                               indent="\t") + "\n")
    return d


class CubinKernel:
    """load_cubin_kernel + CudaKernel::launch (kernel_build.rs:160-198, cuda_shim.rs:464-489)."""

    def __init__(self, stream, directory: Path, name: str = "kernel"):
        self._lib = _lib.load()
        self.meta = json.loads((directory / "meta.json").read_text())
        self.module = unwrap(self._lib.x17ai_cuda_load_module(stream.ctx, str(directory / "kernel.cubin").encode()))
        self.kernel = unwrap(self._lib.x17ai_cuda_get_kernel(self.module, name.encode(), int(self.meta["SMEM_BYTES"])))
        attrs = _lib.CudaKernelAttrs()
        check(self._lib.x17ai_cuda_read_kernel_attrs(self.kernel, ctypes.byref(attrs)))
        self.attrs = attrs

    def launch(self, stream, grid, block, smem, *args):
        """`args` are ctypes values; the shim receives an array of pointers to them, as the Rust host passes."""
        arr = (ctypes.c_void_p * len(args))(*[ctypes.cast(ctypes.pointer(a), ctypes.c_void_p) for a in args])
        check(self._lib.x17ai_cuda_launch_kernel(stream.handle, self.kernel, grid[0], grid[1], grid[2],
                                                 block[0], block[1], block[2], smem, arr))

    def unload(self):
        check(self._lib.x17ai_cuda_del_module(self.module))
