"""Kernel objects in the reference's on-disk form: `cache/kernels/<name>/{kernel.cubin, meta.json}`.

The reference's host renders a template per shape, compiles it with nvcc into a cubin that exports
`extern "C" kernel(...)`, runs a small program that prints launch metadata as JSON, loads the cubin
through the shim and launches it with an array of pointers to the arguments
(src/device/cuda/kernel_build.rs:38-134, cuda_shim.rs:464-489).  This module does the same for the
RMSNorm kernel, the int8 x int8 GEMMs, the e4m3 x int8 GEMM (ffn_y_fwd_f8) and the int8 attention; the
tensor-core objects carry templates of their TMA tensor maps and finish them on the device with the pointers
they are launched with. Every tensor-core object exports four status words (`x17_status`), read with
CubinKernel.status().
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


def build_gemm(stream, config, name: str, force: bool = False) -> Path:
    """One GEMM configuration of the reference's block (a kernels.GemmConfig: int8 x int8, or e4m3 x int8 whose
    object owns the two e4m3 planes of its weights and a `prepare` entry point that fills them) as
    cache/kernels/<name>/kernel.cubin + meta.json, the form GemmKernel::new produces in the reference
    (gemm.rs:368-443): the epilogue
    constants and templates of the two TMA tensor maps come from x17ai_b200_gemm_object_desc (the maps
    need the CUDA driver, so this runs where a GPU is), the kernel patches the maps with the pointers
    and row count it is launched with. Launch it as the reference does: grid
    (c_rows / M_PER_BLOCK, raw_cols / N_PER_BLOCK, 1), arguments (a, a_rows, b, b_rows, c[, rrms][, residual])."""
    d = CACHE / name
    cubin, meta = d / "kernel.cubin", d / "meta.json"
    src = SRC / "gemm.cu"
    newest = max(f.stat().st_mtime for f in (src, SRC.parent / "gemm.cuh", SRC.parent / "ptx.cuh"))
    desc = _lib.GemmObjectDesc()
    cfg = config._c()
    check(_lib.load().x17ai_b200_gemm_object_desc(stream.handle, ctypes.byref(cfg), ctypes.byref(desc)))
    fields = ("epilogue_kind", "n_raw", "k", "k_a", "head_dim", "rrms_cols", "c_stride", "resid_stride", "k0", "k1", "k2", "k3", "k4")
    key = json.dumps([int(getattr(desc, f)) for f in fields] + list(desc.map_a) + list(desc.map_b))
    stamp = d / "config.json"
    if (not force and cubin.exists() and meta.exists() and stamp.exists() and stamp.read_text() == key
            and cubin.stat().st_mtime >= newest):
        return d
    d.mkdir(parents=True, exist_ok=True)
    maps = d / "maps.h"
    maps.write_text("#define X17_MAP_A " + ",".join(str(v) for v in desc.map_a) + "\n"
                    "#define X17_MAP_B " + ",".join(str(v) for v in desc.map_b) + "\n")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    defs = {"X17_EPI": desc.epilogue_kind, "X17_N_RAW": desc.n_raw, "X17_K": desc.k, "X17_HEAD_DIM": desc.head_dim,
            "X17_RRMS_COLS": desc.rrms_cols, "X17_C_STRIDE": desc.c_stride, "X17_RESID_STRIDE": desc.resid_stride,
            "X17_K0": desc.k0, "X17_K1": desc.k1, "X17_K2": desc.k2, "X17_K3": desc.k3, "X17_K4": desc.k4}
    if desc.k_a:
        defs.update({"X17_SPLIT": 1, "X17_K_A": desc.k_a})
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "--ftz=true", "--fmad=true",
           "-include", str(maps)] + [f"-D{k}={int(v)}u" for k, v in defs.items()] + ["--cubin", "-o", str(cubin), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise X17Error(f"nvcc failed for {src}:\n{res.stderr}")
    meta.write_text(json.dumps({"THREADS_PER_BLOCK": int(desc.threads), "SMEM_BYTES": int(desc.smem_bytes),
                                "M_PER_BLOCK": int(desc.m_per_block), "N_PER_BLOCK": int(desc.n_per_block)}, indent="\t") + "\n")
    stamp.write_text(key)
    return d


def build_attn(stream, config, name: str, force: bool = False) -> Path:
    """The int8 attention kernel for one configuration (a kernels.AttnKernelConfig) as
    cache/kernels/<name>/kernel.cubin + meta.json, the form AttnKernel::new produces in the reference
    (attn.rs:300-351). Launch it as the reference does: grid
    (seq_len / Q_PER_BLOCK, n_heads / max(128 / head_dim, 1), 1), arguments
    (seq_len, q, kv, sink_k, sink_v, attn_temperature, out, l, window_size), attn.rs:412-447."""
    d = CACHE / name
    cubin, meta = d / "kernel.cubin", d / "meta.json"
    src = SRC / "attn.cu"
    newest = max(f.stat().st_mtime for f in (src, SRC.parent / "attn.cuh", SRC.parent / "ptx.cuh"))
    desc = _lib.AttnObjectDesc()
    cfg = config._c()
    check(_lib.load().x17ai_b200_attn_object_desc(stream.handle, ctypes.byref(cfg), ctypes.byref(desc)))
    key = json.dumps([config.n_heads, config.head_dim, config.q_stride, config.kv_stride, config.o_stride]
                     + list(desc.map_q) + list(desc.map_kv))
    stamp = d / "config.json"
    if (not force and cubin.exists() and meta.exists() and stamp.exists() and stamp.read_text() == key
            and cubin.stat().st_mtime >= newest):
        return d
    d.mkdir(parents=True, exist_ok=True)
    maps = d / "maps.h"
    maps.write_text("#define X17_MAP_Q " + ",".join(str(v) for v in desc.map_q) + "\n"
                    "#define X17_MAP_KV " + ",".join(str(v) for v in desc.map_kv) + "\n")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    defs = {"X17_HEAD_DIM": config.head_dim, "X17_N_HEADS": config.n_heads, "X17_Q_STRIDE": config.q_stride, "X17_KV_STRIDE": config.kv_stride,
            "X17_O_STRIDE": config.o_stride}
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "--ftz=true", "--fmad=true",
           "-include", str(maps)] + [f"-D{k}={int(v)}u" for k, v in defs.items()] + ["--cubin", "-o", str(cubin), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise X17Error(f"nvcc failed for {src}:\n{res.stderr}")
    meta.write_text(json.dumps({"THREADS_PER_BLOCK": int(desc.threads), "SMEM_BYTES": int(desc.smem_bytes),
                                "Q_PER_BLOCK": int(desc.q_per_block)}, indent="\t") + "\n")
    stamp.write_text(key)
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

    def launch(self, stream, grid, block, smem, *args, kernel=None):
        """`args` are ctypes values; the shim receives an array of pointers to them, as the Rust host passes."""
        arr = (ctypes.c_void_p * len(args))(*[ctypes.cast(ctypes.pointer(a), ctypes.c_void_p) for a in args])
        check(self._lib.x17ai_cuda_launch_kernel(stream.handle, kernel or self.kernel, grid[0], grid[1], grid[2],
                                                 block[0], block[1], block[2], smem, arr))

    def entry(self, name: str, smem: int = 0):
        """Another entry point of the same module (x17ai_cuda_get_kernel)."""
        return unwrap(self._lib.x17ai_cuda_get_kernel(self.module, name.encode(), smem))

    def status(self, stream):
        """The object's four status words (all zero = no bounded wait ran out, no refusal); reading clears them."""
        st = (ctypes.c_uint32 * 4)()
        check(self._lib.x17ai_b200_object_status(stream.handle, self.module, st))
        return [int(v) for v in st]

    def unload(self):
        check(self._lib.x17ai_cuda_del_module(self.module))


class GemmObject:
    """A GEMM kernel object with GemmKernel's launch interface: built once for its configuration, launched
    through the generic shim calls with the reference's grid and argument list (gemm.rs:591-641)."""

    def __init__(self, stream, config, name: str):
        from . import kernels as K
        self.config = config
        self.kernel = CubinKernel(stream, build_gemm(stream, config, name))
        # e4m3 activations x int8 weights: the object keeps two e4m3 planes of the weights, filled by `prepare`
        self.split = config.a_dtype == K.DTYPE_E4M3 and config.b_dtype == K.DTYPE_INT8
        self._prepare = self.kernel.entry("prepare") if self.split else None
        self._prepared_for = None

    def prepare(self, stream, b):
        """The set-up launch of an e4m3 x int8 object: once per weight tensor (the reference's host would add this
        one launch where it loads the weights)."""
        from . import kernels as K
        K.matrix_shape("gemm", "b", b, (self.config.b_rows, self.config.a_cols), K.DTYPE_INT8)
        self.kernel.launch(stream, (296, 1, 1), (256, 1, 1), 0, ctypes.c_void_p(b.data_ptr()), ctypes.c_uint64(b.shape[0]),
                           kernel=self._prepare)
        self._prepared_for = b.data_ptr()

    def launch(self, stream, a, b, c, rrms=None, residual=None):
        from . import kernels as K
        m = self.kernel.meta
        # the same checks as GemmKernel.launch (tensor_check.rs:19-101, gemm.rs:591-641): a wrongly sized
        # output would be written out of bounds
        if self.split:
            K.matrix_shape("gemm", "a", a, (None, self.config.a_cols), K.DTYPE_E4M3)
            K.matrix_shape("gemm", "c", c, (a.shape[0], self.config.b_rows // 2), self.config.c_dtype)
            K.matrix_shape("gemm", "residual", residual, (a.shape[0], self.config.b_rows // 2), K.DTYPE_INT8)
            if self._prepared_for != b.data_ptr():
                self.prepare(stream, b)
        else:
            K.GemmKernel(self.config).check_shapes(a, b, c, rrms, residual)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        args = [ptr(a), ctypes.c_uint64(a.shape[0]), ptr(b), ctypes.c_uint64(b.shape[0]), ptr(c)]
        if rrms is not None:
            args.append(ptr(rrms))
        if residual is not None:
            args.append(ptr(residual))
        grid = (max(1, a.shape[0] // m["M_PER_BLOCK"]), max(1, b.shape[0] // m["N_PER_BLOCK"]), 1)
        self.kernel.launch(stream, grid, (m["THREADS_PER_BLOCK"], 1, 1), m["SMEM_BYTES"], *args)


class AttnObject:
    """The attention kernel object with AttnKernel's launch interface for one sequence (attn.rs:412-447)."""

    def __init__(self, stream, config, name: str):
        self.config = config
        self.kernel = CubinKernel(stream, build_attn(stream, config, name))

    def launch(self, stream, q, kv, sink_k, sink_v, attn_temperature, out, l=None, window_size=0):
        from . import kernels as K
        c, m = self.config, self.kernel.meta
        if q.dim() != 2 or q.shape[0] % m["Q_PER_BLOCK"] != 0:
            raise X17Error(f"attention kernel object takes one sequence [seq, q_stride] with seq a multiple of {m['Q_PER_BLOCK']}, "
                           f"got {list(q.shape)}")
        heads_per_cta = max(128 // c.head_dim, 1)
        if c.n_heads % heads_per_cta != 0:   # attn.rs:108-113: the grid has one CTA per group of 128 / head_dim heads
            raise X17Error(f"attention kernel config requires n_heads to be a multiple of {heads_per_cta} at head_dim "
                           f"{c.head_dim}, got {c.n_heads}")
        if window_size % 16 != 0:
            raise X17Error(f"attention window_size must be zero or divisible by 16, got {window_size}")
        batch, seq = K.AttnKernel(c)._shapes(q, kv, sink_k, sink_v, attn_temperature, out, l)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
        self.kernel.launch(stream, (seq // m["Q_PER_BLOCK"], c.n_heads // heads_per_cta, 1), (m["THREADS_PER_BLOCK"], 1, 1),
                           m["SMEM_BYTES"], ctypes.c_uint64(seq), ptr(q), ptr(kv), ptr(sink_k), ptr(sink_v),
                           ptr(attn_temperature), ptr(out), ptr(l), ctypes.c_uint64(window_size))
