"""ctypes bindings of libx17ai_b200.so (declarations follow include/x17ai_b200.h).

The library is the product; there is no fallback.  Importing this module without the built
library raises, and so does every kernel call on a machine without an sm_100 GPU.
"""
import ctypes
from ctypes import (POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int8, c_size_t,
                    c_uint32, c_uint64, c_uint8, c_void_p)
from pathlib import Path

import os

# X17AI_B200_LIB overrides the in-tree library (an alternative build of the same sources)
LIB_PATH = Path(os.environ.get("X17AI_B200_LIB") or (Path(__file__).resolve().parent / "libx17ai_b200.so"))


class X17Error(RuntimeError):
    """A diagnostic returned through the C ABI (the Rust host's ErrPack, src/lib.rs)."""


class FfiSpan(Structure):
    _fields_ = [("ptr", c_void_p), ("len", c_size_t)]


class FfiBuffer(Structure):
    _fields_ = [("instance", c_void_p), ("vmt", c_void_p)]


class CudaContextHandle(Structure):
    _fields_ = [("refcnt_munus_one", c_size_t), ("device_id", c_size_t), ("capability_major", c_size_t),
                ("capability_minor", c_size_t), ("warp_size", c_size_t), ("device", c_int), ("context", c_void_p)]


class CudaKernelAttrs(Structure):
    _fields_ = [(n, c_int32) for n in (
        "max_threads_per_block", "static_shared_size_bytes", "const_size_bytes", "local_size_bytes", "num_regs",
        "ptx_version", "binary_version", "max_dynamic_shared_size_bytes", "preferred_shared_memory_carveout")]


class PtrResult(Structure):
    _fields_ = [("value", c_void_p), ("diagnostic", c_void_p)]


class AttnConfig(Structure):
    _fields_ = [("n_heads", c_size_t), ("head_dim", c_size_t), ("q_stride", c_size_t), ("kv_stride", c_size_t),
                ("o_stride", c_size_t)]


class AttnMeta(Structure):
    _fields_ = [("threads_per_block", c_size_t), ("smem_bytes", c_size_t), ("q_per_block", c_size_t)]


class GemmConfig(Structure):
    _fields_ = [("a_dtype", c_int32), ("b_dtype", c_int32), ("c_dtype", c_int32), ("epilogue", c_int32),
                ("a_cols", c_size_t), ("b_rows", c_size_t), ("inp_scale", c_double), ("out_scale", c_double),
                ("eps", c_double), ("head_dim", c_size_t)]


class GemmObjectDesc(Structure):
    _fields_ = [("epilogue_kind", c_int32), ("n_raw", c_uint32), ("k", c_uint32), ("head_dim", c_uint32),
                ("rrms_cols", c_uint32), ("c_stride", c_uint64), ("resid_stride", c_uint64),
                ("k0", c_uint32), ("k1", c_uint32), ("k2", c_uint32), ("k3", c_uint32), ("k4", c_uint32),   # f32 bit patterns
                ("smem_bytes", c_uint32), ("threads", c_uint32), ("m_per_block", c_uint32), ("n_per_block", c_uint32),
                ("k_a", c_uint32), ("reserved", c_uint32),
                ("map_a", c_uint8 * 128), ("map_b", c_uint8 * 128)]


class AttnObjectDesc(Structure):
    _fields_ = [("smem_bytes", c_uint32), ("threads", c_uint32), ("q_per_block", c_uint32), ("reserved", c_uint32),
                ("map_q", c_uint8 * 128), ("map_kv", c_uint8 * 128)]


class QkvgConfig(Structure):
    _fields_ = [("model_dim", c_size_t), ("n_heads", c_size_t), ("head_dim", c_size_t), ("gate_cols", c_size_t),
                ("inp_scale", c_double), ("out_scale", c_double), ("eps", c_double)]


class GemmMeta(Structure):
    _fields_ = [("threads_per_block", c_size_t), ("smem_bytes", c_size_t), ("m_per_block", c_size_t),
                ("n_per_block", c_size_t)]


DIAG = c_void_p

# name -> (restype, argtypes); every symbol include/x17ai_b200.h declares
SIGNATURES = {
    "x17ai_move_diagnostic": (None, [DIAG, FfiBuffer]),
    "x17ai_cuda_open_context": (PtrResult, [c_size_t]),
    "x17ai_cuda_close_context": (DIAG, [c_void_p]),
    "x17ai_cuda_context_ptr": (c_void_p, [c_void_p]),
    "x17ai_cuda_open_stream": (PtrResult, [c_void_p]),
    "x17ai_cuda_close_stream": (DIAG, [c_void_p]),
    "x17ai_cuda_synchronize": (DIAG, [c_void_p]),
    "x17ai_cuda_create_timer": (PtrResult, [c_void_p, c_void_p]),
    "x17ai_cuda_destroy_timer": (DIAG, [c_void_p]),
    "x17ai_cuda_timer_start": (DIAG, [c_void_p]),
    "x17ai_cuda_timer_stop": (DIAG, [c_void_p]),
    "x17ai_cuda_timer_elapsed_seconds": (DIAG, [c_void_p, POINTER(c_double)]),
    "x17ai_cuda_alloc": (PtrResult, [c_void_p, c_size_t]),
    "x17ai_cuda_free": (DIAG, [c_void_p, c_void_p]),
    "x17ai_cuda_upload_data": (DIAG, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "x17ai_cuda_download_data": (DIAG, [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "x17ai_cuda_load_module": (PtrResult, [c_void_p, c_char_p]),
    "x17ai_cuda_del_module": (DIAG, [c_void_p]),
    "x17ai_cuda_get_kernel": (PtrResult, [c_void_p, c_char_p, c_size_t]),
    "x17ai_cuda_read_kernel_attrs": (DIAG, [c_void_p, POINTER(CudaKernelAttrs)]),
    "x17ai_cuda_launch_kernel": (DIAG, [c_void_p, c_void_p] + [c_size_t] * 7 + [POINTER(c_void_p)]),
    "x17ai_b200_attn_meta": (DIAG, [POINTER(AttnConfig), POINTER(AttnMeta)]),
    "x17ai_b200_attn_fwd_i8": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_size_t] + [c_void_p] * 7 + [c_size_t]),
    "x17ai_b200_attn_fwd_i8_to_peers": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_size_t] + [c_void_p] * 7
                                        + [c_size_t, c_void_p, c_size_t]),
    "x17ai_b200_attn_fwd_pv_fp8": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_size_t] + [c_void_p] * 8 + [c_size_t]),
    "x17ai_b200_attn_fwd_i8_scaled": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_size_t, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "x17ai_b200_attn_fwd_i8_debug": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_size_t] + [c_void_p] * 7
                                     + [c_size_t] + [c_void_p] * 3),
    "x17ai_b200_attn_decode_i8": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_void_p, c_void_p, c_size_t,
                                         c_size_t] + [c_void_p] * 6 + [c_size_t, c_size_t]),
    "x17ai_b200_attn_decode_i8_noalloc": (DIAG, [c_void_p, POINTER(AttnConfig), c_size_t, c_void_p, c_void_p, c_size_t,
                                                 c_size_t] + [c_void_p] * 6 + [c_size_t, c_size_t]),
    "x17ai_b200_gemm_meta": (DIAG, [POINTER(GemmConfig), POINTER(GemmMeta)]),
    "x17ai_b200_gemm_fwd": (DIAG, [c_void_p, POINTER(GemmConfig), c_void_p, c_size_t, c_void_p, c_size_t,
                                   c_void_p, c_void_p, c_void_p]),
    "x17ai_b200_qkvg_fwd_i8": (DIAG, [c_void_p, POINTER(QkvgConfig), c_void_p, c_size_t] + [c_void_p] * 5),
    "x17ai_b200_split_i8_weights": (DIAG, [c_void_p, c_void_p, c_size_t, c_size_t, c_void_p]),
    "x17ai_b200_rms_norm": (DIAG, [c_void_p, c_int32, c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_double]),
    "x17ai_b200_read_status": (DIAG, [c_void_p, POINTER(c_uint32)]),
    "x17ai_b200_object_status": (DIAG, [c_void_p, c_void_p, POINTER(c_uint32)]),
    "x17ai_b200_take_diagnostic": (c_size_t, [DIAG, c_char_p, c_size_t]),
    "x17ai_b200_graph_begin": (DIAG, [c_void_p]),
    "x17ai_b200_graph_end": (DIAG, [c_void_p, POINTER(c_void_p)]),
    "x17ai_b200_graph_launch": (DIAG, [c_void_p, c_void_p]),
    "x17ai_b200_graph_destroy": (DIAG, [c_void_p, c_void_p]),
    "x17ai_b200_graph_kernel_nodes": (c_uint64, [c_void_p]),
    "x17ai_b200_attn_object_desc": (DIAG, [c_void_p, POINTER(AttnConfig), POINTER(AttnObjectDesc)]),
    "x17ai_b200_gemm_object_desc": (DIAG, [c_void_p, POINTER(GemmConfig), POINTER(GemmObjectDesc)]),
    "x17ai_b200_launch_count": (c_uint64, []),
    "x17ai_b200_set_attn_schedule": (c_int, [c_int, c_uint32]),
    "x17ai_b200_set_gemm_tiling": (c_int, [c_int]),
}

_lib = None


def load():
    """Loads the shared library once and sets the prototypes. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise X17Error(
            f"{LIB_PATH} is missing: build it with `python -m x17ai_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback for this path")
    lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def take_diag(diag) -> str:
    lib = load()
    buf = ctypes.create_string_buffer(4096)
    n = lib.x17ai_b200_take_diagnostic(diag, buf, 4096)
    return buf.raw[:n].decode("utf-8", "replace")


def check(diag) -> None:
    """NULL = success; anything else is moved into an exception (and released)."""
    if diag:
        raise X17Error(take_diag(diag))


def unwrap(res: PtrResult):
    if res.diagnostic:
        raise X17Error(take_diag(res.diagnostic))
    return res.value
