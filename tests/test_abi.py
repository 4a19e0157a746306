"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the header
declares, validates configurations before touching a device, and reports errors through the
diagnostic protocol of the reference's shim (cpp/ffi.hpp:84-175)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "x17ai_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(x17ai_(?:cuda|b200|move)_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from x17ai_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 32
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/x17ai_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes prototypes and the header disagree"


def test_reference_shim_names_present():
    names = set(_declared_symbols())
    shim = """x17ai_move_diagnostic x17ai_cuda_open_context x17ai_cuda_close_context x17ai_cuda_context_ptr
    x17ai_cuda_open_stream x17ai_cuda_close_stream x17ai_cuda_synchronize x17ai_cuda_create_timer
    x17ai_cuda_destroy_timer x17ai_cuda_timer_start x17ai_cuda_timer_stop x17ai_cuda_timer_elapsed_seconds
    x17ai_cuda_alloc x17ai_cuda_free x17ai_cuda_upload_data x17ai_cuda_download_data x17ai_cuda_load_module
    x17ai_cuda_del_module x17ai_cuda_get_kernel x17ai_cuda_read_kernel_attrs x17ai_cuda_launch_kernel""".split()
    assert len(shim) == 21 and set(shim) <= names


def test_struct_layouts_match_reference():
    from x17ai_b200 import _lib
    assert ctypes.sizeof(_lib.PtrResult) == 16
    assert ctypes.sizeof(_lib.CudaKernelAttrs) == 9 * 4
    assert _lib.CudaContextHandle.refcnt_munus_one.offset == 0
    assert ctypes.sizeof(_lib.CudaContextHandle) == 56
    assert ctypes.sizeof(_lib.FfiBuffer) == 16


def test_meta_matches_launch_contract(lib):
    from x17ai_b200 import kernels as K
    a = K.AttnKernel(K.AttnKernelConfig(32, 128, 4096, 8192, 4096))
    assert a.THREADS_PER_BLOCK == 320 and a.Q_PER_BLOCK == 128
    assert a.Q_PER_BLOCK & (a.Q_PER_BLOCK - 1) == 0          # attn.rs:336-339
    g = K.GemmKernel(K.ffn_f_fwd_config(4096, 14336))
    assert (g.M_PER_BLOCK, g.N_PER_BLOCK) == (128, 256)      # powers of two, gemm.rs:563-566


def test_config_validation_messages(lib):
    from x17ai_b200 import X17Error, kernels as K
    with pytest.raises(X17Error, match="requires n_heads > 0"):
        K.AttnKernel(K.AttnKernelConfig(0, 64, 64, 128, 64))
    with pytest.raises(X17Error, match="q_stride >= n_heads \\* head_dim, got 64 vs 256"):
        K.AttnKernel(K.AttnKernelConfig(4, 64, 64, 512, 256))
    with pytest.raises(X17Error, match="kv_stride >= 2 \\* n_heads \\* head_dim"):
        K.AttnKernel(K.AttnKernelConfig(4, 64, 256, 256, 256))
    with pytest.raises(X17Error, match="head_dim 32, 64 or 128, got 48"):
        K.AttnKernel(K.AttnKernelConfig(4, 48, 256, 512, 256))
    with pytest.raises(X17Error, match="rms-norm epilogue requires head_dim"):
        K.GemmKernel(K.GemmConfig(K.DTYPE_INT8, K.DTYPE_INT8, K.DTYPE_INT8, K.EPI_RMS_NORM, 256, 512, head_dim=48))
    with pytest.raises(X17Error, match="geglu epilogue writes e4m3"):
        K.GemmKernel(K.GemmConfig(K.DTYPE_INT8, K.DTYPE_INT8, K.DTYPE_INT8, K.EPI_GEGLU, 256, 512))


def test_host_shape_checks_without_gpu():
    """tensor_check.rs messages; the checks run before any device call."""
    import torch
    from x17ai_b200 import X17Error, kernels as K
    with pytest.raises(X17Error, match="attention input q must be 2D"):
        K.matrix_shape("attention", "q", torch.zeros(4, dtype=torch.int8), (None, 4), K.DTYPE_INT8)
    with pytest.raises(X17Error, match="has zero size"):
        K.matrix_shape("gemm", "a", torch.zeros((0, 4), dtype=torch.int8), (None, 4), K.DTYPE_INT8)
    with pytest.raises(X17Error, match="has 3 columns, but should have 4"):
        K.matrix_shape("gemm", "a", torch.zeros((2, 3), dtype=torch.int8), (None, 4), K.DTYPE_INT8)
    with pytest.raises(X17Error, match="is not on device"):
        K.matrix_shape("gemm", "a", torch.zeros((2, 4), dtype=torch.int8), (None, 4), K.DTYPE_INT8)
    with pytest.raises(X17Error, match=r"must have shape \[4\] or \[4, 1\]"):
        K.vector_shape("attention", "attn_temperature", torch.zeros((2, 2)), 4, K.DTYPE_F32)


def test_no_gpu_means_error_not_fallback(lib):
    """Without a CUDA driver every device entry point returns a diagnostic; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from x17ai_b200 import X17Error, device
    with pytest.raises(X17Error, match="cuInit"):
        device.CudaStream(0)


def test_diagnostic_ownership_protocol(lib):
    """A diagnostic is moved out exactly once through x17ai_move_diagnostic (here via the fixed-buffer helper)."""
    from x17ai_b200 import _lib
    cfg = _lib.AttnConfig(0, 64, 64, 128, 64)
    meta = _lib.AttnMeta()
    d = lib.x17ai_b200_attn_meta(ctypes.byref(cfg), ctypes.byref(meta))
    assert d
    buf = ctypes.create_string_buffer(16)
    n = lib.x17ai_b200_take_diagnostic(d, buf, 16)   # too small: all-or-nothing extend writes nothing
    assert n == 0
    d = lib.x17ai_b200_attn_meta(ctypes.byref(cfg), ctypes.byref(meta))
    assert "n_heads > 0" in _lib.take_diag(d)
    assert lib.x17ai_b200_take_diagnostic(None, buf, 16) == 0
