"""The 21 functions of the reference's driver shim (cpp/cuda_shim.cpp:189-988) exercised the way the
Rust host uses them (src/main.rs:37-385): context and stream, stream-ordered alloc/free, upload and
download, a kernel object loaded from cache/kernels/<name>/kernel.cubin + meta.json, its attributes,
a launch with an array of argument pointers, and the event timer."""
import ctypes

import numpy as np
import pytest

from oracle import formats, rms_norm as o_rms

pytestmark = pytest.mark.gpu


def test_kernel_object_through_the_generic_shim(stream):
    from x17ai_b200 import device, kernel_objects
    rows, dim = 100, 4096
    rng = np.random.default_rng(5)
    x = np.ascontiguousarray(formats.f32_to_e4m3(rng.standard_normal((rows, dim)).astype(np.float32)))
    out = np.zeros((rows, dim), dtype=np.int8)
    assert stream.capability[0] == 10

    d_in, d_out = stream.alloc(x.nbytes), stream.alloc(out.nbytes)
    stream.upload(x.ctypes.data, d_in, 0, x.nbytes)
    kern = kernel_objects.CubinKernel(stream, kernel_objects.build_rms_norm(dim))
    assert kern.attrs.binary_version == 100 and kern.attrs.num_regs > 0 and kern.attrs.local_size_bytes == 0
    timer = device.CudaTimer(stream)
    timer.start()
    grid = ((rows + kernel_objects.ROWS_PER_BLOCK - 1) // kernel_objects.ROWS_PER_BLOCK, 1, 1)
    kern.launch(stream, grid, (kern.meta["THREADS_PER_BLOCK"], 1, 1), kern.meta["SMEM_BYTES"],
                ctypes.c_void_p(d_in), ctypes.c_uint64(rows), ctypes.c_void_p(d_out))
    timer.stop()
    stream.download(d_out, out.ctypes.data, 0, out.nbytes)
    stream.synchronize()
    assert 0.0 < timer.elapsed_seconds() < 1.0
    timer.destroy()
    stream.free(d_in)
    stream.free(d_out)
    kern.unload()
    d = np.abs(out.astype(np.int32) - o_rms.rms_norm_e4m3_i8(x).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() <= 2e-3


def test_shim_error_paths(stream, lib):
    from x17ai_b200 import X17Error, _lib
    with pytest.raises(X17Error, match="cuModuleLoad"):
        _lib.unwrap(lib.x17ai_cuda_load_module(stream.ctx, b"/nonexistent/kernel.cubin"))
    with pytest.raises(X17Error, match="device ID out of range"):
        _lib.unwrap(lib.x17ai_cuda_open_context(4096))
    from x17ai_b200 import kernel_objects
    kern = kernel_objects.CubinKernel(stream, kernel_objects.build_rms_norm(512))
    with pytest.raises(X17Error, match="grid dimensions are out of range"):
        kern.launch(stream, (0, 1, 1), (256, 1, 1), 0, ctypes.c_void_p(0), ctypes.c_uint64(0), ctypes.c_void_p(0))
    with pytest.raises(X17Error, match="cuModuleGetFunction"):
        _lib.unwrap(lib.x17ai_cuda_get_kernel(kern.module, b"no_such_kernel", 0))
    kern.unload()
