"""Host-side mirror of the reference's CUDA device objects over the C ABI.

CudaDevice / CudaStream  <- src/device/cuda.rs:25-77, src/device/cuda/cuda_shim.rs:207-330
CudaTimer                <- src/device/cuda.rs:79-101
Every method is one call into libx17ai_b200.so; errors surface as X17Error.
"""
import ctypes

from . import _lib
from ._lib import check, unwrap


class CudaStream:
    """One primary-context handle plus one non-blocking stream (CudaStream::new, cuda_shim.rs:207-232)."""

    def __init__(self, device_id: int = 0):
        lib = _lib.load()
        self._lib = lib
        self.ctx = unwrap(lib.x17ai_cuda_open_context(device_id))
        try:
            self.handle = unwrap(lib.x17ai_cuda_open_stream(self.ctx))
        except Exception:
            check(lib.x17ai_cuda_close_context(self.ctx))
            raise
        self.device_id = device_id
        self._open = True

    @property
    def capability(self):
        h = ctypes.cast(self.ctx, ctypes.POINTER(_lib.CudaContextHandle)).contents
        return int(h.capability_major), int(h.capability_minor)

    def synchronize(self) -> None:
        check(self._lib.x17ai_cuda_synchronize(self.handle))

    def alloc(self, nbytes: int) -> int:
        return unwrap(self._lib.x17ai_cuda_alloc(self.handle, nbytes))

    def free(self, ptr: int) -> None:
        check(self._lib.x17ai_cuda_free(self.handle, ptr))

    def upload(self, src_host_ptr: int, dst: int, offset: int, nbytes: int) -> None:
        check(self._lib.x17ai_cuda_upload_data(self.handle, src_host_ptr, dst, offset, nbytes))

    def download(self, src: int, dst_host_ptr: int, offset: int, nbytes: int) -> None:
        check(self._lib.x17ai_cuda_download_data(self.handle, src, dst_host_ptr, offset, nbytes))

    def read_status(self):
        """Synchronises and returns the four device status words (all zero = no kernel gave up a wait)."""
        st = (ctypes.c_uint32 * 4)()
        check(self._lib.x17ai_b200_read_status(self.handle, st))
        return [int(v) for v in st]

    def close(self) -> None:
        if self._open:
            self._open = False
            check(self._lib.x17ai_cuda_close_stream(self.handle))
            check(self._lib.x17ai_cuda_close_context(self.ctx))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class TorchStream:
    """Wraps a stream owned by PyTorch (its raw cudaStream_t) so kernels run in torch's stream order."""

    def __init__(self, torch_stream=None):
        import torch
        self._lib = _lib.load()
        s = torch_stream if torch_stream is not None else torch.cuda.current_stream()
        self.handle = s.cuda_stream
        if self.handle == 0:
            raise _lib.X17Error("the legacy default stream has no context of its own: pass a created stream")
        self._torch_stream = s

    def synchronize(self) -> None:
        check(self._lib.x17ai_cuda_synchronize(self.handle))

    def read_status(self):
        st = (ctypes.c_uint32 * 4)()
        check(self._lib.x17ai_b200_read_status(self.handle, st))
        return [int(v) for v in st]


class CudaTimer:
    """CUDA-event timer on a stream (CudaTimer, src/device/cuda.rs:79-101)."""

    def __init__(self, stream: CudaStream):
        self._lib = _lib.load()
        self.handle = unwrap(self._lib.x17ai_cuda_create_timer(stream.ctx, stream.handle))

    def start(self) -> None:
        check(self._lib.x17ai_cuda_timer_start(self.handle))

    def stop(self) -> None:
        check(self._lib.x17ai_cuda_timer_stop(self.handle))

    def elapsed_seconds(self) -> float:
        out = ctypes.c_double(0.0)
        check(self._lib.x17ai_cuda_timer_elapsed_seconds(self.handle, ctypes.byref(out)))
        return out.value

    def destroy(self) -> None:
        if self.handle:
            check(self._lib.x17ai_cuda_destroy_timer(self.handle))
            self.handle = None


class CudaGraph:
    """A recorded sequence of this library's launches on one stream, replayed with one driver call
    (x17ai_b200_graph_begin / _end / _launch). Use as a context manager around the launches to record:

        with CudaGraph(stream) as g:
            kernel.launch(stream, ...)
        g.launch()
    """

    def __init__(self, stream: CudaStream):
        self._lib = _lib.load()
        self.stream = stream
        self.handle = None

    def __enter__(self):
        check(self._lib.x17ai_b200_graph_begin(self.stream.handle))
        return self

    def __exit__(self, exc_type, exc, tb):
        out = ctypes.c_void_p()
        diag = self._lib.x17ai_b200_graph_end(self.stream.handle, ctypes.byref(out))
        if exc_type is None:
            check(diag)
            self.handle = out.value
        elif diag:   # the body failed: drop the end-of-capture diagnostic, the body's error is the one to report
            _lib.take_diag(diag)
        elif out.value:
            check(self._lib.x17ai_b200_graph_destroy(out.value, self.stream.handle))
        return False

    @property
    def kernel_nodes(self) -> int:
        return int(self._lib.x17ai_b200_graph_kernel_nodes(self.handle))

    def launch(self) -> None:
        if self.handle is None:
            raise _lib.X17Error("CudaGraph.launch(): nothing was recorded")
        check(self._lib.x17ai_b200_graph_launch(self.handle, self.stream.handle))

    def destroy(self) -> None:
        if self.handle is not None:
            h, self.handle = self.handle, None
            check(self._lib.x17ai_b200_graph_destroy(h, self.stream.handle))
