// The 21 C-ABI functions of the reference's CUDA driver shim (cpp/cuda_shim.cpp:189-988),
// re-implemented over the CUDA driver API with the same names, argument lists, struct layouts,
// ownership and context discipline: handles are the raw driver objects (CUstream, CUmodule,
// CUfunction, CUdeviceptr), the primary context is retained per open_context and never left
// current on the calling thread, and all device work is stream-ordered.

#include <cuda.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <limits>
#include <mutex>

#include "diag.hpp"

using x17::cu_error_text;
using x17::make_diag;
using x17::ptr_err;
using x17::ptr_ok;
using x17::ScopedContext;
using x17::static_diag;

struct x17ai_CudaTimerHandle {
	CUcontext context;
	CUstream stream;
	CUevent start;
	CUevent end;
};

namespace {

std::once_flag g_init_once;
CUresult g_init_result = CUDA_ERROR_NOT_INITIALIZED;

CUresult ensure_init() {
	if (!x17::driver().ok) return CUDA_ERROR_SHARED_OBJECT_INIT_FAILED;  // no libcuda.so.1 on this machine
	std::call_once(g_init_once, [] { g_init_result = DRV(cuInit)(0); });
	return g_init_result;
}

inline CUstream as_stream(x17ai_CudaStreamHandle *s) { return reinterpret_cast<CUstream>(s); }
inline CUdeviceptr as_devptr(x17ai_CudaDeviceData *p) {
	return static_cast<CUdeviceptr>(reinterpret_cast<uintptr_t>(p));
}

bool fits_u32(size_t v) { return v <= std::numeric_limits<uint32_t>::max(); }

#define X17_CU_CHECK(R, CALL, WHERE)                                                        \
	do {                                                                                    \
		CUresult e_ = (CALL);                                                               \
		if (e_ != CUDA_SUCCESS) {                                                           \
			return R(make_diag(WHERE " failed.", WHERE " failed with cuda error: ",          \
							   cu_error_text(e_)));                                         \
		}                                                                                   \
	} while (0)

inline x17ai_DiagnosticBuffer *same(x17ai_DiagnosticBuffer *d) { return d; }

}  // namespace

extern "C" {

void x17ai_move_diagnostic(x17ai_DiagnosticBuffer *diag, x17ai_FfiBuffer err) {
	if (diag == nullptr) return;
	char const *text = diag->heap ? diag->text.c_str() : diag->static_text;
	size_t const len = std::strlen(text);
	if (err.vmt != nullptr && err.vmt->extend != nullptr) {
		x17ai_FfiSpan dst = err.vmt->extend(err.instance, len);
		if (dst.ptr != nullptr && dst.len == len) std::memcpy(dst.ptr, text, len);
	}
	if (diag->heap) delete diag;
}

x17ai_ContextResult x17ai_cuda_open_context(size_t device_id) {
	using R = x17ai_ContextResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	X17_CU_CHECK(fail, ensure_init(), "x17ai_cuda_open_context(): cuInit()");
	int count = 0;
	X17_CU_CHECK(fail, DRV(cuDeviceGetCount)(&count), "x17ai_cuda_open_context(): cuDeviceGetCount()");
	if (device_id >= size_t(count)) {
		return fail(static_diag("x17ai_cuda_open_context(): CUDA device ID out of range"));
	}
	CUdevice dev;
	X17_CU_CHECK(fail, DRV(cuDeviceGet)(&dev, int(device_id)), "x17ai_cuda_open_context(): cuDeviceGet()");
	int major = 0, minor = 0, warp = 0;
	X17_CU_CHECK(fail, DRV(cuDeviceGetAttribute)(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, dev),
				 "x17ai_cuda_open_context(): cuDeviceGetAttribute(MAJOR)");
	X17_CU_CHECK(fail, DRV(cuDeviceGetAttribute)(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, dev),
				 "x17ai_cuda_open_context(): cuDeviceGetAttribute(MINOR)");
	X17_CU_CHECK(fail, DRV(cuDeviceGetAttribute)(&warp, CU_DEVICE_ATTRIBUTE_WARP_SIZE, dev),
				 "x17ai_cuda_open_context(): cuDeviceGetAttribute(WARP_SIZE)");
	if (major < 0 || minor < 0) {
		return fail(static_diag("x17ai_cuda_open_context(): compute capability out of range"));
	}
	if (warp <= 0 || (warp & (warp - 1)) != 0) {
		return fail(static_diag("x17ai_cuda_open_context(): warp size is not a power of two"));
	}
	CUcontext ctx = nullptr;
	X17_CU_CHECK(fail, DRV(cuDevicePrimaryCtxRetain)(&ctx, dev),
				 "x17ai_cuda_open_context(): cuDevicePrimaryCtxRetain()");
	if (ctx == nullptr) {
		return fail(static_diag("x17ai_cuda_open_context(): cuDevicePrimaryCtxRetain() returned nullptr"));
	}
	auto *h = new (std::nothrow) x17ai_CudaContextHandle{};
	if (h == nullptr) {
		DRV(cuDevicePrimaryCtxRelease)(dev);
		return fail(static_diag("x17ai_cuda_open_context(): out of host memory"));
	}
	h->refcnt_munus_one = 0;
	h->device_id = device_id;
	h->capability_major = size_t(major);
	h->capability_minor = size_t(minor);
	h->warp_size = size_t(warp);
	h->device = dev;
	h->context = ctx;
	return ptr_ok<x17ai_CudaContextHandle, R>(h);
}

x17ai_DiagnosticBuffer *x17ai_cuda_close_context(x17ai_CudaContextHandle *context) {
	if (context == nullptr) return static_diag("x17ai_cuda_close_context(): null context");
	CUdevice dev = context->device;
	delete context;
	X17_CU_CHECK(same, DRV(cuDevicePrimaryCtxRelease)(dev),
				 "x17ai_cuda_close_context(): cuDevicePrimaryCtxRelease()");
	return nullptr;
}

void *x17ai_cuda_context_ptr(x17ai_CudaContextHandle *context) {
	return context != nullptr ? context->context : nullptr;
}

x17ai_StreamResult x17ai_cuda_open_stream(x17ai_CudaContextHandle *ctx) {
	using R = x17ai_StreamResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	if (ctx == nullptr) return fail(static_diag("x17ai_cuda_open_stream(): null context"));
	CUstream stream = nullptr;
	{
		ScopedContext scope(static_cast<CUcontext>(ctx->context));
		X17_CU_CHECK(fail, scope.push_err, "x17ai_cuda_open_stream(): cuCtxPushCurrent()");
		X17_CU_CHECK(fail, DRV(cuStreamCreate)(&stream, CU_STREAM_NON_BLOCKING),
					 "x17ai_cuda_open_stream(): cuStreamCreate()");
	}
	if (stream == nullptr) {
		return fail(static_diag("x17ai_cuda_open_stream(): cuStreamCreate() returned nullptr"));
	}
	return ptr_ok<x17ai_CudaStreamHandle, R>(reinterpret_cast<x17ai_CudaStreamHandle *>(stream));
}

x17ai_DiagnosticBuffer *x17ai_cuda_close_stream(x17ai_CudaStreamHandle *stream) {
	if (stream == nullptr) return static_diag("x17ai_cuda_close_stream(): null stream");
	X17_CU_CHECK(same, DRV(cuStreamDestroy)(as_stream(stream)), "x17ai_cuda_close_stream(): cuStreamDestroy()");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_synchronize(x17ai_CudaStreamHandle *stream) {
	if (stream == nullptr) return static_diag("x17ai_cuda_synchronize(): null stream");
	X17_CU_CHECK(same, DRV(cuStreamSynchronize)(as_stream(stream)),
				 "x17ai_cuda_synchronize(): cuStreamSynchronize()");
	return nullptr;
}

x17ai_TimerResult x17ai_cuda_create_timer(x17ai_CudaContextHandle *context, x17ai_CudaStreamHandle *stream) {
	using R = x17ai_TimerResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	if (context == nullptr || stream == nullptr) {
		return fail(static_diag("x17ai_cuda_create_timer(): null context or stream"));
	}
	auto *t = new (std::nothrow) x17ai_CudaTimerHandle{};
	if (t == nullptr) return fail(static_diag("x17ai_cuda_create_timer(): out of host memory"));
	t->context = static_cast<CUcontext>(context->context);
	t->stream = as_stream(stream);
	CUresult e;
	{
		ScopedContext scope(t->context);
		e = scope.push_err;
		if (e == CUDA_SUCCESS) e = DRV(cuEventCreate)(&t->start, CU_EVENT_DEFAULT);
		if (e == CUDA_SUCCESS) {
			e = DRV(cuEventCreate)(&t->end, CU_EVENT_DEFAULT);
			if (e != CUDA_SUCCESS) DRV(cuEventDestroy)(t->start);
		}
	}
	if (e != CUDA_SUCCESS) {
		delete t;
		return fail(make_diag("x17ai_cuda_create_timer(): cuEventCreate() failed.",
							  "x17ai_cuda_create_timer(): cuEventCreate() failed with cuda error: ",
							  cu_error_text(e)));
	}
	return ptr_ok<x17ai_CudaTimerHandle, R>(t);
}

x17ai_DiagnosticBuffer *x17ai_cuda_destroy_timer(x17ai_CudaTimerHandle *timer) {
	if (timer == nullptr) return static_diag("x17ai_cuda_destroy_timer(): null timer");
	CUresult e1, e2;
	{
		ScopedContext scope(timer->context);
		e1 = DRV(cuEventDestroy)(timer->end);
		e2 = DRV(cuEventDestroy)(timer->start);
	}
	delete timer;
	X17_CU_CHECK(same, e1, "x17ai_cuda_destroy_timer(): cuEventDestroy(end)");
	X17_CU_CHECK(same, e2, "x17ai_cuda_destroy_timer(): cuEventDestroy(start)");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_timer_start(x17ai_CudaTimerHandle *timer) {
	if (timer == nullptr) return static_diag("x17ai_cuda_timer_start(): null timer");
	X17_CU_CHECK(same, DRV(cuEventRecord)(timer->start, timer->stream), "x17ai_cuda_timer_start(): cuEventRecord()");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_timer_stop(x17ai_CudaTimerHandle *timer) {
	if (timer == nullptr) return static_diag("x17ai_cuda_timer_stop(): null timer");
	X17_CU_CHECK(same, DRV(cuEventRecord)(timer->end, timer->stream), "x17ai_cuda_timer_stop(): cuEventRecord()");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_timer_elapsed_seconds(x17ai_CudaTimerHandle *timer, double *seconds) {
	if (timer == nullptr || seconds == nullptr) {
		return static_diag("x17ai_cuda_timer_elapsed_seconds(): null argument");
	}
	float ms = 0.0f;
	CUresult e;
	{
		ScopedContext scope(timer->context);
		e = scope.push_err;
		if (e == CUDA_SUCCESS) e = DRV(cuEventElapsedTime)(&ms, timer->start, timer->end);
	}
	X17_CU_CHECK(same, e, "x17ai_cuda_timer_elapsed_seconds(): cuEventElapsedTime()");
	*seconds = double(ms) / 1000.0;
	return nullptr;
}

x17ai_DeviceDataResult x17ai_cuda_alloc(x17ai_CudaStreamHandle *stream, size_t bytes) {
	using R = x17ai_DeviceDataResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	if (stream == nullptr) return fail(static_diag("x17ai_cuda_alloc(): null stream"));
	CUdeviceptr mem = 0;
	X17_CU_CHECK(fail, DRV(cuMemAllocAsync)(&mem, bytes, as_stream(stream)), "x17ai_cuda_alloc(): cuMemAllocAsync()");
	if (mem == 0) return fail(static_diag("x17ai_cuda_alloc(): cuMemAllocAsync() returned null pointer"));
	return ptr_ok<x17ai_CudaDeviceData, R>(reinterpret_cast<x17ai_CudaDeviceData *>(uintptr_t(mem)));
}

x17ai_DiagnosticBuffer *x17ai_cuda_free(x17ai_CudaStreamHandle *stream, x17ai_CudaDeviceData *ptr) {
	if (stream == nullptr) return static_diag("x17ai_cuda_free(): null stream");
	X17_CU_CHECK(same, DRV(cuMemFreeAsync)(as_devptr(ptr), as_stream(stream)), "x17ai_cuda_free(): cuMemFreeAsync()");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_upload_data(x17ai_CudaStreamHandle *stream, uint8_t const *src,
											   x17ai_CudaDeviceData *dst, size_t offset_bytes,
											   size_t size_bytes) {
	if (stream == nullptr || (src == nullptr && size_bytes != 0)) {
		return static_diag("x17ai_cuda_upload_data(): null argument");
	}
	X17_CU_CHECK(same, DRV(cuMemcpyHtoDAsync)(as_devptr(dst) + offset_bytes, src, size_bytes, as_stream(stream)),
				 "x17ai_cuda_upload_data(): cuMemcpyHtoDAsync()");
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_download_data(x17ai_CudaStreamHandle *stream, x17ai_CudaDeviceData *src,
												 uint8_t *dst, size_t offset_bytes, size_t size_bytes) {
	if (stream == nullptr || (dst == nullptr && size_bytes != 0)) {
		return static_diag("x17ai_cuda_download_data(): null argument");
	}
	X17_CU_CHECK(same, DRV(cuMemcpyDtoHAsync)(dst, as_devptr(src) + offset_bytes, size_bytes, as_stream(stream)),
				 "x17ai_cuda_download_data(): cuMemcpyDtoHAsync()");
	return nullptr;
}

x17ai_ModuleResult x17ai_cuda_load_module(x17ai_CudaContextHandle *ctx, char const *cubin_path) {
	using R = x17ai_ModuleResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	if (ctx == nullptr || cubin_path == nullptr) {
		return fail(static_diag("x17ai_cuda_load_module(): null argument"));
	}
	CUmodule mod = nullptr;
	{
		ScopedContext scope(static_cast<CUcontext>(ctx->context));
		X17_CU_CHECK(fail, scope.push_err, "x17ai_cuda_load_module(): cuCtxPushCurrent()");
		CUresult e = DRV(cuModuleLoad)(&mod, cubin_path);
		if (e != CUDA_SUCCESS) {
			return fail(make_diag("x17ai_cuda_load_module(): cuModuleLoad() failed.",
								  "x17ai_cuda_load_module(): cuModuleLoad(", cubin_path,
								  ") failed with cuda error: ", cu_error_text(e)));
		}
	}
	if (mod == nullptr) return fail(static_diag("x17ai_cuda_load_module(): cuModuleLoad() returned nullptr"));
	return ptr_ok<x17ai_CudaModuleHandle, R>(reinterpret_cast<x17ai_CudaModuleHandle *>(mod));
}

x17ai_DiagnosticBuffer *x17ai_cuda_del_module(x17ai_CudaModuleHandle *module) {
	if (module == nullptr) return static_diag("x17ai_cuda_del_module(): null module");
	X17_CU_CHECK(same, DRV(cuModuleUnload)(reinterpret_cast<CUmodule>(module)), "x17ai_cuda_del_module(): cuModuleUnload()");
	return nullptr;
}

x17ai_KernelResult x17ai_cuda_get_kernel(x17ai_CudaModuleHandle *module, char const *name, size_t smem_size) {
	using R = x17ai_KernelResult;
	auto fail = [](x17ai_DiagnosticBuffer *d) { return ptr_err<R>(d); };
	if (module == nullptr || name == nullptr) return fail(static_diag("x17ai_cuda_get_kernel(): null argument"));
	CUfunction fn = nullptr;
	X17_CU_CHECK(fail, DRV(cuModuleGetFunction)(&fn, reinterpret_cast<CUmodule>(module), name),
				 "x17ai_cuda_get_kernel(): cuModuleGetFunction()");
	if (fn == nullptr) return fail(static_diag("x17ai_cuda_get_kernel(): cuModuleGetFunction() returned nullptr"));
	if (smem_size > size_t(std::numeric_limits<int>::max())) {
		return fail(static_diag("x17ai_cuda_get_kernel(): max dynamic shared memory size is out of range"));
	}
	X17_CU_CHECK(fail, DRV(cuFuncSetAttribute)(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, int(smem_size)),
				 "x17ai_cuda_get_kernel(): cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
	X17_CU_CHECK(fail, DRV(cuFuncSetAttribute)(fn, CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, 100),
				 "x17ai_cuda_get_kernel(): cuFuncSetAttribute(PREFERRED_SHARED_MEMORY_CARVEOUT)");
	return ptr_ok<x17ai_CudaKernelHandle, R>(reinterpret_cast<x17ai_CudaKernelHandle *>(fn));
}

x17ai_DiagnosticBuffer *x17ai_cuda_read_kernel_attrs(x17ai_CudaKernelHandle *kernel, x17ai_CudaKernelAttrs *attrs) {
	if (kernel == nullptr || attrs == nullptr) return static_diag("x17ai_cuda_read_kernel_attrs(): null argument");
	CUfunction fn = reinterpret_cast<CUfunction>(kernel);
	struct Item {
		CUfunction_attribute attr;
		int32_t x17ai_CudaKernelAttrs::*field;
		char const *name;
	};
	static Item const items[] = {
		{CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, &x17ai_CudaKernelAttrs::max_threads_per_block, "MAX_THREADS_PER_BLOCK"},
		{CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, &x17ai_CudaKernelAttrs::static_shared_size_bytes, "SHARED_SIZE_BYTES"},
		{CU_FUNC_ATTRIBUTE_CONST_SIZE_BYTES, &x17ai_CudaKernelAttrs::const_size_bytes, "CONST_SIZE_BYTES"},
		{CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, &x17ai_CudaKernelAttrs::local_size_bytes, "LOCAL_SIZE_BYTES"},
		{CU_FUNC_ATTRIBUTE_NUM_REGS, &x17ai_CudaKernelAttrs::num_regs, "NUM_REGS"},
		{CU_FUNC_ATTRIBUTE_PTX_VERSION, &x17ai_CudaKernelAttrs::ptx_version, "PTX_VERSION"},
		{CU_FUNC_ATTRIBUTE_BINARY_VERSION, &x17ai_CudaKernelAttrs::binary_version, "BINARY_VERSION"},
		{CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, &x17ai_CudaKernelAttrs::max_dynamic_shared_size_bytes, "MAX_DYNAMIC_SHARED_SIZE_BYTES"},
		{CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, &x17ai_CudaKernelAttrs::preferred_shared_memory_carveout, "PREFERRED_SHARED_MEMORY_CARVEOUT"},
	};
	x17ai_CudaKernelAttrs result{};
	for (Item const &it : items) {
		int v = 0;
		CUresult e = DRV(cuFuncGetAttribute)(&v, it.attr, fn);
		if (e != CUDA_SUCCESS) {
			return make_diag("x17ai_cuda_read_kernel_attrs(): cuFuncGetAttribute() failed.",
							 "x17ai_cuda_read_kernel_attrs(): cuFuncGetAttribute(", it.name,
							 ") failed with cuda error: ", cu_error_text(e));
		}
		result.*(it.field) = v;
	}
	*attrs = result;
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_cuda_launch_kernel(x17ai_CudaStreamHandle *stream, x17ai_CudaKernelHandle *kernel,
												 size_t grid_x, size_t grid_y, size_t grid_z,
												 size_t block_x, size_t block_y, size_t block_z,
												 size_t shared_mem_bytes, void **args) {
	if (stream == nullptr || kernel == nullptr) return static_diag("x17ai_cuda_launch_kernel(): null argument");
	if (grid_x < 1 || grid_y < 1 || grid_z < 1 || !fits_u32(grid_x) || !fits_u32(grid_y) || !fits_u32(grid_z)) {
		return static_diag("x17ai_cuda_launch_kernel(): grid dimensions are out of range");
	}
	if (block_x < 1 || block_y < 1 || block_z < 1 || !fits_u32(block_x) || !fits_u32(block_y) || !fits_u32(block_z)) {
		return static_diag("x17ai_cuda_launch_kernel(): block dimensions are out of range");
	}
	if (!fits_u32(shared_mem_bytes)) {
		return static_diag("x17ai_cuda_launch_kernel(): shared memory size is out of range");
	}
	X17_CU_CHECK(same,
				 DRV(cuLaunchKernel)(reinterpret_cast<CUfunction>(kernel), unsigned(grid_x), unsigned(grid_y),
								unsigned(grid_z), unsigned(block_x), unsigned(block_y), unsigned(block_z),
								unsigned(shared_mem_bytes), as_stream(stream), args, nullptr),
				 "x17ai_cuda_launch_kernel(): cuLaunchKernel()");
	return nullptr;
}

}  // extern "C"
