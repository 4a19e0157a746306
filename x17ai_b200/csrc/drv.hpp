// CUDA driver API resolved at run time (dlopen of libcuda.so.1), so that the library loads,
// and its symbol table can be checked, on machines without an NVIDIA driver; every entry point
// then returns a diagnostic instead of computing.
#pragma once

#include <cuda.h>
#include <dlfcn.h>

#include <mutex>

#define X17_DRV_FUNCTIONS(X)      \
	X(cuInit)                     \
	X(cuGetErrorString)           \
	X(cuDeviceGetCount)           \
	X(cuDeviceGet)                \
	X(cuDeviceGetAttribute)       \
	X(cuDevicePrimaryCtxRetain)   \
	X(cuDevicePrimaryCtxRelease)  \
	X(cuCtxPushCurrent)           \
	X(cuCtxPopCurrent)            \
	X(cuCtxGetDevice)             \
	X(cuStreamCreate)             \
	X(cuStreamDestroy)            \
	X(cuStreamSynchronize)        \
	X(cuStreamGetCtx)             \
	X(cuEventCreate)              \
	X(cuEventDestroy)             \
	X(cuEventRecord)              \
	X(cuEventElapsedTime)         \
	X(cuMemAllocAsync)            \
	X(cuMemFreeAsync)             \
	X(cuMemcpyHtoDAsync)          \
	X(cuMemcpyDtoHAsync)          \
	X(cuModuleLoad)               \
	X(cuModuleUnload)             \
	X(cuModuleGetFunction)        \
	X(cuModuleGetGlobal)          \
	X(cuFuncSetAttribute)         \
	X(cuFuncGetAttribute)         \
	X(cuLaunchKernel)             \
	X(cuTensorMapEncodeTiled)

#define X17_STR2(x) #x
#define X17_STR(x) X17_STR2(x)

namespace x17 {

struct Driver {
	bool ok = false;
	char const *missing = "libcuda.so.1";
#define X17_DECL(name) decltype(&name) name##_p = nullptr;
	X17_DRV_FUNCTIONS(X17_DECL)
#undef X17_DECL
};

inline Driver const &driver() {
	static Driver d;
	static std::once_flag once;
	std::call_once(once, [] {
		void *h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
		if (h == nullptr) return;
		bool all = true;
#define X17_LOAD(name)                                                        \
	d.name##_p = reinterpret_cast<decltype(&name)>(dlsym(h, X17_STR(name)));  \
	if (d.name##_p == nullptr) {                                              \
		all = false;                                                          \
		d.missing = X17_STR(name);                                            \
	}
		X17_DRV_FUNCTIONS(X17_LOAD)
#undef X17_LOAD
		d.ok = all;
	});
	return d;
}

}  // namespace x17

// call a driver function: DRV(cuInit)(0)
#define DRV(name) (x17::driver().name##_p)
