// Diagnostics shared by the driver shim and the kernel entry points.
//
// Contract (cpp/ffi.hpp:84-175 of the reference): a function returns NULL on success or a
// DiagnosticBuffer* that the caller owns until it passes it, once, to x17ai_move_diagnostic,
// which appends the text to the caller's FfiBuffer and releases the diagnostic.  Diagnostics
// built from string literals only (allocation failed, or nothing to format) are static and
// are never freed.
#pragma once

#include <cuda.h>

#include "drv.hpp"

#include <cstddef>
#include <new>
#include <sstream>
#include <string>

#include "../../include/x17ai_b200.h"

struct x17ai_DiagnosticBuffer {
	bool heap;
	char const *static_text;
	std::string text;
};

namespace x17 {

inline x17ai_DiagnosticBuffer *static_diag(char const *literal) noexcept {
	// one static object per call site would need a macro; a small pool keyed by the literal's
	// address keeps this a function. Literals live for the life of the library.
	struct Slot {
		x17ai_DiagnosticBuffer d;
	};
	static Slot pool[64];
	static int used = 0;
	for (int i = 0; i < used; ++i) {
		if (pool[i].d.static_text == literal) return &pool[i].d;
	}
	if (used < 64) {
		pool[used].d.heap = false;
		pool[used].d.static_text = literal;
		return &pool[used++].d;
	}
	static x17ai_DiagnosticBuffer overflow{false, "x17ai: error (diagnostic pool exhausted)", {}};
	return &overflow;
}

inline void diag_append(std::ostringstream &) {}
template <typename T, typename... Ts>
void diag_append(std::ostringstream &os, T const &v, Ts const &...rest) {
	os << v;
	diag_append(os, rest...);
}

inline std::string cu_error_text(CUresult e) {
	char const *s = nullptr;
	if (x17::driver().ok && DRV(cuGetErrorString)(e, &s) == CUDA_SUCCESS && s != nullptr) return s;
	return "unknown CUDA error " + std::to_string(int(e));
}

// Formatted diagnostic; falls back to the static literal if anything throws.
template <typename... Ts>
x17ai_DiagnosticBuffer *make_diag(char const *fallback, Ts const &...parts) noexcept {
	try {
		std::ostringstream os;
		diag_append(os, parts...);
		auto *d = new x17ai_DiagnosticBuffer{true, fallback, os.str()};
		return d;
	} catch (...) {
		return static_diag(fallback);
	}
}

template <typename T, typename R>
R ptr_ok(T *v) noexcept {
	R r;
	r.value = v;
	r.diagnostic = nullptr;
	return r;
}
template <typename R>
R ptr_err(x17ai_DiagnosticBuffer *d) noexcept {
	R r;
	r.value = nullptr;
	r.diagnostic = d;
	return r;
}

// RAII push/pop of a context so that no context is left current on the calling thread.
struct ScopedContext {
	CUresult push_err;
	explicit ScopedContext(CUcontext ctx) noexcept : push_err(DRV(cuCtxPushCurrent)(ctx)) {}
	~ScopedContext() {
		if (push_err == CUDA_SUCCESS) {
			CUcontext popped = nullptr;
			DRV(cuCtxPopCurrent)(&popped);
		}
	}
	ScopedContext(ScopedContext const &) = delete;
	ScopedContext &operator=(ScopedContext const &) = delete;
};

}  // namespace x17
