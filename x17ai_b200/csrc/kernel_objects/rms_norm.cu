// Kernel object in the reference's form: a cubin that exports `extern "C" kernel(...)`, loaded with
// x17ai_cuda_load_module / x17ai_cuda_get_kernel and launched with x17ai_cuda_launch_kernel, the shape
// fixed at compile time (-DMODEL_DIM=..., -DL2_NORM_EPS=...) as the reference's templates do.
// Signature of the reference's harness kernel (rms_norm.cu:82-86): (inp e4m3, n_inputs, out FixedI8);
// `usize` is 32 bits on the device there (cuda/utils_core.cuh:46-47) while the host passes 64-bit
// values; 64 bits are declared here and the low half is used.
#include "../rms_norm.cuh"

#ifndef MODEL_DIM
#error "compile with -DMODEL_DIM=<columns>"
#endif
#ifndef L2_NORM_EPS
#define L2_NORM_EPS 8.470329472543003e-22
#endif

extern "C" __global__ void __launch_bounds__(x17::rms_cfg::THREADS)
kernel(unsigned char const *inp, unsigned long long n_inputs, signed char *out) {
	x17::RmsParams p;
	p.inp = inp;
	p.out = out;
	p.row_scale = nullptr;
	p.rows = static_cast<x17::u32>(n_inputs);
	p.cols = MODEL_DIM;
	p.inp_stride = MODEL_DIM;
	p.out_stride = MODEL_DIM;
	p.eps = float(L2_NORM_EPS);
	p.inv_cols = float(1.0 / double(MODEL_DIM));
	if constexpr (MODEL_DIM <= x17::rms_cfg::KEEP_CHUNKS * 32 * 16) {
		x17::rms_norm_body_keep(p);
	} else {
		x17::rms_norm_body<x17::RMS_E4M3_FIXED>(p);
	}
}
