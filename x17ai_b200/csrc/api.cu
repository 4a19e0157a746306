// Kernel entry points of libx17ai_b200.so (part 2 of include/x17ai_b200.h): argument checks in
// the manner of the Rust launchers (src/device/cuda/tensor_check.rs, attn.rs:353-447,
// gemm.rs:591-641), TMA tensor maps, launch configuration, launches.

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <unordered_map>
#include <vector>

#include "attn.cuh"
#include "attn_stream.cuh"
#include "decode.cuh"
#include "diag.hpp"
#include "gemm.cuh"
#include "rms_norm.cuh"

using x17::make_diag;
using x17::static_diag;

namespace {

std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_attn_schedule{X17AI_B200_ATTN_PER_TILE};
std::atomic<int> g_gemm_tiling{X17AI_B200_GEMM_CTA_PAIR};
std::atomic<unsigned> g_attn_item_tiles{0};   // 0 = chosen per launch
std::mutex g_capture_mutex;
std::unordered_map<void *, CUcontext> g_capture_ctx;   // streams between graph_begin and graph_end

// ---- per-device state -----------------------------------------------------------------------

constexpr int MAX_DEVICES = 32;
struct DeviceState {
	std::once_flag once;
	uint32_t *status = nullptr;  // 4 words of device memory
	int sm_count = 0;
	cudaError_t init_err = cudaSuccess;
};
DeviceState g_dev[MAX_DEVICES];

// Makes the stream's context current for the scope (the callers of this library keep no
// context current, cpp/ffi.hpp:195-206) and resolves the device ordinal.
struct StreamScope {
	CUcontext ctx = nullptr;
	int device = -1;
	bool pushed = false;
	x17ai_DiagnosticBuffer *diag = nullptr;

	explicit StreamScope(x17ai_CudaStreamHandle *stream, char const *who) {
		if (stream == nullptr) {
			diag = make_diag("x17ai_b200: null stream", who, ": null stream");
			return;
		}
		if (!x17::driver().ok) {
			diag = make_diag("x17ai_b200: CUDA driver not available", who,
							 ": the CUDA driver is not available on this machine (", x17::driver().missing,
							 " not found); this library has no CPU path");
			return;
		}
		CUresult e = DRV(cuStreamGetCtx)(reinterpret_cast<CUstream>(stream), &ctx);
		if (e == CUDA_SUCCESS) e = DRV(cuCtxPushCurrent)(ctx);
		if (e != CUDA_SUCCESS) {
			diag = make_diag("x17ai_b200: cannot enter the stream's context", who,
							 ": cannot enter the stream's context: ", x17::cu_error_text(e));
			return;
		}
		pushed = true;
		CUdevice dev;
		e = DRV(cuCtxGetDevice)(&dev);
		if (e != CUDA_SUCCESS || int(dev) < 0 || int(dev) >= MAX_DEVICES) {
			diag = make_diag("x17ai_b200: cannot resolve the device", who, ": cannot resolve the device");
			return;
		}
		device = int(dev);
		DeviceState &st = g_dev[device];
		std::call_once(st.once, [&] {
			int major = 0, minor = 0;
			cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
			cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
			if (major != 10) {
				st.init_err = cudaErrorNoKernelImageForDevice;
				return;
			}
			cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device);
			st.init_err = cudaMalloc(&st.status, 4 * sizeof(uint32_t));
			if (st.init_err == cudaSuccess) st.init_err = cudaMemset(st.status, 0, 4 * sizeof(uint32_t));
		});
		if (st.init_err != cudaSuccess) {
			diag = make_diag("x17ai_b200: device initialisation failed", who,
							 ": device initialisation failed (this library needs an sm_100 GPU): ",
							 cudaGetErrorString(st.init_err));
		}
	}
	~StreamScope() {
		if (pushed) {
			CUcontext popped = nullptr;
			DRV(cuCtxPopCurrent)(&popped);
		}
	}
	DeviceState &state() const { return g_dev[device]; }
};

x17ai_DiagnosticBuffer *launch_result(char const *who) {
	cudaError_t e = cudaGetLastError();
	if (e != cudaSuccess) {
		return make_diag("x17ai_b200: kernel launch failed", who, ": kernel launch failed: ",
						 cudaGetErrorString(e));
	}
	g_launches.fetch_add(1, std::memory_order_relaxed);
	return nullptr;
}

// ---- TMA tensor maps ---------------------------------------------------------------------------

CUtensorMapSwizzle swizzle_for(uint32_t inner_bytes) {
	return inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
		   : inner_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
							   : CU_TENSOR_MAP_SWIZZLE_32B;
}

// Byte tensor [d2][d1][d0] (d0 innermost) with row pitch s1 and plane pitch s2, box b0 x b1 x 1.
CUresult make_map_3d(CUtensorMap *map, void const *base, uint64_t d0, uint64_t d1, uint64_t d2,
					 uint64_t s1, uint64_t s2, uint32_t b0, uint32_t b1) {
	cuuint64_t dims[3] = {d0, d1, d2};
	cuuint64_t strides[2] = {s1, s2};
	cuuint32_t box[3] = {b0, b1, 1};
	cuuint32_t estr[3] = {1, 1, 1};
	return DRV(cuTensorMapEncodeTiled)(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims,
								  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(b0),
								  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

CUresult make_map_2d(CUtensorMap *map, void const *base, uint64_t d0, uint64_t d1, uint64_t s1,
					 uint32_t b0, uint32_t b1) {
	cuuint64_t dims[2] = {d0, d1};
	cuuint64_t strides[1] = {s1};
	cuuint32_t box[2] = {b0, b1};
	cuuint32_t estr[2] = {1, 1};
	return DRV(cuTensorMapEncodeTiled)(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims,
								  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(b0),
								  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

bool aligned16(void const *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- attention ---------------------------------------------------------------------------------

x17ai_DiagnosticBuffer *check_attn_config(x17ai_AttnConfig const *cfg, char const *who) {
	if (cfg == nullptr) return make_diag("x17ai_b200: null config", who, ": null config");
	if (cfg->n_heads == 0) {
		return make_diag("x17ai_b200: bad attention config", who, ": attention kernel config requires n_heads > 0");
	}
	if (cfg->head_dim != 32 && cfg->head_dim != 64 && cfg->head_dim != 128) {
		return make_diag("x17ai_b200: bad attention config", who,
						 ": attention kernel config requires head_dim 32, 64 or 128, got ", cfg->head_dim);
	}
	size_t const q_cols = cfg->n_heads * cfg->head_dim;
	if (cfg->q_stride < q_cols) {
		return make_diag("x17ai_b200: bad attention config", who,
						 ": attention kernel config requires q_stride >= n_heads * head_dim, got ",
						 cfg->q_stride, " vs ", q_cols);
	}
	if (cfg->kv_stride < 2 * q_cols) {
		return make_diag("x17ai_b200: bad attention config", who,
						 ": attention kernel config requires kv_stride >= 2 * n_heads * head_dim, got ",
						 cfg->kv_stride, " vs ", 2 * q_cols);
	}
	if (cfg->o_stride < q_cols) {
		return make_diag("x17ai_b200: bad attention config", who,
						 ": attention kernel config requires o_stride >= n_heads * head_dim, got ",
						 cfg->o_stride, " vs ", q_cols);
	}
	if (cfg->q_stride % 16 != 0 || cfg->kv_stride % 16 != 0 || cfg->o_stride % 16 != 0) {
		return make_diag("x17ai_b200: bad attention config", who,
						 ": attention strides must be multiples of 16 bytes");
	}
	return nullptr;
}

uint32_t rounded_window(size_t window_size, size_t seq_len) {
	if (window_size == 0) return 0xFFFFFFFFu;
	size_t const w = ((window_size - 1) / 16 + 1) * 16;  // cuda/attn_fwd_i8.cuh:408-412
	return w >= seq_len ? 0xFFFFFFFFu : uint32_t(w);
}

template <bool DEBUG, bool FP8PV = false, bool SCALED = false>
x17ai_DiagnosticBuffer *attn_launch(
	char const *who, x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch,
	size_t seq_len, int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *temperature, void *out, float *l, size_t window_size, int32_t *dbg_s,
	uint8_t *dbg_p, int32_t *dbg_o, float const *v_scale = nullptr, float const *tok_q = nullptr,
	float const *tok_k = nullptr, float const *tok_v = nullptr, int8_t *const *peer_out = nullptr,
	size_t n_peer_out = 0) {
	if (auto *d = check_attn_config(cfg, who)) return d;
	if (n_peer_out > x17::AttnParams::MAX_PEER_OUT || (n_peer_out > 0 && peer_out == nullptr)) {
		return make_diag("x17ai_b200: bad peer outputs", who, ": at most ", size_t(x17::AttnParams::MAX_PEER_OUT),
						 " peer copies of the output");
	}
	for (size_t i = 0; i < n_peer_out; ++i) {
		if (peer_out[i] == nullptr || !aligned16(peer_out[i])) {
			return make_diag("x17ai_b200: bad peer outputs", who, ": peer outputs must be non-null and 16-byte aligned");
		}
	}
	if (batch == 0 || seq_len == 0) {
		return make_diag("x17ai_b200: empty attention input", who, ": attention input q has zero size");
	}
	if (seq_len >= (size_t(1) << 31) || batch > 65535 || cfg->n_heads > 65535) {
		return make_diag("x17ai_b200: attention shape out of range", who, ": attention shape out of range");
	}
	if (window_size > 0 && window_size % 16 != 0) {
		return make_diag("x17ai_b200: bad window", who,
						 ": attention window_size must be zero or divisible by 16, got ", window_size);
	}
	if (!q || !kv || !sink_k || !sink_v || !temperature || !out) {
		return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	}
	if (!aligned16(q) || !aligned16(kv) || !aligned16(out) || !aligned16(sink_k) || !aligned16(sink_v)) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;

	uint32_t const d = uint32_t(cfg->head_dim);
	CUtensorMap tm_q, tm_kv;
	CUresult e = make_map_3d(&tm_q, q, cfg->n_heads * d, seq_len, batch, cfg->q_stride,
							 cfg->q_stride * seq_len, d, x17::attn_cfg::BQ);
	if (e == CUDA_SUCCESS) {
		e = make_map_3d(&tm_kv, kv, 2 * cfg->n_heads * d, seq_len, batch, cfg->kv_stride,
						cfg->kv_stride * seq_len, d, x17::attn_cfg::BKV);
	}
	if (e != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cuTensorMapEncodeTiled failed", who,
						 ": cuTensorMapEncodeTiled failed: ", x17::cu_error_text(e));
	}
	x17::AttnParams p{};
	p.seq_len = uint32_t(seq_len);
	p.n_heads = uint32_t(cfg->n_heads);
	p.window = rounded_window(window_size, seq_len);
	p.q = q;
	p.q_stride = cfg->q_stride;
	p.q_batch_stride = cfg->q_stride * seq_len;
	p.sink_k = sink_k;
	p.sink_v = sink_v;
	p.temperature = temperature;
	p.out = out;
	p.o_stride = cfg->o_stride;
	p.o_batch_stride = cfg->o_stride * seq_len;
	p.l = l;
	p.l_batch_stride = cfg->n_heads * seq_len;
	p.v_scale = v_scale;
	p.tok_q_scale = tok_q;
	p.tok_k_scale = tok_k;
	p.tok_v_scale = tok_v;
	p.status = scope.state().status;
	p.dbg_s = dbg_s;
	p.dbg_p = dbg_p;
	p.dbg_o = dbg_o;
	p.n_peer_out = uint32_t(n_peer_out);
	for (size_t i = 0; i < n_peer_out; ++i) p.peer_out[i] = peer_out[i];

	cudaError_t ce;
	// (peer copies are written by the one-CTA-per-tile kernel's epilogue only)
	if (!SCALED && n_peer_out == 0 && g_attn_schedule.load(std::memory_order_relaxed) == X17AI_B200_ATTN_PERSISTENT) {
		// items = runs of consecutive query tiles of one (batch, head), dealt round-robin to one CTA per
		// SM. Long runs pay the unfused maximum sweep of their first tile less often; short runs
		// balance the SMs: halve the run while fewer than two items per SM come out.
		x17::AttnItemPlan plan{};
		plan.n_qtiles = uint32_t((seq_len + x17::attn_stream_cfg::BQ - 1) / x17::attn_stream_cfg::BQ);
		uint32_t const sms = uint32_t(scope.state().sm_count);
		uint64_t const bh = uint64_t(batch) * cfg->n_heads;
		uint32_t tiles = g_attn_item_tiles.load(std::memory_order_relaxed);
		if (tiles == 0) {
			tiles = 16;
			while (tiles > 4 && bh * ((plan.n_qtiles + tiles - 1) / tiles) < 2ull * sms) tiles /= 2;
		}
		plan.tiles_per_item = tiles < plan.n_qtiles ? tiles : plan.n_qtiles;
		plan.chunks = (plan.n_qtiles + plan.tiles_per_item - 1) / plan.tiles_per_item;
		uint64_t const items = bh * plan.chunks;
		if (items >= (uint64_t(1) << 31)) {
			return make_diag("x17ai_b200: attention shape out of range", who, ": attention shape out of range");
		}
		plan.n_items = uint32_t(items);
		dim3 grid(plan.n_items < sms ? plan.n_items : sms);
		dim3 block(x17::attn_stream_cfg::THREADS);
		auto go = [&](auto kernel, uint32_t smem) -> cudaError_t {
			cudaError_t e2 = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
			if (e2 != cudaSuccess) return e2;
			kernel<<<grid, block, smem, reinterpret_cast<cudaStream_t>(stream)>>>(tm_q, tm_kv, p, plan);
			return cudaSuccess;
		};
		if (d == 128) {
			ce = go(x17::attn_fwd_stream_kernel<128, DEBUG, FP8PV>, x17::attn_stream_cfg::smem_bytes<128>());
		} else if (d == 64) {
			ce = go(x17::attn_fwd_stream_kernel<64, DEBUG, FP8PV>, x17::attn_stream_cfg::smem_bytes<64>());
		} else {
			ce = go(x17::attn_fwd_stream_kernel<32, DEBUG, FP8PV>, x17::attn_stream_cfg::smem_bytes<32>());
		}
	} else {
		dim3 grid(unsigned((seq_len + x17::attn_cfg::BQ - 1) / x17::attn_cfg::BQ), unsigned(cfg->n_heads),
				  unsigned(batch));
		dim3 block(x17::attn_cfg::THREADS);
		auto go = [&](auto kernel, uint32_t smem) -> cudaError_t {
			// at least 80 KB so that no more than two CTAs (2 x 256 TMEM columns) share an SM
			smem = smem < 80u * 1024u ? 80u * 1024u : smem;
			cudaError_t e2 = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
			if (e2 != cudaSuccess) return e2;
			kernel<<<grid, block, smem, reinterpret_cast<cudaStream_t>(stream)>>>(tm_q, tm_kv, p);
			return cudaSuccess;
		};
		if (d == 128) {
			ce = go(x17::attn_fwd_kernel<128, DEBUG, FP8PV, SCALED>, x17::attn_cfg::smem_bytes<128>());
		} else if (d == 64) {
			ce = go(x17::attn_fwd_kernel<64, DEBUG, FP8PV, SCALED>, x17::attn_cfg::smem_bytes<64>());
		} else {
			ce = go(x17::attn_fwd_kernel<32, DEBUG, FP8PV, SCALED>, x17::attn_cfg::smem_bytes<32>());
		}
	}
	if (ce != cudaSuccess) {
		return make_diag("x17ai_b200: cudaFuncSetAttribute failed", who, ": cudaFuncSetAttribute failed: ",
						 cudaGetErrorString(ce));
	}
	return launch_result(who);
}

// ---- GEMM --------------------------------------------------------------------------------------

struct GemmPlan {
	int epi;     // x17::GemmEpilogue
	bool f8;     // kind::f8f6f4
	bool split;  // e4m3 activations x split int8 weights: K doubled, A repeated
};

x17ai_DiagnosticBuffer *plan_gemm(x17ai_GemmConfig const *cfg, GemmPlan *plan, char const *who) {
	if (cfg == nullptr) return make_diag("x17ai_b200: null config", who, ": null config");
	bool const a_i8 = cfg->a_dtype == X17AI_DTYPE_INT8, a_f8 = cfg->a_dtype == X17AI_DTYPE_E4M3;
	bool const b_i8 = cfg->b_dtype == X17AI_DTYPE_INT8, b_f8 = cfg->b_dtype == X17AI_DTYPE_E4M3;
	if (!(a_i8 || a_f8) || !(b_i8 || b_f8) || (a_i8 && b_f8)) {
		return make_diag("x17ai_b200: unsupported GEMM dtypes", who,
						 ": gemm supports a/b dtypes int8/int8, e4m3/int8 and e4m3/e4m3");
	}
	plan->f8 = a_f8;
	plan->split = a_f8 && b_i8;
	if (cfg->a_cols == 0 || cfg->a_cols % 128 != 0) {
		return make_diag("x17ai_b200: bad GEMM K", who, ": gemm requires a_cols to be a non-zero multiple of 128, got ",
						 cfg->a_cols);
	}
	if (cfg->b_rows == 0 || cfg->b_rows % 128 != 0) {
		return make_diag("x17ai_b200: bad GEMM N", who, ": gemm requires b_rows to be a non-zero multiple of 128, got ",
						 cfg->b_rows);
	}
	switch (cfg->epilogue) {
	case X17AI_EPILOGUE_SCALE:
		if (cfg->c_dtype == X17AI_DTYPE_INT8) plan->epi = x17::EPI_SCALE_I8;
		else if (cfg->c_dtype == X17AI_DTYPE_I32_RAW) plan->epi = x17::EPI_RAW_I32;
		else return make_diag("x17ai_b200: bad GEMM output", who, ": scale epilogue writes int8 (or raw 32-bit)");
		break;
	case X17AI_EPILOGUE_RMS_NORM:
		if (cfg->c_dtype != X17AI_DTYPE_INT8) {
			return make_diag("x17ai_b200: bad GEMM output", who, ": rms-norm epilogue writes int8");
		}
		if (cfg->head_dim != 32 && cfg->head_dim != 64 && cfg->head_dim != 128) {
			return make_diag("x17ai_b200: bad head_dim", who, ": rms-norm epilogue requires head_dim 32, 64 or 128, got ",
							 cfg->head_dim);
		}
		if (cfg->b_rows % (2 * cfg->head_dim) != 0) {
			return make_diag("x17ai_b200: bad GEMM N", who, ": rms-norm epilogue requires b_rows divisible by 2 * head_dim");
		}
		plan->epi = x17::EPI_L2NORM_KV;
		break;
	case X17AI_EPILOGUE_GEGLU:
		if (cfg->c_dtype != X17AI_DTYPE_E4M3) {
			return make_diag("x17ai_b200: bad GEMM output", who, ": geglu epilogue writes e4m3");
		}
		plan->epi = x17::EPI_GEGLU_E4M3;
		break;
	case X17AI_EPILOGUE_RESIDUAL:
		if (cfg->c_dtype == X17AI_DTYPE_E4M3) plan->epi = x17::EPI_RESID_E4M3;
		else if (cfg->c_dtype == X17AI_DTYPE_INT8) plan->epi = x17::EPI_RESID_I8;
		else return make_diag("x17ai_b200: bad GEMM output", who, ": residual epilogue writes e4m3 or int8");
		break;
	default:
		return make_diag("x17ai_b200: unknown epilogue", who, ": unknown epilogue ", cfg->epilogue);
	}
	return nullptr;
}

// Shape and epilogue constants of one GEMM configuration (everything of GemmParams but the pointers).
void fill_gemm_params(x17ai_GemmConfig const *cfg, GemmPlan const &plan, size_t a_rows, x17::GemmParams &p) {
	using namespace x17::gemm_cfg;
	size_t const k_a = cfg->a_cols;
	size_t const k_total = plan.split ? 2 * k_a : k_a;
	p.m = uint32_t(a_rows);
	p.n_raw = uint32_t(cfg->b_rows);
	p.k = uint32_t(k_total);
	p.k_a = uint32_t(k_a);
	p.tiles_m = uint32_t((a_rows + BM - 1) / BM);
	p.tiles_n = uint32_t((cfg->b_rows + BN - 1) / BN);
	p.head_dim = uint32_t(cfg->head_dim);
	double const inp = cfg->inp_scale, out = cfg->out_scale;
	switch (plan.epi) {
	case x17::EPI_SCALE_I8:
	case x17::EPI_RAW_I32:
		p.c_stride = cfg->b_rows;
		p.k0 = float(inp * out);
		break;
	case x17::EPI_L2NORM_KV:
		p.c_stride = cfg->b_rows;
		p.rrms_cols = uint32_t(cfg->b_rows / (2 * cfg->head_dim));
		p.k0 = float(cfg->eps);
		p.k1 = float(out * std::sqrt(double(cfg->head_dim)));  // gemm.rs:146
		p.k2 = float(inp * out);                               // gemm.rs:152
		break;
	case x17::EPI_GEGLU_E4M3: {
		// math::fast::gelu<INP^2, INP^2 * OUT^2, 1> (cuda/utils_core.cuh:426-448)
		p.c_stride = cfg->b_rows / 2;
		double const inp2 = inp * inp;
		double const ck = std::sqrt(inp2 * 2.0 / M_PI);
		p.k0 = float(0.044715 * ck * inp2);
		p.k1 = float(ck);
		p.k2 = float(0.5 * std::sqrt(inp2 * out * out) * std::sqrt(inp2));
		break;
	}
	default:  // residual (cuda/gemm_b8.cuh:484-505, cuda/utils_core.cuh:397-405,468-483)
		p.c_stride = cfg->b_rows / 2;
		p.resid_stride = cfg->b_rows / 2;
		p.k0 = float(0.5 * (1.0 / 8.0));
		p.k1 = float(M_LN2 * -inp);
		p.k2 = float(inp * 2.0);
		p.k3 = float(inp * out / 2.0);
		p.k4 = float(inp * inp * out);
		break;
	}
}

// The CTA-pair form (gemm.cuh): clusters of two CTAs, one 256 x 256 tile per cluster. `tb_half` is B's map with a box
// of half a tile's rows. Used for more than one row tile when the tiling is X17AI_B200_GEMM_CTA_PAIR.
// How many clusters of the pair kernel the device runs at once. The kernel is persistent, so the grid must not be
// larger: a cluster needs two free SMs of one GPC, and a GPU whose GPCs have an odd number of usable SMs holds fewer
// pairs than sm_count / 2; a cluster left over would run alone after all the others. Asked once per kernel and
// device (the answer depends on neither the stream nor the problem).
template <typename Kernel>
uint32_t max_pair_clusters(Kernel kernel, uint32_t smem, int sm_count) {
	static std::atomic<int> cached[MAX_DEVICES];   // 0 = not asked yet
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return uint32_t(sm_count / 2);
	int n = cached[dev].load(std::memory_order_relaxed);
	if (n == 0) {
		cudaLaunchConfig_t cfg{};
		cfg.gridDim = dim3(unsigned(sm_count / 2) * 2);
		cfg.blockDim = dim3(x17::gemm_cfg::THREADS);
		cfg.dynamicSmemBytes = smem;
		cudaLaunchAttribute attr{};
		attr.id = cudaLaunchAttributeClusterDimension;
		attr.val.clusterDim.x = 2;
		attr.val.clusterDim.y = 1;
		attr.val.clusterDim.z = 1;
		cfg.attrs = &attr;
		cfg.numAttrs = 1;
		int active = 0;
		if (cudaOccupancyMaxActiveClusters(&active, kernel, &cfg) != cudaSuccess || active <= 0) {
			(void)cudaGetLastError();
			active = sm_count / 2;
		}
		n = active < sm_count / 2 ? active : sm_count / 2;
		cached[dev].store(n, std::memory_order_relaxed);
	}
	return uint32_t(n);
}

// The CTA-pair form (gemm.cuh): clusters of two CTAs, one 256 x 256 tile per cluster. `tb_half` is B's map with a box
// of half a tile's rows. Used for more than one row tile when the tiling is X17AI_B200_GEMM_CTA_PAIR.
template <int EPI, bool F8>
cudaError_t gemm_go_pair_kind(int sm_count, cudaStream_t stream, CUtensorMap const &ta, CUtensorMap const &tb_half,
							  x17::GemmParams const &p) {
	uint32_t const smem = x17::gemm_cfg::PAIR_SMEM_BYTES;
	auto const kernel = x17::gemm_pair_kernel<EPI, F8>;
	cudaError_t const ce = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
	if (ce != cudaSuccess) return ce;
	uint32_t const tiles = ((p.m + 2 * x17::gemm_cfg::BM - 1) / (2 * x17::gemm_cfg::BM)) * p.tiles_n;
	uint32_t const fit = max_pair_clusters(kernel, smem, sm_count);
	uint32_t const clusters = tiles < fit ? tiles : fit;
	kernel<<<dim3(2 * clusters), x17::gemm_cfg::THREADS, smem, stream>>>(ta, tb_half, p);
	return cudaSuccess;
}
template <int EPI>
cudaError_t gemm_go_pair(bool f8, int sm_count, cudaStream_t stream, CUtensorMap const &ta, CUtensorMap const &tb_half,
						 x17::GemmParams const &p) {
	return f8 ? gemm_go_pair_kind<EPI, true>(sm_count, stream, ta, tb_half, p)
			  : gemm_go_pair_kind<EPI, false>(sm_count, stream, ta, tb_half, p);
}

template <int EPI>
cudaError_t gemm_go(bool f8, dim3 grid, cudaStream_t stream, CUtensorMap const &ta, CUtensorMap const &tb,
					x17::GemmParams const &p) {
	uint32_t const smem = x17::gemm_cfg::SMEM_BYTES;
	cudaError_t ce;
	if (f8) {
		ce = cudaFuncSetAttribute(x17::gemm_kernel<EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
		if (ce != cudaSuccess) return ce;
		x17::gemm_kernel<EPI, true><<<grid, x17::gemm_cfg::THREADS, smem, stream>>>(ta, tb, p);
	} else {
		ce = cudaFuncSetAttribute(x17::gemm_kernel<EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
		if (ce != cudaSuccess) return ce;
		x17::gemm_kernel<EPI, false><<<grid, x17::gemm_cfg::THREADS, smem, stream>>>(ta, tb, p);
	}
	return cudaSuccess;
}

__global__ void split_i8_weights_kernel(int8_t const *w, uint64_t rows, uint64_t cols, uint8_t *out) {
	uint64_t const n = rows * cols;
	for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
		uint64_t const r = i / cols, c = i % cols;
		int const v = w[i];
		int const hi = (v + 128) / 16 - 8;  // floor(v / 16)
		int const lo = v - 16 * hi;         // 0 .. 15
		// standard e4m3 encodings of the integers 16*hi (multiples of 16 up to +-128) and lo
		auto enc = [](int x) -> uint8_t {
			if (x == 0) return 0;
			uint32_t const s = x < 0 ? 0x80u : 0u;
			uint32_t const a = uint32_t(x < 0 ? -x : x);
			int const e = 31 - __clz(int(a));            // a = 1.mmm * 2^e, e <= 7
			uint32_t const mant = e >= 3 ? (a >> (e - 3)) & 7u : (a << (3 - e)) & 7u;
			return uint8_t(s | (uint32_t(e + 7) << 3) | mant);
		};
		out[r * 2 * cols + c] = enc(16 * hi);
		out[r * 2 * cols + cols + c] = enc(lo);
	}
}



// ---- decode without allocation -------------------------------------------------------------------
// Scratch for the split-KV partials of x17ai_b200_attn_decode_i8_noalloc. It lives in the
// library image: every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t NOALLOC_SCRATCH_FLOATS = size_t(1) << 20;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

struct NoAllocDevice {
	std::mutex mutex;
	bool ready = false;        // set once the set-up has succeeded; a failed set-up is tried again by the next call
	float *scratch = nullptr;  // device address of g_noalloc_scratch on this device
	int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[MAX_DEVICES];

// fixed-capacity FfiBuffer for x17ai_b200_take_diagnostic
struct FixedBuf {
	char *ptr;
	size_t cap;
	size_t len;
};
x17ai_FfiSpan fb_span(void *self) {
	auto *b = static_cast<FixedBuf *>(self);
	return x17ai_FfiSpan{b->ptr, b->len};
}
x17ai_FfiSpan fb_buf_span(void *self) {
	auto *b = static_cast<FixedBuf *>(self);
	return x17ai_FfiSpan{b->ptr, b->cap};
}
x17ai_FfiSpan fb_extend(void *self, size_t additional) {
	auto *b = static_cast<FixedBuf *>(self);
	size_t const room = b->cap - b->len;
	size_t const n = additional <= room ? additional : 0;  // all or nothing, like Vec::try_reserve
	x17ai_FfiSpan s{b->ptr + b->len, n};
	b->len += n;
	return s;
}
void fb_clear(void *self) { static_cast<FixedBuf *>(self)->len = 0; }
void fb_set_len(void *self, size_t n) {
	auto *b = static_cast<FixedBuf *>(self);
	if (n <= b->cap) b->len = n;
}
x17ai_FfiBufferVMT const g_fixed_vmt{fb_span, fb_buf_span, fb_extend, fb_clear, fb_set_len};

}  // namespace

extern "C" {

size_t x17ai_b200_take_diagnostic(x17ai_DiagnosticBuffer *diag, char *dst, size_t cap) {
	if (diag == nullptr) return 0;
	FixedBuf buf{dst, dst != nullptr ? cap : 0, 0};
	x17ai_move_diagnostic(diag, x17ai_FfiBuffer{&buf, &g_fixed_vmt});
	return buf.len;
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_object_desc(x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg,
													x17ai_AttnObjectDesc *desc) {
	char const *who = "x17ai_b200_attn_object_desc()";
	if (desc == nullptr) return static_diag("x17ai_b200_attn_object_desc(): null argument");
	if (auto *d = check_attn_config(cfg, who)) return d;
	StreamScope scope(stream, who);   // the driver encodes tensor maps inside a context
	if (scope.diag) return scope.diag;
	std::memset(desc, 0, sizeof(*desc));
	uint32_t const d = uint32_t(cfg->head_dim);
	desc->threads = x17::attn_cfg::THREADS;
	desc->q_per_block = x17::attn_cfg::BQ;
	uint32_t const smem = d == 128 ? x17::attn_cfg::smem_bytes<128>()
						  : d == 64 ? x17::attn_cfg::smem_bytes<64>()
									: x17::attn_cfg::smem_bytes<32>();
	desc->smem_bytes = smem < 80u * 1024u ? 80u * 1024u : smem;
	void *const dummy = reinterpret_cast<void *>(uintptr_t(1) << 20);
	size_t const rows = x17::attn_cfg::BQ;   // placeholder: the kernel object writes the sequence length
	CUtensorMap tq, tkv;
	CUresult e = make_map_3d(&tq, dummy, cfg->n_heads * d, rows, 1, cfg->q_stride, cfg->q_stride * rows, d, x17::attn_cfg::BQ);
	if (e == CUDA_SUCCESS) {
		e = make_map_3d(&tkv, dummy, 2 * cfg->n_heads * d, rows, 1, cfg->kv_stride, cfg->kv_stride * rows, d,
						x17::attn_cfg::BKV);
	}
	if (e != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cuTensorMapEncodeTiled failed", who, ": cuTensorMapEncodeTiled failed: ",
						 x17::cu_error_text(e));
	}
	std::memcpy(desc->map_q, &tq, 128);
	std::memcpy(desc->map_kv, &tkv, 128);
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_gemm_object_desc(x17ai_CudaStreamHandle *stream, x17ai_GemmConfig const *cfg,
													x17ai_GemmObjectDesc *desc) {
	char const *who = "x17ai_b200_gemm_object_desc()";
	if (desc == nullptr) return static_diag("x17ai_b200_gemm_object_desc(): null argument");
	GemmPlan plan{};
	if (auto *d = plan_gemm(cfg, &plan, who)) return d;
	if (plan.f8 && !plan.split) {
		return make_diag("x17ai_b200: unsupported kernel object", who,
						 ": kernel objects exist for the int8 x int8 and the e4m3 x int8 GEMMs of the reference's block");
	}
	StreamScope scope(stream, who);   // the driver encodes tensor maps inside a context
	if (scope.diag) return scope.diag;
	using namespace x17::gemm_cfg;
	x17::GemmParams p{};
	fill_gemm_params(cfg, plan, BM, p);
	std::memset(desc, 0, sizeof(*desc));
	desc->epilogue_kind = plan.epi;
	desc->n_raw = p.n_raw;
	desc->k = p.k;
	desc->head_dim = p.head_dim;
	desc->rrms_cols = p.rrms_cols;
	desc->c_stride = p.c_stride;
	desc->resid_stride = p.resid_stride;
	desc->k0 = p.k0;
	desc->k1 = p.k1;
	desc->k2 = p.k2;
	desc->k3 = p.k3;
	desc->k4 = p.k4;
	desc->smem_bytes = SMEM_BYTES;
	desc->threads = THREADS;
	desc->m_per_block = BM;
	desc->n_per_block = BN;
	desc->k_a = plan.split ? p.k_a : 0;
	// templates of the two tensor maps: shape, strides, box and swizzle are final, the base address and
	// A's row count are written by the kernel object itself at launch
	void *const dummy = reinterpret_cast<void *>(uintptr_t(1) << 20);
	CUtensorMap ta, tb;
	CUresult e = make_map_2d(&ta, dummy, cfg->a_cols, BM, cfg->a_cols, BK, BM);
	// B: the int8 weights [N, K], or the object's own two e4m3 planes [N, 2K] of them
	if (e == CUDA_SUCCESS) e = make_map_2d(&tb, dummy, p.k, cfg->b_rows, p.k, BK, BN);
	if (e != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cuTensorMapEncodeTiled failed", who, ": cuTensorMapEncodeTiled failed: ",
						 x17::cu_error_text(e));
	}
	static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
	std::memcpy(desc->map_a, &ta, 128);
	std::memcpy(desc->map_b, &tb, 128);
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_object_status(x17ai_CudaStreamHandle *stream, x17ai_CudaModuleHandle *module,
												 uint32_t status[4]) {
	char const *who = "x17ai_b200_object_status()";
	if (module == nullptr || status == nullptr) return static_diag("x17ai_b200_object_status(): null argument");
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	CUdeviceptr ptr = 0;
	size_t bytes = 0;
	CUresult e = DRV(cuModuleGetGlobal)(&ptr, &bytes, reinterpret_cast<CUmodule>(module), "x17_status");
	if (e != CUDA_SUCCESS || bytes < 4 * sizeof(uint32_t)) {
		return make_diag("x17ai_b200: no status words", who, ": the module exports no x17_status words: ",
						 x17::cu_error_text(e));
	}
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
	cudaError_t ce = cudaStreamSynchronize(s);
	if (ce == cudaSuccess) ce = cudaMemcpy(status, reinterpret_cast<void *>(ptr), 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
	if (ce == cudaSuccess) ce = cudaMemset(reinterpret_cast<void *>(ptr), 0, 4 * sizeof(uint32_t));
	if (ce != cudaSuccess) {
		return make_diag("x17ai_b200: status read failed", who, ": reading the status words failed: ", cudaGetErrorString(ce));
	}
	return nullptr;
}

uint64_t x17ai_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

x17ai_DiagnosticBuffer *x17ai_b200_read_status(x17ai_CudaStreamHandle *stream, uint32_t status[4]) {
	char const *who = "x17ai_b200_read_status()";
	if (status == nullptr) return static_diag("x17ai_b200_read_status(): null argument");
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
	cudaError_t e = cudaMemcpyAsync(status, scope.state().status, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
	if (e == cudaSuccess) e = cudaMemsetAsync(scope.state().status, 0, 4 * sizeof(uint32_t), s);
	if (e == cudaSuccess) e = cudaStreamSynchronize(s);
	if (e != cudaSuccess) {
		return make_diag("x17ai_b200_read_status(): failed", who, ": ", cudaGetErrorString(e));
	}
	return nullptr;
}

// ---- stream capture: a sequence of this library's launches replayed as one CUDA graph ---------

struct x17ai_b200_Graph {
	cudaGraphExec_t exec = nullptr;
	uint64_t kernel_nodes = 0;
};

x17ai_DiagnosticBuffer *x17ai_b200_graph_begin(x17ai_CudaStreamHandle *stream) {
	char const *who = "x17ai_b200_graph_begin()";
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	cudaError_t e = cudaStreamBeginCapture(reinterpret_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal);
	if (e != cudaSuccess) {
		return make_diag("x17ai_b200_graph_begin(): failed", who, ": cannot begin capture: ", cudaGetErrorString(e));
	}
	// an invalidated capture no longer answers cuStreamGetCtx: graph_end finds the context here
	std::lock_guard<std::mutex> lock(g_capture_mutex);
	g_capture_ctx[stream] = scope.ctx;
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_graph_end(x17ai_CudaStreamHandle *stream, x17ai_b200_Graph **graph) {
	char const *who = "x17ai_b200_graph_end()";
	if (graph == nullptr) return static_diag("x17ai_b200_graph_end(): null argument");
	*graph = nullptr;
	if (stream == nullptr) return static_diag("x17ai_b200_graph_end(): null stream");
	CUcontext ctx = nullptr;
	{
		std::lock_guard<std::mutex> lock(g_capture_mutex);
		auto it = g_capture_ctx.find(stream);
		if (it == g_capture_ctx.end()) return static_diag("x17ai_b200_graph_end(): no capture was begun on this stream");
		ctx = it->second;
		g_capture_ctx.erase(it);
	}
	struct Pushed {
		bool ok;
		explicit Pushed(CUcontext c) : ok(DRV(cuCtxPushCurrent)(c) == CUDA_SUCCESS) {}
		~Pushed() {
			CUcontext popped = nullptr;
			if (ok) DRV(cuCtxPopCurrent)(&popped);
		}
	} pushed(ctx);
	if (!pushed.ok) return static_diag("x17ai_b200_graph_end(): cannot enter the stream's context");
	cudaGraph_t g = nullptr;
	cudaError_t e = cudaStreamEndCapture(reinterpret_cast<cudaStream_t>(stream), &g);
	if (e != cudaSuccess || g == nullptr) {
		cudaGetLastError();   // ending an invalidated capture returns the stream to normal use
		return make_diag("x17ai_b200_graph_end(): failed", who, ": the capture was invalidated: ",
						 cudaGetErrorString(e));
	}
	size_t n = 0;
	uint64_t kernels = 0;
	if (cudaGraphGetNodes(g, nullptr, &n) == cudaSuccess && n > 0) {
		std::vector<cudaGraphNode_t> nodes(n);
		if (cudaGraphGetNodes(g, nodes.data(), &n) == cudaSuccess) {
			for (size_t i = 0; i < n; ++i) {
				cudaGraphNodeType t;
				if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
			}
		}
	}
	cudaGraphExec_t exec = nullptr;
	e = cudaGraphInstantiate(&exec, g, 0);
	cudaGraphDestroy(g);
	if (e != cudaSuccess) {
		return make_diag("x17ai_b200_graph_end(): failed", who, ": cannot instantiate the graph: ", cudaGetErrorString(e));
	}
	auto *out = new (std::nothrow) x17ai_b200_Graph;
	if (out == nullptr) {
		cudaGraphExecDestroy(exec);
		return static_diag("x17ai_b200_graph_end(): out of memory");
	}
	out->exec = exec;
	out->kernel_nodes = kernels;
	*graph = out;
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_graph_launch(x17ai_b200_Graph *graph, x17ai_CudaStreamHandle *stream) {
	char const *who = "x17ai_b200_graph_launch()";
	if (graph == nullptr || graph->exec == nullptr) return static_diag("x17ai_b200_graph_launch(): null graph");
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	cudaError_t e = cudaGraphLaunch(graph->exec, reinterpret_cast<cudaStream_t>(stream));
	if (e != cudaSuccess) {
		return make_diag("x17ai_b200_graph_launch(): failed", who, ": graph launch failed: ", cudaGetErrorString(e));
	}
	g_launches.fetch_add(graph->kernel_nodes, std::memory_order_relaxed);
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_graph_destroy(x17ai_b200_Graph *graph, x17ai_CudaStreamHandle *stream) {
	char const *who = "x17ai_b200_graph_destroy()";
	if (graph == nullptr) return nullptr;
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	if (graph->exec != nullptr) cudaGraphExecDestroy(graph->exec);
	delete graph;
	return nullptr;
}

uint64_t x17ai_b200_graph_kernel_nodes(x17ai_b200_Graph const *graph) { return graph ? graph->kernel_nodes : 0; }

int x17ai_b200_set_attn_schedule(int schedule, unsigned tiles_per_item) {
	if (schedule != X17AI_B200_ATTN_PERSISTENT && schedule != X17AI_B200_ATTN_PER_TILE) return -1;
	if (tiles_per_item > 4096) return -1;
	g_attn_schedule.store(schedule, std::memory_order_relaxed);
	g_attn_item_tiles.store(tiles_per_item, std::memory_order_relaxed);
	return 0;
}

int x17ai_b200_set_gemm_tiling(int tiling) {
	if (tiling != X17AI_B200_GEMM_ONE_CTA && tiling != X17AI_B200_GEMM_CTA_PAIR) return -1;
	g_gemm_tiling.store(tiling, std::memory_order_relaxed);
	return 0;
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_meta(x17ai_AttnConfig const *cfg, x17ai_AttnMeta *meta) {
	char const *who = "x17ai_b200_attn_meta()";
	if (auto *d = check_attn_config(cfg, who)) return d;
	if (meta == nullptr) return static_diag("x17ai_b200_attn_meta(): null argument");
	meta->threads_per_block = x17::attn_cfg::THREADS;
	meta->q_per_block = x17::attn_cfg::BQ;
	uint32_t smem = cfg->head_dim == 128 ? x17::attn_cfg::smem_bytes<128>()
					: cfg->head_dim == 64 ? x17::attn_cfg::smem_bytes<64>()
										  : x17::attn_cfg::smem_bytes<32>();
	meta->smem_bytes = smem < 80u * 1024u ? 80u * 1024u : smem;
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size) {
	return attn_launch<false>("x17ai_b200_attn_fwd_i8()", stream, cfg, batch, seq_len, q, kv, sink_k, sink_v,
							  attn_temperature, out, l, window_size, nullptr, nullptr, nullptr);
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_to_peers(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, int8_t *const *peer_out,
	size_t n_peers) {
	return attn_launch<false>("x17ai_b200_attn_fwd_i8_to_peers()", stream, cfg, batch, seq_len, q, kv, sink_k, sink_v,
							  attn_temperature, out, l, window_size, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
							  nullptr, peer_out, n_peers);
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_pv_fp8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, uint8_t const *kv, int8_t const *sink_k, uint8_t const *sink_v,
	float const *attn_temperature, float const *v_scale, uint16_t *out_bf16, float *l, size_t window_size) {
	if (v_scale == nullptr) return static_diag("x17ai_b200_attn_fwd_pv_fp8(): null v_scale");
	return attn_launch<false, true>("x17ai_b200_attn_fwd_pv_fp8()", stream, cfg, batch, seq_len, q,
									reinterpret_cast<int8_t const *>(kv), sink_k,
									reinterpret_cast<int8_t const *>(sink_v), attn_temperature, out_bf16, l,
									window_size, nullptr, nullptr, nullptr, v_scale);
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_scaled(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, float const *q_scale, int8_t const *kv, float const *k_scale, float const *v_scale,
	int8_t const *sink_k, int8_t const *sink_v, float const *attn_temperature, uint16_t *out_bf16, float *l,
	size_t window_size) {
	if (!q_scale || !k_scale || !v_scale) return static_diag("x17ai_b200_attn_fwd_i8_scaled(): null scale tensor");
	return attn_launch<false, false, true>("x17ai_b200_attn_fwd_i8_scaled()", stream, cfg, batch, seq_len, q, kv, sink_k,
										   sink_v, attn_temperature, out_bf16, l, window_size, nullptr, nullptr, nullptr,
										   nullptr, q_scale, k_scale, v_scale);
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_debug(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size,
	int32_t *dbg_s, uint8_t *dbg_p, int32_t *dbg_o) {
	if (!dbg_s || !dbg_p || !dbg_o) return static_diag("x17ai_b200_attn_fwd_i8_debug(): null debug buffer");
	return attn_launch<true>("x17ai_b200_attn_fwd_i8_debug()", stream, cfg, batch, seq_len, q, kv, sink_k,
							 sink_v, attn_temperature, out, l, window_size, dbg_s, dbg_p, dbg_o);
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_decode_i8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch,
	int8_t const *q, int8_t const *kv_cache, size_t kv_capacity, size_t kv_len,
	uint32_t const *kv_lens, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, size_t n_splits) {
	char const *who = "x17ai_b200_attn_decode_i8()";
	if (auto *d = check_attn_config(cfg, who)) return d;
	if (batch == 0) return make_diag("x17ai_b200: empty decode input", who, ": decode input q has zero size");
	if (batch > 65535 || kv_capacity >= (size_t(1) << 31) || kv_len > kv_capacity) {
		return make_diag("x17ai_b200: decode shape out of range", who, ": decode shape out of range (kv_len ",
						 kv_len, ", kv_capacity ", kv_capacity, ")");
	}
	if (window_size > 0 && window_size % 16 != 0) {
		return make_diag("x17ai_b200: bad window", who,
						 ": attention window_size must be zero or divisible by 16, got ", window_size);
	}
	if (!q || !kv_cache || !sink_k || !sink_v || !attn_temperature || !out) {
		return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	}
	if (!aligned16(q) || !aligned16(kv_cache) || !aligned16(sink_k)) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);

	size_t const pairs = batch * cfg->n_heads;
	if (n_splits == 0) {  // choose: enough CTAs for two waves of 4 CTAs per SM
		size_t const want = size_t(scope.state().sm_count) * 8;
		n_splits = pairs >= want ? 1 : (want + pairs - 1) / pairs;
		size_t const max_splits = kv_len / 256 > 0 ? kv_len / 256 : 1;
		if (n_splits > max_splits) n_splits = max_splits;
	}
	if (n_splits > 65535) n_splits = 65535;

	uint32_t const d = uint32_t(cfg->head_dim);
	x17::DecodeParams p{};
	p.q = q;
	p.q_stride = cfg->q_stride;
	p.kv = kv_cache;
	p.kv_stride = cfg->kv_stride;
	p.kv_batch_stride = cfg->kv_stride * kv_capacity;
	p.kv_lens = kv_lens;
	p.kv_len = uint32_t(kv_len);
	p.kv_capacity = uint32_t(kv_capacity);
	p.window = window_size == 0 ? 0xFFFFFFFFu : uint32_t(((window_size - 1) / 16 + 1) * 16);
	p.sink_k = sink_k;
	p.sink_v = sink_v;
	p.temperature = attn_temperature;
	p.out = out;
	p.o_stride = cfg->o_stride;
	p.l = l;
	p.n_heads = uint32_t(cfg->n_heads);
	p.n_splits = uint32_t(n_splits);
	p.scratch = nullptr;
	if (n_splits > 1) {
		size_t const bytes = pairs * n_splits * (d + 2) * sizeof(float);
		cudaError_t e = cudaMallocAsync(reinterpret_cast<void **>(&p.scratch), bytes, s);
		if (e != cudaSuccess) {
			return make_diag("x17ai_b200: scratch allocation failed", who, ": cudaMallocAsync(", bytes,
							 ") failed: ", cudaGetErrorString(e));
		}
	}
	dim3 grid(unsigned(cfg->n_heads), unsigned(batch), unsigned(n_splits));
	dim3 mgrid(unsigned(cfg->n_heads), unsigned(batch));
	if (d == 128) {
		x17::attn_decode_kernel<128><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<128><<<mgrid, 128, 0, s>>>(p);
	} else if (d == 64) {
		x17::attn_decode_kernel<64><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<64><<<mgrid, 64, 0, s>>>(p);
	} else {
		x17::attn_decode_kernel<32><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<32><<<mgrid, 32, 0, s>>>(p);
	}
	x17ai_DiagnosticBuffer *res = launch_result(who);
	if (n_splits > 1) {
		if (res == nullptr) g_launches.fetch_add(1, std::memory_order_relaxed);
		cudaFreeAsync(p.scratch, s);
	}
	return res;
}

x17ai_DiagnosticBuffer *x17ai_b200_attn_decode_i8_noalloc(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch,
	int8_t const *q, int8_t const *kv_cache, size_t kv_capacity, size_t kv_len,
	uint32_t const *kv_lens, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, size_t n_splits) {
	char const *who = "x17ai_b200_attn_decode_i8_noalloc()";
	if (auto *d = check_attn_config(cfg, who)) return d;
	if (batch == 0) return make_diag("x17ai_b200: empty decode input", who, ": decode input q has zero size");
	if (batch > 65535 || kv_capacity >= (size_t(1) << 31) || kv_len > kv_capacity) {
		return make_diag("x17ai_b200: decode shape out of range", who, ": decode shape out of range (kv_len ",
						 kv_len, ", kv_capacity ", kv_capacity, ")");
	}
	if (window_size > 0 && window_size % 16 != 0) {
		return make_diag("x17ai_b200: bad window", who,
						 ": attention window_size must be zero or divisible by 16, got ", window_size);
	}
	if (!q || !kv_cache || !sink_k || !sink_v || !attn_temperature || !out) {
		return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	}
	if (!aligned16(q) || !aligned16(kv_cache) || !aligned16(sink_k)) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	if (stream == nullptr) return make_diag("x17ai_b200: null stream", who, ": null stream");
	if (!x17::driver().ok) {
		return make_diag("x17ai_b200: CUDA driver not available", who,
						 ": the CUDA driver is not available on this machine; this library has no CPU path");
	}
	// Enter the stream's context by hand: the usual per-device set-up of this library allocates
	// its status words with cudaMalloc, which this entry point must not do.
	CUcontext ctx = nullptr;
	CUresult ce = DRV(cuStreamGetCtx)(reinterpret_cast<CUstream>(stream), &ctx);
	if (ce == CUDA_SUCCESS) ce = DRV(cuCtxPushCurrent)(ctx);
	if (ce != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cannot enter the stream's context", who,
						 ": cannot enter the stream's context: ", x17::cu_error_text(ce));
	}
	struct Pop {
		~Pop() {
			CUcontext popped = nullptr;
			DRV(cuCtxPopCurrent)(&popped);
		}
	} pop;
	CUdevice dev = -1;
	if (DRV(cuCtxGetDevice)(&dev) != CUDA_SUCCESS || int(dev) < 0 || int(dev) >= MAX_DEVICES) {
		return make_diag("x17ai_b200: cannot resolve the device", who, ": cannot resolve the device");
	}
	NoAllocDevice &nd = g_noalloc_dev[int(dev)];
	// First call on this device (with the device current): resolve the device address of the
	// scratch array. In host code the array's name is only a stand-in, not a device pointer.
	// Only a successful set-up is remembered: after a failure (a first call made inside a stream capture, a
	// transient error) the next call tries again.
	{
		std::lock_guard<std::mutex> lock(nd.mutex);
		if (!nd.ready) {
			int major = 0;
			cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, int(dev));
			if (e == cudaSuccess && major != 10) {
				return make_diag("x17ai_b200: device not supported", who, ": this library needs an sm_100 GPU");
			}
			float *ptr = nullptr;
			if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch);
			int sms = 0;
			if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, int(dev));
			if (e != cudaSuccess || ptr == nullptr) {
				(void)cudaGetLastError();
				return make_diag("x17ai_b200: scratch set-up failed", who, ": cudaGetSymbolAddress failed: ",
								 cudaGetErrorString(e));
			}
			nd.scratch = ptr;
			nd.sm_count = sms;
			nd.ready = true;
		}
	}
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
	size_t const pairs = batch * cfg->n_heads;
	if (n_splits == 0) {
		size_t const want = size_t(nd.sm_count) * 8;
		n_splits = pairs >= want ? 1 : (want + pairs - 1) / pairs;
		size_t const max_splits = kv_len / 256 > 0 ? kv_len / 256 : 1;
		if (n_splits > max_splits) n_splits = max_splits;
	}
	uint32_t const d = uint32_t(cfg->head_dim);
	size_t const need = n_splits > 1 ? pairs * n_splits * (d + 2) : 0;
	if (n_splits > 65535 || need > NOALLOC_SCRATCH_FLOATS) {
		return make_diag("x17ai_b200: scratch too small", who, ": batch * n_heads * n_splits * (head_dim + 2) = ",
						 need, " floats exceeds the built-in scratch of ", NOALLOC_SCRATCH_FLOATS,
						 " floats (4 MiB); use fewer splits or x17ai_b200_attn_decode_i8");
	}
	x17::DecodeParams p{};
	p.q = q;
	p.q_stride = cfg->q_stride;
	p.kv = kv_cache;
	p.kv_stride = cfg->kv_stride;
	p.kv_batch_stride = cfg->kv_stride * kv_capacity;
	p.kv_lens = kv_lens;
	p.kv_len = uint32_t(kv_len);
	p.kv_capacity = uint32_t(kv_capacity);
	p.window = window_size == 0 ? 0xFFFFFFFFu : uint32_t(((window_size - 1) / 16 + 1) * 16);
	p.sink_k = sink_k;
	p.sink_v = sink_v;
	p.temperature = attn_temperature;
	p.out = out;
	p.o_stride = cfg->o_stride;
	p.l = l;
	p.n_heads = uint32_t(cfg->n_heads);
	p.n_splits = uint32_t(n_splits);
	p.scratch = nd.scratch;  // every split writes its whole slot before the merge reads it
	dim3 grid(unsigned(cfg->n_heads), unsigned(batch), unsigned(n_splits));
	dim3 mgrid(unsigned(cfg->n_heads), unsigned(batch));
	if (d == 128) {
		x17::attn_decode_kernel<128><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<128><<<mgrid, 128, 0, s>>>(p);
	} else if (d == 64) {
		x17::attn_decode_kernel<64><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<64><<<mgrid, 64, 0, s>>>(p);
	} else {
		x17::attn_decode_kernel<32><<<grid, x17::dec_cfg::THREADS, 0, s>>>(p);
		if (n_splits > 1) x17::attn_decode_merge_kernel<32><<<mgrid, 32, 0, s>>>(p);
	}
	x17ai_DiagnosticBuffer *res = launch_result(who);
	if (res == nullptr && n_splits > 1) g_launches.fetch_add(1, std::memory_order_relaxed);
	return res;
}

x17ai_DiagnosticBuffer *x17ai_b200_gemm_meta(x17ai_GemmConfig const *cfg, x17ai_GemmMeta *meta) {
	GemmPlan plan{};
	if (auto *d = plan_gemm(cfg, &plan, "x17ai_b200_gemm_meta()")) return d;
	if (meta == nullptr) return static_diag("x17ai_b200_gemm_meta(): null argument");
	meta->threads_per_block = x17::gemm_cfg::THREADS;
	meta->smem_bytes = x17::gemm_cfg::SMEM_BYTES;
	meta->m_per_block = x17::gemm_cfg::BM;
	meta->n_per_block = x17::gemm_cfg::BN;
	return nullptr;
}

x17ai_DiagnosticBuffer *x17ai_b200_gemm_fwd(
	x17ai_CudaStreamHandle *stream, x17ai_GemmConfig const *cfg,
	void const *a, size_t a_rows, void const *b, size_t b_rows,
	void *c, float *rrms, int8_t const *residual) {
	char const *who = "x17ai_b200_gemm_fwd()";
	GemmPlan plan{};
	if (auto *d = plan_gemm(cfg, &plan, who)) return d;
	if (a_rows == 0) return make_diag("x17ai_b200: empty GEMM input", who, ": gemm input a has zero size");
	if (b_rows != cfg->b_rows) {
		return make_diag("x17ai_b200: bad GEMM shape", who, ": gemm input b has ", b_rows,
						 " rows, but should have ", cfg->b_rows);
	}
	if (a_rows >= (size_t(1) << 31) || cfg->b_rows >= (size_t(1) << 31) || cfg->a_cols >= (size_t(1) << 30)) {
		return make_diag("x17ai_b200: GEMM shape out of range", who, ": gemm shape out of range");
	}
	if (!a || !b || !c) return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	if (plan.epi == x17::EPI_L2NORM_KV && rrms == nullptr) {
		return make_diag("x17ai_b200: null tensor", who, ": rms-norm epilogue needs the rrms output");
	}
	if ((plan.epi == x17::EPI_RESID_E4M3 || plan.epi == x17::EPI_RESID_I8) && residual == nullptr) {
		return make_diag("x17ai_b200: null tensor", who, ": residual epilogue needs the residual input");
	}
	if (!aligned16(a) || !aligned16(b) || !aligned16(c) || (residual && !aligned16(residual))) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;

	using namespace x17::gemm_cfg;
	size_t const k_a = cfg->a_cols;
	size_t const k_total = plan.split ? 2 * k_a : k_a;
	CUtensorMap ta, tb;
	bool const pair = g_gemm_tiling.load(std::memory_order_relaxed) == X17AI_B200_GEMM_CTA_PAIR && a_rows > BM
					  && cfg->b_rows % BN == 0 && scope.state().sm_count >= 2;
	CUresult e = make_map_2d(&ta, a, k_a, a_rows, k_a, BK, BM);
	if (e == CUDA_SUCCESS) e = make_map_2d(&tb, b, k_total, cfg->b_rows, k_total, BK, pair ? BN / 2 : BN);
	if (e != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cuTensorMapEncodeTiled failed", who,
						 ": cuTensorMapEncodeTiled failed: ", x17::cu_error_text(e));
	}
	x17::GemmParams p{};
	fill_gemm_params(cfg, plan, a_rows, p);
	p.c = c;
	p.residual = residual;
	p.rrms = rrms;
	p.status = scope.state().status;
	uint32_t const n_tiles = p.tiles_m * p.tiles_n;
	uint32_t const ctas = n_tiles < uint32_t(scope.state().sm_count) ? n_tiles : uint32_t(scope.state().sm_count);
	dim3 grid(ctas);
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
	cudaError_t ce;
	if (pair) {
		int const sms = scope.state().sm_count;
		switch (plan.epi) {
		case x17::EPI_SCALE_I8: ce = gemm_go_pair<x17::EPI_SCALE_I8>(plan.f8, sms, s, ta, tb, p); break;
		case x17::EPI_RAW_I32: ce = gemm_go_pair<x17::EPI_RAW_I32>(plan.f8, sms, s, ta, tb, p); break;
		case x17::EPI_L2NORM_KV: ce = gemm_go_pair<x17::EPI_L2NORM_KV>(plan.f8, sms, s, ta, tb, p); break;
		case x17::EPI_GEGLU_E4M3: ce = gemm_go_pair<x17::EPI_GEGLU_E4M3>(plan.f8, sms, s, ta, tb, p); break;
		case x17::EPI_RESID_E4M3: ce = gemm_go_pair<x17::EPI_RESID_E4M3>(plan.f8, sms, s, ta, tb, p); break;
		default: ce = gemm_go_pair<x17::EPI_RESID_I8>(plan.f8, sms, s, ta, tb, p); break;
		}
	} else
	switch (plan.epi) {
	case x17::EPI_SCALE_I8: ce = gemm_go<x17::EPI_SCALE_I8>(plan.f8, grid, s, ta, tb, p); break;
	case x17::EPI_RAW_I32: ce = gemm_go<x17::EPI_RAW_I32>(plan.f8, grid, s, ta, tb, p); break;
	case x17::EPI_L2NORM_KV: ce = gemm_go<x17::EPI_L2NORM_KV>(plan.f8, grid, s, ta, tb, p); break;
	case x17::EPI_GEGLU_E4M3: ce = gemm_go<x17::EPI_GEGLU_E4M3>(plan.f8, grid, s, ta, tb, p); break;
	case x17::EPI_RESID_E4M3: ce = gemm_go<x17::EPI_RESID_E4M3>(plan.f8, grid, s, ta, tb, p); break;
	default: ce = gemm_go<x17::EPI_RESID_I8>(plan.f8, grid, s, ta, tb, p); break;
	}
	if (ce != cudaSuccess) {
		return make_diag("x17ai_b200: cudaFuncSetAttribute failed", who, ": cudaFuncSetAttribute failed: ",
						 cudaGetErrorString(ce));
	}
	return launch_result(who);
}

x17ai_DiagnosticBuffer *x17ai_b200_qkvg_fwd_i8(
	x17ai_CudaStreamHandle *stream, x17ai_QkvgConfig const *cfg, int8_t const *x, size_t rows,
	int8_t const *w_qkvg, int8_t *q, int8_t *kv, float *k_rrms, int8_t *g) {
	char const *who = "x17ai_b200_qkvg_fwd_i8()";
	if (cfg == nullptr) return make_diag("x17ai_b200: null config", who, ": null config");
	size_t const hd = cfg->n_heads * cfg->head_dim;
	size_t const n_q = hd, n_kv = 2 * hd, n_g = cfg->gate_cols;
	if (cfg->n_heads == 0 || (cfg->head_dim != 32 && cfg->head_dim != 64 && cfg->head_dim != 128)) {
		return make_diag("x17ai_b200: bad qkvg config", who, ": qkvg requires n_heads > 0 and head_dim 32, 64 or 128");
	}
	if (cfg->model_dim == 0 || cfg->model_dim % 128 != 0) {
		return make_diag("x17ai_b200: bad qkvg config", who, ": qkvg requires model_dim to be a non-zero multiple of 128, got ",
						 cfg->model_dim);
	}
	if (n_q % x17::gemm_cfg::BN != 0 || n_g % 128 != 0) {
		return make_diag("x17ai_b200: bad qkvg config", who, ": qkvg requires n_heads * head_dim to be a multiple of ",
						 x17::gemm_cfg::BN, " and gate_cols a multiple of 128, got ", n_q, " and ", n_g);
	}
	if (rows == 0) return make_diag("x17ai_b200: empty input", who, ": qkvg input x has zero size");
	if (rows >= (size_t(1) << 31)) return make_diag("x17ai_b200: shape out of range", who, ": too many rows");
	if (!x || !w_qkvg || !q || !kv || !k_rrms || (n_g != 0 && !g)) {
		return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	}
	if (!aligned16(x) || !aligned16(w_qkvg) || !aligned16(q) || !aligned16(kv) || (g && !aligned16(g))) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	using namespace x17::gemm_cfg;
	size_t const n_raw = n_q + n_kv + n_g;
	CUtensorMap ta, tb;
	bool const pair = g_gemm_tiling.load(std::memory_order_relaxed) == X17AI_B200_GEMM_CTA_PAIR && rows > BM
					  && n_raw % BN == 0 && scope.state().sm_count >= 2;
	CUresult e = make_map_2d(&ta, x, cfg->model_dim, rows, cfg->model_dim, BK, BM);
	if (e == CUDA_SUCCESS) e = make_map_2d(&tb, w_qkvg, cfg->model_dim, n_raw, cfg->model_dim, BK, pair ? BN / 2 : BN);
	if (e != CUDA_SUCCESS) {
		return make_diag("x17ai_b200: cuTensorMapEncodeTiled failed", who,
						 ": cuTensorMapEncodeTiled failed: ", x17::cu_error_text(e));
	}
	x17::GemmParams p{};
	p.m = uint32_t(rows);
	p.n_raw = uint32_t(n_raw);
	p.k = p.k_a = uint32_t(cfg->model_dim);
	p.tiles_m = uint32_t((rows + BM - 1) / BM);
	p.tiles_n = uint32_t((n_raw + BN - 1) / BN);
	p.c = q;
	p.c_stride = n_q;
	p.c2 = kv;
	p.c2_stride = n_kv;
	p.c3 = g;
	p.c3_stride = n_g;
	p.n_q = uint32_t(n_q);
	p.n_kv = uint32_t(n_kv);
	p.rrms = k_rrms;
	p.rrms_cols = uint32_t(cfg->n_heads);
	p.head_dim = uint32_t(cfg->head_dim);
	p.status = scope.state().status;
	p.k0 = float(cfg->eps);
	p.k1 = float(cfg->out_scale * std::sqrt(double(cfg->head_dim)));
	p.k2 = float(cfg->inp_scale * cfg->out_scale);
	p.k3 = float(cfg->inp_scale * cfg->out_scale);
	p.k4 = float(cfg->inp_scale * cfg->out_scale);
	uint32_t const n_tiles = p.tiles_m * p.tiles_n;
	uint32_t const ctas = n_tiles < uint32_t(scope.state().sm_count) ? n_tiles : uint32_t(scope.state().sm_count);
	cudaError_t const ce =
		pair ? gemm_go_pair<x17::EPI_QKVG>(false, scope.state().sm_count, reinterpret_cast<cudaStream_t>(stream), ta, tb, p)
			 : gemm_go<x17::EPI_QKVG>(false, dim3(ctas), reinterpret_cast<cudaStream_t>(stream), ta, tb, p);
	if (ce != cudaSuccess) {
		return make_diag("x17ai_b200: cudaFuncSetAttribute failed", who, ": cudaFuncSetAttribute failed: ",
						 cudaGetErrorString(ce));
	}
	return launch_result(who);
}

x17ai_DiagnosticBuffer *x17ai_b200_split_i8_weights(
	x17ai_CudaStreamHandle *stream, int8_t const *w, size_t rows, size_t cols, uint8_t *out) {
	char const *who = "x17ai_b200_split_i8_weights()";
	if (!w || !out || rows == 0 || cols == 0) return make_diag("x17ai_b200: bad argument", who, ": bad argument");
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	split_i8_weights_kernel<<<scope.state().sm_count * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
		w, rows, cols, out);
	return launch_result(who);
}

x17ai_DiagnosticBuffer *x17ai_b200_rms_norm(
	x17ai_CudaStreamHandle *stream, int32_t mode, void const *inp, size_t rows, size_t cols,
	int8_t *out, float *row_scale, double eps) {
	char const *who = "x17ai_b200_rms_norm()";
	if (mode < 0 || mode > 2) return make_diag("x17ai_b200: bad mode", who, ": unknown mode ", mode);
	if (rows == 0 || cols == 0) return make_diag("x17ai_b200: empty input", who, ": rms_norm input has zero size");
	size_t const vals = mode == X17AI_RMS_E4M3_FIXED ? 16 : 8;
	if (cols % 16 != 0 || cols / vals > size_t(x17::rms_cfg::MAX_CHUNKS) * 32) {
		return make_diag("x17ai_b200: bad rms_norm width", who, ": rms_norm requires cols to be a multiple of 16 and at most ",
						 vals * x17::rms_cfg::MAX_CHUNKS * 32, ", got ", cols);
	}
	if (rows >= (size_t(1) << 31)) return make_diag("x17ai_b200: rms_norm shape out of range", who, ": too many rows");
	if (!inp || !out || (mode == X17AI_RMS_BF16_ROWSCALE && !row_scale)) {
		return make_diag("x17ai_b200: null tensor", who, ": null tensor argument");
	}
	if (!aligned16(inp) || !aligned16(out)) {
		return make_diag("x17ai_b200: misaligned tensor", who, ": tensors must be 16-byte aligned");
	}
	StreamScope scope(stream, who);
	if (scope.diag) return scope.diag;
	x17::RmsParams p{};
	p.inp = inp;
	p.out = out;
	p.row_scale = row_scale;
	p.rows = uint32_t(rows);
	p.cols = uint32_t(cols);
	p.inp_stride = cols;
	p.out_stride = cols;
	p.eps = float(eps);
	p.inv_cols = float(1.0 / double(cols));
	dim3 grid(unsigned((rows + x17::rms_cfg::WARPS - 1) / x17::rms_cfg::WARPS));
	cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
	if (mode == X17AI_RMS_E4M3_FIXED) {
		if (cols <= size_t(x17::rms_cfg::KEEP_CHUNKS) * 32 * 16) {
			x17::rms_norm_keep_kernel<<<grid, x17::rms_cfg::THREADS, 0, s>>>(p);
		} else {
			x17::rms_norm_kernel<x17::RMS_E4M3_FIXED><<<grid, x17::rms_cfg::THREADS, 0, s>>>(p);
		}
	} else if (mode == X17AI_RMS_BF16_FIXED) {
		x17::rms_norm_kernel<x17::RMS_BF16_FIXED><<<grid, x17::rms_cfg::THREADS, 0, s>>>(p);
	} else {
		x17::rms_norm_kernel<x17::RMS_BF16_ROWSCALE><<<grid, x17::rms_cfg::THREADS, 0, s>>>(p);
	}
	return launch_result(who);
}

}  // extern "C"
