/*
 * C ABI of libx17ai_b200.so: the B200 (sm_100a) drop-in for the quantized block-forward
 * hot path of x17ai.
 *
 * Part 1 re-exports, with identical names, argument lists, struct layouts and ownership
 * rules, the 21 functions of the reference's driver shim (cpp/cuda_shim.cpp:189-988,
 * declared for the Rust host in src/device/cuda/cuda_shim.rs:76-158).
 *
 * Part 2 adds one entry point per hot-path kernel.  In the reference these kernels are
 * rendered from templates, compiled by nvcc at run time into one cubin per shape and
 * launched through x17ai_cuda_launch_kernel; here they are precompiled for sm_100a and
 * take their shapes and scales at run time, so the Rust launchers
 * (src/device/cuda/attn.rs, gemm.rs) call one function instead of render + nvcc + load +
 * launch.  Every entry point follows the shim's conventions: it returns a
 * DiagnosticBuffer* that is NULL on success and otherwise owned by the caller until it is
 * handed, once, to x17ai_move_diagnostic; all work is enqueued on the given stream and
 * nothing is synchronised; no CUDA context is left current on the calling thread.
 */
#ifndef X17AI_B200_H
#define X17AI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------
 * Part 1: the reference shim (cpp/ffi.hpp, cpp/cuda_shim.cpp)
 * ---------------------------------------------------------------------------------------- */

/* cpp/ffi.hpp:12-23; Rust side src/util/ffi_buffer.rs:14-103 */
typedef struct x17ai_FfiSpan {
	char *ptr;
	size_t len;
} x17ai_FfiSpan;

typedef struct x17ai_FfiBufferVMT {
	x17ai_FfiSpan (*span)(void *self);
	x17ai_FfiSpan (*buf_span)(void *self);
	x17ai_FfiSpan (*extend)(void *self, size_t additional);
	void (*clear)(void *self);
	void (*set_len)(void *self, size_t new_len);
} x17ai_FfiBufferVMT;

typedef struct x17ai_FfiBuffer {
	void *instance;
	x17ai_FfiBufferVMT const *vmt;
} x17ai_FfiBuffer;

/* cpp/ffi.hpp:84-93: opaque to the caller */
typedef struct x17ai_DiagnosticBuffer x17ai_DiagnosticBuffer;

/* cpp/cuda_shim.cpp:56-63; the Rust host reads only the first field (cuda_shim.rs:20-24) */
typedef struct x17ai_CudaContextHandle {
	size_t refcnt_munus_one;
	size_t device_id;
	size_t capability_major;
	size_t capability_minor;
	size_t warp_size;
	int device;    /* CUdevice */
	void *context; /* CUcontext */
} x17ai_CudaContextHandle;

typedef struct x17ai_CudaStreamHandle x17ai_CudaStreamHandle; /* is a CUstream   (cuda_shim.cpp:385) */
typedef struct x17ai_CudaModuleHandle x17ai_CudaModuleHandle; /* is a CUmodule   (cuda_shim.cpp:826) */
typedef struct x17ai_CudaKernelHandle x17ai_CudaKernelHandle; /* is a CUfunction (cuda_shim.cpp:903) */
typedef struct x17ai_CudaDeviceData x17ai_CudaDeviceData;     /* is a CUdeviceptr (cuda_shim.cpp:83-93) */
typedef struct x17ai_CudaTimerHandle x17ai_CudaTimerHandle;   /* cuda_shim.cpp:76-81 */

/* cpp/cuda_shim.cpp:64-74 */
typedef struct x17ai_CudaKernelAttrs {
	int32_t max_threads_per_block;
	int32_t static_shared_size_bytes;
	int32_t const_size_bytes;
	int32_t local_size_bytes;
	int32_t num_regs;
	int32_t ptx_version;
	int32_t binary_version;
	int32_t max_dynamic_shared_size_bytes;
	int32_t preferred_shared_memory_carveout;
} x17ai_CudaKernelAttrs;

/* PtrResult<T> (cpp/ffi.hpp:161-175): returned by value, two pointers */
#define X17AI_PTR_RESULT(T, NAME)            \
	typedef struct NAME {                    \
		T *value;                            \
		x17ai_DiagnosticBuffer *diagnostic;  \
	} NAME
X17AI_PTR_RESULT(x17ai_CudaContextHandle, x17ai_ContextResult);
X17AI_PTR_RESULT(x17ai_CudaStreamHandle, x17ai_StreamResult);
X17AI_PTR_RESULT(x17ai_CudaTimerHandle, x17ai_TimerResult);
X17AI_PTR_RESULT(x17ai_CudaDeviceData, x17ai_DeviceDataResult);
X17AI_PTR_RESULT(x17ai_CudaModuleHandle, x17ai_ModuleResult);
X17AI_PTR_RESULT(x17ai_CudaKernelHandle, x17ai_KernelResult);

/* cuda_shim.cpp:190-205 */
void x17ai_move_diagnostic(x17ai_DiagnosticBuffer *diag, x17ai_FfiBuffer err);
/* cuda_shim.cpp:207-317 */
x17ai_ContextResult x17ai_cuda_open_context(size_t device_id);
/* cuda_shim.cpp:319-341 */
x17ai_DiagnosticBuffer *x17ai_cuda_close_context(x17ai_CudaContextHandle *context);
/* cuda_shim.cpp:343-347 */
void *x17ai_cuda_context_ptr(x17ai_CudaContextHandle *context);
/* cuda_shim.cpp:349-387 */
x17ai_StreamResult x17ai_cuda_open_stream(x17ai_CudaContextHandle *ctx);
/* cuda_shim.cpp:389-408 */
x17ai_DiagnosticBuffer *x17ai_cuda_close_stream(x17ai_CudaStreamHandle *stream);
/* cuda_shim.cpp:410-430 */
x17ai_DiagnosticBuffer *x17ai_cuda_synchronize(x17ai_CudaStreamHandle *stream);
/* cuda_shim.cpp:432-503 */
x17ai_TimerResult x17ai_cuda_create_timer(x17ai_CudaContextHandle *context, x17ai_CudaStreamHandle *stream);
/* cuda_shim.cpp:505-562 */
x17ai_DiagnosticBuffer *x17ai_cuda_destroy_timer(x17ai_CudaTimerHandle *timer);
/* cuda_shim.cpp:564-581 */
x17ai_DiagnosticBuffer *x17ai_cuda_timer_start(x17ai_CudaTimerHandle *timer);
/* cuda_shim.cpp:583-600 */
x17ai_DiagnosticBuffer *x17ai_cuda_timer_stop(x17ai_CudaTimerHandle *timer);
/* cuda_shim.cpp:602-652 */
x17ai_DiagnosticBuffer *x17ai_cuda_timer_elapsed_seconds(x17ai_CudaTimerHandle *timer, double *seconds);
/* cuda_shim.cpp:654-679 */
x17ai_DeviceDataResult x17ai_cuda_alloc(x17ai_CudaStreamHandle *stream, size_t bytes);
/* cuda_shim.cpp:681-700 */
x17ai_DiagnosticBuffer *x17ai_cuda_free(x17ai_CudaStreamHandle *stream, x17ai_CudaDeviceData *ptr);
/* cuda_shim.cpp:702-733 */
x17ai_DiagnosticBuffer *x17ai_cuda_upload_data(x17ai_CudaStreamHandle *stream, uint8_t const *src,
											   x17ai_CudaDeviceData *dst, size_t offset_bytes, size_t size_bytes);
/* cuda_shim.cpp:735-766 */
x17ai_DiagnosticBuffer *x17ai_cuda_download_data(x17ai_CudaStreamHandle *stream, x17ai_CudaDeviceData *src,
												 uint8_t *dst, size_t offset_bytes, size_t size_bytes);
/* cuda_shim.cpp:768-828 */
x17ai_ModuleResult x17ai_cuda_load_module(x17ai_CudaContextHandle *ctx, char const *cubin_path);
/* cuda_shim.cpp:830-846 */
x17ai_DiagnosticBuffer *x17ai_cuda_del_module(x17ai_CudaModuleHandle *module);
/* cuda_shim.cpp:848-905 */
x17ai_KernelResult x17ai_cuda_get_kernel(x17ai_CudaModuleHandle *module, char const *name, size_t smem_size);
/* cuda_shim.cpp:907-927 */
x17ai_DiagnosticBuffer *x17ai_cuda_read_kernel_attrs(x17ai_CudaKernelHandle *kernel, x17ai_CudaKernelAttrs *attrs);
/* cuda_shim.cpp:929-987 */
x17ai_DiagnosticBuffer *x17ai_cuda_launch_kernel(x17ai_CudaStreamHandle *stream, x17ai_CudaKernelHandle *kernel,
												 size_t grid_x, size_t grid_y, size_t grid_z,
												 size_t block_x, size_t block_y, size_t block_z,
												 size_t shared_mem_bytes, void **args);

/* ------------------------------------------------------------------------------------------
 * Part 2: hot-path kernels
 * ---------------------------------------------------------------------------------------- */

/* DType codes of the Rust host (src/dtype.rs:3-8) */
enum {
	X17AI_DTYPE_E4M3 = 0x30,
	X17AI_DTYPE_INT8 = 0x31,
	X17AI_DTYPE_BF16 = 0x40,
	X17AI_DTYPE_F32 = 0x50,
	X17AI_DTYPE_I32_RAW = 0x51 /* validation only: raw 32-bit accumulators as GEMM output */
};

/* AttnKernelConfig (src/device/cuda/attn.rs:45-53); dtype is always Int8.
 * Strides are in elements (bytes) per sequence position. */
typedef struct x17ai_AttnConfig {
	size_t n_heads;
	size_t head_dim; /* 32, 64 or 128 */
	size_t q_stride;
	size_t kv_stride;
	size_t o_stride;
} x17ai_AttnConfig;

/* Launch metadata the reference reads from meta.json (attn.rs:311-316) */
typedef struct x17ai_AttnMeta {
	size_t threads_per_block;
	size_t smem_bytes;
	size_t q_per_block;
} x17ai_AttnMeta;

x17ai_DiagnosticBuffer *x17ai_b200_attn_meta(x17ai_AttnConfig const *cfg, x17ai_AttnMeta *meta);

/*
 * int8 sliding-window attention forward.  Replaces AttnKernel::launch
 * (src/device/cuda/attn.rs:353-447) and the kernel it launches
 * (templates/attn/kernel.cu:9-33 -> AttnForward::run, cuda/attn_fwd_i8.cuh:368-619).
 *   q   [batch][seq_len][q_stride]  int8 FixedI8, head h at columns h*D .. h*D+D-1
 *   kv  [batch][seq_len][kv_stride] int8, head h at columns 2*h*D: [K(D) | V(D)]
 *   sink_k, sink_v [n_heads][D] int8;  attn_temperature [n_heads] f32
 *   out [batch][seq_len][o_stride] int8;  l [batch][n_heads][seq_len] f32 or NULL
 *   window_size: 0 = unbounded, else a multiple of 16 (attn.rs:405-410)
 * batch = 1 is the reference's call; batch > 1 runs independent sequences laid out back to
 * back in one launch.  seq_len need not be a multiple of the query tile.
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size);

/*
 * The same attention with P.V on the fp8 tensor path and bf16 output.  The reference file of this name
 * (attn_y_fwd_fp8.cu:11-47) is a bf16 GEMM of the attention output projection; the kernel described for
 * the benchmark - softmax probabilities quantised to e4m3, V in e4m3 with a per-head f32 scale - has no
 * counterpart in the reference.  Q.K^T, masks, sink, temperature, maximum and normaliser are those of
 * x17ai_b200_attn_fwd_i8; P = e4m3(256 * 2^(s - max)) (OCP e4m3, round to nearest even), O accumulates in
 * f32, out = bf16(O / sum * v_scale[h]), L = log2(256 * sum) + max.
 *   kv: K half int8 FixedI8 as before, V half OCP e4m3 bytes; sink_v [n_heads][D] e4m3 (same scale);
 *   v_scale f32 [n_heads]; out bf16 [batch][seq_len][o_stride] (o_stride in elements).
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_pv_fp8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, uint8_t const *kv, int8_t const *sink_k, uint8_t const *sink_v,
	float const *attn_temperature, float const *v_scale, uint16_t *out_bf16, float *l, size_t window_size);

/*
 * x17ai_b200_attn_fwd_i8 whose epilogue also stores the output into `n_peers` (at most 7) more buffers with the
 * layout of `out`: peer-mapped addresses of other GPUs' memory (CUDA IPC, cuMemMap or symmetric-memory pointers
 * valid in this process), written with plain 16-byte stores over NVLink as each row is finished.  One process per
 * GPU runs its shard of the batch (x17ai_b200/sharding.py) with `out` = its slot of its own gathered buffer and
 * `peer_out[i]` = the same slot of peer i's: when every rank's launch has completed, every GPU holds every shard,
 * and no all-gather pass follows.  The caller orders "all launches completed" before the buffers are read (a
 * barrier between the ranks on the stream); nothing in the kernel waits on another GPU.  Always the
 * one-CTA-per-query-tile kernel.
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_to_peers(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, int8_t *const *peer_out,
	size_t n_peers);

/*
 * The int8 attention for inputs quantised with one symmetric f32 scale per token and head (value = scale * code,
 * scale = absmax / 127: the input format of the benchmark description) and bf16 output.  No counterpart in the
 * reference, whose tensors carry one global FixedI8 scale (cuda/utils_b8.cuh:7-10, 629-632) and whose kernel writes
 * FixedI8 (cuda/attn_fwd_i8.cuh:293-351); masks, sink token, temperature, maximum and normaliser are those of
 * x17ai_b200_attn_fwd_i8, which this call equals for q_scale = k_scale = v_scale = 1/8 up to the output format
 * (out = code / 8).  Q.K^T and P.V stay exact integer products on the int8 tensor path:
 *   x[i][j] = (q_i . k_j)_int32 * q_scale[i] * k_scale[j] * D^-1/2 * log2(min(W', i) + 4) * temp_h
 *   P[i][j] = rint(255 * 2^(x - m_i) * v_scale[j] / g_i),  g_i = the largest v_scale[j] among the keys row i sees  (u8)
 *   out[i]  = bf16((g_i / 255 * sum_j P[i][j] v_j + 2^(sink - m_i) * sink_v / 8) / sum_i),  sum_i as before
 *   q_scale, k_scale, v_scale: f32 [batch][n_heads][seq_len];  sink_k, sink_v FixedI8 as before;
 *   out bf16 [batch][seq_len][o_stride] (o_stride in elements);  l [batch][n_heads][seq_len] or NULL.
 * Always the one-CTA-per-query-tile kernel.
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_scaled(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, float const *q_scale, int8_t const *kv, float const *k_scale, float const *v_scale,
	int8_t const *sink_k, int8_t const *sink_v, float const *attn_temperature, uint16_t *out_bf16, float *l,
	size_t window_size);

/*
 * Which kernel the three attention entry points above and below launch.  No counterpart in the
 * reference (its one kernel, cuda/attn_fwd_i8.cuh:368-619, runs one CTA per 64 queries and head group):
 *   X17AI_B200_ATTN_PER_TILE (default, the faster one on configs[1]): one CTA per 128-query tile, two
 *     CTAs per SM (the kernel the kernel objects embed); tiles_per_item is ignored.
 *   X17AI_B200_ATTN_PERSISTENT: one CTA per SM walks runs of `tiles_per_item` consecutive 128-query
 *     tiles of one (batch, head); probabilities stay in tensor memory (P.V takes its A operand from
 *     there) and the maximum sweep of the next query tile runs inside the probability sweep of the
 *     current one.  tiles_per_item = 0 lets every launch choose (16, halved down to 4 while fewer than
 *     two items per SM come out).
 * Both give the same scores, probabilities and int32 accumulators; the normaliser is summed in a
 * different order and the final rounding differs in its last step, so codes may differ by one step in
 * rare cases.  Process-wide; returns 0, or -1 for an unknown schedule.
 */
enum { X17AI_B200_ATTN_PERSISTENT = 0, X17AI_B200_ATTN_PER_TILE = 1 };
int x17ai_b200_set_attn_schedule(int schedule, unsigned tiles_per_item);

/* Tiling of x17ai_b200_gemm_fwd and x17ai_b200_qkvg_fwd_i8:
 *   X17AI_B200_GEMM_CTA_PAIR (default): clusters of two CTAs on two SMs, 256 x 256 tiles
 *     (tcgen05.mma.cta_group::2): every CTA loads its 128 rows of A and half of the tile's rows of B, a third fewer
 *     bytes per MMA through L2 and shared memory, six ring stages instead of four. Taken for inputs of more than
 *     128 rows whose N is a multiple of 256; other shapes run the one-CTA form.
 *   X17AI_B200_GEMM_ONE_CTA: one CTA per SM, 128 x 256 tiles (tcgen05.mma.cta_group::1), the form the kernel
 *     objects embed (the reference's launch path has no clusters).
 * The same bytes out. Process-wide; returns 0, or -1 for an unknown value. */
enum { X17AI_B200_GEMM_ONE_CTA = 0, X17AI_B200_GEMM_CTA_PAIR = 1 };
int x17ai_b200_set_gemm_tiling(int tiling);

/* Same launch with validation outputs: dbg_s int32 [batch*n_heads][seq][seq] raw scores of the
 * visited tiles, dbg_p uint8 [batch*n_heads][seq][seq] quantised probabilities, dbg_o int32
 * [batch*n_heads][seq][D] the int32 P.V accumulator.  Small shapes only. */
x17ai_DiagnosticBuffer *x17ai_b200_attn_fwd_i8_debug(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch, size_t seq_len,
	int8_t const *q, int8_t const *kv, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size,
	int32_t *dbg_s, uint8_t *dbg_p, int32_t *dbg_o);

/*
 * int8 decode attention: one new token per sequence at position kv_len against an int8 KV
 * cache.  The reference names attn_incremental (attn_incremental.cu:329-481) but ships no
 * int8 decode; semantics are those of row kv_len of x17ai_b200_attn_fwd_i8.
 *   q [batch][q_stride]; kv_cache [batch][kv_capacity][kv_stride]; kv_lens [batch] or NULL
 *   (then every sequence has kv_len cached tokens); out [batch][o_stride]; l [batch][n_heads]
 *   or NULL.
 * When batch*n_heads is too small to fill the GPU the keys are split over several CTAs and
 * the partial results pass through stream-ordered scratch memory that this call allocates
 * and frees (cudaMallocAsync / cudaFreeAsync on `stream`).
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_decode_i8(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch,
	int8_t const *q, int8_t const *kv_cache, size_t kv_capacity, size_t kv_len,
	uint32_t const *kv_lens, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, size_t n_splits);

/*
 * The same decode attention for callers that must not allocate: no counterpart in the
 * reference. Some hosts of this library run where device memory cannot be allocated at call
 * time: inside a serving loop whose memory was carved up front and handed out by the host's own
 * allocator, under a CUDA memory pool that is exhausted or disabled, or in a process whose
 * policy forbids cudaMalloc / cudaMallocAsync after start-up. For them the split-KV partials
 * go to a 4 MiB array built into the library image (every GPU that loads the library holds it
 * until the process exits) instead of stream-ordered scratch.
 *   - Arguments and results are those of x17ai_b200_attn_decode_i8.
 *   - Limit: batch * n_heads * n_splits * (head_dim + 2) <= 1,048,576 floats; larger requests are
 *     rejected with a diagnostic (pass a smaller n_splits, or use the allocating entry point).
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress
 *     with that device current); make that first call before any stream capture.
 *   - All calls share the one array: two calls whose kernels may overlap on the GPU (different
 *     streams, or different threads) race on it. Calls on one stream are safe: each call
 *     overwrites every slot it later reads, so nothing has to be cleared between calls.
 *   - It calls no cudaMalloc, cudaFree, cudaMallocAsync or other allocating routine.
 */
x17ai_DiagnosticBuffer *x17ai_b200_attn_decode_i8_noalloc(
	x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg, size_t batch,
	int8_t const *q, int8_t const *kv_cache, size_t kv_capacity, size_t kv_len,
	uint32_t const *kv_lens, int8_t const *sink_k, int8_t const *sink_v,
	float const *attn_temperature, int8_t *out, float *l, size_t window_size, size_t n_splits);

/* Epilogues of the GEMM (src/device/cuda/gemm.rs: ScaleEpilogue :60-110, RMSNormEpilogue
 * :112-166, ResidualEpilogue :168-212, GeGluEpilogue :214-255) */
enum {
	X17AI_EPILOGUE_SCALE = 0,
	X17AI_EPILOGUE_RMS_NORM = 1,
	X17AI_EPILOGUE_GEGLU = 2,
	X17AI_EPILOGUE_RESIDUAL = 3
};

/* GemmConfig + epilogue config (gemm.rs:257-366).  B is always given transposed, i.e. as
 * [b_rows][a_cols] row-major (gemm.rs:462-467). */
typedef struct x17ai_GemmConfig {
	int32_t a_dtype; /* INT8 or E4M3 */
	int32_t b_dtype; /* INT8, or E4M3 (standard OCP e4m3 x e4m3 tensor-core mode) */
	int32_t c_dtype; /* INT8 or E4M3 (or I32_RAW with the SCALE epilogue) */
	int32_t epilogue;
	size_t a_cols;   /* K */
	size_t b_rows;   /* N_raw */
	double inp_scale;
	double out_scale;
	double eps;      /* RMS_NORM */
	size_t head_dim; /* RMS_NORM: raw columns per head are [K(head_dim) | V(head_dim)] */
} x17ai_GemmConfig;

/* Launch metadata the reference reads from meta.json (gemm.rs:531-537) */
typedef struct x17ai_GemmMeta {
	size_t threads_per_block;
	size_t smem_bytes;
	size_t m_per_block;
	size_t n_per_block;
} x17ai_GemmMeta;

x17ai_DiagnosticBuffer *x17ai_b200_gemm_meta(x17ai_GemmConfig const *cfg, x17ai_GemmMeta *meta);

/*
 * Fused GEMM.  Replaces GemmKernel<E>::launch (gemm.rs:439-443, 591-641) and the kernels
 * rendered from templates/basic_gemm/kernel.cu:9-32 (b8::Gemm, cuda/gemm_b8.cuh:666-754;
 * b16::Gemm, cuda/gemm_b16.cuh:478-566).
 *   a [a_rows][a_cols]; b [b_rows][a_cols]; c [a_rows][b_rows] (SCALE, RMS_NORM) or
 *   [a_rows][b_rows/2] (GEGLU, RESIDUAL); rrms f32 [a_rows][b_rows / (2*head_dim)] (RMS_NORM);
 *   residual int8 [a_rows][b_rows/2] (RESIDUAL).
 * a_dtype E4M3 with b_dtype INT8 (the reference's ffn_y_fwd_f8) needs b in the split form
 * produced by x17ai_b200_split_i8_weights: pass that buffer as b.
 */
x17ai_DiagnosticBuffer *x17ai_b200_gemm_fwd(
	x17ai_CudaStreamHandle *stream, x17ai_GemmConfig const *cfg,
	void const *a, size_t a_rows, void const *b, size_t b_rows,
	void *c, float *rrms, int8_t const *residual);

/* Fused Q / KV / gate projection of one token block: one GEMM over the row-concatenated weights
 * [W_q (H*D rows) ; W_kv (H*2*D rows, per head K then V) ; W_g (gate_cols rows)], each column
 * segment with its own epilogue, so x is read once.  Replaces the two launches attn_q_fwd and
 * attn_kv_fwd of the reference (src/main.rs:387-491; the stale single-kernel form is
 * cuda/qkvg_fwd_i8.cuh:145-219): q = fixedi8(acc * inp * out) (ScaledMatrixWriter), k/v and k_rrms as
 * the RMS_NORM epilogue (L2NormMatrixWriter), g = fixedi8(acc * inp * out) raw gate columns. */
typedef struct x17ai_QkvgConfig {
	size_t model_dim; /* K */
	size_t n_heads;
	size_t head_dim;  /* 32, 64 or 128; n_heads * head_dim a multiple of 256 */
	size_t gate_cols; /* 0 = no gate segment; else a multiple of 128 */
	double inp_scale; /* main.rs:412-421: model_dim^-1/2 / 64 */
	double out_scale; /* 8 */
	double eps;       /* 2^-70 */
} x17ai_QkvgConfig;

/* x [rows][model_dim]; w_qkvg [H*D + 2*H*D + gate_cols][model_dim]; q [rows][H*D]; kv [rows][2*H*D];
 * k_rrms f32 [rows][H]; g [rows][gate_cols] or NULL when gate_cols is 0. */
x17ai_DiagnosticBuffer *x17ai_b200_qkvg_fwd_i8(
	x17ai_CudaStreamHandle *stream, x17ai_QkvgConfig const *cfg, int8_t const *x, size_t rows,
	int8_t const *w_qkvg, int8_t *q, int8_t *kv, float *k_rrms, int8_t *g);

/* One-time weight preparation for e4m3 activations x int8 weights: writes
 * out[rows][2*cols] e4m3 = [16*hi | lo] with w = 16*hi + lo, hi in [-8, 8], lo in [0, 15],
 * both exactly representable in e4m3, so that A.[16*hi|lo]^T with A repeated along K equals
 * A.W^T exactly term by term. */
x17ai_DiagnosticBuffer *x17ai_b200_split_i8_weights(
	x17ai_CudaStreamHandle *stream, int8_t const *w, size_t rows, size_t cols, uint8_t *out);

/* RMSNorm modes */
enum {
	X17AI_RMS_E4M3_FIXED = 0,   /* e4m3 in, FixedI8 out: Rms_norm::kernel (rms_norm.cu:55-113) */
	X17AI_RMS_BF16_FIXED = 1,   /* bf16 in, FixedI8 out */
	X17AI_RMS_BF16_ROWSCALE = 2 /* bf16 in, int8 out + f32 per-row absmax/127 scale */
};

/* Replaces Rms_norm::kernel (rms_norm.cu:55-113): inp [rows][cols] -> out int8 [rows][cols]. */
x17ai_DiagnosticBuffer *x17ai_b200_rms_norm(
	x17ai_CudaStreamHandle *stream, int32_t mode, void const *inp, size_t rows, size_t cols,
	int8_t *out, float *row_scale, double eps);

/* What a builder of a GEMM kernel object (kernel.cubin + meta.json in the reference's form,
 * templates/basic_gemm/kernel.cu:9-16, kernel_build.rs:38-134) needs for one configuration: the
 * epilogue constants as this library computes them, the launch metadata, and templates of the two
 * TMA tensor maps (shape, strides, box, swizzle final; base address and A's row count are patched
 * by the kernel object on the device at launch). int8 x int8 configurations only. */
typedef struct x17ai_GemmObjectDesc {
	int32_t epilogue_kind;
	uint32_t n_raw, k, head_dim, rrms_cols;
	uint64_t c_stride, resid_stride;
	float k0, k1, k2, k3, k4;
	uint32_t smem_bytes, threads, m_per_block, n_per_block;
	uint32_t k_a;      /* e4m3 x int8 objects: K of the activations (k is then 2 * k_a: two weight planes); else 0 */
	uint32_t reserved;
	uint8_t map_a[128], map_b[128];
} x17ai_GemmObjectDesc;
x17ai_DiagnosticBuffer *x17ai_b200_gemm_object_desc(x17ai_CudaStreamHandle *stream, x17ai_GemmConfig const *cfg,
                                                    x17ai_GemmObjectDesc *desc);

/* The same for the attention kernel object (templates/attn/kernel.cu:9-20, attn.rs:336-447): launch
 * metadata and templates of the Q and KV tensor maps for one configuration; the kernel object writes
 * the base addresses and the sequence length on the device and, under the reference's grid of one CTA
 * per 128 / head_dim heads, goes through the heads of its group one after the other. */
typedef struct x17ai_AttnObjectDesc {
	uint32_t smem_bytes, threads, q_per_block, reserved;
	uint8_t map_q[128], map_kv[128];
} x17ai_AttnObjectDesc;
x17ai_DiagnosticBuffer *x17ai_b200_attn_object_desc(x17ai_CudaStreamHandle *stream, x17ai_AttnConfig const *cfg,
                                                    x17ai_AttnObjectDesc *desc);

/* The four status words of a kernel object (a module loaded with x17ai_cuda_load_module whose cubin exports
 * `x17_status`): synchronises the stream, copies them (0 = ok; else code << 16 | detail of the first bounded wait
 * that ran out, or code 15 = an e4m3 x int8 GEMM object launched before its `prepare` entry point ran for the
 * weights it was given; the reporting block; the number of reports; reserved) and clears them. The reference's
 * kernels report nothing (cpp/cuda_shim.cpp:929-987 only reports launch failures); no counterpart there. */
x17ai_DiagnosticBuffer *x17ai_b200_object_status(x17ai_CudaStreamHandle *stream, x17ai_CudaModuleHandle *module,
                                                 uint32_t status[4]);

/* Device-side status of the kernels launched so far on the stream's device: synchronises the
 * stream, copies the four status words (0 = ok; else code << 16 | detail of the first bounded
 * wait that ran out, the reporting block, the number of reports, reserved) and clears them. */
x17ai_DiagnosticBuffer *x17ai_b200_read_status(x17ai_CudaStreamHandle *stream, uint32_t status[4]);

/* For hosts that cannot build the FfiBuffer callback table (its callbacks return a struct by
 * value): moves the diagnostic into dst (at most cap bytes, no terminator) through
 * x17ai_move_diagnostic and a fixed-capacity FfiBuffer, releases it, and returns the number of
 * bytes written.  diag may be NULL (returns 0). */
size_t x17ai_b200_take_diagnostic(x17ai_DiagnosticBuffer *diag, char *dst, size_t cap);

/* Stream capture. The reference's host issues the block's launches one by one (src/main.rs:193-255)
 * and has no graph object; a host that replays the same launches many times (the same buffers,
 * new contents) records them once between graph_begin and graph_end and replays them with
 * graph_launch, one driver call per block instead of six.
 *   - Between begin and end only this library's launch entry points and x17ai_cuda_upload_data /
 *     x17ai_cuda_download_data on page-locked memory may be called on the stream; anything that
 *     synchronises (x17ai_cuda_synchronize, read_status, timers' elapsed time) invalidates the
 *     capture and graph_end then returns a diagnostic.
 *   - Every kernel of the sequence must have been launched once on the device before begin (the
 *     first launch of an entry point sets function attributes and per-device state).
 *   - The graph holds the pointers and sizes of the recorded calls, not the data.
 *   - graph_destroy and graph_launch take the stream to enter its context. */
typedef struct x17ai_b200_Graph x17ai_b200_Graph;
x17ai_DiagnosticBuffer *x17ai_b200_graph_begin(x17ai_CudaStreamHandle *stream);
x17ai_DiagnosticBuffer *x17ai_b200_graph_end(x17ai_CudaStreamHandle *stream, x17ai_b200_Graph **graph);
x17ai_DiagnosticBuffer *x17ai_b200_graph_launch(x17ai_b200_Graph *graph, x17ai_CudaStreamHandle *stream);
x17ai_DiagnosticBuffer *x17ai_b200_graph_destroy(x17ai_b200_Graph *graph, x17ai_CudaStreamHandle *stream);
/* Kernel launches one replay of the graph performs (added to x17ai_b200_launch_count per replay). */
uint64_t x17ai_b200_graph_kernel_nodes(x17ai_b200_Graph const *graph);

/* Number of kernel launches this library has issued since it was loaded (all entry points). */
uint64_t x17ai_b200_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* X17AI_B200_H */
