// GEMM kernel object in the reference's form (templates/basic_gemm/kernel.cu:9-16): a cubin that exports
//   extern "C" kernel(A *a, usize a_rows, B *b, usize b_rows, C *c [, f32 *rrms] [, i8 *residual])
// with the shape and the epilogue constants fixed at compile time, loaded with x17ai_cuda_load_module /
// x17ai_cuda_get_kernel and launched by the reference's host with its own grid
// (c_rows / M_PER_BLOCK, raw_cols / N_PER_BLOCK, 1), gemm.rs:591-641.
//
// The tcgen05 GEMM reads its operands through TMA tensor maps, which only the driver can encode and
// which the reference's argument list has no room for. The builder therefore bakes templates of the two
// maps into this file (X17_MAP_A / X17_MAP_B: shape, strides, box and swizzle final) and every CTA
// finishes them on the device: it copies the templates to shared memory, writes the base addresses it
// was given and A's row count with tensormap.replace, publishes them to a slot in global memory owned by
// its SM (one CTA per SM: the kernel's shared memory does not leave room for two) and acquires them for
// the TMA unit.
//
// The e4m3 x int8 GEMM (the reference's ffn_y_fwd_f8, which converts both operands to bf16 in registers,
// gemm_b16.cuh:72-185) runs here on the fp8 tensor path over two e4m3 planes of the int8 weights,
// w = 16 * hi + lo. The reference's host holds only the int8 weights, so such an object (X17_SPLIT = 1)
// owns a buffer for the planes and exports a second entry point,
//   extern "C" prepare(i8 const *b, usize b_rows)
// which the host launches once per weight tensor (weights are constants of the model) with any grid; `kernel`
// then takes the reference's argument list unchanged and refuses, through the status words, a `b` it was not
// prepared for.
//
// `x17_status` (four words, all zero = no bounded wait ran out and no refusal) can be read by the host
// with cuModuleGetGlobal: x17ai_b200_object_status does that.
//
// Compile with -DX17_EPI=<epilogue id> -DX17_N_RAW= -DX17_K= -DX17_HEAD_DIM= -DX17_RRMS_COLS= -DX17_C_STRIDE=
// -DX17_RESID_STRIDE= -DX17_K0..X17_K4=<float bit patterns> [-DX17_SPLIT=1 -DX17_K_A=] and -include a header
// defining X17_MAP_A, X17_MAP_B.
#include "../gemm.cuh"

#ifndef X17_SPLIT
#define X17_SPLIT 0
#endif

namespace {

struct alignas(128) MapBytes {
	unsigned char b[128];
};

__constant__ MapBytes c_map_a = {{X17_MAP_A}};
__constant__ MapBytes c_map_b = {{X17_MAP_B}};
__device__ MapBytes g_maps[256][2];   // slot per SM
#if X17_SPLIT
// [X17_N_RAW][X17_K] e4m3, X17_K = 2 * X17_K_A: per row the hi plane (16 * hi) then the lo plane
__device__ __align__(128) unsigned char g_planes[size_t(X17_N_RAW) * X17_K];
__device__ unsigned long long g_planes_of;   // the weight tensor the planes were made from
#endif

__device__ __forceinline__ void map_set_address(unsigned smem_map, void const *ptr) {
	asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"l"(
					 static_cast<unsigned long long>(smem_map)),
				 "l"(ptr)
				 : "memory");
}
__device__ __forceinline__ void map_set_rows(unsigned smem_map, unsigned rows) {
	asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"l"(
					 static_cast<unsigned long long>(smem_map)),
				 "r"(rows)
				 : "memory");
}

}  // namespace

extern "C" {
__device__ unsigned x17_status[4];   // read by the host through cuModuleGetGlobal
}

#if X17_SPLIT
extern "C" __global__ void prepare(signed char const *b, unsigned long long b_rows) {
	(void)b_rows;
	unsigned long long const n = (unsigned long long)(X17_N_RAW) * X17_K_A;
	unsigned long long const stride = (unsigned long long)(gridDim.x) * blockDim.x;
	for (unsigned long long i = blockIdx.x * (unsigned long long)(blockDim.x) + threadIdx.x; i < n; i += stride) {
		unsigned long long const r = i / X17_K_A, c = i % X17_K_A;
		int const v = b[i];
		int const hi = (v + 128) / 16 - 8;  // floor(v / 16)
		int const lo = v - 16 * hi;         // 0 .. 15
		// OCP e4m3 encodings of the integers 16 * hi (multiples of 16 up to +-128) and lo, both exact
		auto enc = [](int x) -> unsigned char {
			if (x == 0) return 0;
			unsigned const s = x < 0 ? 0x80u : 0u;
			unsigned const a = unsigned(x < 0 ? -x : x);
			int const e = 31 - __clz(int(a));
			unsigned const mant = e >= 3 ? (a >> (e - 3)) & 7u : (a << (3 - e)) & 7u;
			return (unsigned char)(s | (unsigned(e + 7) << 3) | mant);
		};
		g_planes[r * X17_K + c] = enc(16 * hi);
		g_planes[r * X17_K + X17_K_A + c] = enc(lo);
	}
	if (blockIdx.x == 0 && threadIdx.x == 0) g_planes_of = reinterpret_cast<unsigned long long>(b);
}
#endif

extern "C" __global__ void __launch_bounds__(x17::gemm_cfg::THREADS, 1)
kernel(void const *a, unsigned long long a_rows, void const *b, unsigned long long b_rows, void *c
#if X17_EPI == 1
	   , float *rrms
#endif
#if X17_EPI == 3 || X17_EPI == 4
	   , signed char const *residual
#endif
) {
	using namespace x17;
	(void)b_rows;   // fixed at compile time (X17_N_RAW), as in the reference's templates
	__shared__ MapBytes s_maps[2];
#if X17_SPLIT
	if (g_planes_of != reinterpret_cast<unsigned long long>(b)) {
		// `prepare` has not run for these weights: nothing is computed, the host finds the reason in the status
		if (threadIdx.x == 0) report_status(x17_status, x17::ST_NOT_PREPARED, 1u);
		return;
	}
	b = g_planes;
#endif

	// The reference's grid has one CTA per output tile. One CTA per SM works through the tiles (the loop
	// overlaps the epilogue of a tile with the main loop of the next); the CTAs beyond that leave at once.
	u32 cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
	u32 n_ctas = gridDim.x * gridDim.y * gridDim.z;
	unsigned n_sm;
	asm volatile("mov.u32 %0, %%nsmid;" : "=r"(n_sm));
	if (n_ctas > n_sm) {
		if (cta >= n_sm) return;
		n_ctas = n_sm;
	}

	unsigned smid;
	asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
	MapBytes *const slot = g_maps[smid & 255u];

	if (threadIdx.x < 32) {
		// templates -> shared memory (16 bytes per lane), patch, publish to this SM's slot
		unsigned const lane = threadIdx.x;
		uint4 const *src = reinterpret_cast<uint4 const *>(lane < 8 ? c_map_a.b : c_map_b.b) + (lane & 7u);
		if (lane < 16) reinterpret_cast<uint4 *>(s_maps[lane >> 3].b)[lane & 7u] = *src;
		__syncwarp();
		if (lane == 0) {
			unsigned const ma = smem_u32(s_maps[0].b), mb = smem_u32(s_maps[1].b);
			map_set_address(ma, a);
			map_set_rows(ma, static_cast<unsigned>(a_rows));
			map_set_address(mb, b);
		}
		__syncwarp();
		for (unsigned i = 0; i < 2; ++i) {
			asm volatile(
				"tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
				::"l"(reinterpret_cast<unsigned long long>(slot[i].b)), "r"(smem_u32(s_maps[i].b))
				: "memory");
		}
		for (unsigned i = 0; i < 2; ++i) {
			asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(
							 reinterpret_cast<unsigned long long>(slot[i].b))
						 : "memory");
		}
	}
	__syncthreads();

	GemmParams p{};
	p.m = static_cast<u32>(a_rows);
	p.n_raw = X17_N_RAW;
	p.k = X17_K;
#if X17_SPLIT
	p.k_a = X17_K_A;
#else
	p.k_a = X17_K;
#endif
	p.tiles_m = (p.m + gemm_cfg::BM - 1) / gemm_cfg::BM;
	p.tiles_n = (X17_N_RAW + gemm_cfg::BN - 1) / gemm_cfg::BN;
	p.c = c;
	p.c_stride = X17_C_STRIDE;
	p.resid_stride = X17_RESID_STRIDE;
	p.head_dim = X17_HEAD_DIM;
	p.rrms_cols = X17_RRMS_COLS;
	p.k0 = __uint_as_float(X17_K0);
	p.k1 = __uint_as_float(X17_K1);
	p.k2 = __uint_as_float(X17_K2);
	p.k3 = __uint_as_float(X17_K3);
	p.k4 = __uint_as_float(X17_K4);
	p.status = x17_status;
#if X17_EPI == 1
	p.rrms = rrms;
#endif
#if X17_EPI == 3 || X17_EPI == 4
	p.residual = residual;
#endif
	gemm_body<X17_EPI, X17_SPLIT != 0>(reinterpret_cast<CUtensorMap const *>(slot[0].b),
							  reinterpret_cast<CUtensorMap const *>(slot[1].b), p, cta, n_ctas);
}
