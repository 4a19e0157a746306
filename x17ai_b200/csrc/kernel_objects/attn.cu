// Attention kernel object in the reference's form (templates/attn/kernel.cu:9-20): a cubin that exports
//   extern "C" kernel(usize seq_len, i8 *q, i8 *kv, const i8 *sink_k, const i8 *sink_v,
//                     const f32 *attn_temperature, i8 *out, f32 *l /*nullable*/, usize window_size)
// with heads, head_dim and the row strides fixed at compile time, launched by the reference's host with
// its own grid (seq_len / Q_PER_BLOCK, n_heads / max(128 / head_dim, 1), 1), attn.rs:425-447: one CTA per
// query tile and group of 128 / head_dim heads. This kernel works on one head at a time, so a CTA
// goes through the heads of its group one after the other.
//
// As in kernel_objects/gemm.cu the two TMA tensor maps are baked in as templates (X17_MAP_Q, X17_MAP_KV)
// and finished on the device: base addresses and the sequence length are written with tensormap.replace
// and the maps are published to a slot in global memory. Two CTAs share an SM, so each SM owns a small
// ring of slots handed out by a counter; every CTA of a launch writes the same bytes.
//
// Compile with -DX17_HEAD_DIM= -DX17_N_HEADS= -DX17_Q_STRIDE= -DX17_KV_STRIDE= -DX17_O_STRIDE= and -include a header
// defining X17_MAP_Q and X17_MAP_KV.
#include "../attn.cuh"

namespace {

struct alignas(128) MapBytes {
	unsigned char b[128];
};

constexpr unsigned SLOTS_PER_SM = 16;
__constant__ MapBytes c_map_q = {{X17_MAP_Q}};
__constant__ MapBytes c_map_kv = {{X17_MAP_KV}};
__device__ MapBytes g_maps[256][SLOTS_PER_SM][2];
__device__ unsigned g_next[256];


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

extern "C" __global__ void __launch_bounds__(x17::attn_cfg::THREADS, 2)
kernel(unsigned long long seq_len, signed char const *q, signed char const *kv, signed char const *sink_k,
	   signed char const *sink_v, float const *attn_temperature, signed char *out, float *l,
	   unsigned long long window_size) {
	using namespace x17;
	__shared__ MapBytes s_maps[2];
	__shared__ unsigned s_slot;

	unsigned smid;
	asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
	smid &= 255u;
	if (threadIdx.x == 0) s_slot = atomicAdd(&g_next[smid], 1u) % SLOTS_PER_SM;
	__syncthreads();
	MapBytes *const slot = g_maps[smid][s_slot];

	if (threadIdx.x < 32) {
		unsigned const lane = threadIdx.x;
		uint4 const *src = reinterpret_cast<uint4 const *>(lane < 8 ? c_map_q.b : c_map_kv.b) + (lane & 7u);
		if (lane < 16) reinterpret_cast<uint4 *>(s_maps[lane >> 3].b)[lane & 7u] = *src;
		__syncwarp();
		if (lane == 0) {
			unsigned const mq = smem_u32(s_maps[0].b), mkv = smem_u32(s_maps[1].b);
			map_set_address(mq, q);
			map_set_rows(mq, static_cast<unsigned>(seq_len));
			map_set_address(mkv, kv);
			map_set_rows(mkv, static_cast<unsigned>(seq_len));
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

	AttnParams p{};
	p.seq_len = static_cast<u32>(seq_len);
	p.n_heads = X17_N_HEADS;
	// the window is rounded up to a multiple of 16 keys (cuda/attn_fwd_i8.cuh:408-412); zero or a window
	// that covers the sequence means unbounded
	{
		unsigned long long const w = window_size == 0 ? 0 : ((window_size - 1) / 16 + 1) * 16;
		p.window = (w == 0 || w >= seq_len) ? 0xFFFFFFFFu : static_cast<u32>(w);
	}
	p.q = q;
	p.q_stride = X17_Q_STRIDE;
	p.q_batch_stride = 0;
	p.sink_k = sink_k;
	p.sink_v = sink_v;
	p.temperature = attn_temperature;
	p.out = out;
	p.o_stride = X17_O_STRIDE;
	p.o_batch_stride = 0;
	p.l = l;
	p.l_batch_stride = 0;
	p.status = x17_status;
	constexpr u32 HEADS_PER_CTA = X17_HEAD_DIM >= 128 ? 1 : 128 / X17_HEAD_DIM;
	for (u32 h = 0; h < HEADS_PER_CTA; ++h) {
		u32 const head = blockIdx.y * HEADS_PER_CTA + h;
		if (head >= X17_N_HEADS) break;
		attn_fwd_body<X17_HEAD_DIM, false, false>(reinterpret_cast<CUtensorMap const *>(slot[0].b),
												  reinterpret_cast<CUtensorMap const *>(slot[1].b), p, head,
												  h + 1 < HEADS_PER_CTA);
		__syncthreads();
	}
}
