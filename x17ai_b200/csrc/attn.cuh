// int8 sliding-window attention forward for sm_100a (tcgen05 + TMEM + TMA).
//
// Replaces AttnForward<...>::run (cuda/attn_fwd_i8.cuh:368-619) behind the same argument list
// (templates/attn/kernel.cu:9-20), with a batch dimension added as grid.z.
//
// Semantics kept from the reference: a query i attends keys i-W' .. i-1 (W' = window rounded up
// to 16, 0 = unbounded) plus a per-head sink token; scores are exact int32 dot products times
// the temperature D^-1/2 / 64 * log2(min(W', i) + 4) * temp_h; probabilities are quantised to
// u8 steps of 1/255 and multiplied with V on the int8 tensor cores; the normaliser uses the
// un-rounded probabilities; out = rint(clamp(O / sum)) as FixedI8 and L = log2(sum) + max.
//
// What differs from the reference's schedule: the row maximum is found first (a first sweep of
// Q.K^T over the visible KV tiles that only reduces max), then a second sweep quantises P
// against that final maximum.  P.V therefore accumulates exactly in int32 in TMEM across all
// KV tiles with no rescaling, and the result does not depend on the KV tile size.
//
// One CTA = 128 queries of one (batch, head); two CTAs per SM. 320 threads:
//   warp 0      TMA producer (Q once; K tiles for sweep 1; K and V tiles for sweep 2)
//   warp 1      MMA issuer: S = Q.K^T (kind::i8, M128 N128 K32 x D/32) into TMEM, O += P.V
//               (u8 x s8, V read MN-major straight from its [key][dim] tile) into TMEM columns
//               [128, 128+D). Sweep 1 ping-pongs S between columns [0,128) and [128,256) (O is
//               not live yet) so the tensor core runs one tile ahead of the max scan.
//   warps 2..9  two threads per query row (64 score columns each): tcgen05.ld of the row, max /
//               exp2 / quantise, P written to shared memory in the 128B-swizzled K-major
//               layout, final normalisation and 16-byte stores
// KV tiles wholly outside [i-W', i-1] for every row of the CTA are never loaded.
// The sink score (q . sink_k, exact int32) is taken from the Q tile in shared memory after sweep 1. With peer outputs
// (AttnParams::peer_out) the epilogue collects the output tile in the P buffer and stores it in whole rows to this
// GPU's buffer and to the copies in other GPUs' memory.
#pragma once

#include "ptx.cuh"

namespace x17 {

struct AttnParams {
	u32 seq_len;
	u32 n_heads;
	u32 window;  // already rounded up to 16; 0xFFFFFFFF = unbounded
	i8 const *q;
	u64 q_stride, q_batch_stride;
	i8 const *sink_k;
	i8 const *sink_v;
	f32 const *temperature;
	void *out;  // int8 FixedI8, or bf16 in the fp8 P.V mode
	u64 o_stride, o_batch_stride;  // in elements of the output type
	// FixedI8 output only: copies of `out` in other GPUs' memory (peer-mapped addresses of buffers with the layout of
	// `out`); the epilogue stores every 16 bytes it writes there as well, so a gather of the shards' outputs costs
	// no pass of its own
	static constexpr u32 MAX_PEER_OUT = 7;
	u32 n_peer_out;
	i8 *peer_out[MAX_PEER_OUT];
	f32 const *v_scale;  // fp8 P.V mode: per-head scale of the e4m3 V values
	// per-token-per-head scale mode: value = scale * code, [batch][head][seq] f32 each (null otherwise)
	f32 const *tok_q_scale, *tok_k_scale, *tok_v_scale;
	f32 *l;  // [batch][head][seq] or null
	u64 l_batch_stride;
	u32 *status;
	// validation outputs (only read by the DEBUG instantiation), dense per (batch, head):
	i32 *dbg_s;  // [seq][seq] raw scores of every visited tile
	u8 *dbg_p;   // [seq][seq] quantised probabilities
	i32 *dbg_o;  // [seq][D] int32 P.V accumulator
};

namespace attn_cfg {
constexpr u32 BQ = 128;   // queries per CTA
constexpr u32 BKV = 128;  // keys per tile
constexpr u32 STAGES = 4;
constexpr u32 ROW_WARPS = 8;
constexpr u32 ROW_THREADS = ROW_WARPS * 32;
constexpr u32 THREADS = 64 + ROW_THREADS;
constexpr u32 TMEM_COLS = 256;
constexpr u32 O_COL = 128;
constexpr u32 XCHG_BYTES = ROW_THREADS * 4 + 128 * 4 + 128;  // the row pairs' exchange area, the head's sink values as f32, its sink key
template <u32 D>
constexpr u32 smem_bytes() {
	return BQ * D + STAGES * BKV * D + BQ * BKV + XCHG_BYTES + 1024 + 256;
}
constexpr f32 MAGIC = 12582912.0f;  // 1.5 * 2^23
constexpr u32 MAGIC_BITS = 0x4B400000u;
}  // namespace attn_cfg

X17_DEV uint4 ld_shared_v4(u32 addr) {
	uint4 v;
	asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
	return v;
}
X17_DEV void st_shared_v4(u32 addr, u32 a, u32 b, u32 c, u32 d) {
	asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
				 : "memory");
}

// N score columns of one row -> probabilities: accumulates the un-rounded exp2 into sum[4] and
// returns rint(255 * p) packed four to a word. EDGE: only columns lo <= col < lo + span are visible.
// The four f32 operations per element are issued as packed f32x2 instructions (two elements per
// issue slot); int -> float is one I2FP, float -> u8 uses the 1.5 * 2^23 trick on the FMA pipe. FP8: P is written as OCP e4m3 of 256 * p instead of u8 of 255 * p.
template <bool EDGE, bool FP8 = false, u32 N = 32>
X17_DEV void softmax_chunk(u32 const (&r)[N], u32 col0, f32 temp, f32 neg_m, u32 lo, u32 span,
							  f32 (&sum)[4], u32 (&pk)[N / 4]) {
	using namespace attn_cfg;
	u64 const s256 = pack_f32x2(256.0f, 256.0f);
	u64 const magic2 = pack_f32x2(MAGIC, MAGIC);
	u64 const temp2 = pack_f32x2(temp, temp);
	u64 const negm2 = pack_f32x2(neg_m, neg_m);
	u64 const s255 = pack_f32x2(255.0f, 255.0f);
	u64 sum01 = pack_f32x2(sum[0], sum[1]);
	u64 sum23 = pack_f32x2(sum[2], sum[3]);
#pragma unroll
	for (u32 g = 0; g < N / 4; ++g) {
		u32 q4[4];
#pragma unroll
		for (u32 h = 0; h < 2; ++h) {
			u32 const i = 4 * g + 2 * h;
			// exact int -> float (|acc| < 2^24) with the ALU's I2FP: one instruction, where adding 1.5 * 2^23 to
			// the bits and subtracting it again as a float takes one and a half
			u64 const f2 = pack_f32x2(__int2float_rn(i32(r[i])), __int2float_rn(i32(r[i + 1])));
			u64 const x2 = fma_f32x2(f2, temp2, negm2);
			f32 x0, x1;
			unpack_f32x2(x2, x0, x1);
			if constexpr (EDGE) {
				x0 = (col0 + i - lo) < span ? x0 : -INFINITY;
				x1 = (col0 + i + 1 - lo) < span ? x1 : -INFINITY;
			}
			u64 const e2 = pack_f32x2(ex2_approx(x0), ex2_approx(x1));
			if (h == 0) sum01 = add_f32x2(sum01, e2);
			else sum23 = add_f32x2(sum23, e2);
			if constexpr (FP8) {
				f32 qa, qb;
				unpack_f32x2(mul_f32x2(e2, s256), qa, qb);
				q4[h] = cvt_e4m3x2(qa, qb);
			} else {
				// rint(255 * ex) lands in the low mantissa byte
				u64 const q2 = fma_f32x2(e2, s255, magic2);
				f32 qa, qb;
				unpack_f32x2(q2, qa, qb);
				q4[2 * h] = __float_as_uint(qa);
				q4[2 * h + 1] = __float_as_uint(qb);
			}
		}
		if constexpr (FP8) {
			pk[g] = q4[0] | (q4[1] << 16);
		} else {
			u32 const lo2 = __byte_perm(q4[0], q4[1], 0x0040);
			u32 const hi2 = __byte_perm(q4[2], q4[3], 0x0040);
			pk[g] = __byte_perm(lo2, hi2, 0x5410);
		}
	}
	unpack_f32x2(sum01, sum[0], sum[1]);
	unpack_f32x2(sum23, sum[2], sum[3]);
}

template <bool EDGE, bool WANT_MAX>
X17_DEV void extreme_chunk(u32 const (&r)[32], u32 col0, u32 lo, u32 span, i32 (&ext)[4]) {
#pragma unroll
	for (u32 i = 0; i < 32; ++i) {
		i32 v = i32(r[i]);
		if constexpr (EDGE) {
			bool const valid = (col0 + i - lo) < span;
			v = valid ? v : (WANT_MAX ? INT32_MIN : INT32_MAX);
		}
		ext[i & 3] = WANT_MAX ? max(ext[i & 3], v) : min(ext[i & 3], v);
	}
}

// Per-token-per-head scale mode (the benchmark description's input format; the reference has one global FixedI8
// scale, cuda/utils_b8.cuh:7-10): value = scale[token] * code for q, k and v. The scores carry a per-key factor,
// x = (acc * k_scale[key]) * a_row with a_row = temperature * q_scale[row], and V's per-key scale goes into the
// quantised probabilities: P = rint(255 * 2^(x - m) * v_scale[key] / g), g = the largest v_scale among the row's
// visible keys, so that P <= 255, P.V stays an exact u8 x s8 product and out = O * g / (255 * sum).
// The first sweep reduces t = acc * k_scale[key] (the row maximum of x is a_row times its largest, or for a negative
// temperature its smallest, value) and v_scale; the second computes the probabilities of 32 columns.
template <bool EDGE, bool WANT_MAX>
X17_DEV void scaled_extreme_chunk(u32 const (&r)[32], u32 col0, u32 key0, u32 seq_len, f32 const *ksc, f32 const *vsc,
								  u32 lo, u32 span, f32 &t_ext, f32 &v_max) {
#pragma unroll
	for (u32 i = 0; i < 32; ++i) {
		u32 const key = key0 + i;
		bool vis = key < seq_len;
		if constexpr (EDGE) vis = vis && (col0 + i - lo) < span;
		if (vis) {
			f32 const t = __fmul_rn(__int2float_rn(i32(r[i])), __ldg(ksc + key));
			t_ext = WANT_MAX ? fmaxf(t_ext, t) : fminf(t_ext, t);
			v_max = fmaxf(v_max, __ldg(vsc + key));
		}
	}
}
template <bool EDGE>
X17_DEV void scaled_softmax_chunk(u32 const (&r)[32], u32 col0, u32 key0, u32 seq_len, f32 a_row, f32 const *ksc,
								  f32 const *vsc, f32 neg_m, f32 rg, u32 lo, u32 span, f32 &sum, u32 (&pk)[8]) {
	using namespace attn_cfg;
#pragma unroll
	for (u32 g = 0; g < 8; ++g) {
		u32 q4[4];
#pragma unroll
		for (u32 e4 = 0; e4 < 4; ++e4) {
			u32 const i = 4 * g + e4;
			u32 const key = key0 + i;
			bool vis = key < seq_len;
			if constexpr (EDGE) vis = vis && (col0 + i - lo) < span;
			f32 pq = 0.0f;
			if (vis) {
				f32 const t = __fmul_rn(__int2float_rn(i32(r[i])), __ldg(ksc + key));
				f32 const e = ex2_approx(__fmaf_rn(t, a_row, neg_m));
				sum = __fadd_rn(sum, e);
				pq = fminf(__fmul_rn(__fmul_rn(e, __ldg(vsc + key)), rg), 255.0f);
			}
			q4[e4] = __float_as_uint(__fadd_rn(pq, MAGIC));   // rint(pq) in the low byte
		}
		u32 const lo2 = __byte_perm(q4[0], q4[1], 0x0040);
		u32 const hi2 = __byte_perm(q4[2], q4[3], 0x0040);
		pk[g] = __byte_perm(lo2, hi2, 0x5410);
	}
}

// The same two helpers for a tile that every row sees whole and whose scale vectors can be read four keys at a
// time (16-byte aligned: seq_len a multiple of 4): no masks, no bounds checks (the tile lies below the diagonal,
// so its keys exist), a quarter of the loads, and the multiplications and additions as packed f32x2 instructions;
// the values are those of the general helpers (the same operations in the same order per element).
// EDGE: the tile lies inside the sequence but the row sees only columns lo <= col < lo + span of it
template <bool WANT_MAX, bool EDGE = false>
X17_DEV void scaled_extreme_chunk_full(u32 const (&r)[32], f32 const *ksc, f32 const *vsc, f32 &t_ext, f32 &v_max,
									   u32 col0 = 0, u32 lo = 0, u32 span = 0) {
#pragma unroll
	for (u32 g = 0; g < 8; ++g) {
		float4 const k4 = __ldg(reinterpret_cast<float4 const *>(ksc) + g);
		float4 v4 = __ldg(reinterpret_cast<float4 const *>(vsc) + g);
		f32 t0, t1, t2, t3;
		unpack_f32x2(mul_f32x2(pack_f32x2(__int2float_rn(i32(r[4 * g])), __int2float_rn(i32(r[4 * g + 1]))),
							   pack_f32x2(k4.x, k4.y)), t0, t1);
		unpack_f32x2(mul_f32x2(pack_f32x2(__int2float_rn(i32(r[4 * g + 2])), __int2float_rn(i32(r[4 * g + 3]))),
							   pack_f32x2(k4.z, k4.w)), t2, t3);
		if constexpr (EDGE) {
			f32 const none = WANT_MAX ? -INFINITY : INFINITY;
			bool const s0 = (col0 + 4 * g - lo) < span, s1 = (col0 + 4 * g + 1 - lo) < span;
			bool const s2 = (col0 + 4 * g + 2 - lo) < span, s3 = (col0 + 4 * g + 3 - lo) < span;
			t0 = s0 ? t0 : none; t1 = s1 ? t1 : none; t2 = s2 ? t2 : none; t3 = s3 ? t3 : none;
			v4.x = s0 ? v4.x : 0.0f; v4.y = s1 ? v4.y : 0.0f; v4.z = s2 ? v4.z : 0.0f; v4.w = s3 ? v4.w : 0.0f;
		}
		if constexpr (WANT_MAX) {
			t_ext = fmaxf(fmaxf(t_ext, t0), t1);
			t_ext = fmaxf(fmaxf(t_ext, t2), t3);
		} else {
			t_ext = fminf(fminf(t_ext, t0), t1);
			t_ext = fminf(fminf(t_ext, t2), t3);
		}
		v_max = fmaxf(fmaxf(v_max, v4.x), v4.y);
		v_max = fmaxf(fmaxf(v_max, v4.z), v4.w);
	}
}
template <bool EDGE = false>
X17_DEV void scaled_softmax_chunk_full(u32 const (&r)[32], f32 a_row, f32 const *ksc, f32 const *vsc, f32 neg_m, f32 rg,
									   f32 &sum, u32 (&pk)[8], u32 col0 = 0, u32 lo = 0, u32 span = 0) {
	using namespace attn_cfg;
	u64 const arow2 = pack_f32x2(a_row, a_row);
	u64 const negm2 = pack_f32x2(neg_m, neg_m);
	u64 const rg2 = pack_f32x2(rg, rg);
	u64 const magic2 = pack_f32x2(MAGIC, MAGIC);
	u64 sum2 = pack_f32x2(sum, 0.0f);
#pragma unroll
	for (u32 g = 0; g < 8; ++g) {
		float4 const k4 = __ldg(reinterpret_cast<float4 const *>(ksc) + g);
		float4 const v4 = __ldg(reinterpret_cast<float4 const *>(vsc) + g);
		u32 q4[4];
#pragma unroll
		for (u32 h = 0; h < 2; ++h) {
			u64 const kk = h == 0 ? pack_f32x2(k4.x, k4.y) : pack_f32x2(k4.z, k4.w);
			u64 const vv = h == 0 ? pack_f32x2(v4.x, v4.y) : pack_f32x2(v4.z, v4.w);
			u64 const t2 = mul_f32x2(pack_f32x2(__int2float_rn(i32(r[4 * g + 2 * h])), __int2float_rn(i32(r[4 * g + 2 * h + 1]))), kk);
			f32 x0, x1;
			unpack_f32x2(fma_f32x2(t2, arow2, negm2), x0, x1);
			if constexpr (EDGE) {   // ex2(-inf) = 0: no weight, no share of the sum
				x0 = (col0 + 4 * g + 2 * h - lo) < span ? x0 : -INFINITY;
				x1 = (col0 + 4 * g + 2 * h + 1 - lo) < span ? x1 : -INFINITY;
			}
			u64 const e2 = pack_f32x2(ex2_approx(x0), ex2_approx(x1));
			sum2 = add_f32x2(sum2, e2);
			// e * v_scale * (255 / g) <= 255 up to rounding, so no clamp: rint lands in the low mantissa byte
			f32 qa, qb;
			unpack_f32x2(fma_f32x2(mul_f32x2(e2, vv), rg2, magic2), qa, qb);
			q4[2 * h] = __float_as_uint(qa);
			q4[2 * h + 1] = __float_as_uint(qb);
		}
		u32 const lo2 = __byte_perm(q4[0], q4[1], 0x0040);
		u32 const hi2 = __byte_perm(q4[2], q4[3], 0x0040);
		pk[g] = __byte_perm(lo2, hi2, 0x5410);
	}
	f32 s0, s1;
	unpack_f32x2(sum2, s0, s1);
	sum = __fadd_rn(s0, s1);
}

// FP8PV: P.V on the fp8 tensor path (P as e4m3 of 256 * p, V as e4m3 with a per-head f32 scale, f32
// accumulation in TMEM) and bf16 output; Q.K^T, masks, maximum and normaliser as in the int8 mode.
// The tensor maps are reached through pointers: kernel parameters for the library's entry points, maps
// patched on the device for the kernel object (kernel_objects/attn.cu). `head` is the head this call
// works on; the body may be called again by the same CTA for another head (it invalidates its
// barriers and frees its TMEM columns before it returns) provided `more_calls` was set on the earlier
// calls: a CTA that has given up its TMEM allocation permit must not allocate again.
template <u32 D, bool DEBUG, bool FP8PV = false, bool SCALED = false>
X17_DEV void attn_fwd_body(CUtensorMap const *tm_q_ptr, CUtensorMap const *tm_kv_ptr, AttnParams const &p, u32 head,
						   bool more_calls = false) {
	static_assert(!(SCALED && (FP8PV || DEBUG)), "the per-token-scale mode has no fp8 and no validation form");
	using namespace attn_cfg;
	static_assert(D == 32 || D == 64 || D == 128, "head_dim must be 32, 64 or 128");
	constexpr u32 TILE_BYTES = BKV * D;

	extern __shared__ u8 smem_raw[];
	u32 const smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	u8 *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

	u32 const s_q = smem_base;
	u32 const s_ring = s_q + BQ * D;
	u32 const s_p = s_ring + STAGES * TILE_BYTES;
	constexpr u32 XCHG_OFF = BQ * D + STAGES * TILE_BYTES + BQ * BKV;
	constexpr u32 BAR_OFF = XCHG_OFF + XCHG_BYTES;
	f32 *const xchg = reinterpret_cast<f32 *>(smem_gen + XCHG_OFF);
	f32 *const svf = xchg + ROW_THREADS;
	u8 *const sks = reinterpret_cast<u8 *>(svf + 128);   // the head's sink key (D bytes)
	u32 const bar_base = smem_base + BAR_OFF;
	auto full_bar = [&](u32 s) { return bar_base + 8 * s; };
	auto empty_bar = [&](u32 s) { return bar_base + 8 * (STAGES + s); };
	u32 const q_full_bar = bar_base + 8 * (2 * STAGES + 0);
	u32 const o_full_bar = bar_base + 8 * (2 * STAGES + 1);
	auto s_full_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + 2 + b); };
	auto s_done_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + 4 + b); };
	u32 const p_ready_bar = bar_base + 8 * (2 * STAGES + 6);
	u32 const pv_done_bar = bar_base + 8 * (2 * STAGES + 7);
	u32 const tmem_slot = bar_base + 8 * (2 * STAGES + 8);
	volatile u32 *const tmem_slot_gen =
		reinterpret_cast<volatile u32 *>(smem_gen + BAR_OFF + 8 * (2 * STAGES + 8));
	volatile u32 *const abort_flag = tmem_slot_gen + 1;
	WaitCtx const ctx{abort_flag, p.status};

	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;

	// heavier query tiles (more visible keys) first
	u32 const q_tile = gridDim.x - 1 - blockIdx.x;
	u32 const batch = blockIdx.z;
	u32 const q0 = q_tile * BQ;
	u32 const w = p.window;

	// visible KV tiles: keys max(0, q0 - W') .. q0 + BQ - 2  (the last row sees up to q0+BQ-2)
	u32 const t_begin = (w == 0xFFFFFFFFu || q0 < w) ? 0u : (q0 - w) / BKV;
	u32 const t_end = q_tile;  // inclusive; BQ == BKV, so the diagonal tile has the CTA's index

	// ring entries that thread 0 requests itself right after it has initialised the barriers (below)
	u32 const n_sweep1 = t_end - t_begin + 1;
	u32 const n_early = n_sweep1 < STAGES ? n_sweep1 : STAGES;

	if (threadIdx.x == 0) {
		for (u32 s = 0; s < STAGES; ++s) {
			mbar_init(full_bar(s), 1);
			mbar_init(empty_bar(s), 1);
		}
		mbar_init(q_full_bar, 1);
		mbar_init(o_full_bar, 1);
		for (u32 b = 0; b < 2; ++b) {
			mbar_init(s_full_bar(b), 1);
			mbar_init(s_done_bar(b), ROW_THREADS);
		}
		mbar_init(p_ready_bar, ROW_THREADS);
		mbar_init(pv_done_bar, 1);
		*abort_flag = 0;
		mbar_fence_init();
		fence_proxy_async_smem();
		// Q and the first K tiles are requested before the CTA's set-up barrier: nothing has used the ring yet, so
		// no "empty" wait is needed, and their latency runs under the TMEM allocation
		tma_prefetch_desc(tm_q_ptr);
		tma_prefetch_desc(tm_kv_ptr);
		mbar_expect_tx(q_full_bar, BQ * D);
		tma_load_3d(s_q, tm_q_ptr, q_full_bar, i32(head * D), i32(q0), i32(batch));
		for (u32 s = 0; s < n_early; ++s) {
			mbar_expect_tx(full_bar(s), TILE_BYTES);
			tma_load_3d(s_ring + s * TILE_BYTES, tm_kv_ptr, full_bar(s), i32(2 * head * D), i32((t_begin + s) * BKV),
						i32(batch));
		}
	}
	if (warp == 1) {
		tmem_alloc(tmem_slot, TMEM_COLS);
		if (!more_calls) tmem_relinquish();
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	u32 const tmem_base = *tmem_slot_gen;

	if (warp == 0) {
		// ---------------- TMA producer ----------------
		if (lane == 0) {
			u32 it = n_early;   // thread 0 has already requested Q and the first K tiles of sweep 1
			bool ok = true;
			// one ring entry: the K (item 0) or V (item 1) tile of KV tile t
			auto load = [&](u32 t, u32 item) -> bool {
				u32 const s = it % STAGES;
				u32 const ph = (it / STAGES) & 1;
				if (!mbar_wait(empty_bar(s), ph ^ 1, ctx, ST_WAIT_STAGE_EMPTY, s)) return false;
				mbar_expect_tx(full_bar(s), TILE_BYTES);
				tma_load_3d(s_ring + s * TILE_BYTES, tm_kv_ptr, full_bar(s), i32(2 * head * D + item * D),
							i32(t * BKV), i32(batch));
				++it;
				return true;
			};
			// sweep 1: K tiles. sweep 2, in the order the MMA warp consumes them:
			// K[first], then K[t+1] before V[t] (Q.K^T of the next tile is issued ahead of P.V)
			#pragma unroll 1
			for (u32 t = t_begin + n_early; t <= t_end && ok; ++t) ok = load(t, 0);
			if (ok) ok = load(t_begin, 0);
			#pragma unroll 1
			for (u32 t = t_begin; t <= t_end && ok; ++t) {
				if (t < t_end) ok = load(t + 1, 0);
				if (ok) ok = load(t, 1);
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer ----------------
		if (elect_one()) {
			constexpr u32 idesc_qk = make_idesc(DFMT_S32, FMT_S8, FMT_S8, 0, 0, BQ, BKV);
			constexpr u32 idesc_pv = FP8PV ? make_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 0, 1, BQ, D)
										   : make_idesc(DFMT_S32, FMT_U8, FMT_S8, 0, 1, BQ, D);
			u32 const o_tmem = tmem_base + O_COL;
			bool ok = mbar_wait(q_full_bar, 0, ctx, ST_WAIT_Q_FULL, 0);
			u32 it = 0;
			u32 use0 = 0, use1 = 0;  // Q.K^T tiles issued into S buffer 0 / 1 so far
			u64 const q_desc = make_smem_desc(s_q, D);
			u64 const p_desc = make_smem_desc(s_p, 128);
			u64 const ring_desc = make_smem_desc(s_ring, D);  // + stage * (TILE_BYTES >> 4)

			auto issue_qk = [&](u32 b) -> bool {
				u32 const s = it % STAGES;
				u32 const ph = (it / STAGES) & 1;
				if (!mbar_wait(full_bar(s), ph, ctx, ST_WAIT_TMA_FULL, s)) return false;
				tc_fence_after();
				u64 const bdesc = ring_desc + u64(s * (TILE_BYTES >> 4));
#pragma unroll
				for (u32 ks = 0; ks < D / 32; ++ks) {
					mma_i8_ss(tmem_base + b * BKV, q_desc + 2 * ks, bdesc + 2 * ks, idesc_qk, ks != 0);
				}
				tc_commit(empty_bar(s));
				tc_commit(s_full_bar(b));
				++it;
				use0 += b == 0 ? 1u : 0u;
				use1 += b == 0 ? 0u : 1u;
				return true;
			};
			// O += P.V for one tile; P of that tile is in shared memory
			auto issue_pv = [&](bool first) -> bool {
				u32 const s = it % STAGES;
				u32 const ph = (it / STAGES) & 1;
				if (!mbar_wait(full_bar(s), ph, ctx, ST_WAIT_TMA_FULL, s)) return false;
				tc_fence_after();
				u64 const bdesc = ring_desc + u64(s * (TILE_BYTES >> 4));
#pragma unroll
				for (u32 ks = 0; ks < BKV / 32; ++ks) {
					// A: +32 bytes along the key axis inside the swizzle row;
					// B (MN-major): +32 key rows of D bytes each
					if constexpr (FP8PV) {
						mma_f8_ss(o_tmem, p_desc + 2 * ks, bdesc + ((32 * D) >> 4) * ks, idesc_pv,
								  (!first || ks != 0) ? 1u : 0u);
					} else {
						mma_i8_ss(o_tmem, p_desc + 2 * ks, bdesc + ((32 * D) >> 4) * ks, idesc_pv,
								  (!first || ks != 0) ? 1u : 0u);
					}
				}
				tc_commit(empty_bar(s));
				tc_commit(pv_done_bar);
				++it;
				return true;
			};
			// before S_b is overwritten, its previous contents must have been read
			auto wait_s_read = [&](u32 b, u32 t) -> bool {
				u32 const used = b == 0 ? use0 : use1;
				if (used == 0) return true;
				if (!mbar_wait(s_done_bar(b), (used - 1) & 1, ctx, ST_WAIT_S_DONE, t)) return false;
				tc_fence_after();
				return true;
			};

			// sweep 1: the scores ping-pong between the two halves of the allocation
			#pragma unroll 1
			for (u32 t = t_begin; t <= t_end && ok; ++t) {
				u32 const b = (t - t_begin) & 1u;
				ok = wait_s_read(b, t) && issue_qk(b);
			}
			// sweep 2: S lives in buffer 0 only; the rows copy it to registers and release it at
			// once, so Q.K^T of tile t+1 runs while they work on tile t
			if (ok) ok = wait_s_read(0, t_begin) && issue_qk(0);
			u32 n_p = 0;
			#pragma unroll 1
			for (u32 t = t_begin; t <= t_end && ok; ++t) {
				if (t < t_end) ok = wait_s_read(0, t) && issue_qk(0);
				if (!ok) break;
				if (!mbar_wait(p_ready_bar, n_p & 1, ctx, ST_WAIT_S_DONE, 0x100u + t)) {
					ok = false;
					break;
				}
				++n_p;
				tc_fence_after();
				ok = issue_pv(t == t_begin);
			}
			if (ok) tc_commit(o_full_bar);
		}
	} else {
		// ---------------- two threads per query row ----------------
		u32 const quarter = warp & 3;          // TMEM lanes this warp may touch
		u32 const half = (warp - 2) >> 2;      // which 64 score columns / which half of D
		u32 const row = quarter * 32 + lane;
		u32 const qi = q0 + row;
		bool const row_ok = qi < p.seq_len;
		u32 const lane_addr = (quarter * 32u) << 16;
		u32 const xid = half * BQ + row;       // own slot in the exchange area
		u32 const xpartner = (half ^ 1u) * BQ + row;

		// temperature (attn_fwd_i8.cuh:444-450, :497)
		u32 const n_att = (qi < w ? qi : w) + 4u;
		f32 const base_t = f32((1.0 / 64.0) * (D == 128 ? 0.08838834764831845 : D == 64 ? 0.125 : 0.17677669529663687));
		f32 const row_t = __fmul_rn(base_t, lg2_approx(f32(n_att)));
		f32 const head_t = __ldg(p.temperature + head);
		f32 const temp = __fmul_rn(row_t, head_t);
		bool const pos_t = head_t >= 0.0f;  // uniform over the CTA; row_t > 0 always
		// per-token-scale mode: x = acc * a_row * k_scale[key]; the FixedI8 mode is its case q_scale = k_scale = 1/8
		u64 const tok_base = (u64(batch) * p.n_heads + head) * p.seq_len;
		f32 const a_row = SCALED ? __fmul_rn(__fmul_rn(temp, 64.0f), row_ok ? __ldg(p.tok_q_scale + tok_base + qi) : 0.125f) : 0.0f;
		f32 const *const ksc = SCALED ? p.tok_k_scale + tok_base : nullptr;
		f32 const *const vsc = SCALED ? p.tok_v_scale + tok_base : nullptr;
		// whole tiles may read the scale vectors four keys at a time when every (batch, head) row of them starts
		// on a 16-byte boundary
		bool const scales_by_four = SCALED && (p.seq_len & 3u) == 0
									&& ((reinterpret_cast<u64>(p.tok_k_scale) | reinterpret_cast<u64>(p.tok_v_scale)) & 15u) == 0;
		// the head's sink values as f32 and its sink key, once per CTA (the key is read after sweep 1, one
		// named barrier later; the values in the epilogue)
		if (threadIdx.x - 64u < D) {
			u32 const b = reinterpret_cast<u8 const *>(p.sink_v)[head * D + (threadIdx.x - 64u)];
			svf[threadIdx.x - 64u] = FP8PV ? hw_e4m3_to_f32(b) : f32(i32(i8(b)));
			sks[threadIdx.x - 64u] = reinterpret_cast<u8 const *>(p.sink_k)[head * D + (threadIdx.x - 64u)];
		}

		u32 use0 = 0, use1 = 0;  // how often S buffer 0 / 1 has been consumed
		bool ok = true;
		u32 const col_base = half * 64u;

		// visible columns of this row inside tile k0: lo <= col < lo + span (only used on edge tiles)
		auto visible = [&](u32 k0, u32 &lo, u32 &span) {
			i32 const hi_i = min(i32(BKV), i32(qi) - i32(k0));                                  // col < qi - k0
			i32 const lo_i = (w == 0xFFFFFFFFu) ? 0 : max(0, i32(qi) - i32(w) - i32(k0));      // col >= qi - w - k0
			lo = u32(lo_i);
			span = hi_i > lo_i ? u32(hi_i - lo_i) : 0u;
		};

		// ---- sweep 1: row extreme over the visible keys ----
		i32 ext[4];
#pragma unroll
		for (u32 i = 0; i < 4; ++i) ext[i] = pos_t ? INT32_MIN : INT32_MAX;
		f32 t_ext = pos_t ? -INFINITY : INFINITY, v_max = 0.0f;  // per-token-scale mode: extreme of acc * k_scale, largest v_scale
		#pragma unroll 1
		for (u32 t = t_begin; t <= t_end && ok; ++t) {
			u32 const b = (t - t_begin) & 1u;
			u32 const par = b == 0 ? (use0 & 1u) : (use1 & 1u);
			if (!mbar_wait_warp(s_full_bar(b), par, ctx, ST_WAIT_S_FULL, t)) {
				ok = false;
				break;
			}
			use0 += b == 0 ? 1u : 0u;
			use1 += b == 0 ? 0u : 1u;
			tc_fence_after();
			u32 const k0 = t * BKV;
			bool const edge = (t == t_end) || (w != 0xFFFFFFFFu && k0 + w < q0 + BQ - 1);
			u32 lo = 0, span = BKV;
			if (edge) visible(k0, lo, span);
			u32 r0[32], r1[32];
			u32 const ta = tmem_base + lane_addr + b * BKV + col_base;
			tmem_ld_32x32b_x32(ta, r0);
			tmem_ld_32x32b_x32(ta + 32, r1);
			tmem_wait_ld();
			tc_fence_before();
			mbar_arrive(s_done_bar(b));  // S_b is in registers now
			if constexpr (SCALED) {
				u32 const kc = k0 + col_base;
				if (edge && scales_by_four && k0 + BKV <= p.seq_len) {   // an edge tile whose keys all exist
					if (pos_t) {
						scaled_extreme_chunk_full<true, true>(r0, ksc + kc, vsc + kc, t_ext, v_max, col_base, lo, span);
						scaled_extreme_chunk_full<true, true>(r1, ksc + kc + 32, vsc + kc + 32, t_ext, v_max, col_base + 32, lo, span);
					} else {
						scaled_extreme_chunk_full<false, true>(r0, ksc + kc, vsc + kc, t_ext, v_max, col_base, lo, span);
						scaled_extreme_chunk_full<false, true>(r1, ksc + kc + 32, vsc + kc + 32, t_ext, v_max, col_base + 32, lo, span);
					}
				} else if (edge) {
					if (pos_t) {
						scaled_extreme_chunk<true, true>(r0, col_base, kc, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
						scaled_extreme_chunk<true, true>(r1, col_base + 32, kc + 32, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
					} else {
						scaled_extreme_chunk<true, false>(r0, col_base, kc, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
						scaled_extreme_chunk<true, false>(r1, col_base + 32, kc + 32, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
					}
				} else if (scales_by_four) {
					if (pos_t) {
						scaled_extreme_chunk_full<true>(r0, ksc + kc, vsc + kc, t_ext, v_max);
						scaled_extreme_chunk_full<true>(r1, ksc + kc + 32, vsc + kc + 32, t_ext, v_max);
					} else {
						scaled_extreme_chunk_full<false>(r0, ksc + kc, vsc + kc, t_ext, v_max);
						scaled_extreme_chunk_full<false>(r1, ksc + kc + 32, vsc + kc + 32, t_ext, v_max);
					}
				} else if (pos_t) {
					scaled_extreme_chunk<false, true>(r0, col_base, kc, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
					scaled_extreme_chunk<false, true>(r1, col_base + 32, kc + 32, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
				} else {
					scaled_extreme_chunk<false, false>(r0, col_base, kc, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
					scaled_extreme_chunk<false, false>(r1, col_base + 32, kc + 32, p.seq_len, ksc, vsc, lo, span, t_ext, v_max);
				}
			} else if (!edge) {
				if (pos_t) {
					extreme_chunk<false, true>(r0, col_base, lo, span, ext);
					extreme_chunk<false, true>(r1, col_base + 32, lo, span, ext);
				} else {
					extreme_chunk<false, false>(r0, col_base, lo, span, ext);
					extreme_chunk<false, false>(r1, col_base + 32, lo, span, ext);
				}
			} else {
				if (pos_t) {
					extreme_chunk<true, true>(r0, col_base, lo, span, ext);
					extreme_chunk<true, true>(r1, col_base + 32, lo, span, ext);
				} else {
					extreme_chunk<true, false>(r0, col_base, lo, span, ext);
					extreme_chunk<true, false>(r1, col_base + 32, lo, span, ext);
				}
			}
			if constexpr (DEBUG) {
				if (row_ok) {
					i32 *dst = p.dbg_s + (u64(batch) * p.n_heads + head) * p.seq_len * p.seq_len
							   + u64(qi) * p.seq_len + k0 + col_base;
#pragma unroll
					for (u32 i = 0; i < 32; ++i) {
						if (k0 + col_base + i < p.seq_len) dst[i] = i32(r0[i]);
						if (k0 + col_base + 32 + i < p.seq_len) dst[32 + i] = i32(r1[i]);
					}
				}
			}
		}
		// own candidate, then the partner's (the other 64 columns of the same row)
		f32 cand = -INFINITY;
		{
			i32 const e = pos_t ? max(max(ext[0], ext[1]), max(ext[2], ext[3]))
								: min(min(ext[0], ext[1]), min(ext[2], ext[3]));
			if (e != (pos_t ? INT32_MIN : INT32_MAX)) cand = __fmul_rn(__int2float_rn(e), temp);
		}
		if constexpr (SCALED) cand = (t_ext > -INFINITY && t_ext < INFINITY) ? __fmul_rn(t_ext, a_row) : -INFINITY;
		xchg[xid] = cand;
		named_barrier_sync(1, ROW_THREADS);   // also: sks has been written
		// sink score: exact int32 dot product of this row's q with sink_k (the sink key and value are FixedI8,
		// scale 1/8, in every mode). q comes from the Q tile in shared memory, after the first sweep: reading the
		// row from global memory in front of the sweep cost every CTA some four thousand cycles of load latency.
		i32 sink_dot = 0;
		if (ok && mbar_wait_warp(q_full_bar, 0, ctx, ST_WAIT_Q_FULL, 1)) {
			// 16-byte chunks of a Q row are XOR-swizzled by the row index the way the TMA wrote them
			u32 const q_swz = D == 128 ? (row & 7u) : D == 64 ? ((row >> 1) & 3u) : ((row >> 2) & 1u);
			u8 const *qrow = smem_gen + row * D;
#pragma unroll
			for (u32 i = 0; i < D / 16; ++i) {
				uint4 const a = *reinterpret_cast<uint4 const *>(qrow + ((i ^ q_swz) << 4));
				uint4 const b = *reinterpret_cast<uint4 const *>(sks + 16 * i);
				sink_dot = __dp4a(i32(a.x), i32(b.x), sink_dot);
				sink_dot = __dp4a(i32(a.y), i32(b.y), sink_dot);
				sink_dot = __dp4a(i32(a.z), i32(b.z), sink_dot);
				sink_dot = __dp4a(i32(a.w), i32(b.w), sink_dot);
			}
		} else {
			ok = false;
		}
		f32 const sink_s = SCALED ? __fmul_rn(__fmul_rn(__int2float_rn(sink_dot), a_row), 0.125f)
								  : __fmul_rn(__int2float_rn(sink_dot), temp);
		f32 const m = fmaxf(sink_s, fmaxf(cand, xchg[xpartner]));
		named_barrier_sync(1, ROW_THREADS);  // the exchange area is reused for the sums
		// per-token-scale mode: g = the row's largest v_scale; P = 255 * 2^(x - m) * v_scale / g
		f32 g_row = 0.0f, rg = 0.0f;
		if constexpr (SCALED) {
			xchg[xid] = v_max;
			named_barrier_sync(1, ROW_THREADS);
			g_row = fmaxf(v_max, xchg[xpartner]);   // the largest v_scale among the row's visible keys
			named_barrier_sync(1, ROW_THREADS);
			if (g_row > 0.0f) rg = __fmul_rn(255.0f, rcp_approx(g_row));
		}

		// ---- sweep 2: probabilities against the final maximum ----
		f32 const neg_m = -m;
		f32 sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
		u32 const p_row = s_p + row * 128u;
		u32 const sw = row & 7u;
		u32 const ch0 = half * 4u;  // first of this thread's four 16-byte chunks
		#pragma unroll 1
		for (u32 t = t_begin; t <= t_end && ok; ++t) {
			if (!mbar_wait_warp(s_full_bar(0), use0 & 1, ctx, ST_WAIT_S_FULL, t)) {
				ok = false;
				break;
			}
			++use0;
			tc_fence_after();
			u32 const k0 = t * BKV;
			bool const edge = (t == t_end) || (w != 0xFFFFFFFFu && k0 + w < q0 + BQ - 1);
			u32 lo = 0, span = BKV;
			if (edge) visible(k0, lo, span);
			u32 r0[32], r1[32];
			u32 const ta = tmem_base + lane_addr + col_base;
			u32 pk0[8], pk1[8];
			tmem_ld_32x32b_x32(ta, r0);
			tmem_ld_32x32b_x32(ta + 32, r1);
			tmem_wait_ld();
			tc_fence_before();
			mbar_arrive(s_done_bar(0));  // S is in registers: the next Q.K^T may overwrite it
			if constexpr (SCALED) {
				if (edge && scales_by_four && k0 + BKV <= p.seq_len) {
					scaled_softmax_chunk_full<true>(r0, a_row, ksc + k0 + col_base, vsc + k0 + col_base, neg_m, rg, sum[0], pk0, col_base, lo, span);
					scaled_softmax_chunk_full<true>(r1, a_row, ksc + k0 + col_base + 32, vsc + k0 + col_base + 32, neg_m, rg, sum[1], pk1, col_base + 32, lo, span);
				} else if (edge) {
					scaled_softmax_chunk<true>(r0, col_base, k0 + col_base, p.seq_len, a_row, ksc, vsc, neg_m, rg, lo, span, sum[0], pk0);
					scaled_softmax_chunk<true>(r1, col_base + 32, k0 + col_base + 32, p.seq_len, a_row, ksc, vsc, neg_m, rg, lo, span, sum[1], pk1);
				} else if (scales_by_four) {
					scaled_softmax_chunk_full(r0, a_row, ksc + k0 + col_base, vsc + k0 + col_base, neg_m, rg, sum[0], pk0);
					scaled_softmax_chunk_full(r1, a_row, ksc + k0 + col_base + 32, vsc + k0 + col_base + 32, neg_m, rg, sum[1], pk1);
				} else {
					scaled_softmax_chunk<false>(r0, col_base, k0 + col_base, p.seq_len, a_row, ksc, vsc, neg_m, rg, lo, span, sum[0], pk0);
					scaled_softmax_chunk<false>(r1, col_base + 32, k0 + col_base + 32, p.seq_len, a_row, ksc, vsc, neg_m, rg, lo, span, sum[1], pk1);
				}
			} else if (!edge) {
				softmax_chunk<false, FP8PV>(r0, col_base, temp, neg_m, lo, span, sum, pk0);
				softmax_chunk<false, FP8PV>(r1, col_base + 32, temp, neg_m, lo, span, sum, pk1);
			} else {
				softmax_chunk<true, FP8PV>(r0, col_base, temp, neg_m, lo, span, sum, pk0);
				softmax_chunk<true, FP8PV>(r1, col_base + 32, temp, neg_m, lo, span, sum, pk1);
			}
			if (t > t_begin) {  // P.V of the previous tile has finished reading the P buffer
				if (!mbar_wait_warp(pv_done_bar, (t - t_begin - 1) & 1, ctx, ST_WAIT_O_FULL, 0x100u + t)) {
					ok = false;
					break;
				}
			}
			st_shared_v4(p_row + (((ch0 + 0) ^ sw) << 4), pk0[0], pk0[1], pk0[2], pk0[3]);
			st_shared_v4(p_row + (((ch0 + 1) ^ sw) << 4), pk0[4], pk0[5], pk0[6], pk0[7]);
			st_shared_v4(p_row + (((ch0 + 2) ^ sw) << 4), pk1[0], pk1[1], pk1[2], pk1[3]);
			st_shared_v4(p_row + (((ch0 + 3) ^ sw) << 4), pk1[4], pk1[5], pk1[6], pk1[7]);
			fence_proxy_async_smem();
			mbar_arrive(p_ready_bar);
			if constexpr (DEBUG) {
				if (row_ok) {
					u8 *dst = p.dbg_p + (u64(batch) * p.n_heads + head) * p.seq_len * p.seq_len
							  + u64(qi) * p.seq_len + k0 + col_base;
#pragma unroll
					for (u32 i = 0; i < 32; ++i) {
						if (k0 + col_base + i < p.seq_len) dst[i] = u8(pk0[i >> 2] >> (8 * (i & 3)));
						if (k0 + col_base + 32 + i < p.seq_len) dst[32 + i] = u8(pk1[i >> 2] >> (8 * (i & 3)));
					}
				}
			}
		}

		// ---- normalise and store: each thread of the pair takes half of the D columns ----
		f32 const part = __fadd_rn(__fadd_rn(sum[0], sum[1]), __fadd_rn(sum[2], sum[3]));
		xchg[xid] = part;
		named_barrier_sync(1, ROW_THREADS);
		f32 const other = xchg[xpartner];
		f32 const both = half == 0 ? __fadd_rn(part, other) : __fadd_rn(other, part);
		if (ok && mbar_wait_warp(o_full_bar, 0, ctx, ST_WAIT_O_FULL, 0)) {
			tc_fence_after();
			f32 const sink_e = ex2_approx(__fsub_rn(sink_s, m));
			constexpr f32 PS = FP8PV ? 256.0f : 255.0f;  // scale of the quantised probabilities
			f32 const total = __fmul_rn(__fadd_rn(both, sink_e), PS);
			f32 const w_sink = __fmul_rn(sink_e, PS);
			f32 const recip = rcp_approx(total);
			constexpr u32 HALF_D = D / 2;
			u32 const d0 = half * HALF_D;
			u64 const out_off = u64(batch) * p.o_batch_stride + u64(qi) * p.o_stride + head * D + d0;
			f32 const vs = FP8PV ? __fmul_rn(recip, __ldg(p.v_scale + head)) : recip;
			// all of this thread's O columns are requested at once: one load latency per row instead of four
			u32 r_all[HALF_D / 16][16];
#pragma unroll
			for (u32 c = 0; c < HALF_D; c += 16) tmem_ld_32x32b_x16(tmem_base + lane_addr + O_COL + d0 + c, r_all[c / 16]);
			tmem_wait_ld();
#pragma unroll
			for (u32 c = 0; c < HALF_D; c += 16) {
				u32 const (&r)[16] = r_all[c / 16];
				f32 sv[16];
#pragma unroll
				for (u32 i = 0; i < 16; i += 4) {
					float4 const s4 = *reinterpret_cast<float4 const *>(svf + d0 + c + i);
					sv[i] = s4.x; sv[i + 1] = s4.y; sv[i + 2] = s4.z; sv[i + 3] = s4.w;
				}
				if constexpr (FP8PV) {
					// O is f32 = sum of (256 p) * e4m3(v); sink_v is e4m3 too; out = bf16(value * v_scale)
					u32 o2[8];
#pragma unroll
					for (u32 i = 0; i < 16; i += 2) {
						f32 const oa = __fmul_rn(__fmaf_rn(w_sink, sv[i], __uint_as_float(r[i])), vs);
						f32 const ob = __fmul_rn(__fmaf_rn(w_sink, sv[i + 1], __uint_as_float(r[i + 1])), vs);
						o2[i / 2] = cvt_bf16x2(oa, ob);
					}
					if (row_ok) {
						uint4 *dst = reinterpret_cast<uint4 *>(static_cast<u16 *>(p.out) + out_off + c);
						dst[0] = make_uint4(o2[0], o2[1], o2[2], o2[3]);
						dst[1] = make_uint4(o2[4], o2[5], o2[6], o2[7]);
					}
				} else if constexpr (SCALED) {
					// O = (255 / g) * sum of 2^(x - m) * v; the sink's value is FixedI8 (code / 8); out = bf16(value)
					f32 const ws8 = __fmul_rn(w_sink, 0.125f);
					u32 o2[8];
#pragma unroll
					for (u32 i = 0; i < 16; i += 2) {
						f32 const oa = __fmul_rn(__fmaf_rn(ws8, sv[i], __fmul_rn(__int2float_rn(i32(r[i])), g_row)), recip);
						f32 const ob = __fmul_rn(__fmaf_rn(ws8, sv[i + 1], __fmul_rn(__int2float_rn(i32(r[i + 1])), g_row)), recip);
						o2[i / 2] = cvt_bf16x2(oa, ob);
					}
					if (row_ok) {
						uint4 *dst = reinterpret_cast<uint4 *>(static_cast<u16 *>(p.out) + out_off + c);
						dst[0] = make_uint4(o2[0], o2[1], o2[2], o2[3]);
						dst[1] = make_uint4(o2[4], o2[5], o2[6], o2[7]);
					}
				} else {
					// rint(clamp(o * recip)) through the 1.5 * 2^23 trick: the code is the low byte
					u32 pk[4];
#pragma unroll
					for (u32 g = 0; g < 4; ++g) {
						u32 b4[4];
#pragma unroll
						for (u32 e = 0; e < 4; ++e) {
							f32 const o = __fmaf_rn(w_sink, sv[4 * g + e], __int2float_rn(i32(r[4 * g + e])));
							f32 const q = __fmaf_rn(o, recip, MAGIC);
							b4[e] = __float_as_uint(fminf(fmaxf(q, MAGIC - 127.0f), MAGIC + 127.0f));
						}
						u32 const lo2 = __byte_perm(b4[0], b4[1], 0x0040);
						u32 const hi2 = __byte_perm(b4[2], b4[3], 0x0040);
						pk[g] = __byte_perm(lo2, hi2, 0x5410);
					}
					if (p.n_peer_out != 0) {
						// the tile is collected row-major in the P buffer (free: the last P.V has completed), 16-byte
						// chunks XOR-swizzled by the row, and stored below in whole rows
						u32 const ch = (d0 + c) >> 4;
						st_shared_v4(s_p + row * D + ((ch ^ (row & (D / 16 - 1))) << 4), pk[0], pk[1], pk[2], pk[3]);
					} else if (row_ok) {
						*reinterpret_cast<uint4 *>(static_cast<i8 *>(p.out) + out_off + c) =
							make_uint4(pk[0], pk[1], pk[2], pk[3]);
						if constexpr (DEBUG) {
							i32 *d = p.dbg_o + ((u64(batch) * p.n_heads + head) * p.seq_len + qi) * D + d0 + c;
#pragma unroll
							for (u32 i = 0; i < 16; ++i) d[i] = i32(r[i]);
						}
					}
				}
			}
			if (row_ok && half == 0 && p.l != nullptr) {
				p.l[u64(batch) * p.l_batch_stride + u64(head) * p.seq_len + qi] =
					__fadd_rn(lg2_approx(total), m);
			}
		}
		// Output copies in other GPUs' memory: the rows of the tile leave shared memory whole (eight lanes per 128-byte
		// row of a head), to this GPU's `out` and to every peer's copy with plain stores over NVLink; 16-byte stores of one
		// thread per row, as the direct path above issues them, would cross the link as 16-byte packets. Every row thread
		// reaches this barrier, whatever its waits returned.
		if (p.n_peer_out != 0) {
			if constexpr (!FP8PV && !SCALED) {
				named_barrier_sync(1, ROW_THREADS);
				constexpr u32 CH = D / 16;   // 16-byte chunks per row
				u32 const tid = threadIdx.x - 64u;
#pragma unroll
				for (u32 k = 0; k < (BQ * CH) / ROW_THREADS; ++k) {
					u32 const idx = k * ROW_THREADS + tid;
					u32 const rr = idx / CH, cc = idx % CH;
					if (ok && q0 + rr < p.seq_len) {
						uint4 const v = ld_shared_v4(s_p + rr * D + ((cc ^ (rr & (CH - 1))) << 4));
						u64 const off = u64(batch) * p.o_batch_stride + u64(q0 + rr) * p.o_stride + head * D + cc * 16u;
						*reinterpret_cast<uint4 *>(static_cast<i8 *>(p.out) + off) = v;
						for (u32 pr = 0; pr < p.n_peer_out; ++pr) *reinterpret_cast<uint4 *>(p.peer_out[pr] + off) = v;
					}
				}
			}
		}
	}

	tc_fence_before();
	__syncthreads();
	if (warp == 1) {
		__syncwarp();
		tc_fence_after();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
	if (threadIdx.x == 0) {
		// every phase has completed: the barrier words may be initialised again by a later call
		for (u32 i = 0; i < 2 * STAGES + 8; ++i) mbar_inval(bar_base + 8 * i);
	}
}

template <u32 D, bool DEBUG, bool FP8PV = false, bool SCALED = false>
__global__ void __launch_bounds__(attn_cfg::THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
				const AttnParams p) {
	attn_fwd_body<D, DEBUG, FP8PV, SCALED>(&tm_q, &tm_kv, p, blockIdx.y);
}

}  // namespace x17
