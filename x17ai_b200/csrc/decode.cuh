// int8 decode attention: one new token per sequence against an int8 KV cache. HBM-bound.
//
// The reference has no int8 decode kernel (its attn_incremental.cu:329-481 is a stale bf16
// header); the semantics here are those of row `kv_len` of the prefill kernel
// (cuda/attn_fwd_i8.cuh:368-619): keys kv_len-W' .. kv_len-1 plus the sink, temperature
// D^-1/2 / 64 * log2(min(W', kv_len) + 4) * temp_h, u8 probabilities in steps of 1/255,
// int32 P.V, out = rint(clamp(O / sum)), L = log2(sum) + max.
//
// Grid (head, batch, split). 256 threads; each group of D/16 lanes streams one key row
// (16 bytes per lane, 32 / (D/16) rows per warp instruction): q.k with dp4a + a butterfly
// inside the group, online softmax per group with lazy rescale (the int32 P.V accumulators
// are only flushed to f32 when the group's running maximum moves), P.V with dp4a after a 4x4
// byte transpose of four V rows. Groups, warps and (with n_splits > 1) CTAs are merged with
// the usual (max, sum, O) log-sum-exp combine; the sink token enters as one more partial.
// With n_splits > 1 the CTAs write partials to scratch memory and a second kernel merges them.
#pragma once

#include "ptx.cuh"

namespace x17 {

struct DecodeParams {
	i8 const *q;          // [B, H*D]
	u64 q_stride;
	i8 const *kv;         // [B, T, H*2*D], per head [K(D) | V(D)]
	u64 kv_stride, kv_batch_stride;
	u32 const *kv_lens;   // [B] or null (then kv_len); entries above kv_capacity are clamped to it
	u32 kv_len;
	u32 kv_capacity;      // rows of one sequence's cache
	u32 window;           // rounded up to 16; 0xFFFFFFFF = unbounded
	i8 const *sink_k, *sink_v;
	f32 const *temperature;
	i8 *out;              // [B, H*D]
	u64 o_stride;
	f32 *l;               // [B, H] or null
	u32 n_heads;
	u32 n_splits;
	f32 *scratch;         // [B][H][n_splits][D + 2] partials (n_splits > 1)
};

namespace dec_cfg {
constexpr u32 WARPS = 8;
constexpr u32 THREADS = WARPS * 32;
constexpr u32 UNROLL = 4;  // key rows in flight per lane group (also the dp4a depth of P.V)
}  // namespace dec_cfg

// a: four signed bytes, b: four unsigned bytes
X17_DEV i32 dp4a_s8_u8(u32 a, u32 b, i32 c) {
	i32 d;
	asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
	return d;
}

X17_DEV void transpose4x4_bytes(u32 a, u32 b, u32 c, u32 d, u32 (&o)[4]) {
	u32 const t0 = __byte_perm(a, b, 0x5140);
	u32 const t1 = __byte_perm(c, d, 0x5140);
	u32 const t2 = __byte_perm(a, b, 0x7362);
	u32 const t3 = __byte_perm(c, d, 0x7362);
	o[0] = __byte_perm(t0, t1, 0x5410);
	o[1] = __byte_perm(t0, t1, 0x7632);
	o[2] = __byte_perm(t2, t3, 0x5410);
	o[3] = __byte_perm(t2, t3, 0x7632);
}

// combine partial (m, s, o[16]) <- with (m2, s2, o2[16])
X17_DEV void lse_merge(f32 &m, f32 &s, f32 (&o)[16], f32 m2, f32 s2, f32 const (&o2)[16]) {
	f32 const nm = fmaxf(m, m2);
	f32 const a = ex2_approx(m - nm);
	f32 const b = ex2_approx(m2 - nm);
	s = __fmaf_rn(s, a, s2 * b);
#pragma unroll
	for (u32 i = 0; i < 16; ++i) o[i] = __fmaf_rn(o[i], a, o2[i] * b);
	m = nm;
}

template <u32 D>
__global__ void __launch_bounds__(dec_cfg::THREADS)
attn_decode_kernel(const DecodeParams p) {
	using namespace dec_cfg;
	static_assert(D == 32 || D == 64 || D == 128);
	constexpr u32 LPR = D / 16;        // lanes per key row
	constexpr u32 RPI = 32 / LPR;      // key rows per warp instruction
	constexpr f32 NEG_BIG = -3.0e38f;

	u32 const head = blockIdx.x;
	u32 const batch = blockIdx.y;
	u32 const split = blockIdx.z;
	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;
	u32 const grp = lane / LPR;        // which row of the instruction this lane works on
	u32 const sub = lane % LPR;        // which 16-byte chunk of the row

	u32 const kv_len = p.kv_lens ? min(p.kv_lens[batch], p.kv_capacity) : p.kv_len;
	u32 const w = p.window;
	u32 const k_lo = (w == 0xFFFFFFFFu || kv_len < w) ? 0u : kv_len - w;
	u32 const n_keys = kv_len - k_lo;
	u32 const per_split = ((n_keys + p.n_splits - 1) / p.n_splits + 15u) & ~15u;
	u32 const s_lo = k_lo + split * per_split;
	u32 const s_hi = min(kv_len, s_lo + per_split);

	// this lane's 16 bytes of q
	uint4 const qv = *reinterpret_cast<uint4 const *>(p.q + u64(batch) * p.q_stride + head * D + sub * 16);
	u32 const qw[4] = {qv.x, qv.y, qv.z, qv.w};

	u32 const n_att = (kv_len < w ? kv_len : w) + 4u;
	f32 const base_t = f32((1.0 / 64.0) * (D == 128 ? 0.08838834764831845 : D == 64 ? 0.125 : 0.17677669529663687));
	f32 const temp = __fmul_rn(__fmul_rn(base_t, lg2_approx(f32(n_att))), __ldg(p.temperature + head));

	i8 const *kv_base = p.kv + u64(batch) * p.kv_batch_stride + u64(head) * 2 * D + sub * 16;

	f32 m = NEG_BIG, ssum = 0.0f;
	f32 o_f[16];
	i32 o_i[16];
#pragma unroll
	for (u32 i = 0; i < 16; ++i) {
		o_f[i] = 0.0f;
		o_i[i] = 0;
	}

	u32 const step = WARPS * RPI * UNROLL;
	u32 since_flush = 0;  // an int32 accumulator takes at most 4 * 255 * 127 per step: flush long before 2^31
	for (u32 t0 = s_lo + (warp * UNROLL) * RPI; t0 < s_hi; t0 += step) {
		// ---- scores of UNROLL rows per group ----
		uint4 kq[UNROLL];
		uint4 vq[UNROLL];
		bool valid[UNROLL];
#pragma unroll
		for (u32 u = 0; u < UNROLL; ++u) {
			u32 const t = t0 + u * RPI + grp;
			valid[u] = t < s_hi;
			i8 const *rowp = kv_base + u64(valid[u] ? t : s_lo) * p.kv_stride;
			kq[u] = __ldg(reinterpret_cast<uint4 const *>(rowp));
			vq[u] = __ldg(reinterpret_cast<uint4 const *>(rowp + D));
		}
		f32 s[UNROLL];
		f32 smax = NEG_BIG;
#pragma unroll
		for (u32 u = 0; u < UNROLL; ++u) {
			i32 dot = __dp4a(i32(kq[u].x), i32(qw[0]), 0);
			dot = __dp4a(i32(kq[u].y), i32(qw[1]), dot);
			dot = __dp4a(i32(kq[u].z), i32(qw[2]), dot);
			dot = __dp4a(i32(kq[u].w), i32(qw[3]), dot);
#pragma unroll
			for (u32 mask = 1; mask < LPR; mask <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, mask);
			s[u] = valid[u] ? __fmul_rn(__int2float_rn(dot), temp) : NEG_BIG;
			smax = fmaxf(smax, s[u]);
		}
		// ---- online softmax with lazy flush of the int32 accumulators ----
		if (smax > m || ++since_flush >= 8192u) {
			since_flush = 0;
			smax = fmaxf(smax, m);
			f32 const a = ex2_approx(m - smax);
#pragma unroll
			for (u32 i = 0; i < 16; ++i) {
				o_f[i] = __fmul_rn(__fadd_rn(o_f[i], __int2float_rn(o_i[i])), a);
				o_i[i] = 0;
			}
			ssum = __fmul_rn(ssum, a);
			m = smax;
		}
		u32 pb[UNROLL];
#pragma unroll
		for (u32 u = 0; u < UNROLL; ++u) {
			f32 const e = valid[u] ? __fmul_rn(ex2_approx(__fsub_rn(s[u], m)), 255.0f) : 0.0f;
			ssum = __fadd_rn(ssum, e);
			pb[u] = u32(__float2int_rn(e));
		}
		static_assert(UNROLL == 4);
		u32 const p4 = pack4(pb[0], pb[1], pb[2], pb[3]);
		// ---- O += P . V for this lane's 16 dims ----
		u32 const va[4] = {vq[0].x, vq[0].y, vq[0].z, vq[0].w};
		u32 const vb[4] = {vq[1].x, vq[1].y, vq[1].z, vq[1].w};
		u32 const vc[4] = {vq[2].x, vq[2].y, vq[2].z, vq[2].w};
		u32 const vd[4] = {vq[3].x, vq[3].y, vq[3].z, vq[3].w};
#pragma unroll
		for (u32 wi = 0; wi < 4; ++wi) {
			u32 tr[4];
			transpose4x4_bytes(va[wi], vb[wi], vc[wi], vd[wi], tr);
#pragma unroll
			for (u32 j = 0; j < 4; ++j) o_i[4 * wi + j] = dp4a_s8_u8(tr[j], p4, o_i[4 * wi + j]);
		}
	}
#pragma unroll
	for (u32 i = 0; i < 16; ++i) o_f[i] = __fadd_rn(o_f[i], __int2float_rn(o_i[i]));

	// ---- merge the lane groups of the warp (lanes with equal `sub` hold the same dims) ----
#pragma unroll
	for (u32 mask = LPR; mask < 32; mask <<= 1) {
		f32 const m2 = __shfl_xor_sync(0xffffffffu, m, mask);
		f32 const s2 = __shfl_xor_sync(0xffffffffu, ssum, mask);
		f32 o2[16];
#pragma unroll
		for (u32 i = 0; i < 16; ++i) o2[i] = __shfl_xor_sync(0xffffffffu, o_f[i], mask);
		lse_merge(m, ssum, o_f, m2, s2, o2);
	}

	// ---- merge the warps through shared memory ----
	__shared__ f32 sh_o[WARPS][D];
	__shared__ f32 sh_m[WARPS], sh_s[WARPS];
	if (lane < LPR) {
#pragma unroll
		for (u32 i = 0; i < 16; ++i) sh_o[warp][lane * 16 + i] = o_f[i];
		if (lane == 0) {
			sh_m[warp] = m;
			sh_s[warp] = ssum;
		}
	}
	__syncthreads();
	if (threadIdx.x < D) {
		u32 const d = threadIdx.x;
		f32 fm = sh_m[0], fs = sh_s[0], fo = sh_o[0][d];
#pragma unroll
		for (u32 wq = 1; wq < WARPS; ++wq) {
			f32 const nm = fmaxf(fm, sh_m[wq]);
			f32 const a = ex2_approx(fm - nm), b = ex2_approx(sh_m[wq] - nm);
			fs = __fmaf_rn(fs, a, sh_s[wq] * b);
			fo = __fmaf_rn(fo, a, sh_o[wq][d] * b);
			fm = nm;
		}
		if (p.n_splits > 1) {
			f32 *dst = p.scratch + ((u64(batch) * p.n_heads + head) * p.n_splits + split) * (D + 2);
			dst[d] = fo;
			if (d == 0) {
				dst[D] = fm;
				dst[D + 1] = fs;
			}
		} else {
			// the sink token: max = its score, weight 255, value 255 * sink_v
			i32 sdot = 0;
			uint4 const *qh = reinterpret_cast<uint4 const *>(p.q + u64(batch) * p.q_stride + head * D);
			uint4 const *sk = reinterpret_cast<uint4 const *>(p.sink_k + head * D);
			for (u32 i = 0; i < D / 16; ++i) {
				uint4 a = qh[i], b = __ldg(sk + i);
				sdot = __dp4a(i32(a.x), i32(b.x), sdot);
				sdot = __dp4a(i32(a.y), i32(b.y), sdot);
				sdot = __dp4a(i32(a.z), i32(b.z), sdot);
				sdot = __dp4a(i32(a.w), i32(b.w), sdot);
			}
			f32 const sink_s = __fmul_rn(__int2float_rn(sdot), temp);
			f32 const nm = fmaxf(fm, sink_s);
			f32 const a = ex2_approx(fm - nm), b = ex2_approx(sink_s - nm);
			fs = __fmaf_rn(fs, a, 255.0f * b);
			fo = __fmaf_rn(fo, a, 255.0f * f32(p.sink_v[head * D + d]) * b);
			p.out[u64(batch) * p.o_stride + head * D + d] = i8(f32_to_fixedi8(__fmul_rn(fo, rcp_approx(fs))));
			if (d == 0 && p.l != nullptr) p.l[u64(batch) * p.n_heads + head] = __fadd_rn(lg2_approx(fs), nm);
		}
	}
}

// Second kernel of the split path: one CTA per (head, batch), D threads.
template <u32 D>
__global__ void __launch_bounds__(D)
attn_decode_merge_kernel(const DecodeParams p) {
	u32 const head = blockIdx.x;
	u32 const batch = blockIdx.y;
	u32 const d = threadIdx.x;
	u32 const kv_len = p.kv_lens ? min(p.kv_lens[batch], p.kv_capacity) : p.kv_len;
	u32 const w = p.window;
	u32 const n_att = (kv_len < w ? kv_len : w) + 4u;
	f32 const base_t = f32((1.0 / 64.0) * (D == 128 ? 0.08838834764831845 : D == 64 ? 0.125 : 0.17677669529663687));
	f32 const temp = __fmul_rn(__fmul_rn(base_t, lg2_approx(f32(n_att))), __ldg(p.temperature + head));

	f32 const *src = p.scratch + (u64(batch) * p.n_heads + head) * p.n_splits * (D + 2);
	f32 fm = src[D], fs = src[D + 1], fo = src[d];
	for (u32 s = 1; s < p.n_splits; ++s) {
		f32 const *ps = src + u64(s) * (D + 2);
		f32 const m2 = ps[D];
		f32 const nm = fmaxf(fm, m2);
		f32 const a = ex2_approx(fm - nm), b = ex2_approx(m2 - nm);
		fs = __fmaf_rn(fs, a, ps[D + 1] * b);
		fo = __fmaf_rn(fo, a, ps[d] * b);
		fm = nm;
	}
	i32 sdot = 0;
	uint4 const *qh = reinterpret_cast<uint4 const *>(p.q + u64(batch) * p.q_stride + head * D);
	uint4 const *sk = reinterpret_cast<uint4 const *>(p.sink_k + head * D);
	for (u32 i = 0; i < D / 16; ++i) {
		uint4 a = qh[i], b = __ldg(sk + i);
		sdot = __dp4a(i32(a.x), i32(b.x), sdot);
		sdot = __dp4a(i32(a.y), i32(b.y), sdot);
		sdot = __dp4a(i32(a.z), i32(b.z), sdot);
		sdot = __dp4a(i32(a.w), i32(b.w), sdot);
	}
	f32 const sink_s = __fmul_rn(__int2float_rn(sdot), temp);
	f32 const nm = fmaxf(fm, sink_s);
	f32 const a = ex2_approx(fm - nm), b = ex2_approx(sink_s - nm);
	fs = __fmaf_rn(fs, a, 255.0f * b);
	fo = __fmaf_rn(fo, a, 255.0f * f32(p.sink_v[head * D + d]) * b);
	p.out[u64(batch) * p.o_stride + head * D + d] = i8(f32_to_fixedi8(__fmul_rn(fo, rcp_approx(fs))));
	if (d == 0 && p.l != nullptr) p.l[u64(batch) * p.n_heads + head] = __fadd_rn(lg2_approx(fs), nm);
}

}  // namespace x17
