// Row-wise RMSNorm -> FixedI8, HBM-bound (no tensor cores).
//
// Replaces Rms_norm::kernel (rms_norm.cu:55-113): y = fixedi8(x * rsqrt(mean(x^2) + eps) * 8)
// with x decoded from the reference's e4m3 (cuda/utils_b8.cuh:652-657).  The sum of squares
// is taken in the reference's order (16 consecutive values per lane and 512-value step as an
// fma chain from zero, added to the lane's running sum, then a butterfly over the warp), so
// the result matches the reference kernel bit for bit.
//
// One warp per row, 16-byte loads and stores; the row stays in registers between the two
// passes (up to 8192 columns), so every input byte is read from HBM once.
// Two additional input/output modes: bf16 input, and int8 output with a per-row
// absmax/127 scale instead of the fixed scale 8.
#pragma once

#include "ptx.cuh"

namespace x17 {

enum RmsMode : int {
	RMS_E4M3_FIXED = 0,   // e4m3 in, FixedI8 out (reference form)
	RMS_BF16_FIXED = 1,   // bf16 in, FixedI8 out
	RMS_BF16_ROWSCALE = 2 // bf16 in, int8 out + f32 per-row scale (absmax / 127)
};

struct RmsParams {
	void const *inp;
	i8 *out;
	f32 *row_scale;  // RMS_BF16_ROWSCALE only
	u32 rows, cols;
	u64 inp_stride, out_stride;  // elements
	f32 eps, inv_cols;
};

namespace rms_cfg {
constexpr u32 WARPS = 8;
constexpr u32 THREADS = WARPS * 32;
constexpr u32 MAX_CHUNKS = 16;  // 16-byte chunks per lane held in registers
}  // namespace rms_cfg

// Two e4m3 bytes -> two f32 through the hardware e4m3x2 -> f16x2 converter. For the codes the
// reference's encoder produces (zero and normals, cuda/utils_b8.cuh:636-647) this is exactly
// e4m3_to_bf16 of the reference (utils_b8.cuh:652-657); 0x80 decodes to -0, which squares and
// rounds like +0.
X17_DEV void e4m3x2_to_f32(u32 pair16, f32 &a, f32 &b) {
	u32 h2;
	asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h2) : "r"(pair16));
	asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
		: "=f"(a), "=f"(b)
		: "r"(h2));
}

// rint(clamp(v, -127, 127)) of four values, given as two f32x2 pairs already scaled, packed into
// bytes without the conversion unit: adding 1.5 * 2^23 leaves the rounded integer in the low
// mantissa bits (round half to even, like cvt.rni; valid for |v| < 2^22, here |v| <= 8 * sqrt(cols)),
// a saturating pack clamps to [-128, 127] and a byte-wise max lifts -128 to -127.
X17_DEV u32 pack4_fixedi8_x2(u64 v01, u64 v23) {
	constexpr f32 MAGIC = 12582912.0f;
	constexpr i32 MAGIC_BITS = 0x4B400000;
	u64 const magic2 = pack_f32x2(MAGIC, MAGIC);
	f32 a, b, c, d;
	unpack_f32x2(add_f32x2(v01, magic2), a, b);
	unpack_f32x2(add_f32x2(v23, magic2), c, d);
	i32 const i0 = __float_as_int(a) - MAGIC_BITS, i1 = __float_as_int(b) - MAGIC_BITS;
	i32 const i2 = __float_as_int(c) - MAGIC_BITS, i3 = __float_as_int(d) - MAGIC_BITS;
	u32 hi, packed;
	asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(i3), "r"(i2));
	asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(packed) : "r"(i1), "r"(i0), "r"(hi));
	return __vmaxs4(packed, 0x81818181u);
}

X17_DEV f32 bf16_lo(u32 w) { return __uint_as_float(w << 16); }
X17_DEV f32 bf16_hi(u32 w) { return __uint_as_float(w & 0xFFFF0000u); }

template <int MODE>
X17_DEV void rms_norm_body(RmsParams const &p) {
	using namespace rms_cfg;
	constexpr u32 VALS = MODE == RMS_E4M3_FIXED ? 16 : 8;  // values per 16-byte chunk
	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;
	u32 const row = blockIdx.x * WARPS + warp;
	if (row >= p.rows) return;

	u32 const n_chunks = p.cols / VALS;           // 16-byte chunks per row
	u32 const per_lane = (n_chunks + 31) / 32;    // <= MAX_CHUNKS (checked on the host)
	uint4 const *src = reinterpret_cast<uint4 const *>(
		static_cast<u8 const *>(p.inp) + u64(row) * p.inp_stride * (MODE == RMS_E4M3_FIXED ? 1 : 2));

	uint4 regs[MAX_CHUNKS];
	// all loads of the row are issued before any arithmetic
#pragma unroll
	for (u32 s = 0; s < MAX_CHUNKS; ++s) {
		if (s < per_lane) {
			u32 const ci = s * 32 + lane;
			regs[s] = ci < n_chunks ? __ldg(src + ci) : make_uint4(0, 0, 0, 0);
		}
	}
	f32 local = 0.0f;
	f32 amax = 0.0f;
#pragma unroll
	for (u32 s = 0; s < MAX_CHUNKS; ++s) {
		if (s < per_lane) {
			u32 const wds[4] = {regs[s].x, regs[s].y, regs[s].z, regs[s].w};
			f32 acc = 0.0f;
#pragma unroll
			for (u32 i = 0; i < 4; ++i) {
				if constexpr (MODE == RMS_E4M3_FIXED) {
					f32 x0, x1, x2, x3;
					e4m3x2_to_f32(wds[i] & 0xFFFFu, x0, x1);
					e4m3x2_to_f32(wds[i] >> 16, x2, x3);
					acc = __fmaf_rn(x0, x0, acc);
					acc = __fmaf_rn(x1, x1, acc);
					acc = __fmaf_rn(x2, x2, acc);
					acc = __fmaf_rn(x3, x3, acc);
				} else {
					f32 x0 = bf16_lo(wds[i]), x1 = bf16_hi(wds[i]);
					acc = __fmaf_rn(x0, x0, acc);
					acc = __fmaf_rn(x1, x1, acc);
					amax = fmaxf(amax, fmaxf(fabsf(x0), fabsf(x1)));
				}
			}
			local = __fadd_rn(local, acc);
		}
	}
#pragma unroll
	for (u32 mask = 16; mask > 0; mask >>= 1) {
		local = __fadd_rn(local, __shfl_xor_sync(0xffffffffu, local, mask));
		if constexpr (MODE == RMS_BF16_ROWSCALE) {
			amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
		}
	}
	f32 const rrms = rsqrt_approx(__fmaf_rn(local, p.inv_cols, p.eps));
	f32 mul = rrms;
	if constexpr (MODE == RMS_BF16_ROWSCALE) {
		// scale = absmax(x * rrms) / 127; codes = rint(x * rrms / scale)
		f32 const scale = __fmul_rn(__fmul_rn(amax, rrms), 1.0f / 127.0f);
		if (lane == 0) p.row_scale[row] = scale;
		mul = scale > 0.0f ? __fdiv_rn(rrms, scale) : 0.0f;
	}
	// (x * rrms) * 8 == x * (rrms * 8) exactly: 8 is a power of two
	f32 const mul8 = MODE == RMS_BF16_ROWSCALE ? mul : __fmul_rn(mul, 8.0f);
	u64 const mul8_2 = pack_f32x2(mul8, mul8);  // scaling and rounding run as packed f32x2

	if constexpr (MODE == RMS_E4M3_FIXED) {
		uint4 *dst = reinterpret_cast<uint4 *>(p.out + u64(row) * p.out_stride);
#pragma unroll
		for (u32 s = 0; s < MAX_CHUNKS; ++s) {
			if (s < per_lane) {
				u32 const ci = s * 32 + lane;
				u32 const wds[4] = {regs[s].x, regs[s].y, regs[s].z, regs[s].w};
				u32 o[4];
#pragma unroll
				for (u32 i = 0; i < 4; ++i) {
					f32 x0, x1, x2, x3;
					e4m3x2_to_f32(wds[i] & 0xFFFFu, x0, x1);
					e4m3x2_to_f32(wds[i] >> 16, x2, x3);
					o[i] = pack4_fixedi8_x2(mul_f32x2(pack_f32x2(x0, x1), mul8_2), mul_f32x2(pack_f32x2(x2, x3), mul8_2));
				}
				if (ci < n_chunks) dst[ci] = make_uint4(o[0], o[1], o[2], o[3]);
			}
		}
	} else {
		// 8 bf16 in -> 8 bytes out per chunk
		uint2 *dst = reinterpret_cast<uint2 *>(p.out + u64(row) * p.out_stride);
#pragma unroll
		for (u32 s = 0; s < MAX_CHUNKS; ++s) {
			if (s < per_lane) {
				u32 const ci = s * 32 + lane;
				u32 const wds[4] = {regs[s].x, regs[s].y, regs[s].z, regs[s].w};
				u32 const o0 = pack4_fixedi8_x2(mul_f32x2(pack_f32x2(bf16_lo(wds[0]), bf16_hi(wds[0])), mul8_2),
												mul_f32x2(pack_f32x2(bf16_lo(wds[1]), bf16_hi(wds[1])), mul8_2));
				u32 const o1 = pack4_fixedi8_x2(mul_f32x2(pack_f32x2(bf16_lo(wds[2]), bf16_hi(wds[2])), mul8_2),
												mul_f32x2(pack_f32x2(bf16_lo(wds[3]), bf16_hi(wds[3])), mul8_2));
				if (ci < n_chunks) dst[ci] = make_uint2(o0, o1);
			}
		}
	}
}

// e4m3 -> FixedI8 for rows of up to 4096 columns: the same arithmetic in the same order, with two
// savings in instructions, which (not HBM) bound the general body. The values decoded for the sum
// of squares are kept as f16x2 (exact: every e4m3 value is an f16 value) for the second pass
// instead of being decoded again, and the scaling and the rounding addition run as packed f32x2.
namespace rms_cfg {
constexpr u32 KEEP_CHUNKS = 8;  // 16-byte chunks per lane: 8 x 32 lanes x 16 values = 4096 columns
}
X17_DEV u32 e4m3x2_to_f16x2(u32 pair16) {
	u32 h2;
	// volatile: executed once, not rematerialised from the raw bytes in the second pass
	asm volatile("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h2) : "r"(pair16));
	return h2;
}
X17_DEV void f16x2_to_f32(u32 h2, f32 &a, f32 &b) {
	asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
		: "=f"(a), "=f"(b)
		: "r"(h2));
}
X17_DEV void rms_norm_body_keep(RmsParams const &p) {
	using namespace rms_cfg;
	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;
	u32 const row = blockIdx.x * WARPS + warp;
	if (row >= p.rows) return;
	u32 const n_chunks = p.cols / 16;
	u32 const per_lane = (n_chunks + 31) / 32;  // <= KEEP_CHUNKS (chosen on the host)
	uint4 const *src = reinterpret_cast<uint4 const *>(static_cast<u8 const *>(p.inp) + u64(row) * p.inp_stride);

	uint4 raw[KEEP_CHUNKS];
#pragma unroll
	for (u32 s = 0; s < KEEP_CHUNKS; ++s) {
		if (s < per_lane) {
			u32 const ci = s * 32 + lane;
			raw[s] = ci < n_chunks ? __ldg(src + ci) : make_uint4(0, 0, 0, 0);
		}
	}
	u32 h[KEEP_CHUNKS][8];  // the row as f16x2
	f32 local = 0.0f;
#pragma unroll
	for (u32 s = 0; s < KEEP_CHUNKS; ++s) {
		if (s < per_lane) {
			u32 const wds[4] = {raw[s].x, raw[s].y, raw[s].z, raw[s].w};
			f32 acc = 0.0f;
#pragma unroll
			for (u32 i = 0; i < 4; ++i) {
				h[s][2 * i] = e4m3x2_to_f16x2(wds[i] & 0xFFFFu);
				h[s][2 * i + 1] = e4m3x2_to_f16x2(wds[i] >> 16);
				f32 x0, x1, x2, x3;
				f16x2_to_f32(h[s][2 * i], x0, x1);
				f16x2_to_f32(h[s][2 * i + 1], x2, x3);
				acc = __fmaf_rn(x0, x0, acc);
				acc = __fmaf_rn(x1, x1, acc);
				acc = __fmaf_rn(x2, x2, acc);
				acc = __fmaf_rn(x3, x3, acc);
			}
			local = __fadd_rn(local, acc);
		}
	}
#pragma unroll
	for (u32 mask = 16; mask > 0; mask >>= 1) local = __fadd_rn(local, __shfl_xor_sync(0xffffffffu, local, mask));
	f32 const rrms = rsqrt_approx(__fmaf_rn(local, p.inv_cols, p.eps));
	f32 const mul8 = __fmul_rn(rrms, 8.0f);  // (x * rrms) * 8 == x * (rrms * 8) exactly
	u64 const mul8_2 = pack_f32x2(mul8, mul8);
	uint4 *dst = reinterpret_cast<uint4 *>(p.out + u64(row) * p.out_stride);
#pragma unroll
	for (u32 s = 0; s < KEEP_CHUNKS; ++s) {
		if (s < per_lane) {
			u32 const ci = s * 32 + lane;
			u32 o[4];
#pragma unroll
			for (u32 i = 0; i < 4; ++i) {
				f32 x0, x1, x2, x3;
				f16x2_to_f32(h[s][2 * i], x0, x1);
				f16x2_to_f32(h[s][2 * i + 1], x2, x3);
				o[i] = pack4_fixedi8_x2(mul_f32x2(pack_f32x2(x0, x1), mul8_2), mul_f32x2(pack_f32x2(x2, x3), mul8_2));
			}
			if (ci < n_chunks) dst[ci] = make_uint4(o[0], o[1], o[2], o[3]);
		}
	}
}

__global__ void __launch_bounds__(rms_cfg::THREADS)
rms_norm_keep_kernel(const RmsParams p) {
	rms_norm_body_keep(p);
}

template <int MODE>
__global__ void __launch_bounds__(rms_cfg::THREADS)
rms_norm_kernel(const RmsParams p) {
	rms_norm_body<MODE>(p);
}

}  // namespace x17
