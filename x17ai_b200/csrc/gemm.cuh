// Persistent int8 / e4m3 GEMM for sm_100a with the reference's fused epilogues.
//
//   acc[M, N_raw] = A[M, K] . B[N_raw, K]^T        (both operands K-major, 1 byte per element)
//
// replaces b8::Gemm::run (cuda/gemm_b8.cuh:666-754) and, for e4m3 activations, b16::Gemm::run
// (cuda/gemm_b16.cuh:478-566).  Epilogues replace ScaledMatrixWriter (gemm_b8.cuh:291-339),
// L2NormMatrixWriter (:861-949), GeGluMatrixWriter (:341-441) and ResidualMatrixWriter (:443-622).
//
// Structure (one CTA per SM, 192 threads):
//   warp 0      TMA producer: A tile 128 x 128 B and B tile 256 x 128 B per stage, 128B swizzle
//   warp 1      MMA issuer: tcgen05.mma kind::i8 (or kind::f8f6f4), M128 N256 K32, accumulators
//               in TMEM, two accumulator buffers of 256 columns so the epilogue of tile i
//               overlaps the main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld (thread = row, registers = columns), fused math, 16-byte
//               global stores
// and the same roles as a pair of CTAs on two SMs (gemm_pair_kernel, the library's default): one
// tcgen05.mma.cta_group::2 of M 256, N 256 per K step, issued by the pair's first CTA; each CTA loads its 128 rows
// of A and half of the tile's rows of B and runs the epilogue of its own 128 rows.
// Tiles are walked in groups of row tiles (row tiles fastest inside a group) so that the CTAs running together
// share their A and B rows in L2.
#pragma once

#include "ptx.cuh"

namespace x17 {

enum GemmEpilogue : int {
	EPI_SCALE_I8 = 0,    // c = fixedi8(acc * scale)
	EPI_L2NORM_KV = 1,   // per head [K(D) | V(D)]: K l2-normalised, V scaled; rrms side output
	EPI_GEGLU_E4M3 = 2,  // raw (2j, 2j+1) = (gate, lin) -> e4m3(gelu(gate) * lin)
	EPI_RESID_E4M3 = 3,  // raw (2j, 2j+1) = (gate, value), gated residual -> e4m3
	EPI_RESID_I8 = 4,    // same -> fixedi8
	EPI_RAW_I32 = 5,     // raw 32-bit accumulators (validation of the int32 / f32 accumulation)
	EPI_QKVG = 6,        // fused projection: raw columns [q | kv | g], each segment its own epilogue
};

struct GemmParams {
	u32 m, n_raw, k;
	u32 k_a;  // K extent of A; k == 2 * k_a when B is the split form of int8 weights (A repeats)
	u32 tiles_m, tiles_n;
	void *c;
	u64 c_stride;  // elements of the output type per row
	i8 const *residual;
	u64 resid_stride;
	f32 *rrms;
	u32 rrms_cols;
	u32 head_dim;
	f32 k0, k1, k2, k3, k4;  // epilogue constants, see the epilogue functions
	// EPI_QKVG: raw columns [0, n_q) -> c (q, scale k3); [n_q, n_q + n_kv) -> c2 (kv, L2-norm as
	// EPI_L2NORM_KV with k0..k2, rrms); the rest -> c3 (g, scale k4). Segments are multiples of BN.
	u32 n_q, n_kv;
	void *c2;
	u64 c2_stride;
	void *c3;
	u64 c3_stride;
	u32 *status;
};

namespace gemm_cfg {
constexpr u32 BM = 128;
constexpr u32 BN = 256;
constexpr u32 BK = 128;  // bytes = elements
constexpr u32 STAGES = 4;
constexpr u32 A_BYTES = BM * BK;
constexpr u32 B_BYTES = BN * BK;
constexpr u32 STAGE_BYTES = A_BYTES + B_BYTES;
constexpr u32 THREADS = 192;
constexpr u32 SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr u32 ACC_COLS = 256;

// The CTA-pair form: a cluster of two CTAs on two SMs works on one 256 x 256 tile with tcgen05.mma.cta_group::2.
// Each CTA loads its 128 rows of A and its 128 of the tile's 256 rows of B, so a K block costs a CTA 32 KB instead
// of 48 KB (59 instead of 89 bytes per MMA cycle and SM) and six stages fit where four did.
constexpr u32 PAIR_STAGES = 6;
constexpr u32 PAIR_B_BYTES = (BN / 2) * BK;
constexpr u32 PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr u32 PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
}  // namespace gemm_cfg

// ---- epilogue math ---------------------------------------------------------------------------

// GeGluMatrixWriter::geglu (gemm_b8.cuh:357-372) with math::fast::gelu (utils_core.cuh:426-448):
// k0 = ck3, k1 = ck, k2 = Y_SCALE
X17_DEV f32 geglu_val(f32 gate, f32 lin, GemmParams const &p) {
	f32 x2 = __fmul_rn(gate, gate);
	f32 s = __fmaf_rn(__fmul_rn(p.k0, gate), x2, __fmul_rn(p.k1, gate));
	f32 t = tanh_approx(s);
	f32 yx = __fmul_rn(p.k2, gate);
	f32 g = __fmaf_rn(yx, t, yx);
	return __fmul_rn(g, lin);
}

// ResidualMatrixWriter::residual_gate (gemm_b8.cuh:484-505):
// k0 = 0.5/8, k1 = ln2 * (-INP), k2 = 2*INP, k3 = INP*OUT/2, k4 = INP*INP*OUT
X17_DEV f32 resid_val(f32 gate, f32 new_val, f32 old_val, GemmParams const &p) {
	f32 old_w = __fmaf_rn(p.k0, tanh_approx(__fmul_rn(p.k1, gate)), p.k0);
	f32 line = fmaxf(0.0f, gate);
	if (p.k4 != 1.0f) line = __fmul_rn(line, p.k4);
	f32 e = ex2_approx(-fabsf(__fmul_rn(gate, p.k2)));
	f32 new_w = __fmaf_rn(lg2_approx(__fadd_rn(1.0f, e)), p.k3, line);
	return __fmaf_rn(new_w, new_val, __fmul_rn(old_w, old_val));
}

template <bool F8>
X17_DEV f32 acc_to_f32(u32 bits) {
	if constexpr (F8) {
		return __uint_as_float(bits);
	} else {
		return __int2float_rn(static_cast<i32>(bits));
	}
}

// ---- kernel ----------------------------------------------------------------------------------

// Tile order of the persistent loop: groups of GROUP_M row tiles; inside a group the row tiles run
// fastest and every column tile is visited before the next group starts. The tiles in flight on
// the 148 CTAs then cover a near-square patch of C (16 row tiles x ~9 column tiles) instead of
// every row tile of one column tile, so a wave touches far fewer distinct rows of A and B and
// they stay in L2 while the wave needs them.
template <u32 GROUP_M = 16>
X17_DEV void tile_origin(u32 t, u32 tiles_m, u32 tiles_n, u32 &m_idx, u32 &n_idx) {
	u32 const per_group = GROUP_M * tiles_n;
	u32 const g = t / per_group;
	u32 const first_m = g * GROUP_M;
	u32 const rows = min(GROUP_M, tiles_m - first_m);   // the last group may be short
	u32 const r = t - g * per_group;
	m_idx = first_m + r % rows;
	n_idx = r / rows;
}

// The kernel proper. The tensor maps are reached through pointers: kernel parameters for the library's
// entry points, maps patched on the device for the kernel objects (kernel_objects/gemm.cu). The loop
// strides over the tiles by `n_ctas`, this CTA being number `cta` of them, whatever the grid's shape.
// PAIR: `cta` / `n_ctas` count clusters of two CTAs, a tile is 256 x 256, and this CTA (rank 0 or 1 of its cluster)
// owns rows [128 * rank, +128) of it. Rank 0 issues the MMAs for both; both load, both run the epilogue of their rows.
template <int EPI, bool F8, bool PAIR = false>
X17_DEV void gemm_body(CUtensorMap const *tm_a_ptr, CUtensorMap const *tm_b_ptr, GemmParams const &p, u32 cta,
					   u32 n_ctas) {
	using namespace gemm_cfg;
	constexpr u32 STAGES = PAIR ? PAIR_STAGES : gemm_cfg::STAGES;
	constexpr u32 STAGE_BYTES = PAIR ? PAIR_STAGE_BYTES : gemm_cfg::STAGE_BYTES;
	constexpr u32 TILE_M = PAIR ? 2 * BM : BM;
	u32 const rank = PAIR ? cluster_cta_rank() : 0u;   // 0: the CTA that issues the MMAs
	extern __shared__ u8 smem_raw[];
	u32 const smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	u8 *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

	u32 const bar_base = smem_base + STAGES * STAGE_BYTES;
	auto full_bar = [&](u32 s) { return bar_base + 8 * s; };
	auto empty_bar = [&](u32 s) { return bar_base + 8 * (STAGES + s); };
	auto acc_full_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + b); };
	auto acc_empty_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + 2 + b); };
	u32 const tmem_slot = bar_base + 8 * (2 * STAGES + 4);
	volatile u32 *const tmem_slot_gen =
		reinterpret_cast<volatile u32 *>(smem_gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
	volatile u32 *const abort_flag = tmem_slot_gen + 1;
	WaitCtx const ctx{abort_flag, p.status};

	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;

	if (threadIdx.x == 0) {
		for (u32 s = 0; s < STAGES; ++s) {
			mbar_init(full_bar(s), 1);
			mbar_init(empty_bar(s), 1);
		}
		for (u32 b = 0; b < 2; ++b) {
			mbar_init(acc_full_bar(b), 1);
			mbar_init(acc_empty_bar(b), PAIR ? 8 : 4);  // one arrive per epilogue warp (of both CTAs: rank 0 collects)
		}
		*abort_flag = 0;
		mbar_fence_init();
	}
	if (warp == 1) {
		if constexpr (PAIR) {
			tmem_alloc_pair(tmem_slot, 512);
			tmem_relinquish_pair();
		} else {
			tmem_alloc(tmem_slot, 512);
			tmem_relinquish();
		}
	}
	tc_fence_before();
	__syncthreads();
	if constexpr (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything signals them
	tc_fence_after();
	u32 const tmem_base = *tmem_slot_gen;

	u32 const tiles_m = PAIR ? (p.m + TILE_M - 1) / TILE_M : p.tiles_m;
	u32 const n_tiles = tiles_m * p.tiles_n;
	u32 const k_blocks = p.k / BK;

	if (warp == 0) {
		// ---------------- TMA producer ----------------
		if (elect_one()) {
			tma_prefetch_desc(tm_a_ptr);
			tma_prefetch_desc(tm_b_ptr);
			u32 it = 0;
			bool ok = true;
			for (u32 t = cta; t < n_tiles && ok; t += n_ctas) {
				u32 tm, tn;
				tile_origin<16>(t, tiles_m, p.tiles_n, tm, tn);
				i32 const m0 = i32(tm * TILE_M + rank * BM);
				i32 const n0 = i32(tn * BN + (PAIR ? rank * (BN / 2) : 0u));
				for (u32 kb = 0; kb < k_blocks; ++kb, ++it) {
					u32 const s = it % STAGES;
					u32 const ph = (it / STAGES) & 1;
					if (!mbar_wait(empty_bar(s), ph ^ 1, ctx, ST_WAIT_STAGE_EMPTY, s)) {
						ok = false;
						break;
					}
					u32 const a_dst = smem_base + s * STAGE_BYTES;
					if constexpr (PAIR) {
						// both CTAs' bytes are counted on rank 0's barrier, where the MMA issuer waits
						u32 const bar0 = map_to_cta(full_bar(s), 0);
						if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
						tma_load_2d_pair(a_dst, tm_a_ptr, bar0, i32((kb * BK) % p.k_a), m0);
						tma_load_2d_pair(a_dst + A_BYTES, tm_b_ptr, bar0, i32(kb * BK), n0);
					} else {
						mbar_expect_tx(full_bar(s), STAGE_BYTES);
						tma_load_2d(a_dst, tm_a_ptr, full_bar(s), i32((kb * BK) % p.k_a), m0);
						tma_load_2d(a_dst + A_BYTES, tm_b_ptr, full_bar(s), i32(kb * BK), n0);
					}
				}
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer ----------------
		if (rank == 0 && elect_one()) {
			constexpr u32 idesc = F8 ? make_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 0, 0, TILE_M, BN)
									 : make_idesc(DFMT_S32, FMT_S8, FMT_S8, 0, 0, TILE_M, BN);
			// a commit of the pair form arrives on one barrier: this CTA's and, separately, the peer's copy of it
			auto commit = [&](u32 bar) {
				if constexpr (PAIR) {
					tc_commit_pair(map_to_cta(bar, 0));
					tc_commit_pair(map_to_cta(bar, 1));
				} else {
					tc_commit(bar);
				}
			};
			u32 it = 0;
			u32 local_tile = 0;
			bool ok = true;
			for (u32 t = cta; t < n_tiles && ok; t += n_ctas, ++local_tile) {
				u32 const buf = local_tile & 1;
				u32 const acc_ph = (local_tile >> 1) & 1;
				if (!mbar_wait(acc_empty_bar(buf), acc_ph ^ 1, ctx, ST_WAIT_ACC_EMPTY, buf)) {
					ok = false;
					break;
				}
				tc_fence_after();
				u32 const d_tmem = tmem_base + buf * ACC_COLS;
				for (u32 kb = 0; kb < k_blocks; ++kb, ++it) {
					u32 const s = it % STAGES;
					u32 const ph = (it / STAGES) & 1;
					if (!mbar_wait(full_bar(s), ph, ctx, ST_WAIT_TMA_FULL, s)) {
						ok = false;
						break;
					}
					tc_fence_after();
					u32 const a_addr = smem_base + s * STAGE_BYTES;
					u64 const adesc = make_smem_desc(a_addr, 128);
					u64 const bdesc = make_smem_desc(a_addr + A_BYTES, 128);
#pragma unroll
					for (u32 ks = 0; ks < BK / 32; ++ks) {
						u32 const accumulate = (kb | ks) != 0 ? 1u : 0u;
						// advance 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
						if constexpr (PAIR) {
							if constexpr (F8) mma_f8_ss_pair(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, accumulate);
							else mma_i8_ss_pair(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, accumulate);
						} else if constexpr (F8) {
							mma_f8_ss(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, accumulate);
						} else {
							mma_i8_ss(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, accumulate);
						}
					}
					commit(empty_bar(s));  // frees the stage (in both CTAs) once these MMAs have read it
				}
				if (ok) commit(acc_full_bar(buf));
			}
		}
	} else {
		// ---------------- epilogue warps ----------------
		u32 const quarter = warp & 3;  // TMEM lanes this warp may touch: 32*quarter .. +31
		u32 const row_in_tile = quarter * 32 + lane;
		u32 local_tile = 0;
		bool ok = true;
		for (u32 t = cta; t < n_tiles && ok; t += n_ctas, ++local_tile) {
			u32 const buf = local_tile & 1;
			u32 const acc_ph = (local_tile >> 1) & 1;
			u32 tm, tn;
			tile_origin<16>(t, tiles_m, p.tiles_n, tm, tn);
			u32 const m0 = tm * TILE_M + rank * BM;
			u32 const n0 = tn * BN;
			if (!mbar_wait_warp(acc_full_bar(buf), acc_ph, ctx, ST_WAIT_ACC_FULL, buf)) {
				ok = false;
				break;
			}
			tc_fence_after();
			u32 const row = m0 + row_in_tile;
			bool const row_ok = row < p.m;
			u32 const t_base = tmem_base + buf * ACC_COLS + ((quarter * 32u) << 16);

			if constexpr (EPI == EPI_QKVG) {
				if (n0 < p.n_q || n0 >= p.n_q + p.n_kv) {
					// q or g segment: plain scale -> FixedI8 (ScaledMatrixWriter, gemm_b8.cuh:291-339)
					bool const is_q = n0 < p.n_q;
					i8 *const base = static_cast<i8 *>(is_q ? p.c : p.c3);
					u64 const stride = is_q ? p.c_stride : p.c3_stride;
					u32 const col0 = is_q ? n0 : n0 - p.n_q - p.n_kv;
					u32 const width = is_q ? p.n_q : p.n_raw - p.n_q - p.n_kv;
					f32 const sc = is_q ? p.k3 : p.k4;
					for (u32 c = 0; c < BN && col0 + c < width; c += 32) {
						u32 r[32];
						tmem_ld_32x32b_x32(t_base + c, r);
						tmem_wait_ld();
						u32 w[8];
#pragma unroll
						for (u32 i = 0; i < 8; ++i) {
							w[i] = pack4(u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 0]), sc))),
										 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 1]), sc))),
										 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 2]), sc))),
										 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 3]), sc))));
						}
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(base + u64(row) * stride + col0 + c);
							dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
							dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
						}
					}
				} else {
					// kv segment: per head [K(D) | V(D)] (L2NormMatrixWriter, gemm_b8.cuh:861-949)
					u32 const d = p.head_dim;
					u32 const col0 = n0 - p.n_q;
					for (u32 h0 = 0; h0 < BN && col0 + h0 < p.n_kv; h0 += 2 * d) {
						f32 ssum = 0.0f;
						for (u32 c = 0; c < d; c += 32) {
							u32 r[32];
							tmem_ld_32x32b_x32(t_base + h0 + c, r);
							tmem_wait_ld();
#pragma unroll
							for (u32 i = 0; i < 32; ++i) {
								f32 f = acc_to_f32<F8>(r[i]);
								ssum = __fmaf_rn(f, f, ssum);
							}
						}
						f32 const kscale = __fmul_rn(rsqrt_approx(__fadd_rn(ssum, p.k0)), p.k1);
						if (row_ok) p.rrms[u64(row) * p.rrms_cols + (col0 + h0) / (2 * d)] = kscale;
						for (u32 c = 0; c < 2 * d; c += 32) {
							u32 r[32];
							tmem_ld_32x32b_x32(t_base + h0 + c, r);
							tmem_wait_ld();
							f32 const sc = c < d ? kscale : p.k2;
							u32 w[8];
#pragma unroll
							for (u32 i = 0; i < 8; ++i) {
								w[i] = pack4(u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 0]), sc))),
											 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 1]), sc))),
											 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 2]), sc))),
											 u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 3]), sc))));
							}
							if (row_ok) {
								uint4 *dst = reinterpret_cast<uint4 *>(
									static_cast<i8 *>(p.c2) + u64(row) * p.c2_stride + col0 + h0 + c);
								dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
								dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
							}
						}
					}
				}
			} else if constexpr (EPI == EPI_L2NORM_KV) {
				// raw columns of a head: [K(D) | V(D)]; the tile holds BN / 2D whole heads.
				// k0 = eps, k1 = HEAD_SCALE (= out_scale * sqrt(D)), k2 = SEP_SCALE (= inp * out)
				u32 const d = p.head_dim;
				for (u32 h0 = 0; h0 < BN && n0 + h0 < p.n_raw; h0 += 2 * d) {
					f32 ssum = 0.0f;
					for (u32 c = 0; c < d; c += 32) {
						u32 r[32];
						tmem_ld_32x32b_x32(t_base + h0 + c, r);
						tmem_wait_ld();
#pragma unroll
						for (u32 i = 0; i < 32; ++i) {
							f32 f = acc_to_f32<F8>(r[i]);
							ssum = __fmaf_rn(f, f, ssum);
						}
					}
					f32 const kscale = __fmul_rn(rsqrt_approx(__fadd_rn(ssum, p.k0)), p.k1);
					if (row_ok) {
						p.rrms[u64(row) * p.rrms_cols + (n0 + h0) / (2 * d)] = kscale;
					}
					for (u32 c = 0; c < 2 * d; c += 32) {
						u32 r[32];
						tmem_ld_32x32b_x32(t_base + h0 + c, r);
						tmem_wait_ld();
						f32 const sc = c < d ? kscale : p.k2;
						u32 w[8];
#pragma unroll
						for (u32 i = 0; i < 8; ++i) {
							w[i] = pack4(
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 0]), sc))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 1]), sc))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 2]), sc))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 3]), sc))));
						}
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(
								static_cast<i8 *>(p.c) + u64(row) * p.c_stride + n0 + h0 + c);
							dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
							dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
						}
					}
				}
			} else {
				for (u32 c = 0; c < BN; c += 32) {
					if (n0 + c >= p.n_raw) break;  // uniform across the CTA
					u32 r[32];
					tmem_ld_32x32b_x32(t_base + c, r);
					tmem_wait_ld();
					if constexpr (EPI == EPI_SCALE_I8) {
						// k0 = f32(inp_scale * out_scale)
						u32 w[8];
#pragma unroll
						for (u32 i = 0; i < 8; ++i) {
							w[i] = pack4(
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 0]), p.k0))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 1]), p.k0))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 2]), p.k0))),
								u32(f32_to_fixedi8(__fmul_rn(acc_to_f32<F8>(r[4 * i + 3]), p.k0))));
						}
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(
								static_cast<i8 *>(p.c) + u64(row) * p.c_stride + n0 + c);
							dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
							dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
						}
					} else if constexpr (EPI == EPI_RAW_I32) {
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(
								static_cast<u32 *>(p.c) + u64(row) * p.c_stride + n0 + c);
#pragma unroll
							for (u32 i = 0; i < 8; ++i) {
								dst[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
							}
						}
					} else if constexpr (EPI == EPI_GEGLU_E4M3) {
						u32 w[4];
#pragma unroll
						for (u32 i = 0; i < 4; ++i) {
							u32 b[4];
#pragma unroll
							for (u32 j = 0; j < 4; ++j) {
								f32 gate = acc_to_f32<F8>(r[8 * i + 2 * j]);
								f32 lin = acc_to_f32<F8>(r[8 * i + 2 * j + 1]);
								b[j] = f32_to_e4m3(geglu_val(gate, lin, p));
							}
							w[i] = pack4(b[0], b[1], b[2], b[3]);
						}
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(
								static_cast<u8 *>(p.c) + u64(row) * p.c_stride + (n0 + c) / 2);
							dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
						}
					} else {  // EPI_RESID_E4M3 / EPI_RESID_I8
						uint4 res = make_uint4(0, 0, 0, 0);
						if (row_ok) {
							res = *reinterpret_cast<uint4 const *>(
								p.residual + u64(row) * p.resid_stride + (n0 + c) / 2);
						}
						u32 const rw[4] = {res.x, res.y, res.z, res.w};
						u32 w[4];
#pragma unroll
						for (u32 i = 0; i < 4; ++i) {
							u32 b[4];
#pragma unroll
							for (u32 j = 0; j < 4; ++j) {
								f32 gate = acc_to_f32<F8>(r[8 * i + 2 * j]);
								f32 val = acc_to_f32<F8>(r[8 * i + 2 * j + 1]);
								i32 code = static_cast<i8>((rw[i] >> (8 * j)) & 0xFFu);
								f32 v = resid_val(gate, val, f32(code), p);
								if constexpr (EPI == EPI_RESID_E4M3) {
									b[j] = f32_to_e4m3(v);
								} else {
									b[j] = u32(f32_to_fixedi8(v));
								}
							}
							w[i] = pack4(b[0], b[1], b[2], b[3]);
						}
						if (row_ok) {
							uint4 *dst = reinterpret_cast<uint4 *>(
								static_cast<u8 *>(p.c) + u64(row) * p.c_stride + (n0 + c) / 2);
							dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
						}
					}
				}
			}
			// this warp is done reading the accumulator buffer
			tc_fence_before();
			__syncwarp();
			if (lane == 0) {
				if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(acc_empty_bar(buf), 0));
				else mbar_arrive(acc_empty_bar(buf));
			}
		}
	}

	// teardown: every role falls through to here, also after a wait that gave up
	tc_fence_before();
	__syncthreads();
	if constexpr (PAIR) cluster_sync_all();   // the peer no longer reads this CTA's tiles nor signals its barriers
	if (warp == 1) {
		__syncwarp();
		tc_fence_after();
		if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512);
		else tmem_dealloc(tmem_base, 512);
	}
}

template <int EPI, bool F8>
__global__ void __launch_bounds__(gemm_cfg::THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
			const GemmParams p) {
	gemm_body<EPI, F8>(&tm_a, &tm_b, p, blockIdx.x, gridDim.x);
}

// The CTA-pair form: launched with an even grid; consecutive CTAs form a cluster. The B tensor map's box is the
// half tile (BN / 2 rows).
template <int EPI, bool F8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm_cfg::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
				 const GemmParams p) {
	gemm_body<EPI, F8, true>(&tm_a, &tm_b, p, blockIdx.x / 2, gridDim.x / 2);
}

}  // namespace x17
