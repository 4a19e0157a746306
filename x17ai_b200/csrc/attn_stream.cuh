// int8 sliding-window attention forward for sm_100a, persistent form: one CTA per SM walks a list
// of items, an item being a run of consecutive 128-query tiles of one (batch, head).
//
// Same arithmetic as attn.cuh (AttnForward<...>::run, cuda/attn_fwd_i8.cuh:368-619, with the row
// maximum found before the probabilities are quantised), arranged so that nothing waits on a
// hand-over that another role could have finished earlier:
//
//   * the probabilities stay in tensor memory: a row thread reads its 32 score columns with
//     tcgen05.ld, writes the 32 u8 probabilities back over the first 8 of those columns with
//     tcgen05.st, and P.V takes its A operand from there (no shared-memory P tile, no proxy
//     fence, half the shared-memory reads of the MMA);
//   * the scores of the probability sweep are double-buffered (columns [0,128) and [128,256)),
//     so Q.K^T of key tile t+1 is finished long before the rows are done with tile t;
//   * the maximum sweep of query tile j+1 runs inside the probability sweep of query tile j:
//     for every key tile in shared memory the tensor core also produces Q[j+1].K^T into columns
//     [256,384), and the same row threads reduce it with integer max between their exp2
//     instructions (the max scan needs the ALU pipe, the probabilities the MUFU pipe). Only
//     the first query tile of an item pays for a maximum sweep of its own;
//   * the epilogue of query tile j (O in columns [384,384+D)) and the exchange of the row
//     maxima run while the tensor core already works on the first key tiles of tile j+1.
//
// 576 threads: warp 0 TMA producer (three Q buffers, a ring of K and V tiles), warp 1 MMA
// issuer, warps 2..17 four threads per query row (32 score columns and D/4 output columns each):
// a scheduler needs about four such warps to keep its pipes busy (one warp alone issues an
// instruction every 2.6 cycles at best).
// No load uses cluster multicast; every wait is bounded.
#pragma once

#include "attn.cuh"

namespace x17 {

// How a launch is cut into items (filled in by the host).
struct AttnItemPlan {
	u32 n_qtiles;        // ceil(seq_len / 128)
	u32 tiles_per_item;  // consecutive query tiles of one item
	u32 chunks;          // items per (batch, head) = ceil(n_qtiles / tiles_per_item)
	u32 n_items;         // batch * n_heads * chunks
};

namespace attn_stream_cfg {
constexpr u32 BQ = 128;
constexpr u32 BKV = 128;
constexpr u32 STAGES = 8;     // ring entries of one K or V tile each
constexpr u32 Q_BUFFERS = 3;  // Q of the tile in its probability sweep, of the next (maximum sweep), of the one after
constexpr u32 ROW_WARPS = 16;
constexpr u32 ROW_THREADS = ROW_WARPS * 32;
constexpr u32 THREADS = 64 + ROW_THREADS;
constexpr u32 TMEM_COLS = 512;
constexpr u32 S2_COL = 0;    // two score buffers of the probability sweep, 128 columns each
constexpr u32 S1_COL = 256;  // score buffer of the maximum sweep
constexpr u32 O_COL = 384;
constexpr u32 XCHG_WORDS = 2 * 3 * 4 * BQ;  // two parities x (max candidate, partial sum, partial sink dot) x 4 x rows
constexpr u32 SVF_BYTES = 4 * 2 * 128 * 4;  // per row quarter: the sink values of the current and the previous item's head as f32
constexpr u32 SK_BYTES = Q_BUFFERS * 128;   // the head's sink key beside every Q buffer (loaded with it)
constexpr u32 N_BARRIERS = 2 * STAGES + 2 * Q_BUFFERS + 12;
template <u32 D>
constexpr u32 smem_bytes() {
	return Q_BUFFERS * BQ * D + STAGES * BKV * D + XCHG_WORDS * 4 + SVF_BYTES + SK_BYTES + 512 + 1024;
}
}  // namespace attn_stream_cfg

X17_DEV void tmem_st_32x32b_x8(u32 taddr, u32 const (&r)[8]) {
	asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
				 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
				 : "memory");
}
X17_DEV void tmem_wait_st() {
	asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
X17_DEV void tmem_ld_32x32b_x8(u32 taddr, u32 (&r)[8]) {
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
				 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
				 : "r"(taddr)
				 : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16), completing on an
// mbarrier like a tiled load; no multicast.
X17_DEV void bulk_load(u32 dst, void const *src, u32 bytes, u32 bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
				 "l"(src), "r"(bytes), "r"(bar)
				 : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (lane = row, one
// 32-bit column = four consecutive 8-bit K elements); issued by ONE thread.
X17_DEV void mma_i8_ts(u32 d_tmem, u32 a_tmem, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
X17_DEV void mma_f8_ts(u32 d_tmem, u32 a_tmem, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}

// first key tile that any row of query tile j can see
X17_DEV u32 attn_first_tile(u32 j, u32 w) {
	u32 const q0 = j * attn_stream_cfg::BQ;
	return (w == 0xFFFFFFFFu || q0 < w) ? 0u : (q0 - w) / attn_stream_cfg::BKV;
}

// One pass = the probability sweep of query tile jq2 (if `s2`) together with the maximum sweep
// of query tile jq1 = jq2 + 1 (if `s1`) over the key tiles t_lo..t_hi. Every role derives the
// same sequence of passes and tiles from the item alone.
struct AttnPass {
	u32 jq2, jq1;
	bool s2, s1;
	u32 t_lo, t_hi;
	u32 t1_lo;  // first key tile of the maximum sweep
};
X17_DEV AttnPass attn_pass(u32 j0, u32 j1, u32 pp, u32 w) {
	AttnPass a;
	a.jq1 = j0 + pp;
	a.jq2 = a.jq1 - 1;  // only meaningful when s2
	a.s2 = pp >= 1;
	a.s1 = a.jq1 < j1;
	a.t1_lo = a.s1 ? attn_first_tile(a.jq1, w) : 0u;
	a.t_lo = a.s2 ? attn_first_tile(a.jq2, w) : a.t1_lo;
	a.t_hi = a.s1 ? a.jq1 : a.jq2;
	return a;
}

template <u32 D, bool DEBUG, bool FP8PV = false>
__global__ void __launch_bounds__(attn_stream_cfg::THREADS, 1)
attn_fwd_stream_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
					   const AttnParams p, const AttnItemPlan plan) {
	using namespace attn_stream_cfg;
	using attn_cfg::MAGIC;
	static_assert(D == 32 || D == 64 || D == 128, "head_dim must be 32, 64 or 128");
	constexpr u32 TILE_BYTES = BKV * D;
	constexpr u32 Q_BYTES = BQ * D;

	extern __shared__ u8 smem_raw[];
	u32 const smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	u8 *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

	u32 const s_q = smem_base;
	u32 const s_ring = s_q + Q_BUFFERS * Q_BYTES;
	constexpr u32 XCHG_OFF = Q_BUFFERS * Q_BYTES + STAGES * TILE_BYTES;
	constexpr u32 SVF_OFF = XCHG_OFF + XCHG_WORDS * 4;
	constexpr u32 SK_OFF = SVF_OFF + SVF_BYTES;
	constexpr u32 BAR_OFF = SK_OFF + SK_BYTES;
	u32 *const xchg = reinterpret_cast<u32 *>(smem_gen + XCHG_OFF);
	f32 *const svf_all = reinterpret_cast<f32 *>(smem_gen + SVF_OFF);
	u32 const bar_base = smem_base + BAR_OFF;
	auto full_bar = [&](u32 s) { return bar_base + 8 * s; };
	auto empty_bar = [&](u32 s) { return bar_base + 8 * (STAGES + s); };
	auto q_full_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + b); };
	auto q_empty_bar = [&](u32 b) { return bar_base + 8 * (2 * STAGES + Q_BUFFERS + b); };
	constexpr u32 B0 = 2 * STAGES + 2 * Q_BUFFERS;
	auto s2_full_bar = [&](u32 b) { return bar_base + 8 * (B0 + b); };
	u32 const s1_full_bar = bar_base + 8 * (B0 + 11);
	auto p_ready_bar = [&](u32 b) { return bar_base + 8 * (B0 + 2 + b); };
	u32 const s1_read_bar = bar_base + 8 * (B0 + 8);
	u32 const o_full_bar = bar_base + 8 * (B0 + 9);
	u32 const o_read_bar = bar_base + 8 * (B0 + 10);
	auto xchg_bar = [&](u32 q) { return bar_base + 8 * (B0 + 4 + q); };  // one per row quarter (4 warps share a row)
	u32 const tmem_slot = bar_base + 8 * N_BARRIERS;
	volatile u32 *const tmem_slot_gen = reinterpret_cast<volatile u32 *>(smem_gen + BAR_OFF + 8 * N_BARRIERS);
	volatile u32 *const abort_flag = tmem_slot_gen + 1;
	WaitCtx const ctx{abort_flag, p.status};

	u32 const warp = threadIdx.x >> 5;
	u32 const lane = threadIdx.x & 31;
	u32 const w = p.window;

	if (threadIdx.x == 0) {
		for (u32 s = 0; s < STAGES; ++s) {
			mbar_init(full_bar(s), 1);
			mbar_init(empty_bar(s), 1);
		}
		for (u32 b = 0; b < Q_BUFFERS; ++b) {
			mbar_init(q_full_bar(b), 1);
			mbar_init(q_empty_bar(b), 1);
		}
		for (u32 b = 0; b < 2; ++b) {
			mbar_init(s2_full_bar(b), 1);
			mbar_init(p_ready_bar(b), ROW_WARPS);
		}
		mbar_init(s1_full_bar, 1);
		mbar_init(s1_read_bar, ROW_WARPS);
		mbar_init(o_full_bar, 1);
		mbar_init(o_read_bar, ROW_WARPS);
		for (u32 q = 0; q < 4; ++q) mbar_init(xchg_bar(q), ROW_WARPS / 4);
		*abort_flag = 0;
		mbar_fence_init();
	}
	if (warp == 1) {
		tmem_alloc(tmem_slot, TMEM_COLS);
		tmem_relinquish();
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	u32 const tmem_base = *tmem_slot_gen;

	// item -> (batch, head, first and one-past-last query tile)
	// the last chunks of a sequence come first: with a window the first chunk is the lightest (its
	// queries see fewer keys), without one the cost grows with the position, and the light items
	// fill the end of the launch
	auto decode_item = [&](u32 item, u32 &batch, u32 &head, u32 &j0, u32 &j1) {
		u32 const n_bh = plan.n_items / plan.chunks;
		u32 const c = plan.chunks - 1 - item / n_bh;
		u32 const bh = item % n_bh;
		head = bh % p.n_heads;
		batch = bh / p.n_heads;
		j0 = c * plan.tiles_per_item;
		j1 = min(j0 + plan.tiles_per_item, plan.n_qtiles);
	};

	if (warp == 0) {
		// ---------------- TMA producer ----------------
		if (elect_one()) {
			tma_prefetch_desc(&tm_q);
			tma_prefetch_desc(&tm_kv);
			u32 it = 0;  // ring entries issued
			u32 nq = 0;  // Q tiles issued
			bool ok = true;
			#pragma unroll 1
			for (u32 item = blockIdx.x; item < plan.n_items && ok; item += gridDim.x) {
				u32 batch, head, j0, j1;
				decode_item(item, batch, head, j0, j1);
				auto load_q = [&](u32 j) -> bool {
					u32 const b = nq % Q_BUFFERS;
					u32 const ph = (nq / Q_BUFFERS) & 1;
					if (!mbar_wait(q_empty_bar(b), ph ^ 1, ctx, ST_WAIT_Q_FULL, 0x100u + b)) return false;
					mbar_expect_tx(q_full_bar(b), Q_BYTES + D);
					tma_load_3d(s_q + b * Q_BYTES, &tm_q, q_full_bar(b), i32(head * D), i32(j * BQ), i32(batch));
					bulk_load(smem_base + SK_OFF + b * 128, p.sink_k + head * D, D, q_full_bar(b));
					++nq;
					return true;
				};
				// one ring entry: the K (part 0) or V (part 1) tile of key tile t
				auto load_kv = [&](u32 t, u32 part) -> bool {
					u32 const s = it % STAGES;
					u32 const ph = (it / STAGES) & 1;
					if (!mbar_wait(empty_bar(s), ph ^ 1, ctx, ST_WAIT_STAGE_EMPTY, s)) return false;
					mbar_expect_tx(full_bar(s), TILE_BYTES);
					tma_load_3d(s_ring + s * TILE_BYTES, &tm_kv, full_bar(s), i32(2 * head * D + part * D),
								i32(t * BKV), i32(batch));
					++it;
					return true;
				};
				ok = load_q(j0);
				#pragma unroll 1
				for (u32 pp = 0; pp <= j1 - j0 && ok; ++pp) {
					AttnPass const a = attn_pass(j0, j1, pp, w);
					if (a.jq1 + 1 < j1) ok = load_q(a.jq1 + 1);
					// in the order the MMA thread consumes them: K[t], then V[t-1]
					#pragma unroll 1
					for (u32 t = a.t_lo; t <= a.t_hi && ok; ++t) {
						ok = load_kv(t, 0);
						if (ok && a.s2 && t > a.t_lo && t - 1 <= a.jq2) ok = load_kv(t - 1, 1);
					}
					if (ok && a.s2 && a.t_hi == a.jq2) ok = load_kv(a.jq2, 1);
				}
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer ----------------
		if (elect_one()) {
			constexpr u32 idesc_qk = make_idesc(DFMT_S32, FMT_S8, FMT_S8, 0, 0, BQ, BKV);
			constexpr u32 idesc_pv = FP8PV ? make_idesc(DFMT_F32, FMT_E4M3, FMT_E4M3, 0, 1, BQ, D)
										   : make_idesc(DFMT_S32, FMT_U8, FMT_S8, 0, 1, BQ, D);
			u32 const o_tmem = tmem_base + O_COL;
			u64 const ring_desc = make_smem_desc(s_ring, D);  // + stage * (TILE_BYTES >> 4)
			u32 it = 0;       // ring entries consumed
			u32 nq_base = 0;  // Q tiles of earlier items
			u32 n2 = 0;       // score tiles of the probability sweep issued
			u32 npv = 0;      // P.V tiles issued
			u32 n1 = 0;       // score tiles of the maximum sweep issued
			u32 no = 0;       // probability sweeps finished
			bool ok = true;
			#pragma unroll 1
			for (u32 item = blockIdx.x; item < plan.n_items && ok; item += gridDim.x) {
				u32 batch, head, j0, j1;
				decode_item(item, batch, head, j0, j1);
				#pragma unroll 1
				for (u32 pp = 0; pp <= j1 - j0 && ok; ++pp) {
					AttnPass const a = attn_pass(j0, j1, pp, w);
					u32 const nq1 = nq_base + pp;  // Q index of jq1; jq2 is nq1 - 1
					u64 q1_desc = 0, q2_desc = 0;
					if (a.s1) {
						u32 const b = nq1 % Q_BUFFERS;
						ok = mbar_wait(q_full_bar(b), (nq1 / Q_BUFFERS) & 1, ctx, ST_WAIT_Q_FULL, b);
						if (!ok) break;
						tc_fence_after();
						q1_desc = make_smem_desc(s_q + b * Q_BYTES, D);
					}
					if (a.s2) q2_desc = make_smem_desc(s_q + ((nq1 - 1) % Q_BUFFERS) * Q_BYTES, D);

					// O += P.V of the oldest probability tile not yet multiplied
					bool first_pv = true;
					auto issue_pv = [&]() -> bool {
						u32 const b = npv & 1;
						if (!mbar_wait(p_ready_bar(b), (npv >> 1) & 1, ctx, ST_WAIT_S_DONE, 0x100u)) return false;
						u32 const s = it % STAGES;
						if (!mbar_wait(full_bar(s), (it / STAGES) & 1, ctx, ST_WAIT_TMA_FULL, s)) return false;
						if (first_pv && no > 0) {  // the previous tile's O has been read
							if (!mbar_wait(o_read_bar, (no - 1) & 1, ctx, ST_WAIT_O_FULL, 0x200u)) return false;
						}
						tc_fence_after();
						u64 const bdesc = ring_desc + u64(s * (TILE_BYTES >> 4));
						u32 const a_tmem = tmem_base + S2_COL + b * BKV;
	#pragma unroll
						for (u32 ks = 0; ks < BKV / 32; ++ks) {
							// A: the 32 probabilities of k-step ks sit in columns 32 ks .. 32 ks + 7 of the score
							// buffer; B (MN-major): +32 key rows of D bytes each
							u32 const acc = (!first_pv || ks != 0) ? 1u : 0u;
							u32 const a_ks = a_tmem + 32 * ks;
							if constexpr (FP8PV) mma_f8_ts(o_tmem, a_ks, bdesc + ((32 * D) >> 4) * ks, idesc_pv, acc);
							else mma_i8_ts(o_tmem, a_ks, bdesc + ((32 * D) >> 4) * ks, idesc_pv, acc);
						}
						tc_commit(empty_bar(s));
						++it;
						++npv;
						first_pv = false;
						return true;
					};

					#pragma unroll 1
					for (u32 t = a.t_lo; t <= a.t_hi && ok; ++t) {
						u32 const s = it % STAGES;
						ok = mbar_wait(full_bar(s), (it / STAGES) & 1, ctx, ST_WAIT_TMA_FULL, s);
						if (!ok) break;
						tc_fence_after();
						u64 const bdesc = ring_desc + u64(s * (TILE_BYTES >> 4));
						if (a.s2 && t <= a.jq2) {
							// the buffer's previous contents (two tiles back) were consumed by a P.V that
							// this thread issued earlier: tensor-core operations execute in issue order
							u32 const b = n2 & 1;
	#pragma unroll
							for (u32 ks = 0; ks < D / 32; ++ks) {
								mma_i8_ss(tmem_base + S2_COL + b * BKV, q2_desc + 2 * ks, bdesc + 2 * ks, idesc_qk, ks != 0);
							}
							tc_commit(s2_full_bar(b));
							++n2;
						}
						if (a.s1 && t >= a.t1_lo) {
							if (n1 > 0) {  // the rows have copied the previous scores of this buffer
								ok = mbar_wait(s1_read_bar, (n1 - 1) & 1, ctx, ST_WAIT_S_DONE, t);
								if (!ok) break;
								tc_fence_after();
							}
#pragma unroll
							for (u32 ks = 0; ks < D / 32; ++ks) {
								mma_i8_ss(tmem_base + S1_COL, q1_desc + 2 * ks, bdesc + 2 * ks, idesc_qk, ks != 0);
							}
							tc_commit(s1_full_bar);
							++n1;
						}
						tc_commit(empty_bar(s));
						++it;
						if (a.s2 && t > a.t_lo && t - 1 <= a.jq2) ok = issue_pv();
					}
					if (ok && a.s2 && a.t_hi == a.jq2) ok = issue_pv();
					if (ok && a.s2) {
						tc_commit(o_full_bar);
						tc_commit(q_empty_bar((nq1 - 1) % Q_BUFFERS));
						++no;
					}
				}
				nq_base += j1 - j0;
			}
		}
	} else {
		// ---------------- four threads per query row ----------------
		[&]() {
			u32 const quarter = warp & 3;      // TMEM lanes this warp may touch
			u32 const cq = (warp - 2) >> 2;    // which 32 score columns / which quarter of D
			u32 const row = quarter * 32 + lane;
			u32 const lane_addr = (quarter * 32u) << 16;
			u32 const col_base = cq * 32u;
			constexpr u32 DQ = D / 4;           // output columns of this thread
			constexpr u32 CH = DQ >= 16 ? 16 : 8;
			f32 const base_t = f32((1.0 / 64.0) * (D == 128 ? 0.08838834764831845 : D == 64 ? 0.125 : 0.17677669529663687));
			// 16-byte chunks of a Q row are XOR-swizzled by the row index the way the TMA wrote them
			u32 const q_swz = D == 128 ? (row & 7u) : D == 64 ? ((row >> 1) & 3u) : ((row >> 2) & 1u);

			u32 n1 = 0, n2 = 0, no = 0, nx = 0, nq_base = 0, n_item = 0;

			auto warp_arrive = [&](u32 bar) {
				__syncwarp();
				if (lane == 0) mbar_arrive(bar);
			};
			// bounded wait of a whole warp, inline: every lane polls (a try suspends the lane in hardware
			// while the phase is incomplete), the verdict is made uniform with one vote
			auto wait_rows = [&](u32 bar, u32 parity, u32 code, u32 detail) -> bool {
				bool mine = mbar_try_wait(bar, parity);
				if (!mine) {
	#pragma unroll 1
					for (u32 i = 0; i < WAIT_SLOW_POLLS && !mine; ++i) {
						mine = mbar_try_wait(bar, parity);
						if ((i & 63u) == 63u && *abort_flag != 0) break;
					}
				}
				bool const all = __all_sync(0xffffffffu, mine);
				if (!all && lane == 0) {
					*abort_flag = 1;
					report_status(p.status, code, detail);
				}
				return all;
			};
			// this warp's 32 key columns of the tile starting at key k0 against its 32 rows of the query
			// tile starting at q0: 0 = no row sees any of them, 1 = every row sees all of them, 2 = mixed
			auto classify = [&](u32 q0, u32 k0) -> u32 {
				u32 const kc = k0 + col_base;
				u32 const r_lo = q0 + quarter * 32u, r_hi = r_lo + 31u;
				bool const none = kc >= r_hi || (w != 0xFFFFFFFFu && kc + 31u + w < r_lo);
				bool const every = kc + 31u < r_lo && (w == 0xFFFFFFFFu || kc + w >= r_hi);
				return none ? 0u : every ? 1u : 2u;
			};
			// visible columns of row qi inside the tile that starts at key k0: lo <= col < lo + span
			auto visible = [&](u32 qi, u32 k0, u32 &lo, u32 &span) {
				i32 const hi_i = min(i32(BKV), i32(qi) - i32(k0));
				i32 const lo_i = (w == 0xFFFFFFFFu) ? 0 : max(0, i32(qi) - i32(w) - i32(k0));
				lo = u32(lo_i);
				span = hi_i > lo_i ? u32(hi_i - lo_i) : 0u;
			};

			#pragma unroll 1
			for (u32 item = blockIdx.x; item < plan.n_items; item += gridDim.x) {
				u32 batch, head, j0, j1;
				decode_item(item, batch, head, j0, j1);
				f32 const head_t = __ldg(p.temperature + head);
				bool const pos_t = head_t >= 0.0f;  // uniform over the item; the row factor is positive
				// the sink values of this head as f32, one copy per row quarter (its four warps write it here and
				// read it in the epilogues, which start one pass and one exchange barrier of the quarter later; the
				// buffer of the item before the previous one is free)
				f32 *const svf = svf_all + (quarter * 2 + (n_item & 1)) * 128;
				{
					u32 const rt = cq * 32 + lane;
					if (rt < D) {
						u32 const b = reinterpret_cast<u8 const *>(p.sink_v)[head * D + rt];
						svf[rt] = FP8PV ? hw_e4m3_to_f32(b) : f32(i32(i8(b)));
					}
				}
				++n_item;

				// state of the query tile in its probability sweep (set at the end of the previous pass)
				f32 temp2 = 0.0f, m2 = 0.0f, sink_s2 = 0.0f;

				#pragma unroll 1
				for (u32 pp = 0; pp <= j1 - j0; ++pp) {
					AttnPass const a = attn_pass(j0, j1, pp, w);
					u32 const qi2 = a.jq2 * BQ + row;  // only used when a.s2
					u32 const qi1 = a.jq1 * BQ + row;
					bool const row_ok2 = a.s2 && qi2 < p.seq_len;
					bool const row_ok1 = a.s1 && qi1 < p.seq_len;

					// the next query tile: temperature, this thread's quarter of the sink dot product (q from the
					// Q tile in shared memory: a global load here would stall the warp for thousands of cycles)
					f32 temp1 = 0.0f;
					i32 sdot = 0;
					if (a.s1) {
						u32 const n_att = (qi1 < w ? qi1 : w) + 4u;
						temp1 = __fmul_rn(__fmul_rn(base_t, lg2_approx(f32(n_att))), head_t);
						u32 const nq1 = nq_base + pp;
						u32 const qb = nq1 % Q_BUFFERS;
						if (!wait_rows(q_full_bar(qb), (nq1 / Q_BUFFERS) & 1, ST_WAIT_Q_FULL, 0x200u + qb)) return;
						u8 const *qrow = smem_gen + qb * Q_BYTES + row * D;
						u8 const *sk = smem_gen + SK_OFF + qb * 128 + cq * DQ;
	#pragma unroll
						for (u32 i = 0; i < DQ / 8; ++i) {
							u32 const o = cq * DQ + 8 * i;
							uint2 const x = *reinterpret_cast<uint2 const *>(qrow + ((((o >> 4) ^ q_swz) << 4) | (o & 15u)));
							uint2 const y = *reinterpret_cast<uint2 const *>(sk + 8 * i);
							sdot = __dp4a(i32(x.x), i32(y.x), sdot);
							sdot = __dp4a(i32(x.y), i32(y.y), sdot);
						}
					}
					i32 ext[4];
	#pragma unroll
					for (u32 i = 0; i < 4; ++i) ext[i] = pos_t ? INT32_MIN : INT32_MAX;
					f32 sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
					f32 const neg_m = -m2;

					#pragma unroll 1
					for (u32 t = a.t_lo; t <= a.t_hi; ++t) {
						bool const do2 = a.s2 && t <= a.jq2;
						bool const do1 = a.s1 && t >= a.t1_lo;
						u32 const k0 = t * BKV;
						// first the maximum sweep's scores: copying them frees their buffer for the tensor core
						// a whole softmax before the next ones are needed
						if (do1) {
							if (!wait_rows(s1_full_bar, n1 & 1, ST_WAIT_S_FULL, 0x100u + t)) return;
							tc_fence_after();
							u32 r1[32];
							tmem_ld_32x32b_x32(tmem_base + lane_addr + S1_COL + col_base, r1);
							tmem_wait_ld();
							tc_fence_before();
							warp_arrive(s1_read_bar);
							++n1;
							bool const edge = (t == a.jq1) || (w != 0xFFFFFFFFu && k0 + w < a.jq1 * BQ + BQ - 1);
							u32 const cls = edge ? classify(a.jq1 * BQ, k0) : 1u;
							if (cls == 1u) {
								if (pos_t) extreme_chunk<false, true>(r1, col_base, 0, 0, ext);
								else extreme_chunk<false, false>(r1, col_base, 0, 0, ext);
							} else if (cls == 2u) {
								u32 lo, span;
								visible(qi1, k0, lo, span);
								if (pos_t) extreme_chunk<true, true>(r1, col_base, lo, span, ext);
								else extreme_chunk<true, false>(r1, col_base, lo, span, ext);
							}
							if constexpr (DEBUG) {
								if (row_ok1) {
									i32 *dst = p.dbg_s + (u64(batch) * p.n_heads + head) * p.seq_len * p.seq_len
											   + u64(qi1) * p.seq_len + k0 + col_base;
	#pragma unroll
									for (u32 i = 0; i < 32; ++i) {
										if (k0 + col_base + i < p.seq_len) dst[i] = i32(r1[i]);
									}
								}
							}
						}
						if (do2) {
							u32 const b2 = n2 & 1;
							if (!wait_rows(s2_full_bar(b2), (n2 >> 1) & 1, ST_WAIT_S_FULL, t)) return;
							tc_fence_after();
							u32 const ta = tmem_base + lane_addr + S2_COL + b2 * BKV + col_base;
							bool const edge = (t == a.jq2) || (w != 0xFFFFFFFFu && k0 + w < a.jq2 * BQ + BQ - 1);
							u32 const cls = edge ? classify(a.jq2 * BQ, k0) : 1u;
							u32 pk[8];
							if (cls != 0u) {
								u32 r2[32];
								tmem_ld_32x32b_x32(ta, r2);
								tmem_wait_ld();
								if (cls == 1u) {
									softmax_chunk<false, FP8PV>(r2, col_base, temp2, neg_m, 0, 0, sum, pk);
								} else {
									u32 lo, span;
									visible(qi2, k0, lo, span);
									softmax_chunk<true, FP8PV>(r2, col_base, temp2, neg_m, lo, span, sum, pk);
								}
							} else {
	#pragma unroll
								for (u32 i = 0; i < 8; ++i) pk[i] = 0u;
							}
							// the probabilities go over this thread's own first eight score columns
							tmem_st_32x32b_x8(ta, pk);
							tmem_wait_st();
							tc_fence_before();
							warp_arrive(p_ready_bar(b2));
							++n2;
							if constexpr (DEBUG) {
								if (row_ok2) {
									u8 *dst = p.dbg_p + (u64(batch) * p.n_heads + head) * p.seq_len * p.seq_len
											  + u64(qi2) * p.seq_len + k0 + col_base;
	#pragma unroll
									for (u32 i = 0; i < 32; ++i) {
										if (k0 + col_base + i < p.seq_len) dst[i] = u8(pk[i >> 2] >> (8 * (i & 3)));
									}
								}
							}
						}
					}

					// ---- end of the pass: the four threads of a row exchange their parts ----
					u32 *const xc = xchg + (nx & 1) * (3 * 4 * BQ);
					{
						f32 cand = -INFINITY;
						i32 const e = pos_t ? max(max(ext[0], ext[1]), max(ext[2], ext[3]))
											: min(min(ext[0], ext[1]), min(ext[2], ext[3]));
						if (a.s1 && e != (pos_t ? INT32_MIN : INT32_MAX)) cand = __fmul_rn(__int2float_rn(e), temp1);
						f32 const part = __fadd_rn(__fadd_rn(sum[0], sum[1]), __fadd_rn(sum[2], sum[3]));
						xc[(0 * 4 + cq) * BQ + row] = __float_as_uint(cand);
						xc[(1 * 4 + cq) * BQ + row] = __float_as_uint(part);
						xc[(2 * 4 + cq) * BQ + row] = u32(sdot);
					}
					warp_arrive(xchg_bar(quarter));
					if (!wait_rows(xchg_bar(quarter), nx & 1, ST_WAIT_S_DONE, 0x300u)) return;
					++nx;
					f32 m1 = 0.0f, sink_s1 = 0.0f;
					if (a.s1) {
						i32 const dot = i32(xc[(2 * 4 + 0) * BQ + row]) + i32(xc[(2 * 4 + 1) * BQ + row])
										+ i32(xc[(2 * 4 + 2) * BQ + row]) + i32(xc[(2 * 4 + 3) * BQ + row]);
						sink_s1 = __fmul_rn(__int2float_rn(dot), temp1);
						f32 const c01 = fmaxf(__uint_as_float(xc[(0 * 4 + 0) * BQ + row]), __uint_as_float(xc[(0 * 4 + 1) * BQ + row]));
						f32 const c23 = fmaxf(__uint_as_float(xc[(0 * 4 + 2) * BQ + row]), __uint_as_float(xc[(0 * 4 + 3) * BQ + row]));
						m1 = fmaxf(sink_s1, fmaxf(c01, c23));
					}

					// ---- normalise and store query tile jq2: each thread takes a quarter of the D columns ----
					if (a.s2) {
						f32 const both = __fadd_rn(
							__fadd_rn(__uint_as_float(xc[(1 * 4 + 0) * BQ + row]), __uint_as_float(xc[(1 * 4 + 1) * BQ + row])),
							__fadd_rn(__uint_as_float(xc[(1 * 4 + 2) * BQ + row]), __uint_as_float(xc[(1 * 4 + 3) * BQ + row])));
						if (!wait_rows(o_full_bar, no & 1, ST_WAIT_O_FULL, 0)) return;
						tc_fence_after();
						f32 const sink_e = ex2_approx(__fsub_rn(sink_s2, m2));
						constexpr f32 PS = FP8PV ? 256.0f : 255.0f;  // scale of the quantised probabilities
						f32 const total = __fmul_rn(__fadd_rn(both, sink_e), PS);
						f32 const w_sink = __fmul_rn(sink_e, PS);
						f32 const recip = rcp_approx(total);
						u32 const d0 = cq * DQ;
						u64 const out_off = u64(batch) * p.o_batch_stride + u64(qi2) * p.o_stride + head * D + d0;
						f32 const vs = FP8PV ? __fmul_rn(recip, __ldg(p.v_scale + head)) : recip;
	#pragma unroll
						for (u32 c = 0; c < DQ; c += CH) {
							u32 r[CH];
							if constexpr (CH == 16) tmem_ld_32x32b_x16(tmem_base + lane_addr + O_COL + d0 + c, r);
							else tmem_ld_32x32b_x8(tmem_base + lane_addr + O_COL + d0 + c, r);
							f32 sv[CH];
	#pragma unroll
							for (u32 i = 0; i < CH; i += 4) {
								float4 const s4 = *reinterpret_cast<float4 const *>(svf + d0 + c + i);
								sv[i] = s4.x; sv[i + 1] = s4.y; sv[i + 2] = s4.z; sv[i + 3] = s4.w;
							}
							tmem_wait_ld();
							if constexpr (FP8PV) {
								// O is f32 = sum of (256 p) * e4m3(v); sink_v is e4m3 too; out = bf16(value * v_scale)
								u32 o2[CH / 2];
	#pragma unroll
								for (u32 i = 0; i < CH; i += 2) {
									f32 const oa = __fmul_rn(__fmaf_rn(w_sink, sv[i], __uint_as_float(r[i])), vs);
									f32 const ob = __fmul_rn(__fmaf_rn(w_sink, sv[i + 1], __uint_as_float(r[i + 1])), vs);
									o2[i / 2] = cvt_bf16x2(oa, ob);
								}
								if (row_ok2) {
									uint4 *dst = reinterpret_cast<uint4 *>(static_cast<u16 *>(p.out) + out_off + c);
	#pragma unroll
									for (u32 i = 0; i < CH / 8; ++i) dst[i] = make_uint4(o2[4 * i], o2[4 * i + 1], o2[4 * i + 2], o2[4 * i + 3]);
								}
							} else {
								// rint(clamp(o * recip)) through the 1.5 * 2^23 trick: the code is the low byte
								u32 pk[CH / 4];
	#pragma unroll
								for (u32 g = 0; g < CH / 4; ++g) {
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
								if (row_ok2) {
									i8 *dst = static_cast<i8 *>(p.out) + out_off + c;
									if constexpr (CH == 16) *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
									else *reinterpret_cast<uint2 *>(dst) = make_uint2(pk[0], pk[1]);
									if constexpr (DEBUG) {
										i32 *d = p.dbg_o + ((u64(batch) * p.n_heads + head) * p.seq_len + qi2) * D + d0 + c;
	#pragma unroll
										for (u32 i = 0; i < CH; ++i) d[i] = i32(r[i]);
									}
								}
							}
						}
						tc_fence_before();
						warp_arrive(o_read_bar);  // the next query tile's first P.V may overwrite O
						++no;
						if (row_ok2 && cq == 0 && p.l != nullptr) {
							p.l[u64(batch) * p.l_batch_stride + u64(head) * p.seq_len + qi2] = __fadd_rn(lg2_approx(total), m2);
						}
					}
					temp2 = temp1;
					m2 = m1;
					sink_s2 = sink_s1;
				}
				nq_base += j1 - j0;
			}
		}();
	}

	tc_fence_before();
	__syncthreads();
	if (warp == 1) {
		__syncwarp();
		tc_fence_after();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
	if (threadIdx.x == 0) {
		for (u32 i = 0; i < N_BARRIERS; ++i) mbar_inval(bar_base + 8 * i);
	}
}

}  // namespace x17
