// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA,
// TMEM alloc/ld/st, commit, fences) and shared-memory matrix descriptors.
//
// Every wait in this file is bounded: a wait that runs out records a code in the device-side
// status word and returns false, so that the caller can unwind (free TMEM, return) instead of
// spinning forever.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace x17 {

using i8 = int8_t;
using u8 = uint8_t;
using u16 = uint16_t;
using i32 = int32_t;
using u32 = uint32_t;
using u64 = uint64_t;
using f32 = float;

#define X17_DEV __device__ __forceinline__

// ---------------------------------------------------------------------------------------------
// status words (device memory owned by the library, passed to every kernel):
// [0] first error as (code << 16 | detail), 0 = ok; [1] blockIdx of the reporter;
// [2] number of reports; [3] reserved

enum StatusCode : u32 {
	ST_OK = 0,
	ST_WAIT_TMA_FULL = 1,
	ST_WAIT_STAGE_EMPTY = 2,
	ST_WAIT_ACC_FULL = 3,
	ST_WAIT_ACC_EMPTY = 4,
	ST_WAIT_S_FULL = 5,
	ST_WAIT_S_DONE = 6,
	ST_WAIT_O_FULL = 7,
	ST_WAIT_Q_FULL = 8,
	ST_NOT_PREPARED = 15,  // a kernel object was launched before the set-up launch it needs
};

X17_DEV void report_status(u32 *status, u32 code, u32 detail) {
	u32 v = (code << 16) | (detail & 0xFFFFu);
	if (atomicCAS(&status[0], 0u, v) == 0u) {
		status[1] = blockIdx.x | (blockIdx.y << 16);
	}
	atomicAdd(&status[2], 1u);
}

// What a role needs to give up cleanly: the CTA-wide abort flag (shared memory) that any role
// sets when a wait runs out, and the status words to record why.
struct WaitCtx {
	volatile u32 *abort_flag;
	u32 *status;
};

// ---------------------------------------------------------------------------------------------
// misc

X17_DEV u32 smem_u32(void const *p) {
	return static_cast<u32>(__cvta_generic_to_shared(p));
}

X17_DEV bool elect_one() {
	u32 pred;
	asm volatile(
		"{\n\t.reg .pred P;\n\t"
		"elect.sync _|P, 0xffffffff;\n\t"
		"selp.u32 %0, 1, 0, P;\n\t}"
		: "=r"(pred));
	return pred != 0;
}

X17_DEV f32 ex2_approx(f32 x) {
	f32 r;
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}
X17_DEV f32 lg2_approx(f32 x) {
	f32 r;
	asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}
X17_DEV f32 rcp_approx(f32 x) {
	f32 r;
	asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}
X17_DEV f32 rsqrt_approx(f32 x) {
	f32 r;
	asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}
X17_DEV f32 tanh_approx(f32 x) {
	f32 r;
	asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
	return r;
}

// packed f32x2 arithmetic (two IEEE f32 operations per issue slot on sm_100)
X17_DEV u64 pack_f32x2(f32 lo, f32 hi) {
	u64 r;
	asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
	return r;
}
X17_DEV void unpack_f32x2(u64 v, f32 &lo, f32 &hi) {
	asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
X17_DEV u64 fma_f32x2(u64 a, u64 b, u64 c) {
	u64 d;
	asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
	return d;
}
X17_DEV u64 mul_f32x2(u64 a, u64 b) {
	u64 d;
	asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
	return d;
}
// two f32 -> two OCP e4m3 bytes (round to nearest even, saturating): lo in bits 0-7, hi in 8-15
X17_DEV u32 cvt_e4m3x2(f32 lo, f32 hi) {
	unsigned short r;
	asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
	return r;
}
// two f32 -> two bf16 (round to nearest even): lo in bits 0-15, hi in 16-31
X17_DEV u32 cvt_bf16x2(f32 lo, f32 hi) {
	u32 r;
	asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
	return r;
}
X17_DEV u64 add_f32x2(u64 a, u64 b) {
	u64 d;
	asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
	return d;
}

// ---------------------------------------------------------------------------------------------
// mbarrier

X17_DEV void mbar_init(u32 bar, u32 count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
X17_DEV void mbar_inval(u32 bar) {
	asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
X17_DEV void mbar_fence_init() {
	asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
X17_DEV void mbar_expect_tx(u32 bar, u32 bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
				 : "memory");
}
X17_DEV void mbar_arrive(u32 bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try: the thread may be suspended by the hardware for up to `SUSPEND_NS` while the phase
// is incomplete, which keeps waiting warps from burning issue slots on a polling loop.
constexpr u32 SUSPEND_NS = 20000;
X17_DEV bool mbar_try_wait(u32 bar, u32 parity) {
	u32 ok;
	asm volatile(
		"{\n\t.reg .pred P;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
		"selp.u32 %0, 1, 0, P;\n\t}"
		: "=r"(ok)
		: "r"(bar), "r"(parity), "r"(SUSPEND_NS)
		: "memory");
	return ok != 0;
}

// Bounded wait: returns false when it gives up (after about a second), having set the CTA's
// abort flag so that the other roles leave their waits quickly too.
constexpr u32 WAIT_FAST_POLLS = 1u << 10;
constexpr u32 WAIT_SLOW_POLLS = 1u << 17;  // x up to 20 us of suspension each: a second or two

// The polling loops live in one out-of-line function: inlined and unrolled at every wait they
// made up most of the kernels' code and thrashed the instruction cache.
__device__ __noinline__ bool mbar_wait_slow(u32 bar, u32 parity, volatile u32 *abort_flag, u32 *status,
											u32 code, u32 detail) {
#pragma unroll 1
	for (u32 i = 0; i < WAIT_FAST_POLLS; ++i) {
		if (mbar_try_wait(bar, parity)) return true;
	}
#pragma unroll 1
	for (u32 i = 0; i < WAIT_SLOW_POLLS; ++i) {
		if (mbar_try_wait(bar, parity)) return true;
		if (*abort_flag != 0) return false;
	}
	*abort_flag = 1;
	report_status(status, code, detail);
	return false;
}

X17_DEV bool mbar_wait(u32 bar, u32 parity, WaitCtx const &ctx, u32 code, u32 detail) {
	if (mbar_try_wait(bar, parity)) return true;
	return mbar_wait_slow(bar, parity, ctx.abort_flag, ctx.status, code, detail);
}

// Warp-uniform bounded wait: lane 0 polls, the verdict is broadcast, and on success every lane
// observes the completed phase itself before going on (it cannot advance again before this
// warp has arrived on the matching "empty" barrier). All lanes return the same value, so the
// warp stays converged for the .sync.aligned tcgen05 instructions that follow.
X17_DEV bool mbar_wait_warp(u32 bar, u32 parity, WaitCtx const &ctx, u32 code, u32 detail) {
	// fast path: every lane observes the phase itself (one suspended try each, no polling loop)
	bool mine = mbar_try_wait(bar, parity);
	if (__all_sync(0xffffffffu, mine)) return true;
	// slow path: lane 0 runs the bounded wait and broadcasts the verdict
	u32 ok = 0;
	if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, ctx, code, detail) ? 1u : 0u;
	ok = __shfl_sync(0xffffffffu, ok, 0);
	if (ok) {
#pragma unroll 1
		for (u32 i = 0; i < WAIT_FAST_POLLS; ++i) {
			if (mbar_try_wait(bar, parity)) break;
		}
	}
	__syncwarp();
	return ok != 0;
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma)
X17_DEV void fence_proxy_async_smem() {
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA tiled loads: every CTA fetches its own tiles

X17_DEV void tma_load_2d(u32 dst, CUtensorMap const *map, u32 bar, i32 x, i32 y) {
	asm volatile(
		"cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
		" [%0], [%1, {%3, %4}], [%2];"
		:
		: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
		: "memory");
}
X17_DEV void tma_load_3d(u32 dst, CUtensorMap const *map, u32 bar, i32 x, i32 y, i32 z) {
	asm volatile(
		"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
		" [%0], [%1, {%3, %4, %5}], [%2];"
		:
		: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
		: "memory");
}
X17_DEV void tma_prefetch_desc(CUtensorMap const *map) {
	asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation

X17_DEV void tmem_alloc(u32 smem_dst, u32 ncols) {
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
				 "r"(ncols)
				 : "memory");
}
X17_DEV void tmem_relinquish() {
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
X17_DEV void tmem_dealloc(u32 taddr, u32 ncols) {
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
				 : "memory");
}
X17_DEV void tc_fence_before() {
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
X17_DEV void tc_fence_after() {
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
X17_DEV void tc_commit(u32 bar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
				 : "memory");
}
// ---- the same for a pair of CTAs on two SMs (a cluster of two): one MMA spans both, each CTA holding its
// 128 rows of A, its half of B's rows and its 128 lanes of the accumulator. Allocation, release and free are
// issued by the same warp of both CTAs with the same shared-memory slot offset.
X17_DEV void tmem_alloc_pair(u32 smem_dst, u32 ncols) {
	asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
				 : "memory");
}
X17_DEV void tmem_relinquish_pair() {
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
X17_DEV void tmem_dealloc_pair(u32 taddr, u32 ncols) {
	asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives on `bar` (a shared::cluster address: the issuing CTA's barrier or its peer's) once the pair's MMAs
// issued so far have completed
X17_DEV void tc_commit_pair(u32 bar_cluster) {
	asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
				 : "memory");
}
X17_DEV void mma_i8_ss_pair(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
X17_DEV void mma_f8_ss_pair(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
// TMA tile into this CTA's shared memory whose bytes are counted on a barrier of either CTA of the pair
// (`bar_cluster`: a shared::cluster address). Every CTA fetches its own tiles itself.
X17_DEV void tma_load_2d_pair(u32 dst, CUtensorMap const *map, u32 bar_cluster, i32 x, i32 y) {
	asm volatile(
		"cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
		" [%0], [%1, {%3, %4}], [%2];"
		:
		: "r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
		: "memory");
}
// cluster plumbing
X17_DEV u32 cluster_cta_rank() {
	u32 r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
X17_DEV u32 map_to_cta(u32 smem_addr, u32 rank) {
	u32 r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
	return r;
}
X17_DEV void mbar_arrive_cluster(u32 bar_cluster) {
	asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
X17_DEV void cluster_sync_all() {
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

X17_DEV void tmem_wait_ld() {
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp gets lane (base_lane + t), columns c..c+31
X17_DEV void tmem_ld_32x32b_x32(u32 taddr, u32 (&r)[32]) {
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
		"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
		"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
		  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
		  "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
		  "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
		  "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
		: "r"(taddr)
		: "memory");
}

// 32 lanes x 16 columns
X17_DEV void tmem_ld_32x32b_x16(u32 taddr, u32 (&r)[16]) {
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x16.b32 "
		"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
		  "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
		  "=r"(r[14]), "=r"(r[15])
		: "r"(taddr)
		: "memory");
}

// named barrier among a subset of the CTA's warps
X17_DEV void named_barrier_sync(u32 id, u32 threads) {
	asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: descriptors and MMA

// Shared-memory matrix descriptor (64-bit):
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1
//   [61,64) layout: 0 none, 2 = 128B swizzle, 4 = 64B swizzle, 6 = 32B swizzle
// For swizzled layouts the tile rows are `swizzle_bytes` wide; 8 consecutive rows form one
// swizzle atom and the stride byte offset is the distance between atoms (8 * swizzle_bytes).
// This holds for both K-major operands (row = M/N index, bytes along K) and MN-major operands
// (row = K index, bytes along M/N) as long as the tile is one atom wide.
X17_DEV constexpr u32 swizzle_layout_code(u32 swizzle_bytes) {
	return swizzle_bytes == 128 ? 2u : swizzle_bytes == 64 ? 4u : swizzle_bytes == 32 ? 6u : 0u;
}
X17_DEV u64 make_smem_desc(u32 smem_addr, u32 swizzle_bytes) {
	u64 d = 0;
	d |= u64((smem_addr & 0x3FFFFu) >> 4);
	d |= u64(1) << 16;                              // leading byte offset: unused, 16 B
	d |= u64((8u * swizzle_bytes) >> 4) << 32;      // stride byte offset between 8-row atoms
	d |= u64(1) << 46;                              // descriptor version (Blackwell)
	d |= u64(swizzle_layout_code(swizzle_bytes)) << 61;
	return d;
}

// Instruction descriptor (32-bit) for kind::i8 / kind::f8f6f4 / kind::f16:
//   [4,6) D format: 0 f16, 1 f32, 2 s32      [7,10) A format   [10,13) B format
//   [15] A major (0 = K-major, 1 = MN-major)  [16] B major
//   [17,23) N >> 3                            [24,29) M >> 4
enum : u32 { FMT_U8 = 0, FMT_S8 = 1, FMT_E4M3 = 0, FMT_E5M2 = 1, DFMT_F32 = 1, DFMT_S32 = 2 };
X17_DEV constexpr u32 make_idesc(u32 dfmt, u32 afmt, u32 bfmt, u32 a_mn_major, u32 b_mn_major,
								 u32 m, u32 n) {
	return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | (a_mn_major << 15) | (b_mn_major << 16)
		   | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
X17_DEV void mma_i8_ss(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}
X17_DEV void mma_f8_ss(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
		:
		: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
		: "memory");
}

// ---------------------------------------------------------------------------------------------
// number formats of the reference (cuda/utils_b8.cuh:629-657)

// FixedI8: clamp to +-127, round half to even.
X17_DEV i32 f32_to_fixedi8(f32 x) {
	return __float2int_rn(fmaxf(-127.0f, fminf(127.0f, x)));
}

// Custom e4m3: flush below 1.9375 * 2^-7 to +0, round half up in magnitude, saturate to 0x7E.
X17_DEV u32 f32_to_e4m3(f32 x) {
	u32 bits = __float_as_uint(x);
	u32 sign = (bits >> 24) & 0x80u;
	u32 rest = bits & 0x7FFFFFFFu;
	constexpr u32 lo = (120u << 23) + (0xFu << 19);
	constexpr u32 hi = (135u << 23) + (0xCu << 19);
	u32 rounded = (rest + ((1u << 19) - (120u << 23))) >> 20;
	u32 clamped = rest > hi ? 0x7Eu : rounded;
	return rest < lo ? 0u : (sign | clamped);
}

X17_DEV f32 e4m3_to_f32(u32 code) {
	u32 sign = (code & 0x80u) << 8;
	u32 rest = (code & 0x7Fu) << 4;
	u32 bf = ((sign | rest) + (120u << 7)) & 0xFFFFu;
	return rest == 0 ? 0.0f : __uint_as_float(bf << 16);
}

// one OCP e4m3 byte (subnormals included) -> f32 through the hardware converter
X17_DEV f32 hw_e4m3_to_f32(u32 code) {
	u32 h2;
	asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h2) : "r"(code & 0xFFu));
	f32 r;
	asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.f32.f16 %0, lo;\n\t}" : "=f"(r) : "r"(h2));
	return r;
}

X17_DEV u32 pack4(u32 b0, u32 b1, u32 b2, u32 b3) {
	return (b0 & 0xFFu) | ((b1 & 0xFFu) << 8) | ((b2 & 0xFFu) << 16) | (b3 << 24);
}

}  // namespace x17
