// Shared device helpers for the sm_100a GPTQ kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gptq_b200.h"

namespace gptq {

// ---- nibble -> fp16 conversion -------------------------------------------------
// (q & 0x000F000F) | 0x64006400 is the half2 (1024 + nib_lo, 1024 + nib_hi): 0x6400 is
// 1024.0 and one mantissa ulp there is 1.  With the mask 0x00F000F0 the nibble sits four
// bits higher and the value is 1024 + 16*nib, still exact.
constexpr uint32_t MAGIC_1024 = 0x64006400u;
constexpr uint32_t MASK_LO = 0x000F000Fu;
constexpr uint32_t MASK_HI = 0x00F000F0u;

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
	uint32_t r;
	asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));   // (a & b) | c
	return r;
}

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
	uint32_t r;
	asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
	return r;
}

__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
	uint32_t r;
	asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
	return r;
}

__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
	uint32_t r;
	asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
	return r;
}

// ---- cp.async (16-byte, L2 only) -----------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
	uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
	asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- warp-level fp16 MMA, fp32 accumulate --------------------------------------
// D(16x8) += A(16x16, row) * B(16x8, col).  Fragment ownership (gid = lane/4, tig = lane%4):
//   a0:(gid, 2tig..+1) a1:(gid+8, 2tig..+1) a2:(gid, 2tig+8..+9) a3:(gid+8, 2tig+8..+9)
//   b0:(k=2tig..+1, n=gid) b1:(k=2tig+8..+9, n=gid)
//   d0:(gid, 2tig) d1:(gid, 2tig+1) d2:(gid+8, 2tig) d3:(gid+8, 2tig+1)
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
										 uint32_t b0, uint32_t b1) {
	asm volatile(
		"mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
		: "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
		: "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_nc_v4(const void *p) {
	uint4 r;
	asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
				 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
				 : "l"(p));
	return r;
}

// ---- programmatic dependent launch -------------------------------------------------------
// pdl_trigger(): lets the next kernel in the stream start its independent prologue early.
// pdl_wait(): returns once every kernel this one depends on has completed and its writes are
// visible; nothing produced by an earlier kernel may be touched before it.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + __expf(-x)); }

// ---- host-side launch plumbing -------------------------------------------------
extern thread_local int g_last_cuda_error;
inline int cuda_status(cudaError_t e) {
	if (e == cudaSuccess) return GPTQ_OK;
	g_last_cuda_error = (int)e;
	return GPTQ_ERR_CUDA;
}
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}   // namespace gptq

// ---- mbarrier + TMA (bulk tensor copy) wrappers ---------------------------------------
namespace gptq {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
	uint32_t ok;
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
		"selp.u32 %0, 1, 0, p;\n\t}"
		: "=r"(ok)
		: "r"(bar), "r"(parity)
		: "memory");
	return ok;
}

// Upper half of the 8-byte {value, tag} words that carry partial sums between CTAs without a fence or a
// counter: a quiet-NaN bit pattern, so that a stale fp32 value in the same memory can never look like it.
constexpr unsigned WORD_TAG = 0x7FC0DE01u;

__device__ __forceinline__ unsigned long long global_timer_ns() {
	unsigned long long t;
	asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
	return t;
}

// Bounded wait: returns false when the phase did not complete within `limit` polls or within
// about two seconds of wall time, whichever comes first (a poll may itself suspend the thread
// for a while, so the poll count alone does not bound the time).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
	unsigned long long t0 = 0;
#pragma unroll 1
	for (uint32_t i = 0; i < limit; ++i) {
		if (mbar_try_wait(bar, parity)) return true;
		if ((i & 255u) == 255u) {
			const unsigned long long now = global_timer_ns();
			if (t0 == 0) t0 = now;
			else if (now - t0 > 2000000000ull) return false;
		}
	}
	return false;
}

// 2-D tiled TMA load global -> this CTA's shared memory, completion signalled on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar) {
	asm volatile(
		"cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
		"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar)
		: "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void *tmap) {
	asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

}   // namespace gptq
