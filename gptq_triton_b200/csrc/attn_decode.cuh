// Single-query (decode) attention over a static fp16 KV cache: softmax(q·K^T / sqrt(d)) · V
// for one new token per sequence.  HBM-bound: K and V of every cached position are read once.
//
// Grid (splits, heads, batch).  A CTA of 8 warps takes a contiguous range of cache positions and
// pulls it into shared memory with bulk asynchronous copies (64 keys of K and of V per stage,
// three stages, mbarrier completion).  The copies are issued BEFORE the kernel waits for its
// predecessor in the stream: old cache rows do not depend on it, so the cache streams in while
// the QKV kernel of the same step is still finishing.  Only the newest AT_FRESH positions are
// read from global memory after the wait (they may have been written by that kernel).
// 8 lanes share one key (16 head dims each); each 8-lane group keeps an online softmax (running
// max, running sum, 16 output dims in fp32).  Groups, warps and splits are merged with the usual
// log-sum-exp rescaling; the last CTA of a (batch, head) to arrive (ticket in the workspace)
// merges the split partials in fixed order and writes fp16.
#pragma once

#include "common.cuh"

namespace gptq {

constexpr int AT_D = 128;              // head dim
constexpr int AT_THREADS = 256;         // 8 warps = 32 key groups of 8 lanes
constexpr int AT_GROUPS = AT_THREADS / 8;
constexpr int AT_MAX_SPLITS = 32;
constexpr int AT_TICKET_BYTES = 16384;
constexpr int AT_STATUS_SLOT = AT_TICKET_BYTES / 4 - 1;      // same word as the matmul kernels' status
constexpr int AT_CHUNK = 64;           // keys per stage
constexpr int AT_STAGES = 3;
constexpr int AT_STAGE_BYTES = 2 * AT_CHUNK * AT_D * 2;      // K rows then V rows: 32 KB
constexpr int AT_SMEM_BYTES = AT_STAGES * AT_STAGE_BYTES + 64;
constexpr int AT_FRESH = 16;           // newest positions that are never read ahead of the dependency wait

struct AttnParams {
	const __half *q;          // [b, heads, 128] (row stride q_stride_b)
	long long q_stride_b;
	const __half *kc, *vc;    // [b, heads, max_seq, 128]
	long long kv_stride_b, kv_stride_h;
	const int32_t *pos;       // [b]: index of the newest token; positions 0..pos are attended
	__half *out;              // [b, heads*128]
	long long out_stride_b;
	float scale;
	int heads, splits;
	float *ws_partial;        // [b*heads][splits][130]
	int *ws_ticket;           // [b*heads]
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
				 "r"(bar)
				 : "memory");
}

__global__ void __launch_bounds__(AT_THREADS) attn_decode_kernel(const AttnParams p) {
	extern __shared__ __align__(128) unsigned char at_smem[];
	const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int grp = lane >> 3, sub = lane & 7;           // 4 key groups per warp, 8 lanes per key
	const int g16 = warp * 4 + grp;                      // key group 0..31
	pdl_trigger();
	// positions beyond the cache are never read: the length is clamped to the rows a head owns
	const int len = max(1, min(p.pos[b] + 1, (int)(p.kv_stride_h / AT_D)));
	const int per = (len + p.splits - 1) / p.splits;
	const int k_lo = min(split * per, len), k_hi = min(k_lo + per, len);
	const int nchunks = (k_hi - k_lo + AT_CHUNK - 1) / AT_CHUNK;
	const __half *kbase = p.kc + (size_t)b * p.kv_stride_b + (size_t)head * p.kv_stride_h;
	const __half *vbase = p.vc + (size_t)b * p.kv_stride_b + (size_t)head * p.kv_stride_h;

	__shared__ float s_m[AT_GROUPS], s_l[AT_GROUPS];
	float(*s_acc)[AT_D] = reinterpret_cast<float(*)[AT_D]>(at_smem);      // [AT_GROUPS][128], over the drained stages
	__shared__ int s_last;
	const uint32_t bar0 = smem_u32(at_smem + AT_STAGES * AT_STAGE_BYTES);
	if (tid == 0) {
		for (int s = 0; s < AT_STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
		fence_mbar_init();
	}
	__syncthreads();
	auto issue = [&](int c) {                // one thread: K and V rows of chunk c into stage c % AT_STAGES
		const int stage = c % AT_STAGES, key0 = k_lo + c * AT_CHUNK;
		const uint32_t bytes = (uint32_t)min(AT_CHUNK, k_hi - key0) * AT_D * 2u;
		const uint32_t dst = smem_u32(at_smem + stage * AT_STAGE_BYTES), bar = bar0 + 8 * stage;
		mbar_arrive_expect_tx(bar, 2u * bytes);
		bulk_load_1d(dst, kbase + (size_t)key0 * AT_D, bytes, bar);
		bulk_load_1d(dst + AT_STAGE_BYTES / 2, vbase + (size_t)key0 * AT_D, bytes, bar);
	};
	if (tid == 0)
		for (int c = 0; c < min(nchunks, AT_STAGES); ++c) issue(c);
	pdl_wait();                                          // q and the newest cache rows come from earlier kernels

	// this lane's 16 query dims (sub*8 .. +7 and 64 + sub*8 .. +7), pre-scaled
	float qf[16];
	{
		const __half *qp = p.q + (size_t)b * p.q_stride_b + head * AT_D + sub * 8;
		const uint4 a = *reinterpret_cast<const uint4 *>(qp), c = *reinterpret_cast<const uint4 *>(qp + 64);
		const __half2 *ha = reinterpret_cast<const __half2 *>(&a), *hc = reinterpret_cast<const __half2 *>(&c);
#pragma unroll
		for (int i = 0; i < 4; ++i) {
			const float2 f = __half22float2(ha[i]), g = __half22float2(hc[i]);
			qf[2 * i] = f.x * p.scale;
			qf[2 * i + 1] = f.y * p.scale;
			qf[8 + 2 * i] = g.x * p.scale;
			qf[8 + 2 * i + 1] = g.y * p.scale;
		}
	}
	const int fresh_lo = len - AT_FRESH;

	float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
	for (int i = 0; i < 16; ++i) acc[i] = 0.f;

	constexpr int KPG = AT_CHUNK / AT_GROUPS;       // keys per 8-lane group and chunk
	bool failed = false;
#pragma unroll 1
	for (int c = 0; c < nchunks; ++c) {
		const int stage = c % AT_STAGES, key0 = k_lo + c * AT_CHUNK;
		const int n = min(AT_CHUNK, k_hi - key0);
		const bool got = mbar_wait_bounded(bar0 + 8 * stage, (c / AT_STAGES) & 1);
		if (!__syncthreads_and(got)) {       // the same verdict for every thread
			failed = true;
			break;
		}
		const unsigned char *sK = at_smem + stage * AT_STAGE_BYTES, *sV = sK + AT_STAGE_BYTES / 2;
		uint4 kr[KPG][2], vr[KPG][2];
#pragma unroll
		for (int u = 0; u < KPG; ++u) {
			const int kk = g16 + AT_GROUPS * u, key = key0 + kk;
			if (kk < n) {
				const bool fresh = key >= fresh_lo;
				const __half *kp = fresh ? kbase + (size_t)key * AT_D : reinterpret_cast<const __half *>(sK) + kk * AT_D;
				const __half *vp = fresh ? vbase + (size_t)key * AT_D : reinterpret_cast<const __half *>(sV) + kk * AT_D;
				kr[u][0] = *reinterpret_cast<const uint4 *>(kp + sub * 8);
				kr[u][1] = *reinterpret_cast<const uint4 *>(kp + 64 + sub * 8);
				vr[u][0] = *reinterpret_cast<const uint4 *>(vp + sub * 8);
				vr[u][1] = *reinterpret_cast<const uint4 *>(vp + 64 + sub * 8);
			}
		}
#pragma unroll
		for (int u = 0; u < KPG; ++u) {
			const bool valid = g16 + AT_GROUPS * u < n;          // uniform within an 8-lane group
			float s = 0.f;
			if (valid) {
				const __half2 *h0 = reinterpret_cast<const __half2 *>(&kr[u][0]), *h1 = reinterpret_cast<const __half2 *>(&kr[u][1]);
#pragma unroll
				for (int i = 0; i < 4; ++i) {
					const float2 f = __half22float2(h0[i]), g = __half22float2(h1[i]);
					s = fmaf(qf[2 * i], f.x, s);
					s = fmaf(qf[2 * i + 1], f.y, s);
					s = fmaf(qf[8 + 2 * i], g.x, s);
					s = fmaf(qf[8 + 2 * i + 1], g.y, s);
				}
			}
			// all 32 lanes take part in the shuffles; the xor pattern stays inside the 8-lane group
			s += __shfl_xor_sync(0xffffffffu, s, 1);
			s += __shfl_xor_sync(0xffffffffu, s, 2);
			s += __shfl_xor_sync(0xffffffffu, s, 4);
			if (valid) {
				const float mn = fmaxf(m, s);
				const float corr = __expf(m - mn), pw = __expf(s - mn);
				l = l * corr + pw;
				const __half2 *h0 = reinterpret_cast<const __half2 *>(&vr[u][0]), *h1 = reinterpret_cast<const __half2 *>(&vr[u][1]);
#pragma unroll
				for (int i = 0; i < 4; ++i) {
					const float2 f = __half22float2(h0[i]), g = __half22float2(h1[i]);
					acc[2 * i] = fmaf(pw, f.x, acc[2 * i] * corr);
					acc[2 * i + 1] = fmaf(pw, f.y, acc[2 * i + 1] * corr);
					acc[8 + 2 * i] = fmaf(pw, g.x, acc[8 + 2 * i] * corr);
					acc[8 + 2 * i + 1] = fmaf(pw, g.y, acc[8 + 2 * i + 1] * corr);
				}
				m = mn;
			}
		}
		if (c + AT_STAGES < nchunks) {       // the stage is refilled once every thread has read it
			__syncthreads();
			if (tid == 0) issue(c + AT_STAGES);
		}
	}
	if (failed && tid == 0 && p.ws_ticket) atomicExch(p.ws_ticket + AT_STATUS_SLOT, 1);      // a bulk copy never completed

	// ---- merge the key groups of the CTA (fixed order) --------------------------------------------
	__syncthreads();                                     // every warp is done with the staged rows: the region becomes s_acc
	if (sub == 0) {
		s_m[g16] = m;
		s_l[g16] = l;
	}
#pragma unroll
	for (int i = 0; i < 8; ++i) {
		s_acc[g16][sub * 8 + i] = acc[i];
		s_acc[g16][64 + sub * 8 + i] = acc[8 + i];
	}
	__syncthreads();
	float M = -INFINITY;
#pragma unroll
	for (int g = 0; g < AT_GROUPS; ++g) M = fmaxf(M, s_m[g]);
	float L = 0.f, o = 0.f;            // thread tid < 128 owns output dim tid
	const int dim = tid & (AT_D - 1);
#pragma unroll 4
	for (int g = 0; g < AT_GROUPS; ++g) {
		const float w = (s_m[g] == -INFINITY) ? 0.f : __expf(s_m[g] - M);
		L = fmaf(s_l[g], w, L);
		o = fmaf(s_acc[g][dim], w, o);
	}
	const bool writer = tid < AT_D;

	const int bh = b * p.heads + head;
	if (p.splits == 1) {
		if (writer) p.out[(size_t)b * p.out_stride_b + head * AT_D + tid] = __float2half_rn(o / L);
		return;
	}
	float *wp = p.ws_partial + ((size_t)bh * p.splits + split) * 130;
	if (writer) __stcg(wp + 2 + tid, o);
	if (tid == 0) {
		__stcg(wp, M);
		__stcg(wp + 1, L);
	}
	// The ticket is an acquire-release read-modify-write at GPU scope after a CTA barrier: the partial
	// sums that this CTA's threads stored before the barrier are released with it, and the partials of
	// the CTAs that took a ticket earlier are acquired by it (and, through the next barrier, by every
	// thread of this CTA).  No separate fences.
	__syncthreads();
	if (tid == 0) {
		int t;
		asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.ws_ticket + bh) : "memory");
		const int last = (t == p.splits - 1);
		if (last) p.ws_ticket[bh] = 0;
		s_last = last;
	}
	__syncthreads();
	if (!s_last) {
		return;
	}
	const float *wb = p.ws_partial + (size_t)bh * p.splits * 130;
	if (writer) {
		// all partials of a batch of splits are requested at once, then folded into the running
		// (max, sum, output) in split order
		float Mg = -INFINITY, Lg = 0.f, og = 0.f;
		constexpr int MB = 12;
#pragma unroll 1
		for (int s0 = 0; s0 < p.splits; s0 += MB) {
			float ms[MB], ls[MB], os[MB];
#pragma unroll
			for (int j = 0; j < MB; ++j) {
				if (s0 + j < p.splits) {
					const float *src = wb + (size_t)(s0 + j) * 130;
					ms[j] = __ldcg(src);
					ls[j] = __ldcg(src + 1);
					os[j] = __ldcg(src + 2 + tid);
				}
			}
			float bm = Mg;
#pragma unroll
			for (int j = 0; j < MB; ++j)
				if (s0 + j < p.splits) bm = fmaxf(bm, ms[j]);
			const float keep = (Mg == -INFINITY) ? 0.f : __expf(Mg - bm);
			Lg *= keep;
			og *= keep;
#pragma unroll
			for (int j = 0; j < MB; ++j) {
				if (s0 + j < p.splits) {
					const float w = (ms[j] == -INFINITY) ? 0.f : __expf(ms[j] - bm);
					Lg = fmaf(ls[j], w, Lg);
					og = fmaf(os[j], w, og);
				}
			}
			Mg = bm;
		}
		p.out[(size_t)b * p.out_stride_b + head * AT_D + tid] = __float2half_rn(og / Lg);
	}
}

// ---- RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, fp32 inside, one fp16 rounding ----------------
// One CTA of 512 threads per row.  A thread keeps its first 16-byte unit of x (and of w) in
// registers across the reduction, so rows of up to 4096 elements are read once with a single
// round trip to memory; longer rows loop over the remaining units.
constexpr int RN_THREADS = 512;

__device__ __forceinline__ float rn_sumsq(const uint4 &v) {
	const __half2 *h = reinterpret_cast<const __half2 *>(&v);
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < 4; ++i) {
		const float2 f = __half22float2(h[i]);
		ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
	}
	return ss;
}

__device__ __forceinline__ uint4 rn_scale(const uint4 &v, const uint4 &g, float inv) {
	const __half2 *h = reinterpret_cast<const __half2 *>(&v), *gh = reinterpret_cast<const __half2 *>(&g);
	uint4 o;
	__half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
	for (int i = 0; i < 4; ++i) {
		const float2 f = __half22float2(h[i]), gg = __half22float2(gh[i]);
		oh[i] = __floats2half2_rn(f.x * inv * gg.x, f.y * inv * gg.y);
	}
	return o;
}

// With `rows` the input row m is x[rows[m]] (an embedding lookup: x is the table, the token ids come from an
// earlier kernel) and the row itself is also copied to `copy` (the residual stream of the first layer).
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_kernel(const __half *__restrict__ x, long long ldx, const __half *__restrict__ w,
															 __half *__restrict__ y, long long ldy, int K, float eps,
															 const long long *__restrict__ rows, __half *__restrict__ copy, long long ldc) {
	const int row = blockIdx.x, tid = threadIdx.x;
	const uint4 *wr = reinterpret_cast<const uint4 *>(w);
	uint4 *yr = reinterpret_cast<uint4 *>(y + (size_t)row * ldy);
	const int nu = K >> 3;
	pdl_trigger();
	uint4 g0 = make_uint4(0u, 0u, 0u, 0u), v0 = make_uint4(0u, 0u, 0u, 0u);
	if (tid < nu) g0 = __ldg(wr + tid);                 // the weight does not depend on earlier kernels
	pdl_wait();
	const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)(rows ? rows[row] : (long long)row) * ldx);
	if (tid < nu) v0 = xr[tid];
	if (copy) {
		uint4 *cr = reinterpret_cast<uint4 *>(copy + (size_t)row * ldc);
		if (tid < nu) cr[tid] = v0;
#pragma unroll 1
		for (int u = tid + RN_THREADS; u < nu; u += RN_THREADS) cr[u] = xr[u];
	}
	float ss = rn_sumsq(v0);
#pragma unroll 1
	for (int u = tid + RN_THREADS; u < nu; u += RN_THREADS) ss += rn_sumsq(xr[u]);
	__shared__ float s_part[RN_THREADS / 32];
#pragma unroll
	for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
	if ((tid & 31) == 0) s_part[tid >> 5] = ss;
	__syncthreads();
	float tot = 0.f;
#pragma unroll
	for (int i = 0; i < RN_THREADS / 32; ++i) tot += s_part[i];
	const float inv = rsqrtf(tot / (float)K + eps);
	if (tid < nu) yr[tid] = rn_scale(v0, g0, inv);
#pragma unroll 1
	for (int u = tid + RN_THREADS; u < nu; u += RN_THREADS) yr[u] = rn_scale(xr[u], __ldg(wr + u), inv);
}

}   // namespace gptq
