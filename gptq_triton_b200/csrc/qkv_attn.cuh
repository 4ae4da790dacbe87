// Decode step, one sequence: fused QKV projection + rotary embedding + KV-cache append + single-query attention
// in ONE kernel, one thread-block cluster of 8 CTAs per head.
//
// Why.  Attention of head h needs nothing but head h's q, k, v: the only all-to-all dependency between the QKV
// projection and the attention is inside a head.  A cluster keeps that exchange in distributed shared memory, so the
// kernel boundary between the two (a grid-wide dependency: drain, flush, re-launch, stage again) disappears.
//
//   phase 1  CTA r of the cluster takes K-slice r (K / 8 rows) of the head's 384 weight columns (q, k, v tiles of
//            128): 12 strips of 32 columns x K / 1024 chunks of 128 rows, streamed through per-warp rings of 2 KB
//            slots by 2-D TMA; raw-nibble MMA as in qmm_skinny.cuh; zero points, offsets and scales applied per chunk.
//   exchange every CTA writes its partial sums of q into ALL CTAs of the cluster and of k, v into the last CTA
//            (st.shared::cluster), cluster barrier, fixed-order sum: every CTA holds q, the last one also k, v.
//   phase 2  rotary; the last CTA appends the K / V row to the cache; CTA r attends to key split r of the cache
//            (8 keys x 256 bytes per ring slot, 1-D bulk copies queued in the same ring behind the weight chunks, so they
//            are in flight while phase 1 still runs; these rows were written by earlier decode steps or the prefill),
//            the last one also to the token's own key; online softmax in fp32.
//   merge    (max, sum, 128 outputs) of every CTA go to CTA 0 through distributed shared memory, cluster barrier,
//            CTA 0 folds the eight partials in order and writes the head's 128 outputs as fp16.
//   o_proj   (optional) every CTA receives the partials instead, forms the head's 128 outputs and multiplies them with its
//            share of the head's 128 rows of the output projection (K-slice = head, columns split over the 8 CTAs); the
//            per-head partial sums meet in global memory, where the last CTA to arrive for a column range adds them in
//            head order, adds the residual and writes the new hidden state with its sums of squares.
// RMSNorm of the input is folded in as in the decode kernels (sums of squares from the producing projection).
// Deterministic: every sum runs in a fixed order.  Waits on the rings are bounded (status 1); the cluster barriers are
// hardware barriers between CTAs that are scheduled together, and no CTA leaves before the last of them.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace gptq {

constexpr int QA_THREADS = 256;
#ifndef QA_CLUSTER_SIZE
#define QA_CLUSTER_SIZE 8
#endif
constexpr int QA_CLUSTER = QA_CLUSTER_SIZE;          // CTAs per head (8: measured; 4 halves the CTA count and doubles the K-slice)
constexpr int QA_D = 128;
constexpr int QA_SLOT = 2048;
constexpr int QA_COLS = 3 * QA_D;          // q, k, v columns of one head
constexpr int QA_MAX_NC = 8;               // chunks of 128 K-rows per CTA (K <= 8192)

struct QkvAttnParams {
	const __half *x;              // [K] hidden state of the token
	const int32_t *qz;            // [G, N / 8]
	const __half *sc;             // [G, N]
	int K, N, sec_stride, groupsize, nc, nstage;      // sec_stride: columns between the q, k and v sections (heads * 128)
	const __half *rms_w;          // or nullptr: x is used as it is
	const float *ss_in;
	int ss_tiles;
	float rms_eps;
	const __half *cos_t, *sin_t;  // [max_pos, 128]
	const int32_t *pos;           // [1]: position of the token = keys already cached
	int max_pos;
	__half *kc, *vc;              // [heads, max_pos, 128]
	long long kv_stride_h;
	float scale;
	__half *out;                  // [heads * 128]
	int *status;
	int off_bars, off_xs, off_zz, off_sc, off_part, off_gather, off_merge, off_attn, off_o;     // shared-memory layout
	// Optional third phase: the output projection (o_proj) of the block, y = residual + attn x deq(Wo).  The cluster of
	// head h owns the K-slice h (rows 128 h .. 128 h + 127 of Wo); its CTA r the columns [256 spw r, 256 spw (r + 1)).
	// Partial sums per head go to o_part [heads][o_N] (fp32); the last of the `heads` CTAs with the same r to arrive at
	// o_tickets[r] adds them in head order, adds the residual, writes y (fp16) and the sums of squares of y per 32 columns.
	int o_enable, o_N, o_groupsize, o_spw;          // o_spw: 32-column strips per warp = ceil(o_N / 32 / 64), at most 4
	const int32_t *o_qz;
	const __half *o_sc;
	const __half *o_res;
	float *o_part;
	int *o_tickets;
	__half *o_y;
	float *o_ss;
	// Tensor parallelism (o_proj is the row shard of this rank's heads): the all-reduce over the ranks is part of the final
	// reduction, with the protocol and the buffers of the decode kernel's fused exchange (qmm_skinny.cuh): the CTA that
	// holds a column range PUSHES its sums into every peer's receive buffer as {value, sequence} words, polls its own
	// buffer for the peers' words (bounded: two seconds, status 5) and adds in rank order; the residual is added on every rank.
	int ar_world, ar_rank, ar_tiles;              // ar_tiles = o_N / 128
	unsigned long long *ar_buf[8];
	unsigned *ar_seq;
};

__device__ __forceinline__ uint32_t qa_map_peer(uint32_t local_smem_addr, uint32_t rank) {
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
	return r;
}
__device__ __forceinline__ void qa_st_peer(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void qa_cluster_sync() {
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void qa_bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
				 "r"(bar)
				 : "memory");
}

// AR: with the all-reduce over tensor-parallel ranks in the final reduction (its own instance: the one-GPU kernel keeps
// its register allocation)
template <bool AR>
__global__ void __cluster_dims__(QA_CLUSTER, 1, 1) __launch_bounds__(QA_THREADS, 2)
	qkv_attn_kernel(const __grid_constant__ CUtensorMap tmw, const __grid_constant__ CUtensorMap tmo, const QkvAttnParams p) {
	extern __shared__ __align__(1024) unsigned char smem[];
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
	const int rank = blockIdx.x, head = blockIdx.y;            // cluster rank = K-slice = key split
	const int NST = p.nstage, nc = p.nc;
	unsigned char *xs = smem + p.off_xs;
	__half *s_zz = reinterpret_cast<__half *>(smem + p.off_zz);        // [nc][384] zero point (stored + 1)
	__half *s_sc = reinterpret_cast<__half *>(smem + p.off_sc);        // [nc][384] scale
	float *s_part = reinterpret_cast<float *>(smem + p.off_part);      // [nc][384] this CTA's sums per chunk
	float *s_gather = reinterpret_cast<float *>(smem + p.off_gather);  // [8 ranks][384] written by the peers
	float *s_merge = reinterpret_cast<float *>(smem + p.off_merge);    // [8 ranks][130] written by the peers (read on rank 0)
	float *s_q = reinterpret_cast<float *>(smem + p.off_attn);         // [128] rotated, rounded, pre-scaled query
	__half *s_kn = reinterpret_cast<__half *>(s_q + QA_D);             // [128] new key
	__half *s_vn = s_kn + QA_D;                                        // [128] new value
	float *s_wo = reinterpret_cast<float *>(s_vn + QA_D);              // [8 warps][128]
	float *s_wm = s_wo + 8 * QA_D, *s_wl = s_wm + 8;
	__shared__ float2 s_cs[QA_MAX_NC];                                 // per chunk: C = 1024 (SXe + SXo'), S = SXe + 16 SXo'
	__shared__ float s_inv;

	const uint32_t ring_w = smem_u32(smem + (size_t)warp * NST * QA_SLOT);
	const uint32_t bar_w = smem_u32(smem + p.off_bars) + warp * NST * 8;
	if (lane == 0) {
		for (int s = 0; s < NST; ++s) mbar_init(bar_w + 8 * s, 1);
		fence_mbar_init();
		if (warp == 0) tma_prefetch_desc(&tmw);
		if (warp == 1 && p.o_enable) tma_prefetch_desc(&tmo);
	}
	pdl_trigger();
	// the position comes from the previous decode step (several kernels ago), not from the kernel before this one
	int pos = p.pos[0];
	if (pos < 0 || pos >= p.max_pos) {            // never index the tables / the cache out of range
		if (tid == 0) atomicExch(p.status, 4);
		pos = -1;                                 // the token attends to nothing and its K / V row is dropped
	}
	const int n_old = max(pos, 0);                // keys 0 .. n_old - 1 are in the cache
	// this warp's loads: weight chunks j = warp, warp + 8, ... < 12 * nc (strip j % 12 of chunk j / 12), then the K and V
	// rows of its share of key split `rank`, 8 keys per load
	const int n_wloads = (12 * nc - warp + 7) / 8;
	const int per = ((n_old + QA_CLUSTER - 1) / QA_CLUSTER + 7) & ~7;
	const int k_lo = min(rank * per, n_old), k_hi = min(k_lo + per, n_old);
	const int per_w = (((k_hi - k_lo) + 7) / 8 + 7) & ~7;
	const int wk_lo = min(k_lo + warp * per_w, k_hi), wk_hi = min(wk_lo + per_w, k_hi);
	const int nkeys = wk_hi - wk_lo, n_aloads = 2 * ((nkeys + 7) >> 3);
	// o_proj: strips (rank * 8 + warp) * spw + j of the head's 128 rows of Wo
	const int o_strip0 = (rank * 8 + warp) * p.o_spw;
	const int n_oloads = p.o_enable ? max(0, min(p.o_spw, (p.o_N >> 5) - o_strip0)) : 0;
	const int n_loads = n_wloads + n_aloads + n_oloads;
	const __half *kb = p.kc + (size_t)head * p.kv_stride_h + (size_t)wk_lo * QA_D, *vb = p.vc + (size_t)head * p.kv_stride_h + (size_t)wk_lo * QA_D;
	int pr_j = 0, pr_stage = 0;
	auto produce = [&]() {
		if (pr_j >= n_loads) return;
		if (lane == 0) {
			const uint32_t bar = bar_w + 8 * pr_stage, dst = ring_w + pr_stage * QA_SLOT;
			if (pr_j < n_wloads) {
				const int j = warp + 8 * pr_j, cl = j / 12, strip = j - cl * 12;
				const int n0w = (strip >> 2) * p.sec_stride + head * QA_D + (strip & 3) * 32;
				mbar_arrive_expect_tx(bar, QA_SLOT);
				tma_load_2d(dst, &tmw, n0w, (rank * nc + cl) * 16, bar);
			} else if (pr_j >= n_wloads + n_aloads) {
				mbar_arrive_expect_tx(bar, QA_SLOT);
				tma_load_2d(dst, &tmo, (o_strip0 + pr_j - n_wloads - n_aloads) * 32, head * 16, bar);
			} else {
				const int a = pr_j - n_wloads, c = a >> 1;
				const uint32_t bytes = (uint32_t)min(8, nkeys - 8 * c) * (QA_D * 2);
				mbar_arrive_expect_tx(bar, bytes);
				qa_bulk_load_1d(dst, ((a & 1) ? vb : kb) + (size_t)c * 8 * QA_D, bytes, bar);
			}
		}
		++pr_j;
		if (++pr_stage == NST) pr_stage = 0;
	};
	int cs = 0;
	uint32_t cpar = 0;
	bool failed = false;
	auto slot_wait = [&]() -> bool {
		if (!failed && !__all_sync(0xffffffffu, mbar_wait_bounded(bar_w + 8 * cs, cpar))) failed = true;
		return !failed;
	};
	auto slot_done = [&]() {
		__syncwarp();
		if (++cs == NST) {
			cs = 0;
			cpar ^= 1u;
		}
		produce();
	};
	__syncwarp();
#pragma unroll 1
	for (int s = 0; s < NST; ++s) produce();
	// first half of a cluster barrier whose second half sits in front of the exchange: no CTA writes into a peer's
	// shared memory before every CTA of the cluster is running
	asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

	// ---- before the dependency wait: zero / scale strips of the CTA's chunks and columns, rotary table entry ----
	{
		const int nz = p.N >> 3;
#pragma unroll 1
		for (int i = tid; i < nc * 48; i += QA_THREADS) {
			const int cl = i / 48, u = i - cl * 48;                       // unit of 8 of the head's 384 columns
			const int n = (u >> 4) * p.sec_stride + head * QA_D + (u & 15) * 8;
			const int g = ((rank * nc + cl) * 128) / p.groupsize;
			const uint32_t zv = (uint32_t)__ldg(p.qz + (size_t)g * nz + (n >> 3));
			const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(p.sc + (size_t)g * p.N + n));
			uint4 ze;          // zero point (stored + 1) as fp16, two per word: (0x6401 + nibble) - 1024
			ze.x = h2_sub(0x64016401u + ((zv & 0xFu) | ((zv & 0xF0u) << 12)), MAGIC_1024);
			ze.y = h2_sub(0x64016401u + (((zv >> 8) & 0xFu) | (((zv >> 8) & 0xF0u) << 12)), MAGIC_1024);
			ze.z = h2_sub(0x64016401u + (((zv >> 16) & 0xFu) | (((zv >> 16) & 0xF0u) << 12)), MAGIC_1024);
			ze.w = h2_sub(0x64016401u + (((zv >> 24) & 0xFu) | (((zv >> 24) & 0xF0u) << 12)), MAGIC_1024);
			*reinterpret_cast<uint4 *>(s_zz + (size_t)cl * QA_COLS + u * 8) = ze;
			*reinterpret_cast<uint4 *>(s_sc + (size_t)cl * QA_COLS + u * 8) = sv;
		}
	}
	unsigned char *xs2 = smem + p.off_o;                                  // [8 warps][256 B] attention output of the head, staged like xs
	__half *s_ozz = reinterpret_cast<__half *>(xs2 + 8 * 256);                // [256 spw] zero point (stored + 1) of this CTA's o_proj columns
	__half *s_osc = s_ozz + 256 * 4;                                      // [256 spw] scale
	if (p.o_enable) {
		const int nz = p.o_N >> 3, g = (head * QA_D) / p.o_groupsize;
#pragma unroll 1
		for (int i = tid; i < 32 * p.o_spw; i += QA_THREADS) {            // units of 8 columns
			const int n = rank * 256 * p.o_spw + i * 8;
			if (n < p.o_N) {
				const uint32_t zv = (uint32_t)__ldg(p.o_qz + (size_t)g * nz + (n >> 3));
				const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(p.o_sc + (size_t)g * p.o_N + n));
				uint4 ze;
				ze.x = h2_sub(0x64016401u + ((zv & 0xFu) | ((zv & 0xF0u) << 12)), MAGIC_1024);
				ze.y = h2_sub(0x64016401u + (((zv >> 8) & 0xFu) | (((zv >> 8) & 0xF0u) << 12)), MAGIC_1024);
				ze.z = h2_sub(0x64016401u + (((zv >> 16) & 0xFu) | (((zv >> 16) & 0xF0u) << 12)), MAGIC_1024);
				ze.w = h2_sub(0x64016401u + (((zv >> 24) & 0xFu) | (((zv >> 24) & 0xF0u) << 12)), MAGIC_1024);
				*reinterpret_cast<uint4 *>(s_ozz + i * 8) = ze;
				*reinterpret_cast<uint4 *>(s_osc + i * 8) = sv;
			}
		}
	}
	float rc = 1.f, rs = 0.f;
	if (tid < QA_D) {
		rc = __half2float(__ldg(p.cos_t + (size_t)n_old * QA_D + tid));
		rs = __half2float(__ldg(p.sin_t + (size_t)n_old * QA_D + tid));
	}
	uint4 wq = make_uint4(0u, 0u, 0u, 0u);
	const int units = nc * 16;                                            // 16-byte units of the CTA's K-slice of x
	const bool rms = p.rms_w != nullptr;
	if (rms && tid < units) wq = __ldg(reinterpret_cast<const uint4 *>(p.rms_w + (rank * nc * 16 + tid) * 8));

	pdl_wait();                                   // x (and the sums of squares) come from the kernel before this one
	// ---- stage the K-slice of x (RMSNorm folded in), per-chunk sums of the staged values ----
	if (rms) {
		if (warp == 0) {
			float t = 0.f;
#pragma unroll 4
			for (int i = lane; i < p.ss_tiles; i += 32) t += __ldcg(p.ss_in + i);
#pragma unroll
			for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
			if (lane == 0) s_inv = rsqrtf(t / (float)p.K + p.rms_eps);
		}
		__syncthreads();
	}
	if (tid < 128) {                              // whole warps 0..3 (units <= 128): the shuffles below stay inside half-warps
		float e = 0.f, o = 0.f;
		if (tid < units) {
			uint4 t = __ldcg(reinterpret_cast<const uint4 *>(p.x + (rank * nc * 16 + tid) * 8));
			if (rms) {
				const float inv = s_inv;
				const uint32_t tv[4] = {t.x, t.y, t.z, t.w}, wv[4] = {wq.x, wq.y, wq.z, wq.w};
				uint32_t ov[4];
#pragma unroll
				for (int i = 0; i < 4; ++i) {
					const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&tv[i]));
					const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(&wv[i]));
					const __half2 h = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);      // x * inv_rms * w, one rounding
					ov[i] = *reinterpret_cast<const uint32_t *>(&h);
				}
				t = make_uint4(ov[0], ov[1], ov[2], ov[3]);
			}
			uint4 st;          // k order 0,4,1,5,2,6,3,7, the (1,5) and (3,7) pairs divided by 16
			st.x = __byte_perm(t.x, t.z, 0x5410);
			st.y = h2_mul(__byte_perm(t.x, t.z, 0x7632), 0x2C002C00u);
			st.z = __byte_perm(t.y, t.w, 0x5410);
			st.w = h2_mul(__byte_perm(t.y, t.w, 0x7632), 0x2C002C00u);
			*reinterpret_cast<uint4 *>(xs + tid * 16) = st;
			const float2 a0 = __half22float2(*reinterpret_cast<const __half2 *>(&st.x)), a1 = __half22float2(*reinterpret_cast<const __half2 *>(&st.y));
			const float2 a2 = __half22float2(*reinterpret_cast<const __half2 *>(&st.z)), a3 = __half22float2(*reinterpret_cast<const __half2 *>(&st.w));
			e = (a0.x + a0.y) + (a2.x + a2.y);
			o = (a1.x + a1.y) + (a3.x + a3.y);
		}
#pragma unroll
		for (int d = 1; d < 16; d <<= 1) {        // the 16 units of a chunk sit in one half-warp
			e += __shfl_xor_sync(0xffffffffu, e, d);
			o += __shfl_xor_sync(0xffffffffu, o, d);
		}
		if ((tid & 15) == 0 && tid < units) s_cs[tid >> 4] = make_float2(1024.f * (e + o), e + 16.f * o);
	}
	__syncthreads();

	// the residual values that the last CTA of a column range adds at the very end: fetched by every CTA while its
	// first weight chunks are on their way (not between the dependency wait and the first MMA), so that the reduction does not
	// end with two dependent trips to L2
	unsigned short pre_res0 = 0, pre_res1 = 0, pre_res2 = 0, pre_res3 = 0;      // column j * 256 + tid of the range; only looked at in the reduction
	if (p.o_enable && p.o_res) {
		const int n = rank * 256 * p.o_spw + tid;
		if (0 < p.o_spw && n < p.o_N) pre_res0 = __half_as_ushort(p.o_res[n]);
		if (1 < p.o_spw && n + 256 < p.o_N) pre_res1 = __half_as_ushort(p.o_res[n + 256]);
		if (2 < p.o_spw && n + 512 < p.o_N) pre_res2 = __half_as_ushort(p.o_res[n + 512]);
		if (3 < p.o_spw && n + 768 < p.o_N) pre_res3 = __half_as_ushort(p.o_res[n + 768]);
	}

	// one chunk (128 k x 32 columns in ring slot `cs`) times the staged x of that chunk: g[c][0] = raw sum of column 4 gid + c
	const int row_a = 2 * tig, row_b = 2 * tig + 1;
	const uint32_t ring_even = ring_w + row_a * 128 + ((gid ^ row_a) << 4);
	const uint32_t ring_odd = ring_w + row_b * 128 + ((gid ^ row_b) << 4);
	const bool have_row0 = gid == 0;                                    // one batch row
	auto chunk_mma = [&](const unsigned char *xc, float(&g)[4][2]) {
		const uint32_t ring_c = cs * QA_SLOT;
#pragma unroll
		for (int l = 0; l < 4; ++l) {
			uint4 q;
			asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
						 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
						 : "r"(((l & 1) ? ring_odd : ring_even) + ring_c + (l >> 1) * 1024));
			uint4 xb0 = make_uint4(0u, 0u, 0u, 0u);
			if (have_row0) xb0 = *reinterpret_cast<const uint4 *>(xc + ((l & 1) + 8 * (l >> 1)) * 16);
			const uint32_t qv[4] = {q.x, q.y, q.z, q.w};
			uint32_t a04[4], a15[4], a26[4], a37[4];
#pragma unroll
			for (int c = 0; c < 4; ++c) {
				const uint32_t w = qv[c], w8 = w >> 8;
				a04[c] = lop3_and_or(w, MASK_LO, MAGIC_1024);
				a15[c] = lop3_and_or(w, MASK_HI, MAGIC_1024);
				a26[c] = lop3_and_or(w8, MASK_LO, MAGIC_1024);
				a37[c] = lop3_and_or(w8, MASK_HI, MAGIC_1024);
			}
#pragma unroll
			for (int pr = 0; pr < 2; ++pr) {
				float(&d0)[4] = *reinterpret_cast<float(*)[4]>(&g[2 * pr][0]);
				mma16816(d0, a04[2 * pr], a04[2 * pr + 1], a15[2 * pr], a15[2 * pr + 1], xb0.x, xb0.y);
				mma16816(d0, a26[2 * pr], a26[2 * pr + 1], a37[2 * pr], a37[2 * pr + 1], xb0.z, xb0.w);
			}
		}
	};
	// ---- phase 1: this warp's weight chunks ----
	{
#pragma unroll 1
		for (int i = 0; i < n_wloads; ++i) {
			const int j = warp + 8 * i, cl = j / 12, strip = j - cl * 12;
			float g[4][2];
#pragma unroll
			for (int c = 0; c < 4; ++c) g[c][0] = g[c][1] = 0.f;
			if (!slot_wait()) break;
			chunk_mma(xs + cl * 256 + tig * 32, g);
			slot_done();
			if (tig == 0) {                       // batch row 0: columns strip * 32 + 4 * gid + 0..3
				const int col = strip * 32 + gid * 4;
				const float2 csv = s_cs[cl];
				const uint2 zr = *reinterpret_cast<const uint2 *>(s_zz + (size_t)cl * QA_COLS + col);
				const uint2 sr = *reinterpret_cast<const uint2 *>(s_sc + (size_t)cl * QA_COLS + col);
				const float2 z01 = __half22float2(*reinterpret_cast<const __half2 *>(&zr.x)), z23 = __half22float2(*reinterpret_cast<const __half2 *>(&zr.y));
				const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.x)), s23 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.y));
				float4 o;
				o.x = s01.x * (g[0][0] - fmaf(z01.x, csv.y, csv.x));
				o.y = s01.y * (g[1][0] - fmaf(z01.y, csv.y, csv.x));
				o.z = s23.x * (g[2][0] - fmaf(z23.x, csv.y, csv.x));
				o.w = s23.y * (g[3][0] - fmaf(z23.y, csv.y, csv.x));
				*reinterpret_cast<float4 *>(s_part + (size_t)cl * QA_COLS + col) = o;
			}
		}
	}
	__syncthreads();

	// ---- exchange: q to every CTA of the cluster, k and v to the last one ----
	asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
	{
		const uint32_t gather_local = smem_u32(s_gather + (size_t)rank * QA_COLS);
#pragma unroll 1
		for (int t = tid; t < QA_COLS; t += QA_THREADS) {
			float v = 0.f;
#pragma unroll 1
			for (int cl = 0; cl < nc; ++cl) v += s_part[(size_t)cl * QA_COLS + t];
			if (t < QA_D) {
#pragma unroll
				for (uint32_t r = 0; r < QA_CLUSTER; ++r) qa_st_peer(qa_map_peer(gather_local + t * 4, r), v);
			} else {
				qa_st_peer(qa_map_peer(gather_local + t * 4, QA_CLUSTER - 1), v);
			}
		}
	}
	qa_cluster_sync();
	const bool last = rank == QA_CLUSTER - 1;
	if (tid < QA_D) {
		float qv = 0.f, kv = 0.f, vv = 0.f;
#pragma unroll
		for (int r = 0; r < QA_CLUSTER; ++r) qv += s_gather[(size_t)r * QA_COLS + tid];
		if (last) {
#pragma unroll
			for (int r = 0; r < QA_CLUSTER; ++r) {
				kv += s_gather[(size_t)r * QA_COLS + QA_D + tid];
				vv += s_gather[(size_t)r * QA_COLS + 2 * QA_D + tid];
			}
		}
		// rotate-half through shared memory: out[d] = x[d] cos - x[d+64] sin (d < 64), x[d] cos + x[d-64] sin (d >= 64)
		s_wo[tid] = qv;
		s_wo[QA_D + tid] = kv;
		s_wo[2 * QA_D + tid] = vv;
	}
	__syncthreads();
	if (tid < QA_D) {
		const int d = tid;
		const float sgn = (d < 64) ? -rs : rs;
		s_q[d] = __half2float(__float2half_rn(fmaf(s_wo[d ^ 64], sgn, s_wo[d] * rc))) * p.scale;
		if (last) {
			const __half kh = __float2half_rn(fmaf(s_wo[QA_D + (d ^ 64)], sgn, s_wo[QA_D + d] * rc)), vh = __float2half_rn(s_wo[2 * QA_D + d]);
			s_kn[d] = kh;
			s_vn[d] = vh;
			if (pos >= 0) {
				const size_t off = (size_t)head * p.kv_stride_h + (size_t)pos * QA_D + d;
				p.kc[off] = kh;
				p.vc[off] = vh;
			}
		}
	}
	__syncthreads();

	// ---- phase 2: attention over this warp's keys; 8 lanes per key, a group takes keys g8 and g8 + 4 of a chunk ----
	const int g8 = lane >> 3, sub = lane & 7, rotp = sub >> 2;
	float qreg[2][8];
#pragma unroll
	for (int i = 0; i < 2; ++i)
#pragma unroll
		for (int e = 0; e < 8; ++e) qreg[i][e] = s_q[sub * 16 + ((i + rotp) & 1) * 8 + e];
	float m = -INFINITY, l = 0.f, acc[2][8];
#pragma unroll
	for (int i = 0; i < 2; ++i)
#pragma unroll
		for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
	{
		const int nchunk = (nkeys + 7) >> 3;
		const int n_iter = nchunk + ((last && warp == 0 && pos >= 0) ? 1 : 0);      // + the token's own key / value from shared memory
		const int row_off = g8 * (QA_D * 2) + sub * 32;
#pragma unroll 1
		for (int c = 0; c < n_iter; ++c) {
			const bool from_ring = c < nchunk;
			const int rows = from_ring ? min(8, nkeys - 8 * c) : 1;
			float sc[2] = {0.f, 0.f};
			if (from_ring && !slot_wait()) break;
			{
				const unsigned char *kp = (from_ring ? smem + (size_t)warp * NST * QA_SLOT + cs * QA_SLOT : reinterpret_cast<const unsigned char *>(s_kn)) + row_off;
#pragma unroll
				for (int h = 0; h < 2; ++h) {
					if (g8 + 4 * h < rows) {
#pragma unroll
						for (int i = 0; i < 2; ++i) {
							const uint4 kv4 = *reinterpret_cast<const uint4 *>(kp + h * 4 * (QA_D * 2) + ((i + rotp) & 1) * 16);
							const __half2 *kh = reinterpret_cast<const __half2 *>(&kv4);
#pragma unroll
							for (int e = 0; e < 4; ++e) {
								const float2 f = __half22float2(kh[e]);
								sc[h] = fmaf(qreg[i][2 * e], f.x, fmaf(qreg[i][2 * e + 1], f.y, sc[h]));
							}
						}
					}
					sc[h] += __shfl_xor_sync(0xffffffffu, sc[h], 1);
					sc[h] += __shfl_xor_sync(0xffffffffu, sc[h], 2);
					sc[h] += __shfl_xor_sync(0xffffffffu, sc[h], 4);
				}
			}
			if (from_ring) {
				slot_done();
				if (!slot_wait()) break;
			}
			{
				const unsigned char *vp = (from_ring ? smem + (size_t)warp * NST * QA_SLOT + cs * QA_SLOT : reinterpret_cast<const unsigned char *>(s_vn)) + row_off;
#pragma unroll
				for (int h = 0; h < 2; ++h) {
					if (g8 + 4 * h < rows) {
						const float mn = fmaxf(m, sc[h]);
						const float corr = __expf(m - mn), pw = __expf(sc[h] - mn);
						l = l * corr + pw;
#pragma unroll
						for (int i = 0; i < 2; ++i) {
							const uint4 vv4 = *reinterpret_cast<const uint4 *>(vp + h * 4 * (QA_D * 2) + ((i + rotp) & 1) * 16);
							const __half2 *vh = reinterpret_cast<const __half2 *>(&vv4);
#pragma unroll
							for (int e = 0; e < 4; ++e) {
								const float2 f = __half22float2(vh[e]);
								acc[i][2 * e] = fmaf(pw, f.x, acc[i][2 * e] * corr);
								acc[i][2 * e + 1] = fmaf(pw, f.y, acc[i][2 * e + 1] * corr);
							}
						}
						m = mn;
					}
				}
			}
			if (from_ring) slot_done();
		}
	}
	if (failed && lane == 0) atomicExch(p.status, 1);          // a load never arrived
	// merge the 4 key slots of the warp (lane bits 3, 4), then the 8 warps through shared memory
	{
		float mw = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
		mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
		const float f = (m == -INFINITY) ? 0.f : __expf(m - mw);
		l *= f;
		l += __shfl_xor_sync(0xffffffffu, l, 8);
		l += __shfl_xor_sync(0xffffffffu, l, 16);
		__syncthreads();                          // s_wo was the rotary scratch
#pragma unroll
		for (int i = 0; i < 2; ++i) {
			const int piece = (i + rotp) & 1;
#pragma unroll
			for (int e = 0; e < 8; ++e) {
				float av = acc[i][e] * f;
				av += __shfl_xor_sync(0xffffffffu, av, 8);
				av += __shfl_xor_sync(0xffffffffu, av, 16);
				if (g8 == 0) s_wo[warp * QA_D + sub * 16 + piece * 8 + e] = av;
			}
		}
		if (lane == 0) {
			s_wm[warp] = mw;
			s_wl[warp] = l;
		}
	}
	__syncthreads();
	// ---- merge of the cluster: every CTA's (max, sum, outputs) goes to every CTA; all of them form the same result ----
	if (tid < QA_D) {
		float Mx = -INFINITY;
#pragma unroll
		for (int w = 0; w < 8; ++w) Mx = fmaxf(Mx, s_wm[w]);
		float o = 0.f, Lx = 0.f;
#pragma unroll
		for (int w = 0; w < 8; ++w) {
			const float g = (s_wm[w] == -INFINITY) ? 0.f : __expf(s_wm[w] - Mx);
			o = fmaf(s_wo[w * QA_D + tid], g, o);
			Lx = fmaf(s_wl[w], g, Lx);
		}
		const uint32_t mine = smem_u32(s_merge + (size_t)rank * 130);
		const uint32_t r_hi = p.o_enable ? (uint32_t)QA_CLUSTER : 1u;      // without o_proj only CTA 0 needs it
		for (uint32_t r = 0; r < r_hi; ++r) {
			const uint32_t dst = qa_map_peer(mine, r);
			qa_st_peer(dst + (2 + tid) * 4, o);
			if (tid == 0) {
				qa_st_peer(dst, Mx);
				qa_st_peer(dst + 4, Lx);
			}
		}
	}
	qa_cluster_sync();
	__half *s_ah = s_kn;                                                  // [128] attention output of the head (fp16), over the new key
	if ((rank == 0 || p.o_enable) && tid < QA_D) {
		float Mg = -INFINITY;
#pragma unroll
		for (int r = 0; r < QA_CLUSTER; ++r) Mg = fmaxf(Mg, s_merge[r * 130]);
		float Lg = 0.f, og = 0.f;
#pragma unroll
		for (int r = 0; r < QA_CLUSTER; ++r) {
			const float ms = s_merge[r * 130];
			const float w = (ms == -INFINITY) ? 0.f : __expf(ms - Mg);
			Lg = fmaf(s_merge[r * 130 + 1], w, Lg);
			og = fmaf(s_merge[r * 130 + 2 + tid], w, og);
		}
		const __half ah = __float2half_rn(Lg > 0.f ? og / Lg : 0.f);
		if (rank == 0 && p.out) p.out[head * QA_D + tid] = ah;
		s_ah[tid] = ah;
	}
	if (!p.o_enable) return;

	// ---- phase 3: o_proj.  x = the head's attention output (128 values), this warp's strips of the head's rows of Wo ----
	__shared__ int s_last;
	__syncthreads();
	// every warp stages its own copy like xs (16 units of 8 k, permuted, odd pairs / 16) and forms (C, S) of the chunk for
	// itself: 256 bytes and a few shuffles, and no second CTA barrier
	unsigned char *xs2w = xs2 + warp * 256;
	float2 cs2;
	{
		float e = 0.f, o = 0.f;
		if (lane < 16) {
			const uint4 t = *reinterpret_cast<const uint4 *>(s_ah + lane * 8);
			uint4 st;
			st.x = __byte_perm(t.x, t.z, 0x5410);
			st.y = h2_mul(__byte_perm(t.x, t.z, 0x7632), 0x2C002C00u);
			st.z = __byte_perm(t.y, t.w, 0x5410);
			st.w = h2_mul(__byte_perm(t.y, t.w, 0x7632), 0x2C002C00u);
			*reinterpret_cast<uint4 *>(xs2w + lane * 16) = st;
			const float2 a0 = __half22float2(*reinterpret_cast<const __half2 *>(&st.x)), a1 = __half22float2(*reinterpret_cast<const __half2 *>(&st.y));
			const float2 a2 = __half22float2(*reinterpret_cast<const __half2 *>(&st.z)), a3 = __half22float2(*reinterpret_cast<const __half2 *>(&st.w));
			e = (a0.x + a0.y) + (a2.x + a2.y);
			o = (a1.x + a1.y) + (a3.x + a3.y);
		}
#pragma unroll
		for (int d = 1; d < 16; d <<= 1) {
			e += __shfl_xor_sync(0xffffffffu, e, d);
			o += __shfl_xor_sync(0xffffffffu, o, d);
		}
		e = __shfl_sync(0xffffffffu, e, 0);
		o = __shfl_sync(0xffffffffu, o, 0);
		cs2 = make_float2(1024.f * (e + o), e + 16.f * o);
		__syncwarp();
	}
#pragma unroll 1
	for (int j = 0; j < n_oloads; ++j) {
		float g[4][2];
#pragma unroll
		for (int c = 0; c < 4; ++c) g[c][0] = g[c][1] = 0.f;
		if (!slot_wait()) break;
		chunk_mma(xs2w + tig * 32, g);
		slot_done();
		if (tig == 0) {
			const int lc = (warp * p.o_spw + j) * 32 + gid * 4;          // column inside this CTA's range
			const float2 csv = cs2;
			const uint2 zr = *reinterpret_cast<const uint2 *>(s_ozz + lc);
			const uint2 sr = *reinterpret_cast<const uint2 *>(s_osc + lc);
			const float2 z01 = __half22float2(*reinterpret_cast<const __half2 *>(&zr.x)), z23 = __half22float2(*reinterpret_cast<const __half2 *>(&zr.y));
			const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.x)), s23 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.y));
			float4 o;
			o.x = s01.x * (g[0][0] - fmaf(z01.x, csv.y, csv.x));
			o.y = s01.y * (g[1][0] - fmaf(z01.y, csv.y, csv.x));
			o.z = s23.x * (g[2][0] - fmaf(z23.x, csv.y, csv.x));
			o.w = s23.y * (g[3][0] - fmaf(z23.y, csv.y, csv.x));
			__stcg(reinterpret_cast<float4 *>(p.o_part + (size_t)head * p.o_N + rank * 256 * p.o_spw + lc), o);
		}
	}
	if (failed && lane == 0) atomicExch(p.status, 1);
	// the ticket is an acquire-release atomic at GPU scope after the CTA barrier: it releases the partial sums this CTA
	// stored and acquires those of the CTAs (same rank, other heads) that arrived earlier
	__syncthreads();
	if (tid == 0) {
		int t;
		asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.o_tickets + rank) : "memory");
		const int last_one = (t == (int)gridDim.y - 1);
		if (last_one) p.o_tickets[rank] = 0;      // ready for the next launch
		s_last = last_one;
	}
	__syncthreads();
	if (!s_last) return;
	// The last CTA of this column range adds the heads' partial sums.  256 threads = (64 spw column quads) x (4 / spw head
	// groups): every thread has the float4 loads of its heads in flight at once (one trip to L2), the head groups are then
	// added in order through shared memory (the ring is idle by now), so the sum has a fixed order.
	{
		float *s_red = reinterpret_cast<float *>(smem);                   // [head group][256 spw]
		const int ncol = 256 * p.o_spw, quads = ncol >> 2, hsplit = QA_THREADS / quads;
		const int quad = tid % quads, hg = tid / quads;
		const int H = (int)gridDim.y, hper = (H + hsplit - 1) / hsplit;
		const int h_lo = min(hg * hper, H), h_hi = min(h_lo + hper, H);
		const int n4 = rank * ncol + quad * 4;
		float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
		if (n4 < p.o_N) {
#pragma unroll 1
			for (int h0 = h_lo; h0 < h_hi; h0 += 16) {
				float4 part[16];
#pragma unroll
				for (int k = 0; k < 16; ++k)
					part[k] = (h0 + k < h_hi) ? __ldcg(reinterpret_cast<const float4 *>(p.o_part + (size_t)(h0 + k) * p.o_N + n4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
				for (int k = 0; k < 16; ++k) {
					v.x += part[k].x;
					v.y += part[k].y;
					v.z += part[k].z;
					v.w += part[k].w;
				}
			}
		}
		*reinterpret_cast<float4 *>(s_red + (size_t)hg * ncol + quad * 4) = v;
		__shared__ unsigned s_seq[8];
		const int tile0 = (rank * ncol) >> 7;     // first 128-column tile of this CTA's range; the range holds 2 spw tiles
		if (AR && tid < 2 * p.o_spw && tile0 + tid < p.ar_tiles) s_seq[tid] = p.ar_seq[tile0 + tid] + 1u;      // left by the previous launch on these buffers
		__syncthreads();
		float tsum[4] = {0.f, 0.f, 0.f, 0.f};
		if (AR) {
			// own sums first, pushed to every peer before anything is waited for
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const int c = j * 256 + tid, n = rank * ncol + c;
				if (j < p.o_spw && n < p.o_N) {
					float t = 0.f;
					for (int g = 0; g < hsplit; ++g) t += s_red[(size_t)g * ncol + c];
					tsum[j] = t;
					const unsigned seq = s_seq[(n >> 7) - tile0];
					const size_t slot = (size_t)(seq & 1u) * ((size_t)8 * p.ar_tiles * 2048) + ((size_t)p.ar_rank * p.ar_tiles + (n >> 7)) * 2048 + (n & 127);
					const unsigned long long w = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(t);
#pragma unroll 1
					for (int r = 0; r < p.ar_world; ++r)
						if (r != p.ar_rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.ar_buf[r] + slot), "l"(w) : "memory");
				}
			}
		}
		const unsigned long long t_start = global_timer_ns();
		bool peers_ok = true;
#pragma unroll(AR ? 4 : 1)
		for (int j = 0; j < 4; ++j) {             // a warp takes 32 consecutive columns = one sum-of-squares tile
			if (j >= p.o_spw) break;
			const int c = j * 256 + tid, n = rank * ncol + c;
			float sq = 0.f;
			if (n < p.o_N) {
				float t = 0.f;
				if (AR) {
					const unsigned seq = s_seq[(n >> 7) - tile0];
					const size_t half = (size_t)(seq & 1u) * ((size_t)8 * p.ar_tiles * 2048);
#pragma unroll 1
					for (int r = 0; r < p.ar_world; ++r) {           // rank order: identical sums on every rank
						if (r == p.ar_rank) {
							t += tsum[j];
							continue;
						}
						const unsigned long long *src = p.ar_buf[p.ar_rank] + half + ((size_t)r * p.ar_tiles + (n >> 7)) * 2048 + (n & 127);
						unsigned long long w;
#pragma unroll 1
						for (;;) {
							asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
							if ((unsigned)(w >> 32) == seq) break;
							if (global_timer_ns() - t_start > 2000000000ull) {      // a peer never arrived
								peers_ok = false;
								break;
							}
						}
						t += __uint_as_float((unsigned)w);
					}
				} else {
					for (int g = 0; g < hsplit; ++g) t += s_red[(size_t)g * ncol + c];
				}
				t += __half2float(__ushort_as_half(j == 0 ? pre_res0 : (j == 1 ? pre_res1 : (j == 2 ? pre_res2 : pre_res3))));
				const __half hv = __float2half_rn(t);
				p.o_y[n] = hv;
				const float f = __half2float(hv);
				sq = f * f;
			}
			if (p.o_ss) {
#pragma unroll
				for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
				if (lane == 0 && n < p.o_N) p.o_ss[n >> 5] = sq;
			}
		}
		if (AR) {
			if (!peers_ok) atomicExch(p.status, 5);
			if (tid < 2 * p.o_spw && tile0 + tid < p.ar_tiles) p.ar_seq[tile0 + tid] = s_seq[tid];
		}
	}
}

}   // namespace gptq
