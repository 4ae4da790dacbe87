// One persistent kernel for a whole decode step of a quantised LLaMA decoder (batch rows M <= 8, one GPU).
//
// Why.  Run as one kernel per projection, a decode layer is five short HBM-bound kernels in a dependency
// chain; each pays its own prologue and tail while HBM idles.  Here ONE grid of co-resident CTAs (two per SM,
// cooperative launch) walks through all layers.  Per layer there are five phases separated by grid-wide
// barriers (bounded spins on a counter in global memory):
//     QKV projection -> single-query attention -> o_proj -> fused gate/up -> down_proj.
//
// Streaming.  Every warp owns a ring of 2 KB slots in shared memory and a list of loads that runs through ALL
// phases of ALL layers: its weight chunks (32 columns x 128 K-rows, 2-D tiled bulk copies with the 128-byte
// swizzle) of the projections and, in the attention phases, its rows of the KV cache (8 keys x 256 bytes,
// 1-D bulk copies).  A slot is refilled with the warp's next load as soon as it has been consumed, whatever
// phase that load belongs to: weights and old cache rows do not depend on activations, so the ring never
// drains at a phase boundary and HBM keeps streaming while the CTAs wait at a barrier.
//
// Deferred epilogues.  A projection phase ends by writing its fp32 partial sums per K-split to scratch memory
// (plain stores, released by the barrier).  The NEXT phase folds the reduction over the splits and the
// element-wise work into the staging of its own input:
//     QKV    : h = fp16(residual + sum of down_proj partials) (layer 0: the embedding row); x = fp16(h * w_ln1)
//     ATTN   : q, k, v = inv_rms * sum of QKV partials; rotary; the new K / V row goes into the cache
//     O      : x = merged attention output of the key splits
//     GATE/UP: h = fp16(residual + sum of o_proj partials); x = fp16(h * w_ln2)
//     DOWN   : x = fp16(silu(inv_rms * G) * (inv_rms * U))
// RMSNorm is applied as x = h * w before the projection and the scalar 1 / rms(h) after it (the projection is
// linear), so nobody has to wait for the full sum of squares: the CTAs of column tile 0 leave per-split sums.
// All sums run in a fixed order: results are deterministic.
//
// Math of a projection phase: as in qmm_skinny.cuh (raw nibbles as the A operand of mma.sync.m16n8k16,
// zero points and the 1024-offsets removed from per-group sums of x, scales applied in fp32 per group).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace gptq {

constexpr int CH_THREADS = 256;
constexpr int CH_D = 128;                  // head dim
constexpr int CH_SLOT = 2048;
constexpr int CH_MAX_M = 8;
constexpr int CH_MAX_SPLITS = 8;           // K-splits of a projection, key splits of the attention (one batch of loads when they are summed)

enum { CH_QKV = 0, CH_ATTN = 1, CH_O = 2, CH_GU = 3, CH_DOWN = 4, CH_NPHASE = 5 };
enum { CH_W_QKV = 0, CH_W_O = 1, CH_W_GATE = 2, CH_W_UP = 3, CH_W_DOWN = 4 };

// Status word values (same word as the other kernels' status): 1 a load never completed, 4 position out of
// range, 7 a grid barrier timed out (the grid was not co-resident, or a CTA gave up).

struct alignas(128) ChainLayer {
	CUtensorMap tm[5];                     // qkv, o, gate, up, down: int32 [K/8, N], box 32 columns x 16 rows, 128-byte swizzle
	const int32_t *qz[5];
	const __half *sc[5];
	const __half *ln1, *ln2;               // RMSNorm weights before attention / before the MLP
	__half *kc, *vc;                       // KV cache of the layer [M, heads, max_seq, 128]
};

struct ChainPlan {
	int K, N, tiles, splitk, cps, total_chunks, nstream, w0;      // w0: index of the (first) weight tensor in ChainLayer
};

struct ChainParams {
	const ChainLayer *layers;
	int n_layers, M, hidden, inter, heads, groupsize, spg;
	ChainPlan plan[CH_NPHASE];             // plan[CH_ATTN] is unused
	int attn_splits;
	int nstage;
	int off_bars, off_xs, off_zz, off_sc, off_cs, off_red, strip_groups;      // shared-memory layout
	const __half *embed;                   // [vocab, hidden]
	const long long *tok;                  // [M] token fed in this step
	const int32_t *pos;                    // [M] its position = number of keys already in the cache
	const __half *cos_t, *sin_t;           // [max_pos, 128]
	int max_pos;                           // rows of the tables and of the cache
	long long kv_stride_b, kv_stride_h;    // elements
	float eps, scale;
	float *p_qkv, *p_attn, *p_o, *p_gu, *p_down;       // partial sums per split
	__half *hA, *hB;                       // residual stream entering the layer / after attention [M, hidden]
	float *ss_a, *ss_b;                    // sums of squares of hA / hB per K-split
	__half *h_out;                         // final hidden state [M, hidden] (before the last norm)
	float *ss_f;                           // its sums of squares per 32 columns [M, hidden / 32]
	unsigned *sync;                        // [0] barrier counter, [1] exit counter, [2] abort flag
	int *status;
};

struct ChainJob {
	int n;                                 // loads of this warp in the phase
	int attn;
	const CUtensorMap *tm0, *tm1;
	int n0w, w_lo, nw;                     // weight chunks [w_lo, w_lo + nw) of column strip n0w, stream 0 then stream 1
	const __half *kb, *vb;                 // first cache row of the warp's key range
	int nkeys;
};

__device__ __forceinline__ void ch_bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
				 "r"(bar)
				 : "memory");
}

__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned *p) {
	unsigned v;
	asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
	return v;
}

// The loads of the calling warp in phase idx.  Runs once per warp and phase (twice: for the producer and for the
// consumer side), so it is kept out of line: the streaming loops stay small.
__device__ __noinline__ int chain_make_job(const ChainParams &P, int idx, const int *s_pos, ChainJob *out) {
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, b = blockIdx.x;
	const int wn = warp & 3, kw = warp >> 2;
	ChainJob j;
	j.n = 0; j.attn = 0; j.tm0 = j.tm1 = nullptr; j.n0w = j.w_lo = j.nw = 0; j.kb = j.vb = nullptr; j.nkeys = 0;
	const int layer = idx / CH_NPHASE, kind = idx - layer * CH_NPHASE;
	const ChainLayer *L = P.layers + layer;
	if (kind == CH_ATTN) {
		j.attn = 1;
		const int units = P.M * P.heads;
		if (b < units * P.attn_splits) {
			const int unit = b / P.attn_splits, sp = b - unit * P.attn_splits;
			const int r = unit / P.heads, head = unit - r * P.heads;
			const int n_old = max(s_pos[r], 0);                                   // keys 0 .. n_old-1 are in the cache
			const int per = ((n_old + P.attn_splits - 1) / P.attn_splits + 7) & ~7;
			const int k_lo = min(sp * per, n_old), k_hi = min(k_lo + per, n_old);
			const int per_w = (((k_hi - k_lo) + 7) / 8 + 7) & ~7;
			const int wk_lo = min(k_lo + warp * per_w, k_hi), wk_hi = min(wk_lo + per_w, k_hi);
			j.nkeys = wk_hi - wk_lo;
			j.n = 2 * ((j.nkeys + 7) / 8);
			const size_t off = (size_t)r * P.kv_stride_b + (size_t)head * P.kv_stride_h + (size_t)wk_lo * CH_D;
			j.kb = L->kc + off;
			j.vb = L->vc + off;
		}
	} else {
		const ChainPlan &pl = P.plan[kind];
		if (b < pl.tiles * pl.splitk) {
			const int split = b / pl.tiles, tile = b - split * pl.tiles;
			const int c_lo = split * pl.cps, c_hi = min(c_lo + pl.cps, pl.total_chunks);
			const int per_w = (c_hi - c_lo + 1) / 2;
			const int w_lo = min(c_lo + kw * per_w, c_hi), w_hi = min(w_lo + per_w, c_hi);
			j.tm0 = &L->tm[pl.w0];
			j.tm1 = &L->tm[pl.w0 + pl.nstream - 1];
			j.n0w = tile * 128 + wn * 32;
			j.w_lo = w_lo;
			j.nw = w_hi - w_lo;
			j.n = j.nw * pl.nstream;
		}
	}
	__syncwarp();
	if (lane == 0) *out = j;
	__syncwarp();
	return j.n;
}

// ---- helpers of the staging code -----------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
	const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
	for (int i = 0; i < 4; ++i) {
		const float2 t = __half22float2(h[i]);
		f[2 * i] = t.x;
		f[2 * i + 1] = t.y;
	}
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
	uint4 v;
	__half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
	for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
	return v;
}

// Staged x: units of 8 k in the order 0,4,1,5,2,6,3,7, the (1,5) and (3,7) pairs divided by 16 (the order and
// scaling in which the raw nibble pairs of a packed word meet them in the MMA).
__device__ __forceinline__ void store_x_unit(unsigned char *xs_row, int unit, const uint4 &t) {
	uint4 o;
	o.x = __byte_perm(t.x, t.z, 0x5410);
	o.y = h2_mul(__byte_perm(t.x, t.z, 0x7632), 0x2C002C00u);
	o.z = __byte_perm(t.y, t.w, 0x5410);
	o.w = h2_mul(__byte_perm(t.y, t.w, 0x7632), 0x2C002C00u);
	*reinterpret_cast<uint4 *>(xs_row + unit * 16) = o;
}
// one element (k relative to the slice) of the same layout
__device__ __forceinline__ void store_x_elem(unsigned char *xs_row, int k_rel, float v) {
	const int e = k_rel & 7;
	__half h = __float2half_rn(v);
	if (e & 1) h = __hmul(h, __float2half_rn(0.0625f));
	reinterpret_cast<__half *>(xs_row + (k_rel >> 3) * 16)[((e & 3) << 1) | (e >> 2)] = h;
}

__global__ void __launch_bounds__(CH_THREADS, 2) decode_chain_kernel(const __grid_constant__ ChainParams P) {
	extern __shared__ __align__(1024) unsigned char smem[];
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int wn = warp & 3, kw = warp >> 2, gid = lane >> 2, tig = lane & 3;
	const int b = blockIdx.x, G = gridDim.x;
	const int NST = P.nstage;
	const int n_phase = P.n_layers * CH_NPHASE;

	unsigned char *xs = smem + P.off_xs;
	__half *s_zz = reinterpret_cast<__half *>(smem + P.off_zz);
	__half *s_sc = reinterpret_cast<__half *>(smem + P.off_sc);
	float2 *s_cs = reinterpret_cast<float2 *>(smem + P.off_cs);
	float *red = reinterpret_cast<float *>(smem + P.off_red);
	__shared__ int s_pos[CH_MAX_M];
	__shared__ float s_part[CH_THREADS / 32];
	__shared__ int s_ok;
	__shared__ ChainJob s_job[CH_THREADS / 32], s_cjob[CH_THREADS / 32];      // producer's / consumer's current job per warp

	// ---- per-warp ring ----------------------------------------------------------------------------
	const uint32_t ring_w = smem_u32(smem + (size_t)warp * NST * CH_SLOT);
	const uint32_t bar_w = smem_u32(smem + P.off_bars) + warp * NST * 8;
	if (lane == 0) {
		for (int s = 0; s < NST; ++s) mbar_init(bar_w + 8 * s, 1);
		fence_mbar_init();
	}
	if (tid < P.M) {
		int p = P.pos[tid];
		if (p < 0 || p >= P.max_pos) {            // never index the tables / the cache out of range
			atomicExch(P.status, 4);
			p = -1;                               // the row attends to nothing and its K / V are dropped
		}
		s_pos[tid] = p;
	}
	if (tid == 0 && (smem_u32(smem) & 1023u) != 0) atomicExch(P.status, 2);
	__syncthreads();

	// producer: the warp's loads of all phases in order (the description of the current job lives in shared
	// memory: only lane 0 needs it, and registers are scarce in the main loops); consumer: (stage, parity) of the
	// next slot to read
	int pr_idx = -1, pr_j = 0, pr_n = 0, pr_stage = 0, outstanding = 0;
	auto produce = [&]() {
		if (pr_j >= pr_n) {                        // rare: on to the warp's next phase with loads
			while (pr_j >= pr_n && pr_idx + 1 < n_phase) {
				++pr_idx;
				pr_n = chain_make_job(P, pr_idx, s_pos, &s_job[warp]);
				pr_j = 0;
			}
			if (pr_j >= pr_n) return;
		}
		if (lane == 0) {
			const ChainJob &pj = s_job[warp];
			const uint32_t bar = bar_w + 8 * pr_stage, dst = ring_w + pr_stage * CH_SLOT;
			if (pj.attn) {
				const int c = pr_j >> 1;
				const uint32_t bytes = (uint32_t)min(8, pj.nkeys - 8 * c) * (CH_D * 2);
				mbar_arrive_expect_tx(bar, bytes);
				ch_bulk_load_1d(dst, ((pr_j & 1) ? pj.vb : pj.kb) + (size_t)c * 8 * CH_D, bytes, bar);
			} else {
				const int st = (pr_j >= pj.nw) ? 1 : 0;
				mbar_arrive_expect_tx(bar, CH_SLOT);
				tma_load_2d(dst, st ? pj.tm1 : pj.tm0, pj.n0w, (pj.w_lo + pr_j - st * pj.nw) * 16, bar);
			}
		}
		++pr_j;
		++outstanding;
		if (++pr_stage == NST) pr_stage = 0;
	};
	int cs = 0;
	uint32_t cpar = 0;
	bool failed = false;
	auto slot_wait = [&]() -> bool {
		if (failed) return false;
		if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_w + 8 * cs, cpar))) failed = true;      // one verdict for the whole warp
		return !failed;
	};
	auto slot_done = [&]() {                       // every lane has read the slot: refill it with the next load
		__syncwarp();
		--outstanding;
		if (++cs == NST) {
			cs = 0;
			cpar ^= 1u;
		}
		produce();
	};
#pragma unroll 1
	for (int s = 0; s < NST; ++s) produce();

	// ---- grid barrier ---------------------------------------------------------------------------------
	auto grid_arrive = [&]() {
		__syncthreads();
		if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.sync) : "memory");
	};
	auto grid_wait = [&](unsigned target) -> bool {
		if (tid == 0) {
			bool ok = true;
			unsigned long long t0 = 0;
			unsigned it = 0;
			while (ld_relaxed_u32(P.sync) < target) {
				if ((++it & 63u) == 0) {
					if (ld_relaxed_u32(P.sync + 2) != 0) {          // another CTA gave up
						ok = false;
						break;
					}
					const unsigned long long now = global_timer_ns();
					if (t0 == 0) t0 = now;
					else if (now - t0 > 2000000000ull) {
						atomicExch(P.status, 7);
						atomicExch(P.sync + 2, 1u);
						ok = false;
						break;
					}
				}
			}
			__threadfence();
			s_ok = ok ? 1 : 0;
		}
		__syncthreads();
		return s_ok != 0;
	};

	// ---- loads that do not depend on activations, issued BEFORE the barrier of the phase that uses them ----
	// projection: the CTA's zero / scale strips (two items of 8 columns per thread) and, for QKV and gate/up, the
	// RMSNorm weights of the thread's unit of x; attention: cos / sin of the thread's head dim at the token's position
	uint32_t pre_z[2] = {0u, 0u};
	uint4 pre_sv[2], pre_w;
	pre_sv[0] = pre_sv[1] = pre_w = make_uint4(0u, 0u, 0u, 0u);
	auto pre_issue = [&](int idx) {
		if (idx >= n_phase) return;
		const int layer = idx / CH_NPHASE, kind = idx - layer * CH_NPHASE;
		const ChainLayer *L = P.layers + layer;
		if (kind == CH_ATTN) {
			if (b < P.M * P.heads * P.attn_splits && tid < CH_D) {
				const int r = (b / P.attn_splits) / P.heads;
				const size_t o = (size_t)max(s_pos[r], 0) * CH_D + tid;
				pre_w.x = __half_as_ushort(__ldg(P.cos_t + o));
				pre_w.y = __half_as_ushort(__ldg(P.sin_t + o));
			}
			return;
		}
		const ChainPlan &pl = P.plan[kind];
		if (b >= pl.tiles * pl.splitk) return;
		const int split = b / pl.tiles, tile = b - split * pl.tiles;
		const int n0 = tile * 128;
		const int c_lo = split * pl.cps, c_hi = min(c_lo + pl.cps, pl.total_chunks);
		const int g_lo = (c_lo * 128) / P.groupsize;
		const int ng = (c_hi * 128 - 1) / P.groupsize - g_lo + 1;
		const int n_strip = pl.nstream * ng * 16, nz = pl.N >> 3;
#pragma unroll
		for (int jj = 0; jj < 2; ++jj) {
			const int i = tid + jj * CH_THREADS;
			if (i < n_strip) {
				const int rr = i >> 4, c = i & 15;
				const int s = (rr >= ng) ? 1 : 0, gi = rr - s * ng;
				pre_z[jj] = (uint32_t)__ldg(L->qz[pl.w0 + s] + (size_t)(g_lo + gi) * nz + (n0 >> 3) + c);
				pre_sv[jj] = __ldg(reinterpret_cast<const uint4 *>(L->sc[pl.w0 + s] + (size_t)(g_lo + gi) * pl.N + n0 + c * 8));
			}
		}
		if ((kind == CH_QKV || kind == CH_GU) && tid < (c_hi - c_lo) * 16)
			pre_w = __ldg(reinterpret_cast<const uint4 *>((kind == CH_QKV ? L->ln1 : L->ln2) + (c_lo * 16 + tid) * 8));
	};
	pre_issue(0);

	bool alive = true;
#pragma unroll 1
	for (int idx = 0; idx < n_phase && alive; ++idx) {
		const int layer = idx / CH_NPHASE, kind = idx - layer * CH_NPHASE;
		const ChainLayer *L = P.layers + layer;
		if (idx > 0 && !grid_wait((unsigned)idx * (unsigned)G)) {
			alive = false;
			break;
		}
		chain_make_job(P, idx, s_pos, &s_cjob[warp]);

		if (kind == CH_ATTN) {
			// =========================== single-query attention over the cache ===========================
			const int units = P.M * P.heads;
			if (b < units * P.attn_splits) {
				const int unit = b / P.attn_splits, sp = b - unit * P.attn_splits;
				const int r = unit / P.heads, head = unit - r * P.heads;
				const int pos = s_pos[r];
				const bool last_split = (sp == P.attn_splits - 1);
				float *s_raw = reinterpret_cast<float *>(xs);                      // [3][128] q, k, v before rotary
				float *s_q = s_raw + 3 * CH_D;                                     // [128] rotated, rounded, pre-scaled
				__half *s_kn = reinterpret_cast<__half *>(s_q + CH_D);             // [128] new key
				__half *s_vn = s_kn + CH_D;                                        // [128] new value
				float *s_wo = reinterpret_cast<float *>(s_vn + CH_D);              // [8 warps][128]
				float *s_wm = s_wo + 8 * CH_D, *s_wl = s_wm + 8;                   // [8], [8]
				const ChainPlan &pq = P.plan[CH_QKV];
				if (tid < CH_D) {
					// all partial sums of this thread's q, k, v element and the sums of squares in one batch of loads
					float ssv[CH_MAX_SPLITS], pv[3][CH_MAX_SPLITS];
					const float *src = P.p_qkv + (size_t)r * pq.N + head * CH_D + tid;
#pragma unroll
					for (int s = 0; s < CH_MAX_SPLITS; ++s) {
						if (s < pq.splitk) {
							ssv[s] = __ldcg(P.ss_a + s * P.M + r);
#pragma unroll
							for (int sec = 0; sec < 3; ++sec) pv[sec][s] = __ldcg(src + (size_t)s * P.M * pq.N + sec * P.hidden);
						}
					}
					float ssum = 0.f, v3[3] = {0.f, 0.f, 0.f};
#pragma unroll
					for (int s = 0; s < CH_MAX_SPLITS; ++s) {
						if (s < pq.splitk) {
							ssum += ssv[s];
#pragma unroll
							for (int sec = 0; sec < 3; ++sec) v3[sec] += pv[sec][s];
						}
					}
					const float inv = rsqrtf(ssum / (float)P.hidden + P.eps);
#pragma unroll
					for (int sec = 0; sec < 3; ++sec) s_raw[sec * CH_D + tid] = v3[sec] * inv;
				}
				__syncthreads();
				if (tid < CH_D) {
					const int d = tid;
					const float c = __half2float(__ushort_as_half((unsigned short)pre_w.x)), s = __half2float(__ushort_as_half((unsigned short)pre_w.y));
					const float qa = s_raw[d], qb = s_raw[d ^ 64], ka = s_raw[CH_D + d], kb2 = s_raw[CH_D + (d ^ 64)];
					// rotate-half: out[d] = x[d] cos - x[d+64] sin (d < 64), x[d] cos + x[d-64] sin (d >= 64)
					const float qr = (d < 64) ? qa * c - qb * s : qa * c + qb * s;
					const float kr = (d < 64) ? ka * c - kb2 * s : ka * c + kb2 * s;
					const __half kh = __float2half_rn(kr), vh = __float2half_rn(s_raw[2 * CH_D + d]);
					s_q[d] = __half2float(__float2half_rn(qr)) * P.scale;
					s_kn[d] = kh;
					s_vn[d] = vh;
					if (last_split && pos >= 0) {
						const size_t off = (size_t)r * P.kv_stride_b + (size_t)head * P.kv_stride_h + (size_t)pos * CH_D + d;
						L->kc[off] = kh;
						L->vc[off] = vh;
					}
				}
				__syncthreads();
				// 8 lanes per key: lane (g8 = lane / 8: key slot, sub = lane % 8: 16 dims = two 16-byte pieces); the
				// upper four lanes visit the pieces in the opposite order, so a quarter-warp reads 8 distinct bank groups.
				// A group takes keys g8 and g8 + 4 of a chunk.
				const int g8 = lane >> 3, sub = lane & 7, rotp = sub >> 2;
				float qreg[2][8];
#pragma unroll
				for (int i = 0; i < 2; ++i) {
					const int piece = (i + rotp) & 1;
#pragma unroll
					for (int e = 0; e < 8; ++e) qreg[i][e] = s_q[sub * 16 + piece * 8 + e];
				}
				float m = -INFINITY, l = 0.f, acc[2][8];
#pragma unroll
				for (int i = 0; i < 2; ++i)
#pragma unroll
					for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
				auto score = [&](const unsigned char *krow) -> float {
					float sc = 0.f;
#pragma unroll
					for (int i = 0; i < 2; ++i) {
						const int piece = (i + rotp) & 1;
						float kf[8];
						unpack8(*reinterpret_cast<const uint4 *>(krow + sub * 32 + piece * 16), kf);
#pragma unroll
						for (int e = 0; e < 8; ++e) sc = fmaf(qreg[i][e], kf[e], sc);
					}
					return sc;
				};
				auto accumulate = [&](const unsigned char *vrow, float sc) {
					const float mn = fmaxf(m, sc);
					const float corr = __expf(m - mn), pw = __expf(sc - mn);
					l = l * corr + pw;
#pragma unroll
					for (int i = 0; i < 2; ++i) {
						const int piece = (i + rotp) & 1;
						float vf[8];
						unpack8(*reinterpret_cast<const uint4 *>(vrow + sub * 32 + piece * 16), vf);
#pragma unroll
						for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(pw, vf[e], acc[i][e] * corr);
					}
					m = mn;
				};
				auto reduce8 = [&](float v) -> float {          // sum over the 8 lanes of a key
					v += __shfl_xor_sync(0xffffffffu, v, 1);
					v += __shfl_xor_sync(0xffffffffu, v, 2);
					v += __shfl_xor_sync(0xffffffffu, v, 4);
					return v;
				};
				const int nkeys = s_cjob[warp].nkeys, nchunk = (nkeys + 7) >> 3;
#pragma unroll 1
				for (int c = 0; c < nchunk; ++c) {
					const int rows = min(8, nkeys - 8 * c);
					const bool mine0 = g8 < rows, mine1 = g8 + 4 < rows;
					float sc0 = 0.f, sc1 = 0.f;
					if (!slot_wait()) break;
					{
						const unsigned char *slot = smem + (size_t)warp * NST * CH_SLOT + cs * CH_SLOT;
						if (mine0) sc0 = score(slot + g8 * (CH_D * 2));
						if (mine1) sc1 = score(slot + (g8 + 4) * (CH_D * 2));
					}
					sc0 = reduce8(sc0);
					sc1 = reduce8(sc1);
					slot_done();
					if (!slot_wait()) break;
					{
						const unsigned char *slot = smem + (size_t)warp * NST * CH_SLOT + cs * CH_SLOT;
						if (mine0) accumulate(slot + g8 * (CH_D * 2), sc0);
						if (mine1) accumulate(slot + (g8 + 4) * (CH_D * 2), sc1);
					}
					slot_done();
				}
				if (last_split && warp == 0 && pos >= 0) {          // the token's own key / value, from shared memory
					float sc = 0.f;
					if (g8 == 0) sc = score(reinterpret_cast<const unsigned char *>(s_kn));
					sc = reduce8(sc);
					if (g8 == 0) accumulate(reinterpret_cast<const unsigned char *>(s_vn), sc);
				}
				// merge the 4 key slots of the warp (lane bits 3, 4), then the 8 warps through shared memory
				float mw = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
				mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
				const float f = (m == -INFINITY) ? 0.f : __expf(m - mw);
				l *= f;
				l += __shfl_xor_sync(0xffffffffu, l, 8);
				l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
				for (int i = 0; i < 2; ++i)
#pragma unroll
					for (int e = 0; e < 8; ++e) {
						float av = acc[i][e] * f;
						av += __shfl_xor_sync(0xffffffffu, av, 8);
						av += __shfl_xor_sync(0xffffffffu, av, 16);
						acc[i][e] = av;
					}
				if (g8 == 0) {
#pragma unroll
					for (int i = 0; i < 2; ++i) {
						const int piece = (i + rotp) & 1;
#pragma unroll
						for (int e = 0; e < 8; ++e) s_wo[warp * CH_D + sub * 16 + piece * 8 + e] = acc[i][e];
					}
					if (sub == 0) {
						s_wm[warp] = mw;
						s_wl[warp] = l;
					}
				}
				__syncthreads();
				if (tid < CH_D) {
					float Mx = -INFINITY;
#pragma unroll
					for (int w = 0; w < 8; ++w) Mx = fmaxf(Mx, s_wm[w]);
					float o = 0.f, Lx = 0.f;
#pragma unroll
					for (int w = 0; w < 8; ++w) {
						const float g = (s_wm[w] == -INFINITY) ? 0.f : __expf(s_wm[w] - Mx);
						o = fmaf(s_wo[w * CH_D + tid], g, o);
						Lx = fmaf(s_wl[w], g, Lx);
					}
					float *dst = P.p_attn + ((size_t)unit * P.attn_splits + sp) * 130;
					__stcg(dst + 2 + tid, o);
					if (tid == 0) {
						__stcg(dst, Mx);
						__stcg(dst + 1, Lx);
					}
				}
			}
		} else {
			// =========================== quantised projection ===========================
			const ChainPlan &pl = P.plan[kind];
			if (b < pl.tiles * pl.splitk) {
				const int split = b / pl.tiles, tile = b - split * pl.tiles;
				const int n0 = tile * 128;
				const int NS = pl.nstream;
				const int c_lo = split * pl.cps, c_hi = min(c_lo + pl.cps, pl.total_chunks);
				const int g_lo = (c_lo * 128) / P.groupsize;
				const int ng = (c_hi * 128 - 1) / P.groupsize - g_lo + 1;
				const int units = (c_hi - c_lo) * 16;
				const int xs_stride = pl.cps * 256 + 16;
				const int SG = P.strip_groups;

				// ---- zero / scale strips (loaded before the barrier) into shared memory ----
				{
					const int n_strip = NS * ng * 16;
#pragma unroll
					for (int jj = 0; jj < 2; ++jj) {
						const int i = tid + jj * CH_THREADS;
						if (i < n_strip) {
							const int rr = i >> 4, c = i & 15;
							const int s = (rr >= ng) ? 1 : 0, gi = rr - s * ng;
							const uint32_t zv = pre_z[jj];
							uint4 ze;          // zero point (stored + 1) as fp16, two per word: (0x6401 + nibble) - 1024
							ze.x = h2_sub(0x64016401u + ((zv & 0xFu) | ((zv & 0xF0u) << 12)), MAGIC_1024);
							ze.y = h2_sub(0x64016401u + (((zv >> 8) & 0xFu) | (((zv >> 8) & 0xF0u) << 12)), MAGIC_1024);
							ze.z = h2_sub(0x64016401u + (((zv >> 16) & 0xFu) | (((zv >> 16) & 0xF0u) << 12)), MAGIC_1024);
							ze.w = h2_sub(0x64016401u + (((zv >> 24) & 0xFu) | (((zv >> 24) & 0xF0u) << 12)), MAGIC_1024);
							const size_t o = (size_t)(s * SG + gi) * 128 + c * 8;
							*reinterpret_cast<uint4 *>(s_zz + o) = ze;
							*reinterpret_cast<uint4 *>(s_sc + o) = pre_sv[jj];
						}
					}
				}

				// ---- stage x: the deferred epilogue of the previous phase (every sum over splits is ONE batch of loads) ----
				if (kind == CH_QKV || kind == CH_GU) {
					const bool writer = (tile == 0);
					const bool from_embed = (kind == CH_QKV && layer == 0);
					const int S = P.plan[kind == CH_QKV ? CH_DOWN : CH_O].splitk;
					const float *pbase = (kind == CH_QKV ? P.p_down : P.p_o);
					const __half *rbase = (kind == CH_QKV ? P.hB : P.hA);
					__half *hdst = (kind == CH_QKV ? P.hA : P.hB);
					float wf[8];
					unpack8(pre_w, wf);
#pragma unroll 1
					for (int r = 0; r < P.M; ++r) {
						float sq = 0.f;
						if (tid < units) {
							const int k = (c_lo * 16 + tid) * 8;
							uint4 hv;
							if (from_embed) {
								hv = __ldg(reinterpret_cast<const uint4 *>(P.embed + (size_t)P.tok[r] * P.hidden + k));
							} else {
								const float *part = pbase + (size_t)r * P.hidden + k;
								const size_t stride = (size_t)P.M * P.hidden;
								const uint4 rv = __ldcg(reinterpret_cast<const uint4 *>(rbase + (size_t)r * P.hidden + k));
								float4 pa[CH_MAX_SPLITS], pb[CH_MAX_SPLITS];
#pragma unroll
								for (int s = 0; s < CH_MAX_SPLITS; ++s) {
									if (s < S) {
										pa[s] = __ldcg(reinterpret_cast<const float4 *>(part + s * stride));
										pb[s] = __ldcg(reinterpret_cast<const float4 *>(part + s * stride) + 1);
									}
								}
								float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, res[8];
#pragma unroll
								for (int s = 0; s < CH_MAX_SPLITS; ++s) {
									if (s < S) {
										a8[0] += pa[s].x; a8[1] += pa[s].y; a8[2] += pa[s].z; a8[3] += pa[s].w;
										a8[4] += pb[s].x; a8[5] += pb[s].y; a8[6] += pb[s].z; a8[7] += pb[s].w;
									}
								}
								unpack8(rv, res);
#pragma unroll
								for (int i = 0; i < 8; ++i) a8[i] += res[i];
								hv = pack8(a8);
							}
							float hf[8];
							unpack8(hv, hf);
							if (writer) {
								*reinterpret_cast<uint4 *>(hdst + (size_t)r * P.hidden + k) = hv;
#pragma unroll
								for (int i = 0; i < 8; ++i) sq = fmaf(hf[i], hf[i], sq);
							}
#pragma unroll
							for (int i = 0; i < 8; ++i) hf[i] *= wf[i];
							store_x_unit(xs + (size_t)r * xs_stride, tid, pack8(hf));
						}
						if (writer) {                 // sum of squares of this K-slice of the row, fixed order
#pragma unroll
							for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
							if (lane == 0) s_part[warp] = sq;
							__syncthreads();
							if (tid == 0) {
								float t = 0.f;
#pragma unroll
								for (int w = 0; w < CH_THREADS / 32; ++w) t += s_part[w];
								__stcg((kind == CH_QKV ? P.ss_a : P.ss_b) + split * P.M + r, t);
							}
							__syncthreads();
						}
					}
				} else if (kind == CH_O) {
					// merge the key splits of the attention: items of 2 consecutive k (one head dim pair)
					const int per_row = units * 4;
#pragma unroll 1
					for (int i = tid; i < P.M * per_row; i += CH_THREADS) {
						const int r = i / per_row, k_rel = (i - r * per_row) * 2;
						const int k = c_lo * 128 + k_rel;
						const float *pa = P.p_attn + (size_t)(r * P.heads + (k >> 7)) * P.attn_splits * 130;
						float ms[CH_MAX_SPLITS], ls[CH_MAX_SPLITS];
						float2 ov[CH_MAX_SPLITS];
#pragma unroll
						for (int s = 0; s < CH_MAX_SPLITS; ++s) {
							if (s < P.attn_splits) {
								ms[s] = __ldcg(pa + s * 130);
								ls[s] = __ldcg(pa + s * 130 + 1);
								ov[s] = __ldcg(reinterpret_cast<const float2 *>(pa + s * 130 + 2 + (k & 127)));
							}
						}
						float Mx = -INFINITY;
#pragma unroll
						for (int s = 0; s < CH_MAX_SPLITS; ++s)
							if (s < P.attn_splits) Mx = fmaxf(Mx, ms[s]);
						float Lx = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
						for (int s = 0; s < CH_MAX_SPLITS; ++s) {
							if (s < P.attn_splits) {
								const float g = (ms[s] == -INFINITY) ? 0.f : __expf(ms[s] - Mx);
								Lx = fmaf(ls[s], g, Lx);
								o0 = fmaf(ov[s].x, g, o0);
								o1 = fmaf(ov[s].y, g, o1);
							}
						}
						const float il = (Lx > 0.f) ? 1.f / Lx : 0.f;
						store_x_elem(xs + (size_t)r * xs_stride, k_rel, o0 * il);
						store_x_elem(xs + (size_t)r * xs_stride, k_rel + 1, o1 * il);
					}
				} else {
					// down_proj: x = silu(inv * G) * (inv * U); items of 4 consecutive k, splits in batches of 4
					const ChainPlan &pg = P.plan[CH_GU];
					const int per_row = units * 2;
					const size_t stride = (size_t)2 * P.M * P.inter;
#pragma unroll 1
					for (int i = tid; i < P.M * per_row; i += CH_THREADS) {
						const int r = i / per_row, k_rel = (i - r * per_row) * 4;
						const int k = c_lo * 128 + k_rel;
						const float *gp = P.p_gu + (size_t)r * P.inter + k, *up = gp + (size_t)P.M * P.inter;
						float ssv[CH_MAX_SPLITS];
#pragma unroll
						for (int s = 0; s < CH_MAX_SPLITS; ++s)
							if (s < pg.splitk) ssv[s] = __ldcg(P.ss_b + s * P.M + r);
						float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), ua = ga;
#pragma unroll 1
						for (int s0 = 0; s0 < pg.splitk; s0 += 4) {
							float4 gv[4], uv[4];
#pragma unroll
							for (int j = 0; j < 4; ++j) {
								if (s0 + j < pg.splitk) {
									gv[j] = __ldcg(reinterpret_cast<const float4 *>(gp + (s0 + j) * stride));
									uv[j] = __ldcg(reinterpret_cast<const float4 *>(up + (s0 + j) * stride));
								}
							}
#pragma unroll
							for (int j = 0; j < 4; ++j) {
								if (s0 + j < pg.splitk) {
									ga.x += gv[j].x; ga.y += gv[j].y; ga.z += gv[j].z; ga.w += gv[j].w;
									ua.x += uv[j].x; ua.y += uv[j].y; ua.z += uv[j].z; ua.w += uv[j].w;
								}
							}
						}
						float t = 0.f;
#pragma unroll
						for (int s = 0; s < CH_MAX_SPLITS; ++s)
							if (s < pg.splitk) t += ssv[s];
						const float inv = rsqrtf(t / (float)P.hidden + P.eps);
						unsigned char *xr = xs + (size_t)r * xs_stride;
						store_x_elem(xr, k_rel, silu_f32(ga.x * inv) * (ua.x * inv));
						store_x_elem(xr, k_rel + 1, silu_f32(ga.y * inv) * (ua.y * inv));
						store_x_elem(xr, k_rel + 2, silu_f32(ga.z * inv) * (ua.z * inv));
						store_x_elem(xr, k_rel + 3, silu_f32(ga.w * inv) * (ua.w * inv));
					}
				}
				__syncthreads();

				// ---- group sums of the staged x: C = 1024*(SXe + SXo'), S = SXe + 16*SXo' per (group, row) ----
				{
					const int k_lo = c_lo * 128, k_hi = c_hi * 128;
					const int sub = lane & 3;
					const int total = ng * P.M;
#pragma unroll 1
					for (int it0 = 0; it0 < total; it0 += 8 * 8) {
						const int item = it0 + warp * 8 + (lane >> 2);
						const bool valid = item < total;
						const int gi = valid ? item / P.M : 0, row = valid ? item - gi * P.M : 0;
						const int ka = max((g_lo + gi) * P.groupsize, k_lo), kb = min((g_lo + gi + 1) * P.groupsize, k_hi);
						float e = 0.f, o = 0.f;
						if (valid) {
#pragma unroll 2
							for (int u = (ka - k_lo) / 8 + sub; u < (kb - k_lo) / 8; u += 4) {
								const uint4 v = *reinterpret_cast<const uint4 *>(xs + (size_t)row * xs_stride + u * 16);
								const float2 a0 = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
								const float2 a1 = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
								const float2 a2 = __half22float2(*reinterpret_cast<const __half2 *>(&v.z));
								const float2 a3 = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
								e += (a0.x + a0.y) + (a2.x + a2.y);
								o += (a1.x + a1.y) + (a3.x + a3.y);
							}
						}
						e += __shfl_xor_sync(0xffffffffu, e, 1);
						o += __shfl_xor_sync(0xffffffffu, o, 1);
						e += __shfl_xor_sync(0xffffffffu, e, 2);
						o += __shfl_xor_sync(0xffffffffu, o, 2);
						if (valid && sub == 0) s_cs[gi * 16 + row] = make_float2(1024.f * (e + o), e + 16.f * o);
					}
				}
				__syncthreads();

				// ---- main loop: this warp's chunks, stream 0 then stream 1 ----
				// a warp's sums of a stream go to red[kw][stream][row < M][128] as soon as the stream is done
				// (this lane: columns wn*32 + 4*gid + 0..3 of batch rows 2*tig + {0,1})
				auto put_red = [&](int s, const float(&v)[4][2]) {
#pragma unroll
					for (int h = 0; h < 2; ++h) {
						const int row = 2 * tig + h;
						if (row < P.M) {
							float *rp = red + ((size_t)(kw * NS + s) * P.M + row) * 128 + wn * 32 + gid * 4;
							*reinterpret_cast<float4 *>(rp) = make_float4(v[0][h], v[1][h], v[2][h], v[3][h]);
						}
					}
				};
				const int job_nw = s_cjob[warp].nw, job_w_lo = s_cjob[warp].w_lo;
				if (job_nw == 0) {
					const float zero[4][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
					for (int s = 0; s < NS; ++s) put_red(s, zero);
				} else {
					const bool have_row0 = gid < P.M;
					const int w_lo = job_w_lo, w_hi = job_w_lo + job_nw;
					// step l of a chunk: packed rows 2*tig + (l&1) + 8*(l>>1); swizzled 16-byte unit index ^= row & 7
					const int row_a = 2 * tig, row_b = 2 * tig + 1;
					const unsigned char *xrow0 = xs + (size_t)gid * xs_stride + tig * 32;
					const uint32_t ring_even = ring_w + row_a * 128 + ((gid ^ row_a) << 4);
					const uint32_t ring_odd = ring_w + row_b * 128 + ((gid ^ row_b) << 4);
					const int strip_col = wn * 32 + gid * 4;
#pragma unroll 1
					for (int s = 0; s < NS; ++s) {
						const __half *sc_s = s_sc + (size_t)s * SG * 128 + strip_col;
						float accw[4][2], gA[4][2], gB[4][2];
#pragma unroll
						for (int c = 0; c < 4; ++c) accw[c][0] = accw[c][1] = gA[c][0] = gA[c][1] = gB[c][0] = gB[c][1] = 0.f;
						auto flush = [&](float(&g)[4][2], int gi) {
							const uint2 sr = *reinterpret_cast<const uint2 *>(sc_s + (size_t)gi * 128);
							const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.x));
							const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.y));
							const float sf[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
							for (int c = 0; c < 4; ++c) {
								accw[c][0] = fmaf(sf[c], g[c][0], accw[c][0]);
								accw[c][1] = fmaf(sf[c], g[c][1], accw[c][1]);
								g[c][0] = g[c][1] = 0.f;
							}
						};
						auto step = [&](float(&g)[4][2], uint32_t ring_addr, const unsigned char *x0) {
							uint4 q;
							asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(ring_addr));
							uint4 xb0 = make_uint4(0u, 0u, 0u, 0u);
							if (have_row0) xb0 = *reinterpret_cast<const uint4 *>(x0);
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
						};
						auto xoff_of = [&](int chunk, int l) { return (chunk - c_lo) * 256 + ((l & 1) + 8 * (l >> 1)) * 16; };
						auto ring_of = [&](int l) { return ((l & 1) ? ring_odd : ring_even) + cs * CH_SLOT + (l >> 1) * 1024; };
						// the two accumulator sets alternate by group: while one group's MMAs are in flight the finished
						// set of the previous group is scaled and added
						int chunk = w_lo;
						int gi = (w_lo * 4) / P.spg - g_lo;
						int left = P.spg - (w_lo * 4) % P.spg;
						bool pendA = false, pendB = false, stop = false;
						int giA = 0, giB = 0;
						while (chunk < w_hi && !stop) {
							bool done;
							do {
								if (!slot_wait()) { stop = true; break; }
#pragma unroll
								for (int l = 0; l < 4; ++l) step(gA, ring_of(l), xrow0 + xoff_of(chunk, l));
								if (pendB) {
									flush(gB, giB);
									pendB = false;
								}
								left -= 4;
								++chunk;
								done = (left == 0) || (chunk == w_hi);
								slot_done();
							} while (!done);
							if (stop) break;
							pendA = true;
							giA = gi;
							if (left == 0) {
								++gi;
								left = P.spg;
							}
							if (chunk >= w_hi) break;
							do {
								if (!slot_wait()) { stop = true; break; }
#pragma unroll
								for (int l = 0; l < 4; ++l) step(gB, ring_of(l), xrow0 + xoff_of(chunk, l));
								if (pendA) {
									flush(gA, giA);
									pendA = false;
								}
								left -= 4;
								++chunk;
								done = (left == 0) || (chunk == w_hi);
								slot_done();
							} while (!done);
							if (stop) break;
							pendB = true;
							giB = gi;
							if (left == 0) {
								++gi;
								left = P.spg;
							}
						}
						if (pendA) flush(gA, giA);
						if (pendB) flush(gB, giB);
						put_red(s, accw);
					}
				}

				// ---- reduce the two K-warps, remove the offsets and zero points, store this split's partial sums ----
				__syncthreads();
				{
					const int nelem = NS * P.M * 128;
					float *dst = (kind == CH_QKV ? P.p_qkv : kind == CH_O ? P.p_o : kind == CH_GU ? P.p_gu : P.p_down) + (size_t)split * NS * P.M * pl.N;
#pragma unroll 1
					for (int e = tid; e < nelem; e += CH_THREADS) {
						const int s = (e >= P.M * 128) ? 1 : 0, rc = e - s * (P.M * 128);
						const int row = rc >> 7, col = rc & 127;
						float v = red[((size_t)s * P.M + row) * 128 + col] + red[((size_t)(NS + s) * P.M + row) * 128 + col];
						const __half *zz = s_zz + (size_t)s * SG * 128 + col;
						const __half *sc = s_sc + (size_t)s * SG * 128 + col;
						float corr = 0.f;
#pragma unroll 2
						for (int gi = 0; gi < ng; ++gi) {
							const float2 csv = s_cs[gi * 16 + row];
							corr = fmaf(__half2float(sc[(size_t)gi * 128]), fmaf(__half2float(zz[(size_t)gi * 128]), csv.y, csv.x), corr);
						}
						__stcg(dst + ((size_t)s * P.M + row) * pl.N + n0 + col, v - corr);
					}
				}
			}
		}
		if (failed) {                      // a load never arrived: report, let the other CTAs leave their barriers early
			if (lane == 0) {
				atomicExch(P.status, 1);
				atomicExch(P.sync + 2, 1u);
			}
		}
		grid_arrive();
		pre_issue(idx + 1);                // into registers, consumed after the barrier (issued after the arrival: a release waits for earlier loads)
	}

	// ---- final hidden state: h = fp16(residual + sum of the last down_proj partials), sums of squares per 32 columns ----
	if (alive && grid_wait((unsigned)n_phase * (unsigned)G)) {
		const int tiles32 = P.hidden >> 5;
		const ChainPlan &pd = P.plan[CH_DOWN];
#pragma unroll 1
		for (int t32 = b; t32 < tiles32; t32 += G) {
			const int r = tid >> 5;
			if (r < P.M) {
				const int n = t32 * 32 + lane;
				float pv[CH_MAX_SPLITS];
#pragma unroll
				for (int s = 0; s < CH_MAX_SPLITS; ++s)
					if (s < pd.splitk) pv[s] = __ldcg(P.p_down + ((size_t)s * P.M + r) * P.hidden + n);
				float v = 0.f;
#pragma unroll
				for (int s = 0; s < CH_MAX_SPLITS; ++s)
					if (s < pd.splitk) v += pv[s];
				v += __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short *>(P.hB) + (size_t)r * P.hidden + n)));
				const __half hv = __float2half_rn(v);
				P.h_out[(size_t)r * P.hidden + n] = hv;
				float sq = __half2float(hv);
				sq *= sq;
#pragma unroll
				for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
				if (lane == 0) P.ss_f[(size_t)r * tiles32 + t32] = sq;
			}
		}
	}
	// ---- leave: drain this warp's outstanding loads (bounded), reset the counters behind the last CTA ----
#pragma unroll 1
	while (outstanding > 0) {
		mbar_wait_bounded(bar_w + 8 * cs, cpar, 1u << 16);
		--outstanding;
		if (++cs == NST) {
			cs = 0;
			cpar ^= 1u;
		}
	}
	__syncthreads();
	if (tid == 0) {
		__threadfence();
		const unsigned old = atomicAdd(P.sync + 1, 1u);
		if (old == (unsigned)G - 1u && ld_relaxed_u32(P.sync + 2) == 0) {       // healthy run: ready for the next launch
			P.sync[0] = 0u;
			P.sync[1] = 0u;
		}
	}
}

// ---- lm_head: logits = rmsnorm(h) x W^T (fp16 weights [V, K]), greedy token, position + 1 -------------------
// HBM-bound: every weight is read once, 16 bytes per lane and load.  A warp takes 16 vocabulary rows at a time and
// multiplies them with all (up to 8) batch rows on the tensor cores: the weight rows are the A operand of
// mma.sync.m16n8k16 straight from global memory, the normalised hidden states (shared memory) the B operand.  The
// dot product does not care about the order of k, so the lane (gid, tig) simply takes the 8 consecutive k of rows
// gid and gid + 8 that its 16-byte loads deliver (k = 32 * step + 8 * tig + 0..7) and the same 8 k of batch row gid:
// two MMAs per pair of loads, no shuffles, no conversion.  The arg-max is reduced per warp and CTA; the last CTA to
// arrive (ticket) reduces the per-CTA candidates in CTA order, writes the tokens and advances the positions.
constexpr int LM_THREADS = 256;
constexpr int LM_XPAD = 64;               // bytes added to a row of x in shared memory: conflict-free 16-byte reads

struct LmHeadParams {
	const __half *h;              // [M, K] final hidden state (before the norm)
	const float *ss;              // [M, K / 32] sums of squares of h per 32 columns
	const __half *norm_w;         // [K]
	const __half *W;              // [V, K]
	__half *logits;               // [M, V]
	long long *tok;               // [M] out: arg-max
	int32_t *pos;                 // [M] in/out: += 1
	float *cand_val;              // [grid, M]
	int *cand_idx;                // [grid, M]
	unsigned *ticket;
	int M, K, V;
	float eps;
};

__global__ void __launch_bounds__(LM_THREADS, 2) lm_head_kernel(const LmHeadParams p) {
	extern __shared__ __align__(16) unsigned char lm_smem[];
	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
	constexpr int NW = LM_THREADS / 32;
	__shared__ float s_inv[CH_MAX_M];
	__shared__ float s_bv[NW][CH_MAX_M];
	__shared__ int s_bi[NW][CH_MAX_M];
	__shared__ int s_last;
	const int xs_stride = p.K * 2 + LM_XPAD;                 // bytes; x: [8 rows][K] fp16, rows >= M are zero
	const int tiles32 = p.K >> 5;
	for (int r = warp; r < p.M; r += NW) {
		float t = 0.f;
		for (int i = lane; i < tiles32; i += 32) t += __ldcg(p.ss + (size_t)r * tiles32 + i);
#pragma unroll
		for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
		if (lane == 0) s_inv[r] = rsqrtf(t / (float)p.K + p.eps);
	}
	__syncthreads();
	const int units = p.K >> 3;
	for (int i = tid; i < CH_MAX_M * units; i += LM_THREADS) {
		const int r = i / units, u = i - r * units;
		uint4 xv = make_uint4(0u, 0u, 0u, 0u);
		if (r < p.M) {
			const uint4 hv = __ldcg(reinterpret_cast<const uint4 *>(p.h + (size_t)r * p.K) + u);
			const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(p.norm_w) + u);
			float hf[8], wf[8];
			unpack8(hv, hf);
			unpack8(wv, wf);
			const float inv = s_inv[r];
#pragma unroll
			for (int e = 0; e < 8; ++e) hf[e] = hf[e] * inv * wf[e];          // x * inv * w, one rounding
			xv = pack8(hf);
		}
		*reinterpret_cast<uint4 *>(lm_smem + (size_t)r * xs_stride + u * 16) = xv;
	}
	__syncthreads();
	// this lane's running best of batch columns 2*tig and 2*tig + 1 (the same on all lanes of equal tig)
	float best0 = -INFINITY, best1 = -INFINITY;
	int besti0 = 0x7fffffff, besti1 = 0x7fffffff;
	auto better = [](float f, int i, float bf, int bi) { return f > bf || (f == bf && i < bi); };
	const int gw = blockIdx.x * NW + warp, nwarps = gridDim.x * NW;
	const int ntiles = (p.V + 15) >> 4;
	const unsigned char *xrow = lm_smem + (size_t)gid * xs_stride + tig * 16;
	constexpr int U = 8;                                     // steps of 32 k per batch of loads: 16 loads of 16 bytes in flight per lane
#pragma unroll 1
	for (int tile = gw; tile < ntiles; tile += nwarps) {
		const int ra = tile * 16 + gid, rb = ra + 8;
		const uint4 *pa = reinterpret_cast<const uint4 *>(p.W + (size_t)min(ra, p.V - 1) * p.K) + tig;
		const uint4 *pb = reinterpret_cast<const uint4 *>(p.W + (size_t)min(rb, p.V - 1) * p.K) + tig;
		float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
		for (int k0 = 0; k0 < p.K; k0 += 32 * U) {             // K % 256 == 0
			uint4 wa[U], wb[U];
#pragma unroll
			for (int u = 0; u < U; ++u) {
				wa[u] = ld_nc_v4(pa + (k0 >> 3) + 4 * u);
				wb[u] = ld_nc_v4(pb + (k0 >> 3) + 4 * u);
			}
#pragma unroll
			for (int u = 0; u < U; ++u) {
				const uint4 xv = *reinterpret_cast<const uint4 *>(xrow + (k0 + 32 * u) * 2);
				mma16816(d, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
				mma16816(d, wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
			}
		}
		// d[0], d[1]: row ra, batch columns 2*tig, 2*tig + 1; d[2], d[3]: row rb
		const int c0 = 2 * tig, c1 = c0 + 1;
		const __half h0 = __float2half_rn(d[0]), h1 = __float2half_rn(d[1]), h2 = __float2half_rn(d[2]), h3 = __float2half_rn(d[3]);
		if (ra < p.V) {
			if (c0 < p.M) p.logits[(size_t)c0 * p.V + ra] = h0;
			if (c1 < p.M) p.logits[(size_t)c1 * p.V + ra] = h1;
		}
		if (rb < p.V) {
			if (c0 < p.M) p.logits[(size_t)c0 * p.V + rb] = h2;
			if (c1 < p.M) p.logits[(size_t)c1 * p.V + rb] = h3;
		}
		// the arg-max is taken over the fp16 logits, lowest index wins ties
		float f0 = (ra < p.V) ? __half2float(h0) : -INFINITY, f1 = (ra < p.V) ? __half2float(h1) : -INFINITY;
		int i0 = ra, i1 = ra;
		if (rb < p.V) {
			if (better(__half2float(h2), rb, f0, i0)) { f0 = __half2float(h2); i0 = rb; }
			if (better(__half2float(h3), rb, f1, i1)) { f1 = __half2float(h3); i1 = rb; }
		}
#pragma unroll
		for (int s = 4; s < 32; s <<= 1) {               // over the 8 row pairs of the tile (lanes of equal tig)
			const float of0 = __shfl_xor_sync(0xffffffffu, f0, s), of1 = __shfl_xor_sync(0xffffffffu, f1, s);
			const int oi0 = __shfl_xor_sync(0xffffffffu, i0, s), oi1 = __shfl_xor_sync(0xffffffffu, i1, s);
			if (better(of0, oi0, f0, i0)) { f0 = of0; i0 = oi0; }
			if (better(of1, oi1, f1, i1)) { f1 = of1; i1 = oi1; }
		}
		if (better(f0, i0, best0, besti0)) { best0 = f0; besti0 = i0; }
		if (better(f1, i1, best1, besti1)) { best1 = f1; besti1 = i1; }
	}
	if (gid == 0) {
		s_bv[warp][2 * tig] = best0;
		s_bi[warp][2 * tig] = besti0;
		s_bv[warp][2 * tig + 1] = best1;
		s_bi[warp][2 * tig + 1] = besti1;
	}
	__syncthreads();
	if (tid < p.M) {
		float bv = -INFINITY;
		int bi = 0x7fffffff;
		for (int w = 0; w < NW; ++w) {
			const float f = s_bv[w][tid];
			const int i = s_bi[w][tid];
			if (f > bv || (f == bv && i < bi)) {
				bv = f;
				bi = i;
			}
		}
		__stcg(p.cand_val + (size_t)blockIdx.x * p.M + tid, bv);
		__stcg(p.cand_idx + (size_t)blockIdx.x * p.M + tid, bi);
	}
	__syncthreads();
	if (tid == 0) {
		unsigned t;
		asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(p.ticket) : "memory");
		const int last = (t == gridDim.x - 1);
		if (last) *p.ticket = 0u;
		s_last = last;
	}
	__syncthreads();
	if (!s_last) return;
	for (int r = warp; r < p.M; r += NW) {
		float bv = -INFINITY;
		int bi = 0x7fffffff;
		for (int c = lane; c < (int)gridDim.x; c += 32) {
			const float f = __ldcg(p.cand_val + (size_t)c * p.M + r);
			const int i = __ldcg(p.cand_idx + (size_t)c * p.M + r);
			if (f > bv || (f == bv && i < bi)) {
				bv = f;
				bi = i;
			}
		}
#pragma unroll
		for (int d = 16; d > 0; d >>= 1) {
			const float of = __shfl_xor_sync(0xffffffffu, bv, d);
			const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
			if (of > bv || (of == bv && oi < bi)) {
				bv = of;
				bi = oi;
			}
		}
		if (lane == 0) {
			p.tok[r] = (long long)bi;
			p.pos[r] = p.pos[r] + 1;
		}
	}
}

}   // namespace gptq
