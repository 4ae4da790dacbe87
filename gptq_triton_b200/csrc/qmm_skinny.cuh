// Decode-regime (M <= 16) quantised matmul for sm_100a: an HBM-bound skinny GEMM.
//
// Work split.  A CTA owns 128 output columns (4 warps x 32 columns) and one K-slice
// (grid.y = split-K); its KW warp-rows take contiguous parts of the slice.  The unit of
// streaming is a chunk: 128 K-rows = 16 packed rows x 32 columns = 2 KB per warp.
//
// Weight stream.  Every warp runs a private TMA pipeline: lane 0 issues one 2-D tiled bulk
// copy (box 32 columns x 16 packed rows) per chunk into an NSTAGE-deep ring in shared
// memory and all lanes wait on the stage's mbarrier.  No other warp touches the ring, so
// stage reuse needs only a __syncwarp.  Lane (gid = lane/4, tig = lane%4) reads the 16
// bytes that hold its 4 columns (4*gid..4*gid+3) of packed row 4*step + tig.
//
// Math.  The 8 nibbles of a word are 8 K-values of one column.  Masking with 0x000F000F /
// 0x00F000F0 (and the same after >>8) and OR-ing 0x6400 into each half gives the half2
// pairs (k0,k4) (k2,k6) as 1024+q and (k1,k5) (k3,k7) as 1024+16q: five integer
// instructions per 8 weights and nothing else.  These raw values are the A operand of
// mma.sync.m16n8k16 (16 weight columns x 16 k); the batch rows of x are the B operand,
// staged in shared memory in the matching k order [0,4,1,5,2,6,3,7] with the (k1,k5,k3,k7)
// entries multiplied by 1/16.  Per group the MMA therefore accumulates, in fp32,
//     D = sum x*q + 1024*(SXe + SXo'),   SXe = sum of the unscaled x, SXo' = sum of the x/16,
// the scale is applied in fp32 when the group ends, and the zero point and the 1024-offsets
// are removed once per CTA from the group sums of x:
//     sum x*(q - z) = D - 1024*(SXe + SXo') - z*(SXe + 16*SXo').
// No weight is ever rounded to fp16: the result equals an fp32-accumulated (q-z-1)*s
// reference up to fp32 summation order (x/16 is exact unless |x| < 2^-10, where the
// deviation is below 2^-21 absolute).
//
// Reduction.  Warp-rows reduce through shared memory; split-K CTAs write fp32 partials to
// the workspace and take a ticket; the last CTA of a tile sums the partials in fixed order
// (deterministic) and runs the epilogue: bias/residual, SiLU(gate)*up, or rotary embedding
// with a scatter into Q / K / V (or the KV cache).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace gptq {

enum { EPI_PLAIN = 0, EPI_SILU = 1, EPI_ROPE = 2 };

constexpr int SK_BN = 128;                 // columns per CTA
constexpr int SK_CHUNK_BYTES = 2048;       // one warp-chunk: 16 packed rows x 128 bytes
constexpr int SK_BAR_BYTES = 1024;         // room for the per-warp, per-stage mbarriers
constexpr int SK_TICKET_BYTES = 16384;     // arrival counters; the last int is a status word
constexpr int SK_STATUS_SLOT = SK_TICKET_BYTES / 4 - 1;

struct SkinnyParams {
	const __half *x;
	long long ldx;
	const int32_t *qz0, *qz1;
	const __half *sc0, *sc1;
	const int32_t *perm;   // host side only: request for the gather pass; the kernel reads x in order
	int M, K, N, groupsize;
	int spg;               // 32-row steps per group (1, 2 or a multiple of 4)
	int total_chunks;      // K / 128
	int chunks_per_split;
	int splitk;
	int nstage;
	int xs_stride;         // bytes between rows of the staged x slice
	int xs_bytes;          // M * xs_stride rounded up to 128
	int pdl;               // 1: launched with programmatic stream serialisation (x is loaded after pdl_wait)
	int strip_groups;      // capacity (groups) of the zero / scale strips per stream
	float *ws_partial;
	int *ws_ticket;
	// Split-K exchange without a ticket (M <= 8, all CTAs of the launch co-resident): every split but the
	// last writes its partial sums as 8-byte words {value, tag} (the store carries its own flag: no fence, no
	// counter; the tag is a NaN bit pattern, which no partial sum left in the workspace by another kernel
	// can show in that half of a word); the CTA of the LAST split polls for them, adds them in split order
	// and zeroes the words again, so the area is clean for the next launch.
	unsigned long long *ws_words;      // nullptr: ticket protocol
	// EPI_PLAIN / EPI_SILU
	const __half *bias;
	const __half *residual;
	long long ldr;
	__half *y;
	long long ldy;
	// RMSNorm folded in.  Producer (EPI_PLAIN): ss_out[row][c] = sum over columns 32c .. 32c+31 of
	// the squared fp16 outputs.  Consumer (EPI_SILU / EPI_ROPE, x read in order): x is scaled by
	// rsqrt(sum_t ss_in[row][t] / K + eps) * rms_w while it is staged (one fp16 rounding, as the
	// stand-alone RMSNorm kernel does).
	float *ss_out;
	const __half *rms_w;
	const float *ss_in;
	int ss_tiles;
	float rms_eps;
	// Tensor parallelism, row-parallel projection (EPI_PLAIN): the all-reduce of the partial sums is part
	// of the epilogue.  Every rank PUSHES its tile (fp32, bias included) into the receive buffers of its
	// peers as 8-byte words {value, sequence number} (one store carries the data and its own flag, so no
	// fence and no separate signal is needed), then polls its OWN receive buffer until the words of every
	// peer carry this launch's sequence number, and adds the tiles in rank order: the same bits on every rank.
	int ar_world, ar_rank;
	unsigned long long *ar_buf[8];     // receive buffer of every rank: [parity of the sequence number][source rank < 8][tile][16 rows][128] words
	unsigned *ar_seq;                  // this rank's sequence number per tile (same on every rank: same launches)
	// EPI_ROPE
	const __half *cos_t, *sin_t;
	const int32_t *pos;
	__half *q_out, *k_out, *v_out;
	long long q_stride_m, kv_sb, kv_st, kv_sh, kv_sp;
	int tokens_per_batch, hidden, max_pos;
};

// SPG_T: steps per group known at compile time (1 or 2), or 0 when a group spans whole chunks.
// x is always read in order: for act-order weights the host gathers x[:, perm] once per call with
// gather_x_kernel (every CTA of every tile would otherwise repeat the gather with 2-byte loads).
// KW = 2 or 4: CTA of 4 column-warps x KW K-warps on a 128-column tile, split-K over grid.y.
// KW = 8: "narrow" CTA of 8 K-warps on ONE 32-column strip and the whole of K (grid.y = 1): the
// K-warps are reduced in shared memory only, so the partial sums, the arrival ticket and the
// second pass of a split-K tail disappear; for small outputs (N / 32 CTAs fill the chip).
template <int KW, int NSTREAM, bool M8, int SPG_T, int EPI>
__global__ void __launch_bounds__(KW == 8 ? 256 : KW * 128, KW == 8 ? 2 : 4 / KW)
	skinny_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, const SkinnyParams p) {
	extern __shared__ __align__(1024) unsigned char smem[];
	constexpr bool NARROW = (KW == 8);
	static_assert(!NARROW || (EPI == EPI_PLAIN && NSTREAM == 1), "narrow CTAs: plain epilogue, one weight stream");
	constexpr int NWN = NARROW ? 1 : 4;          // column-warps per CTA
	constexpr int BN = NWN * 32;                 // columns per CTA
	constexpr int BSH = NARROW ? 5 : 7;          // log2(BN)
	constexpr int SU = BN / 8, SUSH = NARROW ? 2 : 4;      // 8-column strip units per group row
	constexpr int NT = NARROW ? 256 : KW * 128;
	constexpr int NWARP = NT / 32;
	constexpr int ROWS = M8 ? 8 : 16;
	constexpr int MB = M8 ? 1 : 2;             // batch-row blocks of 8

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int wn = NARROW ? 0 : (warp & 3), kw = NARROW ? warp : (warp >> 2), gid = lane >> 2, tig = lane & 3;
	const int tile = blockIdx.x, split = blockIdx.y;
	const int n0 = tile * BN, n0w = n0 + wn * 32;
	const bool warp_active = n0w < p.N;

	// shared memory: [ ring | mbarriers | x slice | zero strips | scale strips ]; the ring
	// region is reused as the reduce buffer once the stream has drained
	unsigned char *ring_all = smem;
	const int ring_bytes = NWARP * p.nstage * SK_CHUNK_BYTES;
	uint64_t *bars = reinterpret_cast<uint64_t *>(smem + ring_bytes);
	unsigned char *xs = smem + ring_bytes + SK_BAR_BYTES;
	__half *s_zz = reinterpret_cast<__half *>(xs + p.xs_bytes);                  // [stream][group][128] zero point (stored + 1)
	__half *s_sc = s_zz + NSTREAM * p.strip_groups * BN;                      // [stream][group][128] scale
	float2 *s_cs = reinterpret_cast<float2 *>(s_sc + NSTREAM * p.strip_groups * BN);   // [group][16 rows] (C, S) of x
	float *red = reinterpret_cast<float *>(smem);
	__shared__ int s_last;

	const int c_lo = split * p.chunks_per_split;
	const int c_hi = min(c_lo + p.chunks_per_split, p.total_chunks);
	const int per_w = (c_hi - c_lo + KW - 1) / KW;
	const int w_lo = min(c_lo + kw * per_w, c_hi);
	const int w_hi = min(w_lo + per_w, c_hi);
	const int nw = warp_active ? (w_hi - w_lo) : 0;      // chunks per stream for this warp
	const int nload = nw * NSTREAM;

	// ---- per-warp TMA pipeline -------------------------------------------------------
	const uint32_t ring_w = smem_u32(ring_all + (size_t)warp * p.nstage * SK_CHUNK_BYTES);
	const uint32_t bar_w = smem_u32(bars + warp * p.nstage);
	if (lane == 0) {
		for (int s = 0; s < p.nstage; ++s) mbar_init(bar_w + 8 * s, 1);
		fence_mbar_init();
		if (warp == 0) {
			tma_prefetch_desc(&tm0);
			if (NSTREAM == 2) tma_prefetch_desc(&tm1);
		}
	}
	__syncwarp();
	int pr_j = 0, pr_chunk = w_lo, pr_stream = 0, pr_stage = 0;
	auto produce = [&]() {
		if (pr_j < nload) {
			if (lane == 0) {
				const uint32_t bar = bar_w + 8 * pr_stage;
				mbar_arrive_expect_tx(bar, SK_CHUNK_BYTES);
				tma_load_2d(ring_w + pr_stage * SK_CHUNK_BYTES, (NSTREAM == 2 && pr_stream) ? &tm1 : &tm0, n0w, pr_chunk * 16, bar);
			}
			++pr_j;
			if (++pr_stage == p.nstage) pr_stage = 0;
			if (++pr_chunk == w_hi) {
				pr_chunk = w_lo;
				++pr_stream;
			}
		}
	};

	// ---- stage zero / scale strips and the x slice ---------------------------------------
	// The first batch of these small loads is issued BEFORE the TMA prologue so that it does
	// not queue behind 100+ KB of weight prefetch per SM; the values are stored afterwards.
	const int g_lo = (c_lo * 128) / p.groupsize;
	const int ng = (c_hi * 128 - 1) / p.groupsize - g_lo + 1;
	const int n_strip = NSTREAM * ng * SU;              // items of 8 columns
	const int units = (c_hi - c_lo) * 16;               // 16-byte units per x row
	constexpr int SB = 2, XB = M8 ? 4 : 8;      // 16 rows: eight 16-byte loads of x in flight per thread (two passes instead of four)
	// strips: item -> (stream, group, 8-column unit) without a division (NSTREAM <= 2)
	auto strip_load = [&](int base, uint32_t(&z)[SB], uint4(&sv)[SB]) {
		const int nz = p.N >> 3;
#pragma unroll
		for (int j = 0; j < SB; ++j) {
			const int idx = base + j * NT;
			if (idx < n_strip) {
				const int r = idx >> SUSH, c = idx & (SU - 1);
				const int s = (NSTREAM == 2 && r >= ng) ? 1 : 0, gi = r - s * ng;
				if (n0 + c * 8 < p.N) {
					const int32_t *qz = s ? p.qz1 : p.qz0;
					const __half *sc = s ? p.sc1 : p.sc0;
					z[j] = (uint32_t)__ldg(qz + (size_t)(g_lo + gi) * nz + (n0 >> 3) + c);
					sv[j] = __ldg(reinterpret_cast<const uint4 *>(sc + (size_t)(g_lo + gi) * p.N + n0 + c * 8));
				}
			}
		}
	};
	auto strip_store = [&](int base, const uint32_t(&z)[SB], const uint4(&sv)[SB]) {
#pragma unroll
		for (int j = 0; j < SB; ++j) {
			const int idx = base + j * NT;
			if (idx < n_strip) {
				const int r = idx >> SUSH, c = idx & (SU - 1);
				const int s = (NSTREAM == 2 && r >= ng) ? 1 : 0, gi = r - s * ng;
				if (n0 + c * 8 < p.N) {
					// zero point (stored + 1) as fp16, two per word: (0x6401 + nibble) - 1024
					const uint32_t zv = z[j];
					uint4 ze;
					ze.x = h2_sub(0x64016401u + ((zv & 0xFu) | ((zv & 0xF0u) << 12)), MAGIC_1024);
					ze.y = h2_sub(0x64016401u + (((zv >> 8) & 0xFu) | (((zv >> 8) & 0xF0u) << 12)), MAGIC_1024);
					ze.z = h2_sub(0x64016401u + (((zv >> 16) & 0xFu) | (((zv >> 16) & 0xF0u) << 12)), MAGIC_1024);
					ze.w = h2_sub(0x64016401u + (((zv >> 24) & 0xFu) | (((zv >> 24) & 0xF0u) << 12)), MAGIC_1024);
					const size_t o = (size_t)(s * p.strip_groups + gi) * BN + c * 8;
					*reinterpret_cast<uint4 *>(s_zz + o) = ze;
					*reinterpret_cast<uint4 *>(s_sc + o) = sv[j];
				}
			}
		}
	};
	// x slice: a pass covers XB batch rows of one 16-byte unit per thread
	constexpr bool RMS_OK = (EPI != EPI_PLAIN);
	const bool rms = RMS_OK && p.rms_w != nullptr;
	__shared__ float s_inv[16];
	// x slice: the (row, block of NT units) items of the CTA's slice in row-major order; a pass covers
	// XB consecutive items, so XB loads are in flight per thread whatever the shape (many rows of a
	// short slice, or one row of a long one)
	const int u_blocks = (units + NT - 1) / NT;
	auto x_load = [&](int r, int ub, uint4(&v)[XB], uint4(&wq)[XB]) {
#pragma unroll
		for (int j = 0; j < XB; ++j) {
			const int unit = ub * NT + tid;
			if (r < p.M && unit < units) {
				const int k = (c_lo * 16 + unit) * 8;
				if (rms) wq[j] = __ldg(reinterpret_cast<const uint4 *>(p.rms_w + k));
				v[j] = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)r * p.ldx + k));
			}
			if (++ub == u_blocks) {
				ub = 0;
				++r;
			}
		}
	};
	// one 16-byte unit of x: [row < M][unit of 8 k] in k order 0,4,1,5,2,6,3,7, the (1,5) and (3,7) pairs divided by 16
	auto store_item = [&](int r, int unit, uint4 t, const uint4 &w) {
		if (rms) {
			// x * inv_rms * w: fp32 product, one fp16 rounding (same expression as rmsnorm_kernel)
			const float inv = s_inv[r];
			const uint32_t tv[4] = {t.x, t.y, t.z, t.w}, wv[4] = {w.x, w.y, w.z, w.w};
			uint32_t ov[4];
#pragma unroll
			for (int i = 0; i < 4; ++i) {
				const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&tv[i]));
				const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(&wv[i]));
				const __half2 h = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);
				ov[i] = *reinterpret_cast<const uint32_t *>(&h);
			}
			t = make_uint4(ov[0], ov[1], ov[2], ov[3]);
		}
		uint4 o;
		o.x = __byte_perm(t.x, t.z, 0x5410);                          // (x0, x4)
		o.y = h2_mul(__byte_perm(t.x, t.z, 0x7632), 0x2C002C00u);    // (x1, x5) / 16
		o.z = __byte_perm(t.y, t.w, 0x5410);                          // (x2, x6)
		o.w = h2_mul(__byte_perm(t.y, t.w, 0x7632), 0x2C002C00u);    // (x3, x7) / 16
		*reinterpret_cast<uint4 *>(xs + (size_t)r * p.xs_stride + unit * 16) = o;
	};
	auto x_store = [&](int &r, int &ub, const uint4(&v)[XB], const uint4(&wq)[XB]) {
#pragma unroll
		for (int j = 0; j < XB; ++j) {
			const int unit = ub * NT + tid;
			if (r < p.M && unit < units) store_item(r, unit, v[j], wq[j]);
			if (++ub == u_blocks) {
				ub = 0;
				++r;
			}
		}
	};
	{
		// One copy of the staging code (real loops; the first pass issues its loads before the
		// weight prefetch).  Straight-line code that runs once costs instruction fetch, and this
		// prologue used to be more than half of the kernel's code.
		pdl_trigger();
		const int x_passes = (p.M * u_blocks + XB - 1) / XB;
		const int n_it = max(max(1, x_passes), (n_strip + NT * SB - 1) / (NT * SB));
		int xr = 0, xub = 0;                                 // first (row, unit block) item of the current x pass
		if (p.M == 1 && u_blocks == 1 && p.pdl) {
			// One row, one unit per thread, dependent launch: the shortest chain between the dependency wait and the
			// first MMA.  Everything that does not depend on the previous kernel (strips, the norm weight) is finished
			// before the wait; behind it: one load, the norm factor, one store.
			const bool have = tid < units;
			const int k = (c_lo * 16 + tid) * 8;
			uint4 w1 = make_uint4(0u, 0u, 0u, 0u);
			{
				uint32_t z0[SB];
				uint4 sv0[SB];
				strip_load(tid, z0, sv0);
				if (rms && have) w1 = __ldg(reinterpret_cast<const uint4 *>(p.rms_w + k));
#pragma unroll 1
				for (int s = 0; s < p.nstage; ++s) produce();    // weight prefetch: nstage chunks per warp
				strip_store(tid, z0, sv0);
#pragma unroll 1
				for (int it = 1; it * NT * SB < n_strip; ++it) {
					strip_load(tid + it * NT * SB, z0, sv0);
					strip_store(tid + it * NT * SB, z0, sv0);
				}
			}
			pdl_wait();
			uint4 v1 = make_uint4(0u, 0u, 0u, 0u);
			if (have) v1 = __ldg(reinterpret_cast<const uint4 *>(p.x + k));
			if (rms) {
				if (warp == 0) {
					float t = 0.f;
#pragma unroll 4
					for (int i = lane; i < p.ss_tiles; i += 32) t += __ldcg(p.ss_in + i);
#pragma unroll
					for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
					if (lane == 0) s_inv[0] = rsqrtf(t / (float)p.K + p.rms_eps);
				}
				__syncthreads();
			}
			if (have) store_item(0, tid, v1, w1);
		} else
#pragma unroll 1
		for (int it = 0; it < n_it; ++it) {
			uint32_t z0[SB];
			uint4 sv0[SB], v0[XB], wq[XB];
			strip_load(tid + it * NT * SB, z0, sv0);
			// x comes from the previous kernel: under programmatic dependent launch it may only be
			// read after pdl_wait(), i.e. after the weight prefetch; otherwise it is issued first,
			// ahead of the prefetch burst in the memory queues
			const bool early = !p.pdl || it > 0;
			if (early && it < x_passes) x_load(xr, xub, v0, wq);
			if (it == 0) {
#pragma unroll 1
				for (int s = 0; s < p.nstage; ++s) produce();    // weight prefetch: nstage chunks per warp
				pdl_wait();
				if (!early && x_passes > 0) x_load(xr, xub, v0, wq);
				if (rms) {
					// 1/rms of every row from the per-tile sums the producing kernel left (fixed order)
#pragma unroll 1
					for (int r = warp; r < p.M; r += NWARP) {
						const float *sp = p.ss_in + (size_t)r * p.ss_tiles;
						float t = 0.f;
#pragma unroll 4
						for (int i = lane; i < p.ss_tiles; i += 32) t += __ldcg(sp + i);
#pragma unroll
						for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
						if (lane == 0) s_inv[r] = rsqrtf(t / (float)p.K + p.rms_eps);
					}
					__syncthreads();
				}
			}
			strip_store(tid + it * NT * SB, z0, sv0);
			if (it < x_passes) x_store(xr, xub, v0, wq);      // advances (xr, xub) by XB items
		}
	}
	// Bias and residual of the first epilogue pass (element tid of the M x 128 tile) are fetched now:
	// only the last CTA of a tile uses them, but it then finds them in registers instead of paying
	// a global round trip at the very end of the kernel.
	float pre_bias = 0.f, pre_res = 0.f;
	if (EPI == EPI_PLAIN && tid < p.M * BN) {
		const int n = n0 + (tid & (BN - 1));
		if (n < p.N) {
			if (p.bias) pre_bias = __half2float(__ldg(p.bias + n));
			if (p.residual) pre_res = __half2float(p.residual[(size_t)(tid >> BSH) * p.ldr + n]);
		}
	}
	__syncthreads();

	// ---- group sums of the staged x: C = 1024*(SXe + SXo'), S = SXe + 16*SXo' per (group, row) ----
	// four lanes per (group, row); fixed summation order
	{
		const int k_lo = c_lo * 128, k_hi = c_hi * 128;
		const int sub = lane & 3;
		const int total = ng * p.M;
#pragma unroll 1
		for (int it0 = 0; it0 < total; it0 += NWARP * 8) {       // uniform trip count: shuffles below
			const int item = it0 + warp * 8 + (lane >> 2);
			const bool valid = item < total;
			const int gi = !valid ? 0 : (p.M == 1 ? item : item / p.M), row = !valid ? 0 : (p.M == 1 ? 0 : item - gi * p.M);      // no division on the one-row path
			const int ka = max((g_lo + gi) * p.groupsize, k_lo), kb = min((g_lo + gi + 1) * p.groupsize, k_hi);
			float e = 0.f, o = 0.f;
			if (valid) {
#pragma unroll 2
				for (int u = (ka - k_lo) / 8 + sub; u < (kb - k_lo) / 8; u += 4) {
					const uint4 v = *reinterpret_cast<const uint4 *>(xs + (size_t)row * p.xs_stride + u * 16);
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
	// no barrier here: the sums are read only after the main loop, behind the barrier that ends it

	// ---- main loop ---------------------------------------------------------------------
	// acc[stream][batch block][column 0..3 of this lane][batch row 2*tig + {0,1}]
	float acc[NSTREAM][MB][4][2];
#pragma unroll
	for (int s = 0; s < NSTREAM; ++s)
#pragma unroll
		for (int b = 0; b < MB; ++b)
#pragma unroll
			for (int c = 0; c < 4; ++c) acc[s][b][c][0] = acc[s][b][c][1] = 0.f;

	bool failed = false;
	if (nw > 0) {
		const bool have_row0 = gid < p.M, have_row1 = gid + 8 < p.M;
		// In step l of a chunk this lane works on packed row 2*tig + (l&1) + 8*(l>>1); the ring
		// is written by TMA with the 128-byte swizzle (16-byte unit index ^= row & 7), which
		// makes the quarter-warp reads below conflict-free.  (With 32-row groups a step must
		// stay inside one group, so there the rows are 4*l + tig; that variant has 2-way
		// conflicts.)
		constexpr bool LIN = (SPG_T == 1);
		const int row_a = LIN ? tig : 2 * tig, row_b = LIN ? 4 + tig : 2 * tig + 1;    // steps 0/2 and 1/3
		const unsigned char *xrow0 = xs + (size_t)gid * p.xs_stride + tig * (LIN ? 16 : 32);
		const unsigned char *xrow1 = xs + (size_t)(gid + 8) * p.xs_stride + tig * (LIN ? 16 : 32);
		const uint32_t ring_even = ring_w + row_a * 128 + ((gid ^ row_a) << 4);
		const uint32_t ring_odd = ring_w + row_b * 128 + ((gid ^ row_b) << 4);
		const int strip_col = wn * 32 + gid * 4;
		int stage = 0;
		uint32_t parity = 0;
		bool first = true;
		// The streams share ONE copy of the loop code (a real loop over s, accumulating into accw):
		// instruction fetch is the largest stall of a kernel this short, so code size is kept down.
#pragma unroll 1
		for (int s = 0; s < NSTREAM; ++s) {
			const __half *sc_s = s_sc + (size_t)s * p.strip_groups * BN + strip_col;
			float accw[MB][4][2];
#pragma unroll
			for (int b = 0; b < MB; ++b)
#pragma unroll
				for (int c = 0; c < 4; ++c) accw[b][c][0] = accw[b][c][1] = 0.f;
			// Two accumulator sets: while the MMAs of one group are still in the tensor pipe, the
			// finished set of the previous group is scaled and added, so nothing waits for a drain.
			float gA[MB][4][2], gB[MB][4][2];
			auto clear = [&](float(&g)[MB][4][2]) {
#pragma unroll
				for (int b = 0; b < MB; ++b)
#pragma unroll
					for (int c = 0; c < 4; ++c) g[b][c][0] = g[b][c][1] = 0.f;
			};
			auto flush = [&](float(&g)[MB][4][2], int gi) {
				const uint2 sr = *reinterpret_cast<const uint2 *>(sc_s + (size_t)gi * BN);
				const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.x));
				const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.y));
				const float sf[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
				for (int b = 0; b < MB; ++b)
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						accw[b][c][0] = fmaf(sf[c], g[b][c][0], accw[b][c][0]);
						accw[b][c][1] = fmaf(sf[c], g[b][c][1], accw[b][c][1]);
					}
				clear(g);
			};
			// one step: 2 shared loads, 20 integer ops, 4 (or 8) MMAs
			auto step = [&](float(&g)[MB][4][2], uint32_t ring_addr, const unsigned char *x0, const unsigned char *x1) {
				uint4 q;
				asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(ring_addr));
				uint4 xb0 = make_uint4(0u, 0u, 0u, 0u), xb1 = make_uint4(0u, 0u, 0u, 0u);
				if (have_row0) xb0 = *reinterpret_cast<const uint4 *>(x0);
				if (!M8 && have_row1) xb1 = *reinterpret_cast<const uint4 *>(x1);
				const uint32_t qv[4] = {q.x, q.y, q.z, q.w};
				uint32_t a04[4], a15[4], a26[4], a37[4];
#pragma unroll
				for (int c = 0; c < 4; ++c) {
					const uint32_t w = qv[c], w8 = w >> 8;
					a04[c] = lop3_and_or(w, MASK_LO, MAGIC_1024);       // 1024 + q      (k0, k4)
					a15[c] = lop3_and_or(w, MASK_HI, MAGIC_1024);       // 1024 + 16 q   (k1, k5)
					a26[c] = lop3_and_or(w8, MASK_LO, MAGIC_1024);      // 1024 + q      (k2, k6)
					a37[c] = lop3_and_or(w8, MASK_HI, MAGIC_1024);      // 1024 + 16 q   (k3, k7)
				}
				// A rows (gid, gid+8) = lane columns (2pr, 2pr+1); B = x rows; D = (column, batch row)
#pragma unroll
				for (int pr = 0; pr < 2; ++pr) {
					float(&d0)[4] = *reinterpret_cast<float(*)[4]>(&g[0][2 * pr][0]);
					mma16816(d0, a04[2 * pr], a04[2 * pr + 1], a15[2 * pr], a15[2 * pr + 1], xb0.x, xb0.y);
					mma16816(d0, a26[2 * pr], a26[2 * pr + 1], a37[2 * pr], a37[2 * pr + 1], xb0.z, xb0.w);
					if (!M8) {
						float(&d1)[4] = *reinterpret_cast<float(*)[4]>(&g[MB - 1][2 * pr][0]);
						mma16816(d1, a04[2 * pr], a04[2 * pr + 1], a15[2 * pr], a15[2 * pr + 1], xb1.x, xb1.y);
						mma16816(d1, a26[2 * pr], a26[2 * pr + 1], a37[2 * pr], a37[2 * pr + 1], xb1.z, xb1.w);
					}
				}
			};
			// begin(): refill the stage drained one iteration ago, then wait for this chunk's data
			auto begin = [&]() -> bool {
				if (!first) produce();
				first = false;
				const bool ok = mbar_wait_bounded(bar_w + 8 * stage, parity);
				return ok;
			};
			auto end = [&]() {
				__syncwarp();
				if (++stage == p.nstage) {
					stage = 0;
					parity ^= 1u;
				}
			};
			auto xoff_of = [&](int chunk, int l) { return (chunk - c_lo) * 256 + (LIN ? l * 64 : ((l & 1) + 8 * (l >> 1)) * 16); };
			auto ring_of = [&](int l) { return ((l & 1) ? ring_odd : ring_even) + stage * SK_CHUNK_BYTES + (l >> 1) * 1024; };
			clear(gA);
			clear(gB);

			if (SPG_T == 0) {
				// Groups of 128 rows or more (a multiple of the 4 steps of a chunk).  The two
				// accumulator sets alternate by GROUP: while one group's MMAs are in flight the
				// finished set of the previous group is flushed, one chunk later.
				int chunk = w_lo;
				int gi = (w_lo * 4) / p.spg - g_lo;
				int left = p.spg - (w_lo * 4) % p.spg;          // steps left in the current group
				bool pendA = false, pendB = false;
				int giA = 0, giB = 0;
				while (chunk < w_hi) {
					bool done;
					do {
						if (!begin()) { failed = true; break; }
#pragma unroll
						for (int l = 0; l < 4; ++l) step(gA, ring_of(l), xrow0 + xoff_of(chunk, l), xrow1 + xoff_of(chunk, l));
						if (pendB) {
							flush(gB, giB);
							pendB = false;
						}
						left -= 4;
						++chunk;
						done = (left == 0) || (chunk == w_hi);
						end();
					} while (!done);
					if (failed) break;
					pendA = true;
					giA = gi;
					if (left == 0) {
						++gi;
						left = p.spg;
					}
					if (chunk >= w_hi) break;
					do {
						if (!begin()) { failed = true; break; }
#pragma unroll
						for (int l = 0; l < 4; ++l) step(gB, ring_of(l), xrow0 + xoff_of(chunk, l), xrow1 + xoff_of(chunk, l));
						if (pendA) {
							flush(gA, giA);
							pendA = false;
						}
						left -= 4;
						++chunk;
						done = (left == 0) || (chunk == w_hi);
						end();
					} while (!done);
					if (failed) break;
					pendB = true;
					giB = gi;
					if (left == 0) {
						++gi;
						left = p.spg;
					}
				}
				if (pendA) flush(gA, giA);
				if (pendB) flush(gB, giB);
			} else {
				// 32- or 64-row groups: SPG_T steps per group, flushes at compile-time positions
				constexpr int SP = SPG_T ? SPG_T : 1;
				for (int chunk = w_lo; chunk < w_hi; ++chunk) {
					if (!begin()) { failed = true; break; }
#pragma unroll
					for (int l = 0; l < 4; ++l) {
						step(gA, ring_of(l), xrow0 + xoff_of(chunk, l), xrow1 + xoff_of(chunk, l));
						if ((l + 1) % SP == 0) flush(gA, (chunk * 4 + l) / SP - g_lo);
					}
					end();
				}
			}
			if (NSTREAM == 1 || s == 0) {
#pragma unroll
				for (int b = 0; b < MB; ++b)
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						acc[0][b][c][0] = accw[b][c][0];
						acc[0][b][c][1] = accw[b][c][1];
					}
			} else {
#pragma unroll
				for (int b = 0; b < MB; ++b)
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						acc[NSTREAM - 1][b][c][0] = accw[b][c][0];
						acc[NSTREAM - 1][b][c][1] = accw[b][c][1];
					}
			}
			if (failed) break;
		}
	}
	if (failed && lane == 0) atomicExch(p.ws_ticket + SK_STATUS_SLOT, 1);          // a TMA load never completed
	if (tid == 0 && (smem_u32(smem) & 1023u) != 0) atomicExch(p.ws_ticket + SK_STATUS_SLOT, 2);   // swizzle needs 1 KB alignment
	__syncthreads();            // every warp is done with its ring: the region becomes `red`

	// ---- reduce the KW warp-rows ---------------------------------------------------------
	// red[kw][stream][row][128]; this lane holds columns wn*32 + 4*gid + 0..3 of rows 2*tig + {0,1} (+8)
#pragma unroll
	for (int s = 0; s < NSTREAM; ++s)
#pragma unroll
		for (int b = 0; b < MB; ++b)
#pragma unroll
			for (int h = 0; h < 2; ++h) {
				float *r = red + ((size_t)(kw * NSTREAM + s) * ROWS + (b * 8 + 2 * tig + h)) * BN + wn * 32 + gid * 4;
				*reinterpret_cast<float4 *>(r) = make_float4(acc[s][b][0][h], acc[s][b][1][h], acc[s][b][2][h], acc[s][b][3][h]);
			}
	__syncthreads();

	// tile sums land in red[0][stream][row][col] (slot of warp-row 0); with split-K they are
	// first exchanged through the workspace.
	const int nelem = NSTREAM * p.M * BN;        // only rows < M matter
	float *wsp = p.ws_partial + (size_t)(tile * p.splitk + split) * nelem;   // [stream][row < M][128]
	if (M8) {
		// few rows: one element per thread and pass
#pragma unroll 1
		for (int e = tid; e < nelem; e += NT) {
			const int s = (NSTREAM == 2 && e >= p.M * BN) ? 1 : 0, rc = e - s * (p.M * BN);
			const int row = rc >> BSH, col = rc & (BN - 1);
			float v = 0.f;
#pragma unroll
			for (int k = 0; k < KW; ++k) v += red[((size_t)(k * NSTREAM + s) * ROWS + row) * BN + col];
			{
				// remove the 1024-offsets and the zero points of this CTA's K-slice
				const int ng = (c_hi * 128 - 1) / p.groupsize - g_lo + 1;
				const __half *zz = s_zz + (size_t)s * p.strip_groups * BN + col;
				const __half *sc = s_sc + (size_t)s * p.strip_groups * BN + col;
				float corr = 0.f;
#pragma unroll 2
				for (int gi = 0; gi < ng; ++gi) {
					const float2 cs = s_cs[gi * 16 + row];
					corr = fmaf(__half2float(sc[(size_t)gi * BN]), fmaf(__half2float(zz[(size_t)gi * BN]), cs.y, cs.x), corr);
				}
				v -= corr;
			}
			if (p.splitk == 1 || (p.ws_words && split == p.splitk - 1)) {
				red[((size_t)s * ROWS + row) * BN + col] = v;
			} else if (p.ws_words) {
				const unsigned long long w = ((unsigned long long)WORD_TAG << 32) | (unsigned long long)__float_as_uint(v);
				asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p.ws_words + (size_t)(tile * p.splitk + split) * nelem + e), "l"(w) : "memory");
			} else {
				__stcg(wsp + e, v);
			}
		}
	} else
	{
		// A thread owns one (stream, column) pair and every tpp-th batch row.  It first builds the
		// correction sum_g s*(C + z*S) of its rows (scale and zero are read once per group), then
		// adds the KW warp-row partials and subtracts it.
		constexpr int PAIRS = NSTREAM * BN, TPP = NT / PAIRS, RPT = 16 / TPP;
		const int pair = tid % PAIRS, sub = tid / PAIRS;
		const int s = pair >> BSH, col = pair & (BN - 1);
		const int ng = (c_hi * 128 - 1) / p.groupsize - g_lo + 1;
		const __half *zz = s_zz + (size_t)s * p.strip_groups * BN + col;
		const __half *sc = s_sc + (size_t)s * p.strip_groups * BN + col;
		float corr[RPT];
#pragma unroll
		for (int i = 0; i < RPT; ++i) corr[i] = 0.f;
#pragma unroll 1
		for (int gi = 0; gi < ng; ++gi) {
			const float sv = __half2float(sc[(size_t)gi * BN]);
			const float sz = sv * __half2float(zz[(size_t)gi * BN]);
#pragma unroll
			for (int i = 0; i < RPT; ++i) {
				const int row = sub + i * TPP;
				if (row < p.M) {
					const float2 cs = s_cs[gi * 16 + row];
					corr[i] = fmaf(sv, cs.x, fmaf(sz, cs.y, corr[i]));
				}
			}
		}
#pragma unroll
		for (int i = 0; i < RPT; ++i) {
			const int row = sub + i * TPP;
			if (row < p.M) {
				float v = 0.f;
#pragma unroll
				for (int k = 0; k < KW; ++k) v += red[((size_t)(k * NSTREAM + s) * ROWS + row) * BN + col];
				v -= corr[i];
				if (p.splitk == 1)
					red[((size_t)s * ROWS + row) * BN + col] = v;
				else
					__stcg(wsp + (size_t)s * p.M * BN + row * BN + col, v);
			}
		}
	}
	if (M8 && p.splitk > 1 && p.ws_words) {
		if (split != p.splitk - 1) {                         // partial sums are on their way: done
			return;
		}
		unsigned long long *wt = p.ws_words + (size_t)tile * p.splitk * nelem;
		const unsigned long long t0 = global_timer_ns();
		bool ok = true;
#pragma unroll 1
		for (int e = tid; e < nelem; e += NT) {              // same thread -> element mapping as above and below
			const int s = (NSTREAM == 2 && e >= p.M * BN) ? 1 : 0, rc = e - s * (p.M * BN);
			float *own = red + ((size_t)s * ROWS + (rc >> BSH)) * BN + (rc & (BN - 1));
			float v = 0.f;
#pragma unroll 1
			for (int k0 = 0; k0 < p.splitk - 1; k0 += 8) {
				unsigned long long w[8];
#pragma unroll
				for (int k = 0; k < 8; ++k)
					if (k0 + k < p.splitk - 1) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[k]) : "l"(wt + (size_t)(k0 + k) * nelem + e) : "memory");
#pragma unroll
				for (int k = 0; k < 8; ++k) {
					if (k0 + k < p.splitk - 1) {
						unsigned long long *src = wt + (size_t)(k0 + k) * nelem + e;
						while ((unsigned)(w[k] >> 32) != WORD_TAG) {   // not there yet: poll this word (bounded in time)
							if (global_timer_ns() - t0 > 2000000000ull) {
								ok = false;
								break;
							}
							asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[k]) : "l"(src) : "memory");
						}
						v += __uint_as_float((unsigned)w[k]);        // split order: 0, 1, ..., then this CTA's own share
						asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(src), "l"(0ull) : "memory");
					}
				}
			}
			*own = v + *own;
		}
		if (!ok) atomicExch(p.ws_ticket + SK_STATUS_SLOT, 6);      // a split never delivered its partial sums
	} else if (p.splitk > 1) {
		// the ticket is an acquire-release atomic at GPU scope after the CTA barrier: it releases the partial
		// sums this CTA stored and acquires those of the CTAs that arrived earlier (no separate fences)
		__syncthreads();
		if (tid == 0) {
			int t;
			asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(p.ws_ticket + tile) : "memory");
			const int last = (t == p.splitk - 1);
			if (last) p.ws_ticket[tile] = 0;        // leave the counter ready for the next launch
			s_last = last;
		}
		__syncthreads();
		if (!s_last) {
			return;
		}
		const float *wt = p.ws_partial + (size_t)tile * p.splitk * nelem;
		if (M8) {
#pragma unroll 1
			for (int e = tid; e < nelem; e += NT) {
				const int s = (NSTREAM == 2 && e >= p.M * BN) ? 1 : 0, rc = e - s * (p.M * BN);
				const int row = rc >> BSH, col = rc & (BN - 1);
				float v = 0.f;        // eight loads in flight, then a fixed-order sum
#pragma unroll 1
				for (int k0 = 0; k0 < p.splitk; k0 += 8) {
					float part[8];
#pragma unroll
					for (int k = 0; k < 8; ++k) part[k] = (k0 + k < p.splitk) ? __ldcg(wt + (size_t)(k0 + k) * nelem + e) : 0.f;
#pragma unroll
					for (int k = 0; k < 8; ++k) v += part[k];
				}
				red[((size_t)s * ROWS + row) * BN + col] = v;
			}
		} else {
#pragma unroll 1
			for (int e0 = tid; e0 < nelem; e0 += NT * 4) {        // four elements x eight splits in flight per thread; fixed split order
				float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
				for (int k0 = 0; k0 < p.splitk; k0 += 8) {
					float t[8][4];
#pragma unroll
					for (int kk = 0; kk < 8; ++kk)
#pragma unroll
						for (int j = 0; j < 4; ++j)
							t[kk][j] = (k0 + kk < p.splitk && e0 + j * NT < nelem) ? __ldcg(wt + (size_t)(k0 + kk) * nelem + e0 + j * NT) : 0.f;
#pragma unroll
					for (int kk = 0; kk < 8; ++kk)
#pragma unroll
						for (int j = 0; j < 4; ++j) v[j] += t[kk][j];
				}
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					const int e = e0 + j * NT;
					if (e < nelem) {
						const int s = (NSTREAM == 2 && e >= p.M * BN) ? 1 : 0, rc = e - s * (p.M * BN);
						red[((size_t)s * ROWS + (rc >> BSH)) * BN + (rc & (BN - 1))] = v[j];
					}
				}
			}
		}
	}
	__syncthreads();

	const int epi_n = (EPI == EPI_ROPE) ? p.M * 64 : p.M * BN;
	const int e_lo = 0, e_hi = epi_n;
	const float *fin = red;
	// ---- epilogue from shared memory ---------------------------------------------------------
	if (EPI == EPI_PLAIN || EPI == EPI_SILU) {
		__shared__ float s_ss[64];                           // [row][quarter of the tile]
		const bool want_ss = (EPI == EPI_PLAIN) && p.ss_out != nullptr;
		const bool ar = (EPI == EPI_PLAIN) && !NARROW && p.ar_world > 1;
		if (ar) {
			__shared__ unsigned s_seq;
			if (tid == 0) s_seq = p.ar_seq[tile] + 1u;           // written by the previous launch on this buffer, long complete
			__syncthreads();
			const unsigned seq = s_seq;
			// The receive area is double-buffered by the parity of the sequence number: a rank that runs ahead
			// into call n + 1 on the same buffers writes the other half, so a peer that is still reading the
			// words of call n never sees them overwritten (call n + 2 cannot start before that peer has pushed
			// its own words of call n + 1, i.e. after it has finished reading call n).
			const size_t half = (size_t)(seq & 1u) * ((size_t)8 * gridDim.x * (16 * BN));
			const size_t slot = half + ((size_t)p.ar_rank * gridDim.x + tile) * (16 * BN);      // where this rank's words go in a peer's buffer
#pragma unroll 1
			for (int e = e_lo + tid; e < e_hi; e += NT) {
				const int n = n0 + (e & (BN - 1));
				float v = 0.f;
				if (n < p.N) {
					v = fin[e];                                  // [row][BN] is contiguous: e = row * BN + col
					if (p.bias) v += __half2float(p.bias[n]);
				}
				red[e] = v;                                      // own share, read back by the same thread below
				const unsigned long long w = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
#pragma unroll 1
				for (int r = 0; r < p.ar_world; ++r)
					if (r != p.ar_rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.ar_buf[r] + slot + e), "l"(w) : "memory");
			}
			const unsigned long long t0 = global_timer_ns();
			bool ok = true;
#pragma unroll 1
			for (int e = e_lo + tid; e < e_hi; e += NT) {
				float v = 0.f;
#pragma unroll 1
				for (int r = 0; r < p.ar_world; ++r) {           // rank order: identical sums everywhere
					if (r == p.ar_rank) {
						v += red[e];
						continue;
					}
					const unsigned long long *src = p.ar_buf[p.ar_rank] + half + ((size_t)r * gridDim.x + tile) * (16 * BN) + e;
					unsigned long long w;
#pragma unroll 1
					for (;;) {
						asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
						if ((unsigned)(w >> 32) == seq) break;
						if (global_timer_ns() - t0 > 2000000000ull) {        // a peer never arrived
							ok = false;
							break;
						}
					}
					v += __uint_as_float((unsigned)w);
				}
				red[e] = v;
			}
			if (!ok) atomicExch(p.ws_ticket + SK_STATUS_SLOT, 5);
			if (tid == 0) p.ar_seq[tile] = seq;
		}
#pragma unroll 1
		for (int e = e_lo + tid; e < e_hi; e += NT) {        // whole warps enter or skip (bounds are multiples of 32)
			const int row = e >> BSH, col = e & (BN - 1), n = n0 + col;
			float sq = 0.f;
			if (n < p.N) {
				float v = fin[(size_t)row * BN + col];
				if (EPI == EPI_SILU) {
					v = silu_f32(v) * fin[((size_t)ROWS + row) * BN + col];
				} else if (e == tid) {
					if (p.bias && !ar) v += pre_bias;
					if (p.residual) v += pre_res;
				} else {
					if (p.bias && !ar) v += __half2float(p.bias[n]);
					if (p.residual) v += __half2float(p.residual[(size_t)row * p.ldr + n]);
				}
				const __half hv = __float2half_rn(v);
				p.y[(size_t)row * p.ldy + n] = hv;
				const float f = __half2float(hv);
				sq = f * f;
			}
			if (want_ss) {
#pragma unroll
				for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
				if (lane == 0) s_ss[e >> 5] = sq;
			}
		}
		if (want_ss) {
			__syncthreads();
			// one value per (row, 32 columns): [row][N / 32]
			if (tid < p.M * NWN) p.ss_out[(size_t)(tid / NWN) * (gridDim.x * NWN) + tile * NWN + (tid % NWN)] = s_ss[tid];
		}
	} else {
		// rotary: the tile is exactly one head (head_dim == 128) of section Q, K or V
		const int section = n0 / p.hidden, head = (n0 - section * p.hidden) >> 7;
#pragma unroll 1
		for (int e = e_lo + tid; e < e_hi; e += NT) {
			const int row = e >> 6, d = e & 63;
			const float a = fin[(size_t)row * BN + d], b = fin[(size_t)row * BN + d + 64];
			int pos = p.pos[row];
			if (pos < 0 || pos >= p.max_pos) {          // never index the tables / the cache out of range
				atomicExch(p.ws_ticket + SK_STATUS_SLOT, 4);
				pos = 0;
				if (section != 0) continue;             // K / V of such a row are dropped, not written over cache row 0
			}
			float o1 = a, o2 = b;
			if (section < 2) {
				const __half *ct = p.cos_t + (size_t)pos * 128, *st = p.sin_t + (size_t)pos * 128;
				o1 = a * __half2float(ct[d]) - b * __half2float(st[d]);
				o2 = b * __half2float(ct[d + 64]) + a * __half2float(st[d + 64]);
			}
			__half *dst;
			if (section == 0) {
				dst = p.q_out + (size_t)row * p.q_stride_m + head * 128;
			} else {
				const int bi = row / p.tokens_per_batch, ti = row - bi * p.tokens_per_batch;
				dst = (section == 1 ? p.k_out : p.v_out) + (size_t)bi * p.kv_sb + (size_t)ti * p.kv_st +
					  (size_t)head * p.kv_sh + (size_t)pos * p.kv_sp;
			}
			dst[d] = __float2half_rn(o1);
			dst[d + 64] = __float2half_rn(o2);
		}
	}
}

// ---- act-order gather: out[m][k] = x[m][perm[k]], 8 elements per thread -------------------
__global__ void __launch_bounds__(256) gather_x_kernel(const __half *__restrict__ x, long long ldx, const int32_t *__restrict__ perm,
														__half *__restrict__ out, int K) {
	const int unit = blockIdx.x * 256 + threadIdx.x, row = blockIdx.y;
	pdl_trigger();
	if (unit * 8 >= K) return;
	const int4 pa = __ldg(reinterpret_cast<const int4 *>(perm + unit * 8));       // the permutation does not depend on earlier kernels
	const int4 pb = __ldg(reinterpret_cast<const int4 *>(perm + unit * 8 + 4));
	pdl_wait();
	const unsigned short *xr = reinterpret_cast<const unsigned short *>(x) + (size_t)row * ldx;
	const uint32_t h0 = xr[pa.x], h1 = xr[pa.y], h2 = xr[pa.z], h3 = xr[pa.w];
	const uint32_t h4 = xr[pb.x], h5 = xr[pb.y], h6 = xr[pb.z], h7 = xr[pb.w];
	*reinterpret_cast<uint4 *>(out + (size_t)row * K + unit * 8) = make_uint4(h0 | (h1 << 16), h2 | (h3 << 16), h4 | (h5 << 16), h6 | (h7 << 16));
}

// ---- general kernel: any M, any g_idx, N % 8 == 0, K % 8 == 0 ---------------------------
// One thread per output column, 8 batch rows per CTA row-block; fp32 weights (q-z)*s.
template <int NSTREAM>
__global__ void __launch_bounds__(128) general_kernel(const __half *__restrict__ x, long long ldx,
													  const int32_t *__restrict__ qw0, const int32_t *__restrict__ qz0,
													  const __half *__restrict__ sc0, const int32_t *__restrict__ qw1,
													  const int32_t *__restrict__ qz1, const __half *__restrict__ sc1,
													  const int32_t *__restrict__ g_idx, const int32_t *__restrict__ perm,
													  const __half *__restrict__ bias, const __half *__restrict__ residual,
													  long long ldr, __half *__restrict__ y, long long ldy, int M, int K, int N,
													  int groupsize) {
	const int n = blockIdx.x * 128 + threadIdx.x;
	const int m0 = blockIdx.y * 8;
	if (n >= N) return;
	const int mr = min(8, M - m0);
	float acc[NSTREAM][8];
#pragma unroll
	for (int s = 0; s < NSTREAM; ++s)
#pragma unroll
		for (int m = 0; m < 8; ++m) acc[s][m] = 0.f;
	const int nz = N >> 3, zsh = (n & 7) * 4;
	for (int r = 0; r < K / 8; ++r) {
		uint32_t q[NSTREAM];
		q[0] = (uint32_t)qw0[(size_t)r * N + n];
		if (NSTREAM == 2) q[NSTREAM - 1] = (uint32_t)qw1[(size_t)r * N + n];
#pragma unroll
		for (int i = 0; i < 8; ++i) {
			const int k = r * 8 + i;
			const int g = g_idx ? g_idx[k] : k / groupsize;
			const int kx = perm ? perm[k] : k;
			float w[NSTREAM];
#pragma unroll
			for (int s = 0; s < NSTREAM; ++s) {
				const int32_t *qz = s ? qz1 : qz0;
				const __half *sc = s ? sc1 : sc0;
				const int zz = (int)((((uint32_t)qz[(size_t)g * nz + (n >> 3)]) >> zsh) & 0xFu) + 1;
				w[s] = (float)((int)((q[s] >> (4 * i)) & 0xFu) - zz) * __half2float(sc[(size_t)g * N + n]);
			}
#pragma unroll
			for (int m = 0; m < 8; ++m) {
				if (m < mr) {
					const float xv = __half2float(x[(size_t)(m0 + m) * ldx + kx]);
#pragma unroll
					for (int s = 0; s < NSTREAM; ++s) acc[s][m] = fmaf(xv, w[s], acc[s][m]);
				}
			}
		}
	}
#pragma unroll
	for (int m = 0; m < 8; ++m) {
		if (m < mr) {
			float v = acc[0][m];
			if (NSTREAM == 2) {
				v = silu_f32(v) * acc[NSTREAM - 1][m];
			} else {
				if (bias) v += __half2float(bias[n]);
				if (residual) v += __half2float(residual[(size_t)(m0 + m) * ldr + n]);
			}
			y[(size_t)(m0 + m) * ldy + n] = __float2half_rn(v);
		}
	}
}

}   // namespace gptq
