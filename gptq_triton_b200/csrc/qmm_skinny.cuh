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
// 0x00F000F0 yields the half2 pairs (k0,k4) (k1,k5) and, after >>8, (k2,k6) (k3,k7) as
// 1024+q resp. 1024+16q; one sub / fma per pair turns them into the exact integers
// q - zero.  They are the A operand of mma.sync.m16n8k16 (16 weight columns x 16 k); the
// batch rows of x are the B operand, staged in shared memory in the matching k order
// [0,4,1,5,2,6,3,7].  Integer dot products accumulate in fp32 per group and are scaled by
// the group's fp32 scale when the group ends, so no weight is ever rounded to fp16: the
// result equals an fp32-accumulated (q-z-1)*s reference up to fp32 summation order.
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
	const int32_t *perm;
	int M, K, N, groupsize;
	int spg;               // 32-row steps per group (1, 2 or a multiple of 4)
	int total_chunks;      // K / 128
	int chunks_per_split;
	int splitk;
	int nstage;
	int xs_stride;         // bytes between rows of the staged x slice
	int xs_bytes;          // M * xs_stride rounded up to 128
	int strip_groups;      // capacity (groups) of the zero / scale strips per stream
	float *ws_partial;
	int *ws_ticket;
	// EPI_PLAIN / EPI_SILU
	const __half *bias;
	const __half *residual;
	long long ldr;
	__half *y;
	long long ldy;
	// EPI_ROPE
	const __half *cos_t, *sin_t;
	const int32_t *pos;
	__half *q_out, *k_out, *v_out;
	long long q_stride_m, kv_sb, kv_st, kv_sh, kv_sp;
	int tokens_per_batch, hidden;
};

// SPG_T: steps per group known at compile time (1 or 2), or 0 when a group spans whole chunks.
template <int KW, int NSTREAM, bool M8, int SPG_T, int EPI>
__global__ void __launch_bounds__(KW * 128, 4 / KW)
	skinny_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, const SkinnyParams p) {
	extern __shared__ __align__(1024) unsigned char smem[];
	constexpr int NT = KW * 128;
	constexpr int NWARP = KW * 4;
	constexpr int ROWS = M8 ? 8 : 16;
	constexpr int MB = M8 ? 1 : 2;             // batch-row blocks of 8

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int wn = warp & 3, kw = warp >> 2, gid = lane >> 2, tig = lane & 3;
	const int tile = blockIdx.x, split = blockIdx.y;
	const int n0 = tile * SK_BN, n0w = n0 + wn * 32;
	const bool warp_active = n0w < p.N;

	// shared memory: [ ring | mbarriers | x slice | zero strips | scale strips ]; the ring
	// region is reused as the reduce buffer once the stream has drained
	unsigned char *ring_all = smem;
	const int ring_bytes = NWARP * p.nstage * SK_CHUNK_BYTES;
	uint64_t *bars = reinterpret_cast<uint64_t *>(smem + ring_bytes);
	unsigned char *xs = smem + ring_bytes + SK_BAR_BYTES;
	__half *s_ze = reinterpret_cast<__half *>(xs + p.xs_bytes);                  // [stream][group][128] = 1024 + zero
	__half *s_sc = s_ze + NSTREAM * p.strip_groups * SK_BN;                      // [stream][group][128]
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
				fence_proxy_async();
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
	for (int s = 0; s < p.nstage; ++s) produce();

	// ---- stage zero / scale strips and the x slice ---------------------------------------
	const int g_lo = (c_lo * 128) / p.groupsize;
	{
		const int ng = (c_hi * 128 - 1) / p.groupsize - g_lo + 1;
		const int nz = p.N >> 3;
		for (int idx = tid; idx < NSTREAM * ng * 16; idx += NT) {
			const int s = idx / (ng * 16), r = idx - s * (ng * 16);
			const int gi = r >> 4, c = r & 15;              // 8 columns per item
			if (n0 + c * 8 < p.N) {
				const int32_t *qz = (NSTREAM == 2 && s) ? p.qz1 : p.qz0;
				const __half *sc = (NSTREAM == 2 && s) ? p.sc1 : p.sc0;
				const uint32_t z = (uint32_t)__ldg(qz + (size_t)(g_lo + gi) * nz + (n0 >> 3) + c);
				const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(sc + (size_t)(g_lo + gi) * p.N + n0 + c * 8));
				uint4 ze;       // half(1024 + zero) = 0x6400 + (stored + 1), two per word
				ze.x = 0x64016401u + ((z & 0xFu) | ((z & 0xF0u) << 12));
				ze.y = 0x64016401u + (((z >> 8) & 0xFu) | (((z >> 8) & 0xF0u) << 12));
				ze.z = 0x64016401u + (((z >> 16) & 0xFu) | (((z >> 16) & 0xF0u) << 12));
				ze.w = 0x64016401u + (((z >> 24) & 0xFu) | (((z >> 24) & 0xF0u) << 12));
				const size_t o = (size_t)(s * p.strip_groups + gi) * SK_BN + c * 8;
				*reinterpret_cast<uint4 *>(s_ze + o) = ze;
				*reinterpret_cast<uint4 *>(s_sc + o) = sv;
			}
		}
		// x slice: [row < M][unit of 8 k] in k order 0,4,1,5,2,6,3,7.  Loads of a batch of
		// items are issued together so that their latencies overlap.
		const int units = (c_hi - c_lo) * 16;
		const int nitem = p.M * units;
		constexpr int XB = 4;
		for (int base = tid; base < nitem; base += NT * XB) {
			uint4 v[XB];
			if (p.perm == nullptr) {
#pragma unroll
				for (int j = 0; j < XB; ++j) {
					const int idx = base + j * NT;
					if (idx < nitem) {
						const int row = idx / units, unit = idx - row * units;
						v[j] = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)row * p.ldx + (c_lo * 16 + unit) * 8));
					}
				}
			} else {
				int4 pa[XB], pb[XB];
#pragma unroll
				for (int j = 0; j < XB; ++j) {
					const int idx = base + j * NT;
					if (idx < nitem) {
						const int unit = idx % units;
						const int k = (c_lo * 16 + unit) * 8;
						pa[j] = __ldg(reinterpret_cast<const int4 *>(p.perm + k));
						pb[j] = __ldg(reinterpret_cast<const int4 *>(p.perm + k + 4));
					}
				}
#pragma unroll
				for (int j = 0; j < XB; ++j) {
					const int idx = base + j * NT;
					if (idx < nitem) {
						const unsigned short *xr = reinterpret_cast<const unsigned short *>(p.x) + (size_t)(idx / units) * p.ldx;
						const uint32_t h0 = __ldg(xr + pa[j].x), h1 = __ldg(xr + pa[j].y), h2 = __ldg(xr + pa[j].z), h3 = __ldg(xr + pa[j].w);
						const uint32_t h4 = __ldg(xr + pb[j].x), h5 = __ldg(xr + pb[j].y), h6 = __ldg(xr + pb[j].z), h7 = __ldg(xr + pb[j].w);
						v[j] = make_uint4(h0 | (h1 << 16), h2 | (h3 << 16), h4 | (h5 << 16), h6 | (h7 << 16));
					}
				}
			}
#pragma unroll
			for (int j = 0; j < XB; ++j) {
				const int idx = base + j * NT;
				if (idx < nitem) {
					const int row = idx / units, unit = idx - row * units;
					uint4 o;
					o.x = __byte_perm(v[j].x, v[j].z, 0x5410);    // (x0, x4)
					o.y = __byte_perm(v[j].x, v[j].z, 0x7632);    // (x1, x5)
					o.z = __byte_perm(v[j].y, v[j].w, 0x5410);    // (x2, x6)
					o.w = __byte_perm(v[j].y, v[j].w, 0x7632);    // (x3, x7)
					*reinterpret_cast<uint4 *>(xs + (size_t)row * p.xs_stride + unit * 16) = o;
				}
			}
		}
	}
	__syncthreads();

	// ---- main loop ---------------------------------------------------------------------
	// acc[stream][column 0..3 of this lane][batch row 2*tig + {0,1} (+8 for the second block)]
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
		// makes the quarter-warp reads below conflict-free.
		// (With 32-row groups a step must stay inside one group, so there the rows are
		// 4*l + tig; that variant has 2-way conflicts.)
		constexpr bool LIN = (SPG_T == 1);
		const int row_a = LIN ? tig : 2 * tig, row_b = LIN ? 4 + tig : 2 * tig + 1;    // steps 0/2 and 1/3
		const unsigned char *xrow0 = xs + (size_t)gid * p.xs_stride + tig * (LIN ? 16 : 32);
		const unsigned char *xrow1 = xs + (size_t)(gid + 8) * p.xs_stride + tig * (LIN ? 16 : 32);
		const uint32_t ring_even = ring_w + row_a * 128 + ((gid ^ row_a) << 4);
		const uint32_t ring_odd = ring_w + row_b * 128 + ((gid ^ row_b) << 4);
		const int strip_col = wn * 32 + gid * 4;
		int stage = 0;
		uint32_t parity = 0;
#pragma unroll
		for (int s = 0; s < NSTREAM; ++s) {
			const __half *ze_s = s_ze + (size_t)s * p.strip_groups * SK_BN + strip_col;
			const __half *sc_s = s_sc + (size_t)s * p.strip_groups * SK_BN + strip_col;
			float gacc[MB][4][2];
			uint32_t ZE[4], ZO[4];
			auto load_zero = [&](int gi) {
				const uint2 zr = *reinterpret_cast<const uint2 *>(ze_s + (size_t)gi * SK_BN);
				ZE[0] = __byte_perm(zr.x, zr.x, 0x1010);
				ZE[1] = __byte_perm(zr.x, zr.x, 0x3232);
				ZE[2] = __byte_perm(zr.y, zr.y, 0x1010);
				ZE[3] = __byte_perm(zr.y, zr.y, 0x3232);
#pragma unroll
				for (int c = 0; c < 4; ++c) {
					ZO[c] = h2_sub(0x63806380u, ZE[c]);      // 960 - (1024 + z) = -(64 + z)
#pragma unroll
					for (int b = 0; b < MB; ++b) gacc[b][c][0] = gacc[b][c][1] = 0.f;
				}
			};
			auto flush = [&](int gi) {
				const uint2 sr = *reinterpret_cast<const uint2 *>(sc_s + (size_t)gi * SK_BN);
				const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.x));
				const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&sr.y));
				const float sf[4] = {s01.x, s01.y, s23.x, s23.y};
#pragma unroll
				for (int b = 0; b < MB; ++b)
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						acc[s][b][c][0] = fmaf(sf[c], gacc[b][c][0], acc[s][b][c][0]);
						acc[s][b][c][1] = fmaf(sf[c], gacc[b][c][1], acc[s][b][c][1]);
					}
			};
			for (int chunk = w_lo; chunk < w_hi; ++chunk) {
				if (!mbar_wait_bounded(bar_w + 8 * stage, parity)) {
					failed = true;
					break;
				}
				const int step0 = chunk * 4;
				if (SPG_T == 0) {
					if (chunk == w_lo || (step0 % p.spg) == 0) load_zero(step0 / p.spg - g_lo);
				}
				const uint32_t st_off = stage * SK_CHUNK_BYTES;
				const int xoff = (chunk - c_lo) * 256;
#pragma unroll
				for (int l = 0; l < 4; ++l) {
					if (SPG_T != 0 && (l % (SPG_T ? SPG_T : 1)) == 0) load_zero((step0 + l) / (SPG_T ? SPG_T : 1) - g_lo);
					uint4 q;
					asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
								 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
								 : "r"(((l & 1) ? ring_odd : ring_even) + st_off + (l >> 1) * 1024));
					const int xo = xoff + (LIN ? l * 64 : ((l & 1) + 8 * (l >> 1)) * 16);
					uint4 xb0 = make_uint4(0u, 0u, 0u, 0u), xb1 = make_uint4(0u, 0u, 0u, 0u);
					if (have_row0) xb0 = *reinterpret_cast<const uint4 *>(xrow0 + xo);
					if (!M8 && have_row1) xb1 = *reinterpret_cast<const uint4 *>(xrow1 + xo);
					const uint32_t qv[4] = {q.x, q.y, q.z, q.w};
					uint32_t a04[4], a15[4], a26[4], a37[4];
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						const uint32_t w = qv[c], w8 = w >> 8;
						a04[c] = h2_sub(lop3_and_or(w, MASK_LO, MAGIC_1024), ZE[c]);
						a15[c] = h2_fma(lop3_and_or(w, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[c]);
						a26[c] = h2_sub(lop3_and_or(w8, MASK_LO, MAGIC_1024), ZE[c]);
						a37[c] = h2_fma(lop3_and_or(w8, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[c]);
					}
					// A rows (gid, gid+8) = lane columns (2pr, 2pr+1); B = x rows; D = (column, batch row)
#pragma unroll
					for (int pr = 0; pr < 2; ++pr) {
						float(&d0)[4] = *reinterpret_cast<float(*)[4]>(&gacc[0][2 * pr][0]);
						mma16816(d0, a04[2 * pr], a04[2 * pr + 1], a15[2 * pr], a15[2 * pr + 1], xb0.x, xb0.y);
						mma16816(d0, a26[2 * pr], a26[2 * pr + 1], a37[2 * pr], a37[2 * pr + 1], xb0.z, xb0.w);
						if (!M8) {
							float(&d1)[4] = *reinterpret_cast<float(*)[4]>(&gacc[MB - 1][2 * pr][0]);
							mma16816(d1, a04[2 * pr], a04[2 * pr + 1], a15[2 * pr], a15[2 * pr + 1], xb1.x, xb1.y);
							mma16816(d1, a26[2 * pr], a26[2 * pr + 1], a37[2 * pr], a37[2 * pr + 1], xb1.z, xb1.w);
						}
					}
					if (SPG_T != 0 && ((l + 1) % (SPG_T ? SPG_T : 1)) == 0) flush((step0 + l) / (SPG_T ? SPG_T : 1) - g_lo);
				}
				if (SPG_T == 0) {
					if (chunk + 1 == w_hi || ((step0 + 4) % p.spg) == 0) flush(step0 / p.spg - g_lo);
				}
				__syncwarp();
				produce();
				if (++stage == p.nstage) {
					stage = 0;
					parity ^= 1u;
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
				float *r = red + ((size_t)(kw * NSTREAM + s) * ROWS + (b * 8 + 2 * tig + h)) * SK_BN + wn * 32 + gid * 4;
				*reinterpret_cast<float4 *>(r) = make_float4(acc[s][b][0][h], acc[s][b][1][h], acc[s][b][2][h], acc[s][b][3][h]);
			}
	__syncthreads();

	// tile sums land in red[0][stream][row][col] (slot of warp-row 0); with split-K they are
	// first exchanged through the workspace.
	const int nelem = NSTREAM * p.M * SK_BN;        // only rows < M matter
	float *wsp = p.ws_partial + (size_t)(tile * p.splitk + split) * nelem;   // [stream][row < M][128]
	for (int e = tid; e < nelem; e += NT) {
		const int s = e / (p.M * SK_BN), rc = e - s * (p.M * SK_BN);
		const int row = rc >> 7, col = rc & 127;
		float v = 0.f;
#pragma unroll
		for (int k = 0; k < KW; ++k) v += red[((size_t)(k * NSTREAM + s) * ROWS + row) * SK_BN + col];
		if (p.splitk == 1)
			red[((size_t)s * ROWS + row) * SK_BN + col] = v;
		else
			__stcg(wsp + e, v);
	}
	if (p.splitk > 1) {
		__threadfence();
		__syncthreads();
		if (tid == 0) {
			const int t = atomicAdd(p.ws_ticket + tile, 1);
			const int last = (t == p.splitk - 1);
			if (last) p.ws_ticket[tile] = 0;        // leave the counter ready for the next launch
			s_last = last;
		}
		__syncthreads();
		if (!s_last) return;
		__threadfence();
		const float *wt = p.ws_partial + (size_t)tile * p.splitk * nelem;
		for (int e = tid; e < nelem; e += NT) {
			const int s = e / (p.M * SK_BN), rc = e - s * (p.M * SK_BN);
			const int row = rc >> 7, col = rc & 127;
			float v = 0.f;
			for (int k = 0; k < p.splitk; ++k) v += __ldcg(wt + (size_t)k * nelem + e);
			red[((size_t)s * ROWS + row) * SK_BN + col] = v;
		}
	}
	__syncthreads();

	// ---- epilogue from shared memory ---------------------------------------------------------
	if (EPI == EPI_PLAIN || EPI == EPI_SILU) {
		for (int e = tid; e < p.M * SK_BN; e += NT) {
			const int row = e >> 7, col = e & 127, n = n0 + col;
			if (n >= p.N) continue;
			float v = red[(size_t)row * SK_BN + col];
			if (EPI == EPI_SILU) {
				v = silu_f32(v) * red[((size_t)ROWS + row) * SK_BN + col];
			} else {
				if (p.bias) v += __half2float(p.bias[n]);
				if (p.residual) v += __half2float(p.residual[(size_t)row * p.ldr + n]);
			}
			p.y[(size_t)row * p.ldy + n] = __float2half_rn(v);
		}
	} else {
		// rotary: the tile is exactly one head (head_dim == 128) of section Q, K or V
		const int section = n0 / p.hidden, head = (n0 - section * p.hidden) >> 7;
		for (int e = tid; e < p.M * 64; e += NT) {
			const int row = e >> 6, d = e & 63;
			const float a = red[(size_t)row * SK_BN + d], b = red[(size_t)row * SK_BN + d + 64];
			const int pos = p.pos[row];
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
