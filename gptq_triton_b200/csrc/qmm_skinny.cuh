// Decode-regime (M <= 16) quantised matmul for sm_100a: an HBM-bound skinny GEMM.
//
// Work split.  A CTA owns 128 output columns (4 warps x 32 columns) and one K-slice
// (grid.y = split-K).  Inside the CTA, KW warp-rows split the slice further, segment by
// segment; a segment is a run of 32-row steps that lies inside one quantisation group.
//
// Weight stream.  In one step a warp reads 4 packed rows x 32 columns = 4 x 128
// contiguous bytes: lane (gid = lane/4, tig = lane%4) fetches 16 bytes = 4 columns of
// packed row 4*step + tig with cp.async into a private 8-deep ring in shared memory
// (each lane reads back only what it fetched, so no barrier is involved).
//
// Math.  The 8 nibbles of a word are the 8 K-values of one column.  Masking with
// 0x000F000F / 0x00F000F0 yields the half2 pairs (k0,k4) (k1,k5) and, after >>8,
// (k2,k6) (k3,k7) as 1024+q resp. 1024+16q; one sub / fma per pair turns them into the
// exact integers q - zero.  These feed mma.sync.m16n8k16 as the B operand; the batch rows
// of x are the A operand, staged in shared memory in the matching k order
// [0,4,1,5,2,6,3,7].  The integer dot products accumulate in fp32 per segment and are
// multiplied by the group's scale in fp32 at the segment end, so a weight is never
// rounded to fp16: the result equals an fp32-accumulated (q-z-1)*s reference up to fp32
// summation order.
//
// Reduction.  KW warp-rows reduce through shared memory; split-K CTAs write fp32
// partials to the workspace and take a ticket; the last CTA of a tile sums the partials
// in fixed order (deterministic) and runs the epilogue: bias/residual, SiLU(gate)*up,
// or rotary embedding with a scatter into Q / K / V (or the KV cache).
#pragma once

#include "common.cuh"

namespace gptq {

enum { EPI_PLAIN = 0, EPI_SILU = 1, EPI_ROPE = 2 };

constexpr int SK_BN = 128;      // columns per CTA
constexpr int SK_D = 8;         // cp.async ring depth (steps)
constexpr int SK_TICKET_BYTES = 16384;

struct SkinnyParams {
	const __half *x;
	long long ldx;
	const int32_t *qw0, *qw1;
	const int32_t *qz0, *qz1;
	const __half *sc0, *sc1;
	const int32_t *perm;
	int M, K, N, groupsize;
	int seg_steps;        // steps (of 32 rows) per segment
	int total_steps;      // K / 32
	int total_segs;       // ceil(total_steps / seg_steps)
	int segs_per_split;
	int splitk;
	int xs_stride;        // bytes between rows of the staged x slice
	int xs_bytes;         // rows * xs_stride, rounded up to 128
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

template <int KW, int NSTREAM, bool M8, int EPI>
__global__ void __launch_bounds__(KW * 128, 1) skinny_kernel(const SkinnyParams p) {
	extern __shared__ __align__(128) unsigned char smem[];
	constexpr int NT = KW * 128;
	constexpr int ROWS = M8 ? 8 : 16;
	constexpr int D = SK_D;

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int wn = warp & 3, kw = warp >> 2, gid = lane >> 2, tig = lane & 3;
	const int tile = blockIdx.x, split = blockIdx.y;
	const int n0 = tile * SK_BN, n0w = n0 + wn * 32;
	const bool warp_active = n0w < p.N;

	unsigned char *xs = smem;
	unsigned char *scratch = smem + p.xs_bytes;                        // ring, later the reduce buffer
	uint4 *ring = reinterpret_cast<uint4 *>(scratch) + warp * (D * 32) + lane;
	float *red = reinterpret_cast<float *>(scratch);
	__shared__ int s_last;

	const int seg0 = split * p.segs_per_split;
	const int seg1 = min(seg0 + p.segs_per_split, p.total_segs);
	const int step_lo = seg0 * p.seg_steps;                            // first step of this CTA's slice
	const int step_hi = min(seg1 * p.seg_steps, p.total_steps);

	// number of steps this warp will consume
	int nsteps = 0;
	if (warp_active) {
		for (int s = seg0 + kw; s < seg1; s += KW) nsteps += min(p.seg_steps, p.total_steps - s * p.seg_steps);
		nsteps *= NSTREAM;
	}

	// ---- weight stream: issue side ------------------------------------------------
	int is_seg = seg0 + kw, is_stream = 0, is_local = 0, issued = 0;
	int is_len = min(p.seg_steps, p.total_steps - is_seg * p.seg_steps);
	const size_t col_off = (size_t)(n0w + gid * 4);
	auto issue = [&]() {
		if (issued < nsteps) {
			const int R = (is_seg * p.seg_steps + is_local) * 4 + tig;
			const int32_t *base = (NSTREAM == 2 && is_stream) ? p.qw1 : p.qw0;
			cp_async16(&ring[(issued & (D - 1)) * 32], base + (size_t)R * p.N + col_off);
			++issued;
			if (++is_local == is_len) {
				is_local = 0;
				if (++is_stream == NSTREAM) {
					is_stream = 0;
					is_seg += KW;
					is_len = min(p.seg_steps, p.total_steps - is_seg * p.seg_steps);
				}
			}
		}
		cp_async_commit();
	};
#pragma unroll
	for (int i = 0; i < D - 1; ++i) issue();

	// ---- stage the x slice: [row][unit of 8 k] in k order 0,4,1,5,2,6,3,7 -----------
	{
		const int units = (step_hi - step_lo) * 4;
		for (int idx = tid; idx < ROWS * units; idx += NT) {
			const int row = idx / units, unit = idx - row * units;
			const int k = (step_lo * 4 + unit) * 8;
			uint4 v = make_uint4(0u, 0u, 0u, 0u);
			if (row < p.M) {
				const __half *xr = p.x + (size_t)row * p.ldx;
				if (p.perm == nullptr) {
					v = *reinterpret_cast<const uint4 *>(xr + k);
				} else {
					const int4 pa = *reinterpret_cast<const int4 *>(p.perm + k);
					const int4 pb = *reinterpret_cast<const int4 *>(p.perm + k + 4);
					const uint32_t h0 = __half_as_ushort(xr[pa.x]), h1 = __half_as_ushort(xr[pa.y]);
					const uint32_t h2 = __half_as_ushort(xr[pa.z]), h3 = __half_as_ushort(xr[pa.w]);
					const uint32_t h4 = __half_as_ushort(xr[pb.x]), h5 = __half_as_ushort(xr[pb.y]);
					const uint32_t h6 = __half_as_ushort(xr[pb.z]), h7 = __half_as_ushort(xr[pb.w]);
					v = make_uint4(h0 | (h1 << 16), h2 | (h3 << 16), h4 | (h5 << 16), h6 | (h7 << 16));
				}
			}
			uint4 o;
			o.x = __byte_perm(v.x, v.z, 0x5410);    // (x0, x4)
			o.y = __byte_perm(v.x, v.z, 0x7632);    // (x1, x5)
			o.z = __byte_perm(v.y, v.w, 0x5410);    // (x2, x6)
			o.w = __byte_perm(v.y, v.w, 0x7632);    // (x3, x7)
			*reinterpret_cast<uint4 *>(xs + (size_t)row * p.xs_stride + unit * 16) = o;
		}
	}
	__syncthreads();

	// ---- main loop ---------------------------------------------------------------------
	float acc[NSTREAM][4][4];
#pragma unroll
	for (int s = 0; s < NSTREAM; ++s)
#pragma unroll
		for (int c = 0; c < 4; ++c)
#pragma unroll
			for (int e = 0; e < 4; ++e) acc[s][c][e] = 0.f;

	if (warp_active) {
		const unsigned char *xa_base = xs + (size_t)gid * p.xs_stride + (size_t)tig * 16;
		const int zcol = (n0w >> 3) + (gid >> 1);
		const int zsh = (gid & 1) * 16;
		const int nz = p.N >> 3;
		int consumed = 0;
		for (int seg = seg0 + kw; seg < seg1; seg += KW) {
			const int len = min(p.seg_steps, p.total_steps - seg * p.seg_steps);
			const int g = (seg * p.seg_steps * 32) / p.groupsize;
#pragma unroll
			for (int s = 0; s < NSTREAM; ++s) {
				const int32_t *qz = (NSTREAM == 2 && s) ? p.qz1 : p.qz0;
				const __half *sc = (NSTREAM == 2 && s) ? p.sc1 : p.sc0;
				const uint32_t zw = ((uint32_t)__ldg(qz + (size_t)g * nz + zcol)) >> zsh;
				const uint4 sraw = __ldg(reinterpret_cast<const uint4 *>(sc + (size_t)g * p.N + n0w + 8 * tig));
				uint32_t ZE[4], ZO[4];
#pragma unroll
				for (int c = 0; c < 4; ++c) {
					const uint32_t zz = ((zw >> (4 * c)) & 0xFu) + 1u;
					ZE[c] = (0x6400u + zz) * 0x00010001u;            // half2(1024 + zz)
					ZO[c] = (0xD400u + (zz << 4)) * 0x00010001u;     // half2(-(64 + zz))
				}
				float gacc[4][4];
#pragma unroll
				for (int c = 0; c < 4; ++c)
#pragma unroll
					for (int e = 0; e < 4; ++e) gacc[c][e] = 0.f;

				const unsigned char *xa_ptr = xa_base + (size_t)((seg * p.seg_steps - step_lo) * 4) * 16;
				for (int l = 0; l < len; ++l) {
					cp_async_wait<D - 2>();
					const uint4 q = ring[(consumed & (D - 1)) * 32];
					issue();
					++consumed;
					const uint4 xa = *reinterpret_cast<const uint4 *>(xa_ptr);
					uint4 xb = make_uint4(0u, 0u, 0u, 0u);
					if (!M8) xb = *reinterpret_cast<const uint4 *>(xa_ptr + (size_t)8 * p.xs_stride);
					xa_ptr += 64;
					const uint32_t qv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
					for (int c = 0; c < 4; ++c) {
						const uint32_t w = qv[c], w8 = w >> 8;
						const uint32_t b0 = h2_sub(lop3_and_or(w, MASK_LO, MAGIC_1024), ZE[c]);
						const uint32_t b1 = h2_fma(lop3_and_or(w, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[c]);
						const uint32_t b2 = h2_sub(lop3_and_or(w8, MASK_LO, MAGIC_1024), ZE[c]);
						const uint32_t b3 = h2_fma(lop3_and_or(w8, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[c]);
						mma16816(gacc[c], xa.x, xb.x, xa.y, xb.y, b0, b1);
						mma16816(gacc[c], xa.z, xb.z, xa.w, xb.w, b2, b3);
					}
				}
				// scale the segment's integer dot products: columns n0w + 8*tig + {c, 4+c}
				const __half2 *sh = reinterpret_cast<const __half2 *>(&sraw);
				const float2 s01 = __half22float2(sh[0]), s23 = __half22float2(sh[1]);
				const float2 s45 = __half22float2(sh[2]), s67 = __half22float2(sh[3]);
				const float slo[4] = {s01.x, s01.y, s23.x, s23.y};
				const float shi[4] = {s45.x, s45.y, s67.x, s67.y};
#pragma unroll
				for (int c = 0; c < 4; ++c) {
					acc[s][c][0] = fmaf(slo[c], gacc[c][0], acc[s][c][0]);
					acc[s][c][1] = fmaf(shi[c], gacc[c][1], acc[s][c][1]);
					acc[s][c][2] = fmaf(slo[c], gacc[c][2], acc[s][c][2]);
					acc[s][c][3] = fmaf(shi[c], gacc[c][3], acc[s][c][3]);
				}
			}
		}
	}
	cp_async_wait<0>();
	__syncthreads();            // every warp is done with its ring: the region becomes `red`

	// ---- reduce the KW warp-rows ---------------------------------------------------------
	// red[kw][stream][row][128]
#pragma unroll
	for (int s = 0; s < NSTREAM; ++s) {
		float *r = red + ((size_t)(kw * NSTREAM + s) * ROWS + gid) * SK_BN + wn * 32 + 8 * tig;
		*reinterpret_cast<float4 *>(r) = make_float4(acc[s][0][0], acc[s][1][0], acc[s][2][0], acc[s][3][0]);
		*reinterpret_cast<float4 *>(r + 4) = make_float4(acc[s][0][1], acc[s][1][1], acc[s][2][1], acc[s][3][1]);
		if (!M8) {
			r += 8 * SK_BN;
			*reinterpret_cast<float4 *>(r) = make_float4(acc[s][0][2], acc[s][1][2], acc[s][2][2], acc[s][3][2]);
			*reinterpret_cast<float4 *>(r + 4) = make_float4(acc[s][0][3], acc[s][1][3], acc[s][2][3], acc[s][3][3]);
		}
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
