// extern "C" entry points of libgptq_b200.so: argument checks, kernel selection, launches.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "qmm_skinny.cuh"
#include "qmm_tc.cuh"

namespace gptq {

thread_local int g_last_cuda_error = 0;

static int g_force_splitk = 0;   // test / tuning hook, 0 = automatic

static int sm_count() {
	static int cached[64] = {0};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
	if (cached[dev] == 0) {
		int n = 0;
		if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
		cached[dev] = n;
	}
	return cached[dev];
}

// ---- small utility kernels ----------------------------------------------------------------
__global__ void unpack_qweight_kernel(const uint32_t *__restrict__ qw, uint8_t *__restrict__ out, int R, int N) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)R * N) return;
	const int r = (int)(i / N), n = (int)(i % N);
	const uint32_t q = qw[i];
#pragma unroll
	for (int j = 0; j < 8; ++j) out[((size_t)r * 8 + j) * N + n] = (uint8_t)((q >> (4 * j)) & 0xFu);
}

__global__ void unpack_qzeros_kernel(const uint32_t *__restrict__ qz, uint8_t *__restrict__ out, size_t words) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= words) return;
	const uint32_t q = qz[i];
	uint2 v;
	v.x = (q & 0xFu) | ((q & 0xF0u) << 4) | ((q & 0xF00u) << 8) | ((q & 0xF000u) << 12);
	const uint32_t h = q >> 16;
	v.y = (h & 0xFu) | ((h & 0xF0u) << 4) | ((h & 0xF00u) << 8) | ((h & 0xF000u) << 12);
	reinterpret_cast<uint2 *>(out)[i] = v;
}

__global__ void dequantize_kernel(const uint32_t *__restrict__ qw, const uint32_t *__restrict__ qz,
								  const __half *__restrict__ sc, const int32_t *__restrict__ g_idx,
								  __half *__restrict__ out, int R, int N, int groupsize) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)R * N) return;
	const int r = (int)(i / N), n = (int)(i % N);
	const uint32_t q = qw[i];
#pragma unroll
	for (int j = 0; j < 8; ++j) {
		const int k = r * 8 + j;
		const int g = g_idx ? g_idx[k] : k / groupsize;
		const int zz = (int)((qz[(size_t)g * (N >> 3) + (n >> 3)] >> ((n & 7) * 4)) & 0xFu) + 1;
		const float w = (float)((int)((q >> (4 * j)) & 0xFu) - zz) * __half2float(sc[(size_t)g * N + n]);
		out[(size_t)k * N + n] = __float2half_rn(w);
	}
}

// sorted packed row j, nibble i  <-  original row perm[8j+i]
__global__ void act_order_rows_kernel(const uint32_t *__restrict__ qw, const int32_t *__restrict__ perm,
									  uint32_t *__restrict__ out, int R, int N) {
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)R * N) return;
	const int r = (int)(i / N), n = (int)(i % N);
	uint32_t o = 0;
#pragma unroll
	for (int j = 0; j < 8; ++j) {
		const int k = perm[r * 8 + j];
		const uint32_t q = qw[(size_t)(k >> 3) * N + n];
		o |= ((q >> (4 * (k & 7))) & 0xFu) << (4 * j);
	}
	out[i] = o;
}

// ---- skinny-kernel planning ---------------------------------------------------------------
constexpr int SK_KW = 4;
constexpr int SK_MAX_SPLITK = 16;
constexpr int SK_SMEM_LIMIT = 227 * 1024;

static bool skinny_shape_ok(int K, int N, int groupsize, const int32_t *g_idx) {
	return g_idx == nullptr && N % 32 == 0 && groupsize % 32 == 0 && K % groupsize == 0 && (N / SK_BN + 1) * 4 <= SK_TICKET_BYTES;
}

static size_t skinny_ws_bytes(int M, int N, int nstream) {
	const size_t tiles = (size_t)(N + SK_BN - 1) / SK_BN;
	return SK_TICKET_BYTES + tiles * SK_MAX_SPLITK * nstream * (size_t)std::min(M, 16) * SK_BN * sizeof(float);
}

static void plan_skinny(SkinnyParams &p, int nstream, dim3 &grid, size_t &smem) {
	const int rows = p.M <= 8 ? 8 : 16;
	p.total_steps = p.K / 32;
	const int spg = p.groupsize / 32;
	int seg_steps;
	if (p.groupsize == p.K) {
		seg_steps = std::min(8, p.total_steps);
	} else {
		seg_steps = spg;
		while (seg_steps > 16 && seg_steps % 2 == 0) seg_steps /= 2;
	}
	p.seg_steps = seg_steps;
	p.total_segs = (p.total_steps + seg_steps - 1) / seg_steps;
	const int tiles = (p.N + SK_BN - 1) / SK_BN;
	const int ring = SK_KW * 4 * SK_D * 32 * 16;
	const int xbudget = SK_SMEM_LIMIT - ring - 2048;
	const int ks_max = ((xbudget / rows) - 64) / 2;
	const int segs_max = std::max(1, (ks_max / 32) / seg_steps);
	const int min_split = (p.total_segs + segs_max - 1) / segs_max;
	const int sms = sm_count();
	int best = -1;
	double best_cost = 0;
	for (int sk = min_split; sk <= std::max(min_split, std::min(p.total_segs, SK_MAX_SPLITK)); ++sk) {
		const int sps = (p.total_segs + sk - 1) / sk;
		const int eff = (p.total_segs + sps - 1) / sps;
		const int waves = (tiles * eff + sms - 1) / sms;
		const double per_cta = (double)((sps + SK_KW - 1) / SK_KW) * seg_steps * nstream + 12.0 + 1.5 * eff;
		const double cost = waves * per_cta;
		if (best < 0 || cost < best_cost) {
			best = sk;
			best_cost = cost;
		}
	}
	if (g_force_splitk > 0) best = std::max(min_split, std::min(g_force_splitk, p.total_segs));
	p.segs_per_split = (p.total_segs + best - 1) / best;
	p.splitk = (p.total_segs + p.segs_per_split - 1) / p.segs_per_split;
	const int ks = p.segs_per_split * seg_steps * 32;
	p.xs_stride = ks * 2 + (((ks * 2) % 128 == 0) ? 64 : 0);
	p.xs_bytes = (rows * p.xs_stride + 127) / 128 * 128;
	grid = dim3(tiles, p.splitk, 1);
	smem = (size_t)p.xs_bytes + ring;
}

template <int NSTREAM, int EPI>
static int launch_skinny(SkinnyParams &p, void *workspace, size_t ws_bytes, cudaStream_t stream) {
	dim3 grid;
	size_t smem;
	plan_skinny(p, NSTREAM, grid, smem);
	const size_t need = skinny_ws_bytes(p.M, p.N, NSTREAM);
	if (p.splitk > 1 && (workspace == nullptr || ws_bytes < need)) return GPTQ_ERR_WORKSPACE;
	p.ws_ticket = reinterpret_cast<int *>(workspace);
	p.ws_partial = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + SK_TICKET_BYTES);
	cudaError_t e;
	if (p.M <= 8) {
		auto k = skinny_kernel<SK_KW, NSTREAM, true, EPI>;
		e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
		if (e != cudaSuccess) return cuda_status(e);
		k<<<grid, SK_KW * 128, smem, stream>>>(p);
	} else {
		auto k = skinny_kernel<SK_KW, NSTREAM, false, EPI>;
		e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
		if (e != cudaSuccess) return cuda_status(e);
		k<<<grid, SK_KW * 128, smem, stream>>>(p);
	}
	return cuda_status(cudaGetLastError());
}

static int check_common(const void *x, const void *qw, const void *qz, const void *sc, const void *y, int M, int K, int N,
						int &groupsize, long long ldx, long long ldy) {
	if (!x || !qw || !qz || !sc || !y) return GPTQ_ERR_INVALID;
	if (M < 0 || K <= 0 || N <= 0) return GPTQ_ERR_INVALID;
	if (groupsize == -1) groupsize = K;
	if (groupsize <= 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0 || N % 8 != 0) return GPTQ_ERR_SHAPE;
	if (ldx < K || ldy < N) return GPTQ_ERR_INVALID;
	if (ldx % 8 != 0 || ldy % 8 != 0) return GPTQ_ERR_ALIGN;
	if (!aligned16(x) || !aligned16(qw) || !aligned16(qz) || !aligned16(sc) || !aligned16(y)) return GPTQ_ERR_ALIGN;
	return GPTQ_OK;
}

}   // namespace gptq

using namespace gptq;

extern "C" {

int gptq_version(void) { return 100; }

const char *gptq_error_string(int code) {
	switch (code) {
		case GPTQ_OK: return "ok";
		case GPTQ_ERR_INVALID: return "invalid argument (null pointer, non-positive size or bad leading dimension)";
		case GPTQ_ERR_SHAPE: return "shape not supported: K and N must be multiples of 8";
		case GPTQ_ERR_WORKSPACE: return "workspace missing or smaller than gptq_workspace_bytes()";
		case GPTQ_ERR_ALIGN: return "pointers must be 16-byte aligned and leading dimensions multiples of 8";
		case GPTQ_ERR_CUDA: return "CUDA runtime error at launch (see gptq_last_cuda_error)";
		case GPTQ_ERR_UNSUPPORTED: return "combination not implemented";
		default: return "unknown error code";
	}
}

int gptq_last_cuda_error(void) { return g_last_cuda_error; }

// Tuning / test hook: force the split-K factor of the decode kernel (0 restores the heuristic).
void gptq_debug_force_splitk(int splitk) { g_force_splitk = splitk; }

size_t gptq_workspace_bytes(int M, int K, int N) {
	(void)K;
	if (M <= 0 || N <= 0) return SK_TICKET_BYTES;
	return std::max(skinny_ws_bytes(M, N, 2), tc_ws_bytes(M, N));
}

int gptq_qmatmul(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
				 const int32_t *perm, const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N,
				 int groupsize, int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	int rc = check_common(x, qweight, qzeros, scales, y, M, K, N, groupsize, ldx, ldy);
	if (rc != GPTQ_OK) return rc;
	if (g_idx && perm) return GPTQ_ERR_INVALID;
	if (residual && ldr < N) return GPTQ_ERR_INVALID;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	const bool fast = skinny_shape_ok(K, N, groupsize, g_idx) && (!perm || aligned16(perm));
	if (fast && M <= 16) {
		SkinnyParams p = {};
		p.x = (const __half *)x; p.ldx = ldx;
		p.qw0 = qweight; p.qz0 = qzeros; p.sc0 = (const __half *)scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.bias = (const __half *)bias; p.residual = (const __half *)residual; p.ldr = ldr;
		p.y = (__half *)y; p.ldy = ldy;
		return launch_skinny<1, EPI_PLAIN>(p, workspace, workspace_bytes, st);
	}
	if (fast && tc_shape_ok(M, K, N, groupsize)) {
		TcArgs a = {};
		a.x = (const __half *)x; a.ldx = ldx; a.qw0 = qweight; a.qz0 = qzeros; a.sc0 = (const __half *)scales;
		a.perm = perm; a.M = M; a.K = K; a.N = N; a.groupsize = groupsize;
		a.bias = (const __half *)bias; a.residual = (const __half *)residual; a.ldr = ldr;
		a.y = (__half *)y; a.ldy = ldy;
		return tc_launch(a, TC_EPI_PLAIN, workspace, workspace_bytes, st);
	}
	dim3 grid((N + 127) / 128, (M + 7) / 8);
	general_kernel<1><<<grid, 128, 0, st>>>((const __half *)x, ldx, qweight, qzeros, (const __half *)scales, nullptr, nullptr,
										  nullptr, g_idx, perm, (const __half *)bias, (const __half *)residual, ldr,
										  (__half *)y, ldy, M, K, N, groupsize);
	return cuda_status(cudaGetLastError());
}

int gptq_gateup_silu(const void *x, const int32_t *gate_qweight, const int32_t *gate_qzeros, const void *gate_scales,
					 const int32_t *up_qweight, const int32_t *up_qzeros, const void *up_scales, const int32_t *g_idx,
					 const int32_t *perm, void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
					 void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	int rc = check_common(x, gate_qweight, gate_qzeros, gate_scales, y, M, K, N, groupsize, ldx, ldy);
	if (rc != GPTQ_OK) return rc;
	if (!up_qweight || !up_qzeros || !up_scales) return GPTQ_ERR_INVALID;
	if (!aligned16(up_qweight) || !aligned16(up_qzeros) || !aligned16(up_scales)) return GPTQ_ERR_ALIGN;
	if (g_idx && perm) return GPTQ_ERR_INVALID;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	const bool fast = skinny_shape_ok(K, N, groupsize, g_idx) && (!perm || aligned16(perm));
	if (fast && M <= 16) {
		SkinnyParams p = {};
		p.x = (const __half *)x; p.ldx = ldx;
		p.qw0 = gate_qweight; p.qz0 = gate_qzeros; p.sc0 = (const __half *)gate_scales;
		p.qw1 = up_qweight; p.qz1 = up_qzeros; p.sc1 = (const __half *)up_scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.y = (__half *)y; p.ldy = ldy;
		return launch_skinny<2, EPI_SILU>(p, workspace, workspace_bytes, st);
	}
	if (fast && tc_shape_ok(M, K, N, groupsize)) {
		TcArgs a = {};
		a.x = (const __half *)x; a.ldx = ldx;
		a.qw0 = gate_qweight; a.qz0 = gate_qzeros; a.sc0 = (const __half *)gate_scales;
		a.qw1 = up_qweight; a.qz1 = up_qzeros; a.sc1 = (const __half *)up_scales;
		a.perm = perm; a.M = M; a.K = K; a.N = N; a.groupsize = groupsize;
		a.y = (__half *)y; a.ldy = ldy;
		return tc_launch(a, TC_EPI_SILU, workspace, workspace_bytes, st);
	}
	dim3 grid((N + 127) / 128, (M + 7) / 8);
	general_kernel<2><<<grid, 128, 0, st>>>((const __half *)x, ldx, gate_qweight, gate_qzeros, (const __half *)gate_scales,
										  up_qweight, up_qzeros, (const __half *)up_scales, g_idx, perm, nullptr, nullptr, 0,
										  (__half *)y, ldy, M, K, N, groupsize);
	return cuda_status(cudaGetLastError());
}

int gptq_qkv_rope(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
				  const int32_t *perm, const void *cos, const void *sin, const int32_t *position_ids, void *q_out,
				  int64_t q_stride_m, void *k_out, void *v_out, int tokens_per_batch, int64_t kv_stride_b,
				  int64_t kv_stride_t, int64_t kv_stride_h, int64_t kv_stride_pos, int M, int K, int n_heads, int head_dim,
				  int groupsize, int64_t ldx, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	if (!x || !qweight || !qzeros || !scales || !cos || !sin || !position_ids || !q_out || !k_out || !v_out)
		return GPTQ_ERR_INVALID;
	if (M < 0 || K <= 0 || n_heads <= 0 || tokens_per_batch <= 0) return GPTQ_ERR_INVALID;
	if (head_dim != 128) return GPTQ_ERR_UNSUPPORTED;
	if (groupsize == -1) groupsize = K;
	if (groupsize <= 0) return GPTQ_ERR_INVALID;
	const int hidden = n_heads * head_dim, N = 3 * hidden;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	if (ldx < K) return GPTQ_ERR_INVALID;
	if (ldx % 8 != 0) return GPTQ_ERR_ALIGN;
	if (!aligned16(x) || !aligned16(qweight) || !aligned16(qzeros) || !aligned16(scales)) return GPTQ_ERR_ALIGN;
	if (g_idx) return GPTQ_ERR_UNSUPPORTED;       // act-order must be prepared with gptq_act_order_rows (perm)
	if (!skinny_shape_ok(K, N, groupsize, nullptr) || (perm && !aligned16(perm))) return GPTQ_ERR_UNSUPPORTED;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	if (M <= 16) {
		SkinnyParams p = {};
		p.x = (const __half *)x; p.ldx = ldx;
		p.qw0 = qweight; p.qz0 = qzeros; p.sc0 = (const __half *)scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.cos_t = (const __half *)cos; p.sin_t = (const __half *)sin; p.pos = position_ids;
		p.q_out = (__half *)q_out; p.k_out = (__half *)k_out; p.v_out = (__half *)v_out;
		p.q_stride_m = q_stride_m; p.kv_sb = kv_stride_b; p.kv_st = kv_stride_t; p.kv_sh = kv_stride_h;
		p.kv_sp = kv_stride_pos; p.tokens_per_batch = tokens_per_batch; p.hidden = hidden;
		return launch_skinny<1, EPI_ROPE>(p, workspace, workspace_bytes, st);
	}
	if (tc_shape_ok(M, K, N, groupsize)) {
		TcArgs a = {};
		a.x = (const __half *)x; a.ldx = ldx; a.qw0 = qweight; a.qz0 = qzeros; a.sc0 = (const __half *)scales;
		a.perm = perm; a.M = M; a.K = K; a.N = N; a.groupsize = groupsize;
		a.cos_t = (const __half *)cos; a.sin_t = (const __half *)sin; a.pos = position_ids;
		a.q_out = (__half *)q_out; a.k_out = (__half *)k_out; a.v_out = (__half *)v_out;
		a.q_stride_m = q_stride_m; a.kv_sb = kv_stride_b; a.kv_st = kv_stride_t; a.kv_sh = kv_stride_h;
		a.kv_sp = kv_stride_pos; a.tokens_per_batch = tokens_per_batch; a.hidden = hidden;
		return tc_launch(a, TC_EPI_ROPE, workspace, workspace_bytes, st);
	}
	return GPTQ_ERR_UNSUPPORTED;
}

int gptq_unpack_qweight(const int32_t *qweight, uint8_t *out, int K, int N, gptq_stream_t stream) {
	if (!qweight || !out || K < 0 || N < 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	const size_t words = (size_t)(K / 8) * N;
	if (words == 0) return GPTQ_OK;
	unpack_qweight_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
		(const uint32_t *)qweight, out, K / 8, N);
	return cuda_status(cudaGetLastError());
}

int gptq_unpack_qzeros(const int32_t *qzeros, uint8_t *out, int G, int N, gptq_stream_t stream) {
	if (!qzeros || !out || G < 0 || N < 0) return GPTQ_ERR_INVALID;
	if (N % 8 != 0) return GPTQ_ERR_SHAPE;
	if ((reinterpret_cast<uintptr_t>(out) & 7u) != 0) return GPTQ_ERR_ALIGN;
	const size_t words = (size_t)G * (N / 8);
	if (words == 0) return GPTQ_OK;
	unpack_qzeros_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
		(const uint32_t *)qzeros, out, words);
	return cuda_status(cudaGetLastError());
}

int gptq_dequantize(const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx, void *w_out,
					int K, int N, int groupsize, gptq_stream_t stream) {
	if (!qweight || !qzeros || !scales || !w_out || K <= 0 || N <= 0) return GPTQ_ERR_INVALID;
	if (groupsize == -1) groupsize = K;
	if (groupsize <= 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0 || N % 8 != 0) return GPTQ_ERR_SHAPE;
	const size_t words = (size_t)(K / 8) * N;
	dequantize_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
		(const uint32_t *)qweight, (const uint32_t *)qzeros, (const __half *)scales, g_idx, (__half *)w_out, K / 8, N,
		groupsize);
	return cuda_status(cudaGetLastError());
}

int gptq_act_order_rows(const int32_t *qweight, const int32_t *perm, int32_t *out, int K, int N, gptq_stream_t stream) {
	if (!qweight || !perm || !out || K <= 0 || N <= 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	const size_t words = (size_t)(K / 8) * N;
	act_order_rows_kernel<<<(unsigned)((words + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
		(const uint32_t *)qweight, perm, (uint32_t *)out, K / 8, N);
	return cuda_status(cudaGetLastError());
}

}   // extern "C"
