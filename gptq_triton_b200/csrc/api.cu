// extern "C" entry points of libgptq_b200.so: argument checks, kernel selection, launches.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <utility>

#include <cuda.h>

#include "common.cuh"
#include "attn_decode.cuh"
#include "qkv_attn.cuh"
#include "qmm_skinny.cuh"
#include "qmm_tc.cuh"

namespace gptq {

thread_local int g_last_cuda_error = 0;

static int g_force_splitk = 0;   // test / tuning hook, 0 = automatic
static int g_max_stages2 = 3;    // the same for the two-stream (gate/up) form (gptq_debug_max_stages2): 3 stages 598, 4 stages 593, 2 stages 593 tokens/s on the 7B step
static int g_max_stages = 4;     // tuning hook: upper bound of the ring depth of the decode kernel
static int g_soft_max_splits = 8;  // the planner avoids more splits than this (gptq_debug_soft_max_splits)
static int g_qa_stages = 2;       // ring depth of the attention-block kernel (gptq_debug_qa_stages); 7B step, gate/up at 3 stages: 4 / 3 / 2 stages 589 / 596 / 600 tokens/s at 2.1 k context, 453 / 457 / 457 at 8 k, 660 / 676 / 681 at 300
static int g_pdl = 1;             // programmatic dependent launch for the decode-step kernels (+3 % on the decode step)

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

// Launch with optional programmatic stream serialisation (the kernel may start while its
// predecessor drains; it calls pdl_wait() before touching dependent data).
template <typename... KArgs, typename... Args>
static int launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid;
	cfg.blockDim = block;
	cfg.dynamicSmemBytes = smem;
	cfg.stream = stream;
	cudaLaunchAttribute attr[2];
	int n = 0;
	if (g_pdl) {
		attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
		attr[n].val.programmaticStreamSerializationAllowed = 1;
		++n;
	}
	cfg.attrs = attr;
	cfg.numAttrs = n;
	return cuda_status(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
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
constexpr int SK_MAX_SPLITK = 16;
constexpr int SK_SMEM_LIMIT = 227 * 1024;

static bool skinny_shape_ok(int K, int N, int groupsize, const int32_t *g_idx) {
	const bool gs_ok = groupsize == 32 || groupsize == 64 || groupsize % 128 == 0;
	return g_idx == nullptr && N % 32 == 0 && K % 128 == 0 && gs_ok && K % groupsize == 0 &&
		   (N / SK_BN + 2) * 4 <= SK_TICKET_BYTES - 4;
}

// scratch for x[:, perm] of an act-order decode call, placed behind the partial sums
static size_t gather_offset(size_t base) { return (base + 255) & ~(size_t)255; }
static size_t gather_bytes(int M, int K) { return (size_t)std::min(M, 16) * (size_t)K * sizeof(__half); }
// Workspace of a decode call: [counters | fp32 partial sums][8-byte words of the ticket-free exchange, M <= 8][gathered x]
static size_t words_offset(size_t base) { return (base + 255) & ~(size_t)255; }
static size_t words_bytes(int M, size_t base) { return M <= 8 ? 2 * (base - SK_TICKET_BYTES) : 0; }

static size_t skinny_ws_bytes(int M, int N, int nstream) {
	const size_t tiles = (size_t)(N + SK_BN - 1) / SK_BN;
	return SK_TICKET_BYTES + tiles * SK_MAX_SPLITK * nstream * (size_t)std::min(M, 16) * SK_BN * sizeof(float);
}

EncodeTiledFn tensor_map_encoder() {
	static EncodeTiledFn fn = nullptr;
	static std::once_flag once;
	std::call_once(once, [] {
		void *ptr = nullptr;
		cudaDriverEntryPointQueryResult q;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
			q == cudaDriverEntryPointSuccess)
			fn = reinterpret_cast<EncodeTiledFn>(ptr);
	});
	return fn;
}

// Tensor map over packed weights int32 [K/8, N] with a box of 32 columns x 16 packed rows,
// written to shared memory with the 128-byte swizzle.
static int weight_tensor_map(const int32_t *qw, int K, int N, CUtensorMap *out) {
	EncodeTiledFn enc = tensor_map_encoder();
	if (!enc) return GPTQ_ERR_CUDA;
	cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 8)};
	cuuint64_t strides[1] = {(cuuint64_t)N * 4};
	cuuint32_t box[2] = {32, 16};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(qw), dims, strides, box, estr,
					 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
					 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		g_last_cuda_error = (int)r;
		return GPTQ_ERR_CUDA;
	}
	return GPTQ_OK;
}

// Chooses the split-K factor and the shared-memory layout.  The aim is one wave of
// co-resident CTAs that covers (nearly) all SM slots with equal K-slices: the kernel is
// HBM-bound, so what counts is bytes in flight across the whole chip and no tail wave.
static void plan_skinny(SkinnyParams &p, int nstream, int &kw, dim3 &grid, size_t &smem) {
	p.spg = p.groupsize / 32;
	p.total_chunks = p.K / 128;
	const int tiles = (p.N + SK_BN - 1) / SK_BN;
	const int sms = sm_count();
	auto layout = [&](int sk, int kwarps, int nstage, int &cps, int &eff, int &xs_stride, int &xs_bytes, int &strip_groups) -> size_t {
		cps = (p.total_chunks + sk - 1) / sk;
		eff = (p.total_chunks + cps - 1) / cps;
		const int ks = cps * 128;
		xs_stride = ks * 2 + 16;      // = 16 mod 128: rows gid, gid+1 read disjoint banks
		xs_bytes = (p.M * xs_stride + 127) / 128 * 128;
		strip_groups = (ks + p.groupsize - 1) / p.groupsize + 1;
		const size_t strips = (size_t)nstream * strip_groups * SK_BN * 2 * 2 + (size_t)strip_groups * 16 * 8;
		const size_t ring = (size_t)kwarps * 4 * nstage * SK_CHUNK_BYTES;
		return ring + SK_BAR_BYTES + (size_t)xs_bytes + strips;
	};
	int best_sk = -1, best_kw = 2, best_stage = 4;
	double best_score = -1e30;
	for (int kwarps = 2; kwarps <= (p.spg < 4 ? 2 : 4); kwarps += 2) {
		const int per_sm = 4 / kwarps;
		const size_t cap = kwarps == 2 ? (size_t)113 * 1024 : (size_t)SK_SMEM_LIMIT - 2048;
		const int slots = sms * per_sm;
		for (int sk = 1; sk <= std::min(p.total_chunks, SK_MAX_SPLITK); ++sk) {
			int cps, eff, a, b, c;
			int nstage = nstream == 2 ? g_max_stages2 : g_max_stages;
			while (nstage > 2 && layout(sk, kwarps, nstage, cps, eff, a, b, c) > cap) --nstage;
			if (layout(sk, kwarps, nstage, cps, eff, a, b, c) > cap) continue;
			if (eff != sk) continue;
			const int ctas = tiles * eff;
			const int waves = (ctas + slots - 1) / slots;
			// fraction of the chip's slots kept busy, a strong preference for a single wave,
			// a mild one for fewer splits (less reduction traffic) and deep rings
			double score = (double)ctas / ((double)waves * slots);
			score -= 0.35 * (waves - 1);
			score -= 0.004 * eff;
			score -= 0.02 * std::max(0, 4 - nstage);
			if (cps < kwarps) score -= 0.25;
			if (kwarps == 4) score -= 0.03;
			if (eff > g_soft_max_splits) score -= 0.15;      // measured (7B down_proj, 11008 -> 4096): 8 splits 9.6 us, 9 splits 10.9 us
			if (score > best_score) {
				best_score = score;
				best_sk = sk;
				best_kw = kwarps;
				best_stage = nstage;
			}
		}
	}
	if (g_force_splitk > 0) {
		best_sk = std::min(g_force_splitk, p.total_chunks);
		best_kw = 2;
		best_stage = 4;
		int cps, eff, a, b, c;
		const size_t cap = best_kw == 2 ? (size_t)113 * 1024 : (size_t)SK_SMEM_LIMIT - 2048;
		while (best_stage > 2 && layout(best_sk, best_kw, best_stage, cps, eff, a, b, c) > cap) --best_stage;
	}
	if (best_sk < 0) { best_sk = std::min(p.total_chunks, SK_MAX_SPLITK); best_kw = 4; best_stage = 2; }
	int cps, eff;
	smem = layout(best_sk, best_kw, best_stage, cps, eff, p.xs_stride, p.xs_bytes, p.strip_groups);
	p.chunks_per_split = cps;
	p.splitk = eff;
	p.pdl = g_pdl;
	p.nstage = best_stage;
	kw = best_kw;
	grid = dim3(tiles, p.splitk, 1);
}

// Narrow geometry (one 32-column strip and the whole of K per CTA, no split-K): worth it when
// N / 32 CTAs fill most of the chip in one wave and the x rows of the whole K fit in shared memory.
static int g_allow_narrow = 0;      // opt-in (gptq_debug_allow_narrow): measured slower than the tiled split-K form
static bool plan_narrow(SkinnyParams &p, dim3 &grid, size_t &smem) {
	if (!g_allow_narrow || g_force_splitk > 0) return false;
	if (p.groupsize % 128 != 0 || p.N % 32 != 0) return false;
	const int strips32 = p.N / 32, sms = sm_count();
	if (strips32 * 10 < sms * 6 || strips32 > 2 * sms) return false;
	p.spg = p.groupsize / 32;
	p.total_chunks = p.K / 128;
	const int xs_stride = p.K * 2 + 16;
	const int xs_bytes = (p.M * xs_stride + 127) / 128 * 128;
	const int strip_groups = p.K / p.groupsize + 1;
	const size_t strips = (size_t)strip_groups * 32 * 2 * 2 + (size_t)strip_groups * 16 * 8;
	const size_t cap = strips32 > sms ? (size_t)113 * 1024 : (size_t)SK_SMEM_LIMIT - 2048;      // two CTAs per SM when there are more strips than SMs
	int nstage = 4;
	auto total = [&](int st) { return (size_t)8 * st * SK_CHUNK_BYTES + SK_BAR_BYTES + (size_t)xs_bytes + strips; };
	while (nstage > 2 && total(nstage) > cap) --nstage;
	if (total(nstage) > cap) return false;
	p.xs_stride = xs_stride;
	p.xs_bytes = xs_bytes;
	p.strip_groups = strip_groups;
	p.chunks_per_split = p.total_chunks;
	p.splitk = 1;
	p.pdl = g_pdl;
	p.nstage = nstage;
	smem = total(nstage);
	grid = dim3(strips32, 1, 1);
	return true;
}

// Opt the kernel in to the full dynamic shared memory once per device.
template <typename Kern>
static int ensure_smem_attr(Kern k, bool (&ready)[64]) {
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
	if (!ready[dev]) {
		cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_LIMIT - 1024);
		if (e != cudaSuccess) return cuda_status(e);
		ready[dev] = true;
	}
	return GPTQ_OK;
}

template <int KW, int NSTREAM, bool M8, int SPG_T, int EPI>
static int launch_skinny_inst(const CUtensorMap &tm0, const CUtensorMap &tm1, const SkinnyParams &p, dim3 grid, size_t smem,
							  cudaStream_t stream) {
	auto k = skinny_kernel<KW, NSTREAM, M8, SPG_T, EPI>;
	static bool ready[64] = {false};
	if (int rc = ensure_smem_attr(k, ready)) return rc;
	return launch_ex(k, grid, dim3(KW == 8 ? 256 : KW * 128, 1, 1), smem, stream, tm0, tm1, p);
}

// the narrow kernel exists for the plain epilogue with one weight stream only
template <int NSTREAM, int EPI>
static int launch_narrow(const CUtensorMap &tm0, const CUtensorMap &tm1, const SkinnyParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
	if constexpr (NSTREAM == 1 && EPI == EPI_PLAIN) {
		return p.M <= 8 ? launch_skinny_inst<8, 1, true, 0, EPI_PLAIN>(tm0, tm1, p, grid, smem, stream)
						: launch_skinny_inst<8, 1, false, 0, EPI_PLAIN>(tm0, tm1, p, grid, smem, stream);
	} else {
		return GPTQ_ERR_UNSUPPORTED;
	}
}

template <int NSTREAM, int EPI>
static int launch_skinny(SkinnyParams &p, const int32_t *qw0, const int32_t *qw1, void *workspace, size_t ws_bytes,
						 cudaStream_t stream, size_t gather_off = (size_t)-1) {
	dim3 grid;
	size_t smem;
	int kw;
	const bool narrow = (EPI == EPI_PLAIN && NSTREAM == 1) && p.ar_world <= 1 && plan_narrow(p, grid, smem);
	if (!narrow) plan_skinny(p, NSTREAM, kw, grid, smem);
	if (smem > (size_t)SK_SMEM_LIMIT - 1024) return GPTQ_ERR_UNSUPPORTED;
	const size_t need = skinny_ws_bytes(p.M, p.N, NSTREAM);
	if (workspace == nullptr || ws_bytes < need) return GPTQ_ERR_WORKSPACE;
	// ticket-free split-K exchange: M <= 8, one wave of co-resident CTAs (the polling CTA is the last one dispatched)
	if (gather_off == (size_t)-1 && !narrow && p.M <= 8 && p.splitk > 1 &&
		(int)(grid.x * grid.y) <= sm_count() * (kw == 2 ? 2 : 1) && ws_bytes >= words_offset(need) + words_bytes(p.M, need))
		p.ws_words = reinterpret_cast<unsigned long long *>(reinterpret_cast<unsigned char *>(workspace) + words_offset(need));
	if (p.perm) {
		// act-order: x[:, perm] once, into the workspace behind the partial sums (or at the offset the caller planned)
		const size_t off = (gather_off != (size_t)-1) ? gather_off : gather_offset(words_offset(need) + words_bytes(p.M, need));
		if (ws_bytes < off + gather_bytes(p.M, p.K)) return GPTQ_ERR_WORKSPACE;
		__half *xp = reinterpret_cast<__half *>(reinterpret_cast<unsigned char *>(workspace) + off);
		const dim3 gg((unsigned)((p.K / 8 + 255) / 256), (unsigned)p.M, 1);
		if (int rc = launch_ex(gather_x_kernel, gg, dim3(256, 1, 1), 0, stream, p.x, p.ldx, p.perm, xp, p.K)) return rc;
		p.x = xp;
		p.ldx = p.K;
		p.perm = nullptr;
	}
	p.ws_ticket = reinterpret_cast<int *>(workspace);
	p.ws_partial = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + SK_TICKET_BYTES);
	alignas(64) CUtensorMap tm0, tm1;
	if (int rc = weight_tensor_map(qw0, p.K, p.N, &tm0)) return rc;
	if (NSTREAM == 2) {
		if (int rc = weight_tensor_map(qw1, p.K, p.N, &tm1)) return rc;
	} else {
		tm1 = tm0;
	}
	const bool m8 = p.M <= 8;
	if (narrow) return launch_narrow<NSTREAM, EPI>(tm0, tm1, p, grid, smem, stream);
	if (p.spg == 1) {
		return m8 ? launch_skinny_inst<2, NSTREAM, true, 1, EPI>(tm0, tm1, p, grid, smem, stream)
				  : launch_skinny_inst<2, NSTREAM, false, 1, EPI>(tm0, tm1, p, grid, smem, stream);
	}
	if (p.spg == 2) {
		return m8 ? launch_skinny_inst<2, NSTREAM, true, 2, EPI>(tm0, tm1, p, grid, smem, stream)
				  : launch_skinny_inst<2, NSTREAM, false, 2, EPI>(tm0, tm1, p, grid, smem, stream);
	}
	if (kw == 2) {
		return m8 ? launch_skinny_inst<2, NSTREAM, true, 0, EPI>(tm0, tm1, p, grid, smem, stream)
				  : launch_skinny_inst<2, NSTREAM, false, 0, EPI>(tm0, tm1, p, grid, smem, stream);
	}
	return m8 ? launch_skinny_inst<4, NSTREAM, true, 0, EPI>(tm0, tm1, p, grid, smem, stream)
			  : launch_skinny_inst<4, NSTREAM, false, 0, EPI>(tm0, tm1, p, grid, smem, stream);
}

// Folded RMSNorm (consumer side): decode kernel only, x read in order, at most 256 partial sums per row.
static int check_rms(const void *rms_weight, const float *sumsq_in, int sumsq_tiles, float eps, int M, const int32_t *g_idx,
					 const int32_t *perm) {
	if (!rms_weight) return (sumsq_in == nullptr) ? GPTQ_OK : GPTQ_ERR_INVALID;
	if (!sumsq_in || sumsq_tiles <= 0 || !(eps >= 0.f)) return GPTQ_ERR_INVALID;
	if (!aligned16(rms_weight)) return GPTQ_ERR_ALIGN;
	if (M > 16 || g_idx || perm || sumsq_tiles > 256) return GPTQ_ERR_UNSUPPORTED;
	return GPTQ_OK;
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

// ---- scratch for the allocation-free entry point -------------------------------------------
// Lives in the library image; one copy per GPU that loads the library.  In host code the name
// is only a handle: the device address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[GPTQ_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch_ptr(void **out) {
	static void *cached[64] = {nullptr};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
	if (cached[dev] == nullptr) {
		void *ptr = nullptr;
		cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
		if (e != cudaSuccess || ptr == nullptr) return cuda_status(e == cudaSuccess ? cudaErrorInvalidSymbol : e);
		cached[dev] = ptr;
	}
	*out = cached[dev];
	return GPTQ_OK;
}

// bytes of the array a planned launch touches: counters + [tile][split][row < M][128] fp32
static size_t noalloc_need(const SkinnyParams &p) {
	const size_t tiles = (size_t)(p.N + SK_BN - 1) / SK_BN;
	return SK_TICKET_BYTES + tiles * p.splitk * (size_t)p.M * SK_BN * sizeof(float);
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
		case GPTQ_ERR_WORKSPACE: return "workspace missing or smaller than gptq_workspace_bytes(), or the problem needs more than the built-in scratch of gptq_qmatmul_noalloc";
		case GPTQ_ERR_ALIGN: return "pointers must be 16-byte aligned and leading dimensions multiples of 8";
		case GPTQ_ERR_CUDA: return "CUDA runtime error at launch (see gptq_last_cuda_error)";
		case GPTQ_ERR_UNSUPPORTED: return "combination not implemented";
		default: return "unknown error code";
	}
}

int gptq_last_cuda_error(void) { return g_last_cuda_error; }

// Tuning / test hook: force the split-K factor of the decode kernel (0 restores the heuristic).
void gptq_debug_force_splitk(int splitk) { g_force_splitk = splitk; }
void gptq_debug_max_stages(int n) { g_max_stages = std::max(2, std::min(n, 8)); }
void gptq_debug_max_stages2(int n) { g_max_stages2 = std::max(2, std::min(n, 8)); }
void gptq_debug_set_pdl(int on) { g_pdl = on ? 1 : 0; }
void gptq_debug_qa_stages(int n) { g_qa_stages = n; }
void gptq_debug_soft_max_splits(int n) { g_soft_max_splits = n; }
void gptq_debug_allow_narrow(int on) { g_allow_narrow = on ? 1 : 0; }
size_t gptq_workspace_bytes(int M, int K, int N) {
	if (M <= 0 || N <= 0) return SK_TICKET_BYTES;
	const size_t base = skinny_ws_bytes(M, N, 2);
	return std::max(gather_offset(words_offset(base) + words_bytes(M, base)) + gather_bytes(M, std::max(K, 0)), tc_ws_bytes(M, N));
}

struct ArArgs {
	int world, rank;
	void *const *partials;
	void *const *flags;
};

static int qmatmul_impl(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
						const int32_t *perm, const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N,
						int groupsize, int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes, gptq_stream_t stream,
						float *sumsq_out, const ArArgs *ar = nullptr) {
	int rc = check_common(x, qweight, qzeros, scales, y, M, K, N, groupsize, ldx, ldy);
	if (rc != GPTQ_OK) return rc;
	if (g_idx && perm) return GPTQ_ERR_INVALID;
	if (residual && ldr < N) return GPTQ_ERR_INVALID;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	const bool fast = skinny_shape_ok(K, N, groupsize, g_idx) && (!perm || aligned16(perm));
	// the per-tile sums of squares exist in the decode kernel only (whole 128-column tiles)
	if (sumsq_out && !(fast && M <= 16 && N % 128 == 0)) return GPTQ_ERR_UNSUPPORTED;
	if (ar) {
		// the fused all-reduce lives in the decode kernel's epilogue
		if (ar->world < 2 || ar->world > 8 || ar->rank < 0 || ar->rank >= ar->world || !ar->partials || !ar->flags) return GPTQ_ERR_INVALID;
		if (!(fast && M <= 16 && N % 128 == 0)) return GPTQ_ERR_UNSUPPORTED;
		for (int r = 0; r < ar->world; ++r)
			if (!ar->partials[r] || !ar->flags[r] || !aligned16(ar->partials[r])) return GPTQ_ERR_INVALID;
	}
	if (fast && M <= 16) {
		SkinnyParams p = {};
		p.x = (const __half *)x; p.ldx = ldx;
		p.qz0 = qzeros; p.sc0 = (const __half *)scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.bias = (const __half *)bias; p.residual = (const __half *)residual; p.ldr = ldr;
		p.y = (__half *)y; p.ldy = ldy;
		p.ss_out = sumsq_out;
		if (ar) {
			p.ar_world = ar->world;
			p.ar_rank = ar->rank;
			for (int r = 0; r < ar->world; ++r) p.ar_buf[r] = reinterpret_cast<unsigned long long *>(ar->partials[r]);
			p.ar_seq = reinterpret_cast<unsigned *>(ar->flags[ar->rank]);
		}
		return launch_skinny<1, EPI_PLAIN>(p, qweight, nullptr, workspace, workspace_bytes, st);
	}
	if (fast && !perm && tc_shape_ok(M, K, N, groupsize)) {
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

int gptq_qmatmul(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
				 const int32_t *perm, const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N,
				 int groupsize, int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	return qmatmul_impl(x, qweight, qzeros, scales, g_idx, perm, bias, residual, ldr, y, M, K, N, groupsize, ldx, ldy, workspace,
						workspace_bytes, stream, nullptr);
}

// ---- tensor parallelism: row-parallel projection with the all-reduce in its epilogue ----------------------
size_t gptq_ar_partial_bytes(int N) { return N <= 0 ? 0 : (size_t)2 * 8 * ((N + SK_BN - 1) / SK_BN) * 16 * SK_BN * sizeof(unsigned long long); }
size_t gptq_ar_flag_bytes(int N) { return N <= 0 ? 0 : (((size_t)((N + SK_BN - 1) / SK_BN) * sizeof(unsigned)) + 255) & ~(size_t)255; }

int gptq_qmatmul_ar(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
					const int32_t *perm, const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N,
					int groupsize, int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes, gptq_stream_t stream,
					float *sumsq_out, int world, int rank, void *const *partials, void *const *flags) {
	ArArgs ar = {world, rank, partials, flags};
	return qmatmul_impl(x, qweight, qzeros, scales, g_idx, perm, bias, residual, ldr, y, M, K, N, groupsize, ldx, ldy, workspace,
						workspace_bytes, stream, sumsq_out, &ar);
}

int gptq_qmatmul_sumsq(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
					   const int32_t *perm, const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N,
					   int groupsize, int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes, gptq_stream_t stream,
					   float *sumsq_out) {
	if (!sumsq_out) return GPTQ_ERR_INVALID;
	return qmatmul_impl(x, qweight, qzeros, scales, g_idx, perm, bias, residual, ldr, y, M, K, N, groupsize, ldx, ldy, workspace,
						workspace_bytes, stream, sumsq_out);
}

size_t gptq_attn_workspace_bytes(int batch, int heads) {
	if (batch <= 0 || heads <= 0) return AT_TICKET_BYTES;
	return AT_TICKET_BYTES + (size_t)batch * heads * AT_MAX_SPLITS * 130 * sizeof(float);
}

int gptq_attn_decode(const void *q, int64_t q_stride_b, const void *kcache, const void *vcache, int64_t kv_stride_b,
					 int64_t kv_stride_h, const int32_t *pos, void *out, int64_t out_stride_b, int batch, int heads, int head_dim,
					 int len_hint, float scale, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	if (!q || !kcache || !vcache || !pos || !out) return GPTQ_ERR_INVALID;
	if (batch < 0 || heads <= 0 || len_hint <= 0) return GPTQ_ERR_INVALID;
	if (head_dim != AT_D) return GPTQ_ERR_UNSUPPORTED;
	if (!aligned16(q) || !aligned16(kcache) || !aligned16(vcache) || q_stride_b % 8 || kv_stride_b % 8 || kv_stride_h % 8)
		return GPTQ_ERR_ALIGN;
	if (batch == 0) return GPTQ_OK;
	if ((size_t)batch * heads * 4 > (size_t)AT_TICKET_BYTES - 8) return GPTQ_ERR_UNSUPPORTED;
	// two CTAs (96 KB of staged cache rows each) fit an SM: one wave of at most 2 * SMs CTAs
	int splits = std::max(1, 2 * sm_count() / (batch * heads));
	splits = std::max(1, std::min(splits, std::min(AT_MAX_SPLITS, (len_hint + 63) / 64)));
	if (splits > 1 && (!workspace || workspace_bytes < gptq_attn_workspace_bytes(batch, heads))) return GPTQ_ERR_WORKSPACE;
	AttnParams p = {};
	p.q = (const __half *)q; p.q_stride_b = q_stride_b;
	p.kc = (const __half *)kcache; p.vc = (const __half *)vcache;
	p.kv_stride_b = kv_stride_b; p.kv_stride_h = kv_stride_h;
	p.pos = pos; p.out = (__half *)out; p.out_stride_b = out_stride_b;
	p.scale = scale; p.heads = heads; p.splits = splits;
	p.ws_ticket = reinterpret_cast<int *>(workspace);
	p.ws_partial = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + AT_TICKET_BYTES);
	{
		static bool ready[64] = {false};
		int dev = 0;
		if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
		if (!ready[dev]) {
			cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
			if (e != cudaSuccess) return cuda_status(e);
			ready[dev] = true;
		}
	}
	return launch_ex(attn_decode_kernel, dim3(splits, heads, batch), dim3(AT_THREADS, 1, 1), AT_SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream), p);
}

// Shared-memory layout of qkv_attn_kernel for nc chunks of 128 K-rows per CTA; returns the total.
static size_t qkv_attn_layout(QkvAttnParams &p) {
	size_t o = (size_t)8 * p.nstage * QA_SLOT;
	p.off_bars = (int)o; o += 8 * 8 * 8;
	p.off_xs = (int)o; o += (size_t)p.nc * 256;
	p.off_zz = (int)o; o += (size_t)p.nc * QA_COLS * 2;
	p.off_sc = (int)o; o += (size_t)p.nc * QA_COLS * 2;
	p.off_part = (int)o; o += (size_t)p.nc * QA_COLS * 4;
	p.off_gather = (int)o; o += (size_t)QA_CLUSTER * QA_COLS * 4;
	p.off_merge = (int)o; o += (size_t)QA_CLUSTER * 130 * 4;
	o = (o + 15) & ~(size_t)15;
	p.off_attn = (int)o; o += QA_D * 4 + 2 * QA_D * 2 + 8 * QA_D * 4 + 64;
	p.off_o = (int)o;
	if (p.o_enable) o += 8 * 256 + 2 * 256 * 4 * 2;      // staged attention output (one copy per warp), zero / scale strips of up to 1024 o_proj columns
	return o;
}

int gptq_qkv_attn_supported(int K, int n_heads, int head_dim, int groupsize) {
	if (groupsize == -1) groupsize = K;
	if (K <= 0 || n_heads <= 0 || groupsize <= 0 || head_dim != QA_D) return 0;
	if (K % (QA_CLUSTER * 128) != 0 || K / (QA_CLUSTER * 128) > QA_MAX_NC) return 0;
	if (groupsize % 128 != 0 || K % groupsize != 0) return 0;
	return 1;
}

size_t gptq_qkv_attn_oproj_scratch_bytes(int n_heads, int N) {
	if (n_heads <= 0 || N <= 0) return 0;
	return 256 + (size_t)n_heads * N * sizeof(float);
}

// o: optional fused output projection
struct QaOproj {
	const int32_t *qweight, *qzeros;
	const void *scales, *residual;
	void *y;
	float *sumsq_out;
	int N, groupsize;
	void *scratch;
	size_t scratch_bytes;
	int ar_world, ar_rank;          // > 1: o_proj is this rank's row shard, the all-reduce runs inside the kernel
	void *const *ar_partials;
	void *const *ar_flags;
};

static int qkv_attn_impl(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const void *cos, const void *sin,
						 const int32_t *pos, int max_pos, void *kcache, void *vcache, int64_t kv_stride_h, void *out, int K, int n_heads,
						 int head_dim, int groupsize, float scale, const void *rms_weight, const float *sumsq_in, int sumsq_tiles, float rms_eps,
						 void *workspace, size_t workspace_bytes, gptq_stream_t stream, const QaOproj *o) {
	if (!x || !qweight || !qzeros || !scales || !cos || !sin || !pos || !kcache || !vcache || (!out && !o)) return GPTQ_ERR_INVALID;
	if (max_pos <= 0 || kv_stride_h < (int64_t)max_pos * QA_D) return GPTQ_ERR_INVALID;
	if (groupsize == -1) groupsize = K;
	if (!gptq_qkv_attn_supported(K, n_heads, head_dim, groupsize)) return GPTQ_ERR_UNSUPPORTED;
	if (!aligned16(x) || !aligned16(qweight) || !aligned16(qzeros) || !aligned16(scales) || !aligned16(kcache) || !aligned16(vcache) ||
		(out && !aligned16(out)) || kv_stride_h % 8)
		return GPTQ_ERR_ALIGN;
	if (rms_weight && (!sumsq_in || sumsq_tiles <= 0 || !aligned16(rms_weight))) return GPTQ_ERR_INVALID;
	if (!workspace || workspace_bytes < (size_t)SK_TICKET_BYTES) return GPTQ_ERR_WORKSPACE;
	QkvAttnParams p = {};
	p.x = (const __half *)x; p.qz = qzeros; p.sc = (const __half *)scales;
	p.K = K; p.N = 3 * n_heads * QA_D; p.sec_stride = n_heads * QA_D; p.groupsize = groupsize;
	p.nc = K / (QA_CLUSTER * 128); p.nstage = std::max(2, std::min(4, g_qa_stages));
	p.rms_w = (const __half *)rms_weight; p.ss_in = sumsq_in; p.ss_tiles = sumsq_tiles; p.rms_eps = rms_eps;
	p.cos_t = (const __half *)cos; p.sin_t = (const __half *)sin; p.pos = pos; p.max_pos = max_pos;
	p.kc = (__half *)kcache; p.vc = (__half *)vcache; p.kv_stride_h = kv_stride_h;
	p.scale = scale; p.out = (__half *)out;
	p.status = reinterpret_cast<int *>(workspace) + SK_STATUS_SLOT;
	CUtensorMap tm, tmo;
	if (int rc = weight_tensor_map(qweight, K, p.N, &tm)) return rc;
	tmo = tm;
	if (o) {
		int ogs = o->groupsize == -1 ? n_heads * QA_D : o->groupsize;
		if (!o->qweight || !o->qzeros || !o->scales || !o->y || !o->scratch) return GPTQ_ERR_INVALID;
		if (o->N <= 0 || o->N % 32 != 0 || o->N > 8192 || ogs <= 0 || ogs % 128 != 0 || (n_heads * QA_D) % ogs != 0) return GPTQ_ERR_UNSUPPORTED;
		if (!aligned16(o->qweight) || !aligned16(o->qzeros) || !aligned16(o->scales) || !aligned16(o->y) || !aligned16(o->scratch) ||
			(o->residual && !aligned16(o->residual)))
			return GPTQ_ERR_ALIGN;
		if (o->scratch_bytes < gptq_qkv_attn_oproj_scratch_bytes(n_heads, o->N)) return GPTQ_ERR_WORKSPACE;
		p.o_enable = 1; p.o_N = o->N; p.o_groupsize = ogs;
		p.o_spw = (o->N / 32 + QA_CLUSTER * 8 - 1) / (QA_CLUSTER * 8);
		if (p.o_spw == 3) p.o_spw = 4;          // the reduction divides 256 threads by 64 spw column quads
		if (p.o_spw > 4) return GPTQ_ERR_UNSUPPORTED;
		p.o_qz = o->qzeros; p.o_sc = (const __half *)o->scales; p.o_res = (const __half *)o->residual;
		p.o_tickets = reinterpret_cast<int *>(o->scratch);
		p.o_part = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(o->scratch) + 256);
		p.o_y = (__half *)o->y; p.o_ss = o->sumsq_out;
		if (o->ar_world > 1) {
			if (o->ar_world > 8 || o->ar_rank < 0 || o->ar_rank >= o->ar_world || !o->ar_partials || !o->ar_flags || o->N % 128 != 0) return GPTQ_ERR_INVALID;
			for (int r = 0; r < o->ar_world; ++r)
				if (!o->ar_partials[r] || !o->ar_flags[r] || !aligned16(o->ar_partials[r])) return GPTQ_ERR_INVALID;
			p.ar_world = o->ar_world; p.ar_rank = o->ar_rank; p.ar_tiles = o->N / 128;
			for (int r = 0; r < o->ar_world; ++r) p.ar_buf[r] = reinterpret_cast<unsigned long long *>(o->ar_partials[r]);
			p.ar_seq = reinterpret_cast<unsigned *>(o->ar_flags[o->ar_rank]);
		}
		if (int rc = weight_tensor_map(o->qweight, n_heads * QA_D, o->N, &tmo)) return rc;
	}
	const size_t smem = qkv_attn_layout(p);
	if (smem > (size_t)SK_SMEM_LIMIT - 2048) return GPTQ_ERR_UNSUPPORTED;
	{
		static bool ready[64] = {false};
		int dev = 0;
		if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
		if (!ready[dev]) {
			cudaError_t e = cudaFuncSetAttribute(qkv_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_LIMIT - 2048);      // the kernel has 1 KB of static shared memory
			if (e != cudaSuccess) return cuda_status(e);
			e = cudaFuncSetAttribute(qkv_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_LIMIT - 2048);
			if (e != cudaSuccess) return cuda_status(e);
			ready[dev] = true;
		}
	}
	if (p.ar_world > 1)
		return launch_ex(qkv_attn_kernel<true>, dim3(QA_CLUSTER, n_heads, 1), dim3(QA_THREADS, 1, 1), smem, reinterpret_cast<cudaStream_t>(stream), tm, tmo, p);
	return launch_ex(qkv_attn_kernel<false>, dim3(QA_CLUSTER, n_heads, 1), dim3(QA_THREADS, 1, 1), smem, reinterpret_cast<cudaStream_t>(stream), tm, tmo, p);
}

int gptq_qkv_attn_decode(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const void *cos, const void *sin,
						 const int32_t *pos, int max_pos, void *kcache, void *vcache, int64_t kv_stride_h, void *out, int K, int n_heads,
						 int head_dim, int groupsize, float scale, const void *rms_weight, const float *sumsq_in, int sumsq_tiles, float rms_eps,
						 void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	if (!out) return GPTQ_ERR_INVALID;
	return qkv_attn_impl(x, qweight, qzeros, scales, cos, sin, pos, max_pos, kcache, vcache, kv_stride_h, out, K, n_heads, head_dim, groupsize,
						 scale, rms_weight, sumsq_in, sumsq_tiles, rms_eps, workspace, workspace_bytes, stream, nullptr);
}

int gptq_qkv_attn_oproj_decode(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const void *cos,
							   const void *sin, const int32_t *pos, int max_pos, void *kcache, void *vcache, int64_t kv_stride_h, int K,
							   int n_heads, int head_dim, int groupsize, float scale, const void *rms_weight, const float *sumsq_in,
							   int sumsq_tiles, float rms_eps, const int32_t *o_qweight, const int32_t *o_qzeros, const void *o_scales,
							   int o_N, int o_groupsize, const void *residual, void *y, float *sumsq_out, void *attn_out, void *scratch,
							   size_t scratch_bytes, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	QaOproj o = {o_qweight, o_qzeros, o_scales, residual, y, sumsq_out, o_N, o_groupsize, scratch, scratch_bytes, 0, 0, nullptr, nullptr};
	return qkv_attn_impl(x, qweight, qzeros, scales, cos, sin, pos, max_pos, kcache, vcache, kv_stride_h, attn_out, K, n_heads, head_dim,
						 groupsize, scale, rms_weight, sumsq_in, sumsq_tiles, rms_eps, workspace, workspace_bytes, stream, &o);
}

int gptq_qkv_attn_oproj_decode_ar(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const void *cos,
								  const void *sin, const int32_t *pos, int max_pos, void *kcache, void *vcache, int64_t kv_stride_h, int K,
								  int n_heads, int head_dim, int groupsize, float scale, const void *rms_weight, const float *sumsq_in,
								  int sumsq_tiles, float rms_eps, const int32_t *o_qweight, const int32_t *o_qzeros, const void *o_scales,
								  int o_N, int o_groupsize, const void *residual, void *y, float *sumsq_out, void *attn_out, void *scratch,
								  size_t scratch_bytes, void *workspace, size_t workspace_bytes, gptq_stream_t stream, int world, int rank,
								  void *const *partials, void *const *flags) {
	if (world < 2) return GPTQ_ERR_INVALID;
	QaOproj o = {o_qweight, o_qzeros, o_scales, residual, y, sumsq_out, o_N, o_groupsize, scratch, scratch_bytes, world, rank, partials, flags};
	return qkv_attn_impl(x, qweight, qzeros, scales, cos, sin, pos, max_pos, kcache, vcache, kv_stride_h, attn_out, K, n_heads, head_dim,
						 groupsize, scale, rms_weight, sumsq_in, sumsq_tiles, rms_eps, workspace, workspace_bytes, stream, &o);
}

int gptq_rmsnorm(const void *x, int64_t ldx, const void *weight, void *y, int64_t ldy, int M, int K, float eps, gptq_stream_t stream) {
	if (!x || !weight || !y || M < 0 || K <= 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || ldx % 8 || ldy % 8) return GPTQ_ERR_ALIGN;
	if (M == 0) return GPTQ_OK;
	return launch_ex(rmsnorm_kernel, dim3(M, 1, 1), dim3(RN_THREADS, 1, 1), 0, reinterpret_cast<cudaStream_t>(stream), (const __half *)x, (long long)ldx,
					 (const __half *)weight, (__half *)y, (long long)ldy, K, eps, (const long long *)nullptr, (__half *)nullptr, 0ll);
}

int gptq_embed_rmsnorm(const void *table, int64_t ldt, int64_t n_rows, const int64_t *tok, const void *weight, void *h_out, int64_t ldh, void *y,
					   int64_t ldy, int M, int K, float eps, gptq_stream_t stream) {
	if (!table || !tok || !weight || !h_out || !y || M < 0 || K <= 0 || n_rows <= 0) return GPTQ_ERR_INVALID;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	if (!aligned16(table) || !aligned16(weight) || !aligned16(h_out) || !aligned16(y) || ldt % 8 || ldh % 8 || ldy % 8) return GPTQ_ERR_ALIGN;
	if (M == 0) return GPTQ_OK;
	(void)n_rows;          // the ids are on the device; the caller guarantees 0 <= tok[m] < n_rows
	return launch_ex(rmsnorm_kernel, dim3(M, 1, 1), dim3(RN_THREADS, 1, 1), 0, reinterpret_cast<cudaStream_t>(stream), (const __half *)table, (long long)ldt,
					 (const __half *)weight, (__half *)y, (long long)ldy, K, eps, (const long long *)tok, (__half *)h_out, (long long)ldh);
}

size_t gptq_noalloc_scratch_bytes(int M, int K, int N, int groupsize) {
	if (M <= 0 || M > 16 || K <= 0 || N <= 0) return 0;
	if (groupsize == -1) groupsize = K;
	if (groupsize <= 0 || !skinny_shape_ok(K, N, groupsize, nullptr)) return 0;
	SkinnyParams p = {};
	p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
	dim3 grid;
	size_t smem;
	int kw;
	plan_skinny(p, 1, kw, grid, smem);
	return gather_offset(noalloc_need(p)) + gather_bytes(M, K);      // with room for the act-order gather of x
}

int gptq_qmatmul_noalloc(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *perm,
						 const void *bias, const void *residual, int64_t ldr, void *y, int M, int K, int N, int groupsize,
						 int64_t ldx, int64_t ldy, gptq_stream_t stream) {
	int rc = check_common(x, qweight, qzeros, scales, y, M, K, N, groupsize, ldx, ldy);
	if (rc != GPTQ_OK) return rc;
	if (residual && ldr < N) return GPTQ_ERR_INVALID;
	if (M == 0) return GPTQ_OK;
	if (M > 16 || !skinny_shape_ok(K, N, groupsize, nullptr) || (perm && !aligned16(perm))) return GPTQ_ERR_UNSUPPORTED;
	if (gptq_noalloc_scratch_bytes(M, K, N, groupsize) > GPTQ_NOALLOC_SCRATCH_BYTES) return GPTQ_ERR_WORKSPACE;
	void *scratch = nullptr;
	rc = noalloc_scratch_ptr(&scratch);          // first call on a device: resolves the array's device address
	if (rc != GPTQ_OK) return rc;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	// the arrival counters must start at zero; partial sums need no clearing (every slot that is
	// read is written first by this launch)
	// (the last word of the counter area is the status word: it is kept, gptq_noalloc_status reads it)
	cudaError_t e = cudaMemsetAsync(scratch, 0, SK_TICKET_BYTES - 4, st);
	if (e != cudaSuccess) return cuda_status(e);
	SkinnyParams p = {};
	p.x = (const __half *)x; p.ldx = ldx;
	p.qz0 = qzeros; p.sc0 = (const __half *)scales;
	p.perm = perm;
	p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
	p.bias = (const __half *)bias; p.residual = (const __half *)residual; p.ldr = ldr;
	p.y = (__half *)y; p.ldy = ldy;
	// launch_skinny only checks that the buffer is at least as large as the generic upper bound;
	// the array was checked against the exact need above (partial sums of the planned split, then
	// the gathered x), so pass sizes that satisfy those checks and the planned offset of the gather
	dim3 grid;
	size_t smem;
	int kw;
	SkinnyParams plan = p;
	plan_skinny(plan, 1, kw, grid, smem);
	const size_t off = gather_offset(noalloc_need(plan));
	return launch_skinny<1, EPI_PLAIN>(p, qweight, nullptr, scratch, std::max(skinny_ws_bytes(M, N, 1), off + gather_bytes(M, K)), st, off);
}

int gptq_noalloc_status(int clear) {
	void *scratch = nullptr;
	if (noalloc_scratch_ptr(&scratch) != GPTQ_OK) return GPTQ_ERR_CUDA;
	int *word = reinterpret_cast<int *>(scratch) + SK_STATUS_SLOT;
	int status = 0;
	if (cudaDeviceSynchronize() != cudaSuccess) return GPTQ_ERR_CUDA;
	if (cudaMemcpy(&status, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return GPTQ_ERR_CUDA;
	if (clear && status != 0 && cudaMemset(word, 0, sizeof(int)) != cudaSuccess) return GPTQ_ERR_CUDA;
	return status;
}

static int gateup_impl(const void *x, const int32_t *gate_qweight, const int32_t *gate_qzeros, const void *gate_scales,
					   const int32_t *up_qweight, const int32_t *up_qzeros, const void *up_scales, const int32_t *g_idx,
					   const int32_t *perm, void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
					   void *workspace, size_t workspace_bytes, gptq_stream_t stream, const void *rms_weight,
					   const float *sumsq_in, int sumsq_tiles, float rms_eps) {
	int rc = check_common(x, gate_qweight, gate_qzeros, gate_scales, y, M, K, N, groupsize, ldx, ldy);
	if (rc != GPTQ_OK) return rc;
	if ((rc = check_rms(rms_weight, sumsq_in, sumsq_tiles, rms_eps, M, g_idx, perm)) != GPTQ_OK) return rc;
	if (!up_qweight || !up_qzeros || !up_scales) return GPTQ_ERR_INVALID;
	if (!aligned16(up_qweight) || !aligned16(up_qzeros) || !aligned16(up_scales)) return GPTQ_ERR_ALIGN;
	if (g_idx && perm) return GPTQ_ERR_INVALID;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	const bool fast = skinny_shape_ok(K, N, groupsize, g_idx) && (!perm || aligned16(perm));
	if (fast && M <= 16) {
		SkinnyParams p = {};
		p.x = (const __half *)x; p.ldx = ldx;
		p.qz0 = gate_qzeros; p.sc0 = (const __half *)gate_scales;
		p.qz1 = up_qzeros; p.sc1 = (const __half *)up_scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.y = (__half *)y; p.ldy = ldy;
		p.rms_w = (const __half *)rms_weight; p.ss_in = sumsq_in; p.ss_tiles = sumsq_tiles; p.rms_eps = rms_eps;
		return launch_skinny<2, EPI_SILU>(p, gate_qweight, up_qweight, workspace, workspace_bytes, st);
	}
	if (rms_weight) return GPTQ_ERR_UNSUPPORTED;
	if (fast && !perm && tc_shape_ok(M, K, N, groupsize)) {
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

int gptq_gateup_silu(const void *x, const int32_t *gate_qweight, const int32_t *gate_qzeros, const void *gate_scales,
					 const int32_t *up_qweight, const int32_t *up_qzeros, const void *up_scales, const int32_t *g_idx,
					 const int32_t *perm, void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
					 void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	return gateup_impl(x, gate_qweight, gate_qzeros, gate_scales, up_qweight, up_qzeros, up_scales, g_idx, perm, y, M, K, N,
					   groupsize, ldx, ldy, workspace, workspace_bytes, stream, nullptr, nullptr, 0, 0.f);
}

int gptq_gateup_silu_rms(const void *x, const int32_t *gate_qweight, const int32_t *gate_qzeros, const void *gate_scales,
						 const int32_t *up_qweight, const int32_t *up_qzeros, const void *up_scales, const int32_t *g_idx,
						 const int32_t *perm, void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
						 void *workspace, size_t workspace_bytes, gptq_stream_t stream, const void *rms_weight,
						 const float *sumsq_in, int sumsq_tiles, float rms_eps) {
	if (!rms_weight) return GPTQ_ERR_INVALID;
	return gateup_impl(x, gate_qweight, gate_qzeros, gate_scales, up_qweight, up_qzeros, up_scales, g_idx, perm, y, M, K, N,
					   groupsize, ldx, ldy, workspace, workspace_bytes, stream, rms_weight, sumsq_in, sumsq_tiles, rms_eps);
}

static int qkv_rope_impl(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
						 const int32_t *perm, const void *cos, const void *sin, const int32_t *position_ids, int max_pos, void *q_out,
						 int64_t q_stride_m, void *k_out, void *v_out, int tokens_per_batch, int64_t kv_stride_b,
						 int64_t kv_stride_t, int64_t kv_stride_h, int64_t kv_stride_pos, int M, int K, int n_heads, int head_dim,
						 int groupsize, int64_t ldx, void *workspace, size_t workspace_bytes, gptq_stream_t stream,
						 const void *rms_weight, const float *sumsq_in, int sumsq_tiles, float rms_eps) {
	if (!x || !qweight || !qzeros || !scales || !cos || !sin || !position_ids || !q_out || !k_out || !v_out)
		return GPTQ_ERR_INVALID;
	if (M < 0 || K <= 0 || n_heads <= 0 || tokens_per_batch <= 0 || max_pos <= 0) return GPTQ_ERR_INVALID;
	if (head_dim != 128) return GPTQ_ERR_UNSUPPORTED;
	if (groupsize == -1) groupsize = K;
	if (groupsize <= 0) return GPTQ_ERR_INVALID;
	const int hidden = n_heads * head_dim, N = 3 * hidden;
	if (K % 8 != 0) return GPTQ_ERR_SHAPE;
	if (ldx < K) return GPTQ_ERR_INVALID;
	if (ldx % 8 != 0) return GPTQ_ERR_ALIGN;
	if (!aligned16(x) || !aligned16(qweight) || !aligned16(qzeros) || !aligned16(scales)) return GPTQ_ERR_ALIGN;
	if (g_idx) return GPTQ_ERR_UNSUPPORTED;       // act-order must be prepared with gptq_act_order_rows (perm)
	if (perm && !aligned16(perm)) return GPTQ_ERR_UNSUPPORTED;
	if (M <= 16 && !skinny_shape_ok(K, N, groupsize, nullptr)) return GPTQ_ERR_UNSUPPORTED;
	if (int rc = check_rms(rms_weight, sumsq_in, sumsq_tiles, rms_eps, M, g_idx, perm)) return rc;
	if (M == 0) return GPTQ_OK;
	cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
	if (M <= 16) {
		SkinnyParams p = {};
		p.rms_w = (const __half *)rms_weight; p.ss_in = sumsq_in; p.ss_tiles = sumsq_tiles; p.rms_eps = rms_eps;
		p.x = (const __half *)x; p.ldx = ldx;
		p.qz0 = qzeros; p.sc0 = (const __half *)scales;
		p.perm = perm;
		p.M = M; p.K = K; p.N = N; p.groupsize = groupsize;
		p.cos_t = (const __half *)cos; p.sin_t = (const __half *)sin; p.pos = position_ids;
		p.q_out = (__half *)q_out; p.k_out = (__half *)k_out; p.v_out = (__half *)v_out;
		p.q_stride_m = q_stride_m; p.kv_sb = kv_stride_b; p.kv_st = kv_stride_t; p.kv_sh = kv_stride_h;
		p.kv_sp = kv_stride_pos; p.tokens_per_batch = tokens_per_batch; p.hidden = hidden; p.max_pos = max_pos;
		return launch_skinny<1, EPI_ROPE>(p, qweight, nullptr, workspace, workspace_bytes, st);
	}
	if (!perm && tc_shape_ok(M, K, N, groupsize)) {
		TcArgs a = {};
		a.x = (const __half *)x; a.ldx = ldx; a.qw0 = qweight; a.qz0 = qzeros; a.sc0 = (const __half *)scales;
		a.perm = perm; a.M = M; a.K = K; a.N = N; a.groupsize = groupsize;
		a.cos_t = (const __half *)cos; a.sin_t = (const __half *)sin; a.pos = position_ids;
		a.q_out = (__half *)q_out; a.k_out = (__half *)k_out; a.v_out = (__half *)v_out;
		a.q_stride_m = q_stride_m; a.kv_sb = kv_stride_b; a.kv_st = kv_stride_t; a.kv_sh = kv_stride_h;
		a.kv_sp = kv_stride_pos; a.tokens_per_batch = tokens_per_batch; a.hidden = hidden; a.max_pos = max_pos;
		return tc_launch(a, TC_EPI_ROPE, workspace, workspace_bytes, st);
	}
	return GPTQ_ERR_UNSUPPORTED;
}

int gptq_qkv_rope(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
				  const int32_t *perm, const void *cos, const void *sin, const int32_t *position_ids, int max_pos, void *q_out,
				  int64_t q_stride_m, void *k_out, void *v_out, int tokens_per_batch, int64_t kv_stride_b,
				  int64_t kv_stride_t, int64_t kv_stride_h, int64_t kv_stride_pos, int M, int K, int n_heads, int head_dim,
				  int groupsize, int64_t ldx, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	return qkv_rope_impl(x, qweight, qzeros, scales, g_idx, perm, cos, sin, position_ids, max_pos, q_out, q_stride_m, k_out, v_out,
						 tokens_per_batch, kv_stride_b, kv_stride_t, kv_stride_h, kv_stride_pos, M, K, n_heads, head_dim, groupsize,
						 ldx, workspace, workspace_bytes, stream, nullptr, nullptr, 0, 0.f);
}

int gptq_qkv_rope_rms(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
					  const int32_t *perm, const void *cos, const void *sin, const int32_t *position_ids, int max_pos, void *q_out,
					  int64_t q_stride_m, void *k_out, void *v_out, int tokens_per_batch, int64_t kv_stride_b,
					  int64_t kv_stride_t, int64_t kv_stride_h, int64_t kv_stride_pos, int M, int K, int n_heads, int head_dim,
					  int groupsize, int64_t ldx, void *workspace, size_t workspace_bytes, gptq_stream_t stream,
					  const void *rms_weight, const float *sumsq_in, int sumsq_tiles, float rms_eps) {
	if (!rms_weight) return GPTQ_ERR_INVALID;
	return qkv_rope_impl(x, qweight, qzeros, scales, g_idx, perm, cos, sin, position_ids, max_pos, q_out, q_stride_m, k_out, v_out,
						 tokens_per_batch, kv_stride_b, kv_stride_t, kv_stride_h, kv_stride_pos, M, K, n_heads, head_dim, groupsize,
						 ldx, workspace, workspace_bytes, stream, rms_weight, sumsq_in, sumsq_tiles, rms_eps);
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
