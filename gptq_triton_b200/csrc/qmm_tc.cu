// Prefill-regime (M > 16) quantised matmul on the 5th-generation tensor cores of sm_100a.
//
// Y[M,N] = X[M,K] · deq(W)[K,N] with fp16 operands and fp32 accumulation in tensor memory.
// One CTA computes a 128 or 256 (rows of X) x 128 or 256 (columns of W) tile; K advances in blocks
// of 64.  256-row tiles issue two M = 128 MMAs per K step against the same dequantised B stage.
//
//   warp 0      TMA producer: X tile [128 x 64] fp16, K-major, 128-byte swizzle (one thread)
//   warp 1      MMA issuer: tcgen05.mma.cta_group::1.kind::f16, M=128 N=128 K=16, four per
//               K-block (eight with the second weight stream), tcgen05.commit frees the stage;
//               the warp also owns the TMEM allocation
//   warps 2-17  dequantise, four groups of four warps, group j serving K-blocks j, j+4, ...: a
//               thread owns a weight column of the tile, reads the K-block's 8 packed words of that
//               column from a TMA-fed ring, turns each into 8 fp16 weights
//               (q - zero) * scale with ONE rounding — the fp16 weight of the
//               dequantise-then-matmul path — and stores them as one 16-byte unit of the
//               K-major, 128-byte-swizzled B tile; fence.proxy.async + mbarrier arrive.
//               After the last K-block the same warps drain TMEM (tcgen05.ld 32x32b) and run
//               the epilogue: bias/residual, SiLU(gate)*up, or rotary + scatter to Q/K/V.
//
// Every mbarrier wait is bounded; a wait that runs out sets a status word and the kernel
// unwinds (TMEM is still released).
#include <algorithm>

#include <cuda.h>

#include "qmm_tc.cuh"

namespace gptq {

namespace {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64, TC_STAGES = 4;
constexpr int TC_WORKERS = 512;                             // dequantise / epilogue threads: 4 groups x 4 warps
constexpr int TC_THREADS = 64 + TC_WORKERS;
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 2;            // 16 KB: one A or B stage
constexpr uint32_t TC_SPIN = 1u << 24;
// pipeline depth by tile configuration (shared memory: S * (MH * 16 KB + NSTREAM * BN * 128 B) + packed ring)
__host__ __device__ constexpr int tc_stages(int nstream, int bn, int mh) { return (mh == 2 && nstream * bn == 256) ? 3 : TC_STAGES; }
__host__ __device__ constexpr int tc_pstages(int nstream, int bn, int mh) { return (mh == 2) ? (nstream * bn == 256 ? 3 : 6) : (nstream * bn == 256 ? 4 : 8); }

// ---- tcgen05 / TMEM wrappers -------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
		:
		: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
		: "memory");
}
// arrive on an mbarrier once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i receives row (lane quarter base + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
	uint32_t *r = reinterpret_cast<uint32_t *>(v);
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
		"%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
		  "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
		  "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
		  "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
		: "r"(taddr)
		: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart (SBO), LBO unused (1), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
	uint64_t d = 0;
	d |= (uint64_t)((addr & 0x3FFFFu) >> 4);            // start address, bits [0,14)
	d |= (uint64_t)1 << 16;                             // leading byte offset (ignored for swizzled K-major)
	d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
	d |= (uint64_t)1 << 46;                             // version
	d |= (uint64_t)2 << 61;                             // layout type: SWIZZLE_128B
	return d;
}


struct TcParams {
	TcArgs a;
	int epi;
	int *status;
	int kb_per_split;            // K-blocks of 64 per CTA along grid.z (all of them without split-K)
	float *partial;              // split-K: [split][M][N] fp32 partial sums in the workspace, else nullptr
};

}   // namespace

// forward declaration of the kernel body (second half of this file)
template <int NSTREAM, int EPI, int BN, int MH>
__global__ void __launch_bounds__(TC_THREADS, 1) tc_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw0,
														   const __grid_constant__ CUtensorMap tmw1, const TcParams p);

}   // namespace gptq

#include "qmm_tc_kernel.inl"

// ---- host side -------------------------------------------------------------------------------
namespace gptq {

EncodeTiledFn tensor_map_encoder();      // defined in api.cu
int g_tc_force = 0;                    // tests: 0 = choose by cost, 1 = 128 x 128, 2 = 128 x 256, 3 = 256 x 256 (256 x 128 for two streams), 4 = 256 x 128
constexpr double TC_SPEED_256x128 = 1.6;
extern "C" void gptq_debug_tc_force(int cfg) { g_tc_force = cfg; }

bool tc_shape_ok(int M, int K, int N, int groupsize) {
	return M > 16 && N % TC_BN == 0 && K % TC_BK == 0 && groupsize % TC_BK == 0 && K % groupsize == 0;
}

// Workspace: the status word at the end of the first 16 KB; behind it room for the fp32 partial sums of a split-K
// launch (up to TC_MAX_SPLITK splits of M x N, at most TC_SPLIT_BYTES: larger problems fill the chip without it).
constexpr int TC_MAX_SPLITK = 4;
constexpr size_t TC_SPLIT_BYTES = (size_t)96 << 20;
size_t tc_ws_bytes(int M, int N) {
	const size_t part = (size_t)TC_MAX_SPLITK * (size_t)std::max(M, 0) * (size_t)std::max(N, 0) * 4;
	return 16384 + (M > 16 && part <= TC_SPLIT_BYTES ? part : 0);
}
int g_tc_splitk = 0;                   // tests: 0 = choose by cost, n = force n splits where the epilogue allows
extern "C" void gptq_debug_tc_splitk(int n) { g_tc_splitk = n; }

static int x_tensor_map(const __half *x, int M, int K, long long ldx, CUtensorMap *out) {
	EncodeTiledFn enc = tensor_map_encoder();
	if (!enc) return GPTQ_ERR_CUDA;
	cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
	cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
	cuuint32_t box[2] = {TC_BK, TC_BM};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
					 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		g_last_cuda_error = (int)r;
		return GPTQ_ERR_CUDA;
	}
	return GPTQ_OK;
}

// Tensor map over packed weights int32 [K/8, N]: box bn columns x 8 packed rows (one K-block), no swizzle.
static int w_tensor_map(const int32_t *qw, int K, int N, int bn, CUtensorMap *out) {
	EncodeTiledFn enc = tensor_map_encoder();
	if (!enc) return GPTQ_ERR_CUDA;
	cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 8)};
	cuuint64_t strides[1] = {(cuuint64_t)N * 4};
	cuuint32_t box[2] = {(cuuint32_t)bn, 8};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t *>(qw), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
					 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) {
		g_last_cuda_error = (int)r;
		return GPTQ_ERR_CUDA;
	}
	return GPTQ_OK;
}

template <int NSTREAM, int EPI, int BN, int MH>
static int tc_launch_inst(const CUtensorMap &tmx, const TcParams &p, cudaStream_t stream) {
	auto k = tc_kernel<NSTREAM, EPI, BN, MH>;
	constexpr int S = tc_stages(NSTREAM, BN, MH), PS = tc_pstages(NSTREAM, BN, MH);
	const size_t smem = (size_t)S * (MH * TC_TILE_BYTES + NSTREAM * BN * TC_BK * 2) + (size_t)PS * NSTREAM * 8 * BN * 4 + 512;
	static_assert((size_t)S * (MH * TC_TILE_BYTES + NSTREAM * BN * TC_BK * 2) + (size_t)PS * NSTREAM * 8 * BN * 4 + 512 <= 232448, "shared memory per CTA");
	alignas(64) CUtensorMap tmw0, tmw1;
	if (int rc = w_tensor_map(p.a.qw0, p.a.K, p.a.N, BN, &tmw0)) return rc;
	if (NSTREAM == 2) {
		if (int rc = w_tensor_map(p.a.qw1, p.a.K, p.a.N, BN, &tmw1)) return rc;
	} else {
		tmw1 = tmw0;
	}
	static bool ready[64] = {false};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
	if (!ready[dev]) {
		cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
		if (e != cudaSuccess) return cuda_status(e);
		ready[dev] = true;
	}
	const int nkb = p.a.K / TC_BK;
	const int splits = (nkb + p.kb_per_split - 1) / p.kb_per_split;
	dim3 grid(p.a.N / BN, (p.a.M + TC_BM * MH - 1) / (TC_BM * MH), splits);
	k<<<grid, TC_THREADS, smem, stream>>>(tmx, tmw0, tmw1, p);
	if (int rc = cuda_status(cudaGetLastError())) return rc;
	if (p.partial) {
		const size_t units = (size_t)p.a.M * (p.a.N / 8);
		tc_splitk_finish<<<(unsigned)((units + 255) / 256), 256, 0, stream>>>(p.partial, splits, p.a.M, p.a.N, p.a.bias, p.a.residual, p.a.ldr, p.a.y, p.a.ldy);
		return cuda_status(cudaGetLastError());
	}
	return GPTQ_OK;
}

int tc_launch(const TcArgs &a, int epi, void *workspace, size_t ws_bytes, cudaStream_t stream) {
	if (a.perm) return GPTQ_ERR_UNSUPPORTED;
	if (!workspace || ws_bytes < 16384) return GPTQ_ERR_WORKSPACE;
	if (a.ldx % 8 != 0) return GPTQ_ERR_ALIGN;
	alignas(64) CUtensorMap tmx;
	if (int rc = x_tensor_map(a.x, a.M, a.K, a.ldx, &tmx)) return rc;
	TcParams p;
	p.a = a;
	p.epi = epi;
	p.status = reinterpret_cast<int *>(workspace) + (16384 / 4 - 1);
	p.kb_per_split = a.K / TC_BK;
	p.partial = nullptr;
	// Tile choice: estimated time = waves * (rows * columns of a tile) / relative speed of the configuration
	// (measured per busy SM: 128 x 128 tiles 1.0, 128 x 256 tiles 1.7, 256-row tiles 2.5).
	int dev = 0, sms = 148;
	if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
	auto cost = [&](int bm, int bn, double speed) {
		if (a.N % bn != 0) return 1e30;
		const long long tiles = (long long)(a.N / bn) * ((a.M + bm - 1) / bm);
		const long long waves = (tiles + sms - 1) / sms;
		return (double)waves * bm * bn / speed;
	};
	if (epi == TC_EPI_SILU) {
		const bool tall = g_tc_force ? (g_tc_force >= 3) : (cost(256, 128, 1.5) < cost(128, 128, 1.0));
		return tall ? tc_launch_inst<2, TC_EPI_SILU, 128, 2>(tmx, p, stream) : tc_launch_inst<2, TC_EPI_SILU, 128, 1>(tmx, p, stream);
	}
	// configurations: 0 = 128 x 128, 1 = 128 x 256, 2 = 256 x 256, 3 = 256 x 128
	int pick = 0;
	if (epi == TC_EPI_PLAIN) {
		// Plain epilogue: tile configuration AND split-K by estimated time.  Measured on B200 (M = 512 and 1024,
		// N = 4096, K = 4096 and 11008): a CTA needs t_kb microseconds per K-block of 64 whatever the number of CTAs
		// (0.66 for 128 x 128 tiles, 0.73 for 128 x 256, 0.91 for 256 x 256, 0.82 for 256 x 128) plus about 2.5 us
		// to start and drain; split-K costs about 6 us (second launch, strided fp32 stores) plus the partial sums
		// written and read back at about 4 TB/s.  Short prompts with a long K gain most (M = 512, 11008 -> 4096:
		// 102 -> 62 us); M = 512, 4096 -> 4096 gains 10 %.
		const int bms[4] = {128, 128, 256, 256}, bns[4] = {128, 256, 256, 128};
		const double t_kbs[4] = {0.66, 0.73, 0.91, 0.82};
		const int nkb = a.K / TC_BK;
		const bool room = ws_bytes >= 16384 + (size_t)TC_MAX_SPLITK * a.M * a.N * 4 && (size_t)TC_MAX_SPLITK * a.M * a.N * 4 <= TC_SPLIT_BYTES;
		double best = 1e30;
		int best_sk = 1;
		for (int i = 0; i < 4; ++i) {
			if (a.N % bns[i] != 0) continue;
			if (g_tc_force && i != (((g_tc_force == 2 || g_tc_force == 3) && a.N % 256 != 0) ? 0 : g_tc_force - 1)) continue;
			const double t_kb = t_kbs[i];
			const long long tiles = (long long)(a.N / bns[i]) * ((a.M + bms[i] - 1) / bms[i]);
			for (int sk = 1; sk <= TC_MAX_SPLITK; sk *= 2) {
				if (sk > 1 && (!room || nkb < sk)) break;
				if (g_tc_splitk > 0) {
					if (sk != g_tc_splitk) continue;                 // forced by a test
				} else if (sk > 1 && nkb / sk < 8) {
					break;                                           // too few K-blocks per split to amortise the start / drain
				}
				const int kbps = (nkb + sk - 1) / sk;
				const long long waves = (tiles * ((nkb + kbps - 1) / kbps) + sms - 1) / sms;
				double t = (double)waves * (kbps * t_kb + 2.5);
				if (sk > 1) t += 6.0 + (double)sk * a.M * a.N * 8.0 / 4.0e6;
				if (t < best) {
					best = t;
					pick = i;
					best_sk = sk;
				}
			}
		}
		p.kb_per_split = (nkb + best_sk - 1) / best_sk;
		p.partial = best_sk > 1 ? reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + 16384) : nullptr;
	} else {
		const double c[4] = {cost(128, 128, 1.0), cost(128, 256, 1.7), cost(256, 256, 2.5), cost(256, 128, TC_SPEED_256x128)};
		for (int i = 1; i < 4; ++i)
			if (c[i] < c[pick]) pick = i;
		if (g_tc_force) pick = ((g_tc_force == 2 || g_tc_force == 3) && a.N % 256 != 0) ? 0 : g_tc_force - 1;
	}
	switch (epi) {
		case TC_EPI_PLAIN:
			return pick == 3 ? tc_launch_inst<1, TC_EPI_PLAIN, 128, 2>(tmx, p, stream)
				 : pick == 2 ? tc_launch_inst<1, TC_EPI_PLAIN, 256, 2>(tmx, p, stream)
				 : pick == 1 ? tc_launch_inst<1, TC_EPI_PLAIN, 256, 1>(tmx, p, stream) : tc_launch_inst<1, TC_EPI_PLAIN, 128, 1>(tmx, p, stream);
		case TC_EPI_ROPE:
			return pick == 3 ? tc_launch_inst<1, TC_EPI_ROPE, 128, 2>(tmx, p, stream)
				 : pick == 2 ? tc_launch_inst<1, TC_EPI_ROPE, 256, 2>(tmx, p, stream)
				 : pick == 1 ? tc_launch_inst<1, TC_EPI_ROPE, 256, 1>(tmx, p, stream) : tc_launch_inst<1, TC_EPI_ROPE, 128, 1>(tmx, p, stream);
	}
	return GPTQ_ERR_INVALID;
}

}   // namespace gptq
