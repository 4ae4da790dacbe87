// Host side of the persistent decode-step kernel and of the lm_head kernel: planning, descriptors, launches.
#include <algorithm>
#include <vector>

#include <cuda.h>

#include "common.cuh"
#include "decode_chain.cuh"
#include "qmm_tc.cuh"

namespace gptq {

EncodeTiledFn tensor_map_encoder();      // defined in api.cu

namespace {

constexpr size_t CH_CTRL_BYTES = 16384;              // [sync counters | ... | status word in the last 4 bytes]
constexpr size_t CH_SMEM_CAP = 113 * 1024 - 768;     // two CTAs per SM, static shared memory taken off

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int g_chain_max_stages = 6;          // tuning / test hook (gptq_debug_chain_stages): upper bound of the ring depth per warp

struct ChainLayout {
	ChainParams p;
	size_t smem;
	size_t scratch;
	int grid;
	size_t o_qkv, o_attn, o_o, o_gu, o_down, o_hA, o_hB, o_ssa, o_ssb;
};

int sm_count_now() {
	int dev = 0, n = 148;
	if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
	return n > 0 ? n : 148;
}

// Largest split-K factor <= limit that cuts total_chunks into equal-sized slices (the last may be shorter)
// such that every slice is non-empty.
void plan_projection(ChainPlan &pl, int K, int N, int nstream, int w0, int grid) {
	pl.K = K; pl.N = N; pl.nstream = nstream; pl.w0 = w0;
	pl.tiles = N / 128;
	pl.total_chunks = K / 128;
	const int limit = std::max(1, std::min({grid / std::max(pl.tiles, 1), pl.total_chunks, CH_MAX_SPLITS}));
	pl.splitk = 1;
	pl.cps = pl.total_chunks;
	for (int sk = limit; sk >= 1; --sk) {
		const int cps = (pl.total_chunks + sk - 1) / sk;
		if ((pl.total_chunks + cps - 1) / cps == sk) {
			pl.splitk = sk;
			pl.cps = cps;
			break;
		}
	}
}

// Shapes the chain kernel serves: batch rows <= 8, head_dim 128, one group size (a multiple of 128) that divides
// both K values, every dimension a multiple of 128 (hidden of 256: the lm_head kernel reads 16 bytes per lane).
bool chain_shape_ok(int M, int hidden, int inter, int heads, int groupsize) {
	if (M < 1 || M > CH_MAX_M || heads < 1 || hidden != heads * CH_D) return false;
	if (hidden % 256 != 0 || inter % 128 != 0) return false;
	if (groupsize <= 0 || groupsize % 128 != 0 || hidden % groupsize != 0 || inter % groupsize != 0) return false;
	return true;
}

// grid: CTAs of the launch (two per SM unless given).  Returns false when the shape cannot be laid out.
bool chain_layout(int M, int hidden, int inter, int heads, int groupsize, int grid, ChainLayout &L) {
	if (!chain_shape_ok(M, hidden, inter, heads, groupsize)) return false;
	ChainParams &p = L.p;
	p = ChainParams{};
	p.M = M; p.hidden = hidden; p.inter = inter; p.heads = heads; p.groupsize = groupsize; p.spg = groupsize / 32;
	L.grid = grid;
	if (M * heads > grid) return false;
	plan_projection(p.plan[CH_QKV], hidden, 3 * hidden, 1, CH_W_QKV, grid);
	plan_projection(p.plan[CH_O], hidden, hidden, 1, CH_W_O, grid);
	plan_projection(p.plan[CH_GU], hidden, inter, 2, CH_W_GATE, grid);
	plan_projection(p.plan[CH_DOWN], inter, hidden, 1, CH_W_DOWN, grid);
	p.attn_splits = std::max(1, std::min(grid / (M * heads), CH_MAX_SPLITS));
	int max_cps = 0;
	for (int k : {CH_QKV, CH_O, CH_GU, CH_DOWN}) {
		if (p.plan[k].tiles > grid) return false;          // every (tile, split) pair needs its own CTA
		max_cps = std::max(max_cps, p.plan[k].cps);
	}
	if (max_cps * 16 > CH_THREADS) return false;           // one 16-byte unit of the x slice per thread
	p.strip_groups = (max_cps * 128 + groupsize - 1) / groupsize + 1;
	if (p.strip_groups > 16) return false;                 // the strips are staged in two passes of one item per thread
	size_t xs = align_up((size_t)M * (max_cps * 256 + 16), 128);
	const size_t strips = (size_t)2 * p.strip_groups * 128 * 2;                 // two streams, fp16
	const size_t cs = (size_t)p.strip_groups * 16 * 8;
	const size_t red = (size_t)2 * 2 * M * 128 * 4;
	if (xs + 2 * strips + cs + red < 8192) xs = 8192 - (2 * strips + cs + red);      // the attention phase keeps 7 KB of its own from off_xs on
	xs = align_up(xs, 128);
	const size_t fixed = 512 + xs + 2 * strips + cs + red;
	int nst = std::max(2, std::min(6, g_chain_max_stages));
	while (nst >= 2 && (size_t)8 * nst * CH_SLOT + fixed > CH_SMEM_CAP) --nst;
	if (nst < 2) return false;
	p.nstage = nst;
	size_t off = (size_t)8 * nst * CH_SLOT;
	p.off_bars = (int)off; off += 512;
	p.off_xs = (int)off; off += xs;
	p.off_zz = (int)off; off += strips;
	p.off_sc = (int)off; off += strips;
	p.off_cs = (int)off; off += cs;
	p.off_red = (int)off; off += red;
	L.smem = off;
	// scratch in global memory
	size_t s = CH_CTRL_BYTES;
	auto take = [&](size_t bytes) { const size_t o = s; s = align_up(s + bytes, 256); return o; };
	L.o_qkv = take((size_t)p.plan[CH_QKV].splitk * M * 3 * hidden * 4);
	L.o_attn = take((size_t)M * heads * p.attn_splits * 130 * 4);
	L.o_o = take((size_t)p.plan[CH_O].splitk * M * hidden * 4);
	L.o_gu = take((size_t)p.plan[CH_GU].splitk * 2 * M * inter * 4);
	L.o_down = take((size_t)p.plan[CH_DOWN].splitk * M * hidden * 4);
	L.o_hA = take((size_t)M * hidden * 2);
	L.o_hB = take((size_t)M * hidden * 2);
	L.o_ssa = take((size_t)CH_MAX_SPLITS * M * 4);
	L.o_ssb = take((size_t)CH_MAX_SPLITS * M * 4);
	L.scratch = s;
	return true;
}

int encode_weight_map(const int32_t *qw, int K, int N, CUtensorMap *out) {
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

// CTAs of a chain launch on the current device: two per SM when the kernel fits twice, else what fits
int chain_grid(size_t smem) {
	int occ = 0;
	if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_chain_kernel, CH_THREADS, smem) != cudaSuccess) occ = 0;
	return std::min(occ, 2) * sm_count_now();
}

}   // namespace
}   // namespace gptq

using namespace gptq;

extern "C" {

void gptq_debug_chain_stages(int n) { g_chain_max_stages = n; }

size_t gptq_chain_desc_bytes(int n_layers) { return n_layers <= 0 ? 0 : (size_t)n_layers * sizeof(ChainLayer); }

int gptq_chain_supported(int M, int hidden, int inter, int heads, int groupsize) {
	ChainLayout L;
	return chain_layout(M, hidden, inter, heads, groupsize, 2 * sm_count_now(), L) ? 1 : 0;
}

size_t gptq_chain_scratch_bytes(int M, int hidden, int inter, int heads, int groupsize) {
	ChainLayout L;
	if (!chain_layout(M, hidden, inter, heads, groupsize, 2 * sm_count_now(), L)) return 0;
	return L.scratch;
}

int gptq_chain_build(const gptq_chain_layer *layers, int n_layers, int hidden, int inter, void *desc_dev) {
	if (!layers || n_layers <= 0 || !desc_dev || hidden <= 0 || inter <= 0) return GPTQ_ERR_INVALID;
	if (hidden % 128 != 0 || inter % 128 != 0) return GPTQ_ERR_SHAPE;
	if ((reinterpret_cast<uintptr_t>(desc_dev) & 127u) != 0) return GPTQ_ERR_ALIGN;
	std::vector<ChainLayer> host((size_t)n_layers);
	const int Ks[5] = {hidden, hidden, hidden, hidden, inter};
	const int Ns[5] = {3 * hidden, hidden, inter, inter, hidden};
	for (int l = 0; l < n_layers; ++l) {
		const gptq_chain_layer &src = layers[l];
		ChainLayer &dst = host[(size_t)l];
		for (int w = 0; w < 5; ++w) {
			if (!src.qweight[w] || !src.qzeros[w] || !src.scales[w]) return GPTQ_ERR_INVALID;
			if (!aligned16(src.qweight[w]) || !aligned16(src.qzeros[w]) || !aligned16(src.scales[w])) return GPTQ_ERR_ALIGN;
			if (int rc = encode_weight_map(src.qweight[w], Ks[w], Ns[w], &dst.tm[w])) return rc;
			dst.qz[w] = src.qzeros[w];
			dst.sc[w] = reinterpret_cast<const __half *>(src.scales[w]);
		}
		if (!src.ln1 || !src.ln2 || !src.kcache || !src.vcache) return GPTQ_ERR_INVALID;
		if (!aligned16(src.ln1) || !aligned16(src.ln2) || (reinterpret_cast<uintptr_t>(src.kcache) & 255u) || (reinterpret_cast<uintptr_t>(src.vcache) & 255u))
			return GPTQ_ERR_ALIGN;
		dst.ln1 = reinterpret_cast<const __half *>(src.ln1);
		dst.ln2 = reinterpret_cast<const __half *>(src.ln2);
		dst.kc = reinterpret_cast<__half *>(src.kcache);
		dst.vc = reinterpret_cast<__half *>(src.vcache);
	}
	return cuda_status(cudaMemcpy(desc_dev, host.data(), host.size() * sizeof(ChainLayer), cudaMemcpyHostToDevice));
}

int gptq_decode_chain(const void *desc_dev, int n_layers, int M, int hidden, int inter, int heads, int groupsize, const void *embed,
					  const int64_t *tok, const int32_t *pos, const void *cos, const void *sin, int max_pos, int64_t kv_stride_b,
					  int64_t kv_stride_h, float rms_eps, void *h_out, float *sumsq_out, void *scratch, size_t scratch_bytes,
					  gptq_stream_t stream) {
	if (!desc_dev || !embed || !tok || !pos || !cos || !sin || !h_out || !sumsq_out || !scratch) return GPTQ_ERR_INVALID;
	if (n_layers <= 0 || max_pos <= 0 || !(rms_eps >= 0.f)) return GPTQ_ERR_INVALID;
	if (kv_stride_h < (int64_t)max_pos * CH_D || kv_stride_b < kv_stride_h * heads) return GPTQ_ERR_INVALID;
	if (kv_stride_b % 128 != 0 || kv_stride_h % 128 != 0) return GPTQ_ERR_ALIGN;
	if (!aligned16(embed) || !aligned16(h_out) || (reinterpret_cast<uintptr_t>(scratch) & 255u) || (reinterpret_cast<uintptr_t>(desc_dev) & 127u))
		return GPTQ_ERR_ALIGN;
	if (!chain_shape_ok(M, hidden, inter, heads, groupsize)) return GPTQ_ERR_UNSUPPORTED;
	static bool ready[64] = {false};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
	if (!ready[dev]) {
		cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CH_SMEM_CAP);
		if (e != cudaSuccess) return cuda_status(e);
		ready[dev] = true;
	}
	ChainLayout L;
	// plan for two CTAs per SM; if the device cannot hold that many (co-residency is what the barriers rely on),
	// plan again for what fits
	int grid = 2 * sm_count_now();
	if (!chain_layout(M, hidden, inter, heads, groupsize, grid, L)) return GPTQ_ERR_UNSUPPORTED;
	const int fit = chain_grid(L.smem);
	if (fit <= 0) return GPTQ_ERR_UNSUPPORTED;
	if (fit < grid) {
		grid = fit;
		if (!chain_layout(M, hidden, inter, heads, groupsize, grid, L)) return GPTQ_ERR_UNSUPPORTED;
	}
	if (scratch_bytes < gptq_chain_scratch_bytes(M, hidden, inter, heads, groupsize) || scratch_bytes < L.scratch) return GPTQ_ERR_WORKSPACE;
	ChainParams &p = L.p;
	unsigned char *sb = reinterpret_cast<unsigned char *>(scratch);
	p.layers = reinterpret_cast<const ChainLayer *>(desc_dev);
	p.n_layers = n_layers;
	p.embed = reinterpret_cast<const __half *>(embed);
	p.tok = reinterpret_cast<const long long *>(tok);
	p.pos = pos;
	p.cos_t = reinterpret_cast<const __half *>(cos);
	p.sin_t = reinterpret_cast<const __half *>(sin);
	p.max_pos = max_pos;
	p.kv_stride_b = kv_stride_b;
	p.kv_stride_h = kv_stride_h;
	p.eps = rms_eps;
	p.scale = 0.08838834764831845f;          // 1 / sqrt(128)
	p.p_qkv = reinterpret_cast<float *>(sb + L.o_qkv);
	p.p_attn = reinterpret_cast<float *>(sb + L.o_attn);
	p.p_o = reinterpret_cast<float *>(sb + L.o_o);
	p.p_gu = reinterpret_cast<float *>(sb + L.o_gu);
	p.p_down = reinterpret_cast<float *>(sb + L.o_down);
	p.hA = reinterpret_cast<__half *>(sb + L.o_hA);
	p.hB = reinterpret_cast<__half *>(sb + L.o_hB);
	p.ss_a = reinterpret_cast<float *>(sb + L.o_ssa);
	p.ss_b = reinterpret_cast<float *>(sb + L.o_ssb);
	p.h_out = reinterpret_cast<__half *>(h_out);
	p.ss_f = sumsq_out;
	p.sync = reinterpret_cast<unsigned *>(sb);
	p.status = reinterpret_cast<int *>(sb + CH_CTRL_BYTES - 4);
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((unsigned)grid, 1, 1);
	cfg.blockDim = dim3(CH_THREADS, 1, 1);
	cfg.dynamicSmemBytes = L.smem;
	cfg.stream = reinterpret_cast<cudaStream_t>(stream);
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeCooperative;       // all CTAs co-resident, or the launch fails
	attr[0].val.cooperative = 1;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	return cuda_status(cudaLaunchKernelEx(&cfg, decode_chain_kernel, p));
}


size_t gptq_lm_head_workspace_bytes(int M) { return M <= 0 ? 0 : 256 + (size_t)2 * 2 * sm_count_now() * M * 4 * 2; }

int gptq_lm_head_argmax(const void *h, const float *sumsq, const void *norm_weight, const void *W, int M, int K, int V, float rms_eps,
						void *logits, int64_t *tok_out, int32_t *pos_inout, void *workspace, size_t workspace_bytes, gptq_stream_t stream) {
	if (!h || !sumsq || !norm_weight || !W || !logits || !tok_out || !pos_inout || !workspace) return GPTQ_ERR_INVALID;
	if (M < 1 || K <= 0 || V <= 0 || !(rms_eps >= 0.f)) return GPTQ_ERR_INVALID;
	if (M > CH_MAX_M) return GPTQ_ERR_UNSUPPORTED;
	if (K % 256 != 0) return GPTQ_ERR_SHAPE;
	if (!aligned16(h) || !aligned16(norm_weight) || !aligned16(W) || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return GPTQ_ERR_ALIGN;
	if (workspace_bytes < gptq_lm_head_workspace_bytes(M)) return GPTQ_ERR_WORKSPACE;
	const size_t smem = (size_t)CH_MAX_M * ((size_t)K * 2 + LM_XPAD);          // all 8 rows of x (absent ones zero)
	if (smem > 96 * 1024) return GPTQ_ERR_UNSUPPORTED;
	static bool ready[64] = {false};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GPTQ_ERR_CUDA;
	if (!ready[dev]) {
		cudaError_t e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
		if (e != cudaSuccess) return cuda_status(e);
		ready[dev] = true;
	}
	const int grid = std::max(1, std::min(2 * sm_count_now(), ((V + 15) / 16 + LM_THREADS / 32 - 1) / (LM_THREADS / 32)));      // a warp per 16 vocabulary rows
	unsigned char *wb = reinterpret_cast<unsigned char *>(workspace);
	LmHeadParams p = {};
	p.h = reinterpret_cast<const __half *>(h);
	p.ss = sumsq;
	p.norm_w = reinterpret_cast<const __half *>(norm_weight);
	p.W = reinterpret_cast<const __half *>(W);
	p.logits = reinterpret_cast<__half *>(logits);
	p.tok = reinterpret_cast<long long *>(tok_out);
	p.pos = pos_inout;
	p.ticket = reinterpret_cast<unsigned *>(wb);
	p.cand_val = reinterpret_cast<float *>(wb + 256);
	p.cand_idx = reinterpret_cast<int *>(wb + 256 + (size_t)2 * sm_count_now() * M * 4);
	p.M = M; p.K = K; p.V = V;
	p.eps = rms_eps;
	lm_head_kernel<<<grid, LM_THREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
	return cuda_status(cudaGetLastError());
}

}   // extern "C"
