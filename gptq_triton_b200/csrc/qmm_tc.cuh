// Prefill-regime (M > 16) quantised matmul on the tcgen05 tensor cores.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace gptq {

enum { TC_EPI_PLAIN = 0, TC_EPI_SILU = 1, TC_EPI_ROPE = 2 };

struct TcArgs {
	const __half *x;
	long long ldx;
	const int32_t *qw0, *qw1;
	const int32_t *qz0, *qz1;
	const __half *sc0, *sc1;
	const int32_t *perm;
	int M, K, N, groupsize;
	const __half *bias;
	const __half *residual;
	long long ldr;
	__half *y;
	long long ldy;
	const __half *cos_t, *sin_t;
	const int32_t *pos;
	__half *q_out, *k_out, *v_out;
	long long q_stride_m, kv_sb, kv_st, kv_sh, kv_sp;
	int tokens_per_batch, hidden, max_pos;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
								  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
								  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool tc_shape_ok(int M, int K, int N, int groupsize);
size_t tc_ws_bytes(int M, int N);
int tc_launch(const TcArgs &a, int epi, void *workspace, size_t ws_bytes, cudaStream_t stream);

}   // namespace gptq
