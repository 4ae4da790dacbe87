// Body of the tcgen05 prefill kernel; included by qmm_tc.cu.
namespace gptq {

template <int NSTREAM, int EPI, int BN, int MH>
__global__ void __launch_bounds__(TC_THREADS, 1) tc_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw0,
																 const __grid_constant__ CUtensorMap tmw1, const TcParams p) {
	extern __shared__ __align__(1024) unsigned char smem[];
	// MH = 2: the CTA computes two 128-row halves (256 rows of X) against the same dequantised B
	// stage: every weight is decoded once per 256 rows, and the MMAs of one stage run twice as long,
	// which covers the release -> dequantise -> refill latency of a stage with fewer stages.
	constexpr int S = tc_stages(NSTREAM, BN, MH);
	// Dequantise groups (of 128 threads): as many as B stages, so that a group always returns to the
	// same stage exactly one phase later (a group that ran two phases ahead of a stage's barrier would
	// mistake an old phase for the one it waits for).  With three stages the fourth group only joins
	// the epilogue.
	constexpr int NG = S;
	static_assert(NSTREAM * BN <= 256 && MH * NSTREAM * BN <= 512, "at most 512 TMEM columns");
	constexpr uint32_t TMEM_COLS = MH * NSTREAM * BN;        // 128, 256 or 512 fp32 columns
	constexpr int PS = tc_pstages(NSTREAM, BN, MH);          // stages of the packed-weight ring
	constexpr int A_STAGE = MH * TC_TILE_BYTES;              // X tile(s) of one stage
	constexpr int PW_BYTES = 8 * BN * 4;                     // packed tile of one K-block: 8 words x BN columns
	constexpr int B_TILE = BN * TC_BK * 2;                   // dequantised B stage: BN rows x 128 bytes
	constexpr int CPT = BN / 128;                            // weight columns per dequantise thread
	constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);   // D fp32, A/B fp16 K-major, N = BN, M = 128
	const TcArgs &a = p.a;

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int n0 = blockIdx.x * BN, m0 = blockIdx.y * (TC_BM * MH);
	// split-K (plain epilogue only): blockIdx.z takes the K-blocks [kb0, kb0 + nkb) and leaves fp32 partial sums
	const int kb0 = blockIdx.z * p.kb_per_split;
	const int nkb = min(p.kb_per_split, a.K / TC_BK - kb0);

	unsigned char *sA = smem;                                              // [S][MH][16 KB]
	unsigned char *sB = smem + S * A_STAGE;                                // [NSTREAM][S][B_TILE]
	unsigned char *sW = sB + NSTREAM * S * B_TILE;                         // [PS][NSTREAM][PW_BYTES] packed words
	uint64_t *bars = reinterpret_cast<uint64_t *>(sW + PS * NSTREAM * PW_BYTES);
	const uint32_t bar_full_a = smem_u32(bars), bar_full_b = smem_u32(bars + S), bar_empty = smem_u32(bars + 2 * S);
	const uint32_t bar_acc = smem_u32(bars + 3 * S);
	const uint32_t bar_full_w = smem_u32(bars + 3 * S + 1), bar_empty_w = smem_u32(bars + 3 * S + 1 + PS);
	uint32_t *s_tmem = reinterpret_cast<uint32_t *>(bars + 3 * S + 1 + 2 * PS);
	volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem + 1);

	if (tid == 0) {
		for (int s = 0; s < S; ++s) {
			mbar_init(bar_full_a + 8 * s, 1);
			mbar_init(bar_full_b + 8 * s, 128);               // the 128 threads of the group that owns the stage
			mbar_init(bar_empty + 8 * s, 1);
		}
		mbar_init(bar_acc, 1);
		for (int s = 0; s < PS; ++s) {
			mbar_init(bar_full_w + 8 * s, 1);
			mbar_init(bar_empty_w + 8 * s, 4);                // one arrival per warp of the consuming group
		}
		*s_abort = 0;
		fence_mbar_init();
		tma_prefetch_desc(&tmx);
	}
	if (warp == 1) {                       // the MMA warp owns tensor memory
		tmem_alloc(smem_u32(s_tmem), TMEM_COLS);
		tmem_relinquish();
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = *s_tmem;

	auto fail = [&]() {
		*s_abort = 1;
		atomicExch(p.status, 3);           // 3: a wait inside the tensor-core kernel ran out
	};

	if (warp == 0) {
		// ---------------- TMA producer: packed weight tiles (deep ring) and X tiles ----------------
		if (lane == 0) {
			int kw = 0;                           // next K-block of packed weights to request
			auto feed_w = [&](int upto) -> bool {
				for (; kw < upto && kw < nkb; ++kw) {
					const int s = kw % PS;
					if (!mbar_wait_bounded(bar_empty_w + 8 * s, ((kw / PS) & 1) ^ 1, TC_SPIN)) return false;
					mbar_arrive_expect_tx(bar_full_w + 8 * s, NSTREAM * PW_BYTES);
					tma_load_2d(smem_u32(sW + (s * NSTREAM) * PW_BYTES), &tmw0, n0, (kb0 + kw) * 8, bar_full_w + 8 * s);
					if (NSTREAM == 2) tma_load_2d(smem_u32(sW + (s * NSTREAM + 1) * PW_BYTES), &tmw1, n0, (kb0 + kw) * 8, bar_full_w + 8 * s);
				}
				return true;
			};
			for (int kb = 0; kb < nkb && !*s_abort; ++kb) {
				if (!feed_w(kb + PS)) { fail(); break; }
				const int s = kb % S;
				if (!mbar_wait_bounded(bar_empty + 8 * s, ((kb / S) & 1) ^ 1, TC_SPIN)) { fail(); break; }
				mbar_arrive_expect_tx(bar_full_a + 8 * s, A_STAGE);
#pragma unroll
				for (int h = 0; h < MH; ++h)          // rows beyond M are filled with zeros by the copy
					tma_load_2d(smem_u32(sA + s * A_STAGE + h * TC_TILE_BYTES), &tmx, (kb0 + kb) * TC_BK, m0 + h * TC_BM, bar_full_a + 8 * s);
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer ----------------
		if (lane == 0) {
			for (int kb = 0; kb < nkb && !*s_abort; ++kb) {
				const int s = kb % S;
				const uint32_t ph = (kb / S) & 1;
				if (!mbar_wait_bounded(bar_full_a + 8 * s, ph, TC_SPIN)) { fail(); break; }
				if (!mbar_wait_bounded(bar_full_b + 8 * s, ph, TC_SPIN)) { fail(); break; }
				tc_fence_after();
#pragma unroll
				for (int h = 0; h < MH; ++h) {
					const uint32_t a_addr = smem_u32(sA + s * A_STAGE + h * TC_TILE_BYTES);
#pragma unroll
					for (int st = 0; st < NSTREAM; ++st) {
						const uint32_t b_addr = smem_u32(sB + (st * S + s) * B_TILE);
#pragma unroll
						for (int k = 0; k < TC_BK / 16; ++k)
							umma_f16(tmem_base + (h * NSTREAM + st) * BN, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), IDESC,
									 (kb > 0 || k > 0) ? 1u : 0u);
					}
				}
				umma_commit(bar_empty + 8 * s);          // stage free once these MMAs have read it
			}
			umma_commit(bar_acc);                        // accumulators complete
		}
	} else {
		// ---------------- dequantise producers, then epilogue ----------------
		// Four groups of 128 threads; group j dequantises K-blocks j, j+4, ... (into B stage kb % S), so
		// the groups' barrier round trips and proxy fences overlap.  Thread -> weight column wt of the tile.
		constexpr int RPT = 8, r0 = 0;
		const int wt = (tid - 64) & 127, grp = (tid - 64) >> 7;         // columns wt (+128 when BN = 256)
		const int nz = a.N >> 3, zsh = (wt & 7) * 4;
		const uint32_t b_row = (uint32_t)((wt >> 3) * 1024 + (wt & 7) * 128);
		// a "unit" is one weight column of one stream: NU = NSTREAM * CPT units per thread
		constexpr int NU = NSTREAM * CPT;
		uint32_t cur[NU][RPT];
		// scale / zero of the current and of the next group (fetched one group ahead)
		uint32_t ZE[NU], ZO[NU], S2[NU], zraw[NU];
		unsigned short sraw[NU];
		const int ngroups = a.K / a.groupsize;
		auto fetch_group = [&](int g) {
#pragma unroll
			for (int u = 0; u < NU; ++u) {
				const int st = u / CPT, n = n0 + wt + 128 * (u % CPT);
				const int32_t *qz = (NSTREAM == 2 && st) ? a.qz1 : a.qz0;
				const __half *sc = (NSTREAM == 2 && st) ? a.sc1 : a.sc0;
				zraw[u] = (uint32_t)__ldg(qz + (size_t)g * nz + (n >> 3));
				sraw[u] = __half_as_ushort(__ldg(sc + (size_t)g * a.N + n));
			}
		};
		if (grp < NG) fetch_group(min(((kb0 + grp) * TC_BK) / a.groupsize, ngroups - 1));
		int g_cur = -1;
		bool ok = true;
		for (int kb = (grp < NG ? grp : nkb); kb < nkb; kb += NG) {
			const int g = ((kb0 + kb) * TC_BK) / a.groupsize;
			if (g != g_cur) {
				g_cur = g;
#pragma unroll
				for (int u = 0; u < NU; ++u) {
					const uint32_t zz = ((zraw[u] >> zsh) & 0xFu) + 1u;
					ZE[u] = (0x6400u + zz) * 0x00010001u;            // half2(1024 + zero)
					ZO[u] = (0xD400u + (zz << 4)) * 0x00010001u;     // half2(-(64 + zero))
					S2[u] = (uint32_t)sraw[u] * 0x00010001u;
				}
			}
			{
				const int g_next = ((kb0 + kb + NG) * TC_BK) / a.groupsize;     // group of this thread's next K-block
				if (g_next < ngroups) fetch_group(g_next);                 // always: the registers then hold that group's data
			}
			{
				const int ws = kb % PS;
				if (*s_abort || !mbar_wait_bounded(bar_full_w + 8 * ws, (kb / PS) & 1, TC_SPIN)) { ok = false; break; }
#pragma unroll
				for (int u = 0; u < NU; ++u) {
					const uint32_t *wp = reinterpret_cast<const uint32_t *>(sW + (ws * NSTREAM + u / CPT) * PW_BYTES) + wt + 128 * (u % CPT);
#pragma unroll
					for (int r = 0; r < RPT; ++r) cur[u][r] = wp[(r0 + r) * BN];
				}
				__syncwarp();
				if (lane == 0) mbar_arrive(bar_empty_w + 8 * ws);
			}
			const int s = kb % S;
			if (*s_abort || !mbar_wait_bounded(bar_empty + 8 * s, ((kb / S) & 1) ^ 1, TC_SPIN)) { ok = false; break; }
#pragma unroll
			for (int u = 0; u < NU; ++u) {
				// row (wt + 128j) of the B tile: 8-row groups of 1024 bytes, 16 groups per 128 rows
				unsigned char *bst = sB + ((u / CPT) * S + s) * B_TILE + b_row + (u % CPT) * 16384;
#pragma unroll
				for (int r = 0; r < RPT; ++r) {
					const uint32_t w = cur[u][r], w8 = w >> 8;
					const uint32_t p04 = h2_mul(h2_sub(lop3_and_or(w, MASK_LO, MAGIC_1024), ZE[u]), S2[u]);
					const uint32_t p15 = h2_mul(h2_fma(lop3_and_or(w, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[u]), S2[u]);
					const uint32_t p26 = h2_mul(h2_sub(lop3_and_or(w8, MASK_LO, MAGIC_1024), ZE[u]), S2[u]);
					const uint32_t p37 = h2_mul(h2_fma(lop3_and_or(w8, MASK_HI, MAGIC_1024), 0x2C002C00u, ZO[u]), S2[u]);
					uint4 o;                                   // natural k order k0..k7
					o.x = __byte_perm(p04, p15, 0x5410);
					o.y = __byte_perm(p26, p37, 0x5410);
					o.z = __byte_perm(p04, p15, 0x7632);
					o.w = __byte_perm(p26, p37, 0x7632);
					*reinterpret_cast<uint4 *>(bst + (((r0 + r) ^ (wt & 7)) << 4)) = o;
				}
			}
			fence_proxy_async();                               // generic-proxy stores -> visible to the tensor core
			mbar_arrive(bar_full_b + 8 * s);
		}
		if (!ok) fail();

		// ---------------- epilogue: TMEM -> registers -> global ----------------
		if (ok && !*s_abort && mbar_wait_bounded(bar_acc, 0, TC_SPIN)) {
			tc_fence_after();
			const int q = warp & 3;                             // TMEM lane quarter this warp may read
			const int cq = (warp - 2) >> 2;                     // which 32-column chunk of the tile this warp drains
#pragma unroll 1
			for (int h = 0; h < MH; ++h) {
			const int row = m0 + h * TC_BM + q * 32 + lane;
			const uint32_t t_row = tmem_base + (uint32_t)(h * NSTREAM * BN) + ((uint32_t)(q * 32) << 16);
			const bool live = row < a.M;
			if (EPI == TC_EPI_ROPE) {
				// the tile holds BN/128 heads; warp group cq takes head cq>>1, rotary half cq&1
				const int head_local = cq >> 1;
				const int ncol = n0 + head_local * 128;
				const int section = ncol / a.hidden, head = (ncol - section * a.hidden) >> 7;
				int pos = live ? a.pos[row] : 0;
				bool pos_ok = true;
				if (pos < 0 || pos >= a.max_pos) {      // never index the tables / the cache out of range
					atomicExch(p.status, 4);
					pos = 0;
					pos_ok = false;
				}
				__half *dst = nullptr;
				if (live) {
					if (section == 0) {
						dst = a.q_out + (size_t)row * a.q_stride_m + head * 128;
					} else {
						const int bi = row / a.tokens_per_batch, ti = row - bi * a.tokens_per_batch;
						dst = (section == 1 ? a.k_out : a.v_out) + (size_t)bi * a.kv_sb + (size_t)ti * a.kv_st + (size_t)head * a.kv_sh +
							  (size_t)pos * a.kv_sp;
					}
				}
				const uint32_t t_head = t_row + head_local * 128;
#pragma unroll 1
				for (int hc = (cq & 1); hc < ((cq < 2 * (BN / 128)) ? (cq & 1) + 1 : (cq & 1)); ++hc) {
					float lo[32], hi[32];
					tmem_ld32(t_head + hc * 32, lo);
					tmem_ld32(t_head + 64 + hc * 32, hi);
					tmem_ld_wait();
					if (live && (pos_ok || section == 0)) {      // K / V of an out-of-range position are dropped, not written over cache row 0
						const __half *ct = a.cos_t + (size_t)pos * 128, *stb = a.sin_t + (size_t)pos * 128;
#pragma unroll
						for (int j = 0; j < 32; j += 2) {
							const int d = hc * 32 + j;
							float o1[2], o2[2];
#pragma unroll
							for (int e = 0; e < 2; ++e) {
								const float x1 = lo[j + e], x2 = hi[j + e];
								if (section < 2) {
									o1[e] = x1 * __half2float(ct[d + e]) - x2 * __half2float(stb[d + e]);
									o2[e] = x2 * __half2float(ct[d + e + 64]) + x1 * __half2float(stb[d + e + 64]);
								} else {
									o1[e] = x1;
									o2[e] = x2;
								}
							}
							*reinterpret_cast<__half2 *>(dst + d) = __floats2half2_rn(o1[0], o1[1]);
							*reinterpret_cast<__half2 *>(dst + d + 64) = __floats2half2_rn(o2[0], o2[1]);
						}
					}
				}
			} else {
#pragma unroll 1
				for (int c = cq * (BN / 128); c < (cq + 1) * (BN / 128); ++c) {
					float v[32], u[32];
					tmem_ld32(t_row + c * 32, v);
					if (EPI == TC_EPI_SILU) tmem_ld32(t_row + BN + c * 32, u);
					tmem_ld_wait();
					if (EPI == TC_EPI_PLAIN && p.partial != nullptr) {
						// split-K: this split's fp32 sums; bias, residual and the fp16 rounding follow in tc_splitk_finish
						if (live) {
							float4 *dst = reinterpret_cast<float4 *>(p.partial + ((size_t)blockIdx.z * a.M + row) * a.N + n0 + c * 32);
#pragma unroll
							for (int j = 0; j < 8; ++j) __stcg(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
						}
					} else if (live) {
						const int nc = n0 + c * 32;
#pragma unroll
						for (int j = 0; j < 32; j += 8) {
							float o[8];
#pragma unroll
							for (int e = 0; e < 8; ++e) o[e] = (EPI == TC_EPI_SILU) ? silu_f32(v[j + e]) * u[j + e] : v[j + e];
							if (EPI == TC_EPI_PLAIN) {
								if (a.bias) {
									const uint4 bv = *reinterpret_cast<const uint4 *>(a.bias + nc + j);
									const __half2 *bh = reinterpret_cast<const __half2 *>(&bv);
#pragma unroll
									for (int e = 0; e < 4; ++e) {
										const float2 f = __half22float2(bh[e]);
										o[2 * e] += f.x;
										o[2 * e + 1] += f.y;
									}
								}
								if (a.residual) {
									const uint4 rv = *reinterpret_cast<const uint4 *>(a.residual + (size_t)row * a.ldr + nc + j);
									const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
									for (int e = 0; e < 4; ++e) {
										const float2 f = __half22float2(rh[e]);
										o[2 * e] += f.x;
										o[2 * e + 1] += f.y;
									}
								}
							}
							uint4 ov;
							__half2 *oh = reinterpret_cast<__half2 *>(&ov);
#pragma unroll
							for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(o[2 * e], o[2 * e + 1]);
							*reinterpret_cast<uint4 *>(a.y + (size_t)row * a.ldy + nc + j) = ov;
						}
					}
				}
			}
			}
		} else if (ok) {
			fail();
		}
	}
	tc_fence_before();
	__syncthreads();
	if (warp == 1) {
		// tensor memory goes back only after every MMA issued above has completed (also when unwinding)
		if (lane == 0) mbar_wait_bounded(bar_acc, 0, TC_SPIN);
		__syncwarp();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
}

// Split-K tail of the plain epilogue: y = fp16(sum over splits of the partial sums (in split order) + bias + residual).
__global__ void __launch_bounds__(256) tc_splitk_finish(const float *__restrict__ partial, int splitk, int M, int N, const __half *__restrict__ bias,
														const __half *__restrict__ residual, long long ldr, __half *__restrict__ y, long long ldy) {
	const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;           // unit of 8 columns
	const int upr = N >> 3;
	if (i >= (size_t)M * upr) return;
	const int row = (int)(i / upr), n = (int)(i % upr) * 8;
	float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
	for (int s = 0; s < splitk; ++s) {
		const float4 *src = reinterpret_cast<const float4 *>(partial + ((size_t)s * M + row) * N + n);
		const float4 a = __ldcg(src), b = __ldcg(src + 1);
		o[0] += a.x; o[1] += a.y; o[2] += a.z; o[3] += a.w;
		o[4] += b.x; o[5] += b.y; o[6] += b.z; o[7] += b.w;
	}
	if (bias) {
		const uint4 bv = *reinterpret_cast<const uint4 *>(bias + n);
		const __half2 *bh = reinterpret_cast<const __half2 *>(&bv);
#pragma unroll
		for (int e = 0; e < 4; ++e) {
			const float2 f = __half22float2(bh[e]);
			o[2 * e] += f.x;
			o[2 * e + 1] += f.y;
		}
	}
	if (residual) {
		const uint4 rv = *reinterpret_cast<const uint4 *>(residual + (size_t)row * ldr + n);
		const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
		for (int e = 0; e < 4; ++e) {
			const float2 f = __half22float2(rh[e]);
			o[2 * e] += f.x;
			o[2 * e + 1] += f.y;
		}
	}
	uint4 ov;
	__half2 *oh = reinterpret_cast<__half2 *>(&ov);
#pragma unroll
	for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(o[2 * e], o[2 * e + 1]);
	*reinterpret_cast<uint4 *>(y + (size_t)row * ldy + n) = ov;
}

}   // namespace gptq
