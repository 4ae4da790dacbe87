/*
 * gptq_b200.h — C ABI of libgptq_b200.so: 4-bit GPTQ quantised-linear hot path for
 * NVIDIA B200 (sm_100a).
 *
 * Every pointer is a DEVICE pointer unless a comment says otherwise.  All entry
 * points that take a stream are asynchronous on that stream, never synchronise
 * the host, never allocate and never free.  They return 0 on success and a
 * negative GPTQ_ERR_* code otherwise; they never abort.  The caller owns every
 * buffer; weights are only read.
 *
 * Tensor layouts (those of the reference checkpoint, src/gptq_triton/quant_linear.py:67-71):
 *   qweight  int32 [K/8, N]   word r, nibble i (bit 4i, lowest first) = row 8r+i
 *   qzeros   int32 [G, N/8]   word c, nibble i = column 8c+i, stored value = zero-1
 *   scales   fp16  [G, N]
 *   g_idx    int32 [K]        group of row k; NULL means k / groupsize
 *   x        fp16  [M, K]     row stride ldx (elements)
 *   y        fp16  [M, N]     row stride ldy (elements)
 * decode:  w[k,n] = (q[k,n] - (qzeros[g,n] + 1)) * scales[g,n]        (README.md:93)
 * groupsize == -1 is accepted and means groupsize = K (quant_linear.py:56).
 */
#ifndef GPTQ_B200_H
#define GPTQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GPTQ_OK                 0
#define GPTQ_ERR_INVALID       -1   /* null pointer, non-positive size, bad flag            */
#define GPTQ_ERR_SHAPE         -2   /* shape violates a documented divisibility rule        */
#define GPTQ_ERR_WORKSPACE     -3   /* workspace missing or smaller than gptq_workspace_bytes */
#define GPTQ_ERR_ALIGN         -4   /* pointer or leading dimension not 16-byte aligned     */
#define GPTQ_ERR_CUDA          -5   /* the CUDA runtime reported an error at launch         */
#define GPTQ_ERR_UNSUPPORTED   -6   /* combination not implemented (e.g. head_dim != 128)   */

typedef void *gptq_stream_t;       /* a cudaStream_t */

/* Library/ABI version (major*100 + minor). */
int gptq_version(void);

/* Static, human-readable text for a GPTQ_ERR_* code.  Host pointer, never NULL. */
const char *gptq_error_string(int code);

/* After a GPTQ_ERR_CUDA return: the cudaError_t value seen by the calling thread. */
int gptq_last_cuda_error(void);

/*
 * Bytes of scratch that gptq_qmatmul / gptq_gateup_silu / gptq_qkv_rope need for a
 * problem of this size (split-K partial sums, per-tile arrival counters, and for act-order
 * decode calls the gathered copy of x).  The
 * caller allocates it once per stream, ZEROES it once, and hands it to every call;
 * the kernels leave the counter area zeroed again.  Two calls that overlap on the
 * GPU must not share one workspace.  Replaces the `torch.empty` + 1-D launch grid
 * set-up of the reference wrapper (quant_linear.py:259-263).
 */
size_t gptq_workspace_bytes(int M, int K, int N);

/*
 * y = x · deq(W) (+ bias) (+ residual).  The C-ABI form of
 * triton_matmul4(groupsize, a, qweight, scales, qzeros, bias)
 * (src/gptq_triton/quant_linear.py:228-283) and of the kernel it launches (:125-225).
 *   g_idx     optional int32 [K]: act-order group of each row, rows in checkpoint order.
 *   perm      optional int32 [K]: qweight rows have been re-ordered by
 *             gptq_act_order_rows so that groups are contiguous; perm[j] is the
 *             original row (= index into x) of sorted row j.  g_idx must be NULL then.
 *   bias      optional fp16 [N];  residual optional fp16 [M, N] with row stride ldr.
 * Requirements: K % 8 == 0, N % 8 == 0, ldx % 8 == 0, ldy % 8 == 0, pointers 16-byte aligned.
 * Fast kernels need N % 32 == 0, groupsize % 32 == 0, K % groupsize == 0 and no g_idx;
 * anything else runs on a slower general kernel.
 */
int gptq_qmatmul(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                 const int32_t *g_idx, const int32_t *perm,
                 const void *bias, const void *residual, int64_t ldr,
                 void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
                 void *workspace, size_t workspace_bytes, gptq_stream_t stream);

/*
 * y = silu(x · deq(Wg)) * (x · deq(Wu)), fp32 until the single fp16 store.  The C-ABI form of
 * triton_llama_mlp_4 (src/gptq_triton/fused_mlp.py:241-302) and llama_mlp_fused_4_kernel
 * (:109-233).  Gate and up have identical shapes [K/8, N]; y is [M, N].
 * perm: as in gptq_qmatmul, applies to both matrices.
 */
int gptq_gateup_silu(const void *x,
                     const int32_t *gate_qweight, const int32_t *gate_qzeros, const void *gate_scales,
                     const int32_t *up_qweight, const int32_t *up_qzeros, const void *up_scales,
                     const int32_t *g_idx, const int32_t *perm,
                     void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
                     void *workspace, size_t workspace_bytes, gptq_stream_t stream);

/*
 * Fused QKV projection + rotary embedding: the quantised matmul of
 * QuantLlamaAttention.forward (src/gptq_triton/fused_attention.py:91) with N = 3*hidden,
 * followed by the split into heads and apply_rotary_pos_emb on Q and K (:92-102),
 * done in the epilogue from the fp32 accumulators.
 *   cos, sin      fp16 [max_pos, head_dim] rotate-half tables
 *   position_ids  int32 [M]  (row m = b*tokens_per_batch + t); every value must be in [0, max_pos).
 *                 A value outside is not dereferenced: the row is computed at position 0 and the
 *                 status word at the end of the workspace's counter area is set to 4.
 *   q_out         fp16, element (m, h, d) at  m*q_stride_m + h*head_dim + d
 *   k_out, v_out  fp16, element (m, h, d) at
 *                   (m / tokens_per_batch)*kv_stride_b + (m % tokens_per_batch)*kv_stride_t
 *                   + h*kv_stride_h + position_ids[m]*kv_stride_pos + d
 *                 — plain [M, hidden] output: stride_b = T*hidden, stride_t = hidden,
 *                   stride_h = head_dim, stride_pos = 0;
 *                 — writing straight into a [b, h, max_seq, d] cache: stride_b = h*max_seq*d,
 *                   stride_t = 0, stride_h = max_seq*d, stride_pos = d.
 * head_dim must be 128.
 */
int gptq_qkv_rope(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                  const int32_t *g_idx, const int32_t *perm,
                  const void *cos, const void *sin, const int32_t *position_ids, int max_pos,
                  void *q_out, int64_t q_stride_m,
                  void *k_out, void *v_out, int tokens_per_batch,
                  int64_t kv_stride_b, int64_t kv_stride_t, int64_t kv_stride_h, int64_t kv_stride_pos,
                  int M, int K, int n_heads, int head_dim, int groupsize, int64_t ldx,
                  void *workspace, size_t workspace_bytes, gptq_stream_t stream);

/* uint8 [K, N] <- qweight int32 [K/8, N].  Integer unpack for the bit-exact check of the
 * layout written by pack_linear (quantize.py:262-271). */
int gptq_unpack_qweight(const int32_t *qweight, uint8_t *out, int K, int N, gptq_stream_t stream);

/* uint8 [G, N] <- qzeros int32 [G, N/8]; values as stored (zero point - 1) (quantize.py:275-289). */
int gptq_unpack_qzeros(const int32_t *qzeros, uint8_t *out, int G, int N, gptq_stream_t stream);

/* fp16 [K, N] <- (q - z - 1) * s, one rounding.  The dequantise half of the
 * dequantise-then-matmul comparison path; g_idx optional. */
int gptq_dequantize(const int32_t *qweight, const int32_t *qzeros, const void *scales, const int32_t *g_idx,
                    void *w_out, int K, int N, int groupsize, gptq_stream_t stream);

/* out[j] (int32 [K/8, N]) = packed rows of qweight taken in the order perm[0..K): the
 * load-time re-ordering that makes act-order groups contiguous.  No reference
 * counterpart (the reference refuses act-order with groups, quantize.py:41-42). */
int gptq_act_order_rows(const int32_t *qweight, const int32_t *perm, int32_t *out, int K, int N,
                        gptq_stream_t stream);

/*
 * Single-query attention over a static KV cache: out[b, h*128 + :] = softmax(q·K^T * scale) · V
 * over cache positions 0..pos[b].  Replaces, for one new token, the attention core of
 * QuantLlamaAttention.forward (src/gptq_triton/fused_attention.py:119-146: QK^T / sqrt(d), fp32
 * softmax, ·V) reading the cache that gptq_qkv_rope wrote in place instead of the torch.cat copy
 * (:105-115).  q [b, heads, 128] fp16 (row stride q_stride_b), caches [b, heads, max_seq, 128]
 * fp16 with the given strides, pos int32 [b], out fp16 [b, heads*128].  len_hint (host value,
 * about the current context length) only chooses the split count.  The workspace may be the
 * one used for gptq_qmatmul; size from gptq_attn_workspace_bytes, zeroed once.
 */
size_t gptq_attn_workspace_bytes(int batch, int heads);
int gptq_attn_decode(const void *q, int64_t q_stride_b, const void *kcache, const void *vcache,
                     int64_t kv_stride_b, int64_t kv_stride_h, const int32_t *pos,
                     void *out, int64_t out_stride_b, int batch, int heads, int head_dim,
                     int len_hint, float scale, void *workspace, size_t workspace_bytes,
                     gptq_stream_t stream);

/*
 * One sequence, one new token: QKV projection + rotary + KV-cache append + single-query attention in ONE kernel.
 * Replaces, for that case, the pair gptq_qkv_rope(_rms) + gptq_attn_decode, i.e. QuantLlamaAttention.forward up to
 * o_proj (src/gptq_triton/fused_attention.py:79-146: fused qkv_proj, rotary on q and k, cache concat, QK^T / sqrt(d),
 * fp32 softmax, .V).  A thread-block cluster of 8 CTAs per head splits the K dimension of the projection and the keys
 * of the attention; q / k / v and the softmax partials cross between the CTAs in distributed shared memory.
 * x fp16 [K]; qweight int32 [K/8, 3*n_heads*128] (q, k, v sections of n_heads*128 columns), qzeros, scales as for
 * gptq_qmatmul (no g_idx / perm); cos, sin fp16 [>= max_pos, 128]; pos int32 [1] on the device = keys already cached
 * (a value outside [0, max_pos) sets status 4, drops the K / V row and attends to nothing); kcache / vcache fp16
 * [n_heads, max_seq, 128] with kv_stride_h elements between heads; out fp16 [n_heads*128].
 * rms_weight (optional, fp16 [K]) with sumsq_in (fp32 [sumsq_tiles], sums of squares of x per 32 columns): x is
 * RMS-normalised inside the kernel.  Needs K % 1024 == 0, K <= 8192, head_dim == 128, groupsize % 128 == 0
 * (gptq_qkv_attn_supported); workspace: the one of gptq_qmatmul (only its status word is used).
 */
int gptq_qkv_attn_supported(int K, int n_heads, int head_dim, int groupsize);
int gptq_qkv_attn_decode(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                         const void *cos, const void *sin, const int32_t *pos, int max_pos, void *kcache,
                         void *vcache, int64_t kv_stride_h, void *out, int K, int n_heads, int head_dim,
                         int groupsize, float scale, const void *rms_weight, const float *sumsq_in,
                         int sumsq_tiles, float rms_eps, void *workspace, size_t workspace_bytes,
                         gptq_stream_t stream);

/*
 * gptq_qkv_attn_decode followed by the block's output projection and the residual add, still ONE kernel:
 * y = residual + attention_output x deq(Wo) (src/gptq_triton/fused_attention.py:148, o_proj, and the residual add of
 * the HF decoder layer around it).  The cluster of head h multiplies the head's 128 attention outputs with rows
 * 128 h .. 128 h + 127 of Wo (o_qweight int32 [n_heads*128/8, o_N], o_qzeros, o_scales; no g_idx / perm / bias;
 * o_groupsize % 128 == 0; o_N % 32 == 0, o_N <= 8192); the per-head partial sums are added in head order by the last
 * CTA to arrive, so the result does not depend on timing.  residual (optional) fp16 [o_N]; y fp16 [o_N];
 * sumsq_out (optional) fp32 [o_N / 32]: sums of squares of y per 32 columns (input of the folded RMSNorm of the next
 * projection); attn_out (optional) fp16 [n_heads*128]: the attention output itself.  scratch: device memory of
 * gptq_qkv_attn_oproj_scratch_bytes(n_heads, o_N) bytes, zeroed once, private to this call site.
 */
size_t gptq_qkv_attn_oproj_scratch_bytes(int n_heads, int N);
int gptq_qkv_attn_oproj_decode(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                               const void *cos, const void *sin, const int32_t *pos, int max_pos, void *kcache,
                               void *vcache, int64_t kv_stride_h, int K, int n_heads, int head_dim, int groupsize,
                               float scale, const void *rms_weight, const float *sumsq_in, int sumsq_tiles,
                               float rms_eps, const int32_t *o_qweight, const int32_t *o_qzeros,
                               const void *o_scales, int o_N, int o_groupsize, const void *residual, void *y,
                               float *sumsq_out, void *attn_out, void *scratch, size_t scratch_bytes,
                               void *workspace, size_t workspace_bytes, gptq_stream_t stream);

/*
 * gptq_qkv_attn_oproj_decode for one rank of a tensor-parallel layer: the kernel works on the rank's heads (qweight =
 * column shard of the fused QKV weight, o_qweight = row shard of o_proj) and the all-reduce over the ranks runs inside
 * its final reduction, with the buffers and the protocol of gptq_qmatmul_ar (partials / flags of a buffer set sized for
 * o_N, gptq_ar_partial_bytes / gptq_ar_flag_bytes).  Every rank ends with the same y = residual + sum over ranks.
 * No reference counterpart (the reference has no multi-GPU code).
 */
int gptq_qkv_attn_oproj_decode_ar(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                                  const void *cos, const void *sin, const int32_t *pos, int max_pos, void *kcache,
                                  void *vcache, int64_t kv_stride_h, int K, int n_heads, int head_dim, int groupsize,
                                  float scale, const void *rms_weight, const float *sumsq_in, int sumsq_tiles,
                                  float rms_eps, const int32_t *o_qweight, const int32_t *o_qzeros,
                                  const void *o_scales, int o_N, int o_groupsize, const void *residual, void *y,
                                  float *sumsq_out, void *attn_out, void *scratch, size_t scratch_bytes,
                                  void *workspace, size_t workspace_bytes, gptq_stream_t stream, int world, int rank,
                                  void *const *partials, void *const *flags);

/* y = x * rsqrt(mean(x^2) + eps) * weight, per row, fp32 inside.  The RMSNorm that the HF
 * decoder layer applies in front of the attention and MLP blocks (third-party code the
 * reference model is built from, src/gptq_triton/__init__.py:47). */
int gptq_rmsnorm(const void *x, int64_t ldx, const void *weight, void *y, int64_t ldy,
                 int M, int K, float eps, gptq_stream_t stream);

/* Embedding lookup + RMSNorm for the first decoder layer of a decode step: h_out[m] = table[tok[m]] (the
 * residual stream) and y[m] = rmsnorm(h_out[m]) * weight in one kernel; tok[M] are int64 token ids on the device
 * (0 <= tok[m] < n_rows is the caller's guarantee).  Replaces the embedding module + input_layernorm calls of
 * the HF decoder the reference runs (src/gptq_triton/__init__.py:47). */
int gptq_embed_rmsnorm(const void *table, int64_t ldt, int64_t n_rows, const int64_t *tok, const void *weight,
                       void *h_out, int64_t ldh, void *y, int64_t ldy, int M, int K, float eps,
                       gptq_stream_t stream);

/*
 * RMSNorm folded into the decode kernels (M <= 16).  No counterpart in the reference, whose
 * decoder layer runs the HF LlamaRMSNorm module between its fused ops.  A decode step otherwise
 * spends two extra launches per layer on the norm; here the projection that produces the
 * hidden state also leaves per-tile sums of squares, and the next fused op scales x while it
 * stages it:
 *   gptq_qmatmul_sumsq   = gptq_qmatmul, and sumsq_out[row * (N/32) + c] = sum over columns
 *                          32c .. 32c+31 of y^2 (y as rounded to fp16).  N % 128 == 0.
 *   gptq_gateup_silu_rms = gptq_gateup_silu on x * rsqrt(sum_t sumsq_in[row*sumsq_tiles + t] / K
 *   gptq_qkv_rope_rms      + rms_eps) * rms_weight (fp32 product, one fp16 rounding: the same
 *                          expression as gptq_rmsnorm).  sumsq_tiles (= K/32 after
 *                          gptq_qmatmul_sumsq) <= 256; no g_idx / perm.
 * Shapes outside these limits return GPTQ_ERR_UNSUPPORTED; the caller then runs gptq_rmsnorm.
 */
int gptq_qmatmul_sumsq(const void *x, const int32_t *qweight, const int32_t *qzeros,
                       const void *scales, const int32_t *g_idx, const int32_t *perm,
                       const void *bias, const void *residual, int64_t ldr, void *y,
                       int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
                       void *workspace, size_t workspace_bytes, gptq_stream_t stream,
                       float *sumsq_out);
int gptq_gateup_silu_rms(const void *x, const int32_t *gate_qweight, const int32_t *gate_qzeros,
                         const void *gate_scales, const int32_t *up_qweight,
                         const int32_t *up_qzeros, const void *up_scales, const int32_t *g_idx,
                         const int32_t *perm, void *y, int M, int K, int N, int groupsize,
                         int64_t ldx, int64_t ldy, void *workspace, size_t workspace_bytes,
                         gptq_stream_t stream, const void *rms_weight, const float *sumsq_in,
                         int sumsq_tiles, float rms_eps);
int gptq_qkv_rope_rms(const void *x, const int32_t *qweight, const int32_t *qzeros,
                      const void *scales, const int32_t *g_idx, const int32_t *perm,
                      const void *cos, const void *sin, const int32_t *position_ids, int max_pos,
                      void *q_out, int64_t q_stride_m, void *k_out, void *v_out,
                      int tokens_per_batch, int64_t kv_stride_b, int64_t kv_stride_t,
                      int64_t kv_stride_h, int64_t kv_stride_pos, int M, int K, int n_heads,
                      int head_dim, int groupsize, int64_t ldx, void *workspace,
                      size_t workspace_bytes, gptq_stream_t stream, const void *rms_weight,
                      const float *sumsq_in, int sumsq_tiles, float rms_eps);

/*
 * Tensor parallelism on one node: a row-parallel projection (o_proj, down_proj: this rank holds
 * rows [k_lo, k_hi) of the weight) whose all-reduce is part of the kernel's epilogue.  No
 * counterpart in the reference, which has no multi-GPU code.  Decode sizes only (M <= 16,
 * N % 128 == 0); larger M uses gptq_qmatmul + an NCCL all-reduce.
 *   partials[r]   receive buffer of rank r as mapped into THIS process (own buffer for r == rank),
 *                 gptq_ar_partial_bytes(N) bytes (two halves of [8 source ranks][tiles][16][128] words), zeroed once.
 *   flags[rank]   this rank's per-tile sequence numbers, gptq_ar_flag_bytes(N) bytes, zeroed once
 *                 (the other entries of flags are not used).
 * The receive area is double-buffered by the parity of the call's sequence number, so back-to-back
 * calls on one pair are safe (a rank cannot get two calls ahead of a peer: it needs that peer's
 * words of the call in between).  Calls that may overlap on the GPU need separate pairs.
 * Every rank calls with the same arguments in the same order.  Each rank pushes its tile in fp32
 * (bias included: pass it on one rank only) into its peers' receive buffers as 8-byte words
 * {value, sequence number}, polls its own buffer (at most two seconds, then status word 5) until
 * the words of every peer carry this call's sequence number, and adds the tiles of all ranks in
 * rank order, then residual, fp16 rounding and (optionally) the sums of squares as in
 * gptq_qmatmul_sumsq: every rank ends with the same bits.  `residual` is added on every rank.
 * gptq_peer_* allocate such buffers outside any caching allocator (cudaMalloc) and pass them
 * between the processes of a node as CUDA IPC handles (64 bytes).
 */
size_t gptq_ar_partial_bytes(int N);
size_t gptq_ar_flag_bytes(int N);
int gptq_qmatmul_ar(const void *x, const int32_t *qweight, const int32_t *qzeros,
                    const void *scales, const int32_t *g_idx, const int32_t *perm,
                    const void *bias, const void *residual, int64_t ldr, void *y,
                    int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
                    void *workspace, size_t workspace_bytes, gptq_stream_t stream,
                    float *sumsq_out, int world, int rank, void *const *partials,
                    void *const *flags);
int gptq_peer_alloc(size_t bytes, void **ptr);
int gptq_peer_free(void *ptr);
int gptq_peer_export(void *ptr, void *handle64);
int gptq_peer_open(const void *handle64, void **ptr);
int gptq_peer_close(void *ptr);

/*
 * Allocation-free form of gptq_qmatmul for the decode regime (M <= 16).  No counterpart in the
 * reference.  It exists for callers that cannot provide or obtain scratch memory: a host that has
 * given the whole device to its own memory pool, or a latency-critical serving loop in which
 * cudaMalloc (which synchronises the device) must never run.  The split-K scratch lives in an array
 * that is part of the library image: GPTQ_NOALLOC_SCRATCH_BYTES (4 MiB) per GPU that loads the
 * library, held until the process exits.  The call itself performs no cudaMalloc / cudaFree and
 * calls no allocating routine.
 *
 *   - Shapes: the fast decode path only (M <= 16, N % 32 == 0, K % 128 == 0, groupsize 32, 64 or a
 *     multiple of 128 dividing K, no g_idx; perm is allowed).  Other shapes: GPTQ_ERR_UNSUPPORTED.
 *   - Problems whose split-K partial sums do not fit the array are rejected with
 *     GPTQ_ERR_WORKSPACE (see gptq_noalloc_scratch_bytes for the requirement of a shape).
 *   - The first call on a device looks up the device address of the array (once per device, with
 *     that device current); make that first call before any stream capture.
 *   - All calls on a device share the one array.  The arrival counters are cleared on `stream` at
 *     the start of every call; partial sums of the previous call are simply overwritten.  Two of
 *     these calls that overlap on the GPU (e.g. issued on different streams) race on the array:
 *     keep them on one stream or order them with events.  Calls of the workspace form
 *     (gptq_qmatmul) do not touch the array and may run concurrently with one of these.
 */
#define GPTQ_NOALLOC_SCRATCH_BYTES (4u << 20)
int gptq_qmatmul_noalloc(const void *x, const int32_t *qweight, const int32_t *qzeros, const void *scales,
                         const int32_t *perm, const void *bias, const void *residual, int64_t ldr,
                         void *y, int M, int K, int N, int groupsize, int64_t ldx, int64_t ldy,
                         gptq_stream_t stream);

/* Scratch bytes gptq_qmatmul_noalloc would use for this shape on the current device (0 when the
 * shape is not served by it).  Launches nothing and touches no device memory; it does query the
 * current device's multiprocessor count (the split-K plan depends on it), so call it with the
 * device current on which the matmul will run. */
size_t gptq_noalloc_scratch_bytes(int M, int K, int N, int groupsize);

/* Status word of the allocation-free entry point on the current device: 0 = healthy; 1 = a weight
 * tile never arrived within the kernel's bounded wait; 2 = shared memory misaligned; 6 = a split-K
 * partial sum never arrived (results of that call are wrong).  The word lives in the built-in
 * array, survives later calls and is sticky until read with clear != 0.  The call synchronises the
 * device (cudaDeviceSynchronize + a 4-byte copy): use it after a batch of calls, not in a serving
 * loop, and not during stream capture.  Negative: a GPTQ_ERR_* code.  No counterpart in the reference. */
int gptq_noalloc_status(int clear);

/*
 * A whole decode step of a quantised LLaMA decoder in ONE persistent kernel (batch rows M <= 8, one GPU):
 * per layer RMSNorm, fused QKV projection + rotary embedding + in-place KV-cache append, attention of the
 * new token over the cache, o_proj + residual, RMSNorm, fused gate/up SiLU*mul, down_proj + residual.
 * Replaces, for decode steps, the per-module forward chain of the reference
 * (src/gptq_triton/fused_attention.py:79-153, fused_mlp.py:78-79 and the HF decoder layer around them):
 * the grid stays resident across all layers, phases are separated by grid-wide barriers with bounded
 * waits, and every warp streams its weight tiles and cache rows through one ring that keeps running
 * across the phase boundaries.
 *
 * Set-up (once per model): fill one gptq_chain_layer per decoder layer (device pointers; the five weights
 * are the fused QKV [hidden, 3*hidden], o_proj [hidden, hidden], gate and up [hidden, inter] and down
 * [inter, hidden], all without act-order and without bias, one groupsize % 128 == 0 for all of them;
 * KV caches [M, heads, max_pos, 128] fp16, 256-byte aligned) and call gptq_chain_build, which encodes the
 * tensor maps and copies the descriptors into desc_dev (gptq_chain_desc_bytes(n_layers) bytes of device
 * memory, 128-byte aligned; synchronous host-to-device copy).
 * Per step: gptq_decode_chain.  tok[M] (int64) are the tokens fed, pos[M] (int32) their positions (= keys
 * already cached; the new K / V row is written at pos).  h_out [M, hidden] fp16 receives the final hidden
 * state BEFORE the last RMSNorm and sumsq_out [M, hidden / 32] its sums of squares per 32 columns, which is
 * what gptq_lm_head_argmax takes.  scratch: gptq_chain_scratch_bytes(...) bytes, 256-byte aligned, zeroed
 * once; the last 4 bytes of its first 16 KiB are the status word (1: a load never arrived, 4: position
 * outside [0, max_pos), 7: a grid barrier timed out); after a non-zero status zero the first 16 KiB again.
 * The launch is cooperative (all CTAs co-resident, else it fails with GPTQ_ERR_CUDA).
 * gptq_chain_supported: 1 when the shape is served (M <= 8, head_dim 128, hidden % 256 == 0, inter % 128 == 0,
 * groupsize % 128 == 0 dividing hidden and inter).
 */
typedef struct gptq_chain_layer {
    const int32_t *qweight[5];      /* fused qkv, o_proj, gate, up, down */
    const int32_t *qzeros[5];
    const void *scales[5];
    const void *ln1, *ln2;          /* RMSNorm weights before attention / before the MLP, fp16 [hidden] */
    void *kcache, *vcache;
} gptq_chain_layer;
int gptq_chain_supported(int M, int hidden, int inter, int heads, int groupsize);
size_t gptq_chain_desc_bytes(int n_layers);
size_t gptq_chain_scratch_bytes(int M, int hidden, int inter, int heads, int groupsize);
int gptq_chain_build(const gptq_chain_layer *layers /* host */, int n_layers, int hidden, int inter, void *desc_dev);
int gptq_decode_chain(const void *desc_dev, int n_layers, int M, int hidden, int inter, int heads,
                      int groupsize, const void *embed, const int64_t *tok, const int32_t *pos,
                      const void *cos, const void *sin, int max_pos, int64_t kv_stride_b,
                      int64_t kv_stride_h, float rms_eps, void *h_out, float *sumsq_out,
                      void *scratch, size_t scratch_bytes, gptq_stream_t stream);

/*
 * Final RMSNorm + fp16 lm_head + greedy sampling in one kernel (the tail of a decode step; the reference
 * leaves this to HF's LlamaForCausalLM and generate(), generate.py:41-50).  h [M, K] fp16 is the hidden
 * state before the norm, sumsq [M, K / 32] its sums of squares per 32 columns, W [V, K] fp16 the lm_head
 * weight.  Writes logits [M, V] fp16, tok_out[M] = arg-max (lowest index on ties) and adds 1 to
 * pos_inout[M].  M <= 8, K % 256 == 0.  workspace: gptq_lm_head_workspace_bytes(M) bytes, 256-byte
 * aligned, zeroed once.
 */
size_t gptq_lm_head_workspace_bytes(int M);
int gptq_lm_head_argmax(const void *h, const float *sumsq, const void *norm_weight, const void *W, int M,
                        int K, int V, float rms_eps, void *logits, int64_t *tok_out, int32_t *pos_inout,
                        void *workspace, size_t workspace_bytes, gptq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GPTQ_B200_H */
