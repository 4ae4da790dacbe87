"""CPU oracle for the GPTQ-triton inference hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch-on-CPU / numpy, the arithmetic of the
reference project's quantised linear, fused QKV + rotary and fused gate/up MLP.
It is the checker that the CUDA kernels are compared against.  Nothing in the
product package imports it; only the test-suite, the smoke check and the
benchmark's CPU-baseline leg do.

Parity pinning: the functions below are checked (tests/test_oracle_golden.py)
against fixtures produced by running the reference's own code in a CPU-only
container: its packer and round-to-nearest fake quantiser, and its two Triton
kernels executed by the Triton interpreter.  The rotary embedding is third-party
arithmetic (HF transformers); it is pinned against vectors produced by the
installed transformers `apply_rotary_pos_emb`.

Reference locations (paths inside the reference project):
  packing layout            quantize.py:262-289
  decode formula            README.md:93, src/gptq_triton/quant_linear.py:187-188,211-212
  group of row k            src/gptq_triton/quant_linear.py:200  (k // groupsize)
  accumulate / store        src/gptq_triton/quant_linear.py:194,214,225
  bias                      src/gptq_triton/quant_linear.py:280-281
  fused MLP epilogue        src/gptq_triton/fused_mlp.py:222-233,236-238
  fused attention           src/gptq_triton/fused_attention.py:89-153
  RTN fake quantiser        quantize.py:294-329, gptq.py:174-246
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

_SHIFTS = np.arange(8, dtype=np.uint32) * 4


# ----------------------------------------------------------------------------
# bit layout
# ----------------------------------------------------------------------------

def _as_u32(t) -> np.ndarray:
	if isinstance(t, torch.Tensor):
		t = t.detach().cpu().contiguous().numpy()
	return np.ascontiguousarray(t).view(np.uint32)


def unpack_qweight(qweight) -> np.ndarray:
	"""int32 [K/8, N] -> uint8 [K, N].  Word r, nibble i (i=0 lowest) is row 8r+i.
	Follows quantize.py:262-271 (`qweight[row] |= intweight[j] << (4*(j-i))`)."""
	q = _as_u32(qweight)
	R, N = q.shape
	out = (q[:, None, :] >> _SHIFTS[None, :, None]) & np.uint32(0xF)
	return out.reshape(R * 8, N).astype(np.uint8)


def unpack_qzeros(qzeros) -> np.ndarray:
	"""int32 [G, N/8] -> uint8 [G, N] of STORED values (= zero point - 1).
	Word c, nibble i is column 8c+i.  Follows quantize.py:275-289."""
	z = _as_u32(qzeros)
	G, C = z.shape
	out = (z[:, :, None] >> _SHIFTS[None, None, :]) & np.uint32(0xF)
	return out.reshape(G, C * 8).astype(np.uint8)


def pack_qweight(intweight: np.ndarray) -> np.ndarray:
	"""uint [K, N] (values 0..15) -> int32 [K/8, N]; inverse of unpack_qweight."""
	w = np.asarray(intweight).astype(np.uint32)
	K, N = w.shape
	assert K % 8 == 0
	w = w.reshape(K // 8, 8, N)
	out = np.zeros((K // 8, N), dtype=np.uint32)
	for i in range(8):
		out |= w[:, i, :] << np.uint32(4 * i)
	return out.view(np.int32)


def pack_qzeros(stored: np.ndarray) -> np.ndarray:
	"""uint [G, N] of stored zero values (zero-1, 0..15) -> int32 [G, N/8]."""
	z = np.asarray(stored).astype(np.uint32)
	G, N = z.shape
	assert N % 8 == 0
	z = z.reshape(G, N // 8, 8)
	out = np.zeros((G, N // 8), dtype=np.uint32)
	for i in range(8):
		out |= z[:, :, i] << np.uint32(4 * i)
	return out.view(np.int32)


def group_index(K: int, groupsize: int, g_idx=None) -> np.ndarray:
	"""Group of input row k.  Without act-order it is k // groupsize
	(quant_linear.py:200); groupsize == -1 means one group (quant_linear.py:56).
	With an explicit g_idx (int32 [K]) that vector is used as is."""
	if g_idx is not None:
		g = g_idx.detach().cpu().numpy() if isinstance(g_idx, torch.Tensor) else np.asarray(g_idx)
		assert g.shape == (K,)
		return g.astype(np.int64)
	gs = K if groupsize == -1 else groupsize
	return np.arange(K, dtype=np.int64) // gs


# ----------------------------------------------------------------------------
# decode
# ----------------------------------------------------------------------------

def dequant_f32(qweight, qzeros, scales, groupsize: int, g_idx=None) -> torch.Tensor:
	"""fp32 weights [K, N]:  w = (q - z - 1) * s  with the product in fp32
	(README.md:93).  This is the weight of the fp32-accumulated reference."""
	q = unpack_qweight(qweight).astype(np.int32)
	K, N = q.shape
	z = unpack_qzeros(qzeros).astype(np.int32) + 1
	g = group_index(K, groupsize, g_idx)
	s = scales.detach().cpu().float().numpy() if isinstance(scales, torch.Tensor) else np.asarray(scales, dtype=np.float32)
	w = (q - z[g]).astype(np.float32) * s[g]
	return torch.from_numpy(w)


def dequant_f16(qweight, qzeros, scales, groupsize: int, g_idx=None) -> torch.Tensor:
	"""fp16 weights, single rounding of (q - z - 1) * s.  The integer difference
	is exact and the fp16*fp16 product is exact in fp32, so rounding the fp32
	product once gives the correctly rounded fp16 weight."""
	return dequant_f32(qweight, qzeros, scales, groupsize, g_idx).half()


def dequant_f16_kernel_form(qweight, qzeros, scales, groupsize: int, g_idx=None) -> torch.Tensor:
	"""fp16 weights the way the reference kernel forms them:
	fp16(q*s) - fp16((z+1)*s), difference rounded to fp16
	(quant_linear.py:187-188,211-212)."""
	q = unpack_qweight(qweight).astype(np.float32)
	K, N = q.shape
	z = unpack_qzeros(qzeros).astype(np.float32) + 1.0
	g = group_index(K, groupsize, g_idx)
	s = scales.detach().cpu().numpy().astype(np.float16)
	s32 = s.astype(np.float32)
	a = (q * s32[g]).astype(np.float16)              # q (int32) * scales (fp16) -> fp16
	b = (z * s32).astype(np.float16)[g]              # (zeros + 1) * scales -> fp16
	w = (a.astype(np.float32) - b.astype(np.float32)).astype(np.float16)
	return torch.from_numpy(w)


# ----------------------------------------------------------------------------
# quantised linear
# ----------------------------------------------------------------------------

def _flat(x: torch.Tensor) -> torch.Tensor:
	return x.detach().cpu().reshape(-1, x.shape[-1])


def qmatmul_r32(x, qweight, qzeros, scales, groupsize, g_idx=None, bias=None, residual=None) -> torch.Tensor:
	"""fp32-accumulated reference: fp32 weights, fp32 matmul of the fp16-valued
	activations.  Returns fp32 [M, N] (not rounded) so that callers can measure
	the error of an fp16 result against it.  Bias / residual are added in fp32."""
	w = dequant_f32(qweight, qzeros, scales, groupsize, g_idx)
	y = _flat(x).double() @ w.double()
	if bias is not None:
		y = y + bias.detach().cpu().double()
	if residual is not None:
		y = y + _flat(residual).double()
	return y.float()


def qmatmul_r16(x, qweight, qzeros, scales, groupsize, g_idx=None, bias=None) -> torch.Tensor:
	"""The dequantise-then-matmul path: decode to an fp16 weight, torch.matmul in
	fp16 on the CPU (fp32 accumulation inside the library), fp16 result, bias added
	afterwards in fp16 (quant_linear.py:280-281).  This is what the CPU baseline times."""
	w = dequant_f16(qweight, qzeros, scales, groupsize, g_idx)
	y = torch.matmul(_flat(x).half(), w)
	if bias is not None:
		y = y + bias.detach().cpu().half()
	return y


def qmatmul_kernel_form(x, qweight, qzeros, scales, groupsize) -> torch.Tensor:
	"""Emulates matmul4_kernel: kernel-form fp16 weights, fp32 accumulation, one
	rounding to fp16 at the store (quant_linear.py:194,214,225)."""
	w = dequant_f16_kernel_form(qweight, qzeros, scales, groupsize)
	return (_flat(x).float() @ w.float()).half()


# ----------------------------------------------------------------------------
# fused gate/up MLP
# ----------------------------------------------------------------------------

def silu_f32(x: torch.Tensor) -> torch.Tensor:
	"""x * sigmoid(x) in fp32 (fused_mlp.py:236-238)."""
	return x * torch.sigmoid(x)


def gateup_silu_r32(x, gate, up, groupsize, g_idx=None) -> torch.Tensor:
	"""silu(x·Wg) * (x·Wu) with everything in fp32 until the end; returns fp32.
	`gate` and `up` are (qweight, qzeros, scales) triples."""
	g = qmatmul_r32(x, gate[0], gate[1], gate[2], groupsize, g_idx)
	u = qmatmul_r32(x, up[0], up[1], up[2], groupsize, g_idx)
	return silu_f32(g) * u


def gateup_silu_kernel_form(x, gate, up, groupsize) -> torch.Tensor:
	"""Emulates llama_mlp_fused_4_kernel: kernel-form fp16 weights, two fp32
	accumulators, fp32 silu and product, one fp16 rounding (fused_mlp.py:186-233)."""
	xf = _flat(x).float()
	g = xf @ dequant_f16_kernel_form(gate[0], gate[1], gate[2], groupsize).float()
	u = xf @ dequant_f16_kernel_form(up[0], up[1], up[2], groupsize).float()
	return (silu_f32(g) * u).half()


def mlp_unfused_r16(x, gate, up, down, groupsize, g_idx=None, g_idx_down=None) -> torch.Tensor:
	"""The reference's unfused dequant path for the MLP block: three quantised
	linears each returning fp16, fp16 silu and fp16 multiply in between (HF
	LlamaMLP.forward with QuantLinear children; see fused_mlp.py:13-27)."""
	g = qmatmul_r16(x, gate[0], gate[1], gate[2], groupsize, g_idx)
	u = qmatmul_r16(x, up[0], up[1], up[2], groupsize, g_idx)
	h = torch.nn.functional.silu(g) * u
	return qmatmul_r16(h, down[0], down[1], down[2], groupsize, g_idx_down)


def mlp_r32(x, gate, up, down, groupsize, g_idx=None, g_idx_down=None) -> torch.Tensor:
	"""down(fp16(silu(gate(x)) * up(x))) with fp32 accumulation everywhere and the
	single fp16 rounding of the intermediate that the fused module performs
	(fused_mlp.py:78-79).  Returns fp32."""
	h = gateup_silu_r32(x, gate, up, groupsize, g_idx).half()
	return qmatmul_r32(h, down[0], down[1], down[2], groupsize, g_idx_down)


# ----------------------------------------------------------------------------
# rotary embedding and the fused attention block
# ----------------------------------------------------------------------------

def rope_tables(head_dim: int, max_pos: int, theta: float = 10000.0, dtype=torch.float16) -> Tuple[torch.Tensor, torch.Tensor]:
	"""cos / sin tables [max_pos, head_dim] in the rotate-half convention used by
	HF LLaMA: inv_freq over even dims, angles for the two halves concatenated,
	computed in fp32 and cast to the activation dtype."""
	inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
	t = torch.arange(max_pos, dtype=torch.float32)
	freqs = torch.outer(t, inv_freq)
	emb = torch.cat([freqs, freqs], dim=-1)
	return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
	h = x.shape[-1] // 2
	return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, position_ids: torch.Tensor):
	"""q, k: [b, h, t, d]; cos/sin: [max_pos, d]; position_ids: [b, t].
	out = x*cos + rotate_half(x)*sin, evaluated in the dtype of q
	(the call at fused_attention.py:101-102)."""
	c = cos[position_ids].unsqueeze(1).to(q.dtype)
	s = sin[position_ids].unsqueeze(1).to(q.dtype)
	return q * c + rotate_half(q) * s, k * c + rotate_half(k) * s


def qkv_rope_r32(x, qweight, qzeros, scales, groupsize, cos, sin, position_ids, n_heads: int, head_dim: int, g_idx=None):
	"""Fused QKV projection followed by rotary embedding on Q and K, all in fp32
	from the fp32 accumulator (fp16 cos/sin tables are used at their fp16 values).
	x: [b, t, hidden].  Returns q, k, v as fp32 [b, t, n_heads, head_dim]."""
	b, t, _ = x.shape
	hidden = n_heads * head_dim
	y = qmatmul_r32(x, qweight, qzeros, scales, groupsize, g_idx).view(b, t, 3, n_heads, head_dim)
	q, k, v = y[:, :, 0], y[:, :, 1], y[:, :, 2]
	c = cos[position_ids].float().unsqueeze(2)    # [b, t, 1, d]
	s = sin[position_ids].float().unsqueeze(2)
	q = q * c + rotate_half(q) * s
	k = k * c + rotate_half(k) * s
	return q, k, v


def attention_block_r16(hidden_states, qkv, o, groupsize, cos, sin, position_ids, n_heads: int,
						attention_mask=None, past_key_value=None, use_cache=False, g_idx_qkv=None, g_idx_o=None):
	"""Restatement of QuantLlamaAttention.forward (fused_attention.py:79-153) in
	its own precision: fp16 projections, fp16 rotary, fp32 softmax."""
	bsz, q_len, hidden = hidden_states.shape
	head_dim = hidden // n_heads
	qkv_states = qmatmul_r16(hidden_states, qkv[0], qkv[1], qkv[2], groupsize, g_idx_qkv).view(bsz, q_len, 3 * hidden)
	q, k, v = torch.split(qkv_states, hidden, dim=2)
	q = q.view(bsz, q_len, n_heads, head_dim).transpose(1, 2)
	k = k.view(bsz, q_len, n_heads, head_dim).transpose(1, 2)
	v = v.view(bsz, q_len, n_heads, head_dim).transpose(1, 2)
	q, k = apply_rope(q, k, cos, sin, position_ids)
	if past_key_value is not None:
		k = torch.cat([past_key_value[0], k], dim=2)
		v = torch.cat([past_key_value[1], v], dim=2)
	present = (k.contiguous(), v.contiguous()) if use_cache else None
	w = torch.matmul(q.float(), k.float().transpose(2, 3)) / math.sqrt(head_dim)
	w = w.half()
	if attention_mask is not None:
		w = w + attention_mask
		w = torch.max(w, torch.tensor(torch.finfo(w.dtype).min))
	w = torch.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
	a = torch.matmul(w.float(), v.float()).half()
	a = a.transpose(1, 2).reshape(bsz, q_len, hidden)
	out = qmatmul_r16(a, o[0], o[1], o[2], groupsize, g_idx_o).view(bsz, q_len, hidden)
	return out, present


# ----------------------------------------------------------------------------
# round-to-nearest quantiser + packer (fixture generator of the reference)
# ----------------------------------------------------------------------------

def rtn_find_params(W: torch.Tensor, maxq: int = 15):
	"""Per-row asymmetric min/max parameters (gptq.py:205-246 with
	perchannel=True, sym=False, mse=False).  W: [N, cols]."""
	zero_t = torch.zeros(W.shape[0])
	xmin = torch.minimum(W.min(1)[0], zero_t)
	xmax = torch.maximum(W.max(1)[0], zero_t)
	both = (xmin == 0) & (xmax == 0)
	xmin[both] = -1
	xmax[both] = +1
	scale = (xmax - xmin) / maxq
	zero = torch.round(-xmin / scale)
	return scale, zero


def rtn_quantize(weight: torch.Tensor, groupsize: int):
	"""Restatement of `dumbquant` (quantize.py:294-329) for 4 bits.
	weight: [N, K] (nn.Linear layout).  Returns (fakequant [N,K] fp32,
	scale [N,G] fp32, zero [N,G] fp32)."""
	W = weight.detach().float().clone()
	N, K = W.shape
	gs = K if groupsize == -1 else groupsize
	scales, zeros = [], []
	out = torch.empty_like(W)
	for g0 in range(0, K, gs):
		blk = W[:, g0:g0 + gs]
		s, z = rtn_find_params(blk)
		q = torch.clamp(torch.round(blk / s[:, None]) + z[:, None], 0, 15)   # gptq.py:174-178
		out[:, g0:g0 + gs] = s[:, None] * (q - z[:, None])
		scales.append(s[:, None])
		zeros.append(z[:, None])
	return out, torch.cat(scales, 1), torch.cat(zeros, 1)


def pack_linear(fakequant: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, groupsize: int):
	"""Restatement of `pack_linear` (quantize.py:236-291): recover the integers
	from the fake-quantised weights and pack.  fakequant [N,K]; scale, zero [N,G].
	Returns (qweight int32 [K/8,N], qzeros int32 [G,N/8], scales fp16 [G,N])."""
	N, K = fakequant.shape
	gs = K if groupsize == -1 else groupsize
	s = scale.t().contiguous().float()   # [G, N]
	z = zero.t().contiguous().float()
	sz = z * s
	g = torch.arange(K) // gs
	# q[:, k] = round((w[:, k] + scale_zeros[g]) / scales[g])
	q = torch.round((fakequant.float().t() + sz[g]) / s[g]).to(torch.int32)   # [K, N]
	qweight = pack_qweight(q.numpy().astype(np.uint32) & 0xF)
	qzeros = pack_qzeros((z - 1).to(torch.int32).numpy().astype(np.uint32) & 0xF)
	return torch.from_numpy(qweight.copy()), torch.from_numpy(qzeros.copy()), s.half()


# ----------------------------------------------------------------------------
# error metrics used by the parity tests
# ----------------------------------------------------------------------------

def max_rel_err(y: torch.Tensor, ref32: torch.Tensor) -> float:
	"""max|y - ref| / max|ref| per output tensor: the normalisation under which
	the 2e-3 bound is stated (element-wise relative error is meaningless where
	cancellation makes the reference output small)."""
	ref32 = ref32.double().reshape(-1)
	d = (y.detach().cpu().double().reshape(-1) - ref32).abs().max().item()
	return d / max(ref32.abs().max().item(), 1e-30)
