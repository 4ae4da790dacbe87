"""Fused QKV projection + rotary embedding, and the quantised LLaMA attention block.

Mirrors src/gptq_triton/fused_attention.py of the reference: `make_quant_attn` (:10-45)
concatenates the q/k/v packed tensors along N into one QuantLinear, `QuantLlamaAttention`
(:48-153) runs one QKV matmul, rotary embedding, the KV-cache append, softmax attention
and o_proj.  Here the rotary embedding is applied inside the QKV kernel's epilogue, which
also scatters Q/K/V to [b, h, t, d] (or K/V straight into a static cache).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from .quant_linear import QuantLinear


def rope_tables(head_dim: int, max_pos: int, theta: float = 10000.0, device=None, dtype=torch.float16):
	"""cos/sin [max_pos, head_dim], rotate-half convention, computed in fp32 and cast to the
	activation dtype as the HF rotary module does."""
	inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
	t = torch.arange(max_pos, dtype=torch.float32, device=device)
	freqs = torch.outer(t, inv_freq)
	emb = torch.cat([freqs, freqs], dim=-1)
	return emb.cos().to(dtype).contiguous(), emb.sin().to(dtype).contiguous()


def qkv_rope(groupsize: int, a: torch.Tensor, qweight, scales, qzeros, cos, sin, position_ids, n_heads: int, head_dim: int,
			 perm: Optional[torch.Tensor] = None, kv_cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
			 rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6, sumsq_in: Optional[torch.Tensor] = None):
	"""One kernel: a x deq(Wqkv), rotary on Q and K, scatter to heads.

	a: [b, t, K] fp16 contiguous; position_ids: [b, t] integer.
	Without kv_cache returns (q, k, v) each [b, n_heads, t, head_dim] (k, v freshly allocated).
	With kv_cache = (K, V) each [b, n_heads, max_seq, head_dim] contiguous, K/V rows are written
	in place at their positions and (q, K, V) is returned.
	With rms_weight the input is RMS-normalised first: inside the decode kernel when `sumsq_in`
	(fp32 [M, K // 32], left by the projection that produced `a`) is given and the shape allows,
	else by the RMSNorm kernel.
	"""
	assert a.dim() == 3 and a.is_contiguous(), "A must be [b, t, K] and contiguous"
	assert a.shape[-1] == qweight.shape[0] * 8
	_lib.require_cuda(a, qweight, scales, qzeros, cos, sin, position_ids, perm)
	b, t, K = a.shape
	M = b * t
	hidden = n_heads * head_dim
	assert qweight.shape[1] == 3 * hidden
	pos = position_ids.reshape(-1).to(torch.int32).contiguous()
	assert pos.numel() == M
	# Q is written as [b, t, h, d]; the [b, h, t, d] view is returned
	q = torch.empty((b, t, n_heads, head_dim), device=a.device, dtype=torch.float16)
	if kv_cache is None:
		k = torch.empty((b, n_heads, t, head_dim), device=a.device, dtype=torch.float16)
		v = torch.empty_like(k)
		sb, st, sh, sp = n_heads * t * head_dim, head_dim, t * head_dim, 0
	else:
		k, v = kv_cache
		assert k.is_contiguous() and v.is_contiguous() and k.shape == v.shape and k.shape[0] >= b and k.shape[1] == n_heads and k.shape[3] == head_dim
		S = k.shape[2]
		sb, st, sh, sp = n_heads * S * head_dim, 0, S * head_dim, head_dim
	from .quant_linear import DECODE_MAX_M, dequant_matmul, prefill_kernel_available, rms_fusable
	max_pos = min(cos.shape[0], (kv_cache[0].shape[2] if kv_cache is not None else cos.shape[0]))
	if rms_weight is not None and sumsq_in is not None and rms_fusable(M, K, None, perm):
		assert sumsq_in.dtype == torch.float32 and sumsq_in.is_contiguous() and sumsq_in.numel() >= M * (K // 32)
		ws = _lib.workspace(a.device, M, K, 3 * hidden)
		rc = _lib.lib().gptq_qkv_rope_rms(
			_lib.ptr(a), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), None, None,
			_lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), max_pos, _lib.ptr(q), hidden, _lib.ptr(k), _lib.ptr(v), t, sb, st, sh, sp,
			M, K, n_heads, head_dim, groupsize, K, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device),
			_lib.ptr(rms_weight), _lib.ptr(sumsq_in), K // 32, float(rms_eps))
		_lib.check(rc, 'gptq_qkv_rope_rms')
		return q.transpose(1, 2), k, v
	if rms_weight is not None:
		a = rmsnorm(a, rms_weight, rms_eps)          # the norm runs as its own kernel
	if M > DECODE_MAX_M and perm is not None and prefill_kernel_available(M, K, 3 * hidden, groupsize):
		a = a.view(M, K)[:, perm.long()].contiguous().view(b, t, K)
		perm = None
	if M > DECODE_MAX_M and not prefill_kernel_available(M, K, 3 * hidden, groupsize):
		y = dequant_matmul(a.view(M, K), groupsize, qweight, scales, qzeros, None, perm).float().view(b, t, 3, n_heads, head_dim)
		c = cos[pos.long()].float().view(b, t, 1, head_dim)
		s = sin[pos.long()].float().view(b, t, 1, head_dim)
		rot = lambda z: torch.cat([-z[..., head_dim // 2:], z[..., :head_dim // 2]], dim=-1)
		qf, kf, vf = y[:, :, 0], y[:, :, 1], y[:, :, 2]
		qf = qf * c + rot(qf) * s
		kf = kf * c + rot(kf) * s
		q.copy_(qf.half())
		if kv_cache is None:
			k.copy_(kf.half().transpose(1, 2))
			v.copy_(vf.half().transpose(1, 2))
		else:
			bi = torch.arange(b, device=a.device).view(b, 1).expand(b, t)
			k[bi, :, pos.view(b, t).long()] = kf.half()
			v[bi, :, pos.view(b, t).long()] = vf.half()
		return q.transpose(1, 2), k, v
	ws = _lib.workspace(a.device, M, K, 3 * hidden)
	rc = _lib.lib().gptq_qkv_rope(
		_lib.ptr(a), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), None, _lib.ptr(perm),
		_lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), max_pos, _lib.ptr(q), hidden, _lib.ptr(k), _lib.ptr(v), t, sb, st, sh, sp,
		M, K, n_heads, head_dim, groupsize, K, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device))
	_lib.check(rc, 'gptq_qkv_rope')
	return q.transpose(1, 2), k, v


def _is_llama_attention(m) -> bool:
	return (not isinstance(m, QuantLlamaAttention)
			and all(isinstance(getattr(m, n, None), QuantLinear) for n in ('q_proj', 'k_proj', 'v_proj', 'o_proj')))


def make_quant_attn(model):
	"""Replace every LLaMA attention module (one that owns quantised q/k/v/o projections) by
	QuantLlamaAttention with the three projections fused (reference: fused_attention.py:10-45)."""
	for name, m in list(model.named_modules()):
		if not _is_llama_attention(m):
			continue
		q_proj, k_proj, v_proj = m.q_proj, m.k_proj, m.v_proj
		qweights = torch.cat([q_proj.qweight, k_proj.qweight, v_proj.qweight], dim=1)
		qzeros = torch.cat([q_proj.qzeros, k_proj.qzeros, v_proj.qzeros], dim=1)
		scales = torch.cat([q_proj.scales, k_proj.scales, v_proj.scales], dim=1)
		qkv_layer = QuantLinear(q_proj.bits, q_proj.groupsize, q_proj.infeatures,
								q_proj.outfeatures + k_proj.outfeatures + v_proj.outfeatures, bias=False)
		qkv_layer.qweight = qweights
		qkv_layer.qzeros = qzeros
		qkv_layer.scales = scales
		qkv_layer.bias = None
		gs = [p.g_idx for p in (q_proj, k_proj, v_proj)]
		if any(g is not None for g in gs):
			if any(g is None for g in gs) or not (torch.equal(gs[0], gs[1]) and torch.equal(gs[0], gs[2])):
				raise ValueError('q_proj, k_proj and v_proj must share one g_idx to be fused')
			qkv_layer.set_g_idx(gs[0])
		attn = QuantLlamaAttention(m.config, qkv_layer, m.o_proj, getattr(m, 'rotary_emb', None))
		if '.' in name:
			parent_name, child_name = name.rsplit('.', 1)
			parent = model.get_submodule(parent_name)
		else:
			parent, child_name = model, name
		setattr(parent, child_name, attn)


class QuantLlamaAttention(nn.Module):
	"""LLaMA attention with fused QKV + rotary (reference: fused_attention.py:48-153).
	`rotary_emb` is accepted for signature compatibility; the cos/sin tables are built from
	the config (rope theta, max positions) in the module's dtype."""

	def __init__(self, config, qkv_proj, o_proj, rotary_emb=None):
		super().__init__()
		self.config = config
		self.hidden_size = config.hidden_size
		self.head_dim = getattr(config, 'head_dim', None) or self.hidden_size // config.num_attention_heads
		self.max_position_embeddings = config.max_position_embeddings
		if (self.head_dim * config.num_attention_heads) != self.hidden_size:
			raise ValueError(
				f"hidden_size must be divisible by num_heads (got `hidden_size`: {self.hidden_size}"
				f" and `num_heads`: {config.num_attention_heads}).")
		# heads held by THIS module: all of them, or this rank's share under tensor parallelism
		self.num_heads = qkv_proj.outfeatures // (3 * self.head_dim)
		self.qkv_proj = qkv_proj
		self.o_proj = o_proj
		self.rotary_emb = rotary_emb
		self.rope_theta = float(getattr(config, 'rope_theta', 10000.0) or 10000.0)
		self._tables = None

	def _apply(self, fn, recurse=True):
		self._tables = None
		return super()._apply(fn, recurse)

	def tables(self, device, need: int):
		if self._tables is None or self._tables[0].device != device or self._tables[0].shape[0] < need:
			n = max(need, self.max_position_embeddings)
			self._tables = rope_tables(self.head_dim, n, self.rope_theta, device=device)
		return self._tables

	def project_qkv(self, hidden_states, position_ids, kv_cache=None, rms_weight=None, rms_eps=1e-6, sumsq_in=None, need_positions: int = 0):
		"""`need_positions`: rows the rotary tables must have when there is no static cache (past + new tokens);
		like the reference's rotary cache (fused_attention.py:101) the tables grow beyond max_position_embeddings."""
		qw, g_idx, perm = self.qkv_proj.kernel_operands()
		if g_idx is not None:
			raise NotImplementedError('fused QKV needs act-order groups of equal size')
		bsz, q_len, _ = hidden_states.shape
		if position_ids is None:
			position_ids = torch.arange(q_len, device=hidden_states.device).unsqueeze(0).expand(bsz, q_len)
		need = max(need_positions, q_len) if kv_cache is None else kv_cache[0].shape[2]      # a static cache fixes the position range
		cos, sin = self.tables(hidden_states.device, need)
		return qkv_rope(self.qkv_proj.groupsize, hidden_states, qw, self.qkv_proj.scales, self.qkv_proj.qzeros, cos, sin,
						position_ids, self.num_heads, self.head_dim, perm=perm, kv_cache=kv_cache, rms_weight=rms_weight, rms_eps=rms_eps,
						sumsq_in=sumsq_in)

	def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
				position_ids: Optional[torch.LongTensor] = None, past_key_value: Optional[Tuple[torch.Tensor]] = None,
				output_attentions: bool = False, use_cache: bool = False
				) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[Tuple[torch.Tensor]]]:
		"""Input shape: Batch x Time x Channel.  Same contract as the reference forward
		(fused_attention.py:79-153): returns (attn_output, attn_weights or None, (K, V) or None)."""
		bsz, q_len, _ = hidden_states.size()
		hidden_states = hidden_states.contiguous()
		past = 0 if past_key_value is None else past_key_value[0].shape[-2]
		if position_ids is None:
			position_ids = torch.arange(past, past + q_len, device=hidden_states.device).unsqueeze(0).expand(bsz, q_len)
		query_states, key_states, value_states = self.project_qkv(hidden_states, position_ids, need_positions=past + q_len)
		if past_key_value is not None:
			key_states = torch.cat([past_key_value[0], key_states], dim=2)
			value_states = torch.cat([past_key_value[1], value_states], dim=2)
		kv_seq_len = key_states.shape[-2]
		past_key_value = (key_states, value_states) if use_cache else None

		attn_weights = None
		if output_attentions:
			attn_weights = torch.matmul(query_states, key_states.transpose(2, 3)) / math.sqrt(self.head_dim)
			if attention_mask is not None:
				if attention_mask.size() != (bsz, 1, q_len, kv_seq_len):
					raise ValueError(f"Attention mask should be of size {(bsz, 1, q_len, kv_seq_len)}, but is {attention_mask.size()}")
				attn_weights = attn_weights + attention_mask
				attn_weights = torch.max(attn_weights, torch.tensor(torch.finfo(attn_weights.dtype).min, device=attn_weights.device))
			attn_weights = nn.functional.softmax(attn_weights, dim=-1, dtype=torch.float32).to(query_states.dtype)
			attn_output = torch.matmul(attn_weights, value_states)
		else:
			if attention_mask is not None and attention_mask.size() != (bsz, 1, q_len, kv_seq_len):
				raise ValueError(f"Attention mask should be of size {(bsz, 1, q_len, kv_seq_len)}, but is {attention_mask.size()}")
			attn_output = nn.functional.scaled_dot_product_attention(query_states, key_states, value_states, attn_mask=attention_mask)

		attn_output = attn_output.transpose(1, 2).reshape(bsz, q_len, self.num_heads * self.head_dim)
		attn_output = self.o_proj(attn_output)
		return attn_output, attn_weights, past_key_value


def qkv_attn_supported(K: int, n_heads: int, head_dim: int, groupsize: int) -> bool:
	"""True when one sequence's decode step can run QKV projection + rotary + cache append + attention as one kernel."""
	return bool(_lib.lib().gptq_qkv_attn_supported(K, n_heads, head_dim, groupsize))


def qkv_attn_decode(groupsize: int, a: torch.Tensor, qweight, scales, qzeros, cos, sin, pos: torch.Tensor, kcache: torch.Tensor,
					vcache: torch.Tensor, n_heads: int, rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
					sumsq_in: Optional[torch.Tensor] = None) -> torch.Tensor:
	"""One sequence, one new token: attention output [1, 1, n_heads * 128] from the hidden state `a` [1, 1, K].

	One kernel does what QuantLlamaAttention.forward does up to o_proj (fused_attention.py:79-146 of the reference):
	a x deq(Wqkv), rotary on q and k, K / V row written to the static cache at `pos`, softmax(q K^T / sqrt(d)) V over
	positions 0..pos.  A cluster of 8 CTAs per head splits the K dimension of the projection and the keys of the
	attention, and exchanges q / k / v and the softmax partials through distributed shared memory.
	With rms_weight, `a` is RMS-normalised inside the kernel from `sumsq_in` (fp32 [K // 32], left by the projection
	that produced `a`).  pos: int32 [1] on the device.
	"""
	_lib.require_cuda(a, qweight, scales, qzeros, cos, sin, pos, kcache, vcache)
	K = a.shape[-1]
	assert a.numel() == K and a.is_contiguous() and a.dtype == torch.float16
	assert pos.dtype == torch.int32 and pos.numel() == 1
	assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape == vcache.shape and kcache.shape[-3] == n_heads and kcache.shape[-1] == 128
	S = kcache.shape[-2]
	assert (rms_weight is None) == (sumsq_in is None)
	if sumsq_in is not None:
		assert sumsq_in.dtype == torch.float32 and sumsq_in.is_contiguous() and sumsq_in.numel() >= K // 32
	out = torch.empty((1, 1, n_heads * 128), dtype=torch.float16, device=a.device)
	ws = _lib.workspace(a.device, 1, K, 3 * n_heads * 128)
	rc = _lib.lib().gptq_qkv_attn_decode(
		_lib.ptr(a), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), min(cos.shape[0], S),
		_lib.ptr(kcache), _lib.ptr(vcache), S * 128, _lib.ptr(out), K, n_heads, 128, groupsize, 1.0 / math.sqrt(128),
		_lib.ptr(rms_weight) if rms_weight is not None else None, _lib.ptr(sumsq_in) if sumsq_in is not None else None, K // 32, float(rms_eps),
		_lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device))
	_lib.check(rc, 'gptq_qkv_attn_decode')
	return out


def qkv_attn_oproj_decode(groupsize: int, a: torch.Tensor, qweight, scales, qzeros, cos, sin, pos: torch.Tensor, kcache: torch.Tensor,
						  vcache: torch.Tensor, n_heads: int, o_groupsize: int, o_qweight, o_scales, o_qzeros, scratch: torch.Tensor,
						  residual: Optional[torch.Tensor] = None, sumsq_out: Optional[torch.Tensor] = None,
						  rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6, sumsq_in: Optional[torch.Tensor] = None,
						  attn_out: Optional[torch.Tensor] = None, ar=None) -> torch.Tensor:
	"""qkv_attn_decode + o_proj + residual add in the same kernel: returns residual + attention(a) x deq(Wo) as [1, 1, o_N].

	The whole attention block of a decoder layer for one new token of one sequence (fused_attention.py:79-153 of the
	reference plus the residual add around it).  `scratch`: uint8 tensor of gptq_qkv_attn_oproj_scratch_bytes, zeroed once,
	private to this call site; `sumsq_out`: fp32 [o_N // 32] receives the sums of squares of the result per 32 columns.
	`ar` (tp.PeerExchange sized for o_N): this call is one rank's share (its heads, its row shard of o_proj); the
	all-reduce over the ranks runs inside the kernel and every rank gets residual + the sum.
	"""
	_lib.require_cuda(a, qweight, scales, qzeros, cos, sin, pos, kcache, vcache, o_qweight, o_scales, o_qzeros, scratch, residual)
	K = a.shape[-1]
	o_N = o_qweight.shape[1]
	assert a.numel() == K and a.is_contiguous() and a.dtype == torch.float16
	assert pos.dtype == torch.int32 and pos.numel() == 1
	assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape == vcache.shape and kcache.shape[-3] == n_heads and kcache.shape[-1] == 128
	assert o_qweight.shape[0] * 8 == n_heads * 128
	assert (rms_weight is None) == (sumsq_in is None)
	assert ar is None or o_N % 128 == 0
	if residual is not None:
		assert residual.numel() == o_N and residual.is_contiguous() and residual.dtype == torch.float16
	if sumsq_out is not None:
		assert sumsq_out.dtype == torch.float32 and sumsq_out.is_contiguous() and sumsq_out.numel() >= o_N // 32
	S = kcache.shape[-2]
	y = torch.empty((1, 1, o_N), dtype=torch.float16, device=a.device)
	ws = _lib.workspace(a.device, 1, K, 3 * n_heads * 128)
	P = _lib.ptr
	opt = lambda t: P(t) if t is not None else None
	args = (P(a), P(qweight), P(qzeros), P(scales), P(cos), P(sin), P(pos), min(cos.shape[0], S), P(kcache), P(vcache), S * 128,
			K, n_heads, 128, groupsize, 1.0 / math.sqrt(128), opt(rms_weight), opt(sumsq_in), K // 32, float(rms_eps),
			P(o_qweight), P(o_qzeros), P(o_scales), o_N, o_groupsize, opt(residual), P(y), opt(sumsq_out), opt(attn_out),
			P(scratch), scratch.numel(), P(ws), ws.numel(), _lib.stream_ptr(a.device))
	if ar is not None:
		rc = _lib.lib().gptq_qkv_attn_oproj_decode_ar(*args, ar.world, ar.rank, ar.partials, ar.flags)
		_lib.check(rc, 'gptq_qkv_attn_oproj_decode_ar')
	else:
		rc = _lib.lib().gptq_qkv_attn_oproj_decode(*args)
		_lib.check(rc, 'gptq_qkv_attn_oproj_decode')
	return y


def qkv_attn_oproj_scratch(n_heads: int, o_N: int, device) -> torch.Tensor:
	"""Zeroed scratch area for qkv_attn_oproj_decode (arrival counters + per-head partial sums)."""
	return torch.zeros(_lib.lib().gptq_qkv_attn_oproj_scratch_bytes(n_heads, o_N), dtype=torch.uint8, device=device)


def attn_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: torch.Tensor, len_hint: int) -> torch.Tensor:
	"""Attention of one new token per sequence over a static cache.
	q [b, heads, 1, 128] or [b, 1, heads, 128] memory as produced by qkv_rope (any view whose
	(b, head) slices are 128 contiguous halfs with head stride 128); kcache/vcache [B, heads, S, 128]
	contiguous; pos int32 [b] or [b, 1].  Returns [b, 1, heads*128] fp16."""
	b = q.shape[0]
	heads, S, D = kcache.shape[1], kcache.shape[2], kcache.shape[3]
	_lib.require_cuda(q, kcache, vcache, pos)
	out = torch.empty((b, 1, heads * D), device=q.device, dtype=torch.float16)
	need = _lib.lib().gptq_attn_workspace_bytes(b, heads)
	ws = _lib.workspace(q.device, 1, 128, 128, min_bytes=need)
	rc = _lib.lib().gptq_attn_decode(_lib.ptr(q), heads * D, _lib.ptr(kcache), _lib.ptr(vcache), heads * S * D, S * D, _lib.ptr(pos),
									 _lib.ptr(out), heads * D, b, heads, D, int(len_hint), 1.0 / math.sqrt(D), _lib.ptr(ws), ws.numel(),
									 _lib.stream_ptr(q.device))
	_lib.check(rc, 'gptq_attn_decode')
	return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
	"""RMSNorm over the last dimension in one kernel (fp32 inside, one fp16 rounding)."""
	_lib.require_cuda(x, weight)
	assert x.is_contiguous() and x.dtype == torch.float16
	K = x.shape[-1]
	x2 = x.view(-1, K)
	y = torch.empty_like(x2)
	rc = _lib.lib().gptq_rmsnorm(_lib.ptr(x2), K, _lib.ptr(weight), _lib.ptr(y), K, x2.shape[0], K, float(eps), _lib.stream_ptr(x.device))
	_lib.check(rc, 'gptq_rmsnorm')
	return y.view(x.shape)
