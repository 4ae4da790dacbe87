"""A self-contained LLaMA decoder whose module tree and state-dict keys match the HF
LlamaForCausalLM that the reference builds in load_quant (src/gptq_triton/__init__.py:43-52),
so that make_quant / make_quant_attn / make_fused_mlp and reference checkpoints apply
unchanged, without depending on transformers internals.

Two ways to run it:
  * `forward(input_ids, past_key_values=..., use_cache=...)`: the reference-style path with
    concatenated (K, V) tuples per layer;
  * `DecodeEngine`: static KV cache written in place by the QKV kernel, residual adds fused
    into the o_proj / down_proj epilogues, greedy sampling on the device, the whole decode
    step captured in a CUDA graph.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fused_attention import (QuantLlamaAttention, attn_decode, qkv_attn_decode, qkv_attn_oproj_decode, qkv_attn_oproj_scratch,
							  qkv_attn_supported)
from .fused_attention import rmsnorm as rmsnorm_kernel
from .fused_mlp import QuantLlamaMLP
from .tp import all_reduce_


@dataclass
class LlamaConfig:
	hidden_size: int = 4096
	intermediate_size: int = 11008
	num_hidden_layers: int = 32
	num_attention_heads: int = 32
	vocab_size: int = 32000
	rms_norm_eps: float = 1e-6
	rope_theta: float = 10000.0
	max_position_embeddings: int = 2048

	@classmethod
	def from_json(cls, path):
		import json
		d = json.load(open(path))
		keys = cls.__dataclass_fields__.keys()
		return cls(**{k: d[k] for k in keys if k in d})

	@classmethod
	def llama_7b(cls):
		return cls()

	@classmethod
	def llama_65b(cls):
		return cls(hidden_size=8192, intermediate_size=22016, num_hidden_layers=80, num_attention_heads=64)


class LlamaRMSNorm(nn.Module):
	def __init__(self, hidden_size, eps=1e-6):
		super().__init__()
		self.weight = nn.Parameter(torch.ones(hidden_size))
		self.variance_epsilon = eps

	def forward(self, x):
		v = x.float().pow(2).mean(-1, keepdim=True)
		return self.weight * (x.float() * torch.rsqrt(v + self.variance_epsilon)).to(x.dtype)


class LlamaMLP(nn.Module):
	def __init__(self, config: LlamaConfig):
		super().__init__()
		self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
		self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)
		self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)

	def forward(self, x):
		return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class LlamaAttention(nn.Module):
	"""Unfused attention; only a container until make_quant_attn replaces it, but it also
	runs (fp16 nn.Linear or QuantLinear children) for comparisons."""

	def __init__(self, config: LlamaConfig):
		super().__init__()
		self.config = config
		h = config.hidden_size
		self.num_heads = config.num_attention_heads
		self.head_dim = h // self.num_heads
		self.q_proj = nn.Linear(h, h, bias=False)
		self.k_proj = nn.Linear(h, h, bias=False)
		self.v_proj = nn.Linear(h, h, bias=False)
		self.o_proj = nn.Linear(h, h, bias=False)
		self._tables = None

	def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False, use_cache=False):
		from .fused_attention import rope_tables
		b, t, h = hidden_states.shape
		q = self.q_proj(hidden_states).view(b, t, self.num_heads, self.head_dim).transpose(1, 2)
		k = self.k_proj(hidden_states).view(b, t, self.num_heads, self.head_dim).transpose(1, 2)
		v = self.v_proj(hidden_states).view(b, t, self.num_heads, self.head_dim).transpose(1, 2)
		# the tables cover every position in use: the cached ones plus the new tokens (they grow past
		# max_position_embeddings, as the rotary cache of the HF module does)
		need = (0 if past_key_value is None else past_key_value[0].shape[2]) + t
		if self._tables is None or self._tables[0].device != q.device or self._tables[0].shape[0] < need:
			self._tables = rope_tables(self.head_dim, max(need, self.config.max_position_embeddings), self.config.rope_theta, device=q.device, dtype=q.dtype)
		cos, sin = self._tables
		c, s = cos[position_ids].unsqueeze(1), sin[position_ids].unsqueeze(1)
		rot = lambda x: torch.cat([-x[..., x.shape[-1] // 2:], x[..., :x.shape[-1] // 2]], dim=-1)
		q, k = q * c + rot(q) * s, k * c + rot(k) * s
		if past_key_value is not None:
			k = torch.cat([past_key_value[0], k], dim=2)
			v = torch.cat([past_key_value[1], v], dim=2)
		present = (k, v) if use_cache else None
		o = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask)
		return self.o_proj(o.transpose(1, 2).reshape(b, t, h)), None, present


class LlamaDecoderLayer(nn.Module):
	def __init__(self, config: LlamaConfig):
		super().__init__()
		self.self_attn = LlamaAttention(config)
		self.mlp = LlamaMLP(config)
		self.input_layernorm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)
		self.post_attention_layernorm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)

	def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, use_cache=False):
		r = hidden_states
		a, _, present = self.self_attn(self.input_layernorm(hidden_states), attention_mask=attention_mask, position_ids=position_ids,
									   past_key_value=past_key_value, use_cache=use_cache)
		hidden_states = r + a
		hidden_states = hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))
		return hidden_states, present


class LlamaModel(nn.Module):
	def __init__(self, config: LlamaConfig):
		super().__init__()
		self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
		self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
		self.norm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)


def causal_mask(t: int, past: int, device, dtype=torch.float16):
	m = torch.full((t, past + t), float('-inf'), device=device, dtype=dtype)
	m = torch.triu(m, diagonal=past + 1)
	return m[None, None]


class LlamaForCausalLM(nn.Module):
	def __init__(self, config: LlamaConfig):
		super().__init__()
		self.config = config
		self.model = LlamaModel(config)
		self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

	@torch.no_grad()
	def forward(self, input_ids, past_key_values: Optional[List[Tuple[torch.Tensor, torch.Tensor]]] = None, use_cache: bool = False):
		b, t = input_ids.shape
		past = 0 if past_key_values is None else past_key_values[0][0].shape[2]
		pos = torch.arange(past, past + t, device=input_ids.device).unsqueeze(0).expand(b, t)
		mask = causal_mask(t, past, input_ids.device) if t > 1 else None
		h = self.model.embed_tokens(input_ids)
		presents = []
		for i, layer in enumerate(self.model.layers):
			h, present = layer(h, attention_mask=mask, position_ids=pos,
							   past_key_value=None if past_key_values is None else past_key_values[i], use_cache=use_cache)
			presents.append(present)
		logits = self.lm_head(self.model.norm(h))
		return logits, (presents if use_cache else None)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
	v = x.float().pow(2).mean(-1, keepdim=True)
	return (x.float() * torch.rsqrt(v + eps)).to(x.dtype) * weight


class DecodeEngine:
	"""Greedy decoding with a static KV cache for a model whose attention and MLP blocks have
	been fused (QuantLlamaAttention / QuantLlamaMLP).  One decode step = 32 x (RMSNorm, fused
	QKV+rotary writing K/V into the cache, attention over the cache, o_proj + residual, RMSNorm,
	fused gate/up, down_proj + residual), final norm, fp16 lm_head, argmax."""

	def __init__(self, model: LlamaForCausalLM, batch: int, max_seq: int, use_graph: bool = True, tp_group=None):
		self.model = model
		# tensor parallelism: the model holds this rank's shards (tp.shard_llama); partial sums of the
		# row-parallel projections are all-reduced, the residual is added on rank 0 only
		self.tp_group = tp_group
		self.tp_rank = getattr(model, 'tp_rank', 0)
		self.tp_world = getattr(model, 'tp_world', 1)
		cfg = model.config
		self.cfg = cfg
		dev = model.lm_head.weight.device
		self.device = dev
		self.batch, self.max_seq = batch, max_seq
		for layer in model.model.layers:
			assert isinstance(layer.self_attn, QuantLlamaAttention), 'run make_quant_attn first'
		H, D = model.model.layers[0].self_attn.num_heads, cfg.hidden_size // cfg.num_attention_heads      # local heads
		self.kcache = [torch.zeros((batch, H, max_seq, D), dtype=torch.float16, device=dev) for _ in model.model.layers]
		self.vcache = [torch.zeros((batch, H, max_seq, D), dtype=torch.float16, device=dev) for _ in model.model.layers]
		self.pos = torch.zeros((batch, 1), dtype=torch.int32, device=dev)          # position of the token being fed
		self.tok = torch.zeros((batch, 1), dtype=torch.int64, device=dev)          # token being fed
		self.mask = torch.full((batch, 1, 1, max_seq), float('-inf'), dtype=torch.float16, device=dev)
		# tensor parallelism, decode steps: the all-reduce after o_proj / down_proj is fused into those kernels
		# over peer memory (one exchange buffer per projection); GPTQ_B200_TP_FUSED=0 keeps NCCL
		self.ar_o = self.ar_down = None
		# (row shards of act-order layers look their groups up per row and run on the general kernel, which has no
		# fused exchange: those models use NCCL)
		plain_rows = all(l.self_attn.o_proj.kernel_operands()[1] is None and
						 (not isinstance(l.mlp, QuantLlamaMLP) or l.mlp.down_proj.kernel_operands()[1] is None) for l in model.model.layers)
		if self.tp_world > 1 and batch <= 16 and cfg.hidden_size % 128 == 0 and plain_rows and os.environ.get('GPTQ_B200_TP_FUSED', '1') != '0':
			from .tp import PeerExchange
			try:          # collective: fails on every rank or on none
				self.ar_o = PeerExchange(cfg.hidden_size, self.tp_rank, self.tp_world, tp_group)
				self.ar_down = PeerExchange(cfg.hidden_size, self.tp_rank, self.tp_world, tp_group)
			except RuntimeError:
				if self.ar_o is not None:
					self.ar_o.close()
				self.ar_o = self.ar_down = None          # NCCL all-reduce instead
		self.use_graph = use_graph
		# RMSNorm folded into the decode kernels: o_proj / down_proj leave per-tile sums of squares of
		# the hidden state, the next QKV / gate-up kernel scales x while staging it (one GPU only)
		self.fuse_norm = True
		tiles = max(1, cfg.hidden_size // 32)
		self.ss_attn = torch.zeros((batch, tiles), dtype=torch.float32, device=dev)
		self.ss_mlp = torch.zeros((batch, tiles), dtype=torch.float32, device=dev)
		self.len_hint = max_seq
		self.graph = None
		self.launches_per_step = None
		self._qao_scratch = None
		# captures of the decode step to choose from (see step()); 1 = take the first
		self.graph_candidates = int(os.environ.get('GPTQ_B200_GRAPH_CANDIDATES', '6'))
		self.used_qkv_attn = False          # set when a decode step ran the one-kernel QKV + attention path
		self.used_fused_oproj = False       # ... with o_proj and the residual add in the same kernel
		self.next_pos = 0          # host-side copy of the position the next step() writes (the cache has max_seq rows)
		# One persistent kernel per decode step (gptq_decode_chain) + the lm_head / arg-max kernel, where the model
		# allows it (one GPU, batch <= 8, no act-order, no bias, one group size); opt-in with GPTQ_B200_CHAIN=1 (default: the
		# kernel-per-projection path).
		self.chain = None
		if os.environ.get('GPTQ_B200_CHAIN', '0') != '0':
			self.chain = self._chain_setup()

	def _chain_setup(self):
		"""Descriptors and scratch of the persistent decode-step kernel, or None when the model is not served by it."""
		import ctypes
		from . import _lib
		cfg, model, dev = self.cfg, self.model, self.device
		if self.tp_world != 1 or not (1 <= self.batch <= 8):
			return None
		layers = model.model.layers
		heads = cfg.num_attention_heads
		gs = None
		rows = []
		for i, layer in enumerate(layers):
			attn, mlp = layer.self_attn, layer.mlp
			if not isinstance(mlp, QuantLlamaMLP) or attn.head_dim != 128 or attn.num_heads != heads:
				return None
			qkv_w, qkv_g, qkv_p = attn.qkv_proj.kernel_operands()
			o_w, o_g, o_p = attn.o_proj.kernel_operands()
			d_w, d_g, d_p = mlp.down_proj.kernel_operands()
			if not mlp._ao_ready:
				mlp._prepare()
			if any(v is not None for v in (qkv_g, qkv_p, o_g, o_p, d_g, d_p, mlp._perm, mlp._gidx)):
				return None          # act-order layers keep the kernel-per-projection path
			if any(m.bias is not None for m in (attn.qkv_proj, attn.o_proj, mlp.down_proj)):
				return None
			sizes = {attn.qkv_proj.groupsize, attn.o_proj.groupsize, mlp.groupsize, mlp.down_proj.groupsize}
			if len(sizes) != 1 or (gs is not None and gs not in sizes):
				return None
			gs = sizes.pop()
			if mlp.gate_proj_qweight.shape[1] != cfg.intermediate_size or qkv_w.shape[1] != 3 * cfg.hidden_size:
				return None
			rows.append(((qkv_w, o_w, mlp.gate_proj_qweight, mlp.up_proj_qweight, d_w),
						 (attn.qkv_proj.qzeros, attn.o_proj.qzeros, mlp.gate_proj_qzeros, mlp.up_proj_qzeros, mlp.down_proj.qzeros),
						 (attn.qkv_proj.scales, attn.o_proj.scales, mlp.gate_proj_scales, mlp.up_proj_scales, mlp.down_proj.scales),
						 layer.input_layernorm.weight, layer.post_attention_layernorm.weight, self.kcache[i], self.vcache[i]))
		L = _lib.lib()
		if gs is None or not L.gptq_chain_supported(self.batch, cfg.hidden_size, cfg.intermediate_size, heads, gs):
			return None
		if cfg.hidden_size % 256 != 0 or 8 * (cfg.hidden_size * 2 + 64) > 96 * 1024:
			return None

		class Layer(ctypes.Structure):
			_fields_ = [('qweight', ctypes.c_void_p * 5), ('qzeros', ctypes.c_void_p * 5), ('scales', ctypes.c_void_p * 5),
						('ln1', ctypes.c_void_p), ('ln2', ctypes.c_void_p), ('kcache', ctypes.c_void_p), ('vcache', ctypes.c_void_p)]
		arr = (Layer * len(rows))()
		for dst, (qw, qz, sc, ln1, ln2, kc, vc) in zip(arr, rows):
			for j in range(5):
				dst.qweight[j], dst.qzeros[j], dst.scales[j] = qw[j].data_ptr(), qz[j].data_ptr(), sc[j].data_ptr()
			dst.ln1, dst.ln2, dst.kcache, dst.vcache = ln1.data_ptr(), ln2.data_ptr(), kc.data_ptr(), vc.data_ptr()
		desc = torch.zeros(L.gptq_chain_desc_bytes(len(rows)), dtype=torch.uint8, device=dev)
		with torch.cuda.device(dev):
			_lib.check(L.gptq_chain_build(arr, len(rows), cfg.hidden_size, cfg.intermediate_size, _lib.ptr(desc)), 'gptq_chain_build')
		scratch = torch.zeros(L.gptq_chain_scratch_bytes(self.batch, cfg.hidden_size, cfg.intermediate_size, heads, gs), dtype=torch.uint8, device=dev)
		_lib.register_status_buffer(scratch)
		cos, sin = layers[0].self_attn.tables(dev, self.max_seq)
		return dict(desc=desc, scratch=scratch, groupsize=gs, cos=cos, sin=sin, keep=rows,
					h_out=torch.zeros((self.batch, cfg.hidden_size), dtype=torch.float16, device=dev),
					ss_out=torch.zeros((self.batch, cfg.hidden_size // 32), dtype=torch.float32, device=dev),
					logits=torch.zeros((self.batch, 1, cfg.vocab_size), dtype=torch.float16, device=dev),
					lm_ws=torch.zeros(L.gptq_lm_head_workspace_bytes(self.batch), dtype=torch.uint8, device=dev))

	def _chain_step_body(self):
		from . import _lib
		c, cfg, L = self.chain, self.cfg, _lib.lib()
		H, S, D = cfg.num_attention_heads, self.max_seq, 128
		st = _lib.stream_ptr(self.device)
		eps = float(self.model.model.norm.variance_epsilon)
		rc = L.gptq_decode_chain(_lib.ptr(c['desc']), cfg.num_hidden_layers, self.batch, cfg.hidden_size, cfg.intermediate_size, H, c['groupsize'],
								 _lib.ptr(self.model.model.embed_tokens.weight), _lib.ptr(self.tok), _lib.ptr(self.pos), _lib.ptr(c['cos']), _lib.ptr(c['sin']),
								 S, H * S * D, S * D, eps, _lib.ptr(c['h_out']), _lib.ptr(c['ss_out']), _lib.ptr(c['scratch']), c['scratch'].numel(), st)
		_lib.check(rc, 'gptq_decode_chain')
		rc = L.gptq_lm_head_argmax(_lib.ptr(c['h_out']), _lib.ptr(c['ss_out']), _lib.ptr(self.model.model.norm.weight), _lib.ptr(self.model.lm_head.weight),
								   self.batch, cfg.hidden_size, cfg.vocab_size, eps, _lib.ptr(c['logits']), _lib.ptr(self.tok), _lib.ptr(self.pos),
								   _lib.ptr(c['lm_ws']), c['lm_ws'].numel(), st)
		_lib.check(rc, 'gptq_lm_head_argmax')
		self.logits = c['logits']

	# -- one layer on hidden states h [b, t, hidden]; K/V go to the cache at `pos` --------------
	# ss_in: per-tile sums of squares of h left by the projection that produced it (decode steps
	# with the norms folded into the kernels); returns (h, ss of the new h or None).
	def _layer(self, i, h, pos, attn_mask, kv_len, ss_in=None, x_normed=None):
		"""x_normed: input_layernorm(h), when the caller has computed it already (first layer of a decode step)."""
		layer = self.model.model.layers[i]
		attn: QuantLlamaAttention = layer.self_attn
		decode = h.shape[1] == 1
		ln1, ln2 = layer.input_layernorm, layer.post_attention_layernorm
		b = h.shape[0]
		# tensor parallelism: with the all-reduce inside the projection kernels every rank holds the reduced
		# hidden state (and its sums of squares); with NCCL the norms stay separate kernels
		fused_ar = decode and self.ar_o is not None and b <= 16
		fold = self.fuse_norm and decode and (self.tp_world == 1 or fused_ar) and b <= 16 and self.cfg.hidden_size % 128 == 0 and self.cfg.hidden_size // 32 <= 256
		o = h_attn = None
		if decode and b == 1 and self.batch == 1 and self._one_kernel_attention(attn) and (x_normed is not None or (fold and ss_in is not None)):
			# one sequence: projection, rotary, cache append and attention in one kernel (a cluster of 8 CTAs per head)
			self.used_qkv_attn = True
			qw, _, _ = attn.qkv_proj.kernel_operands()
			cos, sin = attn.tables(h.device, self.max_seq)
			src = x_normed if x_normed is not None else h.contiguous()
			rms_w, rms_ss = (None, None) if x_normed is not None else (ln1.weight, ss_in)
			op = attn.o_proj
			if self._fused_oproj(attn):
				# ... and the output projection with the residual add as well: the whole attention block is one kernel
				self.used_fused_oproj = True
				if self._qao_scratch is None:
					self._qao_scratch = qkv_attn_oproj_scratch(attn.num_heads, op.outfeatures, h.device)
				h_attn = qkv_attn_oproj_decode(attn.qkv_proj.groupsize, src, qw, attn.qkv_proj.scales, attn.qkv_proj.qzeros, cos, sin, pos.view(-1),
											   self.kcache[i], self.vcache[i], attn.num_heads, op.groupsize, op.qweight, op.scales, op.qzeros,
											   self._qao_scratch, residual=h.contiguous(), sumsq_out=self.ss_attn, rms_weight=rms_w,
											   rms_eps=ln1.variance_epsilon, sumsq_in=rms_ss, ar=self.ar_o if self.tp_world > 1 else None)
				o = h_attn
			else:
				o = qkv_attn_decode(attn.qkv_proj.groupsize, src, qw, attn.qkv_proj.scales, attn.qkv_proj.qzeros, cos, sin, pos.view(-1), self.kcache[i],
									self.vcache[i], attn.num_heads, rms_weight=rms_w, rms_eps=ln1.variance_epsilon, sumsq_in=rms_ss)
		elif x_normed is not None:
			q, _, _ = attn.project_qkv(x_normed, pos, kv_cache=(self.kcache[i], self.vcache[i]))
		elif fold:
			q, _, _ = attn.project_qkv(h.contiguous(), pos, kv_cache=(self.kcache[i], self.vcache[i]), rms_weight=ln1.weight,
									   rms_eps=ln1.variance_epsilon, sumsq_in=ss_in)      # ss_in None (first layer): RMSNorm kernel
		else:
			x = rmsnorm_kernel(h.contiguous(), ln1.weight, ln1.variance_epsilon)
			q, _, _ = attn.project_qkv(x, pos, kv_cache=(self.kcache[i], self.vcache[i]))
		if o is not None:
			pass
		elif decode:
			# own single-query kernel over the static cache (length read from `pos` on the device)
			o = attn_decode(q, self.kcache[i], self.vcache[i], pos, self.len_hint)
		else:
			k = self.kcache[i][:b, :, :kv_len]
			v = self.vcache[i][:b, :, :kv_len]
			o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask)
			o = o.transpose(1, 2).reshape(b, h.shape[1], -1)      # local heads x head_dim
		mlp = layer.mlp
		fused_ar = fused_ar and isinstance(mlp, QuantLlamaMLP)
		res = h if (self.tp_rank == 0 or fused_ar) else None          # the fused exchange adds the residual on every rank
		fold_mlp = fold and isinstance(mlp, QuantLlamaMLP) and attn.o_proj.g_idx is None
		ar_o = self.ar_o if fused_ar else None
		if h_attn is not None:
			h = h_attn
		elif fold_mlp:
			h = attn.o_proj(o, residual=res, sumsq_out=self.ss_attn, ar=ar_o)
		else:
			h = attn.o_proj(o, residual=res, ar=ar_o)
		if self.tp_world > 1 and not fused_ar:
			all_reduce_(h, self.tp_group)
		res = h if (self.tp_rank == 0 or fused_ar) else None
		ss_out = None
		if fold_mlp:
			ss_out = self.ss_mlp if mlp.down_proj.g_idx is None else None
			h = mlp(h, residual=res, rms_weight=ln2.weight, rms_eps=ln2.variance_epsilon, sumsq_in=self.ss_attn, sumsq_out=ss_out,
					ar=self.ar_down if fused_ar else None)
		elif isinstance(mlp, QuantLlamaMLP):
			h = mlp(rmsnorm_kernel(h, ln2.weight, ln2.variance_epsilon), residual=res, ar=self.ar_down if fused_ar else None)
		else:
			x = rmsnorm_kernel(h, ln2.weight, ln2.variance_epsilon)
			h = mlp(x) if res is None else res + mlp(x)
		if self.tp_world > 1 and not fused_ar:
			all_reduce_(h, self.tp_group)
		return h, ss_out

	@torch.no_grad()
	def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
		"""Runs the prompt [b, t], fills the cache, returns the first generated token [b, 1]."""
		b, t = input_ids.shape
		assert b == self.batch and t < self.max_seq
		pos = torch.arange(t, device=self.device, dtype=torch.int32).unsqueeze(0).expand(b, t).contiguous()
		mask = causal_mask(t, 0, self.device)
		h = self.model.model.embed_tokens(input_ids)
		for i in range(len(self.model.model.layers)):
			h, _ = self._layer(i, h, pos, mask, t)
		h = rmsnorm(h[:, -1:, :], self.model.model.norm.weight, self.model.model.norm.variance_epsilon)
		logits = self.model.lm_head(h)
		self.logits = logits
		self.tok.copy_(logits.argmax(-1))
		self.pos.fill_(t)
		self.next_pos = t
		self.len_hint = t + 1
		self.mask.fill_(float('-inf'))
		self.mask[..., :t + 1] = 0
		return self.tok.clone()

	def _one_kernel_attention(self, attn) -> bool:
		"""Whether the layer's QKV projection and attention run as one kernel in a decode step of one sequence
		(plain group layout, no bias, head_dim 128, hidden a multiple of 1024; GPTQ_B200_QKV_ATTN=0 turns it off)."""
		if os.environ.get('GPTQ_B200_QKV_ATTN', '1') == '0':
			return False
		qp = attn.qkv_proj
		_, g_idx, perm = qp.kernel_operands()
		if g_idx is not None or perm is not None or qp.bias is not None or attn.head_dim != 128:
			return False
		return qkv_attn_supported(qp.infeatures, attn.num_heads, attn.head_dim, qp.groupsize)

	def _fused_oproj(self, attn) -> bool:
		"""Whether the one-kernel attention also does o_proj and the residual add (plain group layout, no bias, at most
		8192 outputs; under tensor parallelism with the all-reduce inside the kernel; GPTQ_B200_QKV_ATTN_O=0 turns it off)."""
		if os.environ.get('GPTQ_B200_QKV_ATTN_O', '1') == '0':
			return False
		if self.tp_world != 1 and (self.ar_o is None or attn.o_proj.outfeatures % 128 != 0 or os.environ.get('GPTQ_B200_QKV_ATTN_O_TP', '0') == '0'):
			# tensor parallel: needs the exchange buffers of the fused all-reduce; opt-in, because on 2 GPUs it is exactly as fast
			# as the attention kernel followed by o_proj with its own fused all-reduce (632 vs 631 tokens/s)
			return False
		op = attn.o_proj
		_, g_idx, perm = op.kernel_operands()
		return (g_idx is None and perm is None and op.bias is None and op.infeatures == attn.num_heads * 128 and op.outfeatures % 32 == 0
				and op.outfeatures <= 8192 and op.groupsize % 128 == 0 and op.infeatures % op.groupsize == 0)

	def _own_ends(self):
		"""Buffers for the first and last kernel of a decode step when both ends run as own kernels: embedding
		lookup + first RMSNorm in one kernel, final RMSNorm + lm_head + arg-max + position increment in one kernel
		(batch <= 8, hidden a multiple of 256); None otherwise."""
		if getattr(self, '_ends', False) is not False:
			return self._ends
		from . import _lib
		cfg, dev = self.cfg, self.device
		ok = 1 <= self.batch <= 8 and cfg.hidden_size % 256 == 0 and 8 * (cfg.hidden_size * 2 + 64) <= 96 * 1024 \
			and self.model.lm_head.bias is None and self.model.lm_head.weight.dtype == torch.float16
		self._ends = None
		if ok:
			L = _lib.lib()
			self._ends = dict(h0=torch.empty((self.batch, 1, cfg.hidden_size), dtype=torch.float16, device=dev),
							  x0=torch.empty((self.batch, 1, cfg.hidden_size), dtype=torch.float16, device=dev),
							  logits=torch.zeros((self.batch, 1, cfg.vocab_size), dtype=torch.float16, device=dev),
							  lm_ws=torch.zeros(L.gptq_lm_head_workspace_bytes(self.batch), dtype=torch.uint8, device=dev))
		return self._ends

	def _step_body(self):
		if self.chain is not None:
			return self._chain_step_body()
		from . import _lib
		m, cfg = self.model.model, self.cfg
		ends = self._own_ends()
		ss = None
		if ends is not None:
			# embedding row of the token and the first layer's input norm in one kernel
			ln = m.layers[0].input_layernorm
			rc = _lib.lib().gptq_embed_rmsnorm(_lib.ptr(m.embed_tokens.weight), cfg.hidden_size, cfg.vocab_size, _lib.ptr(self.tok), _lib.ptr(ln.weight),
											   _lib.ptr(ends['h0']), cfg.hidden_size, _lib.ptr(ends['x0']), cfg.hidden_size, self.batch, cfg.hidden_size,
											   float(ln.variance_epsilon), _lib.stream_ptr(self.device))
			_lib.check(rc, 'gptq_embed_rmsnorm')
			h = ends['h0']
			h, ss = self._layer(0, h, self.pos, self.mask, self.max_seq, None, x_normed=ends['x0'])
			rest = range(1, len(m.layers))
		else:
			h = m.embed_tokens(self.tok)
			rest = range(len(m.layers))
		for i in rest:
			h, ss = self._layer(i, h, self.pos, self.mask, self.max_seq, ss)
		eps = float(m.norm.variance_epsilon)
		if ends is not None and ss is not None:
			# final norm (from the sums of squares the last down_proj left), lm_head, arg-max, next token and position
			rc = _lib.lib().gptq_lm_head_argmax(_lib.ptr(h), _lib.ptr(ss), _lib.ptr(m.norm.weight), _lib.ptr(self.model.lm_head.weight), self.batch,
												cfg.hidden_size, cfg.vocab_size, eps, _lib.ptr(ends['logits']), _lib.ptr(self.tok), _lib.ptr(self.pos),
												_lib.ptr(ends['lm_ws']), ends['lm_ws'].numel(), _lib.stream_ptr(self.device))
			_lib.check(rc, 'gptq_lm_head_argmax')
			self.logits = ends['logits']
			return
		h = rmsnorm_kernel(h, m.norm.weight, eps)
		logits = self.model.lm_head(h)
		self.logits = logits
		nxt = logits.argmax(-1)
		# advance: next token, next position (the attention kernel reads the length from `pos`)
		self.tok.copy_(nxt)
		self.pos.add_(1)

	@torch.no_grad()
	def step(self) -> torch.Tensor:
		"""Feeds self.tok at self.pos, returns the next token [b, 1] (device tensor)."""
		if self.next_pos >= self.max_seq:
			raise RuntimeError(f'DecodeEngine: the static KV cache holds {self.max_seq} positions and is full; build the engine with a larger max_seq')
		self.next_pos += 1
		if not self.use_graph:
			self._step_body()
			return self.tok
		if self.graph is None:
			if self.ar_o is not None:
				# the fused exchange waits at most two seconds for a peer: start the ranks together
				import torch.distributed as dist
				torch.cuda.synchronize()
				dist.barrier(group=self.tp_group)
			# warm up on a side stream (allocations, workspaces), then capture
			saved = (self.tok.clone(), self.pos.clone(), self.mask.clone())
			s = torch.cuda.Stream()
			s.wait_stream(torch.cuda.current_stream())
			best, best_ms, best_logits = None, None, None
			with torch.cuda.stream(s):
				for _ in range(2):
					self._step_body()
					self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.mask.copy_(saved[2])
				s.synchronize()
				# The activations of a step live in the graph's private memory pool.  Where that pool lands (which physical
				# 2 MB page) decides how fast the few lines that every CTA reads right after a kernel boundary arrive: the same
				# graph replays 7 % faster or slower from one capture to the next (two modes, measured).  So the step is captured several
				# times, every candidate is timed on a few replays, and the fastest one is kept.  The replays write cache rows
				# at the current position onwards, which the real steps write again; token and position are restored.
				n_cand = max(1, self.graph_candidates)          # tensor parallel: every rank replays the same number of times, the choice is per rank
				alive = []          # every candidate keeps its pool until the choice is made: a freed pool would be handed to the next capture
				for _ in range(n_cand):
					g = torch.cuda.CUDAGraph()
					with torch.cuda.graph(g, stream=s):
						self._step_body()
					alive.append(g)
					cand_logits = self.logits          # the capture's own output tensor (it lives in that graph's pool)
					if n_cand == 1:
						best, best_logits = g, cand_logits
						break
					reps = max(1, min(8, self.max_seq - 1 - int(saved[1].max().item())))
					e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
					g.replay()
					e0.record(s)
					for _ in range(reps):
						self.tok.copy_(saved[0]); self.pos.copy_(saved[1])
						g.replay()
					e1.record(s)
					s.synchronize()
					ms = e0.elapsed_time(e1) / reps
					if best_ms is None or ms < best_ms:
						best, best_ms, best_logits = g, ms, cand_logits
				del alive
			torch.cuda.current_stream().wait_stream(s)
			# capture does not execute (and the timed replays started from the saved state): restore it
			self.tok.copy_(saved[0]); self.pos.copy_(saved[1]); self.mask.copy_(saved[2])
			self.graph = best
			self.logits = best_logits
		self.graph.replay()
		return self.tok

	@torch.no_grad()
	def generate(self, input_ids: torch.Tensor, steps: int) -> torch.Tensor:
		"""Greedy generation: returns [b, steps] token ids (the first comes from the prefill)."""
		from . import _lib
		out = [self.prefill(input_ids)]
		for _ in range(steps - 1):
			out.append(self.step().clone())
		toks = torch.cat(out, dim=1)
		# the kernels' bounded waits report through a status word instead of hanging: a non-zero word means
		# that some result of this run cannot be trusted
		status = _lib.kernel_status(self.device)
		if status != 0:
			raise _lib.GptqB200Error(f'a decode kernel reported status {status} (see _lib.kernel_status)')
		return toks

	def close(self):
		"""Releases the tensor-parallel exchange buffers (mapped by the peers: call it on every rank, after the
		last step has completed everywhere) and the captured graph."""
		self.graph = None
		for name in ('ar_o', 'ar_down'):
			ex = getattr(self, name, None)
			if ex is not None:
				ex.close()
				setattr(self, name, None)
