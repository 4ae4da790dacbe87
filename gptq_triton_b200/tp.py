"""Megatron-style tensor parallelism for the quantised LLaMA layer.

Not in the reference (it has no distributed code); layout follows the usual scheme:
  * column parallel (shard N, no communication): q/k/v by heads, gate/up by intermediate columns;
  * row parallel (shard K, partial sums): o_proj over the local heads' columns of the attention
    output, down_proj over the local intermediate range; ONE all-reduce (sum) after each.
Shards are cut on multiples of 128 rows/columns (= the quantisation group and the kernels' tile),
unevenly when the count of 128-blocks does not divide (e.g. 11008/128 = 86 blocks over 4 ranks ->
21/22/21/22), so every shard is again a valid QuantLinear in checkpoint layout.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from .quant_linear import QuantLinear

BLOCK = 128


def partition(n_units: int, world: int) -> List[int]:
	"""world+1 boundaries splitting n_units as evenly as possible (floor(r*n/world))."""
	return [(r * n_units) // world for r in range(world + 1)]


def shard_columns(q: QuantLinear, lo: int, hi: int) -> QuantLinear:
	"""Output columns [lo, hi) of a QuantLinear (multiples of 8)."""
	assert lo % 8 == 0 and hi % 8 == 0 and 0 <= lo < hi <= q.outfeatures
	out = QuantLinear(q.bits, q.groupsize, q.infeatures, hi - lo, q.bias is not None)
	out.qweight = q.qweight[:, lo:hi].contiguous()
	out.qzeros = q.qzeros[:, lo // 8:hi // 8].contiguous()
	out.scales = q.scales[:, lo:hi].contiguous()
	if q.bias is not None:
		out.bias = q.bias[lo:hi].contiguous()
	if q.g_idx is not None:
		out.set_g_idx(q.g_idx)
	return out


def shard_rows(q: QuantLinear, lo: int, hi: int, keep_bias: bool) -> QuantLinear:
	"""Input rows [lo, hi) of a QuantLinear.  Without act-order the cut must fall on group
	boundaries; the shard then owns the groups lo/groupsize .. hi/groupsize.  With act-order (g_idx) any
	cut on a multiple of 8 rows is valid: the rows of a shard may belong to any group, so the shard keeps
	the FULL scale / zero tables (they are small) and its slice of g_idx.  The bias is kept on one rank
	only (the partial sums are added up afterwards)."""
	gs = q.groupsize
	assert lo % 8 == 0 and hi % 8 == 0 and 0 <= lo < hi <= q.infeatures
	if q.g_idx is not None:
		has_bias = q.bias is not None and keep_bias
		out = QuantLinear(q.bits, gs, hi - lo, q.outfeatures, has_bias)
		out.qweight = q.qweight[lo // 8:hi // 8].contiguous()
		out.qzeros = q.qzeros.clone()          # [G, N / 8] of the whole layer, indexed through g_idx
		out.scales = q.scales.clone()
		if has_bias:
			out.bias = q.bias.clone()
		out.set_g_idx(q.g_idx[lo:hi].contiguous())
		return out
	assert (lo % gs == 0 and hi % gs == 0) or gs >= q.infeatures, 'row shards must be cut on group boundaries'
	has_bias = q.bias is not None and keep_bias
	if gs >= q.infeatures:
		# one group for the whole matrix: every shard keeps the single scale/zero row
		out = QuantLinear(q.bits, hi - lo, hi - lo, q.outfeatures, has_bias)
		out.qzeros = q.qzeros.clone()
		out.scales = q.scales.clone()
	else:
		out = QuantLinear(q.bits, gs, hi - lo, q.outfeatures, has_bias)
		out.qzeros = q.qzeros[lo // gs:hi // gs].contiguous()
		out.scales = q.scales[lo // gs:hi // gs].contiguous()
	out.qweight = q.qweight[lo // 8:hi // 8].contiguous()
	if has_bias:
		out.bias = q.bias.clone()
	return out


def shard_plan(hidden: int, heads: int, inter: int, world: int):
	"""Per-rank (head_lo, head_hi, inter_lo, inter_hi)."""
	assert heads % world == 0, 'the number of heads must be divisible by the tensor-parallel size'
	assert inter % BLOCK == 0
	hl = heads // world
	ib = partition(inter // BLOCK, world)
	return [(r * hl, (r + 1) * hl, ib[r] * BLOCK, ib[r + 1] * BLOCK) for r in range(world)]


@torch.no_grad()
def shard_llama(model, rank: int, world: int):
	"""In place: replaces the seven projections of every decoder layer of an UNFUSED quantised
	model (llama.LlamaForCausalLM after make_quant) by this rank's shards.  Embeddings, norms and
	lm_head stay replicated.  Call make_quant_attn / make_fused_mlp afterwards."""
	cfg = model.config
	head_dim = cfg.hidden_size // cfg.num_attention_heads
	h_lo, h_hi, i_lo, i_hi = shard_plan(cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, world)[rank]
	c_lo, c_hi = h_lo * head_dim, h_hi * head_dim
	for layer in model.model.layers:
		a, m = layer.self_attn, layer.mlp
		a.q_proj = shard_columns(a.q_proj, c_lo, c_hi)
		a.k_proj = shard_columns(a.k_proj, c_lo, c_hi)
		a.v_proj = shard_columns(a.v_proj, c_lo, c_hi)
		a.o_proj = shard_rows(a.o_proj, c_lo, c_hi, keep_bias=(rank == 0))
		a.num_heads = h_hi - h_lo
		m.gate_proj = shard_columns(m.gate_proj, i_lo, i_hi)
		m.up_proj = shard_columns(m.up_proj, i_lo, i_hi)
		m.down_proj = shard_rows(m.down_proj, i_lo, i_hi, keep_bias=(rank == 0))
	model.tp_rank, model.tp_world = rank, world
	return model


def all_reduce_(t: torch.Tensor, group=None) -> torch.Tensor:
	"""Sum over the tensor-parallel group, in place; identity without a process group."""
	import torch.distributed as dist
	if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
		dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
	return t


class PeerExchange:
	"""Exchange buffers of one row-parallel projection for the all-reduce fused into the decode
	kernel's epilogue (gptq_qmatmul_ar): every rank allocates a partial-sum buffer and arrival
	counters with cudaMalloc, the ranks of the node trade CUDA IPC handles through the process
	group and map each other's buffers.  `partials` / `flags` are the pointer arrays the C ABI takes."""

	def __init__(self, n_out: int, rank: int, world: int, group=None):
		"""Collective: every rank of `group` must call it.  A failure on any rank (allocation, IPC export or
		open) makes EVERY rank raise RuntimeError after the collectives have completed, so the callers can
		fall back together (to NCCL) without leaving a rank behind in a collective."""
		import ctypes
		import torch.distributed as dist
		from . import _lib
		L = _lib.lib()
		self.rank, self.world = rank, world
		self._opened = []
		self._own = None
		self.flag_bytes = int(L.gptq_ar_flag_bytes(n_out))
		self.bytes = self.flag_bytes + int(L.gptq_ar_partial_bytes(n_out))
		handle = (ctypes.c_ubyte * 64)()
		own = ctypes.c_void_p()
		ok = world <= 8
		if ok and L.gptq_peer_alloc(self.bytes, ctypes.byref(own)) == 0:
			self._own = own
			ok = L.gptq_peer_export(own, handle) == 0
		else:
			ok = False
		gathered = [None] * world
		dist.all_gather_object(gathered, (bool(ok), bytes(handle)), group=group)
		ok = all(g[0] for g in gathered)
		base = []
		if ok:
			for r in range(world):
				if r == rank:
					base.append(own.value)
					continue
				buf = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r][1])
				ptr = ctypes.c_void_p()
				if L.gptq_peer_open(buf, ctypes.byref(ptr)) != 0:
					ok = False
					break
				self._opened.append(ptr)
				base.append(ptr.value)
		verdict = [None] * world
		dist.all_gather_object(verdict, bool(ok), group=group)      # also: every rank has mapped every buffer before the first launch
		if not all(verdict):
			self.close()
			raise RuntimeError('peer exchange buffers could not be set up on every rank')
		# layout of a buffer: [sequence numbers][receive area]
		self.flags = (ctypes.c_void_p * 8)(*([b for b in base] + [None] * (8 - world)))
		self.partials = (ctypes.c_void_p * 8)(*([b + self.flag_bytes for b in base] + [None] * (8 - world)))

	def close(self):
		from . import _lib
		L = _lib.lib()
		for ptr in self._opened:
			L.gptq_peer_close(ptr)
		self._opened = []
		if self._own is not None:
			L.gptq_peer_free(self._own)
			self._own = None
