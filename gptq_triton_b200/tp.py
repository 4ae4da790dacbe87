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
	boundaries; the shard then owns the groups lo/groupsize .. hi/groupsize.  The bias is kept
	on one rank only (the partial sums are added up afterwards)."""
	assert q.g_idx is None, 'row shards of act-order layers are not supported'
	gs = q.groupsize
	assert lo % 8 == 0 and hi % 8 == 0 and 0 <= lo < hi <= q.infeatures
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
