"""Tensor-parallel sharding on the CPU: shard index arithmetic, uneven 128-block splits,
gather-to-full equality, the partial-sum identity against the oracle, and a world_size-2 gloo
run of the all-reduce step."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import gptq_triton_b200 as G
from gptq_triton_b200 import loader, quantize, tp
from gptq_triton_b200.llama import LlamaConfig
from oracle import gptq_oracle as O


def test_partition_even_and_uneven():
	assert tp.partition(86, 4) == [0, 21, 43, 64, 86]
	assert tp.partition(172, 8)[-1] == 172 and all(b - a in (21, 22) for a, b in zip(tp.partition(172, 8), tp.partition(172, 8)[1:]))
	plan = tp.shard_plan(4096, 32, 11008, 4)
	assert [p[3] - p[2] for p in plan] == [2688, 2816, 2688, 2816] and plan[0][:2] == (0, 8) and plan[3][:2] == (24, 32)
	with pytest.raises(AssertionError):
		tp.shard_plan(4096, 32, 11008, 3)


def _quant_linear(K, N, gs, seed, bias=False):
	g = torch.Generator().manual_seed(seed)
	m = G.QuantLinear(4, gs, K, N, bias)
	qw, qz, sc = quantize.quantize_linear_weight(torch.randn((N, K), generator=g) * 0.02, gs)
	m.qweight.copy_(qw); m.qzeros.copy_(qz); m.scales.copy_(sc)
	if bias:
		m.bias.copy_(torch.randn(N, generator=g).half())
	return m


@pytest.mark.parametrize('gs', [128, -1])
def test_row_and_column_shards_reproduce_the_full_product(gs):
	K, N, world = 512, 256, 4
	full = _quant_linear(K, N, gs, seed=1, bias=True)
	x = (torch.randn((3, K), generator=torch.Generator().manual_seed(2))).half()
	ref = O.qmatmul_r32(x, full.qweight, full.qzeros, full.scales, gs, bias=full.bias)
	# column parallel: concatenation of the shards' outputs
	cb = [b * 8 for b in tp.partition(N // 8, world)]
	cols = [tp.shard_columns(full, cb[r], cb[r + 1]) for r in range(world)]
	assert torch.equal(torch.cat([c.qweight for c in cols], dim=1), full.qweight)
	assert torch.equal(torch.cat([c.qzeros for c in cols], dim=1), full.qzeros)
	out = torch.cat([O.qmatmul_r32(x, c.qweight, c.qzeros, c.scales, gs, bias=c.bias) for c in cols], dim=1)
	assert torch.allclose(out, ref, atol=1e-5)
	# row parallel: sum of the shards' partial products; bias only on rank 0
	kb = [b * 128 for b in tp.partition(K // 128, world)]
	rows = [tp.shard_rows(full, kb[r], kb[r + 1], keep_bias=(r == 0)) for r in range(world)]
	assert torch.equal(torch.cat([r_.qweight for r_ in rows], dim=0), full.qweight)
	assert sum(r_.bias is not None for r_ in rows) == 1
	part = sum(O.qmatmul_r32(x[:, kb[r]:kb[r + 1]], rows[r].qweight, rows[r].qzeros, rows[r].scales, rows[r].groupsize, bias=rows[r].bias)
			   for r in range(world))
	assert torch.allclose(part, ref, atol=1e-4)
	with pytest.raises(AssertionError):
		if gs == 128:
			tp.shard_rows(full, 64, 192, keep_bias=False)       # not on a group boundary
		else:
			raise AssertionError


def test_row_shards_of_an_act_order_layer():
	"""g_idx = a random permutation of the group assignment: a row shard keeps the full scale / zero tables and its
	slice of g_idx; the partial products of the shards add up to the full product (any cut on 8 rows is valid)."""
	K, N, gs, world = 512, 128, 128, 4
	full = _quant_linear(K, N, gs, seed=5, bias=True)
	g = torch.Generator().manual_seed(6)
	g_idx = (torch.arange(K) // gs)[torch.randperm(K, generator=g)].to(torch.int32)
	full.set_g_idx(g_idx)
	x = (torch.randn((3, K), generator=g)).half()
	ref = O.qmatmul_r32(x, full.qweight, full.qzeros, full.scales, gs, g_idx=g_idx, bias=full.bias)
	cuts = [0, 72, 200, 384, 512]          # multiples of 8, not of the group size
	rows = [tp.shard_rows(full, cuts[r], cuts[r + 1], keep_bias=(r == 0)) for r in range(world)]
	assert all(torch.equal(r_.qzeros, full.qzeros) and torch.equal(r_.scales, full.scales) for r_ in rows)
	assert torch.equal(torch.cat([r_.g_idx for r_ in rows]), g_idx)
	part = sum(O.qmatmul_r32(x[:, cuts[r]:cuts[r + 1]], rows[r].qweight, rows[r].qzeros, rows[r].scales, gs, g_idx=rows[r].g_idx, bias=rows[r].bias)
			   for r in range(world))
	assert torch.allclose(part, ref, atol=1e-4)
	# column shards carry the whole g_idx
	col = tp.shard_columns(full, 0, 64)
	assert torch.equal(col.g_idx, g_idx)


def test_shard_llama_shapes():
	cfg = LlamaConfig(hidden_size=512, intermediate_size=1408, num_hidden_layers=1, num_attention_heads=4, vocab_size=64, max_position_embeddings=64)
	for world in (2, 4):
		sizes = []
		for rank in range(world):
			model = loader._empty_model(cfg, 4, 128)
			tp.shard_llama(model, rank, world)
			layer = model.model.layers[0]
			assert layer.self_attn.q_proj.outfeatures == 512 // world and layer.self_attn.o_proj.infeatures == 512 // world
			assert layer.mlp.gate_proj.outfeatures == layer.mlp.down_proj.infeatures
			sizes.append(layer.mlp.down_proj.infeatures)
			G.make_quant_attn(model)
			G.make_fused_mlp(model)
			assert model.model.layers[0].self_attn.num_heads == 4 // world
			assert model.model.layers[0].self_attn.qkv_proj.outfeatures == 3 * 512 // world
		assert sum(sizes) == 1408 and all(s % 128 == 0 for s in sizes)


def _gloo_worker(rank, world, port, q):
	os.environ['MASTER_ADDR'] = '127.0.0.1'
	os.environ['MASTER_PORT'] = str(port)
	dist.init_process_group('gloo', rank=rank, world_size=world)
	try:
		K, N, gs = 512, 128, 128
		full = _quant_linear(K, N, gs, seed=3)
		x = (torch.randn((2, K), generator=torch.Generator().manual_seed(4))).half()
		kb = [b * 128 for b in tp.partition(K // 128, world)]
		shard = tp.shard_rows(full, kb[rank], kb[rank + 1], keep_bias=False)
		part = O.qmatmul_r32(x[:, kb[rank]:kb[rank + 1]], shard.qweight, shard.qzeros, shard.scales, gs)
		res = torch.ones((2, N))
		y = part + (res if rank == 0 else 0)          # the residual enters on rank 0 only
		tp.all_reduce_(y)
		ref = O.qmatmul_r32(x, full.qweight, full.qzeros, full.scales, gs) + res
		q.put((rank, bool(torch.allclose(y, ref, atol=1e-4))))
	finally:
		dist.destroy_process_group()


def test_all_reduce_of_row_parallel_partials_gloo():
	world = 2
	ctx = mp.get_context('spawn')
	q = ctx.Queue()
	port = 29500 + (os.getpid() % 500)
	procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
	for p in procs:
		p.start()
	for p in procs:
		p.join(timeout=120)
		assert p.exitcode == 0
	got = sorted(q.get(timeout=10) for _ in range(world))
	assert got == [(0, True), (1, True)]
