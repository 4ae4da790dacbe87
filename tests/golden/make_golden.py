#!/usr/bin/env python
"""Generates the golden fixtures in this directory by running the REFERENCE's own
code on the CPU.  Needs the reference checkout (pass its path as argv[1]); the
fixtures it writes are committed so that the tests never need the reference.

What is recorded:
  pack_*.npz     quantize.dumbquant + quantize.pack_linear on seeded nn.Linear
                 layers: fake-quantised weights, fp32 scale/zero, packed tensors.
  matmul4_*.npz  gptq_triton.quant_linear.matmul4_kernel executed by the Triton
                 interpreter (TRITON_INTERPRET=1) on those packed tensors.
  mlp_*.npz      gptq_triton.fused_mlp.llama_mlp_fused_4_kernel, same way.
  rope.npz       transformers' apply_rotary_pos_emb (third-party arithmetic the
                 reference calls at fused_attention.py:101-102).

usage: python tests/golden/make_golden.py /path/to/reference
"""
import os
import sys
from pathlib import Path

os.environ['TRITON_INTERPRET'] = '1'
ref = sys.argv[1]
sys.path.insert(0, os.path.join(ref, 'src'))
sys.path.insert(0, ref)

import numpy as np
import torch

import quantize                                              # reference: quantize.py
from gptq_triton.quant_linear import QuantLinear, matmul4_kernel
from gptq_triton.fused_mlp import llama_mlp_fused_4_kernel

OUT = Path(__file__).parent


def quantised_layer(K, N, groupsize, seed):
	torch.manual_seed(seed)
	layer = torch.nn.Linear(K, N, bias=False)
	scale, zero = quantize.dumbquant(layer, 4, groupsize)
	ql = QuantLinear(4, groupsize, K, N, False)
	quantize.pack_linear(ql, layer.weight.data, scale, zero, None)
	return layer, scale, zero, ql


def run_matmul4(x, ql, groupsize_arg, BM, BN, BK):
	M, K = x.shape
	N = ql.qweight.shape[1]
	c = torch.zeros(M, N, dtype=torch.float16)
	grid = (((M + BM - 1) // BM) * (N // BN),)
	matmul4_kernel.fn[grid](
		x, ql.qweight, c, ql.scales, ql.qzeros, M, N, K,
		x.stride(0), x.stride(1), ql.qweight.stride(0), ql.qweight.stride(1),
		c.stride(0), c.stride(1), ql.scales.stride(0), ql.scales.stride(1),
		ql.qzeros.stride(0), ql.qzeros.stride(1),
		groupsize_arg, groupsize_arg == K,
		BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK, GROUP_SIZE_M=8)
	return c


def run_mlp(x, g, u, groupsize_arg, BM, BN, BK):
	M, K = x.shape
	N = g.qweight.shape[1]
	c = torch.zeros(M, N, dtype=torch.float16)
	grid = (((M + BM - 1) // BM) * (N // BN),)
	llama_mlp_fused_4_kernel.fn[grid](
		x, c, g.qweight, g.scales, g.qzeros, u.qweight, u.scales, u.qzeros, M, N, K,
		x.stride(0), x.stride(1), g.qweight.stride(0), g.qweight.stride(1),
		c.stride(0), c.stride(1), g.scales.stride(0), g.scales.stride(1),
		g.qzeros.stride(0), g.qzeros.stride(1),
		groupsize_arg, groupsize_arg == K,
		BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK, GROUP_SIZE_M=8)
	return c


def main():
	# (name, K, N, groupsize, M, tile)
	cases = [
		('a', 256, 256, 128, 5, (16, 32, 32)),
		('b', 256, 256, -1, 1, (16, 32, 128)),
		('c', 512, 256, 128, 17, (32, 32, 128)),
		('d', 384, 512, 128, 16, (16, 64, 64)),
	]
	for i, (name, K, N, gs, M, (BM, BN, BK)) in enumerate(cases):
		layer, scale, zero, ql = quantised_layer(K, N, gs, seed=100 + i)
		np.savez_compressed(
			OUT / f'pack_{name}.npz', K=K, N=N, groupsize=gs,
			fakequant=layer.weight.data.numpy(), scale=scale.numpy(), zero=zero.numpy(),
			qweight=ql.qweight.numpy(), qzeros=ql.qzeros.numpy(), scales=ql.scales.numpy())
		torch.manual_seed(200 + i)
		x = torch.randn(M, K).half()
		c = run_matmul4(x, ql, ql.groupsize, BM, BN, BK)
		np.savez_compressed(OUT / f'matmul4_{name}.npz', x=x.numpy(), y=c.numpy(), groupsize=gs, pack=f'pack_{name}.npz')
		print('matmul4', name, float(c.float().abs().max()))

	for i, (name, K, N, gs, M, (BM, BN, BK)) in enumerate([
			('a', 256, 256, 128, 3, (16, 32, 32)),
			('b', 256, 512, -1, 16, (16, 32, 128))]):
		_, _, _, g = quantised_layer(K, N, gs, seed=300 + i)
		_, _, _, u = quantised_layer(K, N, gs, seed=400 + i)
		torch.manual_seed(500 + i)
		x = torch.randn(M, K).half()
		c = run_mlp(x, g, u, g.groupsize, BM, BN, BK)
		np.savez_compressed(
			OUT / f'mlp_{name}.npz', x=x.numpy(), y=c.numpy(), groupsize=gs,
			gate_qweight=g.qweight.numpy(), gate_qzeros=g.qzeros.numpy(), gate_scales=g.scales.numpy(),
			up_qweight=u.qweight.numpy(), up_qzeros=u.qzeros.numpy(), up_scales=u.scales.numpy())
		print('mlp', name, float(c.float().abs().max()))

	# rotary: third-party arithmetic, pinned against the installed transformers
	from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
	torch.manual_seed(600)
	b, h, t, d = 2, 3, 7, 128
	q = torch.randn(b, h, t, d).half()
	k = torch.randn(b, h, t, d).half()
	pos = torch.tensor([[0, 1, 2, 3, 4, 5, 6], [10, 11, 500, 2047, 3, 3, 0]])
	inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
	freqs = pos[:, :, None].float() * inv_freq[None, None, :]
	emb = torch.cat([freqs, freqs], dim=-1)
	cos, sin = emb.cos().half(), emb.sin().half()       # [b, t, d]
	qo, ko = apply_rotary_pos_emb(q, k, cos, sin)        # unsqueeze_dim=1 default
	np.savez_compressed(OUT / 'rope.npz', q=q.numpy(), k=k.numpy(), pos=pos.numpy(), q_out=qo.numpy(), k_out=ko.numpy(), theta=10000.0)
	print('rope done')


if __name__ == '__main__':
	main()
