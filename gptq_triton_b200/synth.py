"""Seeded synthetic GPTQ tensors with the shapes and value distributions of the benchmark
configurations: uniform uint4 weights and zeros, scales ~ U(0.002, 0.02), activations ~ N(0, 1),
optionally an act-order g_idx that is a random permutation of the group assignment.
They stand in for real LLaMA checkpoints, which are not available offline."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


def pack_rows(q: np.ndarray) -> np.ndarray:
	"""uint [K, N] (0..15) -> int32 [K/8, N], lowest nibble = lowest row."""
	K, N = q.shape
	w = q.astype(np.uint32).reshape(K // 8, 8, N)
	out = np.zeros((K // 8, N), dtype=np.uint32)
	for i in range(8):
		out |= w[:, i, :] << np.uint32(4 * i)
	return out.view(np.int32)


def pack_cols(z: np.ndarray) -> np.ndarray:
	"""uint [G, N] (0..15) -> int32 [G, N/8], lowest nibble = lowest column."""
	G, N = z.shape
	w = z.astype(np.uint32).reshape(G, N // 8, 8)
	out = np.zeros((G, N // 8), dtype=np.uint32)
	for i in range(8):
		out |= w[:, :, i] << np.uint32(4 * i)
	return out.view(np.int32)


def quant_tensors(K: int, N: int, groupsize: int, seed: int, act_order: bool = False, bias: bool = False):
	"""Returns dict(qweight, qzeros, scales, g_idx|None, bias|None, groupsize) of CPU tensors."""
	gs = K if groupsize == -1 else groupsize
	G = (K + gs - 1) // gs
	rng = np.random.default_rng(seed)
	qweight = torch.from_numpy(rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint32).view(np.int32))
	qzeros = torch.from_numpy(rng.integers(0, 2 ** 32, size=(G, N // 8), dtype=np.uint32).view(np.int32))
	scales = torch.from_numpy(rng.uniform(0.002, 0.02, size=(G, N)).astype(np.float16))
	g_idx = None
	if act_order:
		g_idx = torch.from_numpy((np.arange(K) // gs)[rng.permutation(K)].astype(np.int32))
	b = torch.from_numpy(rng.normal(0, 1, size=(N,)).astype(np.float16)) if bias else None
	return dict(qweight=qweight, qzeros=qzeros, scales=scales, g_idx=g_idx, bias=b, groupsize=groupsize)


def activations(shape, seed: int, std: float = 1.0) -> torch.Tensor:
	g = torch.Generator().manual_seed(seed)
	return (torch.randn(shape, generator=g) * std).half()


def to_device(d: dict, device) -> dict:
	return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
