"""Round-to-nearest 4-bit quantiser and packer: the fixture generator of the reference
(`dumbquant`, quantize.py:294-329; `Quantizer.find_params` / `quantize`, gptq.py:174-246) and
its packer (`pack_linear`, quantize.py:236-291), vectorised so that they run on the GPU.
Produces tensors in the checkpoint layout that QuantLinear loads."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def rtn_quantize(weight: torch.Tensor, groupsize: int = -1):
	"""weight [N, K] -> (q uint8-valued int32 [N, K], scale fp32 [N, G], zero fp32 [N, G]).
	Asymmetric per-row, per-group min/max quantisation to 0..15 (perchannel=True, sym=False)."""
	W = weight.detach().float()
	N, K = W.shape
	gs = K if groupsize == -1 else groupsize
	assert K % gs == 0
	G = K // gs
	Wg = W.view(N, G, gs)
	zero_t = torch.zeros((), device=W.device)
	xmin = torch.minimum(Wg.amin(dim=2), zero_t)
	xmax = torch.maximum(Wg.amax(dim=2), zero_t)
	both = (xmin == 0) & (xmax == 0)
	xmin = torch.where(both, torch.full_like(xmin, -1.0), xmin)
	xmax = torch.where(both, torch.full_like(xmax, 1.0), xmax)
	scale = (xmax - xmin) / 15.0
	zero = torch.round(-xmin / scale)
	q = torch.clamp(torch.round(Wg / scale[..., None]) + zero[..., None], 0, 15).to(torch.int32).view(N, K)
	return q, scale, zero


def pack(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
	"""q int32 [N, K] in 0..15, scale/zero [N, G] -> (qweight int32 [K/8, N], qzeros int32 [G, N/8],
	scales fp16 [G, N]); lowest nibble = lowest index; the stored zero is zero - 1."""
	N, K = q.shape
	assert K % 8 == 0 and N % 8 == 0
	qt = q.t().contiguous().view(K // 8, 8, N).to(torch.int64)
	sh = (torch.arange(8, device=q.device, dtype=torch.int64) * 4).view(1, 8, 1)
	qweight = (qt << sh).sum(dim=1)
	qweight = torch.where(qweight >= 2 ** 31, qweight - 2 ** 32, qweight).to(torch.int32)
	z = (zero.t().contiguous().to(torch.int64) - 1) & 0xF                 # [G, N]
	G = z.shape[0]
	zt = z.view(G, N // 8, 8)
	sh2 = (torch.arange(8, device=q.device, dtype=torch.int64) * 4).view(1, 1, 8)
	qzeros = (zt << sh2).sum(dim=2)
	qzeros = torch.where(qzeros >= 2 ** 31, qzeros - 2 ** 32, qzeros).to(torch.int32)
	scales = scale.t().contiguous().to(torch.float16)
	return qweight.contiguous(), qzeros.contiguous(), scales


def quantize_linear_weight(weight: torch.Tensor, groupsize: int = -1):
	"""nn.Linear weight [N, K] -> (qweight, qzeros, scales) in checkpoint layout."""
	q, scale, zero = rtn_quantize(weight, groupsize)
	return pack(q, scale, zero)
