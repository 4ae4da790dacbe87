"""Fused gate/up SiLU*mul MLP.

Mirrors src/gptq_triton/fused_mlp.py of the reference: `make_fused_mlp` (:13-27),
`QuantLlamaMLP` (:52-79) and the op `triton_llama_mlp_4` (:241-302), on the sm_100a
C-ABI library.  Unlike the reference kernel this one is not slower for grouped
checkpoints, so load_quant fuses the MLP for every groupsize.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from .quant_linear import QuantLinear


def _is_llama_mlp(m) -> bool:
	"""An MLP block in the LLaMA sense: three quantised projections named gate/up/down."""
	return (not isinstance(m, QuantLlamaMLP)
			and all(isinstance(getattr(m, n, None), QuantLinear) for n in ('gate_proj', 'up_proj', 'down_proj')))


def make_fused_mlp(m, parent_name=''):
	"""Replace all LLaMA MLP modules below `m` by QuantLlamaMLP; returns the (possibly
	replaced) module, like the reference (fused_mlp.py:13-27)."""
	if _is_llama_mlp(m):
		return QuantLlamaMLP(m.gate_proj, m.down_proj, m.up_proj)
	for name, child in m.named_children():
		child = make_fused_mlp(child, parent_name=f"{parent_name}.{name}")
		if isinstance(child, QuantLlamaMLP):
			setattr(m, name, child)
	return m


def autotune_warmup(model):
	"""API shim (reference: fused_mlp.py:30-49); nothing to tune."""
	return iter(())


def gateup_silu(groupsize: int, a: torch.Tensor, gate_qweight, gate_scales, gate_qzeros, up_qweight, up_scales, up_qzeros,
				g_idx: Optional[torch.Tensor] = None, perm: Optional[torch.Tensor] = None,
				rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6,
				sumsq_in: Optional[torch.Tensor] = None) -> torch.Tensor:
	"""silu(a x deq(gate)) * (a x deq(up)); fp32 until the one fp16 store.  With rms_weight the input is
	RMS-normalised first: inside the decode kernel when `sumsq_in` (fp32 [M, K // 32], written by the
	projection that produced `a`, see quant_linear.qmatmul) is given and the shape allows, else by the
	library's RMSNorm kernel."""
	assert gate_qweight.shape == up_qweight.shape and gate_scales.shape == up_scales.shape and gate_qzeros.shape == up_qzeros.shape, "All weights must have the same shape"
	assert a.shape[-1] == (gate_qweight.shape[0] * 8), "A must be a multiple of 8 in the last dimension"
	assert a.is_contiguous(), "A must be contiguous"
	_lib.require_cuda(a, gate_qweight, gate_scales, gate_qzeros, up_qweight, up_scales, up_qzeros, g_idx, perm)
	if a.dtype != torch.float16:
		raise TypeError('A must be float16')
	x = a.view(-1, a.shape[-1])
	M, K = x.shape
	N = gate_qweight.shape[1]
	c = torch.empty((M, N), device=a.device, dtype=torch.float16)
	if M == 0:
		return c.view(a.shape[:-1] + (N,))
	from .quant_linear import DECODE_MAX_M, dequant_matmul, prefill_kernel_available, rms_fusable
	if rms_weight is not None and sumsq_in is not None and rms_fusable(M, K, g_idx, perm):
		assert sumsq_in.dtype == torch.float32 and sumsq_in.is_contiguous() and sumsq_in.numel() >= M * (K // 32)
		ws = _lib.workspace(a.device, M, K, N)
		rc = _lib.lib().gptq_gateup_silu_rms(
			_lib.ptr(x), _lib.ptr(gate_qweight), _lib.ptr(gate_qzeros), _lib.ptr(gate_scales),
			_lib.ptr(up_qweight), _lib.ptr(up_qzeros), _lib.ptr(up_scales), None, None,
			_lib.ptr(c), M, K, N, groupsize, K, N, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device),
			_lib.ptr(rms_weight), _lib.ptr(sumsq_in), K // 32, float(rms_eps))
		_lib.check(rc, 'gptq_gateup_silu_rms')
		return c.view(a.shape[:-1] + (N,))
	if rms_weight is not None:
		from .fused_attention import rmsnorm
		x = rmsnorm(x.contiguous(), rms_weight, rms_eps)
		rms_weight = None
	if M > DECODE_MAX_M and perm is not None and g_idx is None and prefill_kernel_available(M, K, N, groupsize):
		x = x[:, perm.long()].contiguous()
		perm = None
	if M > DECODE_MAX_M and (g_idx is not None or not prefill_kernel_available(M, K, N, groupsize)):
		g = dequant_matmul(x, groupsize, gate_qweight, gate_scales, gate_qzeros, g_idx, perm).float()
		u = dequant_matmul(x, groupsize, up_qweight, up_scales, up_qzeros, g_idx, perm).float()
		c = (torch.nn.functional.silu(g) * u).half()
		return c.view(a.shape[:-1] + (N,))
	ws = _lib.workspace(a.device, M, K, N)
	rc = _lib.lib().gptq_gateup_silu(
		_lib.ptr(x), _lib.ptr(gate_qweight), _lib.ptr(gate_qzeros), _lib.ptr(gate_scales),
		_lib.ptr(up_qweight), _lib.ptr(up_qzeros), _lib.ptr(up_scales), _lib.ptr(g_idx), _lib.ptr(perm),
		_lib.ptr(c), M, K, N, groupsize, K, N, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device))
	_lib.check(rc, 'gptq_gateup_silu')
	return c.view(a.shape[:-1] + (N,))


def triton_llama_mlp_4(groupsize: int, a: torch.FloatTensor, gate_qweight: torch.IntTensor, gate_scales: torch.FloatTensor,
					   gate_qzeros: torch.IntTensor, up_qweight: torch.IntTensor, up_scales: torch.FloatTensor,
					   up_qzeros: torch.IntTensor) -> torch.FloatTensor:
	"""Drop-in for the reference op of the same name (fused_mlp.py:241); no Triton involved."""
	return gateup_silu(groupsize, a, gate_qweight, gate_scales, gate_qzeros, up_qweight, up_scales, up_qzeros)


class QuantLlamaMLP(nn.Module):
	"""down_proj(silu(gate(x)) * up(x)) with gate/up in one kernel; constructor and buffer
	names as in the reference (fused_mlp.py:52-79)."""

	def __init__(self, gate_proj, down_proj, up_proj):
		super().__init__()
		assert gate_proj.groupsize == up_proj.groupsize
		self.register_buffer('gate_proj_qweight', gate_proj.qweight)
		self.register_buffer('gate_proj_scales', gate_proj.scales)
		self.register_buffer('gate_proj_qzeros', gate_proj.qzeros)
		self.register_buffer('up_proj_qweight', up_proj.qweight)
		self.register_buffer('up_proj_scales', up_proj.scales)
		self.register_buffer('up_proj_qzeros', up_proj.qzeros)
		# gate and up see the same input, so they share one act-order; a differing up g_idx is
		# not representable in the fused kernel
		g_gate, g_up = gate_proj.g_idx, up_proj.g_idx
		if (g_gate is None) != (g_up is None) or (g_gate is not None and not torch.equal(g_gate, g_up)):
			raise ValueError('gate_proj and up_proj must share one g_idx to be fused')
		self.register_buffer('g_idx', g_gate)
		self.groupsize = gate_proj.groupsize
		self.infeatures = gate_proj.infeatures
		self.outfeatures = down_proj.outfeatures
		self.down_proj = down_proj
		self._ao_ready = False

	def _apply(self, fn, recurse=True):
		self._ao_ready = False
		return super()._apply(fn, recurse)

	def _prepare(self):
		from .quant_linear import _act_order_perm, act_order_rows
		self._perm = None
		self._gidx = None
		self._gate_qw, self._up_qw = self.gate_proj_qweight, self.up_proj_qweight
		if self.g_idx is not None:
			trivial = torch.arange(self.infeatures, device=self.g_idx.device, dtype=torch.int64) // self.groupsize
			if not torch.equal(self.g_idx.to(torch.int64), trivial):
				perm = _act_order_perm(self.g_idx, self.groupsize)
				if perm is not None:
					self._perm = perm
					self._gate_qw = act_order_rows(self.gate_proj_qweight, perm)
					self._up_qw = act_order_rows(self.up_proj_qweight, perm)
				else:
					self._gidx = self.g_idx
		self._ao_ready = True

	def intermediate(self, x, rms_weight=None, rms_eps=1e-6, sumsq_in=None):
		if not self._ao_ready:
			self._prepare()
		return gateup_silu(self.groupsize, x, self._gate_qw, self.gate_proj_scales, self.gate_proj_qzeros,
						   self._up_qw, self.up_proj_scales, self.up_proj_qzeros, g_idx=self._gidx, perm=self._perm,
						   rms_weight=rms_weight, rms_eps=rms_eps, sumsq_in=sumsq_in)

	def forward(self, x, residual: Optional[torch.Tensor] = None, rms_weight=None, rms_eps=1e-6, sumsq_in=None, sumsq_out=None, ar=None):
		"""`rms_weight` (+ `sumsq_in`): RMS-normalise x first (inside the kernel when sumsq_in is given);
		`sumsq_out`: let down_proj leave the per-tile sums of squares of its output (decode sizes)."""
		h = self.intermediate(x, rms_weight, rms_eps, sumsq_in)
		if residual is None and sumsq_out is None and ar is None:
			return self.down_proj(h)
		return self.down_proj(h, residual=residual, sumsq_out=sumsq_out, ar=ar)      # ar: tensor-parallel exchange (tp.PeerExchange)
