"""QuantLinear, make_quant and the quantised matmul op.

Mirrors src/gptq_triton/quant_linear.py of the reference (module `QuantLinear` :49-77,
`make_quant` :13-32, op `triton_matmul4` :228-283) on top of the sm_100a C-ABI library.
The buffers keep the reference's names, shapes and dtypes, so its checkpoints load
unchanged; an optional `g_idx` buffer (int32 [K], group of each input row) adds act-order.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn as nn

from . import _lib


def make_quant(model, bits, groupsize):
	"""Replace every nn.Linear of `model` except `lm_head` by a QuantLinear
	(reference: quant_linear.py:13-32)."""
	for name, m in list(model.named_modules()):
		if not isinstance(m, nn.Linear):
			continue
		if name == 'lm_head':
			continue
		qlayer = QuantLinear(bits, groupsize, m.in_features, m.out_features, m.bias is not None)
		if '.' in name:
			parent_name, child = name.rsplit('.', 1)
			parent = model.get_submodule(parent_name)
		else:
			parent, child = model, name
		setattr(parent, child, qlayer)


def autotune_warmup(model):
	"""Kept for API compatibility (reference: quant_linear.py:35-46).  Kernel selection is a
	static function of the shape here, so there is nothing to warm up."""
	return iter(())


def _act_order_perm(g_idx: torch.Tensor, groupsize: int) -> Optional[torch.Tensor]:
	"""Stable sort of the rows by group.  Returns perm (int32 [K]) when every group then is a
	contiguous run of exactly `groupsize` rows, else None."""
	K = g_idx.numel()
	perm = torch.argsort(g_idx.to(torch.int64), stable=True)
	expect = torch.arange(K, device=g_idx.device) // groupsize
	if not torch.equal(g_idx.to(torch.int64)[perm], expect):
		return None
	return perm.to(torch.int32)


def act_order_rows(qweight: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
	"""Packed weights with rows taken in `perm` order (groups become contiguous)."""
	_lib.require_cuda(qweight, perm)
	out = torch.empty_like(qweight)
	K, N = qweight.shape[0] * 8, qweight.shape[1]
	rc = _lib.lib().gptq_act_order_rows(_lib.ptr(qweight), _lib.ptr(perm), _lib.ptr(out), K, N, _lib.stream_ptr(qweight.device))
	_lib.check(rc, 'gptq_act_order_rows')
	return out


DECODE_MAX_M = 16


USE_TENSOR_CORE_KERNEL = os.environ.get('GPTQ_B200_TC', '1') != '0'


def prefill_kernel_available(M: int, K: int, N: int, groupsize: int) -> bool:
	"""True when the tensor-core (tcgen05) kernel of the library covers this shape
	(the rule of tc_shape_ok in csrc/qmm_tc.cu)."""
	gs = K if groupsize == -1 else groupsize
	return USE_TENSOR_CORE_KERNEL and M > DECODE_MAX_M and N % 128 == 0 and K % 64 == 0 and gs % 64 == 0 and K % gs == 0


def dequant_matmul(x2d: torch.Tensor, groupsize: int, qweight, scales, qzeros, g_idx=None, perm=None) -> torch.Tensor:
	"""Dequantise-then-matmul on the GPU: the library's dequantise kernel followed by a cuBLAS
	fp16 matmul.  Serves prefill-sized inputs (M > 16) for shapes the tensor-core kernel does not
	cover, and is the comparison path of the tests."""
	w = dequantize(groupsize, qweight, scales, qzeros, g_idx)
	if perm is not None:
		x2d = x2d[:, perm.long()]
	return x2d @ w


def qmatmul(groupsize: int, a: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
			bias: Optional[torch.Tensor] = None, g_idx: Optional[torch.Tensor] = None, perm: Optional[torch.Tensor] = None,
			residual: Optional[torch.Tensor] = None, sumsq_out: Optional[torch.Tensor] = None, ar=None) -> torch.Tensor:
	"""C = A x deq(B) (+ bias) (+ residual).

	A (..., K) fp16 contiguous; qweight (K//8, N) int32; scales (G, N) fp16; qzeros (G, N//8)
	int32; bias (N,) fp16.  Returns (..., N) fp16, freshly allocated, computed asynchronously
	on the current CUDA stream — the contract of the reference op (quant_linear.py:228-283).
	`g_idx` gives act-order groups for rows in checkpoint order; `perm` says that qweight was
	re-ordered with act_order_rows().  `residual` (..., N) is added in the epilogue.
	`sumsq_out` (fp32 [M, N // 32], decode sizes only) receives the sums of squares per 32 columns of
	the output, from which the next fused op derives the RMSNorm factor (see rms_fusable()).
	`ar` (tp.PeerExchange, decode sizes only): this call is one rank's share of a row-parallel
	projection; the partial sums of all ranks are added inside the kernel (every rank gets the
	full result, residual included).
	"""
	assert a.shape[-1] == (qweight.shape[0] * 8), "A must be a multiple of 8 in the last dimension"
	assert a.is_contiguous(), "A must be contiguous"
	_lib.require_cuda(a, qweight, scales, qzeros, bias, g_idx, perm, residual)
	if a.dtype != torch.float16:
		raise TypeError('A must be float16')
	x = a.view(-1, a.shape[-1])
	M, K = x.shape
	N = qweight.shape[1]
	c = torch.empty((M, N), device=a.device, dtype=torch.float16)
	if M == 0:
		return c.view(a.shape[:-1] + (N,))
	res = None
	if residual is not None:
		assert residual.is_contiguous() and residual.numel() == M * N
		res = residual.view(M, N)
	if M > DECODE_MAX_M and perm is not None and g_idx is None and prefill_kernel_available(M, K, N, groupsize):
		x = x[:, perm.long()].contiguous()      # the tensor-core kernel reads x through TMA: gather once up front
		perm = None
	if M > DECODE_MAX_M and (g_idx is not None or not prefill_kernel_available(M, K, N, groupsize)):
		c = dequant_matmul(x, groupsize, qweight, scales, qzeros, g_idx, perm)
		if bias is not None:
			c = c + bias
		if res is not None:
			c = c + res
		return c.view(a.shape[:-1] + (N,))
	ws = _lib.workspace(a.device, M, K, N)
	if ar is not None:
		if sumsq_out is not None:
			assert sumsq_out.dtype == torch.float32 and sumsq_out.is_contiguous() and sumsq_out.numel() >= M * (N // 32)
		rc = _lib.lib().gptq_qmatmul_ar(
			_lib.ptr(x), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), _lib.ptr(g_idx), _lib.ptr(perm),
			_lib.ptr(bias), _lib.ptr(res), N, _lib.ptr(c), M, K, N, groupsize, K, N,
			_lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device), _lib.ptr(sumsq_out),
			ar.world, ar.rank, ar.partials, ar.flags)
		_lib.check(rc, 'gptq_qmatmul_ar')
		return c.view(a.shape[:-1] + (N,))
	if sumsq_out is not None:
		assert sumsq_out.dtype == torch.float32 and sumsq_out.is_contiguous() and sumsq_out.numel() >= M * (N // 32)
		rc = _lib.lib().gptq_qmatmul_sumsq(
			_lib.ptr(x), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), _lib.ptr(g_idx), _lib.ptr(perm),
			_lib.ptr(bias), _lib.ptr(res), N, _lib.ptr(c), M, K, N, groupsize, K, N,
			_lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device), _lib.ptr(sumsq_out))
		_lib.check(rc, 'gptq_qmatmul_sumsq')
		return c.view(a.shape[:-1] + (N,))
	rc = _lib.lib().gptq_qmatmul(
		_lib.ptr(x), _lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), _lib.ptr(g_idx), _lib.ptr(perm),
		_lib.ptr(bias), _lib.ptr(res), N, _lib.ptr(c), M, K, N, groupsize, K, N,
		_lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device))
	_lib.check(rc, 'gptq_qmatmul')
	return c.view(a.shape[:-1] + (N,))


def rms_fusable(M: int, N_producer: int, g_idx, perm) -> bool:
	"""True when the RMSNorm between a producing projection (N_producer outputs) and the next
	fused op can be folded into the two decode kernels (gptq_qmatmul_sumsq -> *_rms)."""
	return 0 < M <= DECODE_MAX_M and N_producer % 128 == 0 and N_producer // 32 <= 256 and g_idx is None and perm is None


def triton_matmul4(groupsize: int, a: torch.FloatTensor, qweight: torch.IntTensor, scales: torch.FloatTensor,
				   qzeros: torch.IntTensor, bias: Optional[torch.FloatTensor] = None) -> torch.FloatTensor:
	"""Drop-in for the reference op of the same name (quant_linear.py:228); no Triton involved."""
	return qmatmul(groupsize, a, qweight, scales, qzeros, bias)


def unpack_qweight(qweight: torch.Tensor) -> torch.Tensor:
	"""uint8 [K, N] integer weights of a packed int32 [K/8, N] tensor (on the GPU)."""
	_lib.require_cuda(qweight)
	R, N = qweight.shape
	out = torch.empty((R * 8, N), dtype=torch.uint8, device=qweight.device)
	_lib.check(_lib.lib().gptq_unpack_qweight(_lib.ptr(qweight), _lib.ptr(out), R * 8, N, _lib.stream_ptr(qweight.device)), 'gptq_unpack_qweight')
	return out


def unpack_qzeros(qzeros: torch.Tensor) -> torch.Tensor:
	"""uint8 [G, N] stored zero values (zero point - 1) of a packed int32 [G, N/8] tensor."""
	_lib.require_cuda(qzeros)
	G, C = qzeros.shape
	out = torch.empty((G, C * 8), dtype=torch.uint8, device=qzeros.device)
	_lib.check(_lib.lib().gptq_unpack_qzeros(_lib.ptr(qzeros), _lib.ptr(out), G, C * 8, _lib.stream_ptr(qzeros.device)), 'gptq_unpack_qzeros')
	return out


def dequantize(groupsize: int, qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
			   g_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
	"""fp16 [K, N] weights (q - z - 1) * s, rounded once."""
	_lib.require_cuda(qweight, scales, qzeros, g_idx)
	R, N = qweight.shape
	out = torch.empty((R * 8, N), dtype=torch.float16, device=qweight.device)
	rc = _lib.lib().gptq_dequantize(_lib.ptr(qweight), _lib.ptr(qzeros), _lib.ptr(scales), _lib.ptr(g_idx), _lib.ptr(out), R * 8, N, groupsize, _lib.stream_ptr(qweight.device))
	_lib.check(rc, 'gptq_dequantize')
	return out


class QuantLinear(nn.Module):
	"""4-bit GPTQ linear layer; constructor and buffers as in the reference
	(quant_linear.py:49-73).  `g_idx` is an optional extra buffer."""

	def __init__(self, bits: int, groupsize: int, infeatures: int, outfeatures: int, bias: bool):
		super().__init__()
		if bits not in [4]:
			raise NotImplementedError("Only 4 bits are supported.")
		groupsize = infeatures if groupsize == -1 else groupsize
		self.infeatures = infeatures
		self.outfeatures = outfeatures
		self.bits = bits
		self.groupsize = groupsize
		features_per_int = 32 // bits
		assert outfeatures % features_per_int == 0, "outfeatures must be a multiple of features_per_int"
		self.register_buffer('qweight', torch.empty((infeatures // features_per_int, outfeatures), dtype=torch.int32))
		self.register_buffer('qzeros', torch.empty((math.ceil(infeatures / groupsize), outfeatures // features_per_int), dtype=torch.int32))
		self.register_buffer('scales', torch.empty((math.ceil(infeatures / groupsize), outfeatures), dtype=torch.float16))
		if bias:
			self.register_buffer('bias', torch.empty(outfeatures, dtype=torch.float16))
		else:
			self.register_parameter('bias', None)
		self.register_buffer('g_idx', None)
		# act-order execution state, derived lazily from g_idx
		self._ao_ready = False
		self._ao_perm = None
		self._ao_qweight = None

	def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
		key = prefix + 'g_idx'
		if key in state_dict and self.g_idx is None:
			self.g_idx = torch.empty(self.infeatures, dtype=torch.int32, device=self.qweight.device)
		self._ao_ready = False
		super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

	def _apply(self, fn, recurse=True):
		# .to()/.cuda()/.half(): the derived act-order tensors are rebuilt on next use
		self._ao_ready = False
		self._ao_perm = None
		self._ao_qweight = None
		return super()._apply(fn, recurse)

	def set_g_idx(self, g_idx: Optional[torch.Tensor]):
		self.g_idx = None if g_idx is None else g_idx.to(device=self.qweight.device, dtype=torch.int32)
		self._ao_ready = False

	def _prepare_act_order(self):
		"""Chooses how g_idx is executed: not at all when it is the trivial k // groupsize;
		through row-sorted weights + an activation gather when the groups are equal-sized;
		else through the general kernel that looks up the group of every row."""
		self._ao_perm = None
		self._ao_qweight = None
		self._ao_mode = 'none'
		if self.g_idx is not None:
			g = self.g_idx
			trivial = torch.arange(self.infeatures, device=g.device, dtype=torch.int64) // self.groupsize
			if not torch.equal(g.to(torch.int64), trivial):
				perm = _act_order_perm(g, self.groupsize)
				if perm is not None:
					self._ao_perm = perm
					self._ao_qweight = act_order_rows(self.qweight, perm)
					self._ao_mode = 'sorted'
				else:
					self._ao_mode = 'general'
		self._ao_ready = True

	def kernel_operands(self):
		"""(qweight, g_idx, perm) as the kernels want them."""
		if not self._ao_ready:
			self._prepare_act_order()
		if self._ao_mode == 'sorted':
			return self._ao_qweight, None, self._ao_perm
		if self._ao_mode == 'general':
			return self.qweight, self.g_idx, None
		return self.qweight, None, None

	def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, sumsq_out: Optional[torch.Tensor] = None, ar=None) -> torch.Tensor:
		qw, g_idx, perm = self.kernel_operands()
		return qmatmul(self.groupsize, x, qw, self.scales, self.qzeros, self.bias, g_idx=g_idx, perm=perm, residual=residual,
					   sumsq_out=sumsq_out, ar=ar)
