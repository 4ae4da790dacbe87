"""ctypes binding of libgptq_b200.so (declared in include/gptq_b200.h).

There is no fallback: if the library is missing or a kernel cannot run, an exception is
raised.  The library is built in-tree by `python -m gptq_triton_b200.build`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / 'libgptq_b200.so'

_lib: Optional[ctypes.CDLL] = None

_P = c_void_p
_SIGNATURES = {
	'gptq_version': (c_int, []),
	'gptq_error_string': (c_char_p, [c_int]),
	'gptq_last_cuda_error': (c_int, []),
	'gptq_workspace_bytes': (c_size_t, [c_int, c_int, c_int]),
	'gptq_qmatmul': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P, c_size_t, _P]),
	'gptq_gateup_silu': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P, c_size_t, _P]),
	'gptq_qkv_rope': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int64, _P, _P, c_int, c_int64, c_int64, c_int64, c_int64,
							  c_int, c_int, c_int, c_int, c_int, c_int64, _P, c_size_t, _P]),
	'gptq_qmatmul_sumsq': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P, c_size_t, _P, _P]),
	'gptq_gateup_silu_rms': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P, c_size_t, _P,
									 _P, _P, c_int, ctypes.c_float]),
	'gptq_qkv_rope_rms': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int64, _P, _P, c_int, c_int64, c_int64, c_int64, c_int64,
								  c_int, c_int, c_int, c_int, c_int, c_int64, _P, c_size_t, _P, _P, _P, c_int, ctypes.c_float]),
	'gptq_ar_partial_bytes': (c_size_t, [c_int]),
	'gptq_ar_flag_bytes': (c_size_t, [c_int]),
	'gptq_qmatmul_ar': (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P, c_size_t, _P, _P,
								c_int, c_int, _P, _P]),
	'gptq_peer_alloc': (c_int, [c_size_t, ctypes.POINTER(c_void_p)]),
	'gptq_peer_free': (c_int, [_P]),
	'gptq_peer_export': (c_int, [_P, _P]),
	'gptq_peer_open': (c_int, [_P, ctypes.POINTER(c_void_p)]),
	'gptq_peer_close': (c_int, [_P]),
	'gptq_unpack_qweight': (c_int, [_P, _P, c_int, c_int, _P]),
	'gptq_unpack_qzeros': (c_int, [_P, _P, c_int, c_int, _P]),
	'gptq_dequantize': (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
	'gptq_act_order_rows': (c_int, [_P, _P, _P, c_int, c_int, _P]),
	'gptq_attn_workspace_bytes': (c_size_t, [c_int, c_int]),
	'gptq_qkv_attn_supported': (c_int, [c_int, c_int, c_int, c_int]),
	'gptq_qkv_attn_decode': (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int, ctypes.c_float, _P, _P, c_int,
									 ctypes.c_float, _P, c_size_t, _P]),
	'gptq_qkv_attn_oproj_scratch_bytes': (c_size_t, [c_int, c_int]),
	'gptq_qkv_attn_oproj_decode': (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int64, c_int, c_int, c_int, c_int, ctypes.c_float, _P, _P, c_int,
										   ctypes.c_float, _P, _P, _P, c_int, c_int, _P, _P, _P, _P, _P, c_size_t, _P, c_size_t, _P]),
	'gptq_qkv_attn_oproj_decode_ar': (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int64, c_int, c_int, c_int, c_int, ctypes.c_float, _P, _P, c_int,
											  ctypes.c_float, _P, _P, _P, c_int, c_int, _P, _P, _P, _P, _P, c_size_t, _P, c_size_t, _P, c_int, c_int, _P, _P]),
	'gptq_attn_decode': (c_int, [_P, c_int64, _P, _P, c_int64, c_int64, _P, _P, c_int64, c_int, c_int, c_int, c_int, ctypes.c_float, _P, c_size_t, _P]),
	'gptq_rmsnorm': (c_int, [_P, c_int64, _P, _P, c_int64, c_int, c_int, ctypes.c_float, _P]),
	'gptq_embed_rmsnorm': (c_int, [_P, c_int64, c_int64, _P, _P, _P, c_int64, _P, c_int64, c_int, c_int, ctypes.c_float, _P]),
	'gptq_qmatmul_noalloc': (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int, c_int64, c_int64, _P]),
	'gptq_noalloc_scratch_bytes': (c_size_t, [c_int, c_int, c_int, c_int]),
	'gptq_noalloc_status': (c_int, [c_int]),
	'gptq_chain_supported': (c_int, [c_int, c_int, c_int, c_int, c_int]),
	'gptq_chain_desc_bytes': (c_size_t, [c_int]),
	'gptq_chain_scratch_bytes': (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
	'gptq_chain_build': (c_int, [_P, c_int, c_int, c_int, _P]),
	'gptq_decode_chain': (c_int, [_P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, c_int64, c_int64, ctypes.c_float,
							  _P, _P, _P, c_size_t, _P]),
	'gptq_lm_head_workspace_bytes': (c_size_t, [c_int]),
	'gptq_lm_head_argmax': (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, ctypes.c_float, _P, _P, _P, _P, c_size_t, _P]),
}
# Entry points outside the header's stable surface (tuning hooks); bound when present.
_OPTIONAL = {
	'gptq_debug_force_splitk': (None, [c_int]),
	'gptq_debug_max_stages': (None, [c_int]),
	'gptq_debug_max_stages2': (None, [c_int]),
	'gptq_debug_set_pdl': (None, [c_int]),
	'gptq_debug_qa_stages': (None, [c_int]),
	'gptq_debug_soft_max_splits': (None, [c_int]),
	'gptq_debug_allow_narrow': (None, [c_int]),
	'gptq_debug_tc_force': (None, [c_int]),
	'gptq_debug_tc_splitk': (None, [c_int]),
	'gptq_debug_chain_stages': (None, [c_int]),
}


def exported_symbols():
	"""Names that include/gptq_b200.h declares."""
	return list(_SIGNATURES)


def lib() -> ctypes.CDLL:
	global _lib
	if _lib is None:
		if not LIB_PATH.exists():
			raise ImportError(
				f'{LIB_PATH} is missing: build it with `python -m gptq_triton_b200.build` '
				'(needs nvcc with sm_100a support). There is no CPU or Triton fallback.')
		l = ctypes.CDLL(str(LIB_PATH))
		for name, (res, args) in _SIGNATURES.items():
			fn = getattr(l, name)
			fn.restype = res
			fn.argtypes = args
		for name, (res, args) in _OPTIONAL.items():
			if hasattr(l, name):
				fn = getattr(l, name)
				fn.restype = res
				fn.argtypes = args
		if os.environ.get('GPTQ_B200_STAGES') and hasattr(l, 'gptq_debug_max_stages'):
			l.gptq_debug_max_stages(int(os.environ['GPTQ_B200_STAGES']))      # ring depth of the decode kernel (A/B measurements)
		if os.environ.get('GPTQ_B200_PDL', '1') == '0' and hasattr(l, 'gptq_debug_set_pdl'):
			l.gptq_debug_set_pdl(0)      # opt out of programmatic dependent launch (A/B measurements)
		_lib = l
	return _lib


class GptqB200Error(RuntimeError):
	pass


def check(code: int, what: str):
	if code != 0:
		l = lib()
		msg = l.gptq_error_string(code).decode()
		extra = f' (cudaError {l.gptq_last_cuda_error()})' if code == -5 else ''
		err = ValueError if code in (-1, -2, -4) else GptqB200Error
		raise err(f'{what}: {msg}{extra}')


def ptr(t: Optional[torch.Tensor]):
	return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device) -> c_void_p:
	return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
	for t in tensors:
		if t is not None and not t.is_cuda:
			raise GptqB200Error('gptq_triton_b200 runs on CUDA tensors only; there is no CPU path')


# One zero-initialised scratch buffer per (device, stream): split-K partial sums and the
# arrival counters that the kernels leave zeroed after each launch.
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def workspace(device: torch.device, M: int, K: int, N: int, min_bytes: int = 0) -> torch.Tensor:
	need = max(lib().gptq_workspace_bytes(M, K, N), min_bytes)
	key = (device.index if device.index is not None else torch.cuda.current_device(),
		   torch.cuda.current_stream(device).cuda_stream)
	ws = _workspaces.get(key)
	if ws is None or ws.numel() < need:
		if ws is not None:
			_retired.append(ws)     # a captured CUDA graph may still point at it
		ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
		_workspaces[key] = ws
	return ws


_retired = []
_status_buffers = []      # scratch areas of other kernels whose status word sits at the same offset (bytes 16380..16383)


def register_status_buffer(buf: torch.Tensor):
	"""Includes the status word of `buf` (a kernel's scratch area, first 16 KiB = control words) in kernel_status()."""
	import weakref
	_status_buffers.append(weakref.ref(buf))


def kernel_status(device=None) -> int:
	"""OR of the status words that the decode kernels keep in their workspaces (0 = healthy;
	1 = a TMA / bulk load never completed within the bounded wait; 2 = shared memory misaligned;
	3 = a wait inside the tensor-core kernel ran out; 4 = position outside the rotary table / cache;
	5 = a peer never arrived in the fused tensor-parallel all-reduce; 6 = a split-K partial sum never arrived;
	7 = a grid barrier of the persistent decode-step kernel timed out)."""
	st = 0
	for (dev, _), ws in _workspaces.items():
		if device is None or dev == (device.index if isinstance(device, torch.device) else device):
			st |= int(ws[16384 - 4:16384].view(torch.int32).item())
	for ref in _status_buffers:
		buf = ref()
		if buf is not None and (device is None or buf.device.index == (device.index if isinstance(device, torch.device) else device)):
			st |= int(buf[16384 - 4:16384].view(torch.int32).item())
	return st


def clear_kernel_status():
	"""Resets the status words (after the cause of a non-zero status has been dealt with)."""
	for ws in _workspaces.values():
		ws[16384 - 4:16384].zero_()
	for ref in _status_buffers:
		buf = ref()
		if buf is not None:
			buf[:16384].zero_()          # also the barrier counters, which a failed run leaves behind
