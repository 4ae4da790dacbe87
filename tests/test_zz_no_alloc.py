"""The allocation-free decode entry point, gptq_qmatmul_noalloc.

Some hosts cannot hand the library scratch memory, or must never trigger an allocation while they
serve requests (their own pool owns the device, or a cudaMalloc-induced device synchronisation is
not acceptable).  For them the library carries a fixed 4 MiB scratch array per GPU and an entry point
that uses it.  This test calls that entry point through the C ABI, twice in a row, and compares
with the regular workspace-based entry point on the same inputs; it also checks that oversized
problems are refused.  The file name keeps it last in collection order.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _ptr(t):
	return None if t is None else ctypes.c_void_p(t.data_ptr())


def _run_both(M, K, N, gs, seed, with_bias_res):
	from gptq_triton_b200 import build, _lib, synth
	from oracle import gptq_oracle as O
	build.build()
	L = _lib.lib()
	dev = torch.device('cuda', 0)
	t = synth.quant_tensors(K, N, gs, seed=seed, bias=with_bias_res)
	x = synth.activations((M, K), seed=seed + 1).to(dev)
	qw, qz, sc = t['qweight'].to(dev), t['qzeros'].to(dev), t['scales'].to(dev)
	bias = t['bias'].to(dev) if with_bias_res else None
	res = synth.activations((M, N), seed=seed + 2).to(dev) if with_bias_res else None
	stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
	# existing entry point (caller-provided workspace)
	ws = _lib.workspace(dev, M, K, N)
	y_ref = torch.empty((M, N), dtype=torch.float16, device=dev)
	rc = L.gptq_qmatmul(_ptr(x), _ptr(qw), _ptr(qz), _ptr(sc), None, None, _ptr(bias), _ptr(res), N, _ptr(y_ref), M, K, N, gs, K, N,
						_ptr(ws), ws.numel(), stream)
	assert rc == 0
	outs = []
	for _ in range(2):          # two calls in a row share the built-in scratch
		y = torch.full((M, N), float('nan'), dtype=torch.float16, device=dev)
		rc = L.gptq_qmatmul_noalloc(_ptr(x), _ptr(qw), _ptr(qz), _ptr(sc), None, _ptr(bias), _ptr(res), N, _ptr(y), M, K, N, gs, K, N, stream)
		assert rc == 0, L.gptq_error_string(rc)
		outs.append(y)
	torch.cuda.synchronize()
	r32 = O.qmatmul_r32(x.cpu(), t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'] if with_bias_res else None,
						residual=res.cpu() if with_bias_res else None)
	return y_ref, outs, r32, O


@pytest.mark.parametrize('M,K,N,gs,extra', [(1, 4096, 4096, 128, False), (5, 1024, 384, 128, True), (16, 2048, 1024, -1, False)])
def test_noalloc_matches_workspace_entry_point(M, K, N, gs, extra):
	y_ref, outs, r32, O = _run_both(M, K, N, gs, seed=7 * M, with_bias_res=extra)
	for y in outs:
		assert not torch.isnan(y).any()
		assert O.max_rel_err(y, y_ref.float().cpu()) <= TOL
		assert O.max_rel_err(y, r32) <= TOL
	assert torch.equal(outs[0], outs[1])


def test_noalloc_act_order_gather_and_status_word():
	"""Act-order weights (rows sorted by group at load, `perm` passed): the gathered x lives in the built-in
	array behind the partial sums.  Afterwards the sticky status word of the array must read healthy."""
	from gptq_triton_b200 import build, _lib, synth
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	from oracle import gptq_oracle as O
	build.build()
	L = _lib.lib()
	dev = torch.device('cuda', 0)
	M, K, N, gs = 3, 2048, 512, 128
	t = synth.quant_tensors(K, N, gs, seed=21, act_order=True)
	x = synth.activations((M, K), seed=22).to(dev)
	g_idx = t['g_idx'].to(dev)
	perm = _act_order_perm(g_idx, gs)
	assert perm is not None
	qw = act_order_rows(t['qweight'].to(dev), perm)
	qz, sc = t['qzeros'].to(dev), t['scales'].to(dev)
	stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
	r32 = O.qmatmul_r32(x.cpu(), t['qweight'], t['qzeros'], t['scales'], gs, g_idx=t['g_idx'])
	for _ in range(2):
		y = torch.full((M, N), float('nan'), dtype=torch.float16, device=dev)
		rc = L.gptq_qmatmul_noalloc(_ptr(x), _ptr(qw), _ptr(qz), _ptr(sc), _ptr(perm), None, None, 0, _ptr(y), M, K, N, gs, K, N, stream)
		assert rc == 0, L.gptq_error_string(rc)
		torch.cuda.synchronize()
		assert O.max_rel_err(y, r32) <= TOL
	assert L.gptq_noalloc_status(0) == 0


def test_noalloc_rejects_what_does_not_fit():
	from gptq_triton_b200 import build, _lib
	build.build()
	L = _lib.lib()
	fake = ctypes.c_void_p(0x1000)
	# unsupported shape for the fast path (N not a multiple of 32): refused before any launch
	assert L.gptq_qmatmul_noalloc(fake, fake, fake, fake, None, None, None, 0, fake, 1, 256, 72, 128, 256, 72, None) == -6
	# M above the decode regime
	assert L.gptq_qmatmul_noalloc(fake, fake, fake, fake, None, None, None, 0, fake, 17, 256, 256, 128, 256, 256, None) == -6
	# a problem whose split-K partial sums exceed the 4 MiB array
	need = L.gptq_noalloc_scratch_bytes(16, 4096, 65536, 128)
	assert need > (4 << 20)
	assert L.gptq_qmatmul_noalloc(fake, fake, fake, fake, None, None, None, 0, fake, 16, 4096, 65536, 128, 4096, 65536, None) == -3
	assert b'scratch' in L.gptq_error_string(-3)
	assert 0 < L.gptq_noalloc_scratch_bytes(1, 4096, 4096, 128) <= (4 << 20)
