"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, and its pure-host entry points answer.  No kernel is launched."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope='module')
def lib():
	from gptq_triton_b200 import build, _lib
	build.build()
	return _lib.lib()


def declared_symbols():
	text = (ROOT / 'include' / 'gptq_b200.h').read_text()
	text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
	return sorted(set(re.findall(r'\b(gptq_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_exported(lib):
	names = declared_symbols()
	assert len(names) >= 10
	for n in names:
		assert hasattr(lib, n), f'{n} declared in include/gptq_b200.h but not exported'


def test_binding_covers_header(lib):
	from gptq_triton_b200 import _lib
	assert sorted(_lib.exported_symbols()) == declared_symbols()


def test_host_entry_points(lib):
	assert lib.gptq_version() >= 100
	assert lib.gptq_error_string(0) == b'ok'
	for code in range(-6, 0):
		assert len(lib.gptq_error_string(code)) > 3
	assert lib.gptq_error_string(-99) == b'unknown error code'
	small = lib.gptq_workspace_bytes(1, 4096, 4096)
	big = lib.gptq_workspace_bytes(16, 4096, 22016)
	assert 0 < small < big < (256 << 20)


def test_argument_errors_before_any_launch(lib):
	"""Invalid arguments are rejected on the host; nothing touches the GPU."""
	fake = ctypes.c_void_p(0x1000)
	args = lambda x=fake, M=1, K=256, N=256, gs=128, ldx=256: (
		x, fake, fake, fake, None, None, None, None, 0, fake, M, K, N, gs, ldx, N, None, 0, None)
	assert lib.gptq_qmatmul(*args(x=None)) == -1
	assert lib.gptq_qmatmul(*args(K=12)) == -2
	assert lib.gptq_qmatmul(*args(x=ctypes.c_void_p(0x1004))) == -4
	assert lib.gptq_qmatmul(*args(ldx=100)) == -1
	assert lib.gptq_qmatmul(*args(M=0)) == 0          # empty batch: nothing to do
	assert lib.gptq_qmatmul(*args(gs=0)) == -1


def test_extension_entry_points_validate_on_the_host(lib):
	"""The entry points without a reference counterpart (folded RMSNorm, fused tensor-parallel all-reduce)
	reject bad arguments before anything touches the GPU; their sizing helpers are pure host code."""
	fake = ctypes.c_void_p(0x1000)
	base = (fake, fake, fake, fake, None, None, None, None, 0, fake, 1, 256, 256, 128, 256, 256, None, 0, None)
	assert lib.gptq_qmatmul_sumsq(*base, None) == -1                      # the extra output is required
	ptrs = (ctypes.c_void_p * 8)(*([0x2000] * 2 + [None] * 6))
	assert lib.gptq_qmatmul_ar(*base, None, 1, 0, ptrs, ptrs) == -1       # a world of one has nothing to exchange
	assert lib.gptq_qmatmul_ar(*base, None, 2, 2, ptrs, ptrs) == -1       # rank outside the world
	assert lib.gptq_qmatmul_ar(*base, None, 9, 0, ptrs, ptrs) == -1       # more than eight ranks
	assert lib.gptq_qmatmul_ar(*base, None, 2, 0, None, ptrs) == -1
	wide = tuple(base[:10]) + (32,) + tuple(base[11:])                     # M = 32: no decode kernel, no fused exchange
	assert lib.gptq_qmatmul_ar(*wide, None, 2, 0, ptrs, ptrs) == -6
	gu = (fake, fake, fake, fake, fake, fake, fake, None, None, fake, 1, 256, 256, 128, 256, 256, None, 0, None)
	assert lib.gptq_gateup_silu_rms(*gu, None, None, 0, 1e-6) == -1      # norm weight required
	assert lib.gptq_gateup_silu_rms(*gu, fake, None, 8, 1e-6) == -1      # ... and the sums of squares
	assert lib.gptq_gateup_silu_rms(*gu, fake, fake, 300, 1e-6) == -6    # more partial sums than the kernel folds
	assert lib.gptq_ar_partial_bytes(4096) == 2 * 8 * 32 * 16 * 128 * 8      # two halves (parity of the sequence number)
	assert lib.gptq_ar_flag_bytes(4096) % 256 == 0 and lib.gptq_ar_flag_bytes(4096) >= 32 * 4
	assert lib.gptq_peer_alloc(0, None) == -1 and lib.gptq_peer_export(None, None) == -1 and lib.gptq_peer_open(None, None) == -1
	assert lib.gptq_peer_free(None) == 0 and lib.gptq_peer_close(None) == 0


def test_attention_block_entry_points_validate_on_the_host(lib):
	"""The one-kernel attention block (gptq_qkv_attn_*): shape rule, scratch size and argument checks are host
	arithmetic; nothing is launched."""
	assert lib.gptq_qkv_attn_supported(4096, 32, 128, 128) == 1
	assert lib.gptq_qkv_attn_supported(4096, 4, 128, -1) == 1          # a tensor-parallel shard: few heads, full K
	assert lib.gptq_qkv_attn_supported(8192, 64, 128, 256) == 1
	assert lib.gptq_qkv_attn_supported(5120, 40, 128, 128) == 1
	assert lib.gptq_qkv_attn_supported(4096 + 512, 32, 128, 128) == 0  # K not a multiple of 1024
	assert lib.gptq_qkv_attn_supported(16384, 32, 128, 128) == 0       # more than 8 chunks of 128 rows per CTA
	assert lib.gptq_qkv_attn_supported(4096, 32, 64, 128) == 0         # head_dim
	assert lib.gptq_qkv_attn_supported(4096, 32, 128, 64) == 0         # groups smaller than a chunk
	assert lib.gptq_qkv_attn_oproj_scratch_bytes(32, 4096) == 256 + 32 * 4096 * 4
	assert lib.gptq_qkv_attn_oproj_scratch_bytes(0, 4096) == 0
	buf = (ctypes.c_ubyte * 64)()
	p = ctypes.cast(buf, ctypes.c_void_p)
	# null pointers and an unsupported shape are refused before anything touches the device
	assert lib.gptq_qkv_attn_decode(None, p, p, p, p, p, p, 64, p, p, 64 * 128, p, 4096, 32, 128, 128, 0.088, None, None, 0, 0.0, p, 1 << 20, None) == -1
	assert lib.gptq_qkv_attn_decode(p, p, p, p, p, p, p, 64, p, p, 64 * 128, p, 4608, 36, 128, 128, 0.088, None, None, 0, 0.0, p, 1 << 20, None) == -6
	assert lib.gptq_qkv_attn_oproj_decode_ar(p, p, p, p, p, p, p, 64, p, p, 64 * 128, 4096, 32, 128, 128, 0.088, None, None, 0, 0.0, p, p, p, 4096, 128,
											 None, p, None, None, p, 1 << 20, p, 1 << 20, None, 1, 0, None, None) == -1          # a world of one rank


def test_python_ops_refuse_cpu_tensors():
	import torch
	import gptq_triton_b200 as g
	from gptq_triton_b200._lib import GptqB200Error
	x = torch.zeros(1, 256, dtype=torch.float16)
	qw = torch.zeros(32, 256, dtype=torch.int32)
	qz = torch.zeros(2, 32, dtype=torch.int32)
	sc = torch.zeros(2, 256, dtype=torch.float16)
	with pytest.raises(GptqB200Error):
		g.triton_matmul4(128, x, qw, sc, qz)
	with pytest.raises(AssertionError):
		g.triton_matmul4(128, torch.zeros(1, 250, dtype=torch.float16), qw, sc, qz)
