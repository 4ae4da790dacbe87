"""Pins the CPU oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py): its packer / RTN quantiser, its two Triton kernels run by
the Triton interpreter, and transformers' rotary embedding."""
import numpy as np
import pytest
import torch

from oracle import gptq_oracle as O

PACKS = ['a', 'b', 'c', 'd']


def _load(golden_dir, name):
	return dict(np.load(golden_dir / name))


@pytest.mark.parametrize('name', PACKS)
def test_unpack_matches_reference_packer(golden_dir, name):
	d = _load(golden_dir, f'pack_{name}.npz')
	K, N, gs = int(d['K']), int(d['N']), int(d['groupsize'])
	gsz = K if gs == -1 else gs
	# integers the reference packed: round((w + z*s)/s) per quantize.py:256
	s = torch.from_numpy(d['scale']).t().contiguous()
	z = torch.from_numpy(d['zero']).t().contiguous()
	g = torch.arange(K) // gsz
	q = torch.round((torch.from_numpy(d['fakequant']).t() + (z * s)[g]) / s[g]).to(torch.int32).numpy()
	assert np.array_equal(O.unpack_qweight(d['qweight']), q.astype(np.uint8))
	assert np.array_equal(O.unpack_qzeros(d['qzeros']).astype(np.int32) + 1, z.numpy().astype(np.int32))
	# our packer is the bit-exact inverse
	assert np.array_equal(O.pack_qweight(q), d['qweight'])
	assert np.array_equal(O.pack_qzeros(z.numpy().astype(np.int32) - 1), d['qzeros'])


@pytest.mark.parametrize('name', PACKS)
def test_rtn_and_pack_restatement(golden_dir, name):
	"""rtn_quantize + pack_linear reproduce dumbquant + pack_linear bit for bit when fed the
	same initial weights; the fixture only holds the fake-quantised weights, and
	quantising those again is idempotent on the integer grid."""
	d = _load(golden_dir, f'pack_{name}.npz')
	gs = int(d['groupsize'])
	fq = torch.from_numpy(d['fakequant'])
	qw, qz, sc = O.pack_linear(fq, torch.from_numpy(d['scale']), torch.from_numpy(d['zero']), gs)
	assert np.array_equal(qw.numpy(), d['qweight'])
	assert np.array_equal(qz.numpy(), d['qzeros'])
	assert np.array_equal(sc.numpy(), d['scales'])


@pytest.mark.parametrize('name', PACKS)
def test_dequant_matches_fakequant(golden_dir, name):
	d = _load(golden_dir, f'pack_{name}.npz')
	gs = int(d['groupsize'])
	w = O.dequant_f32(d['qweight'], d['qzeros'], torch.from_numpy(d['scales']), gs)   # [K, N]
	ref = torch.from_numpy(d['fakequant']).t()
	# only difference: the packed scale is rounded to fp16 (rel 2^-11), |q-z| <= 15
	tol = 15 * torch.from_numpy(d['scale']).max().item() * 2 ** -11 * 1.01
	assert (w - ref).abs().max().item() <= tol


@pytest.mark.parametrize('name', PACKS)
def test_matmul4_kernel_outputs(golden_dir, name):
	d = _load(golden_dir, f'matmul4_{name}.npz')
	p = _load(golden_dir, f'pack_{name}.npz')
	gs = int(d['groupsize'])
	x = torch.from_numpy(d['x'])
	y_ref = torch.from_numpy(d['y']).float()
	sc = torch.from_numpy(p['scales'])
	# emulation of the kernel's own arithmetic: equal up to fp32 summation order
	y_k = O.qmatmul_kernel_form(x, p['qweight'], p['qzeros'], sc, gs).float()
	assert (y_k - y_ref).abs().max().item() <= 2 * 2 ** -10 * y_ref.abs().max().item()
	assert (y_k == y_ref).float().mean().item() > 0.9
	# the fp32-accumulated reference is within the north-star bound of the kernel
	r32 = O.qmatmul_r32(x, p['qweight'], p['qzeros'], sc, gs)
	assert O.max_rel_err(y_ref, r32) < 2e-3
	# and the dequantise-then-matmul path agrees with both
	r16 = O.qmatmul_r16(x, p['qweight'], p['qzeros'], sc, gs)
	assert O.max_rel_err(r16, r32) < 2e-3


@pytest.mark.parametrize('name', ['a', 'b'])
def test_fused_mlp_kernel_outputs(golden_dir, name):
	d = _load(golden_dir, f'mlp_{name}.npz')
	gs = int(d['groupsize'])
	x = torch.from_numpy(d['x'])
	gate = (d['gate_qweight'], d['gate_qzeros'], torch.from_numpy(d['gate_scales']))
	up = (d['up_qweight'], d['up_qzeros'], torch.from_numpy(d['up_scales']))
	y_ref = torch.from_numpy(d['y']).float()
	y_k = O.gateup_silu_kernel_form(x, gate, up, gs).float()
	assert (y_k - y_ref).abs().max().item() <= 2 * 2 ** -10 * y_ref.abs().max().item()
	r32 = O.gateup_silu_r32(x, gate, up, gs)
	assert O.max_rel_err(y_ref, r32) < 2e-3


def test_rope_matches_transformers(golden_dir):
	d = _load(golden_dir, 'rope.npz')
	q, k = torch.from_numpy(d['q']), torch.from_numpy(d['k'])
	pos = torch.from_numpy(d['pos'])
	cos, sin = O.rope_tables(q.shape[-1], 2048, float(d['theta']))
	qo, ko = O.apply_rope(q, k, cos, sin, pos)
	assert torch.equal(qo, torch.from_numpy(d['q_out']))
	assert torch.equal(ko, torch.from_numpy(d['k_out']))


def test_g_idx_default_equals_explicit():
	K, N, gs = 256, 64, 128
	rng = np.random.default_rng(0)
	qw = O.pack_qweight(rng.integers(0, 16, (K, N)))
	qz = O.pack_qzeros(rng.integers(0, 16, (K // gs, N)))
	sc = torch.from_numpy(rng.uniform(0.002, 0.02, (K // gs, N)).astype(np.float16))
	a = O.dequant_f32(qw, qz, sc, gs)
	b = O.dequant_f32(qw, qz, sc, gs, g_idx=np.arange(K) // gs)
	assert torch.equal(a, b)
	perm = rng.permutation(K)
	c = O.dequant_f32(qw, qz, sc, gs, g_idx=(np.arange(K) // gs)[perm])
	assert not torch.equal(a, c)
