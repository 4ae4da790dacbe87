"""GPU parity at the sizes the benchmark configurations name (LLaMA-7B projections, M up to 2048).

The shape grid follows the reference's own verification procedure (Verify.ipynb:96-139: M up to 2048,
N and K in {4096, 11008}; :251-306 for the fused MLP).  Every output is compared
  * with the CPU oracle (oracle.gptq_oracle, fp32-accumulated reference R32) — on the whole output where that
    is a matter of seconds, else on a slice of output columns cut on multiples of 8 (the packed tensors are
    sliced, so the oracle computes exactly those columns), and
  * at M = 2048 also with the dequantise-then-matmul path on the GPU (bit-exact dequantise kernel + fp32
    matmul) on the whole output.
Tolerance: max|y - R32| / max|R32| <= 2e-3.
"""
import pytest
import torch

from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3
GS = 128


@pytest.fixture(scope='module')
def G():
	import gptq_triton_b200 as g
	from gptq_triton_b200 import build
	build.build()
	return g


def synth(K, N, gs, seed, act_order=False):
	from gptq_triton_b200 import synth as S
	return S.quant_tensors(K, N, gs, seed, act_order=act_order)


def acts(shape, seed):
	from gptq_triton_b200 import synth as S
	return S.activations(shape, seed)


def cuda(t):
	return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in t.items()}


def col_slice(t, lo, hi):
	"""Columns [lo, hi) of a set of packed tensors (multiples of 8)."""
	assert lo % 8 == 0 and hi % 8 == 0
	return dict(qweight=t['qweight'][:, lo:hi].contiguous(), qzeros=t['qzeros'][:, lo // 8:hi // 8].contiguous(),
				scales=t['scales'][:, lo:hi].contiguous(), g_idx=t['g_idx'])


def gpu_fp32_matmul(x, w32):
	prev = torch.backends.cuda.matmul.allow_tf32
	torch.backends.cuda.matmul.allow_tf32 = False
	try:
		return x.float() @ w32
	finally:
		torch.backends.cuda.matmul.allow_tf32 = prev


# ---------------------------------------------------------------- benchmark configuration 0, exactly
@pytest.fixture(scope='module')
def config0():
	K = N = 4096
	t = synth(K, N, GS, seed=0)
	x = acts((1, 512, K), seed=1)
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], GS)          # 17 GFLOP on the host
	return t, x, r32


@pytest.mark.parametrize('cfg', [0, 1, 2, 3, 4])
def test_config0_prefill_every_tile_configuration_against_the_oracle(G, config0, cfg):
	"""x [1, 512, 4096] through triton_matmul4 (the tcgen05 kernel; 64 K-blocks per tile, so every ring
	wraps many times), once with the automatic tile choice and once per forced tile configuration."""
	from gptq_triton_b200 import _lib
	t, x, r32 = config0
	d = cuda(t)
	try:
		_lib.lib().gptq_debug_tc_force(cfg)
		y = G.triton_matmul4(GS, x.cuda(), d['qweight'], d['scales'], d['qzeros'])
		torch.cuda.synchronize()
	finally:
		_lib.lib().gptq_debug_tc_force(0)
	assert y.shape == (1, 512, 4096) and y.dtype == torch.float16
	assert O.max_rel_err(y.view(512, 4096), r32) <= TOL
	assert _lib.kernel_status() == 0


# ---------------------------------------------------------------- M = 2048 prefill at the 7B shapes (configuration 2 and the bench's prompt)
@pytest.mark.parametrize('gs', [128, -1])
@pytest.mark.parametrize('K,N', [(4096, 4096), (11008, 4096)])
def test_prefill_m2048_projection(G, K, N, gs):
	from gptq_triton_b200 import _lib
	M = 2048
	t = synth(K, N, gs, seed=K + N + (1 if gs == -1 else 0))
	d = cuda(t)
	x = acts((M, K), seed=3)
	y = G.qmatmul(gs, x.cuda(), d['qweight'], d['scales'], d['qzeros'])
	w32 = G.dequantize(gs, d['qweight'], d['scales'], d['qzeros']).float()
	assert O.max_rel_err(y, gpu_fp32_matmul(x.cuda(), w32).cpu()) <= TOL
	for lo in (0, N - 256):                                                  # first and last 256 columns through the CPU oracle
		s = col_slice(t, lo, lo + 256)
		r32 = O.qmatmul_r32(x, s['qweight'], s['qzeros'], s['scales'], gs)
		assert O.max_rel_err(y[:, lo:lo + 256], r32) <= TOL
	assert _lib.kernel_status() == 0


@pytest.mark.parametrize('gs', [128, -1])
def test_prefill_m2048_fused_gateup(G, gs):
	"""silu(x Wg) * (x Wu), 4096 -> 2 x 11008 through the two-stream tile of the tensor-core kernel."""
	from gptq_triton_b200 import _lib
	M, K, N = 2048, 4096, 11008
	g, u = synth(K, N, gs, 71), synth(K, N, gs, 72)
	dg, du = cuda(g), cuda(u)
	x = acts((M, K), seed=5)
	y = G.triton_llama_mlp_4(gs, x.cuda(), dg['qweight'], dg['scales'], dg['qzeros'], du['qweight'], du['scales'], du['qzeros'])
	a = gpu_fp32_matmul(x.cuda(), G.dequantize(gs, dg['qweight'], dg['scales'], dg['qzeros']).float())
	b = gpu_fp32_matmul(x.cuda(), G.dequantize(gs, du['qweight'], du['scales'], du['qzeros']).float())
	assert O.max_rel_err(y, (a * torch.sigmoid(a) * b).cpu()) <= TOL
	for lo in (0, N - 256):
		sg, su = col_slice(g, lo, lo + 256), col_slice(u, lo, lo + 256)
		r32 = O.gateup_silu_r32(x, (sg['qweight'], sg['qzeros'], sg['scales']), (su['qweight'], su['qzeros'], su['scales']), gs)
		assert O.max_rel_err(y[:, lo:lo + 256], r32) <= TOL
	assert _lib.kernel_status() == 0


def test_prefill_m2048_full_mlp_block_against_unfused_reference(G):
	"""Configuration 2 at M = 2048, groupsize 128: down(silu(gate(x)) * up(x)) through QuantLlamaMLP against the
	unfused dequantise path (three matmuls, each rounded to fp16) computed on the GPU in fp32 from the
	bit-exact dequantised weights; threshold as Verify.ipynb:300 scaled to the output range."""
	import gptq_triton_b200 as g
	M, K, I = 2048, 4096, 11008
	tg, tu, td = synth(K, I, GS, 81), synth(K, I, GS, 82), synth(I, K, GS, 83)
	mods = []
	for t, (kin, kout) in zip((tg, td, tu), ((K, I), (I, K), (K, I))):
		m = g.QuantLinear(4, GS, kin, kout, False)
		m.qweight, m.qzeros, m.scales = t['qweight'], t['qzeros'], t['scales']
		mods.append(m.cuda())
	mlp = g.QuantLlamaMLP(*mods)
	x = acts((1, M, K), seed=9) * 0.25
	y = mlp(x.cuda())
	W = [G.dequantize(GS, m.qweight, m.scales, m.qzeros).float() for m in mods]          # gate, down, up
	xs = x.cuda().view(M, K)
	a, b = gpu_fp32_matmul(xs, W[0]), gpu_fp32_matmul(xs, W[2])
	h = (a * torch.sigmoid(a) * b).half()
	ref = gpu_fp32_matmul(h, W[1])
	assert O.max_rel_err(y.view(M, K), ref.cpu()) <= TOL


def test_prefill_m2048_qkv_rope_into_cache(G):
	"""4096 -> 12288 at M = 2048 (the bench's prompt): Q to [b, h, t, d], K / V rows written into a static cache
	at their positions.  Whole output against the GPU dequantise path + rotary in fp32; heads 0 and 31 of all three
	sections against the CPU oracle."""
	from gptq_triton_b200 import _lib
	M, K, H, D = 2048, 4096, 32, 128
	hidden = H * D
	t = synth(K, 3 * hidden, GS, seed=33)
	d = cuda(t)
	x = acts((1, M, K), seed=34)
	S = M + 8
	cos, sin = O.rope_tables(D, S)
	pos = torch.arange(M).unsqueeze(0)
	kc = torch.zeros((1, H, S, D), dtype=torch.float16, device='cuda')
	vc = torch.zeros_like(kc)
	q, k, v = G.qkv_rope(GS, x.cuda(), d['qweight'], d['scales'], d['qzeros'], cos.cuda(), sin.cuda(), pos.cuda(), H, D, kv_cache=(kc, vc))
	torch.cuda.synchronize()
	assert k.data_ptr() == kc.data_ptr() and bool((kc[0, :, M:] == 0).all()) and bool((vc[0, :, M:] == 0).all())
	# whole output on the GPU
	y = gpu_fp32_matmul(x.cuda().view(M, K), G.dequantize(GS, d['qweight'], d['scales'], d['qzeros']).float()).view(M, 3, H, D)
	c, s = cos.cuda().float()[:M].view(M, 1, D), sin.cuda().float()[:M].view(M, 1, D)
	rot = lambda z: torch.cat([-z[..., D // 2:], z[..., :D // 2]], dim=-1)
	rq, rk, rv = y[:, 0] * c + rot(y[:, 0]) * s, y[:, 1] * c + rot(y[:, 1]) * s, y[:, 2]
	assert O.max_rel_err(q[0].transpose(0, 1), rq.cpu()) <= TOL                 # q: [h, t, d] view -> [t, h, d]
	assert O.max_rel_err(kc[0, :, :M].transpose(0, 1), rk.cpu()) <= TOL
	assert O.max_rel_err(vc[0, :, :M].transpose(0, 1), rv.cpu()) <= TOL
	# two heads through the CPU oracle: build the 2-head fused projection from the column slices
	heads = (0, H - 1)
	parts = [col_slice(t, sec * hidden + h * D, sec * hidden + (h + 1) * D) for sec in range(3) for h in heads]
	sub = {n: torch.cat([p[n] for p in parts], dim=1) for n in ('qweight', 'qzeros', 'scales')}
	oq, ok, ov = O.qkv_rope_r32(x, sub['qweight'], sub['qzeros'], sub['scales'], GS, cos, sin, pos, 2, D)      # [1, t, 2, d]
	idx = torch.tensor(heads)
	assert O.max_rel_err(q[0].cpu()[idx].transpose(0, 1), oq[0]) <= TOL                # oracle layout: [t, heads, d]
	assert O.max_rel_err(kc[0].cpu()[idx][:, :M].transpose(0, 1), ok[0]) <= TOL
	assert O.max_rel_err(vc[0].cpu()[idx][:, :M].transpose(0, 1), ov[0]) <= TOL
	assert _lib.kernel_status() == 0


# ---------------------------------------------------------------- benchmark configuration 1: decode sweep, act-order
@pytest.mark.parametrize('M', [1, 4, 16])
@pytest.mark.parametrize('K,N', [(4096, 12288), (4096, 4096), (11008, 4096)])
def test_config1_decode_act_order_against_the_oracle(G, M, K, N):
	"""g_idx = a seeded random permutation of the group assignment; the module path (rows sorted by group at
	load + one gather of x).  The CPU oracle checks 256 output columns at each end."""
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	t = synth(K, N, GS, seed=K + N + 5, act_order=True)
	d = cuda(t)
	x = acts((M, K), seed=M)
	perm = _act_order_perm(d['g_idx'], GS)
	assert perm is not None
	y = G.qmatmul(GS, x.cuda(), act_order_rows(d['qweight'], perm), d['scales'], d['qzeros'], perm=perm)
	w32 = G.dequantize(GS, d['qweight'], d['scales'], d['qzeros'], d['g_idx']).float()
	assert O.max_rel_err(y, gpu_fp32_matmul(x.cuda(), w32).cpu()) <= TOL
	for lo in (0, N - 256):
		s = col_slice(t, lo, lo + 256)
		r32 = O.qmatmul_r32(x, s['qweight'], s['qzeros'], s['scales'], GS, g_idx=t['g_idx'])
		assert O.max_rel_err(y[:, lo:lo + 256], r32) <= TOL


@pytest.mark.parametrize('M', [1, 4, 16])
def test_config1_decode_act_order_gateup_pair(G, M):
	"""The 4096 -> 22016 entry of the sweep: gate and up (2 x 11008) share one act-order g_idx and run as the
	fused kernel; compared as the concatenated projection [gate | up] would be, through silu(g) * u."""
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	K, N = 4096, 11008
	g = synth(K, N, GS, seed=301, act_order=True)
	u = synth(K, N, GS, seed=302)
	u['g_idx'] = g['g_idx']
	dg, du = cuda(g), cuda(u)
	x = acts((M, K), seed=40 + M)
	perm = _act_order_perm(dg['g_idx'], GS)
	y = G.gateup_silu(GS, x.cuda(), act_order_rows(dg['qweight'], perm), dg['scales'], dg['qzeros'],
					  act_order_rows(du['qweight'], perm), du['scales'], du['qzeros'], perm=perm)
	a = gpu_fp32_matmul(x.cuda(), G.dequantize(GS, dg['qweight'], dg['scales'], dg['qzeros'], dg['g_idx']).float())
	b = gpu_fp32_matmul(x.cuda(), G.dequantize(GS, du['qweight'], du['scales'], du['qzeros'], du['g_idx']).float())
	assert O.max_rel_err(y, (a * torch.sigmoid(a) * b).cpu()) <= TOL
	for lo in (0, N - 256):
		sg, su = col_slice(g, lo, lo + 256), col_slice(u, lo, lo + 256)
		r32 = O.gateup_silu_r32(x, (sg['qweight'], sg['qzeros'], sg['scales']), (su['qweight'], su['qzeros'], su['scales']), GS, g_idx=g['g_idx'])
		assert O.max_rel_err(y[:, lo:lo + 256], r32) <= TOL


@pytest.mark.parametrize('gs', [128, -1])
def test_config2_mlp_block_m1(G, gs):
	"""Configuration 2 at M = 1: the fused MLP against the oracle's fp32 MLP (all of it: 3 x 45 M weights at M = 1)."""
	import gptq_triton_b200 as g
	K, I = 4096, 11008
	tg, tu, td = synth(K, I, gs, 91), synth(K, I, gs, 92), synth(I, K, gs, 93)
	mods = []
	for t, (kin, kout) in zip((tg, td, tu), ((K, I), (I, K), (K, I))):
		m = g.QuantLinear(4, gs, kin, kout, False)
		m.qweight, m.qzeros, m.scales = t['qweight'], t['qzeros'], t['scales']
		mods.append(m.cuda())
	mlp = g.QuantLlamaMLP(*mods)
	x = acts((1, 1, K), seed=11) * 0.25
	y = mlp(x.cuda())
	ref = O.mlp_r32(x.view(1, K), (tg['qweight'], tg['qzeros'], tg['scales']), (tu['qweight'], tu['qzeros'], tu['scales']),
					(td['qweight'], td['qzeros'], td['scales']), gs)
	assert O.max_rel_err(y.view(1, K), ref) <= TOL
