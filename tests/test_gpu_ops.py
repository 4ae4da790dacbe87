"""GPU parity tests of the quantised-linear ops (through the C-ABI library) against the CPU oracle.

Tolerances:
  * integer unpack and fp16 dequantise: bit-exact;
  * fp16 matmul outputs: max|y - R32| / max|R32| <= 2e-3 against the fp32-accumulated
    reference (the north-star bound), and <= 0.004 absolute against the golden outputs of the
    reference's own kernel (the Verify.ipynb bound).
"""
import numpy as np
import pytest
import torch

from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3


@pytest.fixture(scope='module')
def G():
	import gptq_triton_b200 as g
	from gptq_triton_b200 import build
	build.build()
	return g


def dev(t):
	return None if t is None else t.cuda()


def synth(K, N, gs, seed, act_order=False, bias=False):
	from gptq_triton_b200 import synth as S
	return S.quant_tensors(K, N, gs, seed, act_order=act_order, bias=bias)


def acts(shape, seed):
	from gptq_triton_b200 import synth as S
	return S.activations(shape, seed)


# ---------------------------------------------------------------- integers, bit-exact
@pytest.mark.parametrize('K,N', [(8, 8), (256, 64), (1024, 4096), (11008, 256)])
def test_unpack_bit_exact(G, K, N):
	t = synth(K, N, 128 if K % 128 == 0 else -1, seed=K + N)
	got = G.unpack_qweight(t['qweight'].cuda()).cpu().numpy()
	assert np.array_equal(got, O.unpack_qweight(t['qweight']))
	gotz = G.unpack_qzeros(t['qzeros'].cuda()).cpu().numpy()
	assert np.array_equal(gotz, O.unpack_qzeros(t['qzeros']))


@pytest.mark.parametrize('K,N,gs,ao', [(256, 64, 128, False), (512, 256, 128, True), (384, 128, -1, False), (1024, 512, 32, True)])
def test_dequantize_bit_exact(G, K, N, gs, ao):
	t = synth(K, N, gs, seed=7, act_order=ao)
	got = G.dequantize(gs, t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), dev(t['g_idx'])).cpu()
	ref = O.dequant_f16(t['qweight'], t['qzeros'], t['scales'], gs, t['g_idx'])
	assert torch.equal(got, ref)


def test_act_order_rows_bit_exact(G):
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	K, N, gs = 512, 128, 128
	t = synth(K, N, gs, seed=11, act_order=True)
	perm = _act_order_perm(t['g_idx'].cuda(), gs)
	assert perm is not None
	sorted_qw = act_order_rows(t['qweight'].cuda(), perm).cpu()
	q = O.unpack_qweight(t['qweight'])
	assert np.array_equal(O.unpack_qweight(sorted_qw), q[perm.cpu().numpy()])
	assert np.array_equal(np.sort(perm.cpu().numpy()), np.arange(K))


# ---------------------------------------------------------------- decode-regime matmul
SHAPES = [
	(256, 256, 128), (512, 384, 128), (1024, 160, 32), (2048, 4096, 128), (4096, 512, -1),
	(1408, 256, 128), (11008, 128, 128), (256, 4096 + 32, 64),
]


@pytest.mark.parametrize('K,N,gs', SHAPES)
@pytest.mark.parametrize('M', [1, 3, 8, 9, 16])
def test_qmatmul_decode(G, M, K, N, gs):
	t = synth(K, N, gs, seed=K * 7 + N)
	x = acts((M, K), seed=M)
	y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda())
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs)
	assert y.shape == (M, N) and y.dtype == torch.float16
	assert O.max_rel_err(y, r32) <= TOL
	# the kernel keeps fp32 weights, so it should sit at fp16 output rounding
	assert O.max_rel_err(y, r32) <= 6e-4


@pytest.mark.parametrize('M', [1, 4, 16])
def test_qmatmul_leading_dims_bias_residual(G, M):
	K, N, gs = 512, 256, 128
	t = synth(K, N, gs, seed=5, bias=True)
	x = acts((2, M, K), seed=3)
	res = acts((2, M, N), seed=4)
	y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda())
	assert y.shape == (2, M, N)
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'], residual=res)
	assert O.max_rel_err(y, r32) <= TOL


@pytest.mark.parametrize('M', [1, 5, 16])
@pytest.mark.parametrize('K,N,gs', [(512, 256, 128), (4096, 384, 128), (1024, 128, 32)])
def test_qmatmul_act_order_sorted_and_general(G, M, K, N, gs):
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	t = synth(K, N, gs, seed=21, act_order=True)
	x = acts((M, K), seed=8)
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, g_idx=t['g_idx'])
	d = {k: dev(v) for k, v in t.items() if isinstance(v, torch.Tensor)}
	# general kernel: g_idx looked up per row, checkpoint layout
	y_gen = G.qmatmul(gs, x.cuda(), d['qweight'], d['scales'], d['qzeros'], g_idx=d['g_idx'])
	assert O.max_rel_err(y_gen, r32) <= TOL
	# prepared path: rows sorted by group + activation gather
	perm = _act_order_perm(d['g_idx'], gs)
	y_srt = G.qmatmul(gs, x.cuda(), act_order_rows(d['qweight'], perm), d['scales'], d['qzeros'], perm=perm)
	assert O.max_rel_err(y_srt, r32) <= TOL


def test_quantlinear_module_act_order_and_state_dict(G):
	K, N, gs = 512, 256, 128
	t = synth(K, N, gs, seed=33, act_order=True, bias=True)
	m = G.QuantLinear(4, gs, K, N, True)
	sd = {'qweight': t['qweight'], 'qzeros': t['qzeros'], 'scales': t['scales'], 'bias': t['bias'], 'g_idx': t['g_idx']}
	m.load_state_dict(sd)
	m = m.cuda()
	x = acts((1, 3, K), seed=9)
	y = m(x.cuda())
	assert m._ao_mode == 'sorted'
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, g_idx=t['g_idx'], bias=t['bias'])
	assert O.max_rel_err(y, r32) <= TOL
	# uneven groups cannot be sorted into equal runs: the general kernel takes over
	g2 = t['g_idx'].clone()
	g2[:7] = g2[7]
	m.set_g_idx(g2)
	y2 = m(x.cuda())
	assert m._ao_mode == 'general'
	r2 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, g_idx=g2, bias=t['bias'])
	assert O.max_rel_err(y2, r2) <= TOL


def test_split_k_variants_agree_and_are_deterministic(G):
	from gptq_triton_b200 import _lib
	K, N, gs, M = 4096, 512, 128, 4
	t = synth(K, N, gs, seed=2)
	x = acts((M, K), seed=2).cuda()
	d = {k: dev(v) for k, v in t.items() if isinstance(v, torch.Tensor)}
	r32 = O.qmatmul_r32(x.cpu(), t['qweight'], t['qzeros'], t['scales'], gs)
	outs = []
	try:
		for sk in (1, 2, 3, 8, 16):
			_lib.lib().gptq_debug_force_splitk(sk)
			a = G.qmatmul(gs, x, d['qweight'], d['scales'], d['qzeros'])
			b = G.qmatmul(gs, x, d['qweight'], d['scales'], d['qzeros'])
			assert torch.equal(a, b), 'same launch configuration must be bit-reproducible'
			assert O.max_rel_err(a, r32) <= 6e-4
			outs.append(a)
	finally:
		_lib.lib().gptq_debug_force_splitk(0)


@pytest.mark.parametrize('name', ['a', 'b', 'c', 'd'])
def test_against_reference_kernel_golden(G, golden_dir, name):
	d = dict(np.load(golden_dir / f'matmul4_{name}.npz'))
	p = dict(np.load(golden_dir / f'pack_{name}.npz'))
	gs = int(d['groupsize'])
	x = torch.from_numpy(d['x'])
	y = G.triton_matmul4(gs if gs != -1 else int(p['K']), x.cuda(), torch.from_numpy(p['qweight']).cuda(),
						 torch.from_numpy(p['scales']).cuda(), torch.from_numpy(p['qzeros']).cuda())
	y_ref = torch.from_numpy(d['y']).float()
	assert (y.cpu().float() - y_ref).abs().max().item() <= 0.004       # Verify.ipynb bound
	assert O.max_rel_err(y, y_ref) <= TOL


# ---------------------------------------------------------------- fused gate/up
@pytest.mark.parametrize('M', [1, 7, 16])
@pytest.mark.parametrize('K,N,gs', [(256, 256, 128), (4096, 1376, 128), (512, 512, -1)])
def test_gateup_silu_decode(G, M, K, N, gs):
	g = synth(K, N, gs, seed=41)
	u = synth(K, N, gs, seed=42)
	x = acts((M, K), seed=43)
	y = G.triton_llama_mlp_4(gs if gs != -1 else K, x.cuda(), g['qweight'].cuda(), g['scales'].cuda(), g['qzeros'].cuda(),
							 u['qweight'].cuda(), u['scales'].cuda(), u['qzeros'].cuda())
	r32 = O.gateup_silu_r32(x, (g['qweight'], g['qzeros'], g['scales']), (u['qweight'], u['qzeros'], u['scales']), gs)
	assert O.max_rel_err(y, r32) <= TOL


@pytest.mark.parametrize('name', ['a', 'b'])
def test_gateup_against_reference_kernel_golden(G, golden_dir, name):
	d = dict(np.load(golden_dir / f'mlp_{name}.npz'))
	gs = int(d['groupsize'])
	x = torch.from_numpy(d['x'])
	K = x.shape[1]
	c = lambda k: torch.from_numpy(d[k]).cuda()
	y = G.triton_llama_mlp_4(gs if gs != -1 else K, x.cuda(), c('gate_qweight'), c('gate_scales'), c('gate_qzeros'),
							 c('up_qweight'), c('up_scales'), c('up_qzeros'))
	y_ref = torch.from_numpy(d['y']).float()
	assert (y.cpu().float() - y_ref).abs().max().item() < 1e-3          # Verify.ipynb fused-MLP bound
	assert O.max_rel_err(y, y_ref) <= TOL


def test_fused_mlp_module_matches_unfused_path(G):
	"""QuantLlamaMLP vs three separate QuantLinear calls + fp16 silu*mul (the reference's
	unfused dequant path), both on the GPU, and both against the oracle."""
	K, I, gs, M = 512, 1408, 128, 5
	g, u, dn = synth(K, I, gs, 51), synth(K, I, gs, 52), synth(I, K, gs, 53)
	x = acts((M, K), seed=54)

	def ql(t, k, n):
		m = G.QuantLinear(4, gs, k, n, False)
		m.load_state_dict({'qweight': t['qweight'], 'qzeros': t['qzeros'], 'scales': t['scales']})
		return m.cuda()
	gate, up, down = ql(g, K, I), ql(u, K, I), ql(dn, I, K)
	fused = G.QuantLlamaMLP(gate, down, up)
	y_f = fused(x.cuda())
	y_u = down(torch.nn.functional.silu(gate(x.cuda())) * up(x.cuda()))
	tri = lambda t: (t['qweight'], t['qzeros'], t['scales'])
	r32 = O.mlp_r32(x, tri(g), tri(u), tri(dn), gs)
	assert O.max_rel_err(y_f, r32) <= TOL
	assert O.max_rel_err(y_u, r32) <= 2 * TOL      # unfused rounds the intermediate three times
	assert O.max_rel_err(y_f, y_u.float().cpu()) <= 2 * TOL


# ---------------------------------------------------------------- fused QKV + rotary
@pytest.mark.parametrize('b,t', [(1, 1), (2, 3), (4, 4), (1, 16)])
@pytest.mark.parametrize('ao', [False, True])
def test_qkv_rope_decode(G, b, t, ao):
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	H, D, K, gs = 2, 128, 512, 128
	hidden = H * D
	w = synth(K, 3 * hidden, gs, seed=61, act_order=ao)
	x = acts((b, t, K), seed=62)
	rng = np.random.default_rng(63)
	pos = torch.from_numpy(rng.integers(0, 2048, size=(b, t)).astype(np.int64))
	cos, sin = O.rope_tables(D, 2048)
	qw = w['qweight'].cuda()
	perm = None
	if ao:
		perm = _act_order_perm(w['g_idx'].cuda(), gs)
		qw = act_order_rows(qw, perm)
	q, k, v = G.qkv_rope(gs, x.cuda(), qw, w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D, perm=perm)
	rq, rk, rv = O.qkv_rope_r32(x, w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D, g_idx=w['g_idx'])
	assert q.shape == (b, H, t, D) and k.shape == (b, H, t, D) and v.shape == (b, H, t, D)
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL
	assert O.max_rel_err(k.transpose(1, 2), rk) <= TOL
	assert O.max_rel_err(v.transpose(1, 2), rv) <= TOL


def test_qkv_rope_writes_kv_cache_in_place(G):
	H, D, K, gs, b, S = 2, 128, 256, 128, 3, 64
	hidden = H * D
	w = synth(K, 3 * hidden, gs, seed=71)
	x = acts((b, 1, K), seed=72)
	pos = torch.tensor([[5], [0], [63]])
	cos, sin = O.rope_tables(D, S)
	kc = torch.full((b, H, S, D), 7.0, dtype=torch.float16, device='cuda')
	vc = torch.full((b, H, S, D), 7.0, dtype=torch.float16, device='cuda')
	q, k2, v2 = G.qkv_rope(gs, x.cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(),
						   pos.cuda(), H, D, kv_cache=(kc, vc))
	assert k2 is kc and v2 is vc
	rq, rk, rv = O.qkv_rope_r32(x, w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D)
	for bi in range(b):
		p = int(pos[bi, 0])
		assert O.max_rel_err(kc[bi, :, p, :], rk[bi, 0]) <= TOL
		assert O.max_rel_err(vc[bi, :, p, :], rv[bi, 0]) <= TOL
		mask = torch.ones(S, dtype=torch.bool)
		mask[p] = False
		assert bool((kc[bi][:, mask, :] == 7.0).all()) and bool((vc[bi][:, mask, :] == 7.0).all())


def test_attention_module_fused_equals_unfused(G):
	"""Verify.ipynb's second check: the fused-QKV module gives the same result as separate q/k/v
	projections followed by rotary, here within fp16 rounding of the rotary arithmetic."""
	from types import SimpleNamespace
	H, D, gs, b, t = 2, 128, 128, 1, 8
	hidden = H * D
	cfg = SimpleNamespace(hidden_size=hidden, num_attention_heads=H, max_position_embeddings=256, rope_theta=10000.0)
	ws = [synth(hidden, hidden, gs, seed=80 + i) for i in range(4)]

	def ql(tn):
		m = G.QuantLinear(4, gs, hidden, hidden, False)
		m.load_state_dict({'qweight': tn['qweight'], 'qzeros': tn['qzeros'], 'scales': tn['scales']})
		return m.cuda()
	holder = torch.nn.Module()
	attn = torch.nn.Module()
	attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj = (ql(w) for w in ws)
	attn.config = cfg
	holder.self_attn = attn
	G.make_quant_attn(holder)
	fused = holder.self_attn
	assert isinstance(fused, G.QuantLlamaAttention) and fused.qkv_proj.outfeatures == 3 * hidden
	x = acts((b, t, hidden), seed=85)
	pos = torch.arange(t).unsqueeze(0)
	mask = torch.full((t, t), float('-inf')).triu(1)[None, None].half()
	out, _, present = fused(x.cuda(), attention_mask=mask.cuda(), position_ids=pos.cuda(), use_cache=True)
	cos, sin = O.rope_tables(D, 256)
	tri = lambda w: (w['qweight'], w['qzeros'], w['scales'])
	qkv = tuple(torch.cat([ws[i][k] for i in range(3)], dim=1) for k in ('qweight', 'qzeros', 'scales'))
	ref, ref_present = O.attention_block_r16(x, qkv, tri(ws[3]), gs, cos, sin, pos, H, attention_mask=mask, use_cache=True)
	assert O.max_rel_err(out, ref.float()) <= 2 * TOL
	assert O.max_rel_err(present[0], ref_present[0].float()) <= 2 * TOL
	# decode one more token with the cache
	x2 = acts((b, 1, hidden), seed=86)
	out2, _, present2 = fused(x2.cuda(), position_ids=torch.tensor([[t]]).cuda(), past_key_value=present, use_cache=True)
	ref2, _ = O.attention_block_r16(x2, qkv, tri(ws[3]), gs, cos, sin, torch.tensor([[t]]), H, past_key_value=ref_present, use_cache=True)
	assert present2[0].shape[2] == t + 1
	assert O.max_rel_err(out2, ref2.float()) <= 2 * TOL


# ---------------------------------------------------------------- full benchmark shapes
@pytest.mark.parametrize('K,N', [(4096, 12288), (4096, 4096), (11008, 4096)])
@pytest.mark.parametrize('M', [1, 16])
def test_full_size_against_gpu_dequant_matmul(G, M, K, N):
	"""At the 7B projection sizes the CPU oracle would take minutes, so the check is the
	dequantise-then-matmul path on the GPU (bit-exact dequantise kernel + fp32 matmul) plus
	linearity in x."""
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	gs = 128
	t = synth(K, N, gs, seed=K + N, act_order=True)
	d = {k: dev(v) for k, v in t.items() if isinstance(v, torch.Tensor)}
	x1, x2 = acts((M, K), 1).cuda(), acts((M, K), 2).cuda()
	perm = _act_order_perm(d['g_idx'], gs)
	qws = act_order_rows(d['qweight'], perm)
	w32 = G.dequantize(gs, d['qweight'], d['scales'], d['qzeros'], d['g_idx']).float()
	prev = torch.backends.cuda.matmul.allow_tf32
	torch.backends.cuda.matmul.allow_tf32 = False
	try:
		r1 = x1.float() @ w32
		r12 = (x1.float() + x2.float()) @ w32
	finally:
		torch.backends.cuda.matmul.allow_tf32 = prev
	y1 = G.qmatmul(gs, x1, qws, d['scales'], d['qzeros'], perm=perm)
	assert O.max_rel_err(y1, r1.cpu()) <= TOL
	y2 = G.qmatmul(gs, x2, qws, d['scales'], d['qzeros'], perm=perm)
	x12 = (x1.float() + x2.float()).half()
	if torch.equal(x12.float(), x1.float() + x2.float()):
		y12 = G.qmatmul(gs, x12, qws, d['scales'], d['qzeros'], perm=perm)
		assert O.max_rel_err(y12, r12.cpu()) <= TOL
	assert O.max_rel_err((y1.float() + y2.float()), (r12).cpu()) <= 2 * TOL


def test_full_size_gateup(G):
	K, N, gs, M = 4096, 11008, 128, 4
	g, u = synth(K, N, gs, 91), synth(K, N, gs, 92)
	x = acts((M, K), 93).cuda()
	dg = {k: dev(v) for k, v in g.items() if isinstance(v, torch.Tensor)}
	du = {k: dev(v) for k, v in u.items() if isinstance(v, torch.Tensor)}
	y = G.gateup_silu(gs, x, dg['qweight'], dg['scales'], dg['qzeros'], du['qweight'], du['scales'], du['qzeros'])
	wg = G.dequantize(gs, dg['qweight'], dg['scales'], dg['qzeros']).float()
	wu = G.dequantize(gs, du['qweight'], du['scales'], du['qzeros']).float()
	prev = torch.backends.cuda.matmul.allow_tf32
	torch.backends.cuda.matmul.allow_tf32 = False
	try:
		a, b = x.float() @ wg, x.float() @ wu
	finally:
		torch.backends.cuda.matmul.allow_tf32 = prev
	ref = a * torch.sigmoid(a) * b
	assert O.max_rel_err(y, ref.cpu()) <= TOL


# ---------------------------------------------------------------- general kernel for M > 16 / odd shapes
@pytest.mark.parametrize('M,K,N,gs', [(17, 256, 256, 128), (40, 512, 72, 128), (100, 256, 256, -1)])
def test_qmatmul_larger_m_and_odd_n(G, M, K, N, gs):
	t = synth(K, N, gs, seed=M)
	x = acts((M, K), seed=M + 1)
	y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda())
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs)
	assert O.max_rel_err(y, r32) <= TOL


def test_empty_batch(G):
	t = synth(256, 256, 128, seed=1)
	x = torch.zeros((0, 256), dtype=torch.float16, device='cuda')
	y = G.qmatmul(128, x, t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda())
	assert y.shape == (0, 256)


# ---------------------------------------------------------------- decode attention + RMSNorm kernels
@pytest.mark.parametrize('b,heads,S,positions', [(1, 4, 300, [0]), (1, 32, 2100, [2047]), (3, 4, 513, [5, 512, 63]), (2, 2, 64, [63, 1]),
												  (16, 8, 2200, [2100 - 37 * i for i in range(16)])])
def test_attn_decode_matches_fp32_reference(G, b, heads, S, positions):
	"""softmax(q K^T / sqrt(d)) V over cache positions 0..pos, fp32 softmax as in
	fused_attention.py:119-137 of the reference, against a float64 evaluation."""
	from gptq_triton_b200.fused_attention import attn_decode
	D = 128
	g = torch.Generator().manual_seed(b * 1000 + S)
	q = torch.randn((b, 1, heads, D), generator=g).half()
	kc = torch.randn((b, heads, S, D), generator=g).half()
	vc = torch.randn((b, heads, S, D), generator=g).half()
	pos = torch.tensor(positions, dtype=torch.int32).view(b, 1)
	out = attn_decode(q.cuda().transpose(1, 2), kc.cuda(), vc.cuda(), pos.cuda(), len_hint=max(positions) + 1).cpu()
	ref = torch.empty((b, heads * D), dtype=torch.float64)
	for i in range(b):
		n = positions[i] + 1
		s = torch.einsum('hd,hsd->hs', q[i, 0].double(), kc[i, :, :n].double()) / D ** 0.5
		ref[i] = torch.einsum('hs,hsd->hd', torch.softmax(s, dim=-1), vc[i, :, :n].double()).reshape(-1)
	assert out.shape == (b, 1, heads * D)
	assert O.max_rel_err(out.view(b, -1), ref.float()) <= TOL


@pytest.mark.parametrize('M,K', [(1, 4096), (5, 512), (16, 11008)])
def test_rmsnorm_kernel(G, M, K):
	from gptq_triton_b200.fused_attention import rmsnorm
	g = torch.Generator().manual_seed(M + K)
	x = (torch.randn((M, K), generator=g) * 3).half()
	w = (torch.rand((K,), generator=g) + 0.5).half()
	y = rmsnorm(x.cuda(), w.cuda(), 1e-6).cpu()
	xd = x.double()
	ref = xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + 1e-6) * w.double()
	assert O.max_rel_err(y, ref.float()) <= 1e-3


# ---------------------------------------------------------------- prefill (M > 16): tcgen05 kernel
TC_SHAPES = [(256, 256, 128), (512, 384, 128), (4096, 512, -1), (1408, 256, 64), (2048, 1024, 128)]


@pytest.mark.parametrize('K,N,gs', TC_SHAPES)
@pytest.mark.parametrize('M', [17, 128, 200, 512])
def test_qmatmul_prefill_tensor_core(G, M, K, N, gs):
	from gptq_triton_b200 import _lib
	from gptq_triton_b200.quant_linear import prefill_kernel_available
	assert prefill_kernel_available(M, K, N, gs)
	t = synth(K, N, gs, seed=K + N + M, bias=True)
	x = acts((M, K), seed=M)
	res = acts((M, N), seed=M + 1)
	y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda())
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'], residual=res)
	assert O.max_rel_err(y, r32) <= TOL
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 0


@pytest.mark.parametrize('M', [64, 300])
def test_prefill_act_order_and_gateup_and_rope(G, M):
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	K, N, gs = 512, 256, 128
	t = synth(K, N, gs, seed=5, act_order=True)
	x = acts((M, K), seed=6)
	d = {k: dev(v) for k, v in t.items() if isinstance(v, torch.Tensor)}
	perm = _act_order_perm(d['g_idx'], gs)
	y = G.qmatmul(gs, x.cuda(), act_order_rows(d['qweight'], perm), d['scales'], d['qzeros'], perm=perm)
	assert O.max_rel_err(y, O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, g_idx=t['g_idx'])) <= TOL
	# fused gate/up
	g, u = synth(K, N, gs, 41), synth(K, N, gs, 42)
	h = G.gateup_silu(gs, x.cuda(), g['qweight'].cuda(), g['scales'].cuda(), g['qzeros'].cuda(), u['qweight'].cuda(), u['scales'].cuda(), u['qzeros'].cuda())
	rh = O.gateup_silu_r32(x, (g['qweight'], g['qzeros'], g['scales']), (u['qweight'], u['qzeros'], u['scales']), gs)
	assert O.max_rel_err(h, rh) <= TOL
	# fused QKV + rotary, prefill layout [1, M, K]
	H, D = 2, 128
	w = synth(K, 3 * H * D, gs, seed=61)
	pos = torch.arange(M).unsqueeze(0)
	cos, sin = O.rope_tables(D, 512)
	q, k, v = G.qkv_rope(gs, x.view(1, M, K).cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D)
	rq, rk, rv = O.qkv_rope_r32(x.view(1, M, K), w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D)
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL and O.max_rel_err(k.transpose(1, 2), rk) <= TOL and O.max_rel_err(v.transpose(1, 2), rv) <= TOL
	# ... and straight into a KV cache
	S = 512
	kc = torch.zeros((1, H, S, D), dtype=torch.float16, device='cuda')
	vc = torch.zeros_like(kc)
	G.qkv_rope(gs, x.view(1, M, K).cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D, kv_cache=(kc, vc))
	assert O.max_rel_err(kc[0, :, :M].transpose(0, 1), rk[0]) <= TOL and O.max_rel_err(vc[0, :, :M].transpose(0, 1), rv[0]) <= TOL
	assert bool((kc[0, :, M:] == 0).all())


@pytest.mark.parametrize('cfg', [1, 2, 3, 4])
@pytest.mark.parametrize('M', [100, 256, 300, 700])
def test_prefill_every_tile_configuration(G, M, cfg):
	"""128 x 128, 128 x 256, 256 x 256 and 256 x 128 tiles of the tensor-core kernel give the same results
	(M = 100 / 300 / 700 leave the last 128-row half partly or wholly empty)."""
	from gptq_triton_b200 import _lib
	K, N, gs, H, D = 512, 768, 128, 2, 128
	t = synth(K, N, gs, seed=cfg + M, bias=True)
	g, u = synth(K, N, gs, 43), synth(K, N, gs, 44)
	w = synth(K, 3 * H * D, gs, seed=62)
	x = acts((M, K), seed=7)
	res = acts((M, N), seed=8)
	pos = torch.arange(M).unsqueeze(0)
	cos, sin = O.rope_tables(D, 1024)
	try:
		_lib.lib().gptq_debug_tc_force(cfg)
		y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda())
		h = G.gateup_silu(gs, x.cuda(), g['qweight'].cuda(), g['scales'].cuda(), g['qzeros'].cuda(), u['qweight'].cuda(), u['scales'].cuda(), u['qzeros'].cuda())
		q, k, v = G.qkv_rope(gs, x.view(1, M, K).cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D)
		torch.cuda.synchronize()
	finally:
		_lib.lib().gptq_debug_tc_force(0)
	assert O.max_rel_err(y, O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'], residual=res)) <= TOL
	assert O.max_rel_err(h, O.gateup_silu_r32(x, (g['qweight'], g['qzeros'], g['scales']), (u['qweight'], u['qzeros'], u['scales']), gs)) <= TOL
	rq, rk, rv = O.qkv_rope_r32(x.view(1, M, K), w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D)
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL and O.max_rel_err(k.transpose(1, 2), rk) <= TOL and O.max_rel_err(v.transpose(1, 2), rv) <= TOL
	assert _lib.kernel_status() == 0


def test_qkv_rope_position_outside_tables_is_reported_not_dereferenced(G):
	"""A position beyond the cos/sin tables must not be used as an index: the kernel computes that
	row at position 0 and raises status 4 in the workspace."""
	from gptq_triton_b200 import _lib
	H, D, K, gs = 2, 128, 256, 128
	w = synth(K, 3 * H * D, gs, seed=5)
	x = acts((1, 2, K), seed=6)
	cos, sin = O.rope_tables(D, 16)
	pos = torch.tensor([[3, 99]])                 # 99 >= 16 rows
	assert _lib.kernel_status() == 0
	q, k, v = G.qkv_rope(gs, x.cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D)
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 4
	rq, _, _ = O.qkv_rope_r32(x, w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, torch.tensor([[3, 0]]), H, D)
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL
	_lib.clear_kernel_status()
	assert _lib.kernel_status() == 0


# ---------------------------------------------------------------- RMSNorm folded into the decode kernels
@pytest.mark.parametrize('M', [1, 5, 16])
@pytest.mark.parametrize('ao', [False, True])
def test_fused_rmsnorm_in_gateup_and_qkv(G, M, ao):
	from gptq_triton_b200.quant_linear import _act_order_perm, act_order_rows
	K, N, gs, H, D = 1024, 384, 128, 2, 128
	rng = torch.Generator().manual_seed(M)
	x = (torch.randn((1, M, K), generator=rng) * 2.5).half()
	gamma = (torch.rand((K,), generator=rng) + 0.5).half()
	xd = x.double()
	xn = (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.double()).half()       # one rounding, as in the kernel
	g, u = synth(K, N, gs, 71, act_order=ao), synth(K, N, gs, 72)
	w = synth(K, 3 * H * D, gs, 73, act_order=ao)
	perm = None
	gq, uq, wq = g['qweight'].cuda(), u['qweight'].cuda(), w['qweight'].cuda()
	if ao:
		perm = _act_order_perm(g['g_idx'].cuda(), gs)
		gq, uq = act_order_rows(gq, perm), act_order_rows(uq, perm)
	y = G.gateup_silu(gs, x.cuda(), gq, g['scales'].cuda(), g['qzeros'].cuda(), uq, u['scales'].cuda(), u['qzeros'].cuda(), perm=perm,
					  rms_weight=gamma.cuda(), rms_eps=1e-6)
	ref = O.gateup_silu_r32(xn, (g['qweight'], g['qzeros'], g['scales']), (u['qweight'], u['qzeros'], u['scales']), gs, g_idx=g['g_idx'])
	assert O.max_rel_err(y, ref) <= TOL
	permw = None
	if ao:
		permw = _act_order_perm(w['g_idx'].cuda(), gs)
		wq = act_order_rows(wq, permw)
	pos = torch.arange(M).unsqueeze(0)
	cos, sin = O.rope_tables(D, 64)
	q, k, v = G.qkv_rope(gs, x.cuda(), wq, w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D, perm=permw,
						 rms_weight=gamma.cuda(), rms_eps=1e-6)
	rq, rk, rv = O.qkv_rope_r32(xn, w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D, g_idx=w['g_idx'])
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL and O.max_rel_err(k.transpose(1, 2), rk) <= TOL and O.max_rel_err(v.transpose(1, 2), rv) <= TOL


@pytest.mark.parametrize('M', [1, 5, 16])
def test_rmsnorm_folded_into_decode_kernels(G, M):
	"""The projection that produces the hidden state leaves per-tile sums of squares; the next
	fused op turns them into the RMSNorm factor while it stages x.  Checked against the
	stand-alone norm (oracle arithmetic) and against the RMSNorm kernel path of the same ops."""
	from gptq_triton_b200 import _lib
	Kp, hidden, inter, gs, H, D = 512, 1024, 384, 128, 8, 128           # hidden = H * D
	rng = torch.Generator().manual_seed(100 + M)
	t = synth(Kp, hidden, gs, 81, bias=True)
	xin = acts((M, Kp), seed=82)
	res = (torch.randn((M, hidden), generator=rng) * 1.5).half()
	ss = torch.zeros((M, hidden // 32), dtype=torch.float32, device='cuda')
	h = G.qmatmul(gs, xin.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda(), sumsq_out=ss)
	h_plain = G.qmatmul(gs, xin.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda())
	assert torch.equal(h, h_plain), 'the extra output must not change y'
	ss_ref = h.float().pow(2).view(M, hidden // 32, 32).sum(-1)
	assert torch.allclose(ss, ss_ref, rtol=1e-5, atol=1e-6)
	# consumers
	gamma = (torch.rand((hidden,), generator=rng) + 0.5).half()
	hd = h.cpu().double()
	xn = (hd * torch.rsqrt(hd.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.double()).half().view(1, M, hidden)
	g, u = synth(hidden, inter, gs, 83), synth(hidden, inter, gs, 84)
	args = (h.view(1, M, hidden), g['qweight'].cuda(), g['scales'].cuda(), g['qzeros'].cuda(), u['qweight'].cuda(), u['scales'].cuda(), u['qzeros'].cuda())
	y = G.gateup_silu(gs, *args, rms_weight=gamma.cuda(), rms_eps=1e-6, sumsq_in=ss)
	y_sep = G.gateup_silu(gs, *args, rms_weight=gamma.cuda(), rms_eps=1e-6)
	ref = O.gateup_silu_r32(xn, (g['qweight'], g['qzeros'], g['scales']), (u['qweight'], u['qzeros'], u['scales']), gs)
	assert O.max_rel_err(y, ref) <= TOL
	assert O.max_rel_err(y, y_sep.float().cpu()) <= 1e-3
	w = synth(hidden, 3 * H * D, gs, 85)
	pos = torch.arange(M).unsqueeze(0)
	cos, sin = O.rope_tables(D, 64)
	qa = (h.view(1, M, hidden), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(), pos.cuda(), H, D)
	q, k, v = G.qkv_rope(gs, *qa, rms_weight=gamma.cuda(), rms_eps=1e-6, sumsq_in=ss)
	rq, rk, rv = O.qkv_rope_r32(xn, w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, pos, H, D)
	assert O.max_rel_err(q.transpose(1, 2), rq) <= TOL and O.max_rel_err(k.transpose(1, 2), rk) <= TOL and O.max_rel_err(v.transpose(1, 2), rv) <= TOL
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 0


def test_rms_folding_rejects_unsupported_shapes(G):
	"""More than 64 producer tiles, or a prefill-sized M, are refused (the caller then uses the RMSNorm kernel)."""
	from gptq_triton_b200 import _lib
	K, N, gs = 256, 256, 128
	t = synth(K, N, gs, 90)
	x = acts((32, K), seed=91).cuda()
	ss = torch.zeros((32, N // 32), dtype=torch.float32, device='cuda')
	with pytest.raises(_lib.GptqB200Error):
		G.qmatmul(gs, x, t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), sumsq_out=ss)


@pytest.mark.parametrize('M', [1, 4, 9, 16])
@pytest.mark.parametrize('K,gs', [(512, 128), (1536, 128), (1024, -1)])
def test_decode_narrow_geometry(G, M, K, gs):
	"""Opt-in geometry: one 32-column strip per CTA over the whole of K (no split-K); same results as the
	tiled split-K form, with bias, residual and the sums of squares."""
	from gptq_triton_b200 import _lib
	N = 4096
	t = synth(K, N, gs, seed=K + M, bias=True)
	x = acts((M, K), seed=M + 3)
	res = acts((M, N), seed=M + 4)
	d = {k: dev(v) for k, v in t.items() if isinstance(v, torch.Tensor)}
	ss = torch.zeros((M, N // 32), dtype=torch.float32, device='cuda')
	ss2 = torch.zeros_like(ss)
	y2 = G.qmatmul(gs, x.cuda(), d['qweight'], d['scales'], d['qzeros'], bias=d['bias'], residual=res.cuda(), sumsq_out=ss2)      # tiled split-K form
	try:
		_lib.lib().gptq_debug_allow_narrow(1)
		y = G.qmatmul(gs, x.cuda(), d['qweight'], d['scales'], d['qzeros'], bias=d['bias'], residual=res.cuda(), sumsq_out=ss)
	finally:
		_lib.lib().gptq_debug_allow_narrow(0)
	r32 = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'], residual=res)
	assert O.max_rel_err(y, r32) <= 6e-4 and O.max_rel_err(y2, r32) <= 6e-4
	assert torch.allclose(ss, y.float().pow(2).view(M, N // 32, 32).sum(-1), rtol=1e-5, atol=1e-6)
	assert torch.allclose(ss2, y2.float().pow(2).view(M, N // 32, 32).sum(-1), rtol=1e-5, atol=1e-6)
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 0


def test_row_parallel_shards_of_an_act_order_layer_on_the_gpu(G):
	"""Tensor-parallel row shards of an act-order layer (full scale / zero tables + a slice of g_idx each), run one
	after the other on this GPU: decode and prefill sizes, the partial sums add up to the oracle's full product."""
	from gptq_triton_b200 import tp
	K, N, gs, world = 1024, 256, 128, 2
	t = synth(K, N, gs, seed=77, act_order=True)
	full = G.QuantLinear(4, gs, K, N, False)
	full.qweight, full.qzeros, full.scales = t['qweight'], t['qzeros'], t['scales']
	full.set_g_idx(t['g_idx'])
	cuts = [0, 520, 1024]
	shards = [tp.shard_rows(full, cuts[r], cuts[r + 1], keep_bias=False).cuda() for r in range(world)]
	for M in (1, 16, 40):
		x = acts((M, K), seed=M)
		ref = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, g_idx=t['g_idx'])
		y = sum(shards[r](x[:, cuts[r]:cuts[r + 1]].contiguous().cuda()).float() for r in range(world))
		assert O.max_rel_err(y, ref) <= 2 * TOL


@pytest.mark.parametrize('sk', [2, 4])
@pytest.mark.parametrize('cfg', [1, 2, 3, 4])
def test_prefill_split_k(G, cfg, sk):
	"""Split-K of the tensor-core kernel (plain epilogue): every tile configuration with 2 and 4 splits, uneven last
	split (K = 1216 = 19 blocks of 64), bias and residual applied by the finishing kernel."""
	from gptq_triton_b200 import _lib
	M, K, N, gs = 300, 1216, 512, 64
	t = synth(K, N, gs, seed=cfg * 10 + sk, bias=True)
	x, res = acts((M, K), seed=3), acts((M, N), seed=4)
	ref = O.qmatmul_r32(x, t['qweight'], t['qzeros'], t['scales'], gs, bias=t['bias'], residual=res)
	try:
		_lib.lib().gptq_debug_tc_force(cfg)
		_lib.lib().gptq_debug_tc_splitk(sk)
		y = G.qmatmul(gs, x.cuda(), t['qweight'].cuda(), t['scales'].cuda(), t['qzeros'].cuda(), bias=t['bias'].cuda(), residual=res.cuda())
		torch.cuda.synchronize()
	finally:
		_lib.lib().gptq_debug_tc_force(0)
		_lib.lib().gptq_debug_tc_splitk(0)
	assert O.max_rel_err(y, ref) <= TOL
	assert _lib.kernel_status() == 0
