"""GPU parity of the one-kernel decode attention (QKV projection + rotary + cache append + single-query attention,
one cluster of 8 CTAs per head) against the CPU oracle and against the two-kernel path.

Tolerance: max|y - R| / max|R| <= 2e-3 for q-side results compared through the attention output, K / V cache rows
against the fp32 oracle projection at the same bound; untouched cache rows must stay bit-identical.
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


def synth(K, N, gs, seed):
	from gptq_triton_b200 import synth as S
	return S.quant_tensors(K, N, gs, seed)


def acts(shape, seed):
	from gptq_triton_b200 import synth as S
	return S.activations(shape, seed)


def oracle_attention(x, w, gs, cos, sin, pos, H, D, kc, vc):
	"""fp64 attention over the cache rows 0..pos-1 plus the token's own fp16-rounded key / value."""
	p = torch.tensor([[pos]])
	rq, rk, rv = O.qkv_rope_r32(x.view(1, 1, -1), w['qweight'], w['qzeros'], w['scales'], gs, cos, sin, p, H, D)
	q, k, v = rq[0, 0].half().double(), rk[0, 0].half().double(), rv[0, 0].half().double()
	keys = torch.cat([kc[:, :pos].double(), k.view(H, 1, D)], dim=1)
	vals = torch.cat([vc[:, :pos].double(), v.view(H, 1, D)], dim=1)
	s = torch.einsum('hd,hsd->hs', q, keys) / D ** 0.5
	return torch.einsum('hs,hsd->hd', torch.softmax(s, dim=-1), vals).reshape(-1).float(), rk[0, 0], rv[0, 0]


@pytest.mark.parametrize('K,H,gs,S,pos', [(1024, 2, 128, 96, 0), (1024, 2, 128, 96, 7), (1024, 4, 128, 700, 699), (2048, 3, 256, 300, 130),
										  (4096, 32, 128, 2304, 2111), (1024, 2, -1, 96, 64), (8192, 2, 128, 160, 100)])
def test_qkv_attn_against_oracle(G, K, H, gs, S, pos):
	from gptq_triton_b200.fused_attention import qkv_attn_decode, qkv_attn_supported
	from gptq_triton_b200 import _lib
	D = 128
	assert qkv_attn_supported(K, H, D, gs)
	w = synth(K, 3 * H * D, gs, seed=K + H)
	x = acts((1, 1, K), seed=pos + 5)
	g = torch.Generator().manual_seed(S + pos)
	kc = torch.randn((1, H, S, D), generator=g).half()
	vc = torch.randn((1, H, S, D), generator=g).half()
	cos, sin = O.rope_tables(D, S)
	kd, vd = kc.cuda(), vc.cuda()
	out = qkv_attn_decode(gs, x.cuda(), w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(),
						  torch.tensor([pos], dtype=torch.int32).cuda(), kd, vd, H)
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 0
	ref, rk, rv = oracle_attention(x, w, gs, cos, sin, pos, H, D, kc[0], vc[0])
	assert out.shape == (1, 1, H * D)
	assert O.max_rel_err(out.view(-1).cpu(), ref) <= TOL
	# the cache: row `pos` holds the new key / value, every other row is untouched
	assert O.max_rel_err(kd[0, :, pos].cpu(), rk) <= TOL
	assert O.max_rel_err(vd[0, :, pos].cpu(), rv) <= TOL
	mask = torch.ones(S, dtype=torch.bool)
	mask[pos] = False
	assert torch.equal(kd[0][:, mask].cpu(), kc[0][:, mask]) and torch.equal(vd[0][:, mask].cpu(), vc[0][:, mask])


def test_qkv_attn_equals_two_kernel_path_with_folded_rmsnorm(G):
	"""Same inputs through gptq_qkv_rope_rms + gptq_attn_decode: the cache rows agree to the last bit or one fp16 ulp of
	the largest value (the K dimension is summed in a different order), the attention outputs within the parity bound."""
	from gptq_triton_b200.fused_attention import attn_decode, qkv_attn_decode, qkv_rope
	K, H, D, gs, S, pos = 4096, 32, 128, 128, 2304, 2050
	w = synth(K, 3 * H * D, gs, seed=11)
	h = acts((1, 1, K), seed=12).cuda()
	lnw = (1.0 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(13))).half().cuda()
	ss = (h.float().view(K // 32, 32) ** 2).sum(-1).contiguous()
	g = torch.Generator().manual_seed(14)
	kc = torch.randn((1, H, S, D), generator=g).half().cuda()
	vc = torch.randn((1, H, S, D), generator=g).half().cuda()
	cos, sin = O.rope_tables(D, S)
	cos, sin = cos.cuda(), sin.cuda()
	p = torch.tensor([[pos]], dtype=torch.int32).cuda()
	qw, sc, qz = w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda()
	k1, v1 = kc.clone(), vc.clone()
	o1 = qkv_attn_decode(gs, h, qw, sc, qz, cos, sin, p.view(-1), k1, v1, H, rms_weight=lnw, rms_eps=1e-6, sumsq_in=ss)
	k2, v2 = kc.clone(), vc.clone()
	q, _, _ = qkv_rope(gs, h, qw, sc, qz, cos, sin, p, H, D, kv_cache=(k2, v2), rms_weight=lnw, rms_eps=1e-6, sumsq_in=ss)
	o2 = attn_decode(q, k2, v2, p, len_hint=pos + 1)
	torch.cuda.synchronize()
	assert O.max_rel_err(k1[0, :, pos].cpu(), k2[0, :, pos].float().cpu()) <= 1e-3
	assert O.max_rel_err(v1[0, :, pos].cpu(), v2[0, :, pos].float().cpu()) <= 1e-3
	assert O.max_rel_err(o1.view(-1).cpu(), o2.view(-1).float().cpu()) <= TOL
	# deterministic: a second run gives the same bits
	k3, v3 = kc.clone(), vc.clone()
	o3 = qkv_attn_decode(gs, h, qw, sc, qz, cos, sin, p.view(-1), k3, v3, H, rms_weight=lnw, rms_eps=1e-6, sumsq_in=ss)
	assert torch.equal(o1, o3) and torch.equal(k1, k3) and torch.equal(v1, v3)


@pytest.mark.parametrize('K,H,gs,S,pos,resid', [(1024, 8, 128, 96, 7, True), (4096, 32, 128, 2304, 2111, True), (2048, 16, 256, 300, 130, False),
												(1024, 8, -1, 64, 0, True)])
def test_qkv_attn_oproj_against_oracle(G, K, H, gs, S, pos, resid):
	"""The whole attention block in one kernel: y = residual + attention x deq(Wo), with the sums of squares of y."""
	from gptq_triton_b200.fused_attention import qkv_attn_oproj_decode, qkv_attn_oproj_scratch
	from gptq_triton_b200 import _lib
	D = 128
	hidden = H * D
	assert hidden == K
	w = synth(K, 3 * hidden, gs, seed=K + H)
	wo = synth(hidden, hidden, gs, seed=K + H + 1)
	x = acts((1, 1, K), seed=pos + 5)
	g = torch.Generator().manual_seed(S + pos)
	kc = torch.randn((1, H, S, D), generator=g).half()
	vc = torch.randn((1, H, S, D), generator=g).half()
	cos, sin = O.rope_tables(D, S)
	kd, vd = kc.cuda(), vc.cuda()
	scratch = qkv_attn_oproj_scratch(H, hidden, 'cuda')
	ss = torch.zeros(hidden // 32, dtype=torch.float32, device='cuda')
	attn_out = torch.zeros((1, 1, hidden), dtype=torch.float16, device='cuda')
	xd = x.cuda()
	outs = []
	for _ in range(2):          # the second call finds the arrival counters as the first one left them
		kd.copy_(kc), vd.copy_(vc)
		y = qkv_attn_oproj_decode(gs, xd, w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(),
								  torch.tensor([pos], dtype=torch.int32).cuda(), kd, vd, H, gs, wo['qweight'].cuda(), wo['scales'].cuda(),
								  wo['qzeros'].cuda(), scratch, residual=xd if resid else None, sumsq_out=ss, attn_out=attn_out)
		outs.append((y.clone(), ss.clone()))
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 0
	assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
	ref_attn, rk, rv = oracle_attention(x, w, gs, cos, sin, pos, H, D, kc[0], vc[0])
	assert O.max_rel_err(attn_out.view(-1).cpu(), ref_attn) <= TOL
	# o_proj on the kernel's own fp16 attention output, fp32 accumulation, then the residual
	a16 = attn_out.view(1, -1).cpu()
	ref = O.qmatmul_r32(a16, wo['qweight'], wo['qzeros'], wo['scales'], gs).view(-1)
	if resid:
		ref = ref + x.view(-1).float()
	assert y.shape == (1, 1, hidden)
	assert O.max_rel_err(y.view(-1).cpu(), ref) <= TOL
	yf = y.view(-1).float().cpu()
	assert torch.allclose(ss.cpu(), (yf.view(-1, 32) ** 2).sum(-1), rtol=1e-5, atol=1e-6)
	assert O.max_rel_err(kd[0, :, pos].cpu(), rk) <= TOL and O.max_rel_err(vd[0, :, pos].cpu(), rv) <= TOL


def test_qkv_attn_position_outside_the_cache_is_reported(G):
	from gptq_triton_b200.fused_attention import qkv_attn_decode
	from gptq_triton_b200 import _lib
	K, H, D, gs, S = 1024, 2, 128, 128, 64
	w = synth(K, 3 * H * D, gs, seed=3)
	x = acts((1, 1, K), seed=4).cuda()
	kc = torch.full((1, H, S, D), 3.0, dtype=torch.float16, device='cuda')
	vc = torch.full((1, H, S, D), 3.0, dtype=torch.float16, device='cuda')
	cos, sin = O.rope_tables(D, S)
	assert _lib.kernel_status() == 0
	out = qkv_attn_decode(gs, x, w['qweight'].cuda(), w['scales'].cuda(), w['qzeros'].cuda(), cos.cuda(), sin.cuda(),
						  torch.tensor([S], dtype=torch.int32).cuda(), kc, vc, H)
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 4
	assert bool((kc == 3.0).all()) and bool((vc == 3.0).all())        # nothing was written
	assert bool((out == 0).all())
	_lib.clear_kernel_status()
	assert _lib.kernel_status() == 0


def test_unsupported_shapes_are_refused(G):
	from gptq_triton_b200.fused_attention import qkv_attn_supported
	assert not qkv_attn_supported(512, 2, 128, 128)          # K not a multiple of 1024
	assert not qkv_attn_supported(1024, 2, 64, 128)          # head_dim
	assert not qkv_attn_supported(1024, 2, 128, 32)          # groups smaller than a chunk of 128 rows
	assert not qkv_attn_supported(16384, 2, 128, 128)        # more than 8 chunks per CTA
