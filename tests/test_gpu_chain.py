"""The persistent decode-step kernel (gptq_decode_chain) and the lm_head / arg-max kernel (gptq_lm_head_argmax).

The chain kernel has no separate CPU oracle of its own: a decode step is a composition of the ops that the other
GPU tests pin to the oracle one by one (quantised matmuls, rotary, attention, RMSNorm), so it is compared
  * with the kernel-per-projection engine on the same model and tokens (logits of every step to fp16 rounding,
    tokens identical), for batch sizes 1, 2, 4 and 8, and
  * through the greedy-decoding tests of test_gpu_decode.py against the dequantise-then-matmul twin.
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def G():
	import gptq_triton_b200 as g
	from gptq_triton_b200 import build
	build.build()
	return g


@pytest.mark.parametrize('M,K,V', [(1, 4096, 32000), (3, 512, 1000), (8, 1024, 517)])
def test_lm_head_argmax_kernel(G, M, K, V):
	"""logits = rmsnorm(h) @ W^T within 2e-3 of an fp32 reference, identical arg-max, positions advanced."""
	from gptq_triton_b200 import _lib
	L = _lib.lib()
	gen = torch.Generator().manual_seed(M * 7 + K)
	h = (torch.randn((M, K), generator=gen) * 3).half().cuda()
	w_norm = (1 + 0.1 * torch.randn((K,), generator=gen)).half().cuda()
	W = (torch.randn((V, K), generator=gen) * 0.02).half().cuda()
	ss = h.float().pow(2).view(M, K // 32, 32).sum(-1).contiguous()
	logits = torch.zeros((M, V), dtype=torch.float16, device='cuda')
	tok = torch.full((M,), -1, dtype=torch.int64, device='cuda')
	pos = torch.arange(10, 10 + M, dtype=torch.int32, device='cuda')
	ws = torch.zeros(L.gptq_lm_head_workspace_bytes(M), dtype=torch.uint8, device='cuda')
	eps = 1e-6
	for _ in range(2):          # the ticket is left ready for the next call
		rc = L.gptq_lm_head_argmax(_lib.ptr(h), _lib.ptr(ss), _lib.ptr(w_norm), _lib.ptr(W), M, K, V, eps, _lib.ptr(logits), _lib.ptr(tok), _lib.ptr(pos),
								   _lib.ptr(ws), ws.numel(), _lib.stream_ptr(h.device))
		assert rc == 0, L.gptq_error_string(rc)
	torch.cuda.synchronize()
	x = (h.float() * torch.rsqrt(h.float().pow(2).mean(-1, keepdim=True) + eps) * w_norm.float()).half()
	ref = x.float() @ W.float().t()
	err = (logits.float() - ref).abs().max().item() / ref.abs().max().item()
	assert err <= 2e-3, err
	assert torch.equal(tok.cpu(), logits.float().argmax(-1).cpu())
	assert torch.equal(pos.cpu(), torch.arange(12, 12 + M, dtype=torch.int32))


def _engines(G, cfg, batch, max_seq, seed):
	model = G.synthetic_quantized_llama(cfg, groupsize=128, seed=seed, device='cuda')
	old = os.environ.get('GPTQ_B200_CHAIN')
	try:
		os.environ['GPTQ_B200_CHAIN'] = '1'
		chain = G.DecodeEngine(model, batch=batch, max_seq=max_seq, use_graph=False)
		os.environ['GPTQ_B200_CHAIN'] = '0'
		plain = G.DecodeEngine(model, batch=batch, max_seq=max_seq, use_graph=False)
	finally:
		if old is None:
			os.environ.pop('GPTQ_B200_CHAIN', None)
		else:
			os.environ['GPTQ_B200_CHAIN'] = old
	assert chain.chain is not None, 'the chain kernel should serve this model'
	assert plain.chain is None
	return model, chain, plain


@pytest.mark.parametrize('batch', [1, 2, 4, 8])
def test_chain_step_matches_kernel_per_projection_engine(G, batch):
	"""Same model, same prompt: after the (shared) prefill path, every decode step of the chain engine gives the
	logits of the kernel-per-projection engine up to fp16 rounding of the intermediate activations, and the same
	K / V rows in the cache.  Teacher forcing: both engines are fed the plain engine's tokens."""
	from gptq_triton_b200 import _lib
	from gptq_triton_b200.llama import LlamaConfig
	cfg = LlamaConfig(hidden_size=512, intermediate_size=1408, num_hidden_layers=3, num_attention_heads=4, vocab_size=512,
					  max_position_embeddings=256)
	prompt_len, steps = 37, 12
	model, chain, plain = _engines(G, cfg, batch, prompt_len + steps + 8, seed=5)
	prompt = torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=torch.Generator().manual_seed(batch)).cuda()
	chain.prefill(prompt)
	plain.prefill(prompt)
	assert torch.equal(chain.tok, plain.tok)
	for step in range(steps):
		chain.tok.copy_(plain.tok)
		plain.step()
		chain.step()
		torch.cuda.synchronize()
		assert _lib.kernel_status() == 0, f'status {_lib.kernel_status()} at step {step}'
		a, b = chain.logits.float().view(batch, -1), plain.logits.float().view(batch, -1)
		scale = b.abs().max().item()
		err = (a - b).abs().max().item()
		assert err <= 4e-3 * scale, (step, err, scale)
		assert torch.equal(chain.pos, plain.pos)
		p = int(plain.pos[0, 0].item()) - 1
		for l in range(cfg.num_hidden_layers):
			ka, kb = chain.kcache[l][:, :, p].float(), plain.kcache[l][:, :, p].float()
			va, vb = chain.vcache[l][:, :, p].float(), plain.vcache[l][:, :, p].float()
			assert (ka - kb).abs().max().item() <= 4e-3 * kb.abs().max().item() + 1e-3
			assert (va - vb).abs().max().item() <= 4e-3 * vb.abs().max().item() + 1e-3
		# the sampled token is the arg-max of the chain's own logits
		assert torch.equal(chain.tok.view(-1).cpu(), chain.logits.float().view(batch, -1).argmax(-1).cpu())


def test_chain_at_7b_layer_dimensions(G):
	"""Two layers at the benchmark's dimensions (hidden 4096, MLP 11008, 32 heads, vocabulary 32000), 300-token
	prompt: the shape-dependent plans (96 x 3, 32 x 8, 86 x 3, 32 x 9 CTAs, 9 key splits) against the
	kernel-per-projection engine."""
	from gptq_triton_b200 import _lib
	from gptq_triton_b200.llama import LlamaConfig
	cfg = LlamaConfig(num_hidden_layers=2, max_position_embeddings=512)
	prompt_len, steps = 300, 6
	model, chain, plain = _engines(G, cfg, 1, prompt_len + steps + 8, seed=9)
	prompt = torch.randint(0, cfg.vocab_size, (1, prompt_len), generator=torch.Generator().manual_seed(3)).cuda()
	chain.prefill(prompt)
	plain.prefill(prompt)
	for step in range(steps):
		chain.tok.copy_(plain.tok)
		plain.step()
		chain.step()
		torch.cuda.synchronize()
		assert _lib.kernel_status() == 0
		a, b = chain.logits.float().view(-1), plain.logits.float().view(-1)
		assert (a - b).abs().max().item() <= 4e-3 * b.abs().max().item(), step


def test_chain_position_outside_the_cache_is_reported(G):
	"""A position beyond the cache rows must not be used as an index: the row attends to nothing, its K / V are
	dropped and status 4 is raised (the engine's host-side bound normally prevents this)."""
	from gptq_triton_b200 import _lib
	from gptq_triton_b200.llama import LlamaConfig
	cfg = LlamaConfig(hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=4, vocab_size=512,
					  max_position_embeddings=64)
	model, chain, _ = _engines(G, cfg, 1, 32, seed=2)
	prompt = torch.randint(0, cfg.vocab_size, (1, 8), generator=torch.Generator().manual_seed(1)).cuda()
	chain.prefill(prompt)
	before = [k.clone() for k in chain.kcache]
	chain.pos.fill_(1000)
	assert _lib.kernel_status() == 0
	chain.step()
	torch.cuda.synchronize()
	assert _lib.kernel_status() == 4
	for k0, k1 in zip(before, chain.kcache):
		assert torch.equal(k0, k1)
	_lib.clear_kernel_status()
	assert _lib.kernel_status() == 0
