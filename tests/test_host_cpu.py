"""CPU tests of the host-side layer: packer/quantiser against the oracle, module surgery,
state-dict compatibility with the reference checkpoint layout, checkpoint round trip."""
import json

import numpy as np
import pytest
import torch

import gptq_triton_b200 as G
from gptq_triton_b200 import loader, quantize
from gptq_triton_b200.llama import LlamaConfig
from oracle import gptq_oracle as O

SMALL = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2, vocab_size=128, max_position_embeddings=64)


@pytest.mark.parametrize('gs', [128, -1, 32])
def test_rtn_quantiser_and_packer_match_oracle(gs):
	torch.manual_seed(0)
	W = torch.randn(64, 256) * 0.02
	qw, qz, sc = quantize.quantize_linear_weight(W, gs)
	fq, s, z = O.rtn_quantize(W, gs)
	a, b, c = O.pack_linear(fq, s, z, gs)
	assert torch.equal(qw, a) and torch.equal(qz, b) and torch.equal(sc, c)


def test_packer_matches_reference_fixture(golden_dir):
	d = dict(np.load(golden_dir / 'pack_a.npz'))
	gs = int(d['groupsize'])
	fq = torch.from_numpy(d['fakequant'])
	# quantising the fake-quantised weights again reproduces the reference's integers
	qw, qz, sc = quantize.quantize_linear_weight(fq, gs)
	assert np.array_equal(O.unpack_qweight(qw), O.unpack_qweight(d['qweight']))


def test_quantlinear_contract():
	with pytest.raises(NotImplementedError):
		G.QuantLinear(3, 128, 256, 256, False)
	with pytest.raises(AssertionError):
		G.QuantLinear(4, 128, 256, 252, False)
	m = G.QuantLinear(4, -1, 256, 64, True)
	assert m.groupsize == 256 and m.qweight.shape == (32, 64) and m.qzeros.shape == (1, 8) and m.scales.shape == (1, 64)
	assert m.qweight.dtype == torch.int32 and m.scales.dtype == torch.float16 and m.bias.shape == (64,)
	assert set(m.state_dict()) == {'qweight', 'qzeros', 'scales', 'bias'}
	m2 = G.QuantLinear(4, 128, 256, 64, False)
	assert set(m2.state_dict()) == {'qweight', 'qzeros', 'scales'}
	sd = dict(m2.state_dict())
	sd['g_idx'] = torch.arange(256, dtype=torch.int32) // 128
	m2.load_state_dict(sd)
	assert 'g_idx' in m2.state_dict()


def test_module_surgery_and_checkpoint_round_trip(tmp_path):
	model = loader._empty_model(SMALL, 4, 128)
	names = [n for n, m in model.named_modules() if isinstance(m, G.QuantLinear)]
	assert len(names) == 7 * SMALL.num_hidden_layers and 'lm_head' not in names
	assert isinstance(model.lm_head, torch.nn.Linear)
	gen = torch.Generator().manual_seed(1)
	for n, m in model.named_modules():
		if isinstance(m, G.QuantLinear):
			qw, qz, sc = quantize.quantize_linear_weight(torch.randn((m.outfeatures, m.infeatures), generator=gen) * 0.02, 128)
			m.qweight.copy_(qw); m.qzeros.copy_(qz); m.scales.copy_(sc)
	for prm in model.parameters():
		prm.data.normal_(0, 0.02, generator=gen)
	keys = set(model.state_dict())
	assert 'model.layers.0.self_attn.q_proj.qweight' in keys and 'model.layers.1.mlp.down_proj.scales' in keys
	assert 'model.embed_tokens.weight' in keys and 'lm_head.weight' in keys and 'model.norm.weight' in keys
	loader.save_quant(model, tmp_path, 128)
	assert json.load(open(tmp_path / 'quant_config.json')) == {'wbits': 4, 'groupsize': 128}
	loaded = G.load_quant(str(tmp_path), warmup_autotune=False, device=None)
	layer = loaded.model.layers[0]
	assert isinstance(layer.self_attn, G.QuantLlamaAttention) and isinstance(layer.mlp, G.QuantLlamaMLP)
	qkv = layer.self_attn.qkv_proj
	assert qkv.outfeatures == 3 * SMALL.hidden_size and qkv.qweight.shape == (SMALL.hidden_size // 8, 3 * SMALL.hidden_size)
	src = model.model.layers[0].self_attn
	assert torch.equal(qkv.qweight, torch.cat([src.q_proj.qweight, src.k_proj.qweight, src.v_proj.qweight], dim=1))
	assert torch.equal(qkv.qzeros, torch.cat([src.q_proj.qzeros, src.k_proj.qzeros, src.v_proj.qzeros], dim=1))
	assert torch.equal(layer.mlp.gate_proj_qweight, model.model.layers[0].mlp.gate_proj.qweight)
	assert torch.equal(loaded.lm_head.weight, model.lm_head.weight)
	assert loaded.seqlen == 2048
	unfused = G.load_quant(str(tmp_path), warmup_autotune=False, device=None, fuse_mlp=False)
	assert not isinstance(unfused.model.layers[0].mlp, G.QuantLlamaMLP)
	with pytest.raises(FileNotFoundError):
		(tmp_path / 'model.safetensors').unlink()
		G.load_quant(str(tmp_path), warmup_autotune=False, device=None)


@pytest.mark.parametrize('safetensors', [True, False])
def test_checkpoint_with_rotary_inv_freq_keys_loads(tmp_path, safetensors):
	"""Checkpoints written under the transformers versions the reference names carry
	`self_attn.rotary_emb.inv_freq` per layer; they must load, in both file formats, and any OTHER
	unexpected key of a safetensors file must still be refused."""
	model = loader._empty_model(SMALL, 4, 128)
	gen = torch.Generator().manual_seed(2)
	for n, m in model.named_modules():
		if isinstance(m, G.QuantLinear):
			qw, qz, sc = quantize.quantize_linear_weight(torch.randn((m.outfeatures, m.infeatures), generator=gen) * 0.02, 128)
			m.qweight.copy_(qw); m.qzeros.copy_(qz); m.scales.copy_(sc)
	for prm in model.parameters():
		prm.data.normal_(0, 0.02, generator=gen)
	loader.save_quant(model, tmp_path, 128, safetensors=safetensors)
	head_dim = SMALL.hidden_size // SMALL.num_attention_heads
	extra = {f'model.layers.{i}.self_attn.rotary_emb.inv_freq': 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))
			 for i in range(SMALL.num_hidden_layers)}
	if safetensors:
		from safetensors.torch import load_file, save_file
		sd = load_file(str(tmp_path / 'model.safetensors'))
		save_file({**sd, **extra}, str(tmp_path / 'model.safetensors'))
	else:
		sd = torch.load(tmp_path / 'model.pt')
		torch.save({**sd, **extra}, tmp_path / 'model.pt')
	loaded = G.load_quant(str(tmp_path), warmup_autotune=False, device=None)
	assert torch.equal(loaded.model.layers[1].self_attn.o_proj.qweight, model.model.layers[1].self_attn.o_proj.qweight)
	if safetensors:
		save_file({**sd, **extra, 'model.layers.0.bogus.weight': torch.zeros(1)}, str(tmp_path / 'model.safetensors'))
		with pytest.raises(RuntimeError):
			G.load_quant(str(tmp_path), warmup_autotune=False, device=None)


def test_decode_engine_refuses_to_step_past_its_cache():
	"""Host-side guard: step() raises before a position beyond the static cache could reach a kernel
	(checked without a GPU by calling the guard on a bare object)."""
	from gptq_triton_b200.llama import DecodeEngine
	e = DecodeEngine.__new__(DecodeEngine)
	e.next_pos, e.max_seq = 8, 8
	with pytest.raises(RuntimeError, match='is full'):
		e.step()


def test_make_fused_mlp_returns_module():
	model = loader._empty_model(SMALL, 4, 128)
	mlp = model.model.layers[0].mlp
	fused = G.make_fused_mlp(mlp)
	assert isinstance(fused, G.QuantLlamaMLP) and fused.infeatures == 256 and fused.outfeatures == 256
	assert G.make_fused_mlp(torch.nn.Linear(4, 4)).__class__ is torch.nn.Linear


def test_bench_reference_arm_prints_one_json_line():
	"""`bench.py --impl reference` (the CPU port of the reference path) runs without a GPU and prints the contract's
	JSON line with its own cpu_baseline and e2e records."""
	import subprocess, sys
	from pathlib import Path
	root = Path(__file__).resolve().parent.parent
	r = subprocess.run([sys.executable, str(root / 'bench.py'), '--impl', 'reference', '--steps', '1', '--warmup', '0'], capture_output=True, text=True, timeout=600)
	assert r.returncode == 0, r.stderr[-2000:]
	line = json.loads(r.stdout.strip().splitlines()[-1])
	assert line['impl'] == 'reference' and line['unit'] == 'tokens/s' and line['value'] > 0
	assert line['cpu_baseline']['kind'] == 'port' and line['cpu_baseline']['cores'] >= 1 and line['cpu_baseline']['factor'] == 32
	assert line['e2e'] == {'value': line['value'], 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}
