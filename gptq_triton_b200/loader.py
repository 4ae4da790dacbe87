"""load_quant and synthetic model construction.

`load_quant` mirrors src/gptq_triton/__init__.py:16-93 of the reference: same arguments,
same checkpoint directory layout (quant_config.json, config.json, model.safetensors or
model.pt with HF LLaMA key names and .qweight/.qzeros/.scales(/.bias/.g_idx) tensors),
same order of module surgery (make_quant, load, bias pruning, make_quant_attn, make_fused_mlp).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from .fused_attention import make_quant_attn
from .fused_mlp import make_fused_mlp
from .llama import LlamaConfig, LlamaForCausalLM
from .quant_linear import QuantLinear, make_quant
from .quantize import quantize_linear_weight


def _empty_model(config: LlamaConfig, wbits: int, groupsize: int) -> LlamaForCausalLM:
	prev = torch.get_default_dtype()
	torch.set_default_dtype(torch.half)
	try:
		with torch.device('meta'):
			model = LlamaForCausalLM(config)
		make_quant(model, wbits, groupsize)          # QuantLinear buffers are created on the CPU
		for name, mod in model.named_modules():
			for pn, prm in list(mod.named_parameters(recurse=False)):
				if prm.is_meta:
					mod.register_parameter(pn, torch.nn.Parameter(torch.empty(prm.shape, dtype=torch.half), requires_grad=False))
	finally:
		torch.set_default_dtype(prev)
	return model


def autotune_warmup(model):
	"""No-op kept for API compatibility (reference: __init__.py:96-113): kernels are chosen by a
	static rule on the shape, there is no autotuner to warm."""
	return None


def _load_checkpoint_state(model, state, strict: bool):
	"""Checkpoints written under the transformers versions the reference names (README.md:66) carry
	`...self_attn.rotary_emb.inv_freq`, a persistent buffer of the HF attention module of that time; the
	reference loads them into the HF model as they are (__init__.py:60-63).  The decoder here builds its
	rotary tables from the config, so those keys are dropped; every other key is loaded as given (strictly
	for safetensors, non-strictly for model.pt, as the reference does)."""
	state = {k: v for k, v in state.items() if not k.endswith('.rotary_emb.inv_freq')}
	model.load_state_dict(state, strict=strict)


def load_quant(checkpoint: str, warmup_autotune: bool = True, device: Optional[str] = 'cuda', fuse_mlp: Optional[bool] = None):
	"""Load a quantised model from a checkpoint directory.
	fuse_mlp: None fuses for every groupsize (the fused kernel here is not slower for grouped
	checkpoints, unlike the reference's); False keeps three separate projections."""
	ck = Path(checkpoint)
	quant_config = json.load(open(ck / 'quant_config.json'))
	wbits, groupsize = quant_config['wbits'], quant_config['groupsize']
	config = LlamaConfig.from_json(ck / 'config.json')
	model = _empty_model(config, wbits, groupsize)
	if (ck / 'model.safetensors').exists():
		from safetensors.torch import load_file as safe_load
		_load_checkpoint_state(model, safe_load(str(ck / 'model.safetensors')), strict=True)
	elif (ck / 'model.pt').exists():
		_load_checkpoint_state(model, torch.load(ck / 'model.pt'), strict=False)
	else:
		raise FileNotFoundError(f"Could not find model checkpoint at {checkpoint}; please ensure that the path is correct and contains a `model.pt` or `model.safetensors` file.")
	for _, m in model.named_modules():
		if isinstance(m, QuantLinear) and m.bias is not None and bool((m.bias == 0).all()):
			m.bias = None
	make_quant_attn(model)
	if fuse_mlp is None or fuse_mlp:
		make_fused_mlp(model)
	if device is not None:
		model = model.to(device)
	elif warmup_autotune:
		raise ValueError("You must specify a device when warmup_autotune is True.")
	model.seqlen = 2048
	return model


def save_quant(model: LlamaForCausalLM, checkpoint: str, groupsize: int, safetensors: bool = True):
	"""Writes an UNFUSED quantised model in the reference's checkpoint layout (quantize.py:60-79)."""
	ck = Path(checkpoint)
	ck.mkdir(parents=True, exist_ok=True)
	json.dump({'wbits': 4, 'groupsize': groupsize}, open(ck / 'quant_config.json', 'w'))
	json.dump(model.config.__dict__, open(ck / 'config.json', 'w'))
	sd = {k: v.contiguous().cpu() for k, v in model.state_dict().items() if v is not None}
	if safetensors:
		from safetensors.torch import save_file
		save_file(sd, str(ck / 'model.safetensors'))
	else:
		torch.save(sd, ck / 'model.pt')


@torch.no_grad()
def synthetic_quantized_llama(config: LlamaConfig, groupsize: int = 128, seed: int = 0, device='cuda', fuse: bool = True,
							  weight_std: float = 0.02) -> LlamaForCausalLM:
	"""Random-init model of the given architecture: every q/k/v/o/gate/up/down weight ~ N(0, std),
	round-to-nearest quantised to 4 bits with `groupsize`; fp16 embeddings and lm_head ~ N(0, std).
	Stands in for a real checkpoint (none is available offline)."""
	model = _empty_model(config, 4, groupsize).to(device)
	gen = torch.Generator(device=device).manual_seed(seed)
	for name, m in model.named_modules():
		if isinstance(m, QuantLinear):
			W = torch.randn((m.outfeatures, m.infeatures), generator=gen, device=device, dtype=torch.float32) * weight_std
			qweight, qzeros, scales = quantize_linear_weight(W, groupsize)
			m.qweight.copy_(qweight)
			m.qzeros.copy_(qzeros)
			m.scales.copy_(scales)
			del W
	model.model.embed_tokens.weight.copy_(torch.randn(model.model.embed_tokens.weight.shape, generator=gen, device=device) * weight_std)
	model.lm_head.weight.copy_(torch.randn(model.lm_head.weight.shape, generator=gen, device=device) * weight_std)
	for layer in model.model.layers:
		layer.input_layernorm.weight.fill_(1.0)
		layer.post_attention_layernorm.weight.fill_(1.0)
	model.model.norm.weight.fill_(1.0)
	if fuse:
		make_quant_attn(model)
		make_fused_mlp(model)
	model.seqlen = 2048
	return model


@torch.no_grad()
def dense_reference_copy(model: LlamaForCausalLM) -> LlamaForCausalLM:
	"""The dequantise-then-matmul twin of an UNFUSED quantised model: every QuantLinear becomes an
	fp16 nn.Linear holding the dequantised weight (cuBLAS matmuls).  Used as the comparison path
	for greedy decoding."""
	return _dense_like(model)


def _dense_like(model: LlamaForCausalLM) -> LlamaForCausalLM:
	from .quant_linear import dequantize
	prev = torch.get_default_dtype()
	torch.set_default_dtype(torch.half)
	try:
		with torch.device('meta'):
			dense = LlamaForCausalLM(model.config)
	finally:
		torch.set_default_dtype(prev)
	dev = model.lm_head.weight.device
	dense = dense.to_empty(device=dev)
	src = dict(model.named_modules())
	for name, m in dense.named_modules():
		if isinstance(m, torch.nn.Linear) and name != 'lm_head':
			q = src[name]
			assert isinstance(q, QuantLinear), f'{name}: pass the unfused quantised model'
			w = dequantize(q.groupsize, q.qweight, q.scales, q.qzeros, q.g_idx)      # [K, N]
			m.weight = torch.nn.Parameter(w.t().contiguous(), requires_grad=False)
	dense.model.embed_tokens.weight = model.model.embed_tokens.weight
	dense.lm_head.weight = model.lm_head.weight
	dense.model.norm.weight = model.model.norm.weight
	for a, b in zip(dense.model.layers, model.model.layers):
		a.input_layernorm.weight = b.input_layernorm.weight
		a.post_attention_layernorm.weight = b.post_attention_layernorm.weight
	return dense
