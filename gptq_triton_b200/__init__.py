"""gptq_triton_b200: B200-native implementation of the GPTQ-triton inference hot path.

Same public names as the reference package (src/gptq_triton/__init__.py:10-13); the
`triton_*` names are kept as aliases although no Triton is involved.
"""
from . import fused_mlp, quant_linear
from .fused_attention import QuantLlamaAttention, make_quant_attn, qkv_rope
from .fused_mlp import QuantLlamaMLP, gateup_silu, make_fused_mlp, triton_llama_mlp_4
from .llama import DecodeEngine, LlamaConfig, LlamaForCausalLM
from .loader import autotune_warmup, load_quant, save_quant, synthetic_quantized_llama
from .quant_linear import QuantLinear, dequantize, make_quant, qmatmul, triton_matmul4, unpack_qweight, unpack_qzeros

__all__ = [
	'load_quant', 'autotune_warmup', 'save_quant', 'synthetic_quantized_llama', 'DecodeEngine', 'LlamaConfig', 'LlamaForCausalLM',
	'QuantLinear', 'make_quant', 'triton_matmul4', 'qmatmul',
	'QuantLlamaAttention', 'make_quant_attn', 'qkv_rope',
	'QuantLlamaMLP', 'make_fused_mlp', 'triton_llama_mlp_4', 'gateup_silu',
	'dequantize', 'unpack_qweight', 'unpack_qzeros',
	'quant_linear', 'fused_mlp',
]
