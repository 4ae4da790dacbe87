"""Multi-GPU self-check of the tensor-parallel decode path; run one process per GPU, e.g.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \\
        tests/tp_check.py

Every rank builds the same small synthetic model twice (same seed): once whole, once as this
rank's shards.  Greedy tokens of the tensor-parallel engine must equal those of the single-GPU
engine; the logits of the last step must agree to fp16 rounding.  Exits non-zero on mismatch."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
	import gptq_triton_b200 as G
	from gptq_triton_b200 import _lib, tp
	from gptq_triton_b200.llama import LlamaConfig
	rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
	local = int(os.environ.get('LOCAL_RANK', rank))
	torch.cuda.set_device(local)
	dev = torch.device('cuda', local)
	dist.init_process_group('nccl', device_id=dev)
	cfg = LlamaConfig(hidden_size=1024, intermediate_size=2816, num_hidden_layers=3, num_attention_heads=8, vocab_size=512,
					  max_position_embeddings=256)
	steps, prompt_len = 16, 40
	ok = True
	engines = []          # kept alive: their exchange buffers are mapped by the peers until the end
	for seed in range(6):
		whole = G.synthetic_quantized_llama(cfg, groupsize=128, seed=seed, device=dev, fuse=True)
		part = G.synthetic_quantized_llama(cfg, groupsize=128, seed=seed, device=dev, fuse=False)
		tp.shard_llama(part, rank, world)
		G.make_quant_attn(part)
		G.make_fused_mlp(part)
		prompt = torch.randint(0, cfg.vocab_size, (2, prompt_len), generator=torch.Generator().manual_seed(seed)).to(dev)
		def run(model, use_graph, batch=2):
			"""Greedy generation; returns tokens [b, steps] and the top-1/top-2 logit margin before every
			token."""
			e = G.DecodeEngine(model, batch=batch, max_seq=prompt_len + steps + 4, use_graph=use_graph)
			engines.append(e)
			toks = [e.prefill(prompt[:batch])]
			top2 = e.logits.float().topk(2, dim=-1).values
			margins = [float((top2[..., 0] - top2[..., 1]).min())]
			for _ in range(steps - 1):
				toks.append(e.step().clone())
				top2 = e.logits.float().topk(2, dim=-1).values
				margins.append(float((top2[..., 0] - top2[..., 1]).min()))
			return torch.cat(toks, dim=1), margins, e.logits.float().clone()
		t1, margins, logits1 = run(whole, False)
		# both forms of the all-reduce: fused into the projection kernels over peer memory, and NCCL
		for use_graph, fused in ((False, True), (True, True), (True, False)):
			os.environ['GPTQ_B200_TP_FUSED'] = '1' if fused else '0'
			t2, _, logits2 = run(part, use_graph)
			diff = (t1 != t2).any(dim=0).nonzero()
			first = int(diff[0]) if diff.numel() else -1
			if first < 0:
				# same tokens fed at every step: the logits of the last step agree to fp16 rounding (the summation
				# order of the row-parallel projections differs, nothing else)
				scale = float(logits1.abs().max())
				err = float((logits1 - logits2).abs().max())
				if err > 4e-3 * scale:
					ok = False
					if rank == 0:
						print(f'seed {seed} graph={use_graph} fused={fused}: last-step logits differ by {err:.4g} (scale {scale:.4g})', flush=True)
			# random-init logits are flat: a flip at a step whose reference margin is tiny is a tie, not an
			# error (and everything after the first flip legitimately differs)
			tie = first >= 0 and margins[first] < 0.05
			if rank == 0:
				print(f'seed {seed} graph={use_graph} fused={fused}: first differing step {first} (margin there {margins[first] if first >= 0 else 0:.3f})'
					  f' -> {"identical" if first < 0 else ("tie" if tie else "MISMATCH")}', flush=True)
			if first >= 0 and not tie:
				ok = False
		# one sequence: the attention block runs as the cluster kernel on the rank's heads, once followed by o_proj with its
		# fused all-reduce and once with o_proj and the all-reduce inside the same kernel
		if seed < 3:
			t1, margins, logits1 = run(whole, True, batch=1)
			os.environ['GPTQ_B200_TP_FUSED'] = '1'
			for inside in ('0', '1'):
				os.environ['GPTQ_B200_QKV_ATTN_O_TP'] = inside
				t2, _, logits2 = run(part, True, batch=1)
				assert engines[-1].used_qkv_attn and engines[-1].used_fused_oproj == (inside == '1')
				diff = (t1 != t2).any(dim=0).nonzero()
				first = int(diff[0]) if diff.numel() else -1
				tie = first >= 0 and margins[first] < 0.05
				if first < 0:
					scale = float(logits1.abs().max())
					err = float((logits1 - logits2).abs().max())
					if err > 4e-3 * scale:
						ok = False
						if rank == 0:
							print(f'seed {seed} batch 1 o_proj inside={inside}: last-step logits differ by {err:.4g} (scale {scale:.4g})', flush=True)
				if rank == 0:
					print(f'seed {seed} batch 1, o_proj + all-reduce inside the attention kernel={inside}: first differing step {first} -> '
						  f'{"identical" if first < 0 else ("tie" if tie else "MISMATCH")}', flush=True)
				if first >= 0 and not tie:
					ok = False
			os.environ.pop('GPTQ_B200_QKV_ATTN_O_TP', None)
		del whole, part
	torch.cuda.synchronize()
	status = _lib.kernel_status(dev)
	if status != 0:
		print(f'rank {rank}: kernel status word {status} (5 = a peer never arrived in the fused all-reduce)', flush=True)
		ok = False
	flag = torch.tensor([1 if ok else 0], device=dev)
	dist.all_reduce(flag, op=dist.ReduceOp.MIN)
	res = int(flag.item())
	if rank == 0:
		print('TP_CHECK', 'OK' if res else 'FAIL', flush=True)
	torch.cuda.synchronize()
	dist.barrier()
	for e in engines:          # every rank is past its last step: the exchange buffers can be unmapped and freed
		e.close()
	sys.stdout.flush()
	os._exit(0 if res else 1)        # no communicator teardown while captured graphs are alive


if __name__ == '__main__':
	main()
