#!/usr/bin/env python
"""Benchmark of the hot path: greedy decode of a LLaMA-7B-architecture model with 4-bit g128
GPTQ weights (synthetic, random-init) at batch 1 after a 2048-token prompt.

One "step" is one decode step (one token): 32 x (fused QKV+rotary, o_proj, fused gate/up,
down_proj quantised matmuls + attention over the KV cache) + fp16 lm_head + argmax.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line (rank 0).  `value` is device-timed (CUDA-graph replays, inputs resident
in HBM); `e2e` goes through the public DecodeEngine.step() API with the token fed from pinned
host memory and the result read back every step.  `roofline` is the dominant kernel (fused
gate/up decode kernel) timed live with CUDA events while rotating over all 32 layers' weights
(1.4 GB, larger than L2).  `--impl reference` times the CPU dequantise-then-matmul oracle on the
host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = 'decode tokens/s (7B-arch, 4-bit g128, 2k ctx)'
UNIT = 'tokens/s'
WORKLOAD = 'llama7b-arch 4-bit g128 greedy decode, batch 1, 2048-token prompt'
PROMPT = 2048
GROUPSIZE = 128


def measured_peaks():
	p = ROOT / 'MEASURED_PEAKS.json'
	if p.exists():
		d = json.load(open(p))
		return float(d['hbm_gbs']), 'measured'
	return 6650.0, 'fallback'


def quantised_bytes(K, N, g=GROUPSIZE):
	return K * N // 2 + (K // g) * N * 2 + (K // g) * N // 2


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's dequantise-then-matmul path on the host cores
# ------------------------------------------------------------------------------------------
def cpu_model_name() -> str:
	try:
		for line in open('/proc/cpuinfo'):
			if line.lower().startswith('model name'):
				return line.split(':', 1)[1].strip()
	except OSError:
		pass
	return 'unknown'


def cpu_layer_seconds(reps: int):
	"""One decoder layer of the decode step at batch 1 on the host cores through the CPU oracle: the four
	quantised projections at their real shapes (dequantise to fp16 + torch.matmul, the reference's CPU-runnable
	path), attention of one query over a 2112-token fp16 cache, and 1/32 of the fp16 lm_head.
	Returns (median seconds per layer, cores)."""
	import torch
	from gptq_triton_b200 import synth
	from oracle import gptq_oracle as O
	cores = os.cpu_count() or 1
	torch.set_num_threads(cores)
	h, inter, ctx, heads = 4096, 11008, 2112, 32
	shapes = [(h, 3 * h), (h, h), (h, inter), (h, inter), (inter, h)]
	ws = [synth.quant_tensors(K, N, GROUPSIZE, seed=i) for i, (K, N) in enumerate(shapes)]
	xs = [synth.activations((1, K), seed=10 + i) for i, (K, N) in enumerate(shapes)]
	g = torch.Generator().manual_seed(5)
	kc = torch.randn((heads, ctx, 128), generator=g).half()
	vc = torch.randn((heads, ctx, 128), generator=g).half()
	q = torch.randn((heads, 1, 128), generator=g).half()
	lm = (torch.randn((32000 // 32, h), generator=g) * 0.02).half()
	times = []
	for _ in range(reps):
		t0 = time.perf_counter()
		for w, x in zip(ws, xs):
			O.qmatmul_r16(x, w['qweight'], w['qzeros'], w['scales'], GROUPSIZE)
		att = torch.softmax((q.float() @ kc.float().transpose(1, 2)) / 128 ** 0.5, dim=-1)
		(att @ vc.float()).half()
		xs[0] @ lm.t()
		times.append(time.perf_counter() - t0)
	times.sort()
	return times[len(times) // 2], cores


def cpu_config0():
	"""The reference's CPU-runnable case: one 4096 x 4096 g128 QuantLinear, x [1, 512, 4096] through the torch
	dequantise + matmul path; unpack + dequantise and the matmul are timed separately."""
	import torch
	from gptq_triton_b200 import synth
	from oracle import gptq_oracle as O
	cores = os.cpu_count() or 1
	torch.set_num_threads(cores)
	t = synth.quant_tensors(4096, 4096, GROUPSIZE, seed=0)
	x = synth.activations((1, 512, 4096), seed=1)
	d, m = [], []
	for _ in range(3):
		t0 = time.perf_counter()
		w = O.dequant_f16(t['qweight'], t['qzeros'], t['scales'], GROUPSIZE)
		t1 = time.perf_counter()
		torch.matmul(x.view(512, 4096), w)
		t2 = time.perf_counter()
		d.append(t1 - t0)
		m.append(t2 - t1)
	d.sort(); m.sort()
	return {'x': [1, 512, 4096], 'K': 4096, 'N': 4096, 'groupsize': GROUPSIZE, 'dequant_s': d[1], 'matmul_s': m[1], 'total_s': d[1] + m[1],
			'gflops': 2 * 512 * 4096 * 4096 / (d[1] + m[1]) / 1e9, 'cores': cores}


LAYERS = 32


def cpu_baseline_record(reps: int):
	sec, cores = cpu_layer_seconds(reps)
	tok_s = 1.0 / (sec * LAYERS)
	return {'value': tok_s, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'cpu_model': cpu_model_name(),
			'sample': 'one decoder layer of the decode step at batch 1 (4 quantised projections at their real shapes through dequantise + fp16 torch.matmul, '
					  'attention of one query over a 2112-token cache, 1/32 of the lm_head), median of %d; a token = %d such layers' % (reps, LAYERS),
			'extrapolated': True, 'factor': LAYERS, 'layer_s': sec}


def reference_arm(args):
	rank = int(os.environ.get('RANK', '0'))
	if rank != 0:
		return
	for _ in range(max(0, min(args.warmup, 2))):
		cpu_layer_seconds(1)
	rec = cpu_baseline_record(max(1, min(args.steps, 24)))
	tok_s = rec['value']
	line = {
		'impl': 'reference', 'metric': METRIC, 'value': tok_s, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
		'ms_per_step': 1e3 / tok_s, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16',
		'data': 'synthetic', 'config': {'workload': WORKLOAD, 'path': 'CPU port of the reference path: unpack + dequantise + torch.matmul fp16 on the host cores'},
		'cpu_baseline': rec,
		'e2e': {'value': tok_s, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
	}
	print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
	"""SM clock and clock-event reasons of one GPU, read (never set) every few milliseconds through
	NVML while the timed region runs; falls back to an `nvidia-smi -lms` child process."""
	Q = 'index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'
	BITS = {'sw_power_cap': 0x4, 'hw_slowdown': 0x8, 'sw_thermal_slowdown': 0x20, 'hw_thermal_slowdown': 0x40}

	def __init__(self, gpu_index: int, uuid: str = None):
		self.idx = gpu_index
		self.uuid = uuid
		self.proc = None
		self.lines = []
		self.nvml = None
		self.samples = []          # (sm_mhz, reason bits)
		self.stop_flag = False
		self.max_mhz = None

	def start(self):
		try:
			import pynvml
			pynvml.nvmlInit()
			h = None
			if self.uuid:
				try:
					h = pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode() if hasattr(self.uuid, 'encode') else self.uuid)
				except Exception:
					h = None
			if h is None:
				h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
			self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
			reasons_fn = getattr(pynvml, 'nvmlDeviceGetCurrentClocksEventReasons', None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
			self.nvml = (pynvml, h, reasons_fn)
			self.thread = threading.Thread(target=self._poll, daemon=True)
			self.thread.start()
			return
		except Exception:
			self.nvml = None
		try:
			self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.idx), '--query-gpu=' + self.Q, '--format=csv,noheader,nounits', '-lms', '100'],
										 stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
			self.thread = threading.Thread(target=self._read, daemon=True)
			self.thread.start()
		except Exception:
			self.proc = None

	def _poll(self):
		pynvml, h, reasons_fn = self.nvml
		while not self.stop_flag:
			try:
				self.samples.append((float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), int(reasons_fn(h))))
			except Exception:
				pass
			time.sleep(0.005)

	def _read(self):
		for line in self.proc.stdout:
			self.lines.append(line.strip())

	def stop(self):
		if self.nvml is not None:
			self.stop_flag = True
			self.thread.join(timeout=1)
			sm = sorted(s for s, _ in self.samples)
			bits = 0
			for _, r in self.samples:
				bits |= r
			reasons = sorted(n for n, b in self.BITS.items() if bits & b)
			return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': self.max_mhz, 'samples': len(sm), 'reasons': reasons}
		if self.proc is None:
			return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
		self.proc.terminate()
		try:
			self.proc.wait(timeout=2)
		except Exception:
			self.proc.kill()
		sm, mx, reasons = [], None, set()
		names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
		for l in self.lines:
			f = [x.strip() for x in l.split(',')]
			if len(f) < 9:
				continue
			try:
				sm.append(float(f[1])); mx = float(f[2])
			except ValueError:
				continue
			for n, v in zip(names, f[5:9]):
				if v.lower().startswith('active'):
					reasons.add(n)
		sm.sort()
		return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': mx, 'samples': len(sm), 'reasons': sorted(reasons)}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def greedy_reference(model_fn, prompt, steps):
	"""Reference-style greedy decoding (concatenated K/V tuples): tokens [b, steps], logits of the last step and the
	smallest top-1/top-2 margin."""
	import torch
	logits, past = model_fn(prompt, None)
	toks, margin = [], float('inf')
	last = None
	for _ in range(steps):
		last = logits[:, -1, :].float()
		top2 = last.topk(2, dim=-1).values
		margin = min(margin, float((top2[:, 0] - top2[:, 1]).min()))
		nxt = last.argmax(-1, keepdim=True)
		toks.append(nxt)
		logits, past = model_fn(nxt, past)
	return torch.cat(toks, dim=1), last, margin


def parity_check(G, engine_factory, reference, cfg, batch, dev, steps=8):
	"""Greedy tokens and last-step logits of the engine that is about to be timed against `reference`
	(prompt -> (tokens, last logits, margin)).  The prompt is chosen by seed so that every top-1/top-2 margin of
	the reference run is clear of fp16 noise (random-init logits over 32000 entries are nearly flat)."""
	import torch
	best = None
	for seed in range(6):
		prompt = torch.randint(0, cfg.vocab_size, (batch, PROMPT), generator=torch.Generator().manual_seed(500 + seed)).to(dev)
		toks, last, margin = reference(prompt, steps)
		if best is None or margin > best[3]:
			best = (prompt, toks, last, margin)
		if margin > 0.05:
			break
	prompt, ref_toks, ref_last, margin = best
	engine = engine_factory()
	out = [engine.prefill(prompt)]
	for _ in range(steps - 1):
		out.append(engine.step().clone())
	# the logits that produced the last token: those of step `steps - 1`
	got = torch.cat(out, dim=1)
	logits = engine.logits.float().view(batch, -1)
	diff = (got != ref_toks).any(dim=0).nonzero()
	first = int(diff[0]) if diff.numel() else -1
	scale = float(ref_last.abs().max())
	err = float((logits - ref_last.view(batch, -1)).abs().max()) / max(scale, 1e-30) if first < 0 else None
	# Tokens must be identical.  The logits of the last step are compared as max|a - b| / max|b|; both runs round the
	# residual stream and the activations to fp16 at 2 x 32 places with different summation orders (and the twin also
	# rounds the weights to fp16), so the bound is that of accumulated fp16 rounding over 32 layers, not of one op.
	return engine, {'steps': steps, 'first_diff_step': first, 'min_reference_margin': margin, 'last_logits_max_err_over_max': err,
					'tolerance': 2e-2, 'ok': bool(first < 0 and err is not None and err <= 2e-2)}


def prefill_record(G, model, cfg, dev, peak_tflops):
	"""The tcgen05 prefill kernel at M = 512 and 2048 on the model's own weights, rotating over all layers
	(32 x 8 MB / 32 x 43 MB of packed weights: larger than L2), timed with CUDA events."""
	import torch
	layers = model.model.layers
	out = []
	for M in (512, 2048):
		x = (torch.randn((1, M, cfg.hidden_size), device=dev) * 0.5).half()
		for name, fn, flops in (
				('o_proj %dx%d' % (cfg.hidden_size, cfg.hidden_size), lambda l: l.self_attn.o_proj(x), 2.0 * M * cfg.hidden_size * cfg.hidden_size),
				('gate/up %dx2x%d fused' % (cfg.hidden_size, cfg.intermediate_size), lambda l: l.mlp.intermediate(x), 4.0 * M * cfg.hidden_size * cfg.intermediate_size)):
			for l in layers[:3]:
				fn(l)
			torch.cuda.synchronize()
			e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
			e0.record()
			for l in layers:
				fn(l)
			e1.record()
			torch.cuda.synchronize()
			us = e0.elapsed_time(e1) * 1e3 / len(layers)
			tf = flops / us / 1e6
			out.append({'M': M, 'op': name, 'us': us, 'tflops': tf, 'frac': tf / peak_tflops})
	return out


def measure_exchange(G, tp, dev, rank, world, barrier, dist):
	"""The all-reduce that is fused into the row-parallel decode kernel, alone: a projection with a one-chunk K-slice
	(128 rows per rank, 4096 outputs, one row of x) with and without the exchange over peer memory, 64 launches per CUDA
	graph, CUDA events, max over ranks.  The difference is what one exchange adds to a kernel; a 7B decode step has 64."""
	import torch
	from gptq_triton_b200 import synth
	N, K = 4096, 128
	t = synth.quant_tensors(K, N, 128, seed=77 + rank)
	w = tuple(v.to(dev) for v in (t['qweight'], t['scales'], t['qzeros']))
	x = synth.activations((1, K), seed=5).to(dev)
	res = torch.zeros((1, N), dtype=torch.float16, device=dev)
	try:
		ex = tp.PeerExchange(N, rank, world, group=None)
	except RuntimeError:
		return None
	out = {}
	for name, ar in (('with_exchange_us', ex), ('without_exchange_us', None)):
		fn = lambda: G.qmatmul(128, x, *w, residual=res, ar=ar)
		s = torch.cuda.Stream()
		with torch.cuda.stream(s):
			for _ in range(3):
				fn()
			s.synchronize()
			barrier()
			g = torch.cuda.CUDAGraph()
			with torch.cuda.graph(g, stream=s):
				for _ in range(64):
					fn()
			barrier()
			g.replay()
			s.synchronize()
			barrier()
			e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
			e0.record(s)
			for _ in range(5):
				g.replay()
			e1.record(s)
			s.synchronize()
		us = torch.tensor([e0.elapsed_time(e1) * 1e3 / (5 * 64)], device=dev)
		dist.all_reduce(us, op=dist.ReduceOp.MAX)
		out[name] = float(us.item())
		del g
	barrier()
	ex.close()
	out['exchange_us'] = out['with_exchange_us'] - out['without_exchange_us']
	out['what'] = 'o_proj-shaped decode kernel (M = 1, 128 rows per rank -> 4096) inside a CUDA graph, with and without the fused all-reduce'
	return out


def measure_config4(G, tp, dev, rank, world, barrier, dist, steps=16, warmup=4):
	"""Benchmark configuration 4: LLaMA-65B architecture, 4-bit g128, batch 16, 2048-token prompts, greedy decode,
	tensor parallel over the ranks of this run.  Device-timed like the main measurement (barrier, CUDA events, max over
	ranks).  Reports tokens/s over all sequences, the bytes one rank streams per step and the fraction of that rank's
	HBM roofline."""
	import torch
	from gptq_triton_b200 import _lib
	from gptq_triton_b200.llama import LlamaConfig
	cfg = LlamaConfig.llama_65b()
	batch = 16
	model = G.synthetic_quantized_llama(cfg, groupsize=GROUPSIZE, seed=4321, device=dev, fuse=False)
	if world > 1:
		tp.shard_llama(model, rank, world)
	G.make_quant_attn(model)
	G.make_fused_mlp(model)
	torch.cuda.empty_cache()
	engine = G.DecodeEngine(model, batch=batch, max_seq=PROMPT + warmup + steps + 16, use_graph=True)
	prompt = torch.randint(0, cfg.vocab_size, (batch, PROMPT), generator=torch.Generator().manual_seed(77)).to(dev)
	engine.prefill(prompt)
	for _ in range(warmup):
		engine.step()
	barrier()
	e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
	e0.record()
	for _ in range(steps):
		engine.step()
	e1.record()
	barrier()
	t = torch.tensor([e0.elapsed_time(e1)], device=dev)
	if dist is not None:
		dist.all_reduce(t, op=dist.ReduceOp.MAX)
	ms = float(t.item())
	wbytes = 0
	for n, b_ in model.named_buffers():
		if n.endswith(('qweight', 'qzeros', 'scales')):
			wbytes += b_.numel() * b_.element_size()
	wbytes += model.lm_head.weight.numel() * 2
	heads_local = model.model.layers[0].self_attn.num_heads
	ctx = PROMPT + warmup + steps / 2.0
	kv = 2.0 * cfg.num_hidden_layers * batch * heads_local * ctx * 128 * 2
	peak, which = measured_peaks()
	ach = (wbytes + kv) / (ms / steps) / 1e6
	rec = {'workload': 'llama65b-arch 4-bit g128 greedy decode, batch 16, 2048-token prompts, tp%d' % world, 'value': batch * steps / (ms / 1e3), 'unit': UNIT,
		   'ms_per_step': ms / steps, 'steps': steps, 'warmup': warmup, 'weight_bytes_per_rank': wbytes, 'kv_bytes_per_rank_per_step': kv,
		   'achieved_gbs_per_rank': ach, 'hbm_peak_gbs': peak, 'frac_of_rank_roofline': ach / peak, 'peak_source': which,
		   'fused_all_reduce': engine.ar_o is not None, 'kernel_status': _lib.kernel_status(dev)}
	barrier()
	engine.close()
	return rec


def gpu_arm(args):
	import torch
	import torch.distributed as dist

	rank = int(os.environ.get('RANK', '0'))
	local_rank = int(os.environ.get('LOCAL_RANK', '0'))
	world = int(os.environ.get('WORLD_SIZE', '1'))
	if not torch.cuda.is_available():
		raise SystemExit('bench.py needs a CUDA device (B200); there is no CPU path for the product kernels')
	torch.cuda.set_device(local_rank)
	dev = torch.device('cuda', local_rank)
	if world > 1:
		dist.init_process_group('nccl', device_id=dev)

	import gptq_triton_b200 as G
	from gptq_triton_b200 import _lib, loader
	from gptq_triton_b200.llama import LlamaConfig

	from gptq_triton_b200 import tp
	big = args.workload == 'llama65b-b16'
	cfg = LlamaConfig.llama_65b() if big else LlamaConfig.llama_7b()
	batch = 16 if big else 1
	if args.layers:
		cfg.num_hidden_layers = args.layers            # debugging aid only; the default is the full model
	max_seq = PROMPT + args.warmup + 2 * args.steps + 32

	# ---- the model, and the parity check of the engine that is timed below --------------------------------
	# N = 1: against the dequantise-then-matmul twin (fp16 nn.Linear holding the dequantised weights, cuBLAS);
	# N > 1: ONE model, tensor-parallel over the N GPUs (same seed on every rank, each keeps its shards), against the
	# un-sharded engine built on the same rank.
	parity = None
	if world > 1:
		model = G.synthetic_quantized_llama(cfg, groupsize=GROUPSIZE, seed=1234, device=dev, fuse=False)
		tp.shard_llama(model, rank, world)
		G.make_quant_attn(model)
		G.make_fused_mlp(model)
		torch.cuda.empty_cache()
		factory = lambda: G.DecodeEngine(model, batch=batch, max_seq=max_seq, use_graph=not args.no_graph)
		if not big and not args.no_parity:
			whole = G.synthetic_quantized_llama(cfg, groupsize=GROUPSIZE, seed=1234, device=dev)
			def reference(prompt, steps):
				e = G.DecodeEngine(whole, batch=batch, max_seq=PROMPT + steps + 8, use_graph=False)
				toks = [e.prefill(prompt)]
				margin = float('inf')
				for i in range(steps):
					top2 = e.logits.float().view(batch, -1).topk(2, dim=-1).values
					margin = min(margin, float((top2[:, 0] - top2[:, 1]).min()))
					last = e.logits.float().view(batch, -1).clone()
					if i < steps - 1:
						toks.append(e.step().clone())
				return torch.cat(toks, dim=1), last, margin
			engine, parity = parity_check(G, factory, reference, cfg, batch, dev)
			parity['against'] = 'un-sharded engine on the same rank'
			flag = torch.tensor([1 if parity['ok'] else 0], device=dev)
			dist.all_reduce(flag, op=dist.ReduceOp.MIN)
			parity['ok_on_every_rank'] = bool(int(flag.item()))
			del whole
			torch.cuda.empty_cache()
		else:
			engine = factory()
	else:
		model = G.synthetic_quantized_llama(cfg, groupsize=GROUPSIZE, seed=1234, device=dev, fuse=False)
		dense = None if (big or args.no_parity) else loader.dense_reference_copy(model)
		G.make_quant_attn(model)
		G.make_fused_mlp(model)
		factory = lambda: G.DecodeEngine(model, batch=batch, max_seq=max_seq, use_graph=not args.no_graph)
		if dense is not None:
			def model_fn(ids, past):
				return dense(ids, past_key_values=past, use_cache=True)
			engine, parity = parity_check(G, factory, lambda prompt, steps: greedy_reference(model_fn, prompt, steps), cfg, batch, dev)
			parity['against'] = 'dequantise-then-matmul twin (fp16 cuBLAS) of the same model'
			del dense
			torch.cuda.empty_cache()
		else:
			engine = factory()
	gen = torch.Generator().manual_seed(99)
	prompt = torch.randint(0, cfg.vocab_size, (batch, PROMPT), generator=gen).to(dev)
	engine.prefill(prompt)
	torch.cuda.synchronize()

	def barrier():
		torch.cuda.synchronize()
		if world > 1:
			dist.barrier()
		torch.cuda.synchronize()

	# ---- device-timed: K graph replays -------------------------------------------------------
	try:
		gpu_uuid = 'GPU-' + str(torch.cuda.get_device_properties(local_rank).uuid)
	except Exception:
		gpu_uuid = None
	sampler = ClockSampler(local_rank, gpu_uuid)
	if rank == 0:
		sampler.start()           # before the warm-up: the timed region follows the warm-up without a pause
	for _ in range(args.warmup):
		engine.step()
	barrier()
	if rank == 0:
		sampler.samples.clear()
	e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
	torch.cuda.profiler.start()           # lets a profiler restrict itself to the timed region
	e0.record()
	for _ in range(args.steps):
		engine.step()
	e1.record()
	barrier()
	torch.cuda.profiler.stop()
	ms = e0.elapsed_time(e1)
	clocks = sampler.stop() if rank == 0 else None
	t = torch.tensor([ms], device=dev)
	if world > 1:
		dist.all_reduce(t, op=dist.ReduceOp.MAX)
	ms = float(t.item())
	tok_s = batch * args.steps / (ms / 1e3)            # every rank works on the same tokens (tensor parallel)

	# ---- end to end through DecodeEngine.step(): token in from pinned host memory, token out ----
	host_tok = torch.zeros((batch, 1), dtype=torch.int64).pin_memory()
	host_out = torch.zeros((batch, 1), dtype=torch.int64).pin_memory()
	host_tok.copy_(engine.tok.cpu())
	barrier()
	t0 = time.perf_counter()
	for _ in range(args.steps):
		engine.tok.copy_(host_tok, non_blocking=True)       # H2D: the token chosen on the host side
		out = engine.step()
		host_out.copy_(out, non_blocking=True)              # D2H: the next token
		torch.cuda.current_stream().synchronize()
		host_tok.copy_(host_out)
	e2e_s = time.perf_counter() - t0
	t = torch.tensor([e2e_s], device=dev)
	if world > 1:
		dist.all_reduce(t, op=dist.ReduceOp.MAX)
	e2e_tok_s = batch * args.steps / float(t.item())

	# ---- roofline of the dominant kernel: fused gate/up decode kernel, live, rotating weights ----
	roof = None
	status = None
	prefill = None
	if rank == 0:
		layers = model.model.layers
		x = torch.randn((batch, 1, cfg.hidden_size), device=dev, dtype=torch.float16)
		for l in layers[:4]:
			l.mlp.intermediate(x)
		torch.cuda.synchronize()
		reps = max(1, 256 // len(layers))
		k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
		g = torch.cuda.CUDAGraph()
		s = torch.cuda.Stream()
		s.wait_stream(torch.cuda.current_stream())
		with torch.cuda.stream(s):
			for l in layers:
				l.mlp.intermediate(x)
			s.synchronize()
			with torch.cuda.graph(g, stream=s):
				for l in layers:
					l.mlp.intermediate(x)
			g.replay()
			s.synchronize()
			k0.record(s)
			for _ in range(reps):
				g.replay()
			k1.record(s)
			s.synchronize()
		us = k0.elapsed_time(k1) * 1e3 / (reps * len(layers))
		K, N = cfg.hidden_size, int(layers[0].mlp.gate_proj_qweight.shape[1])      # N is this rank's share under tensor parallelism
		alg = 2 * quantised_bytes(K, N) + batch * (2 * K + 2 * N)           # two weight streams + x + y
		peak, which = measured_peaks()
		ach = alg / us / 1e3
		full = world == 1 and not big
		roof = {'bound': 'hbm', 'kernel': 'skinny_kernel<gate/up, SiLU epilogue> M=%d K=%d N=%d' % (batch, K, N), 'achieved': ach, 'peak': peak, 'unit': 'GB/s',
				'frac': ach / peak, 'peak_source': which, 'us_per_launch': us, 'algorithmic_bytes': alg,
				'traffic': 46.95e6 if full else None,
				'traffic_source': 'ncu capture of the same kernel and shape (dram__bytes_read + dram__bytes_write per launch), profiles/skinny_gateup_m1_ncu_full.md' if full else None}
		if world == 1 and not big and not args.no_prefill:
			tf_peak = 1618.5
			pk = ROOT / 'MEASURED_PEAKS.json'
			if pk.exists():
				tf_peak = float(json.load(open(pk)).get('bf16_tflops', tf_peak))
			prefill = {'bound': 'tensor', 'peak': tf_peak, 'peak_source': 'measured cuBLAS bf16 burst' if pk.exists() else 'fallback', 'unit': 'TFLOP/s',
					   'kernels': prefill_record(G, model, cfg, dev, tf_peak)}
		status = _lib.kernel_status(dev)

	# ---- CPU baseline (rank 0, N=1 only) -----------------------------------------------------------
	cpu = None
	if rank == 0 and world == 1 and not args.no_cpu_baseline:
		cpu = cpu_baseline_record(9)
		cpu['config0'] = cpu_config0()

	exchange = None
	# ---- benchmark configuration 4 as a sub-record: 65B architecture, batch 16, tensor parallel (N >= 2 by default) ----
	config4 = None
	want4 = (args.config4 == 'on') or (args.config4 == 'auto' and world > 1)
	if want4 and not big and not args.layers:
		launches_7b = None
		chain_used = engine.chain is not None
		qa_used = int(engine.used_qkv_attn) + int(engine.used_fused_oproj)
		fused_ar = engine.ar_o is not None
		folded_7b = engine.fuse_norm and batch <= 16 and (world == 1 or engine.ar_o is not None)
		barrier()
		engine.close()
		del engine, model
		torch.cuda.empty_cache()
		exchange = measure_exchange(G, tp, dev, rank, world, barrier, dist) if (world > 1 and fused_ar) else None
		config4 = measure_config4(G, tp, dev, rank, world, barrier, dist if world > 1 else None)
		engine = None
	else:
		chain_used = engine.chain is not None
		qa_used = int(engine.used_qkv_attn) + int(engine.used_fused_oproj)
		fused_ar = engine.ar_o is not None
		folded_7b = engine.fuse_norm and batch <= 16 and (world == 1 or engine.ar_o is not None)

	rc = 0
	if rank == 0:
		# own kernels per rank and step: 4 quantised matmuls + attention per layer (batch 1: the QKV projection and the attention
		# and on one GPU also o_proj are one kernel), embedding + first norm in one kernel,
		# final norm + lm_head + arg-max in one kernel; RMSNorm is otherwise folded into the matmul kernels.  The persistent
		# kernel path: one chain kernel + lm_head.
		if chain_used:
			launches_per_step = 2
		else:
			launches_per_step = ((5 - qa_used) * cfg.num_hidden_layers + 2) if folded_7b else (7 * cfg.num_hidden_layers + 1)
		line = {
			'metric': METRIC, 'value': tok_s, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
			'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16',
			'data': 'synthetic',
			'config': {'workload': WORKLOAD if not big else 'llama65b-arch 4-bit g128 greedy decode, batch 16, 2048-token prompts', 'layers': cfg.num_hidden_layers, 'hidden': cfg.hidden_size, 'groupsize': GROUPSIZE,
					   'parallelism': (('tp%d: QKV and gate/up by columns, o_proj and down by rows, ' % world) + ('all-reduce fused into those kernels over peer memory' if fused_ar else 'one NCCL all-reduce after each')) if world > 1 else 'single GPU',
					   'step': 'persistent chain kernel' if chain_used else (('attention block (QKV projection, rotary, attention, o_proj, residual) in one kernel, gate/up and down_proj one kernel each, CUDA graph' if qa_used == 2 else 'QKV projection + attention in one kernel, one kernel per other projection, CUDA graph') if qa_used else 'one kernel per projection, CUDA graph'),
					   'l2': 'inputs larger than L2: 3.6 GB of weights + KV cache are streamed every step'},
			'e2e': {'value': e2e_tok_s, 'unit': UNIT, 'h2d_bytes_per_step': 8 * batch, 'd2h_bytes_per_step': 8 * batch},
			'gpu_launches': launches_per_step * args.steps,
			'roofline': roof, 'prefill': prefill, 'parity': parity, 'config4': config4, 'exchange': exchange, 'cpu_baseline': cpu, 'clocks': clocks, 'kernel_status': status,
		}
		print(json.dumps(line), flush=True)
		if config4 is not None and config4.get('kernel_status'):
			status = status or config4['kernel_status']
		if status != 0:
			sys.stderr.write('bench.py: a kernel reported status %d (see gptq_triton_b200._lib.kernel_status)\n' % status)
			rc = 3
	if world > 1:
		# Leave without tearing the communicator down: destroying a process group while CUDA graphs
		# that captured its collectives are alive was seen to block until the NCCL watchdog fired.
		torch.cuda.synchronize()
		dist.barrier()
		sys.stdout.flush()
		os._exit(rc)
	if rc:
		sys.exit(rc)


def kernel_case(args):
	"""Small stand-alone case for profilers: a few launches of one decode kernel over rotating
	weight copies (larger than L2 together), nothing else.  `--kernel-case gateup|qkv|o|down`."""
	import torch
	import gptq_triton_b200 as G
	from gptq_triton_b200 import synth
	dev = torch.device('cuda', 0)
	M = args.m
	if args.kernel_case == 'prefill':
		# tensor-core kernel: M x 4096 x 4096 quantised matmul, three launches
		K, N = 4096, 4096
		t = synth.quant_tensors(K, N, GROUPSIZE, seed=2)
		w = tuple(v.to(dev) for v in (t['qweight'], t['scales'], t['qzeros']))
		x = synth.activations((max(M, 2048), K), seed=1).to(dev)
		for i in range(3):
			G.qmatmul(GROUPSIZE, x, *w)
		torch.cuda.synchronize()
		print(json.dumps({'kernel_case': 'prefill', 'M': int(x.shape[0]), 'launches': 3}))
		return
	if args.kernel_case == 'chain':
		# the persistent decode-step kernel on four layers of the 7B architecture after a 2048-token prompt (about 1 GB on
		# the device): a few steps, nothing else; also prints the step time of both engines
		from gptq_triton_b200.llama import LlamaConfig
		cfg = LlamaConfig(num_hidden_layers=4, max_position_embeddings=4096)
		model = G.synthetic_quantized_llama(cfg, groupsize=GROUPSIZE, seed=1, device=dev)
		prompt = torch.randint(0, cfg.vocab_size, (1, PROMPT), generator=torch.Generator().manual_seed(3)).to(dev)
		out = {'kernel_case': 'chain', 'layers': 4}
		for name, flag in (('chain', '1'), ('kernel_per_projection', '0')):
			os.environ['GPTQ_B200_CHAIN'] = flag
			e = G.DecodeEngine(model, batch=1, max_seq=PROMPT + 64, use_graph=(flag == '0'))
			assert (e.chain is not None) == (flag == '1')
			e.prefill(prompt)
			for _ in range(5):
				e.step()
			torch.cuda.synchronize()
			e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
			e0.record()
			for _ in range(20):
				e.step()
			e1.record()
			torch.cuda.synchronize()
			out[name + '_ms_per_step'] = e0.elapsed_time(e1) / 20
		print(json.dumps(out))
		return
	if args.kernel_case == 'lmhead':
		# final RMSNorm + fp16 lm_head + arg-max: 32000 x 4096 weights (262 MB, larger than L2), timed with CUDA events
		from gptq_triton_b200 import _lib
		L = _lib.lib()
		V, K = 32000, 4096
		h = (torch.randn((M, K), device=dev) * 2).half()
		wn = torch.ones((K,), device=dev, dtype=torch.float16)
		W = (torch.randn((V, K), device=dev) * 0.02).half()
		ss = h.float().pow(2).view(M, K // 32, 32).sum(-1).contiguous()
		logits = torch.zeros((M, V), dtype=torch.float16, device=dev)
		tok = torch.zeros((M,), dtype=torch.int64, device=dev)
		pos = torch.zeros((M,), dtype=torch.int32, device=dev)
		ws = torch.zeros(L.gptq_lm_head_workspace_bytes(M), dtype=torch.uint8, device=dev)
		def run():
			rc = L.gptq_lm_head_argmax(_lib.ptr(h), _lib.ptr(ss), _lib.ptr(wn), _lib.ptr(W), M, K, V, 1e-6, _lib.ptr(logits), _lib.ptr(tok), _lib.ptr(pos),
									   _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
			assert rc == 0
		for _ in range(3):
			run()
		torch.cuda.synchronize()
		e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
		e0.record()
		for _ in range(10):
			run()
		e1.record()
		torch.cuda.synchronize()
		us = e0.elapsed_time(e1) * 100
		x = (h.float() * torch.rsqrt(h.float().pow(2).mean(-1, keepdim=True) + 1e-6)).half()
		t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
		for _ in range(3):
			(x @ W.t()).argmax(-1)
		t0.record()
		for _ in range(10):
			(x @ W.t()).argmax(-1)
		t1.record()
		torch.cuda.synchronize()
		peak, which = measured_peaks()
		alg = V * K * 2 + M * K * 2 + M * V * 2
		print(json.dumps({'kernel_case': 'lmhead', 'M': M, 'us': us, 'gbs': alg / us / 1e3, 'frac': alg / us / 1e3 / peak, 'peak_source': which,
						  'cublas_plus_argmax_us': t0.elapsed_time(t1) * 100, 'launches': 13}))
		return
	if args.kernel_case == 'attn':
		# single-query attention over rotating caches (together larger than L2) at 2100 tokens of context:
		# --m sequences x --heads heads (1 x 32: the 7B decode step; 16 x 8 / 16 x 16 / 16 x 32: configuration 4 per rank at tp8 / 4 / 2)
		from gptq_triton_b200.fused_attention import attn_decode
		B, H, S, D = M, args.heads, 2200, 128
		per = 2 * B * H * S * D * 2
		ncache = max(2, min(8, (300 << 20) // per + 1))
		caches = [(torch.randn((B, H, S, D), device=dev).half(), torch.randn((B, H, S, D), device=dev).half()) for _ in range(ncache)]
		q = torch.randn((B, 1, H, D), device=dev).half().transpose(1, 2)
		pos = torch.full((B, 1), 2100, dtype=torch.int32, device=dev)
		for i in range(ncache):
			attn_decode(q, caches[i][0], caches[i][1], pos, 2101)
		torch.cuda.synchronize()
		e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
		reps = 4
		e0.record()
		for _ in range(reps):
			for i in range(ncache):
				attn_decode(q, caches[i][0], caches[i][1], pos, 2101)
		e1.record()
		torch.cuda.synchronize()
		us = e0.elapsed_time(e1) * 1e3 / (reps * ncache)
		alg = 2 * B * H * 2101 * D * 2
		peak, which = measured_peaks()
		print(json.dumps({'kernel_case': 'attn', 'batch': B, 'heads': H, 'ctx': 2101, 'us': us, 'gbs': alg / us / 1e3, 'frac': alg / us / 1e3 / peak,
						  'peak_source': which, 'launches': ncache * (reps + 1)}))
		return
	if args.kernel_case == 'qkvattn':
		# decode attention block of one sequence at 2100 tokens of context, 7B shapes: the one-kernel form (projection + rotary +
		# cache append + attention, one cluster per head) against the pair qkv_rope + attn_decode, over rotating copies of the
		# weights and caches (together larger than L2), timed with CUDA events
		from gptq_triton_b200.fused_attention import attn_decode, qkv_attn_decode, qkv_attn_oproj_decode, qkv_attn_oproj_scratch, qkv_rope, rope_tables
		K, H, S, D, ctx = 4096, 32, 2200, 128, 2100
		t = synth.quant_tensors(K, 3 * H * D, GROUPSIZE, seed=2)
		ncopy = 8
		ws = [tuple(v.to(dev).clone() for v in (t['qweight'], t['scales'], t['qzeros'])) for _ in range(ncopy)]
		to = synth.quant_tensors(K, K, GROUPSIZE, seed=3)
		wo = [tuple(v.to(dev).clone() for v in (to['qweight'], to['scales'], to['qzeros'])) for _ in range(ncopy)]
		scratch = qkv_attn_oproj_scratch(H, K, dev)
		ss = torch.zeros(K // 32, dtype=torch.float32, device=dev)
		caches = [(torch.randn((1, H, S, D), device=dev).half(), torch.randn((1, H, S, D), device=dev).half()) for _ in range(ncopy)]
		x = synth.activations((1, 1, K), seed=1).to(dev)
		cos, sin = rope_tables(D, S, 10000.0, device=dev)
		pos = torch.full((1, 1), ctx, dtype=torch.int32, device=dev)
		def one(i):
			qw, sc, qz = ws[i]
			return qkv_attn_decode(GROUPSIZE, x, qw, sc, qz, cos, sin, pos.view(-1), caches[i][0], caches[i][1], H)
		def pair(i):
			qw, sc, qz = ws[i]
			q, _, _ = qkv_rope(GROUPSIZE, x, qw, sc, qz, cos, sin, pos, H, D, kv_cache=caches[i])
			return attn_decode(q, caches[i][0], caches[i][1], pos, ctx + 1)
		def block(i):          # the whole attention block: + o_proj + residual, still one kernel
			qw, sc, qz = ws[i]
			return qkv_attn_oproj_decode(GROUPSIZE, x, qw, sc, qz, cos, sin, pos.view(-1), caches[i][0], caches[i][1], H, GROUPSIZE, wo[i][0], wo[i][1],
										 wo[i][2], scratch, residual=x, sumsq_out=ss)
		def pair_o(i):
			return G.qmatmul(GROUPSIZE, pair(i).view(1, K), *wo[i], residual=x.view(1, K), sumsq_out=ss.view(1, -1))
		out = {'kernel_case': 'qkvattn', 'heads': H, 'ctx': ctx + 1, 'timing': 'eager launches, CUDA events (includes launch gaps)'}
		reps = 4
		for name, fn in (('one_kernel_us', one), ('two_kernels_us', pair), ('block_one_kernel_us', block), ('block_three_kernels_us', pair_o)):
			for i in range(ncopy):
				fn(i)
			torch.cuda.synchronize()
			e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
			e0.record()
			for _ in range(reps):
				for i in range(ncopy):
					fn(i)
			e1.record()
			torch.cuda.synchronize()
			out[name] = e0.elapsed_time(e1) * 1e3 / (reps * ncopy)
		alg = K * 3 * H * D // 2 + (K // GROUPSIZE) * 3 * H * D * 5 // 2 + 2 * H * (ctx + 1) * D * 2
		alg_block = alg + K * K // 2 + (K // GROUPSIZE) * K * 5 // 2
		peak, which = measured_peaks()
		out.update({'alg_bytes_block': alg_block, 'frac_block_one_kernel': alg_block / out['block_one_kernel_us'] / 1e3 / peak, 'alg_bytes': alg, 'frac_one_kernel': alg / out['one_kernel_us'] / 1e3 / peak, 'frac_two_kernels': alg / out['two_kernels_us'] / 1e3 / peak,
					'peak_source': which, 'max_abs_diff': float((one(0).float() - pair(0).float()).abs().max()), 'launches': 8 * ncopy * (reps + 1) + 3})
		from gptq_triton_b200 import _lib
		out['kernel_status'] = _lib.kernel_status()
		print(json.dumps(out))
		return
	if args.kernel_case == 'gateup':
		K, N = 4096, 11008
		g, u = synth.quant_tensors(K, N, GROUPSIZE, seed=2), synth.quant_tensors(K, N, GROUPSIZE, seed=3)
		copies = [tuple(t.to(dev).clone() for t in (g['qweight'], g['scales'], g['qzeros'], u['qweight'], u['scales'], u['qzeros'])) for _ in range(4)]
		x = synth.activations((M, K), seed=1).to(dev)
		for i in range(8):
			G.gateup_silu(GROUPSIZE, x, *copies[i % 4])
	else:
		K, N = {'qkv': (4096, 12288), 'o': (4096, 4096), 'down': (11008, 4096)}[args.kernel_case]
		t = synth.quant_tensors(K, N, GROUPSIZE, seed=2)
		copies = [tuple(v.to(dev).clone() for v in (t['qweight'], t['scales'], t['qzeros'])) for _ in range(8)]
		x = synth.activations((M, K), seed=1).to(dev)
		for i in range(8):
			G.qmatmul(GROUPSIZE, x, *copies[i % 8])
	torch.cuda.synchronize()
	print(json.dumps({'kernel_case': args.kernel_case, 'M': M, 'launches': 8}))


def main():
	ap = argparse.ArgumentParser()
	ap.add_argument('--gpus', type=int, default=1)
	ap.add_argument('--steps', type=int, default=64)
	ap.add_argument('--warmup', type=int, default=8)
	ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
	ap.add_argument('--layers', type=int, default=0, help='debug: fewer decoder layers')
	ap.add_argument('--no-cpu-baseline', action='store_true')
	ap.add_argument('--no-parity', action='store_true', help='skip the greedy-decoding parity check before the timed region')
	ap.add_argument('--no-prefill', action='store_true', help='skip the prefill-kernel record')
	ap.add_argument('--config4', default='auto', choices=['auto', 'on', 'off'], help='also measure the 65B-architecture batch-16 configuration as a sub-record (auto: with 2 or more GPUs)')
	ap.add_argument('--workload', default='llama7b', choices=['llama7b', 'llama65b-b16'], help='llama65b-b16: 65B architecture, batch 16 (tensor-parallel runs)')
	ap.add_argument('--no-graph', action='store_true', help='do not capture the decode step in a CUDA graph')
	ap.add_argument('--kernel-case', default=None, choices=['gateup', 'qkv', 'o', 'down', 'prefill', 'attn', 'lmhead', 'chain', 'qkvattn'], help='profiling aid: run a few launches of one kernel and exit')
	ap.add_argument('--m', type=int, default=1, help='batch rows for --kernel-case')
	ap.add_argument('--heads', type=int, default=32, help='heads for --kernel-case attn')
	args = ap.parse_args()
	if args.kernel_case:
		kernel_case(args)
	elif args.impl == 'reference':
		reference_arm(args)
	else:
		gpu_arm(args)


if __name__ == '__main__':
	main()
