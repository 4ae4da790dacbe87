"""Tensor-parallel decode on 2 GPUs (skipped with fewer): tests/tp_check.py run as one
process per GPU must report identical greedy tokens for the sharded and the whole model."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tp_two_gpus_matches_single_gpu():
	if torch.cuda.device_count() < 2:
		pytest.skip('needs 2 GPUs')
	env = dict(os.environ, NCCL_NVLS_ENABLE='0')
	cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr', '127.0.0.1',
		   '--master-port', '29533', str(Path(__file__).resolve().parent / 'tp_check.py')]
	r = subprocess.run(cmd, cwd=Path(__file__).resolve().parent.parent, env=env, capture_output=True, text=True, timeout=900)
	assert 'TP_CHECK OK' in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
