"""Builds libgptq_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Usage:  python -m gptq_triton_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / 'csrc'
LIB = PKG / 'libgptq_b200.so'

NVCC_FLAGS = [
	'-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
	'--compiler-options', '-fPIC', '-shared',
]


def _nvcc() -> str:
	for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
		if cand and Path(cand).exists():
			return cand
	raise RuntimeError('nvcc not found; set NVCC or put it on PATH')


def sources():
	return sorted(CSRC.glob('*.cu'))


def up_to_date() -> bool:
	if not LIB.exists():
		return False
	t = LIB.stat().st_mtime
	deps = list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh')) + list(CSRC.glob('*.inl')) + list((PKG.parent / 'include').glob('*.h'))
	return all(d.stat().st_mtime <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
	if not force and up_to_date():
		return LIB
	cmd = [_nvcc(), *NVCC_FLAGS, '-o', str(LIB), *map(str, sources())]
	if verbose:
		cmd.insert(1, '-Xptxas')
		cmd.insert(2, '-v')
		print(' '.join(cmd))
	r = subprocess.run(cmd, capture_output=True, text=True)
	if verbose or r.returncode != 0:
		sys.stderr.write(r.stdout + r.stderr)
	if r.returncode != 0:
		raise RuntimeError('nvcc failed building libgptq_b200.so')
	return LIB


if __name__ == '__main__':
	build(force='--force' in sys.argv, verbose='--verbose' in sys.argv)
	print(LIB)
