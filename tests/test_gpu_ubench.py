"""Builds and runs the tcgen05.mma micro-benchmark (tests/ubench/tcgen05_mma_rate.cu) and checks
that the figures the decode kernel's design rests on still hold on the GPU at hand: a 128-column
k-step takes about 67 cycles and holds its issuing thread for nearly as long; a 16-column k-step is
barely cheaper (about 59 cycles), whatever the accumulator or M; one decode tile's 29 instructions
keep the tensor path busy for about 1.5 K cycles."""
import os
import re
import shutil
import subprocess

import pytest
import torch

from conftest import REPO

pytestmark = pytest.mark.gpu


def test_tcgen05_mma_cycle_table(tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed on this machine")
    exe = tmp_path / "tcgen05_mma_rate"
    src = os.path.join(REPO, "tests", "ubench", "tcgen05_mma_rate.cu")
    subprocess.run([nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(exe), src],
                   check=True, capture_output=True, timeout=300)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    print("\n" + r.stdout)
    rows = {}
    for line in r.stdout.splitlines():
        m = re.match(r"(.+?)\s*:\s+([\d.]+) cycles.*?([\d.]+) cycles", line)
        if m:
            rows[m.group(1).strip()] = (float(m.group(2)), float(m.group(3)))
    assert 55 <= rows["m128 n128 TS (A in tensor memory)"][0] <= 85
    assert rows["m128 n128 TS (A in tensor memory)"][1] >= 40            # the issuing thread is held at the pipe's rate
    assert 45 <= rows["m128 n16 TS"][0] <= 75
    assert rows["m128 n16 TS, two accumulators alternating"][0] >= 0.8 * rows["m128 n16 TS"][0]
    tile = rows["one decode tile: 13 x n128 + 8 x n16 TS + 8 x n16 SS"]
    assert 1200 <= tile[0] <= 2200
    # the same with the P.V operand laid out as the kernel's V tile, alone and beside other warps'
    # shared-memory traffic: traffic can only slow the tensor path down
    tile_mn = rows["one decode tile, P.V operand MN-major as in the kernel"]
    heavy = rows["one decode tile (MN-major) + 15 warps of heavy shared-memory traffic"]
    assert 1200 <= tile_mn[0] <= 3000
    assert heavy[0] >= 0.95 * tile_mn[0]
