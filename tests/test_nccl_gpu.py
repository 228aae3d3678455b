"""Collectives of this repository's libnccl.so.2 between several processes.

Like k0zi/Vulkanizer's tests/nccl.cpp:233-262 the ranks are separate processes started before any CUDA call; with one GPU
they all share device 0 (the ranks then meet on the host), with more GPUs each rank gets its own and the ranks meet on
device-side flags over NVLink. Results are compared exactly.
"""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

WORKER = Path(__file__).with_name("nccl_worker.py")


def run_ranks(nranks, devices):
    with tempfile.TemporaryDirectory() as tmp:
        id_file = Path(tmp) / "nccl_id"
        env = dict(os.environ, VKZB_NCCL_TIMEOUT_S="60")
        procs = [subprocess.Popen([sys.executable, str(WORKER), str(id_file), str(nranks), str(r), str(devices[r])], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(nranks)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n[timed out]"
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and f"rank {r} ok" in out, f"rank {r} failed:\n{out[-3000:]}"


@pytest.mark.gpu
def test_three_ranks_sharing_one_gpu(cuda):
    run_ranks(3, [0, 0, 0])


@pytest.mark.gpu
def test_one_rank_per_gpu(cuda):
    n = cuda.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = min(n, 4)
    run_ranks(n, list(range(n)))


@pytest.mark.gpu
def test_single_rank_communicator(cuda):
    run_ranks(1, [0])
