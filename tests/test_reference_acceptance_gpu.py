"""k0zi/Vulkanizer's own acceptance tests, unmodified, against this repository's drop-in libraries.

oracle/Makefile compiles the reference's tests/cublas.cpp and tests/nccl.cpp from where they lie in its tree, against its own
headers, and links them with vulkanizer_b200/lib/libcublas.so.12, libcublasLt.so.12 and libnccl.so.2 (oracle/_ref/ holds the
binaries; the reference tree itself is not needed at run time). Each must exit 0 on a B200: every GEMM case of the reference's
table, its trsm / LU / QR checks, grouped and pointer-array batches, cublasLt epilogues, and every collective of its NCCL test
run through the hand-written CUDA kernels of this repository.
"""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF_BIN = ROOT / "oracle" / "_ref"


def run_binary(name, limit=600):
    binary = REF_BIN / name
    if not binary.exists():
        pytest.skip(f"{binary} was not built (the reference tree was absent when oracle/Makefile ran)")
    env = dict(os.environ, LD_LIBRARY_PATH=str(ROOT / "vulkanizer_b200" / "lib") + ":" + os.environ.get("LD_LIBRARY_PATH", ""),
               VKZB_NCCL_TIMEOUT_S="60")
    done = subprocess.run([str(binary)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=limit)
    tail = done.stdout[-4000:]
    assert done.returncode == 0, f"{name} exited {done.returncode}:\n{tail}"
    assert "FAILED" not in done.stdout, tail
    return done.stdout


@pytest.mark.gpu
def test_reference_cublas_acceptance_test_passes_unmodified(cuda):
    out = run_binary("ref_cublas_test")
    assert "OK" in out.splitlines()[-1] or "ok" in out.lower()


@pytest.mark.gpu
def test_reference_nccl_acceptance_test_passes_unmodified(cuda):
    out = run_binary("ref_nccl_test")
    assert out.strip().endswith("OK")
