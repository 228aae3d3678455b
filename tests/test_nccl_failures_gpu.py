"""Failure detection of libnccl.so.2 (the reference's counterpart: bounded waits and ncclCommAbort, src/nccl/nccl.cpp:238,
554-557). Every failure is made on the host or is a bounded wait that runs out; no test faults or hangs a GPU. The ranks of a
scenario are child processes on device 0, so the ranks meet on the host (kernels of different ranks never wait on one another
on one GPU); the device-side wait is exercised by a single rank against a flag that nobody writes.
"""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

WORKER = Path(__file__).with_name("nccl_failure_worker.py")


def run(scenario, ranks, env_extra, limit=120):
    with tempfile.TemporaryDirectory() as tmp:
        id_file = Path(tmp) / "nccl_id"
        env = dict(os.environ, **env_extra)
        procs = [subprocess.Popen([sys.executable, str(WORKER), scenario, str(id_file), str(r)], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in ranks]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=limit)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n[hung: killed by the test]"
            outs.append(out)
        for p, out in zip(procs, outs):
            assert p.returncode == 0 and ": ok" in out, out[-3000:]
        return outs


@pytest.mark.gpu
def test_a_rank_that_never_joins_ends_the_init_with_an_error(cuda):
    run("missing-rank", [0, 1], {"VKZB_NCCL_TIMEOUT_S": "2"})


@pytest.mark.gpu
def test_a_skipped_collective_times_out_cleanly(cuda):
    run("skipped-collective", [0, 1], {"VKZB_NCCL_TIMEOUT_S": "2"})


@pytest.mark.gpu
def test_abort_from_another_thread_releases_a_waiting_rank(cuda):
    run("abort", [0, 1], {"VKZB_NCCL_TIMEOUT_S": "60"})


@pytest.mark.gpu
def test_device_side_wait_runs_out_and_reports(cuda):
    run("lost-peer-on-device", [0], {"VKZB_NCCL_DEVICE_WAIT_MS": "50"})
