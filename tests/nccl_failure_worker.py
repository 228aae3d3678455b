"""Failure paths of libnccl.so.2, one scenario per invocation; run as a child process by tests/test_nccl_failures_gpu.py.

    python tests/nccl_failure_worker.py <scenario> <id file> <rank>

No scenario makes a GPU fault or hang: the failures are made on the host (a rank that stays away, a communicator aborted from
another thread) or are a bounded device-side wait that runs out and reports a status.
"""
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    scenario, id_file, rank = sys.argv[1], Path(sys.argv[2]), int(sys.argv[3])
    import torch
    from vulkanizer_b200 import capi

    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    if rank == 0 and not id_file.exists():
        tmp = id_file.with_suffix(".tmp")
        tmp.write_bytes(capi.NcclComm.unique_id())
        tmp.rename(id_file)
    deadline = time.time() + 30
    while not id_file.exists():
        assert time.time() < deadline
        time.sleep(0.01)
    uid = id_file.read_bytes()

    if scenario == "missing-rank":
        # three ranks expected, two come: the init gives up after VKZB_NCCL_TIMEOUT_S with ncclRemoteError
        t0 = time.time()
        try:
            capi.NcclComm(3, rank, uid)
        except capi.NcclError as e:
            assert "remote" in str(e), e
            print(f"rank {rank} gave up after {time.time() - t0:.1f} s: ok", flush=True)
            return
        raise AssertionError("init returned although a rank never joined")

    if scenario == "skipped-collective":
        # two ranks on one GPU; rank 1 never enters the all-reduce: rank 0's call ends with ncclRemoteError, nothing hangs
        comm = capi.NcclComm(2, rank, uid)
        x = torch.ones(8, device="cuda")
        if rank == 0:
            try:
                comm.all_reduce(x.data_ptr(), x.data_ptr(), 8, "float32")
            except capi.NcclError as e:
                assert "remote" in str(e) and "timed out" in str(e), e
                print("rank 0 timed out cleanly: ok", flush=True)
                return
            raise AssertionError("the collective returned although the peer skipped it")
        time.sleep(3.0)  # stays away, between steps, with nothing in flight
        print("rank 1 stayed away: ok", flush=True)
        return

    if scenario == "abort":
        # two ranks; rank 1 stays away; a second thread of rank 0 aborts the communicator while the main thread waits
        comm = capi.NcclComm(2, rank, uid)
        x = torch.ones(8, device="cuda")
        if rank == 0:
            threading.Timer(0.5, comm.abort).start()
            t0 = time.time()
            try:
                comm.all_reduce(x.data_ptr(), x.data_ptr(), 8, "float32")
            except capi.NcclError as e:
                took = time.time() - t0
                assert "aborted" in str(e), e
                assert took < 5.0, f"the abort took {took:.1f} s to release the waiter"
                assert comm.async_error() == 6  # ncclRemoteError
                print(f"rank 0 released by the abort after {took:.2f} s: ok", flush=True)
                return
            raise AssertionError("the collective returned although the peer never came")
        time.sleep(2.0)
        print("rank 1 stayed away: ok", flush=True)
        return

    if scenario == "lost-peer-on-device":
        # one rank: the device-side barrier waits (50 ms, VKZB_NCCL_DEVICE_WAIT_MS) for a flag nobody writes, gives up, and
        # the status word says so; the stream and the context stay usable
        comm = capi.NcclComm(1, 0, uid)
        stream = torch.cuda.Stream()
        assert comm.async_error() == 0
        t0 = time.time()
        comm.self_test_lost_peer(stream.cuda_stream)
        stream.synchronize()
        took = time.time() - t0
        assert 0.03 < took < 5.0, took
        assert comm.async_error() == 6  # ncclRemoteError
        y = torch.arange(8, device="cuda").sum().item()  # the context still works
        assert y == 28
        comm.destroy()
        print(f"device wait ran out after {took * 1e3:.0f} ms: ok", flush=True)
        return
    raise SystemExit(f"unknown scenario {scenario}")


if __name__ == "__main__":
    main()
