"""One rank of the collective test: run as a child process by tests/test_nccl_gpu.py (and by hand on a multi-GPU box).

    python tests/nccl_worker.py <id file> <nranks> <rank> <device>

Every collective of this repository's libnccl.so.2 is run on integer-valued data, so the expected results are exact
(`==` comparisons, as in k0zi/Vulkanizer's tests/nccl.cpp:88, 111-112). Prints "rank <r> ok" on success.
"""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    id_file, nranks, rank, device = Path(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
    import torch
    from vulkanizer_b200 import capi

    torch.cuda.set_device(device)
    torch.zeros(1, device="cuda")
    if rank == 0:
        tmp = id_file.with_suffix(".tmp")
        tmp.write_bytes(capi.NcclComm.unique_id())
        tmp.rename(id_file)
    deadline = time.time() + 60
    while not id_file.exists():
        assert time.time() < deadline, "rank 0 never published the unique id"
        time.sleep(0.01)
    comm = capi.NcclComm(nranks, rank, id_file.read_bytes())
    stream = torch.cuda.Stream()
    s = stream.cuda_stream
    n = 1000

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def val(r, count=n):  # what rank r contributes
        return (np.arange(count) % 17 - 8 + 3 * r).astype(np.float32)

    with torch.cuda.stream(stream):
        # all-gather, out of place and in place
        send, recv = dev(val(rank)), torch.zeros(n * nranks, device="cuda")
        comm.all_gather(send.data_ptr(), recv.data_ptr(), n, "float32", s)
        stream.synchronize()
        assert np.array_equal(recv.cpu().numpy(), np.concatenate([val(r) for r in range(nranks)]))
        inplace = torch.zeros(n * nranks, device="cuda")
        inplace[rank * n:(rank + 1) * n] = send
        comm.all_gather(inplace.data_ptr() + 4 * rank * n, inplace.data_ptr(), n, "float32", s)
        stream.synchronize()
        assert np.array_equal(inplace.cpu().numpy(), np.concatenate([val(r) for r in range(nranks)]))
        # all-reduce: sum in place, max out of place, bf16 average, int64 product-free sum
        x = dev(val(rank))
        comm.all_reduce(x.data_ptr(), x.data_ptr(), n, "float32", capi.NCCL_SUM, s)
        stream.synchronize()
        assert np.array_equal(x.cpu().numpy(), sum(val(r) for r in range(nranks)))
        y, out = dev(val(rank)), torch.zeros(n, device="cuda")
        comm.all_reduce(y.data_ptr(), out.data_ptr(), n, "float32", capi.NCCL_MAX, s)
        stream.synchronize()
        assert np.array_equal(out.cpu().numpy(), np.max([val(r) for r in range(nranks)], axis=0))
        h = dev(val(rank)).to(torch.bfloat16)
        comm.all_reduce(h.data_ptr(), h.data_ptr(), n, "bfloat16", capi.NCCL_AVG, s)
        stream.synchronize()
        want = torch.from_numpy(sum(val(r) for r in range(nranks)) / nranks).to(torch.bfloat16)
        assert torch.equal(h.cpu(), want)
        i64 = dev((np.arange(7) + rank * 10).astype(np.int64))  # fewer elements than ranks would leave empty slices: 7 > nranks here
        comm.all_reduce(i64.data_ptr(), i64.data_ptr(), 7, "int64", capi.NCCL_SUM, s)
        stream.synchronize()
        assert np.array_equal(i64.cpu().numpy(), sum(np.arange(7) + r * 10 for r in range(nranks)))
        # broadcast from the last rank
        root = nranks - 1
        b = dev(val(rank))
        comm.broadcast(b.data_ptr(), b.data_ptr(), n, "float32", root, s)
        stream.synchronize()
        assert np.array_equal(b.cpu().numpy(), val(root))
        # reduce-scatter
        full = dev(np.concatenate([val(rank) + 100 * q for q in range(nranks)]))
        part = torch.zeros(n, device="cuda")
        comm.reduce_scatter(full.data_ptr(), part.data_ptr(), n, "float32", capi.NCCL_SUM, s)
        stream.synchronize()
        assert np.array_equal(part.cpu().numpy(), sum(val(r) + 100 * rank for r in range(nranks)))
        # reduce to rank 0, gather to rank 1 % nranks, all-to-all
        r0 = torch.zeros(n, device="cuda")
        comm.reduce(dev(val(rank)).data_ptr(), r0.data_ptr(), n, "float32", 0, capi.NCCL_SUM, s)
        stream.synchronize()
        if rank == 0:
            assert np.array_equal(r0.cpu().numpy(), sum(val(r) for r in range(nranks)))
        groot = 1 % nranks
        g = torch.zeros(n * nranks, device="cuda")
        keep = dev(val(rank))
        comm.gather(keep.data_ptr(), g.data_ptr(), n, "float32", groot, s)
        stream.synchronize()
        if rank == groot:
            assert np.array_equal(g.cpu().numpy(), np.concatenate([val(r) for r in range(nranks)]))
        a2a_send = dev(np.concatenate([val(rank) + 1000 * q for q in range(nranks)]))
        a2a_recv = torch.zeros(n * nranks, device="cuda")
        comm.all_to_all(a2a_send.data_ptr(), a2a_recv.data_ptr(), n, "float32", s)
        stream.synchronize()
        assert np.array_equal(a2a_recv.cpu().numpy(), np.concatenate([val(r) + 1000 * rank for r in range(nranks)]))
        # a large, repeated gather: buffers are mapped once and reused
        big = 1 << 22
        src = torch.full((big,), float(rank + 1), device="cuda")
        dst = torch.zeros(big * nranks, device="cuda")
        for _ in range(3):
            comm.all_gather(src.data_ptr(), dst.data_ptr(), big, "float32", s)
        stream.synchronize()
        assert torch.equal(dst.view(nranks, big)[:, ::4096].cpu(), torch.arange(1, nranks + 1, dtype=torch.float32)[:, None].expand(nranks, big // 4096))
    with torch.cuda.stream(stream):
        # one group of ten collectives on this communicator, each with buffers of its own: more than the ring of posted
        # addresses holds, so the group runs in batches and no operation may see another one's buffers
        ins = [dev(val(rank) + 7 * j) for j in range(10)]
        outs = [torch.zeros(n * nranks if j % 2 == 0 else n, device="cuda") for j in range(10)]
        comm.group_start()
        for j in range(10):
            if j % 2 == 0:
                comm.all_gather(ins[j].data_ptr(), outs[j].data_ptr(), n, "float32", s)
            else:
                comm.all_reduce(ins[j].data_ptr(), outs[j].data_ptr(), n, "float32", capi.NCCL_SUM, s)
        comm.group_end()
        stream.synchronize()
        for j in range(10):
            want = np.concatenate([val(r) + 7 * j for r in range(nranks)]) if j % 2 == 0 else sum(val(r) + 7 * j for r in range(nranks))
            assert np.array_equal(outs[j].cpu().numpy(), want), f"grouped operation {j}"
        # twenty ungrouped collectives in a row with changing buffers: the ring wraps twice, a fast rank may not overwrite
        # addresses a slower one has yet to read
        for j in range(20):
            src_j = dev(val(rank) + j)
            dst_j = torch.zeros(n * nranks, device="cuda")
            comm.all_gather(src_j.data_ptr(), dst_j.data_ptr(), n, "float32", s)
            stream.synchronize()
            assert np.array_equal(dst_j.cpu().numpy(), np.concatenate([val(r) + j for r in range(nranks)])), f"gather {j}"
        # a sum with premultiplied contributions: rank r scales by r + 1 (tests/nccl.cpp:122-133)
        op = comm.premul_sum(float(rank + 1))
        ones = torch.ones(16, device="cuda")
        comm.all_reduce(ones.data_ptr(), ones.data_ptr(), 16, "float32", op, s)
        stream.synchronize()
        assert (ones.cpu().numpy() == nranks * (nranks + 1) / 2).all()
        comm.destroy_op(op)
        # point to point: a ring, then an exchange with every rank (itself included), each in one group (tests/nccl.cpp:178-200)
        sbuf = torch.full((32,), rank, dtype=torch.int32, device="cuda")
        rbuf = torch.full((32,), -1, dtype=torch.int32, device="cuda")
        comm.group_start()
        comm.send(sbuf.data_ptr(), 32, "int32", (rank + 1) % nranks, s)
        comm.recv(rbuf.data_ptr(), 32, "int32", (rank + nranks - 1) % nranks, s)
        comm.group_end()
        stream.synchronize()
        assert (rbuf.cpu().numpy() == (rank + nranks - 1) % nranks).all()
        got = [torch.full((32,), -1, dtype=torch.int32, device="cuda") for _ in range(nranks)]
        comm.group_start()
        for q in range(nranks):
            comm.send(sbuf.data_ptr(), 32, "int32", q, s)
            comm.recv(got[q].data_ptr(), 32, "int32", q, s)
        comm.group_end()
        stream.synchronize()
        for q in range(nranks):
            assert (got[q].cpu().numpy() == q).all(), f"exchange with rank {q}"
        # even and odd ranks part ways, keys descending so the order inside each half is reversed (tests/nccl.cpp:201-220)
        half = comm.split(rank % 2, -rank)
        members = [r for r in range(nranks) if r % 2 == rank % 2]
        assert half.nranks == len(members) and half.rank == sum(1 for r in members if r > rank)
        v = torch.full((4,), rank, dtype=torch.int32, device="cuda")
        half.all_reduce(v.data_ptr(), v.data_ptr(), 4, "int32", capi.NCCL_SUM, s)
        stream.synchronize()
        assert (v.cpu().numpy() == sum(members)).all()
        half.destroy()
        assert comm.split(-1, 0) is None   # NCCL_SPLIT_NOCOLOR
    # a GEMM whose tiles are written to every rank's copy of D as they are produced (output mirrors): rank r computes
    # columns [r * w, (r + 1) * w) of D = A^T B, and afterwards every rank holds all of D
    from oracle import pyoracle as orc
    m, k, w = 384, 192, 256
    lt = capi.CublasLt()
    A, av = orc.fill_lcg("f16", m * k, 1)
    Bfull, bv = orc.fill_lcg("f16", k * w * nranks, 2)
    dA = torch.from_numpy(A.view(np.int16)).cuda()
    dB = torch.from_numpy(Bfull.view(np.int16)).cuda()
    D = torch.full((m * w * nranks,), -1.0, device="cuda")
    peers = comm.exchange_buffer(D.data_ptr())
    lt.set_output_mirrors(D.data_ptr(), D.numel() * 4, [peers[p] for p in range(nranks) if p != rank])
    with torch.cuda.stream(stream):
        comm.barrier(s)
        mine = D.data_ptr() + 4 * rank * w * m
        lt.matmul(capi.OP_T, capi.OP_N, m, w, k, 1.0, dA.data_ptr(), capi.CUDA_R_16F, k, dB.data_ptr() + 2 * rank * w * k, capi.CUDA_R_16F, k, 0.0,
                  mine, capi.CUDA_R_32F, m, mine, capi.CUDA_R_32F, m, stream=s)
        comm.barrier(s)
        stream.synchronize()
    want = (av.reshape(m, k).astype(np.float64) @ bv.reshape(w * nranks, k).astype(np.float64).T).T  # [col, row]
    assert np.allclose(D.cpu().numpy().reshape(w * nranks, m), want, atol=1e-3), "mirrored tiles did not arrive on every rank"
    # a result the bulk stores cannot write (column length not a multiple of 16 bytes) must be refused, not silently left unmirrored
    status = lt.matmul(capi.OP_T, capi.OP_N, m - 2, w, k, 1.0, dA.data_ptr(), capi.CUDA_R_16F, k, dB.data_ptr(), capi.CUDA_R_16F, k, 0.0,
                       mine, capi.CUDA_R_32F, m, mine, capi.CUDA_R_32F, m, stream=s, check=False)
    assert status == (capi.STATUS_NOT_SUPPORTED if nranks > 1 else capi.STATUS_SUCCESS), status
    lt.set_output_mirrors(0, 0, [])
    torch.cuda.synchronize()
    comm.barrier(s)
    torch.cuda.synchronize()
    lt.destroy()
    assert comm.async_error() == 0
    comm.destroy()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
