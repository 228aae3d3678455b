"""Host-side logic of the multi-GPU path on CPU: the block-cyclic column partition, and two gloo ranks agreeing on it and
on the communicator id they would hand to ncclCommInitRank."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from bench_multi_gpu import column_chunks, round_widths, shard

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("n, ranks", [(32768, 1), (32768, 2), (32768, 4), (32768, 8), (8192, 2), (8192, 8), (4096, 4)])
def test_partition_covers_every_column_once_in_gather_order(n, ranks):
    rounds = column_chunks(n, ranks)
    covered = []
    expect_first = 0
    for j, w, round_first, firsts in rounds:
        assert round_first == expect_first and w % 256 == 0
        # ncclAllGather puts rank r's block at offset r * count: the chunks of a round must lie in rank order, side by side
        assert firsts == [round_first + r * w for r in range(ranks)]
        covered += [(f, f + w) for f in firsts]
        expect_first += ranks * w
    assert expect_first == n
    covered.sort()
    assert covered[0][0] == 0 and all(a[1] == b[0] for a, b in zip(covered, covered[1:])) and covered[-1][1] == n
    per_rank = [sum(w for _, w, _, _ in rounds)] * ranks
    assert sum(per_rank) == n


@pytest.mark.parametrize("units, ranks", [(256, 1), (256, 2), (256, 8), (256, 3), (5, 8), (0, 4)])
def test_batch_entries_are_dealt_in_contiguous_shares_that_differ_by_at_most_one(units, ranks):
    shares = [shard(units, ranks, r) for r in range(ranks)]
    assert shares[0][0] == 0 and sum(c for _, c in shares) == units
    assert all(a[0] + a[1] == b[0] for a, b in zip(shares, shares[1:]))
    assert max(c for _, c in shares) - min(c for _, c in shares) <= 1


def test_rounds_are_uniform_so_each_gather_hides_behind_the_next_product():
    assert round_widths(32768, 8) == [512] * 8
    assert round_widths(32768, 4) == [1024] * 8
    assert round_widths(32768, 2) == [1024] * 16
    assert round_widths(32768, 1) == [2048] * 16
    assert round_widths(8192, 8) == [256] * 4
    assert round_widths(32768, 4, 2048) == [2048] * 4


def test_uneven_split_is_refused():
    with pytest.raises(AssertionError):
        column_chunks(1000, 3)


WORKER = r'''
import os, sys, hashlib
sys.path.insert(0, sys.argv[1])
import torch.distributed as dist
from bench_multi_gpu import column_chunks, round_widths, shard
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
box = [bytes(range(128)) if rank == 0 else None]          # stands in for ncclGetUniqueId on rank 0
dist.broadcast_object_list(box, src=0)
assert box[0] == bytes(range(128))
rounds = column_chunks(8192, world)
mine = [(firsts[rank], w) for _, w, _, firsts in rounds]
gathered = [None] * world
dist.all_gather_object(gathered, mine)
flat = sorted(c for part in gathered for c in part)
assert flat[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(flat, flat[1:])) and flat[-1][0] + flat[-1][1] == 8192, flat
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_gloo_ranks_agree_on_partition_and_id(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29577", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for r, p in enumerate(procs):
        out, _ = p.communicate(timeout=120)
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-2000:]


def test_reference_arm_samples_the_workload_the_other_arm_runs():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.reference_sample_of("cfg2_f16_tn_8192") == ("f16", "T", "N", 2048, 0.02)
    assert bench.reference_sample_of("cfg2_bf16_tn_8192")[0] == "bf16"
    assert bench.reference_sample_of("cfg5b_bf16_32768_nsharded") == ("bf16", "T", "N", 2048, 1.0)
    kind, ta, tb, size, _ = bench.reference_sample_of("cfg1_sgemm_nn_512")
    assert (kind, ta, tb, size) == ("f32", "N", "N", 512)
    assert bench.reference_sample_of("cfg3_s8_tn_11008x512x4096")[0] == "f32"  # int8 values as f32: timing only
