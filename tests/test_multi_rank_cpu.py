"""The N > 1 path on CPU: two gloo ranks agree on a disjoint, complete partition of the work
and on the whole-job throughput (all tokens over the slowest rank's time)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from openkimi_b200.partition import aggregate_throughput, shard_batch, shard_documents
    from openkimi_b200.synthetic import random_cu_seqlens

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cu = random_cu_seqlens(65536, 16, seed=0)
    lengths = (cu[1:] - cu[:-1]).tolist()
    mine = shard_documents(lengths, world, rank)
    batch = list(shard_batch(16, world, rank))
    # gather every rank's view
    views = [None] * world
    dist.all_gather_object(views, (mine, batch, sum(lengths[i] for i in mine)))

    def reduce_max(ms):
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    local_ms = 10.0 * (rank + 1)  # rank 1 is the slow one
    tput = aggregate_throughput(local_ms, 32768, 5, world, reduce_max)
    if rank == 0:
        out.put((views, tput, lengths))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_partition_and_aggregate():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    views, tput, lengths = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    docs = sorted(views[0][0] + views[1][0])
    assert docs == list(range(16))                       # complete and disjoint
    assert sorted(views[0][1] + views[1][1]) == list(range(16))
    loads = [views[0][2], views[1][2]]
    assert sum(loads) == 65536 and abs(loads[0] - loads[1]) <= max(lengths)
    assert abs(tput - 2 * 32768 * 5 / 0.020) < 1e-6      # slowest rank: 20 ms


def test_shard_helpers_edge_cases():
    sys.path.insert(0, ROOT)
    from openkimi_b200.partition import shard_batch, shard_documents

    assert [len(shard_batch(4, 8, r)) for r in range(8)] == [1, 1, 1, 1, 0, 0, 0, 0]
    assert [list(shard_batch(10, 4, r)) for r in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert shard_documents([5, 5, 5], 1, 0) == [0, 1, 2]
    assert shard_documents([], 2, 1) == []
