"""The N > 1 plumbing of the benchmark on CPU: two `gloo` ranks, the barrier, the max-over-ranks
of the timings and the whole-job aggregate.  The data path itself has no collective (replicas
only), so this is all the multi-rank logic there is besides the replica sharding, which
tests/test_plan.py and tests/test_packing.py cover."""
import os
import socket
import sys

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    sys.path.insert(0, ROOT)
    import bench
    ranks = bench.Ranks(world, rank, backend="gloo")
    ranks.barrier()
    ms = 10.0 if rank == 0 else 25.0          # rank 1 is the slow one
    tokens = 1000.0 if rank == 0 else 3000.0  # and processed more units
    value = bench.whole_job_throughput(ranks, tokens, steps=4, ms_this_rank=ms)
    mx = ranks.max(float(rank))
    sm = ranks.sum(1.0)
    ranks.close()
    out.put((rank, value, mx, sm))


def test_two_gloo_ranks_aggregate_like_the_contract_says():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, value, mx, sm in results:
        # (1000 + 3000) tokens x 4 steps / 25 ms = 640,000 tokens/s on every rank
        assert abs(value - 640000.0) < 1e-6
        assert mx == 1.0 and sm == 2.0


def test_single_rank_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    ranks = bench.Ranks(1, 0, backend="gloo")
    assert bench.whole_job_throughput(ranks, 500.0, 2, 10.0) == 100000.0
    ranks.close()
