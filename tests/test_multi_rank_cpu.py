"""The multi-GPU path of bench.py shards by request (one independent stream per rank, no data-path
collective): what crosses ranks is the reduction of the counters (tokens: sum, seconds: max).  Exercised
here with two gloo ranks on CPU."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _rank(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    produced, sec = 100.0 + 10 * rank, 1.0 + 0.5 * rank          # rank 1 is the slower stream
    p_all, s_all, e_all, es_all = bench.reduce_counters(dist, torch, world, produced, sec, 30.0 + rank, 2.0 + rank,
                                                        torch.device("cpu"))
    if rank == 0:
        out.put((p_all, s_all, e_all, es_all))
    dist.barrier()
    dist.destroy_process_group()


def test_counter_reduction_across_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res == (210.0, 1.5, 61.0, 3.0)        # tokens add up, time is the slowest rank's


def test_single_rank_reduction_is_identity():
    import bench
    assert bench.reduce_counters(None, torch, 1, 5.0, 2.0, 3.0, 1.0, torch.device("cpu")) == (5.0, 2.0, 3.0, 1.0)
