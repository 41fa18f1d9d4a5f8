"""Tensor-parallel target (column/row-parallel shards, NCCL all-reduce of the row-parallel partial products,
vocabulary-parallel argmax) on two GPUs: greedy speculative generation must equal the committed oracle output.
Skipped when fewer than two GPUs are visible."""
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _rank(rank, world, port, out):
    import torch
    import torch.distributed as dist
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import b200_eagle as be
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    g = json.load(open(os.path.join(ROOT, "tests", "golden", "generation_tiny_qwen2.json")))
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=dev, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=dev, gen_device="cpu")
    base.norm.mul_(8.0)
    draft.norm.mul_(8.0)
    shard = base.shard(rank, world).relayout()
    draft.relayout()
    res = be.generate_step(torch.tensor(g["prompt"]), shard, draft, depth=3, verify_num_tokens=15, max_tokens=40, N=40,
                           verbose=False)
    if rank == 0:
        out.put((res["tokens"], res["accept_lengths"], res["decoder"].graph is not None))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_tensor_parallel_target_matches_golden_generation(cuda):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    g = json.load(open(os.path.join(ROOT, "tests", "golden", "generation_tiny_qwen2.json")))
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        tokens, accept, graphed = out.get(timeout=150)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:                      # a rank that is stuck must not keep the test run alive
            if p.is_alive():
                p.kill()
    assert tokens == g["random_draft_d3_t15"]["tokens"]
    assert accept == g["random_draft_d3_t15"]["accept_lengths"]
