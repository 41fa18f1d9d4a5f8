"""Tensor-parallel target (column/row-parallel shards, vocabulary-parallel argmax) on two GPUs, the row-parallel
partial products reduced either by NCCL between per-op kernels or inside the persistent kernel over peer
memory: greedy speculative generation must equal the committed oracle output both ways, and the two ways
must agree on the logits.  Skipped when fewer than two GPUs are visible."""
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
    prompt = torch.tensor(g["prompt"])
    assert not shard.can_fuse()
    res = be.generate_step(prompt, shard, draft, depth=3, verify_num_tokens=15, max_tokens=40, N=40, verbose=False)
    cache = shard.make_cache(128)
    per_op = shard(prompt[None], cache=cache)[0].float().cpu()
    # the same shard with the all-reduce inside the persistent kernel
    shard.tp.open_exchange(args.hidden_size)
    assert shard.can_fuse() and shard.launches_per_forward == 1
    cache = shard.make_cache(128)
    fused = shard(prompt[None], cache=cache)[0].float().cpu()
    shard.check_fused_error()
    res2 = be.generate_step(prompt, shard, draft, depth=3, verify_num_tokens=15, max_tokens=40, N=40, verbose=False)
    shard.check_fused_error()
    err = float(((fused - per_op).abs() - 2.0 ** -6 * per_op.abs()).max())      # <= 2e-2 wanted
    if rank == 0:
        out.put((res["tokens"], res["accept_lengths"], res2["tokens"], res2["accept_lengths"], err,
                 res2["decoder"].graph is not None))
    dist.barrier()
    # the reset a host does after a reported timeout leaves the group usable (no timeout is provoked here)
    shard.tp.reset_exchange()
    again = shard(prompt[None], cache=shard.make_cache(128))[0].float().cpu()
    shard.check_fused_error()
    assert torch.equal(again, fused)
    # the two-step exchange (each GPU reduces its slice of the columns and stores it to every GPU), forced on two GPUs:
    # same sums in the same rank order, so the same bits as the one-step exchange
    shard.tp.reset_exchange()
    shard.tp_two_shot = 1
    two = shard(prompt[None], cache=shard.make_cache(128))[0].float().cpu()
    shard.check_fused_error()
    assert torch.equal(two, fused)
    # ... and the one-step exchange behind the hierarchical all-GPU barrier (one remote arrival per GPU)
    shard.tp.reset_exchange()
    shard.tp_two_shot = 2
    hier = shard(prompt[None], cache=shard.make_cache(128))[0].float().cpu()
    shard.check_fused_error()
    assert torch.equal(hier, fused)
    # ... and the push form (partial products stored into every GPU's buffer, the reduce reads local memory only)
    # and the pull form (every GPU reads the peers' partial products after the barrier), each forced
    for form in (3, 4):
        shard.tp.reset_exchange()
        shard.tp_two_shot = form
        forced = shard(prompt[None], cache=shard.make_cache(128))[0].float().cpu()
        shard.check_fused_error()
        assert torch.equal(forced, fused)
    shard.tp.reset_exchange()
    shard.tp_two_shot = 0
    # a tensor-parallel DRAFT next to the tensor-parallel target: layers cut, vocabulary projection whole
    draft2 = be.Model.random_init(args, seed=12, device=dev, gen_device="cpu")
    draft2.norm.mul_(8.0)
    dshard = draft2.shard(rank, world, shard_head=False).relayout()
    dshard.tp.open_exchange(args.hidden_size)
    assert dshard.can_fuse() and dshard.vocab_local == args.vocab_size
    res3 = be.generate_step(prompt, shard, dshard, depth=3, verify_num_tokens=15, max_tokens=40, N=40, verbose=False)
    shard.check_fused_error()
    dshard.check_fused_error()
    gold = g["random_draft_d3_t15"]
    assert res3["tokens"] == gold["tokens"] and res3["accept_lengths"] == gold["accept_lengths"]
    dist.barrier()
    dshard.tp.close_exchange()
    shard.tp.close_exchange()
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
        tokens, accept, tokens2, accept2, err, graphed = out.get(timeout=200)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:                      # a rank that is stuck must not keep the test run alive
            if p.is_alive():
                p.kill()
    assert tokens == g["random_draft_d3_t15"]["tokens"]
    assert accept == g["random_draft_d3_t15"]["accept_lengths"]
    assert err <= 2e-2                       # |fused - per-op| <= 2^-6 |per-op| + 2e-2 on every logit
    assert tokens2 == g["random_draft_d3_t15"]["tokens"]
    assert accept2 == g["random_draft_d3_t15"]["accept_lengths"]
    assert graphed                           # with the exchange inside the kernels the step replays as one CUDA graph
