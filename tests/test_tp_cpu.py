"""Host logic of the tensor-parallel target on CPU: the shards of Model.shard() tile the unsharded weights
exactly (column-parallel q|k|v, gate, up and head by rows; row-parallel o_proj, down_proj by K columns), and the
vocabulary-parallel greedy argmax over two gloo ranks equals the argmax of the whole row, ties to the lower id."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@pytest.mark.parametrize("preset,world", [("tiny-qwen2", 2)])
def test_shards_tile_the_unsharded_weights(be, preset, world):
    args = be.shape_preset(preset)
    full = be.Model.random_init(args, seed=3, device="cpu")
    shards = [full.shard(r, world) for r in range(world)]
    nq, nkv = full.nq, full.nkv
    for li, lw in enumerate(full.layers):
        for name in ("weight", "scales", "biases"):
            whole = getattr(lw["qkv"], name)
            parts = [getattr(s.layers[li]["qkv"], name) for s in shards]
            lq, lkv = nq // world, nkv // world
            assert torch.equal(torch.cat([p[:lq] for p in parts]), whole[:nq])                       # q heads
            assert torch.equal(torch.cat([p[lq:lq + lkv] for p in parts]), whole[nq:nq + nkv])        # k heads
            assert torch.equal(torch.cat([p[lq + lkv:] for p in parts]), whole[nq + nkv:])            # v heads
            for key in ("gate", "up"):                                                                # MLP rows
                assert torch.equal(torch.cat([getattr(s.layers[li][key], name) for s in shards]), getattr(lw[key], name))
            for key in ("o", "down"):                                                                 # K columns
                assert torch.equal(torch.cat([getattr(s.layers[li][key], name) for s in shards], dim=1),
                                   getattr(lw[key], name))
        if lw["qkv"].bias is not None:
            lq, lkv = nq // world, nkv // world
            b = [s.layers[li]["qkv"].bias for s in shards]
            assert torch.equal(torch.cat([x[:lq] for x in b]), lw["qkv"].bias[:nq])
        for s in shards:                                                                              # replicated
            assert s.layers[li]["input_norm"] is lw["input_norm"] and s.layers[li]["post_norm"] is lw["post_norm"]
    assert torch.equal(torch.cat([s.lm_head.weight for s in shards]), full.lm_head.weight)
    assert [s.vocab_offset for s in shards] == [r * args.vocab_size // world for r in range(world)]
    assert all(s.vocab_local == args.vocab_size // world and s.embed is full.embed for s in shards)
    assert all(s.args.num_attention_heads == args.num_attention_heads // world and
               s.args.intermediate_size == args.intermediate_size // world and s.args.head_dim == args.head_dim
               for s in shards)
    assert not shards[0].can_fuse()              # a shard fuses only once the peers' exchange buffers are mapped


def test_shard_refuses_degrees_that_do_not_divide(be):
    args = be.shape_preset("tiny-qwen2")
    full = be.Model.random_init(args, seed=3, device="cpu")
    with pytest.raises(be._lib.B200Error):
        full.shard(0, 3)


def _rank(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import b200_eagle as be
    args = be.shape_preset("tiny-qwen2")
    m = be.Model.random_init(args, seed=3, device="cpu").shard(rank, world)
    V = args.vocab_size
    g = torch.Generator().manual_seed(5)
    got = []
    for case in range(4):
        row = torch.randn(V, generator=g).half()
        if case == 1:                             # the maximum sits in both halves: the lower id wins
            row[7], row[V // 2 + 3] = 9.0, 9.0
        if case == 2:                             # ... and twice inside the upper half only
            row[V // 2 + 5], row[V - 1] = 9.0, 9.0
        want = int(torch.argmax(row.float()))     # first maximum
        mine = row[rank * (V // world):(rank + 1) * (V // world)]
        got.append((m.greedy_token(mine), want))
    if rank == 1:
        out.put(got)
    dist.barrier()
    dist.destroy_process_group()


def test_vocabulary_parallel_greedy_token_over_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    try:
        got = out.get(timeout=120)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    assert all(a == b for a, b in got), got
