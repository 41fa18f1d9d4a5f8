"""Several requests sharing every forward pass (``b200_forward`` with ``requests > 1``, ``BatchSpecDecoder``):
each request gets what it would get alone, checked against single-request passes, the single-request decoder and
the free-running CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import eagle_ref, model_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(be, cuda):
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=cuda, gen_device="cpu")
    base.norm.mul_(8.0)
    draft.norm.mul_(8.0)
    states = (base.state_numpy(), draft.state_numpy())
    base.relayout()
    draft.relayout()
    return args, base, draft, states


def _close(got, want, rel=2.0 ** -6, abs_=2e-2):
    got, want = got.float().cpu().numpy().astype(np.float64), want.float().cpu().numpy().astype(np.float64)
    err = np.abs(got - want)
    assert np.all(err <= rel * np.abs(want) + abs_), f"max err {err.max()} (scale {np.abs(want).max()})"


def _tree_inputs(model, rows, prefix, seed):
    """A plausible tree pass: row m sees the committed prefix and a random subset of the earlier rows plus itself."""
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, model.args.vocab_size, (rows,), generator=g, dtype=torch.int32)
    masks, depth = [], []
    for m in range(rows):
        bits = 1 << m
        d = 0
        for j in range(m):
            if torch.rand((), generator=g) < 0.4:
                bits |= 1 << j
                d += 1
        masks.append(bits)
        depth.append(d)
    pos = prefix + torch.tensor(depth, dtype=torch.int32)
    return tokens, pos, torch.tensor(masks, dtype=torch.int64)


@pytest.mark.parametrize("requests,rows", [(2, 16), (2, 8), (4, 8), (3, 8)])
def test_a_shared_pass_gives_every_request_the_logits_and_cache_rows_of_its_own_pass(be, cuda, models, requests, rows):
    args, base, _, _ = models
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=torch.Generator().manual_seed(100 + n), dtype=torch.int32)
               for n in (13, 29, 40, 7)[:requests]]
    batch = base.make_batch_cache(128, requests)
    alone = [base.make_cache(128) for _ in range(requests)]
    for r, pr in enumerate(prompts):
        base(pr[None], cache=batch.slabs[r], logits_last_only=True)
        base(pr[None], cache=alone[r], logits_last_only=True)
        assert torch.equal(batch.slabs[r].data, alone[r].data)
    f = base.fwd
    want = []
    ins = [_tree_inputs(base, rows, int(pr.numel()), 7 + r) for r, pr in enumerate(prompts)]
    for r, (tok, pos, mask) in enumerate(ins):
        f.tokens[:rows].copy_(tok); f.pos[:rows].copy_(pos); f.mask[:rows].copy_(mask)
        f.prefix.fill_(int(prompts[r].numel()))
        want.append(base.forward_device(rows, alone[r], 0, rows).clone())
    for r, (tok, pos, mask) in enumerate(ins):
        f.tokens[r * rows:(r + 1) * rows].copy_(tok)
        f.pos[r * rows:(r + 1) * rows].copy_(pos)
        f.mask[r * rows:(r + 1) * rows].copy_(mask)
        f.prefix[r] = int(prompts[r].numel())
    got = base.forward_device(rows * requests, batch, 0, rows, requests=requests).clone()
    torch.cuda.synchronize()
    base.check_fused_error()
    assert got.shape == (requests * rows, args.vocab_size)
    for r in range(requests):
        _close(got[r * rows:(r + 1) * rows], want[r])
        n = int(prompts[r].numel())
        _close(batch.slabs[r].data[:, :, :, n:n + rows], alone[r].data[:, :, :, n:n + rows])
        assert torch.equal(batch.slabs[r].data[:, :, :, :n], alone[r].data[:, :, :, :n])        # committed rows untouched


def test_selected_head_rows_per_request(be, cuda, models):
    args, base, _, _ = models
    R, rows = 2, 8
    batch = base.make_batch_cache(128, R)
    prompts = [torch.arange(3, 3 + n, dtype=torch.int32) for n in (9, 17)]
    for r, pr in enumerate(prompts):
        base(pr[None], cache=batch.slabs[r], logits_last_only=True)
    f = base.fwd
    for r, pr in enumerate(prompts):
        tok, pos, mask = _tree_inputs(base, rows, int(pr.numel()), 50 + r)
        f.tokens[r * rows:(r + 1) * rows].copy_(tok)
        f.pos[r * rows:(r + 1) * rows].copy_(pos)
        f.mask[r * rows:(r + 1) * rows].copy_(mask)
        f.prefix[r] = int(pr.numel())
    full = base.forward_device(rows * R, batch, 0, rows, requests=R).clone()
    sel = torch.tensor([5, 2], dtype=torch.int32, device=cuda)
    one = base.forward_device(rows * R, batch, 0, rows, logits_rows=1, row_index=sel, requests=R).clone()
    assert one.shape == (R, args.vocab_size)
    assert torch.equal(one[0], full[5]) and torch.equal(one[1], full[rows + 2])


def test_two_requests_decode_like_each_alone_and_like_the_oracle(be, cuda, models):
    args, base, draft, states = models
    rng = np.random.default_rng(21)
    prompts = [torch.from_numpy(rng.integers(0, args.vocab_size, n)) for n in (33, 19)]
    dec = be.BatchSpecDecoder(base, draft, depth=3, verify_num_tokens=15, cache_rows=512, requests=2,
                              max_out_tokens=512, max_steps=128)
    dec.warmup()
    res = dec.generate(prompts, max_tokens=40, N=60)
    ob, od = model_ref.OracleModel(args, states[0]), model_ref.OracleModel(args, states[1])
    for r, pr in enumerate(prompts):
        single = be.generate_step(pr, base, draft, depth=3, verify_num_tokens=15, max_tokens=40, N=60, verbose=False)
        ref = eagle_ref.generate_step(pr.numpy(), ob, od, depth=3, verify_num_tokens=15, max_tokens=40, N=60)
        assert res[r]["tokens"] == single["tokens"] == ref["tokens"]
        assert res[r]["accept_lengths"] == single["accept_lengths"] == ref["accept_lengths"]
        assert res[r]["generated"] >= 40


def test_four_self_draft_requests_accept_whole_paths(be, cuda, models):
    """Draft = target: every step accepts depth + 1 tokens, so compaction and catch-up run on every request with
    different committed lengths."""
    args, base, _, states = models
    rng = np.random.default_rng(5)
    prompts = [torch.from_numpy(rng.integers(0, args.vocab_size, n)) for n in (11, 25, 8, 31)]
    dec = be.BatchSpecDecoder(base, base, depth=3, verify_num_tokens=7, cache_rows=512, requests=4,
                              max_out_tokens=512, max_steps=128)
    dec.warmup()
    res = dec.generate(prompts, max_tokens=30, N=40, clip=True)
    ob = model_ref.OracleModel(args, states[0])
    for r, pr in enumerate(prompts):
        ref = eagle_ref.generate_step(pr.numpy(), ob, ob, depth=3, verify_num_tokens=7, max_tokens=30, N=40, clip=True)
        assert res[r]["tokens"] == ref["tokens"]
        assert res[r]["accept_lengths"][:len(ref["accept_lengths"])] == ref["accept_lengths"]
        assert max(res[r]["accept_lengths"]) >= 3


def test_bad_batch_shapes_are_rejected(be, cuda, models):
    _, base, draft, _ = models
    with pytest.raises(be._lib.B200Error):
        be.BatchSpecDecoder(base, draft, depth=3, verify_num_tokens=23, cache_rows=512, requests=2)     # 48 rows
    with pytest.raises(be._lib.B200Error):
        base.forward_device(16, base.make_cache(128), 0, 8, requests=2)                                # not a batch cache
    long_cache = base.make_batch_cache(4096, 2)                                                       # single-phase attention only
    with pytest.raises(be._lib.B200Error):
        base.forward_device(16, long_cache, 0, 8, requests=2)


def test_batched_sampling_is_reproducible_per_seed(be, cuda, models):
    args, base, draft, _ = models
    rng = np.random.default_rng(8)
    prompts = [torch.from_numpy(rng.integers(0, args.vocab_size, n)) for n in (14, 22)]
    outs = []
    for seed in (3, 3, 4):
        dec = be.BatchSpecDecoder(base, draft, depth=3, verify_num_tokens=15, cache_rows=512, requests=2,
                                  max_out_tokens=512, max_steps=128, temperature=0.9, seed=seed)
        dec.warmup()
        outs.append([r["tokens"] for r in dec.generate(prompts, max_tokens=24, N=40)])
    assert outs[0] == outs[1] and outs[0] != outs[2]
    assert all(len(t) >= 25 for t in outs[0])
