"""The CPU oracle of the model and the decode loop, checked against the properties the reference asserts."""
import numpy as np
import pytest
import torch

from oracle import eagle_ref, model_ref, tree_ref as tr


@pytest.fixture(scope="module")
def tiny(be):
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device="cpu")
    draft = be.Model.random_init(args, seed=12, device="cpu")
    # random-init logits are nearly flat, so cumulative scores never favour deep nodes; a larger
    # final-norm gain sharpens the distributions and lets trees grow deep
    base.norm.mul_(8.0)
    draft.norm.mul_(8.0)
    return args, model_ref.OracleModel(args, base.state_numpy()), model_ref.OracleModel(args, draft.state_numpy())


def _plain_greedy(model, prompt, n, rows=256):
    cache = model_ref.make_prompt_cache(model, rows)
    logits = model(np.asarray(prompt), cache)
    out = [int(tr.first_argmax(logits[-1].astype(np.float32)))]
    for _ in range(n - 1):
        logits = model(np.array([out[-1]]), cache)
        out.append(int(tr.first_argmax(logits[-1].astype(np.float32))))
    return out, cache


def test_array_position_rope_equals_contiguous_rope_under_permutation():
    # property asserted at mlx_arrayed_rope_kernel.py:211-236
    rng = np.random.default_rng(0)
    B, H, L, D, off = 2, 3, 17, 64, 467
    x = rng.standard_normal((B, H, L, D)).astype(np.float16)
    inv = (2.0 ** (-np.log2(1e6) * np.arange(0, D, 2) / D)).astype(np.float32)
    perm = np.stack([rng.permutation(L) for _ in range(B)])
    contiguous = model_ref.rope_positions(np.take_along_axis(x, np.argsort(perm, 1)[:, None, :, None], 2),
                                          off + np.arange(L)[None].repeat(B, 0), inv, 1.0)
    gathered = np.take_along_axis(contiguous, perm[:, None, :, None], 2)
    assert np.array_equal(model_ref.rope_positions(x, perm + off, inv, 1.0), gathered)


def test_verify_then_compaction_equals_sequential_cache(tiny):
    """mlx_eagle_tests.py:17-180 restated on a random-init model: decode a path sequentially, decode the
    same tokens as a tree, accept, and compare every K/V row of every layer."""
    args, base, _ = tiny
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, args.vocab_size, 12)
    greedy, _ = _plain_greedy(base, prompt, 7)
    van = model_ref.make_prompt_cache(base, 128)
    spec = model_ref.make_prompt_cache(base, 128)
    base(prompt, van)
    base(prompt, spec)
    # tree of the golden test: path 1 = nodes 0,1,2,3,5,7 carries the greedy continuation
    retrieve = np.array([[0, 1, 2, 4, 6, -1], [0, 1, 2, 3, 5, 7]])
    mask_index = np.array([0, 1, 2, 2, 3, 4, 5])
    tokens = np.zeros(8, dtype=np.int64)
    tokens[[0, 1, 2, 3, 5, 7]] = greedy[:6]
    tokens[[4, 6]] = [(greedy[3] + 1) % args.vocab_size, (greedy[4] + 1) % args.vocab_size]
    tm = np.eye(8, dtype=bool)
    for i in range(7):
        tm[i + 1] |= tm[mask_index[i]]
    pos = tm.sum(1) - 1
    seq_logits = base(tokens[[0, 1, 2, 3, 5, 7]], van)
    offset = spec[0].offset
    tree_logits = eagle_ref.tree_decoding(tokens[None], tm, pos, base, spec)
    best, a, sample = tr.evaluate_posterior_greedy(tree_logits[retrieve], tokens[retrieve])
    assert (best, a) == (1, 5)
    assert int(sample.argmax()) == greedy[6] == int(seq_logits[-1].argmax())
    idx = retrieve[best, 1:1 + a]
    new = tr.accept_candidate([c.keys for c in spec], [c.values for c in spec], idx, a, offset)
    assert new == van[0].offset
    for g, s in zip(van, spec):
        kd = np.abs(g.keys[:, :, :new].astype(np.float32) - s.keys[:, :, :new].astype(np.float32)).max()
        vd = np.abs(g.values[:, :, :new].astype(np.float32) - s.values[:, :, :new].astype(np.float32)).max()
        assert kd <= 2e-2 and vd <= 2e-2       # mx.allclose-level agreement (mlx_eagle_tests.py:144-170)


def test_self_draft_accepts_full_depth_and_matches_plain_greedy(tiny):
    args, base, _ = tiny
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, args.vocab_size, 10)
    res = eagle_ref.generate_step(prompt, base, base, depth=2, verify_num_tokens=7, max_tokens=16, N=8)
    plain, _ = _plain_greedy(base, prompt, len(res["tokens"]))
    agree = sum(int(a == b) for a, b in zip(res["tokens"], plain))
    assert agree >= len(plain) - 1 or res["tokens"][:8] == plain[:8]
    assert np.mean(res["accept_lengths"]) >= 2.0           # drafting with the target itself accepts deep paths


def test_random_draft_still_yields_the_targets_greedy_tokens(tiny):
    args, base, draft = tiny
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, args.vocab_size, 9)
    res = eagle_ref.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=8, N=8)
    plain, _ = _plain_greedy(base, prompt, len(res["tokens"]))
    assert res["tokens"][:6] == plain[:6]
    assert res["generated"] == sum(1 + a for a in res["accept_lengths"])


def test_stop_rules_of_the_oracle_loop(tiny):
    """End-of-sequence stop and exact clipping, as restated for the product's loop: prefixes of the free run."""
    args, base, _ = tiny
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, args.vocab_size, 10)
    free = eagle_ref.generate_step(prompt, base, base, depth=2, verify_num_tokens=7, max_tokens=16, N=8)
    clipped = eagle_ref.generate_step(prompt, base, base, depth=2, verify_num_tokens=7, max_tokens=5, N=8, clip=True)
    assert clipped["tokens"] == free["tokens"][:6] and clipped["generated"] == 5 and clipped["finish_reason"] == "length"
    eos = free["tokens"][4]
    first = free["tokens"].index(eos)
    stopped = eagle_ref.generate_step(prompt, base, base, depth=2, verify_num_tokens=7, max_tokens=16, N=8, eos_token_id=eos)
    assert stopped["tokens"] == free["tokens"][:first + 1] and stopped["finish_reason"] == "eos"
    assert stopped["generated"] == first
