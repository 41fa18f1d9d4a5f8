"""The whole-pass persistent kernel (b200_forward) against the CPU oracle and against the per-op kernels."""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import eagle_ref, model_ref

pytestmark = pytest.mark.gpu
f64 = np.float64


def _close(got, want, rel, abs_):
    got, want = np.asarray(got).astype(f64), np.asarray(want).astype(f64)
    err = np.abs(got - want)
    assert np.all(err <= rel * np.abs(want) + abs_), f"max err {err.max()} (want scale {np.abs(want).max()})"


@pytest.fixture(scope="module", params=["tiny-qwen2", "tiny-llama"])
def pair(request, be, cuda):
    args = be.shape_preset(request.param)
    m = be.Model.random_init(args, seed=5, device=cuda, gen_device="cpu")
    om = model_ref.OracleModel(args, m.state_numpy())
    m.relayout()
    assert m.can_fuse() and m.launches_per_forward == 1
    return args, m, om


def test_causal_prompt_matches_oracle_logits_and_cache(pair):
    args, m, om = pair
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, args.vocab_size, 45)          # passes of 32 and 13 rows
    cache = m.make_cache(128)
    logits = m(torch.from_numpy(prompt)[None], cache=cache)[0].cpu().numpy()
    m.check_fused_error()
    oc = model_ref.make_prompt_cache(om, 128)
    want = om(prompt, oc)
    _close(logits, want, 2.0 ** -6, 2e-2)                  # stated tolerance: |d| <= 2^-6 |want| + 2e-2
    assert np.mean(logits.argmax(-1) == want.argmax(-1)) >= 0.9
    for li, c in enumerate(oc):
        _close(cache.data[li, 0, :, :45].cpu().numpy(), c.keys[0, :, :45], 2.0 ** -6, 2e-2)
        _close(cache.data[li, 1, :, :45].cpu().numpy(), c.values[0, :, :45], 2.0 ** -6, 2e-2)


def test_tree_pass_with_golden_mask_matches_oracle(be, pair):
    args, m, om = pair
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, args.vocab_size, 70)          # prefix longer than one key block
    tokens = rng.integers(0, args.vocab_size, 8)
    mask_index = np.array([0, 1, 2, 2, 3, 4, 5])           # mlx_eagle_tests.py:80
    tm = np.eye(8, dtype=bool)
    for i in range(7):
        tm[i + 1] |= tm[mask_index[i]]
    pos = tm.sum(1) - 1
    cache = m.make_cache(192)
    m(torch.from_numpy(prompt)[None], cache=cache, logits_last_only=True)
    got = be.eagle.tree_decoding(torch.from_numpy(tokens)[None], torch.from_numpy(tm), torch.from_numpy(pos), m, cache)
    m.check_fused_error()
    oc = model_ref.make_prompt_cache(om, 192)
    om(prompt, oc)
    want = eagle_ref.tree_decoding(tokens[None], tm, pos, om, oc)
    _close(got[0].cpu().numpy(), want, 2.0 ** -6, 2e-2)


def test_split_key_attention_equals_single_phase_attention(pair):
    """Short caches use one CTA per kv head walking all key blocks; long ones split the keys across CTAs
    and merge.  Forcing the split on a short cache must give the same logits within the logits tolerance."""
    args, m, _ = pair
    rng = np.random.default_rng(6)
    prompt = torch.from_numpy(rng.integers(0, args.vocab_size, 90))
    outs = []
    for split in (0, -1):
        m.attn_split_blocks = split
        cache = m.make_cache(192)
        outs.append(m(prompt[None], cache=cache)[0].float().cpu().numpy())
    m.attn_split_blocks = 0
    m.check_fused_error()
    _close(outs[0], outs[1], 2.0 ** -7, 1e-2)


def test_row_results_do_not_depend_on_the_row_count(pair):
    """One token alone and the same token as row 0 of a 16-row pass give the same logits up to the order of
    the fp32 partial sums (the K range is cut differently for 8 and for 16 rows): a few fp16 ulps, far
    below the logits tolerance.  This is what makes speculative greedy output equal plain greedy decoding."""
    args, m, _ = pair
    rng = np.random.default_rng(4)
    prompt = torch.from_numpy(rng.integers(0, args.vocab_size, 40))
    c1, c2 = m.make_cache(128), m.make_cache(128)
    m(prompt[None], cache=c1, logits_last_only=True)
    m(prompt[None], cache=c2, logits_last_only=True)
    toks = torch.from_numpy(rng.integers(0, args.vocab_size, 16))
    one = m(toks[None, :1], cache=c1)[0, 0].clone()
    many = m(toks[None], cache=c2)[0, 0].clone()
    _close(one.float().cpu().numpy(), many.float().cpu().numpy(), 2.0 ** -8, 4e-3)


SHAPES = [
    ("qwen2-0.5b", 3),      # hidden 896 (7 k-chunks), 14/2 heads of 64, tied head
    ("qwen2-7b", 2),        # hidden 3584, 28/4 heads of 128, MLP 18944
    ("llama3.2-1b", 2),     # 32/8 heads of 64
]


@pytest.mark.parametrize("plen", [300, 620])            # 5 key blocks (single-phase attention) / 10 (split keys)
@pytest.mark.parametrize("name,layers", SHAPES)
def test_fused_pass_equals_per_op_kernels_at_benchmark_shapes(be, cuda, name, layers, plen):
    """Full-width layers of the benchmark shapes (few of them): the persistent kernel against the nine
    launches per layer, same weights, same inputs; prompt passes of 32 rows, then a 16-row tree pass
    over a 300- or 620-row prefix, then a one-row pass."""
    args = dataclasses.replace(be.shape_preset(name), num_hidden_layers=layers)
    m = be.Model.random_init(args, seed=21, device=cuda).relayout()
    assert m.can_fuse()
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, args.vocab_size, (plen,), generator=g)
    tree = torch.randint(0, args.vocab_size, (16,), generator=g)
    tm = torch.tril(torch.ones(16, 16, dtype=torch.bool))
    tm[9:, 5:9] = False                                    # a branching tree: rows 9.. skip nodes 5..8
    tm |= torch.eye(16, dtype=torch.bool)
    pos = tm.sum(1) - 1
    outs = {}
    for fused in (True, False):
        m.fused = fused
        cache = m.make_cache(704)
        last = m(prompt[None], cache=cache, logits_last_only=True)[0, 0].float().cpu()
        t = be.eagle.tree_decoding(tree[None], tm, pos, m, cache)[0].float().cpu()
        cache.offset = plen
        one = m(tree[None, :1], cache=cache)[0, 0].float().cpu()
        outs[fused] = (last, t, one, cache.data[:, :, :, :plen + 16].float().cpu())
    m.fused = True
    m.check_fused_error()
    for a, b in zip(outs[True], outs[False]):
        assert torch.isfinite(a).all()
        _close(a.numpy(), b.numpy(), 2.0 ** -6, 2e-2)
    # the row-0 logits of the tree pass and the one-row pass agree up to the fp32 summation order
    # (different row counts take different work splits; through full-width layers a hidden state can move by one fp16
    # unit, which at logits of magnitude 4..8 is 3.9e-3: two such units as the absolute term)
    _close(outs[True][1][0].numpy(), outs[True][2].numpy(), 2.0 ** -8, 8e-3)


def test_forward_rejects_bad_descriptors(be, pair):
    import ctypes
    args, m, _ = pair
    cache = m.make_cache(64)
    d = m._fused_desc(8, cache, 0, 8, m.fwd, 8, None)
    lib = be._lib.lib()
    bad = be._lib.ForwardDesc.from_buffer_copy(d)
    bad.M = 33
    assert lib.b200_forward(ctypes.byref(bad), None) == -1
    bad = be._lib.ForwardDesc.from_buffer_copy(d)
    bad.tail = 4                                            # write_off + M > tail
    assert lib.b200_forward(ctypes.byref(bad), None) == -1
    bad = be._lib.ForwardDesc.from_buffer_copy(d)
    bad.workspace_bytes = 1024
    assert lib.b200_forward(ctypes.byref(bad), None) == -4
    bad = be._lib.ForwardDesc.from_buffer_copy(d)
    bad.h = d.h + 2
    assert lib.b200_forward(ctypes.byref(bad), None) == -2


def test_short_nibble_expansion_gives_the_same_bits_and_is_refused_for_out_of_range_scales(be, cuda):
    """The kernel's shorter expansion (nibble as an fp16 subnormal times scale * 2^20) must equal the long one bit
    for bit whenever it is allowed, and must not be chosen when a scale is zero, subnormal or >= 2^-4."""
    args = be.shape_preset("tiny-qwen2")
    rng = np.random.default_rng(8)
    prompt = torch.from_numpy(rng.integers(0, args.vocab_size, 29))          # one pass of the persistent kernel
    m = be.Model.random_init(args, seed=5, device=cuda, gen_device="cpu").relayout()
    outs = []
    for fast in (True, False):
        m.fast_dequant = fast
        outs.append(m(prompt[None], cache=m.make_cache(128))[0].clone())
    assert m._scales_fast is True                       # N(0, 0.02) weights: scales around 1e-2
    m.check_fused_error()
    assert torch.equal(outs[0], outs[1])
    # one zero scale, one large scale: the model must fall back to the long expansion and still match the oracle
    m2 = be.Model.random_init(args, seed=5, device=cuda, gen_device="cpu")
    m2.layers[0]["gate"].scales[3, 1] = 0.0
    m2.layers[1]["down"].scales[7, 0] = 0.125
    om = model_ref.OracleModel(args, m2.state_numpy())
    m2.relayout()
    got = m2(prompt[None], cache=m2.make_cache(128))[0].cpu().numpy()
    assert m2._scales_fast is False
    want = om(prompt.numpy(), model_ref.make_prompt_cache(om, 128))
    _close(got, want, 2.0 ** -6, 2e-2)


def test_prompt_through_the_large_m_path_matches_the_oracle_and_the_32_row_passes(pair):
    """A 300-token prompt goes through b200_qmm_umma 128 rows at a time (mlx_eagle.py:522-535): logits and every
    K/V row against the CPU oracle, and against the same prompt ingested 32 rows at a time."""
    args, m, om = pair
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, args.vocab_size, 300)
    assert m.can_prefill_large_m()
    cache = m.make_cache(384)
    logits = m(torch.from_numpy(prompt)[None], cache=cache)[0].cpu().numpy()
    assert cache.offset == 300
    oc = model_ref.make_prompt_cache(om, 384)
    want = om(prompt, oc)
    _close(logits, want, 2.0 ** -6, 2e-2)
    for li, c in enumerate(oc):
        _close(cache.data[li, 0, :, :300].cpu().numpy(), c.keys[0, :, :300], 2.0 ** -6, 2e-2)
        _close(cache.data[li, 1, :, :300].cpu().numpy(), c.values[0, :, :300], 2.0 ** -6, 2e-2)
    m.prefill_large_m = False
    try:
        cache2 = m.make_cache(384)
        small = m(torch.from_numpy(prompt)[None], cache=cache2)[0].cpu().numpy()
    finally:
        m.prefill_large_m = True
    m.check_fused_error()
    _close(logits, small, 2.0 ** -6, 2e-2)
    last = m(torch.from_numpy(prompt)[None], cache=m.make_cache(384), logits_last_only=True)[0].cpu().numpy()
    _close(last[0], want[-1], 2.0 ** -6, 2e-2)


def test_plan_hint_changes_the_work_split_not_the_result(be, pair):
    """``b200_forward_plan_hint`` (a measurement aid) moves work between K-parts, stages and split-K; the logits stay
    within the summation-order tolerance, hints that do not fit the shape are ignored, and "" restores the planner."""
    args, m, _ = pair
    lib = be._lib.lib()
    rng = np.random.default_rng(3)
    prompt = torch.from_numpy(rng.integers(0, args.vocab_size, 24))

    def run():
        m._fwd_ws = None                                     # the workspace size depends on the split
        out = m(prompt[None], cache=m.make_cache(128))[0].float().cpu().numpy()
        m.check_fused_error()
        return out

    want = run()
    try:
        lib.b200_forward_plan_hint(b"A=1:1:2,C=2:2:1,D=1:1:1,E=1:2:2,H=2:2:1")
        _close(run(), want, 2.0 ** -8, 4e-3)
        lib.b200_forward_plan_hint(b"A=8:99:99,E=3:1:1")   # infeasible values: the planner's own choice is used
        assert np.array_equal(run(), want)
    finally:
        lib.b200_forward_plan_hint(b"")
    assert np.array_equal(run(), want)


@pytest.mark.parametrize("world", [4, 8])
def test_fused_pass_equals_per_op_kernels_at_tensor_parallel_shard_shapes(be, cuda, world):
    """The layer shapes one rank of a 70B-shape target cut over 4 or 8 GPUs multiplies (hidden 8192, 64/8 heads
    and 28672 MLP rows divided by the world size, a vocabulary shard), as a whole model on one GPU with a 24-row
    tree pass: the planner's splits for these narrow, deep matrices against the per-op kernels."""
    full = be.shape_preset("llama3-70b")
    args = dataclasses.replace(full, num_hidden_layers=1, head_dim=128,
                               num_attention_heads=full.num_attention_heads // world,
                               num_key_value_heads=full.num_key_value_heads // world,
                               intermediate_size=full.intermediate_size // world,
                               vocab_size=full.vocab_size // world)
    m = be.Model.random_init(args, seed=33, device=cuda).relayout()
    assert m.can_fuse()
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, args.vocab_size, (140,), generator=g)
    tree = torch.randint(0, args.vocab_size, (24,), generator=g)
    tm = torch.tril(torch.ones(24, 24, dtype=torch.bool))
    tm[13:, 6:12] = False
    tm |= torch.eye(24, dtype=torch.bool)
    pos = tm.sum(1) - 1
    outs = {}
    for fused in (True, False):
        m.fused = fused
        cache = m.make_cache(256)
        m(prompt[None], cache=cache, logits_last_only=True)
        t = be.eagle.tree_decoding(tree[None], tm, pos, m, cache)[0].float().cpu()
        outs[fused] = (t, cache.data[:, :, :, :140 + 24].float().cpu())
    m.fused = True
    m.check_fused_error()
    for a, b in zip(outs[True], outs[False]):
        assert torch.isfinite(a).all()
        # hidden 8192 with random weights gives logits of magnitude ~10: the absolute term follows their scale
        _close(a.numpy(), b.numpy(), 2.0 ** -6, max(2e-2, 2.0 ** -8 * float(b.abs().max())))
