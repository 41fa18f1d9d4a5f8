"""End-to-end generation on the GPU against the free-running CPU oracle, plus loop properties."""
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
    base.relayout()          # both models on the streaming weight layout
    draft.relayout()
    return args, base, draft, states


def _plain_greedy_gpu(model, prompt, n):
    cache = model.make_cache(256)
    logits = model(prompt[None], cache=cache, logits_last_only=True)
    out = [int(torch.argmax(logits[0, -1].float()))]
    for _ in range(n - 1):
        logits = model(torch.tensor([[out[-1]]]), cache=cache)
        out.append(int(torch.argmax(logits[0, -1].float())))
    return out


def _first_divergence(a, b):
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            return i
    return None


@pytest.mark.parametrize("self_draft,depth,T", [(False, 3, 15), (True, 3, 15), (True, 4, 31)])
def test_generation_matches_the_cpu_oracle(be, models, self_draft, depth, T):
    args, base, draft, states = models
    d = base if self_draft else draft
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, args.vocab_size, 33)
    res = be.generate_step(torch.from_numpy(prompt), base, d, depth=depth, verify_num_tokens=T, max_tokens=40, N=40,
                           verbose=False)
    ob = model_ref.OracleModel(args, states[0])
    od = ob if self_draft else model_ref.OracleModel(args, states[1])
    ref = eagle_ref.generate_step(prompt, ob, od, depth=depth, verify_num_tokens=T, max_tokens=40, N=40)
    div = _first_divergence(res["tokens"], ref["tokens"])
    # Free-running CPU and GPU differ in fp32 summation order; with the sharpened test models the
    # argmax margins are far above that noise, so the token streams and accept lengths are identical.
    assert div is None, f"first divergence at token {div}: gpu {res['tokens'][div]} vs oracle {ref['tokens'][div]}"
    assert res["accept_lengths"] == ref["accept_lengths"]
    assert res["generated"] == ref["generated"] >= 40
    dec = res["decoder"]
    assert dec.base_cache.offset == 33 + sum(1 + a for a in res["accept_lengths"][:res["steps"]]) or res["steps_launched"] > res["steps"]


def test_graph_replay_equals_eager_and_plain_greedy(be, models):
    args, base, draft, _ = models
    rng = np.random.default_rng(9)
    prompt = torch.from_numpy(rng.integers(0, args.vocab_size, 21))
    g = be.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=30, N=30, verbose=False)
    e = be.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=30, N=30, verbose=False,
                         use_graph=False)
    assert g["tokens"] == e["tokens"] and g["accept_lengths"] == e["accept_lengths"]
    plain = _plain_greedy_gpu(base, prompt, len(g["tokens"]))
    assert g["tokens"] == plain        # speculative greedy output == the target's own greedy decoding


def test_bad_configurations_are_rejected(be, models):
    _, base, draft, _ = models
    with pytest.raises(be._lib.B200Error):
        be.SpecDecoder(base, draft, depth=7, verify_num_tokens=15, cache_rows=256)
    with pytest.raises(be._lib.B200Error):
        be.SpecDecoder(base, draft, depth=0, verify_num_tokens=15, cache_rows=256)     # README: depth 0 needs T=7
    with pytest.raises(be._lib.B200Error):
        be.SpecDecoder(base, draft, depth=3, verify_num_tokens=15, cache_rows=256, k=4)


def test_eos_stop_clipping_and_final_token_match_the_oracle_loop(be, models):
    """The stop rules a serving loop needs on top of the reference's: stop at an end-of-sequence token (found on
    the device), cut to exactly max_tokens, keep the last token (``mlx_eagle.py:544-546,573,596-601``)."""
    args, base, draft, states = models
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, args.vocab_size, 33)
    ob, od = model_ref.OracleModel(args, states[0]), model_ref.OracleModel(args, states[1])
    free = eagle_ref.generate_step(prompt, ob, od, depth=3, verify_num_tokens=15, max_tokens=40, N=40)
    # an "end of sequence" that the free-running generation produces in the middle of a multi-token step
    steps_tok = []
    n = 1
    for a in free["accept_lengths"]:
        steps_tok.append(free["tokens"][n:n + a + 1])
        n += a + 1
    pick = next((st for st in steps_tok[2:] if len(st) > 1), steps_tok[3])
    eos = pick[min(1, len(pick) - 1)]
    if eos in free["tokens"][:free["tokens"].index(eos)]:
        pytest.skip("token repeats earlier")
    ref = eagle_ref.generate_step(prompt, ob, od, depth=3, verify_num_tokens=15, max_tokens=40, N=40, eos_token_id=eos)
    res = be.generate_step(torch.from_numpy(prompt), base, draft, depth=3, verify_num_tokens=15, max_tokens=40, N=40,
                           verbose=False, eos_token_id=eos)
    assert res["finish_reason"] == ref["finish_reason"] == "eos"
    assert res["tokens"] == ref["tokens"] and res["tokens"][-1] == eos and res["tokens"].count(eos) == 1
    assert res["generated"] == ref["generated"] == len(res["tokens"]) - 1
    # exact clipping: 17 tokens, not a whole number of steps
    ref = eagle_ref.generate_step(prompt, ob, od, depth=3, verify_num_tokens=15, max_tokens=17, N=40, clip=True)
    res = be.generate_step(torch.from_numpy(prompt), base, draft, depth=3, verify_num_tokens=15, max_tokens=17, N=40,
                           verbose=False, clip=True)
    assert res["tokens"] == ref["tokens"] == free["tokens"][:18] and res["generated"] == 17
    assert res["finish_reason"] == ref["finish_reason"] == "length"
    # the first token itself is the end of sequence: no step runs
    res = be.generate_step(torch.from_numpy(prompt), base, draft, depth=3, verify_num_tokens=15, max_tokens=17, N=40,
                           verbose=False, eos_token_id=free["tokens"][0])
    assert res["tokens"] == [free["tokens"][0]] and res["generated"] == 0 and res["steps_launched"] == 0


def test_step_log_does_not_overflow_when_replayed_past_its_capacity(be, models):
    """Replaying more steps than the step log holds must not write past it (the counters keep counting)."""
    args, base, draft, _ = models
    dec = be.SpecDecoder(base, draft, depth=3, verify_num_tokens=15, cache_rows=512, max_out_tokens=64, max_steps=6)
    big = torch.full((2 * 6 + 64,), -7, dtype=torch.int32, device=dec.device)
    dec.step_log = big[:12]                      # the log, followed by a canary in the same allocation
    dec.prefill(torch.arange(3, 20, dtype=torch.int32))
    dec.step_log.fill_(-7)
    for _ in range(9):
        dec.step()
    torch.cuda.synchronize()
    assert int(dec.ctl[4]) == 9                  # CTL_STEP
    assert bool((big[12:] == -7).all())          # nothing written behind the log
    assert bool((big[:12:2] >= 0).all())         # the six logged steps are there


@pytest.mark.parametrize("depth,T", [(2, 10), (1, 3), (5, 20), (0, 7)])
def test_tree_sizes_outside_the_reference_s_four_match_the_oracle(be, models, depth, T):
    """The reference's kernel restricts verify_num_tokens to 7, 15, 23, 31 (README.md:18); here any size up to 31
    and any depth up to 6 runs (the passes take any row count), and the result still equals the CPU oracle's."""
    args, base, draft, states = models
    rng = np.random.default_rng(100 + T)
    prompt = rng.integers(0, args.vocab_size, 17)
    res = be.generate_step(torch.from_numpy(prompt), base, draft, depth=depth, verify_num_tokens=T, max_tokens=24, N=24,
                           verbose=False)
    ob, od = model_ref.OracleModel(args, states[0]), model_ref.OracleModel(args, states[1])
    ref = eagle_ref.generate_step(prompt, ob, od, depth=depth, verify_num_tokens=T, max_tokens=24, N=24)
    assert res["tokens"] == ref["tokens"] and res["accept_lengths"] == ref["accept_lengths"]
