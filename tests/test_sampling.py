"""Sampling acceptance (temperature > 0): the CPU restatement draws from the target's distribution, and the GPU
kernels take the same decisions as the restatement bit for bit."""
import numpy as np
import pytest
import torch

from oracle import eagle_ref, model_ref, tree_ref as tr


def test_draws_are_reproducible_and_spread():
    a = [tr.rand40(7, i) for i in range(2000)]
    assert a == [tr.rand40(7, i) for i in range(2000)] and len(set(a)) == 2000
    assert all(0 <= x < (1 << 40) for x in a)
    assert abs(np.mean(a) / float(1 << 40) - 0.5) < 0.02
    assert tr.rand40(7, 0) != tr.rand40(8, 0)


def test_every_emitted_token_follows_the_target_distribution():
    """A tree with a root, two children and a grandchild: the first emitted token (accepted child or bonus) must be
    distributed as softmax(root logits / T), and, given that child 1 was accepted, the second one as softmax(node 1
    logits / T): chi-square over 20 000 streams."""
    rng = np.random.default_rng(0)
    V, temp, n = 12, 0.8, 20000
    logits = (rng.normal(size=(4, V)) * 2).astype(np.float16)
    dt, mi = np.array([0, 3, 7, 5]), np.array([0, 0, 1])
    first, second, n2 = np.zeros(V), np.zeros(V), 0
    for seed in range(n):
        acc, toks, bonus, _ = tr.evaluate_posterior_sample(logits, dt, mi, temp, seed, 0)
        seq = [int(t) for t in toks] + [bonus]
        first[seq[0]] += 1
        if len(acc) >= 1 and acc[0] == 1:
            second[seq[1]] += 1
            n2 += 1

    def chi2(cnt, row, total):
        p = np.exp(row.astype(np.float64) / temp)
        p /= p.sum()
        return float(((cnt - total * p) ** 2 / (total * p)).sum())

    assert chi2(first, logits[0], n) < 31.3                  # 99.9th percentile of chi-square with 11 degrees of freedom
    assert n2 > 200 and chi2(second, logits[1], n2) < 31.3


def test_low_temperature_reproduces_greedy_acceptance():
    rng = np.random.default_rng(1)
    logits = (rng.normal(size=(8, 50)) * 4).astype(np.float16)
    mi = np.array([0, 1, 2, 2, 3, 4, 5])                       # mlx_eagle_tests.py:80
    dt = np.zeros(8, dtype=np.int64)
    dt[1:] = rng.integers(0, 50, 7)
    am = logits.argmax(-1)
    dt[1], dt[2], dt[4] = am[0], am[1], am[2]                  # the greedy path 0-1-2-4 matches, then stops
    dt[6] = (am[4] + 1) % 50
    acc, toks, bonus, _ = tr.evaluate_posterior_sample(logits, dt, mi, 1e-3, 3, 0)
    assert acc.tolist() == [1, 2, 4] and bonus == int(am[4])


@pytest.mark.gpu
@pytest.mark.parametrize("V,T,temp", [(1000, 7, 0.7), (5000, 15, 1.0), (151936, 15, 0.9), (32064, 31, 1.6)])
def test_gpu_decisions_equal_the_restatement_on_the_same_logits(be, cuda, V, T, temp):
    """b200_tree_accept_sample against tree_ref.evaluate_posterior_sample on identical inputs: random trees, peaked
    random logits whose argmax is often a child (so that paths of every length get accepted), many seeds; accepted
    nodes, tokens, bonus token, draw counter and counters bit-identical."""
    lib, p = be._lib.lib(), be._lib.ptr
    st = be._lib.stream_ptr(cuda)
    rng = np.random.default_rng(V + T)
    ws = torch.zeros(lib.b200_tree_accept_sample_workspace_bytes(V), dtype=torch.uint8, device=cuda)
    row_max = torch.zeros(32, dtype=torch.int32, device=cuda)
    row_sum = torch.zeros(32, dtype=torch.int64, device=cuda)
    lengths = set()
    for trial in range(12):
        parents = np.array([rng.integers(0, n + 1) for n in range(T)])            # parent of node n + 1 is an earlier node
        tokens = rng.integers(0, V, T + 1)
        logits = (rng.normal(size=(T + 1, V)) * 1.5).astype(np.float16)
        for n in range(T):                                                         # make most children likely tokens
            if rng.random() < 0.8:
                logits[parents[n], tokens[n + 1]] = np.float16(5.0 + 1.2 * np.log(V) + rng.random())
        seed, draw0 = int(rng.integers(0, 2 ** 31)), int(rng.integers(0, 1000))
        ctl = torch.zeros(16, dtype=torch.int32)
        ctl[0], ctl[1], ctl[3], ctl[4], ctl[5], ctl[6], ctl[8], ctl[12], ctl[13] = 100, 90, 17, 3, 95, 64, 16, seed, draw0
        d_ctl = ctl.to(cuda)
        y = torch.zeros(8, dtype=torch.int32, device=cuda)
        rows = torch.zeros(16, dtype=torch.int32, device=cuda)
        out = torch.zeros(64, dtype=torch.int32, device=cuda)
        log = torch.zeros(32, dtype=torch.int32, device=cuda)
        d_logits = torch.from_numpy(logits).to(cuda)
        d_tok = torch.from_numpy(tokens.astype(np.int32)).to(cuda)
        d_mi = torch.from_numpy(parents.astype(np.int32)).to(cuda)
        rc = lib.b200_tree_accept_sample(T, V, p(d_logits), p(row_max), p(row_sum), p(d_tok), p(d_mi), temp, p(d_ctl), p(y),
                                         p(rows), p(out), p(log), p(ws), ws.numel(), st)
        assert rc == 0
        torch.cuda.synchronize()
        acc, toks, bonus, draw = tr.evaluate_posterior_sample(logits, tokens, parents, temp, seed, draw0)
        a = len(acc)
        lengths.add(a)
        assert int(rows[0]) == a and rows[1:1 + a].cpu().tolist() == acc.tolist()
        assert y[:a + 1].cpu().tolist() == [int(t) for t in toks] + [bonus]
        got = d_ctl.cpu().tolist()
        assert got[13] == draw and got[2] == a and got[3] == 17 + a + 1 and got[0] == 100 + a + 1 and got[4] == 4
        assert out[17:17 + a + 1].cpu().tolist() == [int(t) for t in toks] + [bonus]
        assert not row_max.any() and not row_sum.any()                            # scratch left clean
    assert max(lengths) >= 2 and len(lengths) >= 2                                # paths of different lengths occurred


@pytest.mark.gpu
def test_gpu_sampling_generation_in_lock_step_with_the_restatement(be, cuda):
    """Whole steps on the GPU; after every step's target pass the restatement's decision on the GPU's own logits and
    tree must be what the acceptance kernels then produce.  (Free-running CPU and GPU streams may part ways: a draw
    that falls within rounding noise of a boundary picks a neighbouring token; on identical logits they cannot.)"""
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=cuda, gen_device="cpu")
    base.norm.mul_(8.0)                                        # peaked distributions: children do get accepted
    draft.norm.mul_(8.0)
    base.relayout()
    draft.relayout()
    prompt = torch.from_numpy(np.random.default_rng(4).integers(0, args.vocab_size, 25))
    accepted = []
    for temp, seed, d in ((0.8, 5, draft), (1.2, 9, base)):
        dec = be.SpecDecoder(base, d, 3, 15, cache_rows=512, temperature=temp, seed=seed)
        first = dec.prefill(prompt)
        plogits = base(prompt[None].to(torch.int32), cache=base.make_cache(512), logits_last_only=True)[0, -1]
        assert first == tr.sample_token(plogits.float().cpu().numpy().astype(np.float16), temp, seed, 0)
        draw = 1                                               # the first token took draw 0
        for _ in range(12):
            dec._draft_tree()
            logits = dec._finalize_and_verify().float().cpu().numpy().astype(np.float16)
            dt = dec.draft_tokens[:16].cpu().numpy()
            mi = dec.mask_index[:15].cpu().numpy()
            acc, toks, bonus, draw = tr.evaluate_posterior_sample(logits, dt, mi, temp, seed, draw)
            dec._accept()
            a = int(dec.accept_rows[0])
            assert a == len(acc) and dec.accept_rows[1:1 + a].cpu().tolist() == acc.tolist()
            assert dec.y[:a + 1].cpu().tolist() == [int(t) for t in toks] + [bonus]
            assert int(dec.ctl[13]) == draw
            accepted.append(a)
    assert max(accepted) >= 1
    # and the public call: sampled output differs from the greedy one, two runs with one seed agree
    s1 = be.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=30, N=30, verbose=False,
                          temperature=0.9, seed=3)
    s2 = be.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=30, N=30, verbose=False,
                          temperature=0.9, seed=3)
    g = be.generate_step(prompt, base, draft, depth=3, verify_num_tokens=15, max_tokens=30, N=30, verbose=False)
    assert s1["tokens"] == s2["tokens"] and s1["tokens"] != g["tokens"]


@pytest.mark.gpu
@pytest.mark.parametrize("V", [1000, 151936])
def test_first_token_draw_equals_the_restatement(be, cuda, V):
    lib, p = be._lib.lib(), be._lib.ptr
    rng = np.random.default_rng(V)
    ws = torch.zeros(lib.b200_tree_accept_sample_workspace_bytes(V), dtype=torch.uint8, device=cuda)
    row_max = torch.zeros(32, dtype=torch.int32, device=cuda)
    row_sum = torch.zeros(32, dtype=torch.int64, device=cuda)
    tok = torch.zeros(1, dtype=torch.int32, device=cuda)
    seen = set()
    for trial in range(10):
        logits = (rng.normal(size=V) * 3).astype(np.float16)
        seed, counter, temp = int(rng.integers(0, 2 ** 31)), int(rng.integers(0, 50)), float(rng.choice([0.6, 1.0, 1.5]))
        assert lib.b200_sample_token(p(torch.from_numpy(logits).to(cuda)), V, temp, seed, counter, p(row_max), p(row_sum),
                                     p(ws), ws.numel(), p(tok), be._lib.stream_ptr(cuda)) == 0
        torch.cuda.synchronize()
        assert int(tok) == tr.sample_token(logits, temp, seed, counter)
        assert not row_max.any() and not row_sum.any()
        seen.add(int(tok))
    assert len(seen) >= 5


@pytest.mark.gpu
def test_sampling_is_refused_for_a_sharded_target_and_bad_temperatures(be, cuda):
    lib = be._lib.lib()
    z = torch.zeros(64, dtype=torch.int64, device=cuda)
    p = be._lib.ptr
    assert lib.b200_tree_accept_sample(7, 1000, p(z), p(z), p(z), p(z), p(z), 0.0, p(z), p(z), p(z), p(z), p(z), p(z), 512,
                                       be._lib.stream_ptr(cuda)) == -1
    assert lib.b200_tree_accept_sample(7, 1000, p(z), p(z), p(z), p(z), p(z), 1.0, p(z), p(z), p(z), p(z), p(z), p(z), 8,
                                       be._lib.stream_ptr(cuda)) == -4
