"""Committed golden fixtures (tests/golden/, written by tests/golden/make_golden.py).

CPU part: the oracle reproduces every fixture bit for bit, and agrees with the reference's own known-answer
vectors.  GPU part: the CUDA path, through the C ABI, against the same committed numbers."""
import json
import os

import numpy as np
import pytest

from oracle import qmm_ref, tree_ref as tr

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
QMM_CASES = ["qmm_m8_n64_k256", "qmm_m16_n96_k896", "qmm_m1_n40_k128"]


def _load(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def test_reference_known_answers_hold_for_the_oracle():
    ka = json.load(open(os.path.join(GOLD, "reference_known_answers.json")))
    mi = np.array(ka["mask_index"])
    mask = np.eye(len(mi) + 1, dtype=bool)
    for i, parent in enumerate(mi):
        mask[i + 1] |= mask[parent]
    assert mask.astype(int).tolist() == ka["tree_mask_rows"]
    pos = mask.sum(1) - 1
    assert pos.tolist() == ka["tree_position_ids"]
    retrieve = tr.post_process_draft_tree(pos, len(mi), mi)
    assert retrieve.tolist() == ka["retrieve_indices"]
    tokens = np.arange(10, 18)
    argmax = np.zeros(8, dtype=np.int64)
    path = ka["retrieve_indices"][ka["best_candidate"]]
    for a, b in zip(path[:-1], path[1:]):
        argmax[a] = tokens[b]
    argmax[path[-1]] = ka["bonus_token"]
    best, alen, _, _, bonus = tr.evaluate_posterior_from_node_argmax(argmax, tokens, retrieve)
    assert (best, alen, bonus) == (ka["best_candidate"], ka["accept_length"], ka["bonus_token"])


@pytest.mark.parametrize("name", QMM_CASES)
def test_oracle_reproduces_qmm_fixture(name):
    d = _load(name)
    assert np.array_equal(qmm_ref.qmm(d["x"], d["wq"], d["scales"], d["biases"]), d["y"])
    assert np.array_equal(qmm_ref.qmm(d["x"], d["wq"], d["scales"], d["biases"], bias=d["bias"]), d["y_bias"])


def test_oracle_reproduces_tree_selection_fixture():
    d = _load("tree_selection")
    K, T, depth = 8, 15, 3
    sizes = [K] + [K * K] * depth
    cuts = np.cumsum([0] + sizes)
    scores = [d["scores"][a:b].reshape(-1, K) for a, b in zip(cuts[:-1], cuts[1:])]
    tokens = [d["tokens"][a:b].reshape(-1, K) for a, b in zip(cuts[:-1], cuts[1:])]
    pcuts = np.cumsum([0, 1] + [K] * depth)
    parents = [d["parents"][a:b] for a, b in zip(pcuts[:-1], pcuts[1:])]
    pos, mi, dt, mask = tr.process_draft_tree(scores, tokens, parents, 7, K, T)
    assert np.array_equal(pos, d["tree_position_ids"]) and np.array_equal(mi, d["mask_index"])
    assert np.array_equal(dt, d["draft_tokens"]) and np.array_equal(mask, d["tree_mask"])
    assert np.array_equal(tr.post_process_draft_tree(pos, T, mi), d["retrieve"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", QMM_CASES)
def test_cuda_qmm_against_fixture(be, cuda, name):
    import torch
    d = _load(name)
    t = lambda a: torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(cuda)
    x, wq, s, b, bias = t(d["x"]), t(d["wq"]), t(d["scales"]), t(d["biases"]), t(d["bias"])
    y = be.matmul(x, wq, s, b, 64)[0].cpu().numpy().astype(np.float64)
    want = d["y"].astype(np.float64)
    # fp16 tolerance of the matmul path: |d| <= 2^-10 |want| + 2e-3 (fp32 summation order differs from numpy's)
    assert np.all(np.abs(y - want) <= 2.0 ** -10 * np.abs(want) + 2e-3)
    yb = be.matmul(x, wq, s, b, 64, bias=bias)[0].cpu().numpy().astype(np.float64)
    wantb = d["y_bias"].astype(np.float64)
    assert np.all(np.abs(yb - wantb) <= 2.0 ** -10 * np.abs(wantb) + 4e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("case,self_draft", [("random_draft_d3_t15", False), ("self_draft_d3_t15", True)])
def test_cuda_generation_against_fixture(be, cuda, case, self_draft):
    """Greedy speculative generation of the seeded tiny model pair equals the committed oracle output
    (tokens and accept lengths bit for bit) without running the oracle."""
    import torch
    g = json.load(open(os.path.join(GOLD, "generation_tiny_qwen2.json")))
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=cuda, gen_device="cpu")
    base.norm.mul_(8.0)
    draft.norm.mul_(8.0)
    base.relayout()
    draft.relayout()
    res = be.generate_step(torch.tensor(g["prompt"]), base, base if self_draft else draft, depth=3, verify_num_tokens=15,
                           max_tokens=40, N=40, verbose=False)
    assert res["tokens"] == g[case]["tokens"]
    assert res["accept_lengths"] == g[case]["accept_lengths"]
