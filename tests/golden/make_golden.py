"""Writes the golden fixtures of this directory.  Run from the repository root:

    python tests/golden/make_golden.py

Two kinds of vectors:
  * reference_known_answers.json - the known-answer vectors the reference's own test file holds for this
    path (mlx_eagle_tests.py:80 retrieve indices, :97-113 tree mask and position ids, :124-126 accept
    length / best candidate / bonus token), transcribed as data.  The reference (MLX / Metal) cannot be
    imported or run on Linux, so these are the only reference-side pins that exist.
  * qmm_*.npz, tree_selection.npz, generation_tiny_qwen2.json - seeded inputs with the outputs of the CPU
    oracle (oracle/), so that the CUDA path can be checked against committed numbers and the oracle
    itself cannot drift unnoticed.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import eagle_ref, model_ref, qmm_ref, tree_ref as tr   # noqa: E402


def reference_known_answers():
    d = {
        "source": "0seba/mlx-eagle-spec-decoding-tree mlx_eagle_tests.py",
        "tree_mask_rows": [[1, 0, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0, 0],
                           [1, 1, 1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 1, 0, 0, 0], [1, 1, 1, 1, 0, 1, 0, 0],
                           [1, 1, 1, 0, 1, 0, 1, 0], [1, 1, 1, 1, 0, 1, 0, 1]],      # :97-113
        "tree_position_ids": [0, 1, 2, 3, 3, 4, 4, 5],                              # :97-113
        "mask_index": [0, 1, 2, 2, 3, 4, 5],                                         # parents implied by the mask rows
        "retrieve_indices": [[0, 1, 2, 4, 6, -1], [0, 1, 2, 3, 5, 7]],               # :80
        "accept_length": 5, "best_candidate": 1, "bonus_token": 33894,               # :124-126
    }
    with open(os.path.join(HERE, "reference_known_answers.json"), "w") as f:
        json.dump(d, f, indent=1)


def qmm_cases():
    for name, (m, n, k, seed) in {"qmm_m8_n64_k256": (8, 64, 256, 1), "qmm_m16_n96_k896": (16, 96, 896, 2),
                                  "qmm_m1_n40_k128": (1, 40, 128, 3)}.items():
        rng = np.random.default_rng(seed)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        x = rng.standard_normal((m, k)).astype(np.float16)
        wq, s, b = qmm_ref.quantize(w)
        bias = (rng.standard_normal(n) * 0.02).astype(np.float16)
        y = qmm_ref.qmm(x, wq, s, b)
        yb = qmm_ref.qmm(x, wq, s, b, bias=bias)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x, wq=wq, scales=s, biases=b, bias=bias, y=y, y_bias=yb)


def tree_selection():
    """A seeded candidate pool (depth 3, 8 children per node) through process_draft_tree / post_process_draft_tree."""
    rng = np.random.default_rng(5)
    depth, T, K = 3, 15, 8
    scores = [np.sort(rng.uniform(-3, 0, (1, K)).astype(np.float32))[:, ::-1].copy()]
    tokens = [rng.integers(0, 1000, (1, K))]
    parents = [np.zeros(1, dtype=np.int64)]
    cur = scores[0].reshape(K, 1)
    for i in range(depth):
        child = np.sort(rng.uniform(-3, 0, (K, K)).astype(np.float32))[:, ::-1]
        cu = (child + cur).astype(np.float32)
        scores.append(cu.copy())
        tokens.append(rng.integers(0, 1000, (K, K)))
        best = tr.topk(cu.reshape(-1), K)[0]
        parents.append(tr.level_parents(best, i, K))
        cur = cu.reshape(-1)[best].reshape(K, 1)
    pos, mask_index, draft_tokens, tree_mask = tr.process_draft_tree(scores, tokens, parents, 7, K, T)
    retrieve = tr.post_process_draft_tree(pos, T, mask_index)
    np.savez_compressed(os.path.join(HERE, "tree_selection.npz"),
                        scores=np.concatenate([s.reshape(-1) for s in scores]),
                        tokens=np.concatenate([t.reshape(-1) for t in tokens]),
                        parents=np.concatenate([p_.reshape(-1) for p_ in parents]),
                        draft_tokens=np.asarray(draft_tokens), mask_index=np.asarray(mask_index),
                        tree_mask=np.asarray(tree_mask), tree_position_ids=np.asarray(pos), retrieve=np.asarray(retrieve))


def generation_tiny():
    """Free-running oracle generation on the seeded tiny model pair the GPU tests build (seeds 11 / 12)."""
    import torch
    import b200_eagle as be
    args = be.shape_preset("tiny-qwen2")
    out = {}
    states = []
    for seed in (11, 12):
        m = be.Model.random_init(args, seed=seed, device="cpu", gen_device="cpu")
        m.norm.mul_(8.0)
        states.append(m.state_numpy())
    prompt = np.random.default_rng(7).integers(0, args.vocab_size, 33)
    for name, draft_state, depth, T in (("random_draft_d3_t15", states[1], 3, 15), ("self_draft_d3_t15", states[0], 3, 15)):
        ref = eagle_ref.generate_step(prompt, model_ref.OracleModel(args, states[0]), model_ref.OracleModel(args, draft_state),
                                      depth=depth, verify_num_tokens=T, max_tokens=40, N=40)
        out[name] = {"tokens": [int(t) for t in ref["tokens"]], "accept_lengths": [int(a) for a in ref["accept_lengths"]]}
    out["prompt"] = [int(t) for t in prompt]
    with open(os.path.join(HERE, "generation_tiny_qwen2.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    reference_known_answers()
    qmm_cases()
    tree_selection()
    generation_tiny()
    print("golden fixtures written to", HERE)
