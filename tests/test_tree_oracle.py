"""Tree logic of the CPU oracle against the reference's own known-answer vectors and invariants."""
import numpy as np
import pytest

from oracle import detmath, tree_ref as tr

# mlx_eagle_tests.py:97-113 (tree mask and position ids) and :80 (retrieve indices)
GOLDEN_TREE_MASK = np.array([
    [1, 0, 0, 0, 0, 0, 0, 0],
    [1, 1, 0, 0, 0, 0, 0, 0],
    [1, 1, 1, 0, 0, 0, 0, 0],
    [1, 1, 1, 1, 0, 0, 0, 0],
    [1, 1, 1, 0, 1, 0, 0, 0],
    [1, 1, 1, 1, 0, 1, 0, 0],
    [1, 1, 1, 0, 1, 0, 1, 0],
    [1, 1, 1, 1, 0, 1, 0, 1]], dtype=bool)
GOLDEN_POSITION_IDS = [0, 1, 2, 3, 3, 4, 4, 5]
GOLDEN_RETRIEVE = [[0, 1, 2, 4, 6, -1], [0, 1, 2, 3, 5, 7]]
GOLDEN_MASK_INDEX = [0, 1, 2, 2, 3, 4, 5]      # parents implied by the mask rows


def _mask_from_parents(mask_index):
    t = len(mask_index)
    m = np.eye(t + 1, dtype=bool)
    for i in range(t):
        m[i + 1] |= m[mask_index[i]]
    return m


def test_golden_mask_positions_and_paths():
    m = _mask_from_parents(GOLDEN_MASK_INDEX)
    assert np.array_equal(m, GOLDEN_TREE_MASK)
    pos = m.sum(1) - 1
    assert pos.tolist() == GOLDEN_POSITION_IDS
    r = tr.post_process_draft_tree(pos, 7, np.array(GOLDEN_MASK_INDEX))
    assert r.tolist() == GOLDEN_RETRIEVE


def test_golden_acceptance_picks_second_path_with_length_5():
    # mlx_eagle_tests.py:124-126: accept length 5, best candidate 1; the target predicts each next token of path 1
    tokens = np.array([10, 11, 12, 13, 14, 15, 16, 17])
    retrieve = np.array(GOLDEN_RETRIEVE)
    argmax = np.zeros(8, dtype=np.int64)
    path = GOLDEN_RETRIEVE[1]
    for a, b in zip(path[:-1], path[1:]):
        argmax[a] = tokens[b]
    argmax[7] = 33894
    best, a, idx, acc, bonus = tr.evaluate_posterior_from_node_argmax(argmax, tokens, retrieve)
    assert (best, a, bonus) == (1, 5, 33894)
    assert idx.tolist() == [1, 2, 3, 5, 7] and acc.tolist() == [11, 12, 13, 15, 17]


def test_posterior_from_argmax_equals_logit_version():
    rng = np.random.default_rng(0)
    for _ in range(50):
        T, V = 15, 40
        mask_index = np.array([rng.integers(0, i + 1) for i in range(T)])
        pos = _mask_from_parents(mask_index).sum(1) - 1
        retrieve = tr.post_process_draft_tree(pos, T, mask_index)
        tokens = rng.integers(0, V, T + 1)
        logits = rng.standard_normal((T + 1, V)).astype(np.float16)
        # plant an accepted chain now and then
        if rng.random() < 0.7:
            p = retrieve[rng.integers(0, len(retrieve))]
            for a, b in zip(p[:-1], p[1:]):
                if b >= 0 and rng.random() < 0.8:
                    logits[a, tokens[b]] = 50
        best, a, sample = tr.evaluate_posterior_greedy(logits[retrieve], tokens[retrieve])
        b2, a2, idx, acc, bonus = tr.evaluate_posterior_from_node_argmax(logits.argmax(-1), tokens, retrieve)
        assert (best, a) == (b2, a2) and bonus == int(sample.argmax())
        assert idx.tolist() == retrieve[best, 1:1 + a].tolist()


def test_topk_order_and_ties():
    x = np.array([1.0, 3.0, 3.0, -2.0, 3.0, 0.5], dtype=np.float32)
    idx, val = tr.topk(x, 4)
    assert idx.tolist() == [1, 2, 4, 0] and val.tolist() == [3.0, 3.0, 3.0, 1.0]
    idx2, _ = tr.topk(x, 4, stable=True)
    assert idx2.tolist() == idx.tolist()


def test_search_sorted_matches_numpy_for_present_values():
    rng = np.random.default_rng(1)
    for size in (7, 15, 23, 31):
        arr = np.sort(rng.choice(500, size, replace=False)).astype(np.uint32)
        tgt = np.concatenate([arr, [0]]).astype(np.uint32)
        got = tr.search_sorted(arr, tgt)
        assert np.array_equal(got, np.searchsorted(arr, tgt, side="left"))
        # the wrapped "parent - 1" of a root child runs off the end (for size 23 the reference probes
        # one element past the array on the way); process_draft_tree masks that entry
        assert tr.search_sorted(arr, np.array([0xFFFFFFFF], dtype=np.uint32))[0] >= size


def _random_tree(rng, depth, T, V=600, k=8):
    root = (rng.standard_normal(V) * 3).astype(np.float16)
    ti, tp = tr.root_expand(root, k)
    pool = tr.DraftPool(ti, tp, k)
    scores, rows, out_ids = tp, None, None
    for i in range(depth):
        pool.begin_level()
        rows = tr.draft_level_mask(rows, out_ids, i, k)
        logits = (rng.standard_normal((1, k, V)) * 3).astype(np.float16)
        _, scores, out_ids, tki, cu, tcs = tr.process_generate_tree_iteration(logits, scores, k)
        pool.end_level(tki, cu, tcs)
    return pool, tr.process_draft_tree(pool.saved_cu_scores, pool.saved_topk_indices, pool.parents_list, 7, k, T)


@pytest.mark.parametrize("depth,T", [(0, 7), (1, 7), (3, 15), (4, 31), (3, 23), (6, 31)])
def test_random_trees_are_well_formed(depth, T):
    rng = np.random.default_rng(depth * 100 + T)
    for _ in range(10):
        pool, (pos, mi, dt, tm) = _random_tree(rng, depth, T)
        assert dt.shape == (1, T + 1) and dt[0, 0] == 7
        assert np.all(mi < np.arange(1, T + 1))                   # parents precede children
        assert np.array_equal(tm, _mask_from_parents(mi))
        assert np.array_equal(pos, tm.sum(1) - 1) and pos.max() <= depth + 1
        assert np.all(pos[1:] == pos[mi] + 1)
        r = tr.post_process_draft_tree(pos, T, mi)
        leaves = [i for i in range(T + 1) if i not in set(mi.tolist())]
        assert r.shape == (len(leaves), pos.max() + 1)
        for row, leaf in zip(r, leaves):
            d = pos[leaf]
            assert row[d] == leaf and row[0] == 0 and np.all(row[d + 1:] == -1)
            for j in range(d, 0, -1):
                assert mi[row[j] - 1] == row[j - 1]


def test_selected_nodes_always_include_their_parent():
    # the bisection in process_draft_tree relies on it: a parent never scores below its child
    rng = np.random.default_rng(5)
    for _ in range(20):
        pool, _ = _random_tree(rng, 3, 15)
        scores = np.concatenate([s.reshape(-1) for s in pool.saved_cu_scores])
        parents = np.concatenate(pool.parents_list)
        sel, _ = tr.topk(scores, 15, stable=True)
        sel = set(sel.tolist())
        for f in sel:
            p = int(parents[f // 8])
            assert p == 0 or (p - 1) in sel


def test_draft_level_masks_follow_the_parent_rows():
    m0 = tr.draft_level_mask(None, None, 0)
    assert np.array_equal(m0, np.eye(8, dtype=bool))
    out_ids = np.array([2, 2, 0, 7, 1, 1, 1, 3])
    m1 = tr.draft_level_mask(m0, out_ids, 1)
    assert m1.shape == (8, 16)
    for r in range(8):
        assert m1[r, :8].tolist() == np.eye(8, dtype=bool)[out_ids[r]].tolist() and m1[r, 8 + r]


def test_deterministic_logsumexp_is_accurate_and_order_free():
    rng = np.random.default_rng(3)
    l = (rng.standard_normal((4, 5000)) * 4).astype(np.float16)
    lse = detmath.logsumexp(l)
    x = l.astype(np.float64)
    ref = np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1)) + x.max(-1)
    assert np.max(np.abs(lse - ref)) < 1e-9
    perm = rng.permutation(5000)
    assert np.array_equal(detmath.logsumexp(l[:, perm]), lse)           # integer sum: exact under reordering
    lp = detmath.log_probs(l)
    assert lp.dtype == np.float32 and np.all(lp <= 0)
    assert abs(float(np.exp(lp.astype(np.float64)).sum(-1)[0]) - 1.0) < 1e-5


def test_accept_candidate_moves_rows_like_an_array_assignment():
    rng = np.random.default_rng(0)
    keys = [rng.standard_normal((1, 2, 40, 8)).astype(np.float16) for _ in range(2)]
    vals = [rng.standard_normal((1, 2, 40, 8)).astype(np.float16) for _ in range(2)]
    k0 = [k.copy() for k in keys]
    new = tr.accept_candidate(keys, vals, np.array([2, 3, 7]), 3, 10)
    assert new == 14
    for k, ko in zip(keys, k0):
        assert np.array_equal(k[:, :, 11], ko[:, :, 12]) and np.array_equal(k[:, :, 12], ko[:, :, 13])
        assert np.array_equal(k[:, :, 13], ko[:, :, 17]) and np.array_equal(k[:, :, :11], ko[:, :, :11])
