"""CPU restatement (numpy) of the reference's draft-tree logic, function for function.

Test infrastructure.  Follows ``mlx_eagle.py``; each function cites the lines
it restates.  Conventions fixed here because MLX's are unspecified or
unavailable:

* every top-k / argsort orders by descending value and breaks ties by ascending
  index (``mx.argpartition`` / ``mx.argsort`` tie order is MLX's, not the
  reference's);
* log-probabilities come from ``detmath.log_probs`` (fp32, reproducible bit for
  bit on a GPU); cumulative scores are fp32 sums.  The reference keeps them in
  the model dtype.
* ``-1`` entries of ``retrieve_indices`` index the LAST node, as MLX's negative
  indexing does (``mlx_eagle.py:582-589``); restated literally.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np

from . import detmath


# ----------------------------------------------------------------------------- mlx_eagle.py:24-58
def topk(x: np.ndarray, k: int, axis: int = -1, stable: bool = False):
    """Indices and values of the k largest along the last axis, sorted descending.

    Both modes of the reference (argpartition+argsort, or a full stable argsort
    of ``-x``) give the same result under the tie rule "lower index first".
    """
    assert axis in (-1, x.ndim - 1)
    order = np.argsort(-x, axis=-1, kind="stable")[..., :k]
    return order.astype(np.uint32), np.take_along_axis(x, order, axis=-1)


# ----------------------------------------------------------------------------- mlx_eagle.py:61-93
def search_sorted(arr: np.ndarray, target: np.ndarray, left: bool = True) -> np.ndarray:
    """Vectorised bisection with ceil(log2(size)) steps on uint32 values.

    ``target`` may hold 0xFFFFFFFF (the reference's ``draft_parents - 1`` underflows for root
    children, ``mlx_eagle.py:236``); such entries run off the end and are masked by the caller.
    For some sizes (23) the last step of such an entry probes ``mid == size``, one element past
    the end in the reference; the probe is clamped to the last element here.  Entries whose
    target is present in ``arr`` never probe past the end.
    """
    arr = arr.astype(np.uint32)
    target = target.astype(np.uint32)
    low = np.zeros_like(target, dtype=np.uint32)
    high = np.full(target.shape, arr.size, dtype=np.uint32)
    for _ in range(int(math.ceil(math.log2(arr.size)))):
        mid = (low + high) // 2
        mid_values = arr[np.minimum(mid, arr.size - 1)]
        if left:
            low = np.where(mid_values < target, mid + 1, low)
            high = np.where(mid_values >= target, mid, high)
        else:
            low = np.where(mid_values <= target, mid + 1, low)
            high = np.where(mid_values > target, mid, high)
    return low


# ----------------------------------------------------------------------------- mlx_eagle.py:410-412
def root_expand(logits_row: np.ndarray, k: int = 8):
    """Top-k of the raw logits of the catch-up pass, scored as ``logit - logsumexp``.

    Returns ``topk_index (1,k) uint32`` and ``topk_p (1,k,1) float32``.
    """
    logits_row = np.asarray(logits_row).reshape(1, -1)
    idx, _ = topk(logits_row.astype(np.float32), k)
    logp = detmath.log_probs(logits_row)
    return idx, np.take_along_axis(logp, idx.astype(np.int64), axis=-1)[..., None]


# ----------------------------------------------------------------------------- mlx_eagle.py:97-115
def process_generate_tree_iteration(logits: np.ndarray, current_scores: np.ndarray, k: int = 8):
    """One tree level: per-parent top-k of log-softmax, cumulative rescoring, top-k of the k*k.

    logits ``(1,k,V)``, current_scores ``(1,k,1)`` ->
    next_input_ids ``(1,k)``, next_scores ``(1,k,1)``, out_ids ``(k,)``, topk_index ``(1,k,k)``,
    cu_scores ``(1,k,k)``, topk_cs_index ``(k,)``.
    """
    logp = detmath.log_probs(logits)                              # softmax(logits).log()
    topk_index, topk_p = topk(logp, k)
    cu_scores = (topk_p + current_scores.astype(np.float32)).astype(np.float32)
    topk_cs_index, topk_cs_p = topk(cu_scores.reshape(-1), k)
    out_ids = topk_cs_index // k
    next_input_ids = topk_index.reshape(-1)[topk_cs_index][None]
    next_scores = topk_cs_p[None, :, None]
    return next_input_ids, next_scores, out_ids, topk_index, cu_scores, topk_cs_index


def level_parents(topk_cs_index: np.ndarray, i: int, k: int = 8) -> np.ndarray:
    """``parents`` of level i (``mlx_eagle.py:158-162``): flat pool index of each row's parent, plus 1."""
    bias1 = k if i > 0 else 0
    bias2 = max(0, i - 1)
    return (topk_cs_index.astype(np.uint32) + np.uint32(1 + k * k * bias2 + bias1)).astype(np.uint32)


def draft_level_mask(prev_rows: np.ndarray | None, out_ids: np.ndarray | None, i: int, k: int = 8) -> np.ndarray:
    """Visibility of the tree columns for the k queries of level i (``mlx_eagle.py:143-146,171,207``).

    Returns a bool matrix ``(k, k*(i+1))``: the rows of the previous level's mask permuted by
    ``out_ids`` (each query inherits its parent's row) with an identity block appended.  The
    committed prefix ``[:offset]`` is fully visible and not represented.
    """
    eye = np.eye(k, dtype=bool)
    if i == 0:
        return eye
    inherited = prev_rows[out_ids.astype(np.int64)]
    return np.concatenate([inherited, eye], axis=1)


# ----------------------------------------------------------------------------- mlx_eagle.py:217-250
def process_draft_tree(scores_list: Sequence[np.ndarray], ss_token: Sequence[np.ndarray],
                       parents_list: Sequence[np.ndarray], sampled_token_id: int, k: int,
                       total_tokens: int):
    """Select the ``total_tokens`` best pool nodes and derive the verify batch.

    Returns ``tree_position_ids (T+1,)``, ``mask_index (T,)``, ``draft_tokens (1,T+1)``,
    ``tree_mask (T+1,T+1) bool`` (True = visible; the reference turns it into 0/-inf).
    """
    scores = np.concatenate([np.asarray(s, dtype=np.float32).reshape(1, -1, k) for s in scores_list], axis=1).reshape(-1)
    tokens = np.concatenate([np.asarray(t).reshape(1, -1, k) for t in ss_token], axis=1).reshape(-1)
    parents = np.concatenate([np.asarray(p, dtype=np.uint32).reshape(-1) for p in parents_list], axis=0)

    top_scores_index, _ = topk(scores, total_tokens, stable=True)
    top_scores_index = np.sort(top_scores_index)

    draft_tokens = tokens[top_scores_index]
    draft_tokens = np.concatenate([np.asarray([sampled_token_id], dtype=draft_tokens.dtype), draft_tokens])

    draft_parents = parents[top_scores_index // k]
    mask_index = search_sorted(top_scores_index, draft_parents - np.uint32(1))   # uint32 wrap for roots
    mask_index = np.where(draft_parents == 0, -1, mask_index.astype(np.int64)) + 1

    tree_mask = np.eye(total_tokens + 1, dtype=bool)
    for i in range(total_tokens):
        tree_mask[i + 1] = tree_mask[i + 1] | tree_mask[mask_index[i]]

    tree_position_ids = tree_mask.sum(1) - 1
    return tree_position_ids.astype(np.int32), mask_index.astype(np.int32), draft_tokens[None], tree_mask


# ----------------------------------------------------------------------------- mlx_eagle.py:254-295
def post_process_draft_tree(tree_position_ids: np.ndarray, total_tokens: int, mask_index: np.ndarray) -> np.ndarray:
    """Root-to-leaf index paths ``(leaf_num, max_depth)`` padded with -1, leaves in ascending order."""
    max_depth = int(tree_position_ids.max()) + 1
    noleaf_index = set(int(v) for v in mask_index.tolist())
    noleaf_num = len(noleaf_index) - 1
    leaf_num = total_tokens - noleaf_num
    pos = tree_position_ids.tolist()
    mi = mask_index.tolist()
    retrieve = [[-1] * max_depth for _ in range(leaf_num)]
    rid = 0
    for i in range(total_tokens + 1):
        if i not in noleaf_index:
            cid = i
            for j in range(pos[i], -1, -1):
                retrieve[rid][j] = cid
                cid = mi[-1] if cid == 0 else mi[cid - 1]
            rid += 1
    return np.asarray(retrieve, dtype=np.int32).reshape(leaf_num, max_depth)


# ----------------------------------------------------------------------------- mlx_eagle.py:311-326
def evaluate_posterior_greedy(logits: np.ndarray, candidates: np.ndarray):
    """Longest greedily-accepted path.  logits ``(leaf, depth, V)``, candidates ``(leaf, depth)``.

    Returns ``best_candidate``, ``accept_length`` and ``logits[best, accept_length]``.
    """
    argm = first_argmax(logits[:, :-1])
    return _with_sample(logits, argm, candidates)


def first_argmax(x: np.ndarray) -> np.ndarray:
    """argmax over the last axis, first occurrence on ties (what ``mx.argmax`` returns)."""
    return np.argmax(x, axis=-1)


def _posterior_from_argmax(argm: np.ndarray, candidates: np.ndarray):
    posterior_mask = (candidates[:, 1:] == argm).astype(np.int32)
    lens = np.cumprod(posterior_mask, axis=1).sum(axis=1)
    accept_length = int(lens.max()) if lens.size else 0
    best = 0 if accept_length == 0 else int(np.argmax(lens))
    return best, accept_length


def _with_sample(logits, argm, candidates):
    best, accept_length = _posterior_from_argmax(argm, candidates)
    return best, accept_length, logits[best, accept_length]


def evaluate_posterior_from_node_argmax(node_argmax: np.ndarray, draft_tokens: np.ndarray,
                                        retrieve_indices: np.ndarray):
    """Same decision from one argmax per verify node (what the GPU path computes).

    ``node_argmax[i]`` = argmax of the target logits at node i.  Gathering with ``retrieve_indices``
    (negative entries wrap, as in ``mlx_eagle.py:582-585``) and comparing is exactly
    ``evaluate_posterior_greedy`` on the gathered logits.  Returns ``best``, ``accept_length``,
    ``accept_indices`` (``retrieve_indices[best, 1:1+a]``), ``accepted_tokens`` and the bonus token
    ``argmax(logits[best, a])``.
    """
    cand = draft_tokens.reshape(-1)[retrieve_indices]                # -1 wraps to the last node
    argm = node_argmax.reshape(-1)[retrieve_indices]
    best, a = _posterior_from_argmax(argm[:, :-1], cand)
    accept_indices = retrieve_indices[best, 1:1 + a]
    accepted_tokens = cand[best, 1:1 + a]
    bonus = int(argm[best, a])
    return best, a, accept_indices, accepted_tokens, bonus


# ----------------------------------------------------------------------------- sampling acceptance
# The reference is greedy only (README.md:9: "no sampling yet").  This is the restatement of the product's
# speculative sampling on the verify tree (include/b200_eagle.h, b200_tree_accept_sample): integer arithmetic on the
# masses e(v) = round(exp((l_v - max) / temperature) * 2^40) of detmath.exp_fixed and a counter-based generator, so
# that CPU and GPU take the same decisions.
_M64 = (1 << 64) - 1


def rand40(seed: int, counter: int) -> int:
    """40-bit draw number ``counter`` of the stream ``seed`` (splitmix64 of the pair)."""
    z = ((((seed & 0xFFFFFFFF) << 32) | (counter & 0xFFFFFFFF)) + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return z >> 24


def node_masses(logits_row: np.ndarray, temperature: float) -> np.ndarray:
    """Fixed-point masses of one row of fp16 logits at ``temperature`` (int64, 2^40 scale)."""
    from .detmath import exp_fixed
    x = np.asarray(logits_row).astype(np.float64)
    return exp_fixed((x - x.max()) / np.float64(temperature))


def sample_token(logits_row: np.ndarray, temperature: float, seed: int, counter: int) -> int:
    """One draw from softmax(logits_row / temperature): the token whose cumulative mass (token order) first exceeds
    rand40(seed, counter) * total / 2^40."""
    e = node_masses(logits_row, temperature)
    total = int(e.sum(dtype=np.int64))
    target = (rand40(seed, counter) * total) >> 40
    cum = np.cumsum(e.astype(object))
    return int(np.searchsorted(np.asarray(cum, dtype=object), target, side="right"))


def evaluate_posterior_sample(node_logits: np.ndarray, draft_tokens: np.ndarray, mask_index: np.ndarray,
                              temperature: float, seed: int, draw: int):
    """Walk the verify tree from the root: a node's children (ascending node index) are accepted with probability
    mass(token) / remaining mass of the node's row, a rejected token's mass is removed; the bonus token is drawn from
    what is left at the node where the walk stops.  ``node_logits`` ``(T+1, V)``, ``draft_tokens`` ``(T+1,)``,
    ``mask_index[n]`` = parent of node ``n + 1``.  Returns ``accept_indices`` (node indices), ``accepted_tokens``,
    ``bonus`` and the advanced draw counter."""
    dt = np.asarray(draft_tokens).reshape(-1)
    mi = np.asarray(mask_index).reshape(-1)
    T = mi.size
    cur, accepted = 0, []
    while True:
        e = node_masses(node_logits[cur], temperature)
        rem = int(e.sum(dtype=np.int64))
        removed = []
        taken = -1
        for c in range(1, T + 1):
            if int(mi[c - 1]) != cur or len(accepted) >= 7:
                continue
            x = int(dt[c])
            ex = int(e[x])
            u = rand40(seed, draw)
            draw += 1
            if u * rem < (ex << 40):
                taken = c
                break
            rem -= ex
            removed.append(x)
        if taken < 0:
            break
        accepted.append(taken)
        cur = taken
    u = rand40(seed, draw)
    draw += 1
    target = (u * rem) >> 40
    e = e.copy()
    for x in removed:
        e[x] = 0
    cum = np.cumsum(e.astype(object))                      # exact Python integers
    bonus = int(np.searchsorted(np.asarray(cum, dtype=object), target, side="right"))
    accept_indices = np.asarray(accepted, dtype=np.int64)
    return accept_indices, dt[accept_indices] if accepted else np.zeros(0, dtype=dt.dtype), bonus, draw


# ----------------------------------------------------------------------------- mlx_eagle.py:349-376
def accept_candidate(keys: List[np.ndarray], values: List[np.ndarray], accept_indices: np.ndarray,
                     accept_length: int, offset: int) -> int:
    """Move the accepted nodes' K/V rows to ``offset+1 ..`` in every layer; returns the new offset.

    ``keys[l]`` / ``values[l]`` are ``(1, Hkv, S, hd)`` arrays modified in place.  The right-hand
    side is gathered before the store, as an array assignment does.
    """
    if accept_length > 0:
        src = offset + np.asarray(accept_indices, dtype=np.int64)
        for kk, vv in zip(keys, values):
            kk[:, :, offset + 1: offset + accept_length + 1] = kk[:, :, src].copy()
            vv[:, :, offset + 1: offset + accept_length + 1] = vv[:, :, src].copy()
    return offset + accept_length + 1


# ----------------------------------------------------------------------------- pool bookkeeping
class DraftPool:
    """The lists ``generate_draft_tree`` accumulates (``mlx_eagle.py:147-150,200-201``)."""

    def __init__(self, topk_index: np.ndarray, topk_p: np.ndarray, k: int = 8):
        self.k = k
        self.saved_topk_indices = [np.asarray(topk_index).reshape(1, 1, k)]
        self.saved_cu_scores = [np.asarray(topk_p, dtype=np.float32).reshape(1, 1, k)]
        self.parents_list = [np.zeros((1,), dtype=np.uint32)]
        self.topk_cs_index = np.arange(k, dtype=np.uint32)
        self.level = 0

    def begin_level(self):
        self.parents_list.append(level_parents(self.topk_cs_index, self.level, self.k))

    def end_level(self, topk_index, cu_scores, topk_cs_index):
        self.saved_topk_indices.append(np.asarray(topk_index).reshape(1, self.k, self.k))
        self.saved_cu_scores.append(np.asarray(cu_scores, dtype=np.float32).reshape(1, self.k, self.k))
        self.topk_cs_index = np.asarray(topk_cs_index, dtype=np.uint32)
        self.level += 1
