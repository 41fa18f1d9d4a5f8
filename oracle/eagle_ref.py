"""CPU restatement of the reference's speculative decoding loop (``mlx_eagle.py``), free running.

Test infrastructure and timed CPU baseline.  ``spec_step`` follows
``mlx_eagle.py:379-463`` (including the M=1 catch-up pass when nothing was accepted and the
zero-padding to 8 rows otherwise), ``generate_draft_tree`` follows ``:118-213`` (additive mask
built and row-permuted exactly as there), ``generate_step`` follows ``:503-606``.
"""
from __future__ import annotations

import time
from typing import List

import numpy as np

from . import tree_ref as tr
from .model_ref import OracleKVCache, OracleModel, make_prompt_cache


def generate_draft_tree(topk_index, topk_p, draft_model: OracleModel, cache: List[OracleKVCache], depth=5, k=8,
                        logits_hook=None):
    offset = cache[0].offset
    current_input_ids = topk_index.reshape(-1)
    scores = topk_p
    mask = np.full((k, offset + depth * k), -np.inf, dtype=np.float32)
    mask[:, :offset] = 0
    eye = np.where(np.eye(k, dtype=bool), 0.0, -np.inf).astype(np.float32)
    pool = tr.DraftPool(topk_index, topk_p, k)
    for i in range(depth):
        pool.begin_level()
        mask[:, offset + i * k: offset + (i + 1) * k] = eye
        logits = draft_model(current_input_ids, cache, position_ids=offset + i, flat_rope=True,
                             mask=mask[:, : offset + (i + 1) * k])
        if logits_hook is not None:
            logits = logits_hook(i, logits)
        new_ids, scores, out_ids, topk_idx, cu_scores, topk_cs_index = tr.process_generate_tree_iteration(
            logits[None], scores, k)
        current_input_ids = new_ids.reshape(-1)
        pool.end_level(topk_idx, cu_scores, topk_cs_index)
        mask = mask[out_ids.astype(np.int64)]
    return pool.parents_list, pool.saved_topk_indices, pool.saved_cu_scores


def tree_decoding(token_ids, tree_mask_bool, tree_position_ids, base_model: OracleModel, cache):
    offset = cache[0].offset
    tm = np.where(tree_mask_bool, 0.0, -np.inf).astype(np.float32)
    mask = np.concatenate([np.zeros((tm.shape[0], offset), dtype=np.float32), tm], axis=-1)
    return base_model(token_ids.reshape(-1), cache, position_ids=tree_position_ids.astype(np.int64) + offset, mask=mask)


def spec_step(y, base_model, draft_model, base_cache, draft_cache, accept_length, k=8, depth=5, verify_num_tokens=15):
    base_offset = base_cache[0].offset
    draft_offset = draft_cache[0].offset + 1 + accept_length
    _y = np.asarray(y).reshape(-1)
    if accept_length > 0:
        pad_size = 8 - accept_length - 1
        yy = np.concatenate([_y, np.zeros(pad_size, dtype=_y.dtype)])
        draft_logits = draft_model(yy, draft_cache)[[accept_length]]
        for c in draft_cache:
            c.offset = draft_offset
    else:
        draft_logits = draft_model(_y, draft_cache)[[accept_length]]
    topk_index, topk_p = tr.root_expand(draft_logits[0], k)
    parents, tokens, scores = generate_draft_tree(topk_index, topk_p, draft_model, draft_cache, depth, k)
    tpi, mi, dt, tm = tr.process_draft_tree(scores, tokens, parents, int(_y[-1]), k, verify_num_tokens)
    base_logits = tree_decoding(dt, tm, tpi, base_model, base_cache)
    return tpi, mi, dt, base_logits, base_offset, draft_offset


def generate_step(prompt, base_model: OracleModel, draft_model: OracleModel, prefill_step_size=512, k=8, depth=5,
                  verify_num_tokens=15, max_tokens=128, N=20, cache_rows=None, eos_token_id=None, clip=False,
                  temperature=0.0, seed=0):
    """Returns ``dict(tokens, accept_lengths, steps, seconds, tokens_per_second)``; timer starts after
    prompt ingestion (``mlx_eagle.py:541``).  ``eos_token_id`` / ``clip`` are the two stop rules the
    product adds to the reference loop (stop after the first end-of-sequence token; cut to exactly
    ``max_tokens``), restated here so the GPU loop can be checked against them.  ``temperature > 0`` switches the
    acceptance from greedy to speculative sampling (``tree_ref.evaluate_posterior_sample``; the first token is a draw
    from the prompt's last logits, ``tree_ref.sample_token``) with the random stream ``seed``."""
    y = np.asarray(prompt).reshape(-1)
    rows = cache_rows or (y.size + max_tokens + 8 * (depth + 2) + verify_num_tokens + 128)
    base_cache = make_prompt_cache(base_model, rows)
    draft_cache = make_prompt_cache(draft_model, rows)
    while y.size > prefill_step_size:
        draft_model(y[:prefill_step_size], draft_cache)
        base_model(y[:prefill_step_size], base_cache)
        y = y[prefill_step_size:]
    draft_model(y, draft_cache)
    base_logits = base_model(y, base_cache)
    if temperature > 0.0:
        y = np.array([tr.sample_token(base_logits[-1], temperature, seed, 0)])
    else:
        y = np.array([int(tr.first_argmax(base_logits[-1].astype(np.float32)))])
    tokens = [int(y[0])]
    n, accept_length, accept_lengths = 0, 0, []
    tic = time.perf_counter()
    steps = 0
    finish = "steps"
    stop_n = 0 if (eos_token_id is not None and tokens[0] == eos_token_id) else None
    draw = 1 if temperature > 0.0 else 0                    # the first token took draw 0
    for _ in range(N):
        if n >= max_tokens or stop_n is not None:
            break
        tpi, mi, dt, logits, base_offset, draft_offset = spec_step(
            y, base_model, draft_model, base_cache, draft_cache, accept_length, k, depth, verify_num_tokens)
        if temperature > 0.0:
            accept_indices, accepted_tokens, sampled, draw = tr.evaluate_posterior_sample(
                logits, dt[0], mi, temperature, seed, draw)
            accept_length = int(accept_indices.size)
        else:
            retrieve = tr.post_process_draft_tree(tpi, verify_num_tokens, mi)
            candidates = dt[0][retrieve]
            best, accept_length, sample_p = tr.evaluate_posterior_greedy(logits[retrieve], candidates)
            accept_indices = retrieve[best, 1: 1 + accept_length]
            accepted_tokens = candidates[best, 1: 1 + accept_length]
        tr.accept_candidate([c.keys for c in base_cache], [c.values for c in base_cache], accept_indices,
                            accept_length, base_offset)
        for c in base_cache:
            c.offset = base_offset + accept_length + 1
        for c in draft_cache:
            c.offset = draft_offset
        next_token = sampled if temperature > 0.0 else int(tr.first_argmax(sample_p.astype(np.float32)))
        y = np.concatenate([accepted_tokens.astype(np.int64), [next_token]])
        tokens.extend(int(t) for t in y)
        accept_lengths.append(int(accept_length))
        if eos_token_id is not None and eos_token_id in [int(t) for t in y]:
            stop_n = n + [int(t) for t in y].index(eos_token_id) + 1
        n += 1 + accept_length
        steps += 1
    total = time.perf_counter() - tic
    if stop_n is not None:
        n, finish = stop_n, "eos"
    if n >= max_tokens:
        finish = "eos" if (finish == "eos" and n <= max_tokens) else "length"
        if clip:
            n = max_tokens
    tokens = tokens[: 1 + n]
    return dict(tokens=tokens, generated=n, finish_reason=finish, accept_lengths=accept_lengths, steps=steps, seconds=total,
                tokens_per_second=n / total if total > 0 else 0.0, base_cache=base_cache, draft_cache=draft_cache)
