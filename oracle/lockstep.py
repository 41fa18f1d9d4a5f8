"""Lock-step checker of the on-device tree logic (test infrastructure; also the pre-flight parity check of
``bench.py``): one speculative step is launched kernel by kernel and after every kernel the integer logic of
the CPU restatement (``tree_ref``: ``mlx_eagle.py:24-376``) runs on the GPU-produced logits."""
from __future__ import annotations

import numpy as np
import torch

from . import tree_ref as tr

K = 8


def _bits(mask_rows):
    return [int(sum(1 << j for j, v in enumerate(row) if v)) for row in mask_rows]


def _u64(t):
    return [int(v) & 0xFFFFFFFFFFFFFFFF for v in t.cpu().tolist()]


def lockstep(be, base, draft, depth, T, steps, prompt_len, seed, cache_rows=512, check_kv=True):
    """Runs ``steps`` speculative steps kernel by kernel and, after each kernel, the CPU restatement's integer
    logic on the logits the GPU produced; asserts that pool, parents, masks, positions, retrieve paths, accept
    length, tokens, counters and (``check_kv``) the compacted cache rows are bit-identical.  Returns the accept
    lengths.  ``be`` is the product package (passed in: this module never imports it)."""
    _lib = be._lib
    L, p, ck = _lib.lib(), _lib.ptr, _lib.check
    dev = base.device
    rng = np.random.default_rng(seed)
    prompt = torch.from_numpy(rng.integers(0, base.args.vocab_size, prompt_len))
    dec = be.SpecDecoder(base, draft, depth, T, cache_rows=cache_rows, max_out_tokens=512, max_steps=64)
    first = dec.prefill(prompt)
    st = _lib.stream_ptr(dev)
    V = draft.args.vocab_size
    y_host, a_prev, base_len, draft_len, n_gen = [first], 0, prompt_len, prompt_len, 0
    accept_hist = []
    for step in range(steps):
        f = draft.fwd
        ck(L.b200_prep_catchup(p(dec.ctl), p(dec.y), p(f.tokens), p(f.pos), p(f.mask), p(f.prefix), p(dec.sel_row), st), "prep")
        assert f.tokens[:K].cpu().tolist() == (y_host + [0] * K)[:K]
        assert f.pos[:K].cpu().tolist() == [draft_len + m for m in range(K)]
        assert _u64(f.mask[:K]) == [(2 << m) - 1 for m in range(K)]
        assert int(f.prefix[0]) == draft_len and int(dec.sel_row) == a_prev
        logits = draft.forward_device(K, dec.draft_cache, 0, K, logits_rows=1, row_index=dec.sel_row).cpu().numpy()
        dec._expand(draft.logits[:1], 1, V, -1, st)
        # ---- root expansion (mlx_eagle.py:410-412)
        ti, tp = tr.root_expand(logits[0], K)
        off = draft_len + a_prev + 1
        assert dec.pool_tokens[:K].cpu().tolist() == ti.reshape(-1).tolist()
        assert np.array_equal(dec.pool_scores[:K].cpu().numpy(), tp.reshape(-1))
        assert int(dec.ctl[5]) == off and int(f.prefix[0]) == off
        assert f.tokens[:K].cpu().tolist() == ti.reshape(-1).tolist()
        assert f.pos[:K].cpu().tolist() == [off] * K
        pool = tr.DraftPool(ti, tp, K)
        scores, rows, out_ids = tp, None, None
        for i in range(depth):
            pool.begin_level()
            rows = tr.draft_level_mask(rows, out_ids, i, K)
            assert _u64(f.mask[:K]) == _bits(rows)
            lg = draft.forward_device(K, dec.draft_cache, K * i, K * (i + 1)).cpu().numpy()
            dec._expand(draft.logits[:K], K, V, i, st)
            nid, scores, out_ids, tki, cu, tcs = tr.process_generate_tree_iteration(lg[None], scores, K)
            pool.end_level(tki, cu, tcs)
            lo = K + K * K * i
            assert dec.pool_tokens[lo:lo + 64].cpu().tolist() == tki.reshape(-1).tolist()
            assert np.array_equal(dec.pool_scores[lo:lo + 64].cpu().numpy(), cu.reshape(-1))
            assert dec.topk_cs_index.cpu().tolist() == tcs.tolist()
            assert np.array_equal(dec.cur_scores.cpu().numpy(), scores.reshape(-1))
            assert f.tokens[:K].cpu().tolist() == nid.reshape(-1).tolist()
            assert f.pos[:K].cpu().tolist() == [off + i + 1] * K
            assert dec.pool_parents[1 + K * i: 1 + K * (i + 1)].cpu().tolist() == pool.parents_list[-1].tolist()
        # ---- finalisation (mlx_eagle.py:217-295)
        bf = base.fwd
        ck(L.b200_tree_finalize(depth, T, p(dec.pool_scores), p(dec.pool_tokens), p(dec.pool_parents), p(dec.ctl),
                                p(dec.y), p(bf.tokens), p(bf.pos), p(bf.mask), p(bf.prefix), p(dec.tree_position_ids),
                                p(dec.mask_index), p(dec.draft_tokens), p(dec.retrieve), p(dec.tree_info), st), "fin")
        tpi, mi, dt, tm = tr.process_draft_tree(pool.saved_cu_scores, pool.saved_topk_indices, pool.parents_list,
                                                y_host[-1], K, T)
        retrieve = tr.post_process_draft_tree(tpi, T, mi)
        assert dec.tree_position_ids[:T + 1].cpu().tolist() == tpi.tolist()
        assert dec.mask_index[:T].cpu().tolist() == mi.tolist()
        assert dec.draft_tokens[:T + 1].cpu().tolist() == dt[0].tolist() == bf.tokens[:T + 1].cpu().tolist()
        assert _u64(bf.mask[:T + 1]) == _bits(tm)
        assert bf.pos[:T + 1].cpu().tolist() == (tpi + base_len).tolist() and int(bf.prefix[0]) == base_len
        leaf_num, max_depth = dec.tree_info.cpu().tolist()
        assert (leaf_num, max_depth) == retrieve.shape
        got_r = dec.retrieve.cpu().numpy().reshape(-1, 9)[:leaf_num, :max_depth]
        assert np.array_equal(got_r, retrieve)
        # ---- verify, acceptance (mlx_eagle.py:311-326,582-599) and compaction (:349-376)
        blog = base.forward_device(T + 1, dec.base_cache, 0, T + 1)
        dec.base_logits = blog
        blog_h = blog.cpu().numpy()
        before = dec.base_cache.data.clone() if check_kv else None
        dec._accept()
        cand = dt[0][retrieve]
        best, a, sample = tr.evaluate_posterior_greedy(blog_h[retrieve], cand)
        idx = retrieve[best, 1:1 + a]
        acc = cand[best, 1:1 + a]
        bonus = int(tr.first_argmax(sample.astype(np.float32)))
        y_host = [int(t) for t in acc] + [bonus]
        ctl = dec.ctl.cpu().tolist()
        assert dec.accept_rows[: 1 + a].cpu().tolist() == [a] + idx.tolist()
        assert dec.y.cpu().tolist() == (y_host + [0] * K)[:K]
        assert dec.out_tokens[n_gen:n_gen + a + 1].cpu().tolist() == y_host
        n_gen += a + 1
        assert ctl[:6] == [base_len + a + 1, off, a, n_gen, step + 1, off] and ctl[7] == (best if a > 0 else 0)
        assert dec.step_log[2 * step: 2 * step + 2].cpu().tolist() == [a, best if a > 0 else 0]
        if check_kv:
            kk = [before[l, 0][None].cpu().numpy() for l in range(before.shape[0])]
            vv = [before[l, 1][None].cpu().numpy() for l in range(before.shape[0])]
            tr.accept_candidate(kk, vv, idx, a, base_len)
            after = dec.base_cache.data.cpu().numpy()
            for l in range(before.shape[0]):
                assert np.array_equal(after[l, 0], kk[l][0]) and np.array_equal(after[l, 1], vv[l][0])
        assert int(dec.argmax_key.abs().sum()) == 0 and int(dec.row_sum.abs().sum()) == 0
        base_len, draft_len, a_prev = base_len + a + 1, off, a
        accept_hist.append(a)
    return accept_hist
