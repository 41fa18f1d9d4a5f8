"""EAGLE-2-style tree speculative decoding loop, greedy, one request per GPU.

Keeps the generate-loop API of the reference's ``mlx_eagle.py`` (``generate_step``,
``spec_step``, ``tree_decoding``, ``post_process_draft_tree``,
``evaluate_posterior_greedy``, ``accept_candidate``, the CLI flags), but one
decode step is a fixed sequence of kernel launches whose every data-dependent
quantity (cache lengths, accept length, tree shape, tokens) lives in device
memory: the host never waits for the device inside a step, and the whole step is
replayed as one CUDA graph.

Step (``mlx_eagle.py:379-463`` then ``:576-599``):
  catch-up pass of the draft on the last accepted tokens (always padded to 8 rows)
  -> root expansion -> ``depth`` draft passes of 8 tokens, each followed by one
  tree level -> selection of the ``verify_num_tokens`` best nodes, ancestor masks,
  depths, root-to-leaf paths -> one target pass on the tree -> per-node argmax ->
  longest accepted path -> KV compaction of the target cache, both cache lengths,
  next input tokens.
"""
from __future__ import annotations

import argparse
import time
from typing import List, Optional

import torch

from . import _lib
from .llama import KVCache, Model, ModelArgs, MAX_ROWS, MAX_REQUESTS, shape_preset

K = 8                      # children per node (mlx_eagle.py:750)
RETRIEVE_W = 9             # row width of the retrieve-index matrix (max depth 7 + 2)
CTL_BASE_LEN, CTL_DRAFT_LEN, CTL_ACCEPT, CTL_NGEN, CTL_STEP, CTL_DRAFT_OFF, CTL_OUT_CAP, CTL_BEST = range(8)
CTL_LOG_CAP, CTL_EOS, CTL_DONE, CTL_STOP_N, CTL_SEED, CTL_DRAW = 8, 9, 10, 11, 12, 13


class SpecDecoder:
    """Device-resident state and launch sequence of the speculative decoding loop."""

    def __init__(self, base_model: Model, draft_model: Model, depth: int, verify_num_tokens: int,
                 cache_rows: int, max_out_tokens: int = 4096, max_steps: int = 4096, k: int = K,
                 base_cache: Optional[KVCache] = None, draft_cache: Optional[KVCache] = None, req: int = 0,
                 temperature: float = 0.0, seed: int = 0):
        if k != K:
            raise _lib.B200Error("k is fixed to 8, as in the reference (mlx_eagle.py:750)")
        if not (0 <= depth <= 6):
            raise _lib.B200Error("depth must be in 0..6 (accepted tokens + 1 must fit the 8-row catch-up pass)")
        T = verify_num_tokens
        if not (1 <= T <= 31) or T > K + K * K * depth:
            raise _lib.B200Error("verify_num_tokens must be <= 31 and <= pool size (README: 7, 15, 23 or 31)")
        self.base, self.draft = base_model, draft_model
        self.depth, self.T = depth, T
        # temperature > 0: speculative sampling instead of greedy acceptance (b200_tree_accept_sample), the first
        # token drawn from the prompt's last logits (b200_sample_token); the reference is greedy only (README.md:9).
        self.temperature, self.seed = float(temperature), int(seed)
        if self.temperature > 0.0 and base_model.tp is not None:
            raise _lib.B200Error("sampling acceptance needs the whole vocabulary on one GPU (no tensor-parallel target)")
        dev = base_model.device
        self.device = dev
        # (a request of a BatchSpecDecoder gets its slabs of the shared caches and its row group ``req``)
        self.base_cache = base_cache if base_cache is not None else base_model.make_cache(cache_rows)
        self.draft_cache = draft_cache if draft_cache is not None else draft_model.make_cache(cache_rows)
        self.req = req
        i32 = dict(dtype=torch.int32, device=dev)
        i64 = dict(dtype=torch.int64, device=dev)
        pool = K + K * K * max(depth, 1)
        self.ctl = torch.zeros(16, **i32)
        self.y = torch.zeros(K, **i32)
        self.sel_row = torch.zeros(1, **i32)
        self.pool_scores = torch.zeros(pool, dtype=torch.float32, device=dev)
        self.pool_tokens = torch.zeros(pool, **i32)
        self.pool_parents = torch.zeros(64, **i32)
        self.cur_scores = torch.zeros(K, dtype=torch.float32, device=dev)
        self.topk_cs_index = torch.zeros(K, **i32)
        self.row_max = torch.zeros(MAX_ROWS, **i32)
        self.row_sum = torch.zeros(MAX_ROWS, **i64)
        nblk = _lib.lib().b200_topk_blocks(draft_model.args.vocab_size)
        self.cand = torch.zeros(K * nblk * K, **i64)
        self.argmax_key = torch.zeros(MAX_ROWS, **i64)
        self.tree_position_ids = torch.zeros(MAX_ROWS, **i32)
        self.mask_index = torch.zeros(MAX_ROWS, **i32)
        self.draft_tokens = torch.zeros(MAX_ROWS, **i32)
        self.retrieve = torch.full((MAX_ROWS * RETRIEVE_W,), -1, **i32)
        self.tree_info = torch.zeros(2, **i32)
        self.accept_rows = torch.zeros(16, **i32)
        nws = _lib.lib().b200_tree_accept_sample_workspace_bytes(base_model.args.vocab_size)
        self.sample_ws = torch.zeros(nws, dtype=torch.uint8, device=dev) if self.temperature > 0.0 else None
        self.out_tokens = torch.zeros(max_out_tokens, **i32)
        self.step_log = torch.zeros(2 * max_steps, **i32)
        self.max_steps = max_steps
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.base_logits = None
        self.kernel_launches_per_step = (
            (depth + 1) * draft_model.launches_per_forward + base_model.launches_per_forward
            + 1 + (depth + 1) * 4 + 1 + 1 + 1 + 1)
        if base_model.tp is not None:                    # argmax combine over peer memory, or two key shifts around NCCL
            self.kernel_launches_per_step += 1 if base_model.tp.peers is not None else 2

    # ------------------------------------------------------------------ prompt ingestion
    def prefill(self, prompt: torch.Tensor, prefill_step_size: int = 512, eos_token_id: Optional[int] = None) -> int:
        """Feed the prompt to both models (``mlx_eagle.py:522-535``) and take the first token greedily.
        ``eos_token_id`` arms the device-side stop test of ``b200_tree_accept`` for this request."""
        prompt = prompt.reshape(-1).to(torch.int32).to(self.device)
        n = prompt.numel()
        need = n + 8 * (self.depth + 1) + 40
        if need > self.base_cache.rows:
            raise _lib.B200Error(f"cache of {self.base_cache.rows} rows cannot hold a {n}-token prompt")
        self.base_cache.offset = 0
        self.draft_cache.offset = 0
        self.draft(prompt[None], cache=self.draft_cache, logits_last_only=True)
        logits = self.base(prompt[None], cache=self.base_cache, logits_last_only=True)
        draws = 0
        if self.temperature > 0.0:
            # sampling mode: the first token is a draw from the prompt's last logits (draw 0 of the stream)
            self.row_max.zero_()
            self.row_sum.zero_()
            tok = torch.zeros(1, dtype=torch.int32, device=self.device)
            row = logits[0, -1].contiguous()
            _lib.check(_lib.lib().b200_sample_token(
                _lib.ptr(row), self.base.args.vocab_size, self.temperature, self.seed & 0xFFFFFFFF, 0,
                _lib.ptr(self.row_max), _lib.ptr(self.row_sum), _lib.ptr(self.sample_ws), self.sample_ws.numel(),
                _lib.ptr(tok), _lib.stream_ptr(self.device)), "b200_sample_token")
            first, draws = int(tok), 1
        else:
            first = self.base.greedy_token(logits[0, -1])
        self.ctl.zero_()
        host = torch.zeros(16, dtype=torch.int32)
        host[CTL_BASE_LEN] = n
        host[CTL_DRAFT_LEN] = n
        host[CTL_OUT_CAP] = self.out_tokens.numel()
        host[CTL_LOG_CAP] = self.max_steps
        host[CTL_EOS] = 0 if eos_token_id is None else int(eos_token_id) + 1
        host[CTL_SEED] = ((self.seed + 0x80000000) % (1 << 32)) - 0x80000000       # the 32-bit pattern of the seed
        host[CTL_DRAW] = draws
        if eos_token_id is not None and first == int(eos_token_id):
            host[CTL_DONE], host[CTL_STOP_N] = 1, 0
        self.ctl.copy_(host)
        self.y.zero_()
        self.y[0] = first
        self.step_log.zero_()
        self.out_tokens.zero_()
        self.row_max.zero_()
        self.row_sum.zero_()
        self.argmax_key.zero_()
        return first

    # ------------------------------------------------------------------ one step, device only
    def _inputs(self, f, rows_per_request):
        """This request's rows of a model's forward inputs (row group ``req``) and its committed-length word."""
        o = self.req * rows_per_request
        return f.tokens[o:], f.pos[o:], f.mask[o:], f.prefix[self.req:]

    def _prep_catchup(self):
        L, p, ck = _lib.lib(), _lib.ptr, _lib.check
        tok, pos, mask, prefix = self._inputs(self.draft.fwd, K)
        ck(L.b200_prep_catchup(p(self.ctl), p(self.y), p(tok), p(pos), p(mask), p(prefix),
                               p(self.sel_row), _lib.stream_ptr(self.device)), "b200_prep_catchup")

    def _draft_tree(self):
        st = _lib.stream_ptr(self.device)
        d = self.draft
        V = d.args.vocab_size
        self._prep_catchup()
        logits = d.forward_device(K, self.draft_cache, 0, K, logits_rows=1, row_index=self.sel_row)
        self._expand(logits, 1, V, -1, st)
        for i in range(self.depth):
            logits = d.forward_device(K, self.draft_cache, K * i, K * (i + 1))
            self._expand(logits, K, V, i, st)

    def _expand(self, logits, R, V, level, st):
        L, p, ck = _lib.lib(), _lib.ptr, _lib.check
        tok, pos, mask, prefix = self._inputs(self.draft.fwd, K)
        ck(L.b200_logits_rowstats(p(logits), R, V, p(self.row_max), p(self.row_sum), st), "b200_logits_rowstats")
        ck(L.b200_logits_topk_candidates(p(logits), R, V, p(self.row_max), p(self.row_sum),
                                         0 if level < 0 else 1, p(self.cand), st), "b200_logits_topk_candidates")
        ck(L.b200_tree_expand(p(logits), V, level, p(self.cand), p(self.row_max), p(self.row_sum), p(self.ctl),
                              p(self.pool_scores), p(self.pool_tokens), p(self.pool_parents), p(self.cur_scores),
                              p(self.topk_cs_index), p(tok), p(pos), p(mask), p(prefix), st),
           "b200_tree_expand")

    def _finalize(self):
        L, p, ck = _lib.lib(), _lib.ptr, _lib.check
        st = _lib.stream_ptr(self.device)
        tok, pos, mask, prefix = self._inputs(self.base.fwd, self.T + 1)
        ck(L.b200_tree_finalize(self.depth, self.T, p(self.pool_scores), p(self.pool_tokens), p(self.pool_parents),
                                p(self.ctl), p(self.y), p(tok), p(pos), p(mask), p(prefix),
                                p(self.tree_position_ids), p(self.mask_index), p(self.draft_tokens),
                                p(self.retrieve), p(self.tree_info), st), "b200_tree_finalize")

    def _finalize_and_verify(self):
        self._finalize()
        self.base_logits = self.base.forward_device(self.T + 1, self.base_cache, 0, self.T + 1)
        return self.base_logits

    def draft_tree_step(self):
        """The draft side of a step alone (``mlx_eagle.py:400-440`` up to the selected tree): catch-up pass, root
        expansion, ``depth`` tree levels, selection of the ``verify_num_tokens`` best nodes with their masks,
        depths and root-to-leaf paths.  No target pass, nothing accepted: the decode state does not advance, so the
        call can be repeated (what the draft-only benchmark configuration times)."""
        self._draft_tree()
        self._finalize()

    def _accept(self):
        L, p, ck = _lib.lib(), _lib.ptr, _lib.check
        st = _lib.stream_ptr(self.device)
        a = self.base.args
        base = self.base
        if self.temperature > 0.0:
            ck(L.b200_tree_accept_sample(self.T, a.vocab_size, p(self.base_logits), p(self.row_max), p(self.row_sum),
                                         p(self.draft_tokens), p(self.mask_index), self.temperature, p(self.ctl), p(self.y),
                                         p(self.accept_rows), p(self.out_tokens), p(self.step_log), p(self.sample_ws),
                                         self.sample_ws.numel(), st), "b200_tree_accept_sample")
            ck(L.b200_kv_compact(p(self.base_cache.data), a.num_hidden_layers, a.num_key_value_heads,
                                 self.base_cache.rows, a.head_dim, p(self.accept_rows), p(self.ctl), st),
               "b200_kv_compact")
            return
        ck(L.b200_logits_argmax(p(self.base_logits), self.T + 1, base.vocab_local, p(self.argmax_key), st),
           "b200_logits_argmax")
        if base.tp is not None and base.tp.peers is not None:
            # vocabulary-parallel head: every shard's per-node (max, argmax) keys, combined over peer memory
            tp = base.tp
            ck(L.b200_tp_argmax_combine(p(self.argmax_key), self.T + 1, base.vocab_offset, tp.world, tp.rank,
                                        tp.peer_array, st), "b200_tp_argmax_combine")
        elif base.tp is not None:
            # ... or, without exchange buffers, by a MAX all-reduce through torch.distributed
            ck(L.b200_argmax_key_shift(p(self.argmax_key), self.T + 1, base.vocab_offset, st), "b200_argmax_key_shift")
            base.tp.all_reduce_max(self.argmax_key[: self.T + 1])
            ck(L.b200_argmax_key_shift(p(self.argmax_key), self.T + 1, 0, st), "b200_argmax_key_shift")
        ck(L.b200_tree_accept(self.T, p(self.argmax_key), p(self.draft_tokens), p(self.retrieve), p(self.tree_info),
                              p(self.ctl), p(self.y), p(self.accept_rows), p(self.out_tokens), p(self.step_log), st),
           "b200_tree_accept")
        ck(L.b200_kv_compact(p(self.base_cache.data), a.num_hidden_layers, a.num_key_value_heads,
                             self.base_cache.rows, a.head_dim, p(self.accept_rows), p(self.ctl), st),
           "b200_kv_compact")

    def step(self):
        """Launch one whole speculative step (no host synchronisation)."""
        self._draft_tree()
        self._finalize_and_verify()
        self._accept()

    def capture(self):
        """Record ``step`` into a CUDA graph (after at least one eager step, which also sets the
        kernels' shared-memory attributes).  Shapes are static; lengths are read on the device."""
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.graph = g
        return g

    def replay(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()

    def warmup(self, capture: bool = True):
        """One eager step on a dummy prompt (sets kernel attributes, sizes workspaces), then the graph
        capture.  Call once after construction; ``generate`` then only replays."""
        g = torch.Generator().manual_seed(0)
        v = min(self.base.args.vocab_size, self.draft.args.vocab_size)
        self.prefill(torch.randint(0, v, (8,), generator=g, dtype=torch.int32))
        self.step()
        if capture and (self.base.tp is None or self.base.can_fuse()):
            # (a tensor-parallel target without exchange buffers all-reduces through torch.distributed: its
            # step is launched eagerly)
            self.capture()
        torch.cuda.synchronize(self.device)

    def generate(self, prompt: torch.Tensor, max_tokens: int = 128, N: int = 20, prefill_step_size: int = 512,
                 eos_token_id: Optional[int] = None, clip: bool = False):
        """Greedy tree-speculative generation for one prompt (host or device tensor of token ids).

        Runs at most ``N`` steps and stops at the first step boundary where ``max_tokens`` were generated
        (``mlx_eagle.py:544-546``).  Steps are enqueued ahead of the host: the stop test reads a pinned
        copy of the device counters that trails the device by two steps, so the device never waits for
        the host; steps launched past the stop point are discarded from the result.

        Two stop rules the reference lacks: with ``eos_token_id`` the request ends at the first generated
        token equal to it (found on the device by ``b200_tree_accept``; the token itself is kept, everything
        after it is dropped), and ``clip=True`` cuts the result to exactly ``max_tokens`` generated tokens
        instead of a whole number of steps.  The token fed to the step that never ran (the last ``y``, which
        the reference computes but never prints, ``mlx_eagle.py:573,596-601``) is part of the result.

        Returns a dict: tokens (first token + every step's accepted tokens and bonus token),
        accept_lengths, generated, steps, steps_launched, finish_reason ("eos", "length" or "steps"),
        seconds (decode loop only, as the reference times it, ``:541``), tokens_per_second, and the byte
        counts copied between host and device.
        """
        if N + 4 > self.max_steps or max_tokens + 8 * 4 > self.out_tokens.numel():
            raise _lib.B200Error("generate: N / max_tokens exceed the decoder's log capacity")
        if prompt.numel() + max_tokens + 8 * (self.depth + 2) + self.T + 64 > self.base_cache.rows:
            raise _lib.B200Error("generate: prompt + max_tokens do not fit the KV cache")
        first = self.prefill(prompt, prefill_step_size, eos_token_id)
        torch.cuda.synchronize(self.device)
        tic = time.perf_counter()
        lead = 2
        if not hasattr(self, "_pinned"):
            self._pinned = [torch.zeros(16, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._events = [torch.cuda.Event() for _ in range(4)]
        pinned, events = self._pinned, self._events
        i = 0
        first_is_eos = eos_token_id is not None and first == int(eos_token_id)
        while i < N and not first_is_eos:
            self.replay()
            pinned[i % 4].copy_(self.ctl, non_blocking=True)
            events[i % 4].record()
            i += 1
            j = i - 1 - lead
            if j >= 0:
                events[j % 4].synchronize()
                if int(pinned[j % 4][CTL_NGEN]) >= max_tokens or int(pinned[j % 4][CTL_DONE]):
                    break
        torch.cuda.synchronize(self.device)
        total = time.perf_counter() - tic
        self.base.check_fused_error()
        self.draft.check_fused_error()
        return self._result(first, i, total, max_tokens, clip, int(prompt.numel()))

    def _result(self, first: int, steps_run: int, total: float, max_tokens: int, clip: bool, prompt_len: int):
        """The result dict of ``generate`` from the device-side logs after ``steps_run`` launched steps."""
        ctl = self.ctl.cpu().tolist()
        stop_n = ctl[CTL_STOP_N] if ctl[CTL_DONE] else None
        log = self.step_log[: 2 * steps_run].cpu().tolist()
        produced = sum(1 + log[2 * s] for s in range(steps_run))
        toks = self.out_tokens[:produced].cpu().tolist()
        n, steps, accept_lengths = 0, 0, []
        for s in range(steps_run):
            if n >= max_tokens or (stop_n is not None and n >= stop_n):
                break
            accept_lengths.append(log[2 * s])
            n += 1 + log[2 * s]
            steps += 1
        reason = "steps"
        if stop_n is not None and stop_n <= n:
            n, reason = stop_n, "eos"
        if n >= max_tokens:
            reason = "length" if not (reason == "eos" and n <= max_tokens) else "eos"
            if clip:
                n = max_tokens
        d2h = steps_run * 64 + 8 * steps_run + 4 * produced
        return dict(tokens=[first] + toks[:n], generated=n, steps=steps, steps_launched=steps_run,
                    accept_lengths=accept_lengths, mean_tokens_per_step=n / max(steps, 1), seconds=total,
                    tokens_per_second=produced / total if total > 0 else 0.0, produced=produced,
                    finish_reason=reason, h2d_bytes=prompt_len * 4, d2h_bytes=d2h)

    # ------------------------------------------------------------------ host views
    def read_ctl(self) -> List[int]:
        return self.ctl.cpu().tolist()

    def sync_offsets(self):
        c = self.read_ctl()
        self.base_cache.offset = c[CTL_BASE_LEN]
        self.draft_cache.offset = c[CTL_DRAFT_LEN]
        return c


# ---------------------------------------------------------------------- reference-style functions
class BatchSpecDecoder:
    """Several requests decoded in lock step on one GPU: every draft pass and the target pass run ONCE for all of
    them (request r owns row group r of the pass, its own slab of the KV caches and its own committed length), so
    each weight read is shared; the tree kernels, the acceptance and the compaction run per request.  The reference
    decodes one request (``mlx_eagle.py:503-606``); this is the same step for ``requests`` of them, and every request's
    tokens are what ``SpecDecoder`` produces for it alone (up to the fp32 summation order of a wider pass).

    ``requests * (verify_num_tokens + 1)`` and ``requests * 8`` rows must fit one pass (32 rows): 2 requests at 15
    verify tokens, 4 at 7."""

    def __init__(self, base_model: Model, draft_model: Model, depth: int, verify_num_tokens: int, cache_rows: int,
                 requests: int, max_out_tokens: int = 4096, max_steps: int = 4096, temperature: float = 0.0,
                 seed: int = 0):
        R, T = int(requests), verify_num_tokens
        if not (1 <= R <= MAX_REQUESTS) or R * (T + 1) > MAX_ROWS or R * K > MAX_ROWS:
            raise _lib.B200Error("requests x (verify_num_tokens + 1) rows must fit one 32-row pass")
        if not (base_model.can_fuse() and draft_model.can_fuse()) or base_model.tp is not None:
            raise _lib.B200Error("BatchSpecDecoder needs relayouted, unsharded models")
        self.base, self.draft, self.depth, self.T, self.requests = base_model, draft_model, depth, T, R
        self.device = base_model.device
        self.base_cache = base_model.make_batch_cache(cache_rows, R)
        self.draft_cache = draft_model.make_batch_cache(cache_rows, R)
        self.ctl = torch.zeros(R, 16, dtype=torch.int32, device=self.device)
        self.sel_rows = torch.zeros(R, dtype=torch.int32, device=self.device)
        self.slots: List[SpecDecoder] = []
        for r in range(R):
            # (sampling acceptance: request r draws from the stream seed + r)
            s = SpecDecoder(base_model, draft_model, depth, T, cache_rows, max_out_tokens, max_steps,
                            base_cache=self.base_cache.slabs[r], draft_cache=self.draft_cache.slabs[r], req=r,
                            temperature=temperature, seed=seed + r)
            s.ctl = self.ctl[r]                       # one device array for all requests: one read-back per step
            s.sel_row = self.sel_rows[r:r + 1]
            self.slots.append(s)
        self.max_steps = max_steps
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # the per-request kernels of a step (tree levels, selection, acceptance, compaction) touch only their own
        # request's state: they go to one side stream per request, so that the captured graph has parallel branches
        self.side = [torch.cuda.Stream(device=self.device) for _ in range(R)]
        one = self.slots[0].kernel_launches_per_step
        fwd = (depth + 1) * draft_model.launches_per_forward + base_model.launches_per_forward
        self.kernel_launches_per_step = fwd + R * (one - fwd)

    def _per_request(self, fn):
        """Run ``fn(r, slot)`` for every request, each on its own side stream, between two joins with the main
        stream (the shared passes before and after see all of them done)."""
        main = torch.cuda.current_stream(self.device)
        for r, s in enumerate(self.slots):
            self.side[r].wait_stream(main)
            with torch.cuda.stream(self.side[r]):
                fn(r, s)
        for r in range(self.requests):
            main.wait_stream(self.side[r])

    def step(self):
        """One speculative step of every request (no host synchronisation)."""
        R, T, d, b = self.requests, self.T, self.draft, self.base
        V = d.args.vocab_size
        self._per_request(lambda r, s: s._prep_catchup())
        logits = d.forward_device(K * R, self.draft_cache, 0, K, logits_rows=1, row_index=self.sel_rows, requests=R)
        self._per_request(lambda r, s: s._expand(logits[r:r + 1], 1, V, -1, _lib.stream_ptr(self.device)))
        for i in range(self.depth):
            logits = d.forward_device(K * R, self.draft_cache, K * i, K * (i + 1), requests=R)
            self._per_request(lambda r, s: s._expand(logits[r * K:(r + 1) * K], K, V, i, _lib.stream_ptr(self.device)))
        self._per_request(lambda r, s: s._finalize())
        bl = b.forward_device((T + 1) * R, self.base_cache, 0, T + 1, requests=R)

        def accept(r, s):
            s.base_logits = bl[r * (T + 1):(r + 1) * (T + 1)]
            s._accept()
        self._per_request(accept)

    def capture(self):
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.graph = g
        return g

    def replay(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()

    def prefill(self, prompts, prefill_step_size: int = 512, eos_token_id: Optional[int] = None) -> List[int]:
        """Feed every request's prompt to both models (one request at a time: prompts differ in length) and take
        their first tokens."""
        if len(prompts) != self.requests:
            raise _lib.B200Error(f"need {self.requests} prompts")
        return [s.prefill(pr, prefill_step_size, eos_token_id) for s, pr in zip(self.slots, prompts)]

    def warmup(self, capture: bool = True):
        g = torch.Generator().manual_seed(0)
        v = min(self.base.args.vocab_size, self.draft.args.vocab_size)
        self.prefill([torch.randint(0, v, (8,), generator=g, dtype=torch.int32) for _ in range(self.requests)])
        self.step()
        if capture:
            self.capture()
        torch.cuda.synchronize(self.device)

    def generate(self, prompts, max_tokens: int = 128, N: int = 20, prefill_step_size: int = 512,
                 eos_token_id: Optional[int] = None, clip: bool = False):
        """Greedy tree-speculative generation for ``requests`` prompts at once.  Steps run until every request has
        ``max_tokens`` tokens (or met ``eos_token_id``), at most ``N``; a request that finishes early keeps stepping
        with the others and its surplus is dropped.  Returns one result dict per request (as ``SpecDecoder.generate``)
        with the shared ``seconds``, plus ``"total_tokens_per_second"`` over all requests in each."""
        s0 = self.slots[0]
        longest = max(int(pr.numel()) for pr in prompts)
        if N + 4 > self.max_steps or N * (self.depth + 2) + 8 * 4 > s0.out_tokens.numel():
            raise _lib.B200Error("generate: N steps exceed the decoder's log capacity")
        if longest + N * (self.depth + 2) + 8 * (self.depth + 2) + self.T + 64 > self.base_cache.rows:
            raise _lib.B200Error("generate: prompt + N steps do not fit the KV cache")
        firsts = self.prefill(prompts, prefill_step_size, eos_token_id)
        torch.cuda.synchronize(self.device)
        tic = time.perf_counter()
        lead = 2
        if not hasattr(self, "_pinned"):
            self._pinned = [torch.zeros(self.requests, 16, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._events = [torch.cuda.Event() for _ in range(4)]
        pinned, events = self._pinned, self._events
        i = 0
        while i < N:
            self.replay()
            pinned[i % 4].copy_(self.ctl, non_blocking=True)
            events[i % 4].record()
            i += 1
            j = i - 1 - lead
            if j >= 0:
                events[j % 4].synchronize()
                c = pinned[j % 4]
                if all(int(c[r][CTL_NGEN]) >= max_tokens or int(c[r][CTL_DONE]) for r in range(self.requests)):
                    break
        torch.cuda.synchronize(self.device)
        total = time.perf_counter() - tic
        self.base.check_fused_error()
        self.draft.check_fused_error()
        out = [s._result(f, i, total, max_tokens, clip, int(pr.numel())) for s, f, pr in zip(self.slots, firsts, prompts)]
        agg = sum(o["generated"] for o in out) / total if total > 0 else 0.0
        for o in out:
            o["total_tokens_per_second"] = agg
        return out


def post_process_draft_tree(tree_position_ids: torch.Tensor, total_tokens: int, mask_index: torch.Tensor) -> torch.Tensor:
    """Root-to-leaf index paths ``(leaf_num, max_depth)``, -1 padded (``mlx_eagle.py:254-295``).

    Host-side helper for callers that hold the tree on the host; the decode loop gets the same matrix
    from ``b200_tree_finalize`` without leaving the device."""
    pos = tree_position_ids.reshape(-1).tolist()
    mi = mask_index.reshape(-1).tolist()
    max_depth = max(pos) + 1
    nonleaf = set(mi)
    leaf_num = total_tokens - (len(nonleaf) - 1)
    out = [[-1] * max_depth for _ in range(leaf_num)]
    rid = 0
    for i in range(total_tokens + 1):
        if i not in nonleaf:
            cid = i
            for j in range(pos[i], -1, -1):
                out[rid][j] = cid
                cid = mi[-1] if cid == 0 else mi[cid - 1]
            rid += 1
    return torch.tensor(out, dtype=torch.int32).reshape(leaf_num, max_depth)


def tree_decoding(token_ids: torch.Tensor, tree_mask: torch.Tensor, tree_position_ids: torch.Tensor,
                  base_model: Model, cache: KVCache) -> torch.Tensor:
    """One target pass over the tree (``mlx_eagle.py:329-346``); ``tree_mask`` is additive 0/-inf
    or boolean ``(T+1, T+1)``."""
    offset = cache.offset
    tm = tree_mask
    if tm.dtype == torch.bool:
        tm = torch.where(tm, 0.0, float("-inf"))
    tm = tm.float().cpu()
    mask = torch.cat([torch.zeros(tm.shape[0], offset), tm], dim=-1)[None, None]
    return base_model(token_ids, cache, position_ids=tree_position_ids.reshape(1, -1).cpu() + offset, mask=mask)


def evaluate_posterior_greedy(logits: torch.Tensor, candidates: torch.Tensor):
    """``mlx_eagle.py:311-326``: logits ``(leaf, depth, V)``, candidates ``(leaf, depth)``."""
    posterior_mask = (candidates[:, 1:] == torch.argmax(logits[:, :-1].float(), dim=-1)).to(torch.int32)
    lens = torch.cumprod(posterior_mask, dim=1).sum(dim=1)
    accept_length = lens.max()
    best = torch.where(accept_length == 0, torch.zeros((), dtype=torch.int64, device=lens.device), torch.argmax(lens))
    return best, accept_length, logits[best, accept_length]


def accept_candidate(cache: KVCache, accept_indices: torch.Tensor, accept_length: int, offset: int):
    """``mlx_eagle.py:349-376`` on the single-allocation cache."""
    if accept_length > 0:
        src = (offset + accept_indices.reshape(-1).to(torch.int64)).to(cache.data.device)
        rows = cache.data[:, :, :, src].clone()
        cache.data[:, :, :, offset + 1: offset + accept_length + 1] = rows
    cache.offset = offset + accept_length + 1


def spec_step(dec: SpecDecoder):
    """Device graph of one step up to the target logits, like ``mlx_eagle.py:379-463``.

    Returns ``(tree_position_ids, mask_index, draft_tokens, base_logits, base_offset, draft_offset)``
    as device tensors / device scalars (no synchronisation)."""
    dec._draft_tree()
    logits = dec._finalize_and_verify()
    T = dec.T
    return (dec.tree_position_ids[: T + 1], dec.mask_index[:T], dec.draft_tokens[None, : T + 1], logits[None],
            dec.ctl[CTL_BASE_LEN], dec.ctl[CTL_DRAFT_OFF])


def generate_step(prompt: torch.Tensor, base_model: Model, draft_model: Model, prefill_step_size: int = 512,
                  k: int = 8, depth: int = 5, verify_num_tokens: int = 31, max_tokens: int = 128, tokenizer=None,
                  N: int = 20, use_graph: bool = True, verbose: bool = True, eos_token_id: Optional[int] = None,
                  clip: bool = False, temperature: float = 0.0, seed: int = 0):
    """Greedy tree-speculative generation (``mlx_eagle.py:503-606``), same arguments as the reference
    (``verify_num_tokens`` is limited to 31 here) plus the two stop rules of ``SpecDecoder.generate``
    (``eos_token_id``, ``clip``) and, with ``temperature > 0``, sampling acceptance from the random stream ``seed``.  Builds a ``SpecDecoder`` for the request, captures
    its step graph and calls ``SpecDecoder.generate``; prints the reference's three summary lines.
    Returns the result dict of ``generate`` plus the decoder under ``"decoder"``."""
    rows = prompt.numel() + max_tokens + 8 * (depth + 2) + verify_num_tokens + 128
    rows = ((rows + 63) // 64) * 64
    dec = SpecDecoder(base_model, draft_model, depth, verify_num_tokens, rows,
                      max_out_tokens=max_tokens + 128, max_steps=N + 8, k=k, temperature=temperature, seed=seed)
    dec.warmup(capture=use_graph)
    stats = dec.generate(prompt, max_tokens=max_tokens, N=N, prefill_step_size=prefill_step_size,
                         eos_token_id=eos_token_id, clip=clip)
    if verbose:
        if tokenizer is not None:
            print(tokenizer.decode(stats["tokens"]))
        print("Generated Tokens", stats["generated"])
        print("Mean Tokens Per Step:", stats["mean_tokens_per_step"])
        print("Tokens Per Second:", round(stats["tokens_per_second"], 1))
    dec.sync_offsets()
    stats["decoder"] = dec
    return stats


def parse_args(argv=None):
    """CLI flags of ``mlx_eagle.py:620-681``; a model is a local checkpoint directory or a shape preset
    (random-init weights: nothing can be downloaded where this was written)."""
    p = argparse.ArgumentParser(description="Tree speculative decoding on B200 with seeded random-init models.")
    p.add_argument("--draft-model", type=str, default="qwen2-0.5b")
    p.add_argument("--base-model", type=str, default="qwen2-7b")
    p.add_argument("--prompt", type=str, required=True,
                   help="text (with a checkpoint that has a tokenizer), comma-separated token ids, or a number of seeded "
                        "random prompt tokens")
    p.add_argument("--depth", type=int, default=1)
    p.add_argument("--verify-num-tokens", type=int, default=15, help="7, 15, 23 or 31")
    p.add_argument("--max-tokens", type=int, default=300)
    p.add_argument("--max-generation-steps", "-N", type=int, default=300)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--eos-token-id", type=int, default=None, help="stop at the first generated token with this id")
    p.add_argument("--clip", action="store_true", help="cut the output to exactly --max-tokens tokens")
    p.add_argument("--temp", type=float, default=0.0,
                   help="0: greedy acceptance (the reference); > 0: sampling acceptance at this temperature, stream --seed")
    return p.parse_args(argv)


def main(argv=None):
    """``python -m`` entry with the reference's flags (``mlx_eagle.py:683-756``).  ``--draft-model`` / ``--base-model``
    name either a local MLX-format 4-bit checkpoint directory (``load.load``, the counterpart of ``mlx_utils.load``)
    or a shape preset with seeded random-init weights; ``--prompt`` is text (needs the checkpoint's tokenizer),
    comma-separated token ids, or a count of seeded random tokens."""
    import os
    from . import load as _load
    args = parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())

    def get(name, seed):
        if os.path.isdir(name):
            m, tok = _load.load(name, dev)
            return m.relayout(), tok
        return Model.random_init(shape_preset(name), seed, dev).relayout(), None

    draft, _ = get(args.draft_model, args.seed + 1)
    base, tokenizer = get(args.base_model, args.seed + 2)
    if args.prompt.isdigit():
        g = torch.Generator().manual_seed(args.seed)
        ids = torch.randint(0, min(draft.args.vocab_size, base.args.vocab_size), (int(args.prompt),), generator=g,
                            dtype=torch.int32)
    elif all(t.strip().lstrip("-").isdigit() for t in args.prompt.split(",")):
        ids = torch.tensor([int(t) for t in args.prompt.split(",")], dtype=torch.int32)
    elif tokenizer is not None:
        ids = torch.tensor(tokenizer.encode(args.prompt), dtype=torch.int32)
    else:
        raise SystemExit("a text prompt needs a checkpoint directory with tokenizer files as --base-model")
    eos = args.eos_token_id
    if eos is None and tokenizer is not None and getattr(tokenizer, "eos_token_id", None) is not None:
        eos = int(tokenizer.eos_token_id)
    generate_step(ids, base, draft, k=8, depth=args.depth, verify_num_tokens=args.verify_num_tokens,
                  max_tokens=args.max_tokens, prefill_step_size=512, N=args.max_generation_steps,
                  eos_token_id=eos, clip=args.clip, tokenizer=tokenizer, temperature=args.temp, seed=args.seed)


if __name__ == "__main__":
    main()
