"""Benchmark of the tree speculative decoding hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c3|c2|c4|tp70b|tp7b]

Default workload ``c3`` (N = 1 and every rank at N > 1): full speculative decode steps, greedy, Qwen2-7B-shape
4-bit target + Qwen2-0.5B-shape 4-bit draft (random-init weights, seeded), 256-token seeded random prompt,
depth 3, 15 verify tokens; one "step" is one speculative step (draft catch-up pass, 3 draft tree passes, tree
finalisation, one target pass on 16 tokens, acceptance, KV compaction).  Metric: accepted tokens per second
(tokens produced by the timed steps / device time).  The block of K steps is repeated from the same decode
state until at least two seconds have been timed; the median block gives ``value``, the spread is reported.

The JSON line also carries: the end-to-end number through ``SpecDecoder.generate`` with a pinned host prompt
(``e2e``), the roofline of the target pass (``roofline``: the persistent forward kernel at 16 rows) and of the
draft pass (``roofline_draft``: the same kernel on the draft at 8 rows), the quantised-matmul operator sweep of
the metric's second half (``qmm_sweep``: 8192 x 2048 at 1..32 rows, GB/s against the HBM peak), a lock-step
parity check of the very models that are timed (``config.parity_checked``) and a CPU baseline (the CPU
restatement of the reference's path on a bounded sample on this host's cores).  At N > 1 the ranks afterwards
run the tensor-parallel workload ``tp70b`` for a few steps and attach its numbers under
``config.tensor_parallel``.  At N = 1 two more attachments: ``config.batched_requests`` (the same step for as many
requests as fit one 32-row pass, all passes shared) and ``config.accept_length_sensitivity`` (the step time at accept
length 0 and above: random-init pairs accept nothing, so the headline counts one token per step).

Other workloads: ``c2`` draft-only tree build (0.5B-shape draft, prompt 128, depth 3, 7 nodes), ``c4``
Llama-3-8B-shape target + Llama-3.2-1B-shape draft (prompt 1024, depth 4, 31 verify tokens, also reports the
time to the first token of the 1024-token prompt), ``tp70b`` / ``tp7b`` one stream with the target cut across
all ranks.  ``--impl reference`` times the CPU restatement only (the reference itself is MLX/Metal and cannot
run on Linux), on the same configuration, and prints the same line with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

UNIT = "tokens/s"
# name -> (target preset, draft preset, prompt tokens, depth, verify tokens, metric)
STREAM_WORKLOADS = {
    "c3": ("qwen2-7b", "qwen2-0.5b", 256, 3, 15,
           "accepted tokens/s (7B-shape 4-bit target + 0.5B draft, 15-node tree)"),
    "c4": ("llama3-8b", "llama3.2-1b", 1024, 4, 31,
           "accepted tokens/s (Llama-3-8B-shape 4-bit target + 3.2-1B-shape draft, 31-node tree, prompt 1024)"),
    "c2": (None, "qwen2-0.5b", 128, 3, 7, "draft trees/s (0.5B-shape 4-bit draft, depth 3, 7 of 200 nodes selected)"),
}
METRIC = STREAM_WORKLOADS["c3"][5]
MIN_TIMED_SECONDS = 2.0


def workload_text(name):
    t, d, prompt, depth, verify, _ = STREAM_WORKLOADS[name]
    if t is None:
        return f"draft-only tree build, {d}-shape draft, prompt {prompt}, depth {depth}, top-8 expansion, {verify} nodes selected, greedy"
    return f"spec-decode {t}-shape target + {d}-shape draft, prompt {prompt}, depth {depth}, verify {verify}, greedy"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs (one query every 100 ms from a
    looping nvidia-smi process; if that produced nothing, one direct query under load is taken instead)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc, self.note = gpu_index, [], None, None

    def _cmd(self, loop):
        cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index)]
        return cmd + (["-lms", "100"] if loop else [])

    def start(self):
        try:
            self.proc = subprocess.Popen(self._cmd(True), stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError as e:
            self.proc, self.note = None, f"nvidia-smi could not be started: {e}"

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def sample_once(self):
        """One direct query (used under load when the looping process has not printed yet)."""
        try:
            out = subprocess.run(self._cmd(False), capture_output=True, text=True, timeout=10).stdout
            for line in out.splitlines():
                self.rows.append([c.strip() for c in line.split(",")])
        except (OSError, subprocess.TimeoutExpired) as e:
            self.note = f"direct nvidia-smi query failed: {e}"

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [v for v in sm if v > 500] or sm
        out = {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
               "reasons": sorted(reasons), "samples": len(sm)}
        if not sm:
            out["note"] = self.note or "nvidia-smi printed no parsable row during the timed region"
        return out


def _qmm_bytes(m, n, k, bias=False):
    return n * k // 2 + 4 * n * k // 64 + 2 * m * k + 2 * m * n + (2 * n if bias else 0)


def forward_algorithmic_bytes(model, rows, kv_rows):
    """Bytes one forward pass of `rows` tokens has to move: every linear layer's packed weights, scales and
    biases plus its activations in and out (the per-matmul formula), and the K/V rows attention reads."""
    a = model.args
    H, I = a.hidden_size, a.intermediate_size
    nqkv = model.nq + 2 * model.nkv
    resid = 2 * rows * H
    per_layer = (_qmm_bytes(rows, nqkv, H, a.attention_bias)
                 + _qmm_bytes(rows, H, model.nq) + resid
                 + 2 * _qmm_bytes(rows, I, H) - 2 * rows * H - 2 * rows * I
                 + _qmm_bytes(rows, H, I) + resid
                 + 2 * kv_rows * a.num_key_value_heads * a.head_dim * 2)
    return len(model.layers) * per_layer + _qmm_bytes(rows, model.vocab_local, H)


def forward_roofline(torch, model, cache, rows, prefix, reps):
    """Time one forward pass alone (one launch of the persistent kernel = one pass of `rows` tokens over a
    `prefix`-row cache) as a CUDA graph, with CUDA events on the launching stream."""
    f = model.fwd
    g = torch.Generator().manual_seed(99)
    f.tokens[:rows].copy_(torch.randint(0, model.args.vocab_size, (rows,), generator=g, dtype=torch.int32))
    f.pos[:rows].copy_(prefix + torch.arange(rows, dtype=torch.int32))
    f.mask[:rows].copy_(torch.tensor([(2 << i) - 1 for i in range(rows)], dtype=torch.int64))
    f.prefix.fill_(prefix)

    def run():
        model.forward_device(rows, cache, 0, rows)

    run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    model.check_fused_error()
    return forward_algorithmic_bytes(model, rows, prefix + rows), e0.elapsed_time(e1) / 1e3 / reps


# dram__bytes_read.sum + dram__bytes_write.sum of one forward-kernel launch over its algorithmic bytes, from ncu
# captures of few-layer models of the same layer shapes (profiles/): the full launches hold several GB and are
# not captured.  Traffic grows with the layers streamed, so the ratio carries over to the launch timed here.
# Measured: 0.995 on the 7B layer shape at 16 rows, 1.007 on the 0.5B layer shape at 8 rows (small layers: the share of
# activations and KV that miss L2 is larger).
FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC = 0.995
FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC_SMALL = 1.007        # hidden size below 2048


def roofline_block(torch, model, cache, rows, prefix, name, reps=20):
    peak, peak_src = _peaks()
    alg, sec = forward_roofline(torch, model, cache, rows, prefix, reps)
    a = model.args
    return {"bound": "hbm", "achieved": alg / sec / 1e9, "peak": peak, "unit": "GB/s", "frac": alg / sec / 1e9 / peak,
            "traffic": (FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC if a.hidden_size >= 2048
                        else FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC_SMALL) * alg,
            "traffic_source": "dram bytes of an ncu capture of a 4-layer model of the same layer shape, scaled by the "
                              "algorithmic bytes (traffic grows with the layers streamed)",
            "peak_source": peak_src,
            "kernel": f"{name}: one pass of {rows} rows over a {prefix}-row cache (embedding, {a.num_hidden_layers} layers, "
                      "vocabulary projection)",
            "algorithmic_bytes_per_launch": alg, "us_per_launch": 1e6 * sec, "launches_timed": reps}


def qmm_sweep(torch, be, dev, launches=100, sets=32, rows=(1, 8, 16, 24, 32)):
    """The operator half of the metric: y = x . dequant(W)^T at N 8192, K 2048 (W ~ N(0, 0.02), 4 bit, group 64,
    x ~ N(0, 1) fp16) for 1, 8, 16, 24, 32 rows.  Every launch reads another of `sets` weight sets (302 MB in
    all, more than the 126 MB L2), each launch is timed by its own pair of CUDA events, the median of `launches`
    launches is reported, as GB/s of the algorithmic bytes and as a fraction of the measured HBM peak and of the
    8 TB/s nominal figure.  The method is the reference bench's (qmm_kernel.py:167-390, utils.py:49-78: a
    wash-out between timed launches; here the rotation of the weight sets).  `chain` is a back-to-back run of
    `sets` different matrices replayed from a CUDA graph (programmatic dependent launch), what a model pass presents
    to the operator."""
    qk = be.qmm_kernel
    N, K = 8192, 2048
    peak, _ = _peaks()
    g = torch.Generator(device=dev).manual_seed(7)
    plain, tiled = [], []
    for _ in range(sets):
        wq, s, b = be.quantize.quantize(torch.randn(N, K, generator=g, device=dev) * 0.02)
        plain.append((wq, s, b))
        tiled.append(qk.relayout(wq, s, b))
    out = []
    for m in rows:
        x = torch.randn(m, K, generator=g, device=dev).half()
        y = torch.empty(m, N, dtype=torch.float16, device=dev)
        alg = _qmm_bytes(m, N, K)
        row = {"M": m, "N": N, "K": K, "algorithmic_bytes": alg, "flop_per_byte": 2.0 * m * N * K / alg}

        def run_plain(i):
            qk.matmul_fused(x, *plain[i % sets], out=y)

        def run_tiled(i):
            qk.matmul_tiled(x, tiled[i % sets], N, out=y)

        for name, fn in (("b200_qmm", run_plain), ("b200_qmm_tiled", run_tiled)):
            for i in range(sets):
                fn(i)
            torch.cuda.synchronize()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(launches)]
            for i, (a0, a1) in enumerate(ev):
                a0.record()
                fn(i)
                a1.record()
            torch.cuda.synchronize()
            us = sorted(a0.elapsed_time(a1) * 1e3 for a0, a1 in ev)
            med = us[len(us) // 2]
            # back-to-back chain over all weight sets, recorded once into a CUDA graph (no host time between the
            # launches), one pair of events around three replays
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(sets):
                    fn(i)
            graph.replay()
            torch.cuda.synchronize()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(3):
                graph.replay()
            c1.record()
            torch.cuda.synchronize()
            chain_us = c0.elapsed_time(c1) * 1e3 / (3 * sets)
            row[name] = {"median_us": med, "min_us": us[0], "GBs": alg / med / 1e3, "frac_of_measured_peak": alg / med / 1e3 / peak,
                         "frac_of_8TBs": alg / med / 1e3 / 8000.0, "chain_us_per_launch": chain_us,
                         "chain_GBs": alg / chain_us / 1e3, "chain_frac_of_measured_peak": alg / chain_us / 1e3 / peak}
        out.append(row)
    return {"shape": "N 8192 x K 2048, 4 bit, group 64, fp16", "weight_sets": sets, "launches": launches,
            "timing": "CUDA events per launch, median; weight sets rotate (302 MB > L2)", "rows": out}


def cpu_sample(steps, warm=0, seed=0, workload="c3"):
    """The CPU restatement on a bounded sample: `warm` untimed + `steps` timed speculative steps at the
    full shapes, with the committed KV rows of the prompt pre-filled (prompt ingestion is outside the metric's
    timer).  Returns (tokens produced by the timed steps, their seconds, host threads used)."""
    import numpy as np
    import b200_eagle as be
    from oracle import eagle_ref, model_ref, qmm_c
    from oracle import tree_ref as tr

    cores = qmm_c.use_all_cores()          # launchers export OMP_NUM_THREADS=1; the baseline gets every core
    try:
        import torch
        torch.set_num_threads(cores)
    except Exception:
        pass
    tname, dname, prompt, depth, verify, _ = STREAM_WORKLOADS[workload]
    rng = np.random.default_rng(seed)

    def lin(n, k, bias=False):
        s = (rng.random((n, k // 64), dtype=np.float32) * 0.004 + 0.002).astype(np.float16)
        return dict(weight=rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint32), scales=s,
                    biases=(-7.5 * s.astype(np.float32)).astype(np.float16),
                    bias=(rng.standard_normal(n) * 0.02).astype(np.float16) if bias else None)

    def state(args):
        H, I, hd = args.hidden_size, args.intermediate_size, args.head_dim
        nq, nkv = args.num_attention_heads * hd, args.num_key_value_heads * hd
        layers = [dict(qkv=lin(nq + 2 * nkv, H, args.attention_bias), o=lin(H, nq), gate=lin(I, H), up=lin(I, H),
                       down=lin(H, I), input_norm=np.ones(H, np.float16), post_norm=np.ones(H, np.float16))
                  for _ in range(args.num_hidden_layers)]
        inv, sc = be.llama.rope_inv_freqs(args)
        return dict(layers=layers, embed=lin(args.vocab_size, H), norm=np.ones(H, np.float16),
                    lm_head=None if args.tie_word_embeddings else lin(args.vocab_size, H),
                    inv_freqs=inv.numpy(), rope_scaling_factor=sc)

    da = be.shape_preset(dname)
    draft = model_ref.OracleModel(da, state(da))
    rows = prompt + 8 * (steps + warm + depth + 2) + verify + 64
    dc = model_ref.make_prompt_cache(draft, rows)
    caches = [dc]
    if tname is not None:
        ba = be.shape_preset(tname)
        base = model_ref.OracleModel(ba, state(ba))
        bc = model_ref.make_prompt_cache(base, rows)
        caches.append(bc)
    for cs in caches:
        for c in cs:
            c.keys[:, :, :prompt] = (rng.standard_normal(c.keys[:, :, :prompt].shape) * 0.5).astype(np.float16)
            c.values[:, :, :prompt] = (rng.standard_normal(c.values[:, :, :prompt].shape) * 0.5).astype(np.float16)
            c.offset = prompt
    y, a, n, sec = np.array([1]), 0, 0, 0.0
    for it in range(warm + steps):
        tic = time.perf_counter()
        if tname is None:
            # draft-only tree build (mlx_eagle.py:400-440 without the target pass)
            logits = draft(np.asarray(y).reshape(-1), dc)[[0]]
            ti, tp = tr.root_expand(logits[0], 8)
            parents, tokens, scores = eagle_ref.generate_draft_tree(ti, tp, draft, dc, depth, 8)
            tr.process_draft_tree(scores, tokens, parents, int(y[-1]), 8, verify)
            for c in dc:
                c.offset = prompt
            produced = 1
        else:
            tpi, mi, dt, logits, bo, do = eagle_ref.spec_step(y, base, draft, bc, dc, a, 8, depth, verify)
            retrieve = tr.post_process_draft_tree(tpi, verify, mi)
            cand = dt[0][retrieve]
            best, a, sample = tr.evaluate_posterior_greedy(logits[retrieve], cand)
            idx, acc = retrieve[best, 1:1 + a], cand[best, 1:1 + a]
            tr.accept_candidate([c.keys for c in bc], [c.values for c in bc], idx, a, bo)
            for c in bc:
                c.offset = bo + a + 1
            for c in dc:
                c.offset = do
            y = np.concatenate([acc.astype(np.int64), [min(int(sample.argmax()), da.vocab_size - 1)]])
            produced = 1 + a
        if it >= warm:
            n += produced
            sec += time.perf_counter() - tic
    return n, sec, cores


def reduce_counters(dist, torch, world, produced, sec, e2e_tokens, e2e_sec, dev):
    """Whole-job numbers from per-rank ones: tokens add up over the independent request streams, the time
    is the slowest rank's.  The only collective of the multi-GPU path."""
    if world <= 1:
        return float(produced), float(sec), float(e2e_tokens), float(e2e_sec)
    tot = torch.tensor([float(produced), sec, float(e2e_tokens), e2e_sec], dtype=torch.float64, device=dev)
    sums, maxs = tot.clone(), tot.clone()
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dist.all_reduce(maxs, op=dist.ReduceOp.MAX)
    return float(sums[0]), float(maxs[1]), float(sums[2]), float(maxs[3])


# Tensor-parallel workloads (--workload): one request stream, the target cut across all ranks, the draft
# replicated.  name -> (target preset, draft preset, prompt, depth, verify tokens)
TP_WORKLOADS = {
    "tp70b": ("llama3-70b", "llama3-8b", 512, 3, 23),
    "tp7b": ("qwen2-7b", "qwen2-0.5b", 256, 3, 15),
}


def tensor_parallel_numbers(torch, dist, be, workload, rank, world, dev, K, warmup, with_e2e=True):
    """One request stream with a tensor-parallel target on an initialised process group: column/row-parallel
    shards, the all-reduce of the row-parallel partial products inside the persistent kernel over peer memory,
    vocabulary-parallel argmax.  Also times one target pass both ways: the persistent kernel, and the per-op
    kernels with NCCL all-reduces.  Returns a dict of numbers (the same on every rank)."""
    tname, dname, prompt_len, depth, verify = TP_WORKLOADS[workload]
    tshape, dshape = be.shape_preset(tname), be.shape_preset(dname)
    shard_draft = os.environ.get("B200_TP_DRAFT", "replicated") == "sharded"
    if shard_draft:          # the draft's layers are cut like the target's; its vocabulary projection stays whole
        draft = be.Model.random_init_shard(dshape, 1000, dev, rank, world, shard_head=False).relayout()
        draft.tp.open_exchange(dshape.hidden_size)
    else:
        draft = be.Model.random_init(dshape, seed=1000, device=dev).relayout()      # same weights on every rank
    base = be.Model.random_init_shard(tshape, 2000, dev, rank, world).relayout()
    base.tp.open_exchange(tshape.hidden_size)
    base.tp_two_shot = draft.tp_two_shot = int(os.environ.get("B200_TP_TWO_SHOT", "0"))      # 0 = library default
    assert base.can_fuse() and draft.can_fuse()
    rows = ((prompt_len + 8 * (warmup + K + depth + 8) + verify + 128 + 63) // 64) * 64
    dec = be.SpecDecoder(base, draft, depth, verify, cache_rows=rows, max_out_tokens=8 * (warmup + K) + 512,
                         max_steps=warmup + K + 64)
    dec.warmup(capture=True)
    assert dec.graph is not None
    g = torch.Generator().manual_seed(1234)
    prompt_host = torch.randint(0, min(dshape.vocab_size, tshape.vocab_size), (prompt_len,), generator=g,
                                dtype=torch.int32).pin_memory()
    dec.prefill(prompt_host)
    for _ in range(warmup):
        dec.replay()
    torch.cuda.synchronize()
    n0 = int(dec.ctl[3])
    sampler = ClockSampler(dev.index)
    sampler.start()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        dec.replay()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    sec = e0.elapsed_time(e1) / 1e3
    clocks = sampler.stop()
    produced = int(dec.ctl[3]) - n0
    base.check_fused_error()
    log = dec.step_log[2 * warmup: 2 * (warmup + K)].cpu().view(-1, 2)
    mean_accept = float(log[:, 0].float().mean())

    res, e2e_sec = None, 0.0
    if with_e2e:
        n_e2e = min(K, 300)
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        res = dec.generate(prompt_host, max_tokens=n_e2e, N=n_e2e)
        torch.cuda.synchronize()
        e2e_sec = time.perf_counter() - t0

    # one target pass alone, both ways (collective: every rank runs it)
    prefix_now = int(dec.ctl[0])
    alg, fsec = forward_roofline(torch, base, dec.base_cache, verify + 1, prefix_now, reps=10)
    dalg, dsec = forward_roofline(torch, draft, dec.draft_cache, 8, prefix_now, reps=10)
    base.fused = False                                # per-op kernels + NCCL all-reduce, launched eagerly
    for _ in range(2):
        base.forward_device(verify + 1, dec.base_cache, 0, verify + 1)
    torch.cuda.synchronize()
    dist.barrier()
    n0e, n1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0e.record()
    for _ in range(5):
        base.forward_device(verify + 1, dec.base_cache, 0, verify + 1)
    n1e.record()
    torch.cuda.synchronize()
    nccl_sec = n0e.elapsed_time(n1e) / 1e3 / 5
    base.fused = True
    # the same pass in the pull form of the exchange (every GPU reads the peers' partial products after the barrier)
    chosen = base.tp_two_shot
    base.tp.reset_exchange()
    base.tp_two_shot = 4
    _, pull_sec = forward_roofline(torch, base, dec.base_cache, verify + 1, prefix_now, reps=10)
    base.check_fused_error()
    base.tp.reset_exchange()
    base.tp_two_shot = chosen

    t = torch.tensor([sec, e2e_sec, fsec, nccl_sec, dsec, pull_sec], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec, e2e_sec, fsec, nccl_sec, dsec, pull_sec = (float(v) for v in t)
    step_bytes = base.linear_weight_bytes() + (depth + 1) * draft.linear_weight_bytes()
    out = dict(tname=tname, dname=dname, prompt_len=prompt_len, depth=depth, verify=verify, sec=sec, produced=produced,
               mean_accept=mean_accept, clocks=clocks, res=res, e2e_sec=e2e_sec, alg=alg, fsec=fsec, nccl_sec=nccl_sec, pull_sec=pull_sec,
               dsec=dsec, step_bytes=step_bytes, prefix_now=prefix_now, launches=dec.kernel_launches_per_step * K,
               head_dim=tshape.head_dim, draft_mode="layers cut across the GPUs, whole vocabulary projection" if shard_draft
               else "replicated")
    dist.barrier()
    base.tp.close_exchange()
    if shard_draft:
        draft.tp.close_exchange()
    del dec, base, draft
    torch.cuda.empty_cache()
    return out


def run_tensor_parallel(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import b200_eagle as be

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world < 2:
        raise SystemExit("--workload tp*: launch under torch.distributed.run with 2, 4 or 8 ranks")
    dist.init_process_group("nccl", device_id=dev)
    warmup, K = max(args.warmup, 3), args.steps
    r = tensor_parallel_numbers(torch, dist, be, args.workload, rank, world, dev, K, warmup)
    if rank == 0:
        peak, peak_src = _peaks()
        achieved = r["alg"] / r["fsec"] / 1e9
        res, sec = r["res"], r["sec"]
        e2e_steps = max(res["steps_launched"], 1)
        mt = (r["verify"] + 1 + 7) // 8
        line = {
            "metric": "accepted tokens/s (one request stream, tensor-parallel target)", "value": r["produced"] / sec,
            "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup, "ms_per_step": 1e3 * sec / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic (random-init weights drawn at shard shapes from one seed on every rank)",
            "config": {"workload": f"spec-decode {r['tname']}-shape target cut over {world} GPUs + replicated {r['dname']}-shape "
                                   f"draft, prompt {r['prompt_len']}, depth {r['depth']}, verify {r['verify']}, greedy",
                       "parallelism": f"tp{world} target (all-reduce inside the persistent kernel over peer memory), "
                                      f"draft {r['draft_mode']}, replicated tree logic",
                       "l2": "inputs larger than L2 (weights streamed every step)", "mean_accept_length": r["mean_accept"],
                       "weight_bytes_per_step_per_gpu": r["step_bytes"],
                       "step_weight_stream_frac_of_peak": r["step_bytes"] / (sec / K) / 1e9 / peak,
                       "target_pass_ms": {"persistent_kernel_peer_memory_allreduce": 1e3 * r["fsec"],
                                          "persistent_kernel_pull_form_of_the_exchange": 1e3 * r["pull_sec"],
                                          "per_op_kernels_nccl_allreduce_eager": 1e3 * r["nccl_sec"]},
                       "draft_pass_ms": 1e3 * r["dsec"], "draft": r["draft_mode"]},
            "clocks": r["clocks"],
            "e2e": {"value": res["produced"] / r["e2e_sec"], "unit": UNIT,
                    "h2d_bytes_per_step": res["h2d_bytes"] / e2e_steps, "d2h_bytes_per_step": res["d2h_bytes"] / e2e_steps,
                    "region": "SpecDecoder.generate on every rank: pinned-host prompt copy, prompt ingestion, decode loop "
                              "with a pinned read-back of the counters every step, token read-back"},
            "gpu_launches": r["launches"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src,
                         "kernel": f"forward_kernel<{mt},{r['head_dim']}>: one target pass of {r['verify'] + 1} rows over a "
                                   f"{r['prefix_now']}-row cache on one shard of {world}, exchanges with the peers included",
                         "algorithmic_bytes_per_launch": r["alg"], "us_per_launch": 1e6 * r["fsec"]},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def operator_sweep(torch, be, dev, reps=20):
    """The two matmul operators on re-laid-out weights at the 7B-shape target's big layers, at decode row counts and
    at 128 rows (prompt ingestion; the streaming kernel then needs four launches): the streaming kernel on mma.sync
    (b200_qmm_tiled) and the tcgen05 kernel (b200_qmm_umma).  CUDA events; the launches rotate
    through more than 126 MB of weights so that no launch finds its weights in L2."""
    qk = be.qmm_kernel
    out = []

    def tiled_blocks(x, wt, n, out):              # the streaming kernel takes 32 rows per launch
        for r in range(0, x.shape[0], 32):
            qk.matmul_tiled(x[r:r + 32], wt, n, out=out[r:r + 32])

    for (m, n, k) in [(16, 18944, 3584), (16, 152064, 3584), (8, 151936, 896), (128, 18944, 3584), (128, 152064, 3584)]:
        g = torch.Generator(device=dev).manual_seed(1)
        nbytes = n * k // 2 + n * k // 16
        copies = max(2, int(300e6 // nbytes) + 1)
        wts = []
        for _ in range(copies):
            wq, s, b = be.quantize.quantize(torch.randn(n, k, generator=g, device=dev) * 0.02)
            wts.append(qk.relayout(wq, s, b))
        x = torch.randn(m, k, generator=g, device=dev).half()
        y = torch.empty(m, n, dtype=torch.float16, device=dev)
        row = {"M": m, "N": n, "K": k, "weight_bytes": nbytes}
        for name, fn in (("qmm_tiled", tiled_blocks if m > 32 else qk.matmul_tiled), ("qmm_umma", qk.matmul_umma)):
            for i in range(3):
                fn(x, wts[i % copies], n, out=y)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                fn(x, wts[i % copies], n, out=y)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / reps * 1e3
            row[name] = {"us": us, "GBs": nbytes / us / 1e3}
        row["umma_error_word"] = qk.umma_error(dev)
        out.append(row)
        del wts
    return out


def run_reference(args, rank):
    """The reference arm: the CPU restatement of the path on every core this process may use (rank 0 only)."""
    if rank != 0:
        return
    wl = args.workload if args.workload in STREAM_WORKLOADS else "c3"
    steps = max(1, min(args.steps, 4))
    warm = 1 if args.warmup > 0 else 0
    n, sec, cores = cpu_sample(steps, warm, workload=wl)
    value = n / sec
    tname, dname, prompt, depth, verify, metric = STREAM_WORKLOADS[wl]
    sample = (f"{steps} of the requested {args.steps} steps at the full shapes on {cores} host threads (thread count set "
              f"explicitly, OMP_NUM_THREADS ignored); weights drawn directly in packed 4-bit form, {prompt} committed KV rows "
              "pre-filled (prompt ingestion untimed)")
    line = {"impl": "reference", "metric": metric, "value": value, "unit": UNIT if tname else "trees/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sec / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_text(wl), "note": "CPU restatement of the reference path (MLX/Metal cannot run "
                       "on Linux)", "host_threads": cores},
            "cpu_baseline": {"value": value, "unit": UNIT if tname else "trees/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT if tname else "trees/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def parity_check(be, base, draft, depth, verify, prompt_len, steps=3):
    """Three speculative steps of the very models that are timed, kernel by kernel, with the CPU restatement's
    integer logic run on the GPU's logits after every kernel: tree indices, masks, positions, accept lengths and
    tokens must be bit-identical.  Raises AssertionError otherwise."""
    from oracle.lockstep import lockstep
    rows = ((prompt_len + 8 * (steps + depth + 8) + verify + 128 + 63) // 64) * 64
    hist = lockstep(be, base, draft, depth, verify, steps=steps, prompt_len=prompt_len, seed=4321, cache_rows=rows,
                    check_kv=False)
    return {"steps": steps, "ok": True, "accept_lengths": hist,
            "what": "oracle integer logic on the GPU logits after every kernel of a step: pool, parents, masks, positions, "
                    "retrieve paths, accept length, tokens, counters bit-identical"}


def timed_blocks(torch, dist, world, dec, K, snapshot, min_seconds=MIN_TIMED_SECONDS):
    """Replays the K-step block from the same decode state until MIN_TIMED_SECONDS have been timed (at least 3
    blocks); CUDA events around each block, barrier + synchronize on both sides.  Returns the per-block seconds
    and the tokens one block produces."""
    ctl0, y0 = snapshot
    secs, produced = [], None
    while len(secs) < 3 or (sum(secs) < min_seconds and len(secs) < 400):
        dec.ctl.copy_(ctl0)
        dec.y.copy_(y0)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            dec.replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        secs.append(e0.elapsed_time(e1) / 1e3)
        p = int(dec.ctl[3]) - int(ctl0[3])
        produced = p if produced is None else produced
    return secs, produced


def accept_length_numbers(torch, be, draft, dname, depth, verify, prompt_len, dev):
    """Does the step time depend on how many tokens are accepted?  Random-init pairs accept nothing, so the headline
    runs at one token per step.  Here the draft-shape model is the target too, once with a different random model as
    its draft (accept length 0) and once with itself (the draft agrees with the target wherever the 8-row and the
    wider pass round alike): same shapes, same launch sequence, different accept lengths."""
    other = be.Model.random_init(be.shape_preset(dname), seed=777, device=dev).relayout()
    out = []
    for name, d in (("a different random model as draft", other), ("the target as its own draft", draft)):
        dec = be.SpecDecoder(draft, d, depth, verify, cache_rows=2048, max_out_tokens=2048, max_steps=256)
        dec.warmup()
        dec.prefill(torch.randint(0, draft.args.vocab_size, (prompt_len,), generator=torch.Generator().manual_seed(5),
                                  dtype=torch.int32))
        for _ in range(5):
            dec.replay()
        torch.cuda.synchronize()
        ctl0, y0 = dec.ctl.clone(), dec.y.clone()
        ts = []
        for _ in range(5):
            dec.ctl.copy_(ctl0)
            dec.y.copy_(y0)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                dec.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 50)
        out.append({"draft": name, "ms_per_step": statistics.median(ts),
                    "tokens_per_step": (int(dec.ctl[3]) - int(ctl0[3])) / 50})
        del dec
    del other
    torch.cuda.empty_cache()
    return {"models": f"{dname} shape as target and draft, depth {depth}, verify {verify}", "cases": out,
            "reading": "the step is a fixed launch sequence: its time does not depend on the accept length, tokens/s does"}


def batched_requests_numbers(torch, be, base, draft, depth, verify, prompt_len, K, warmup, dev, min_seconds):
    """The same step for several requests at once on this GPU (``BatchSpecDecoder``: every pass is shared, so each
    weight read serves all requests): as many requests as fit a 32-row pass, K-step blocks replayed from one decode
    state like the headline, CUDA events; plus the public call from pinned host prompts.  Not the headline: the
    workload of the metric is one request per GPU."""
    R = min(4, 32 // (verify + 1), 32 // 8)
    if R < 2:
        return None
    Kb = min(K, 100)
    rows = min(2048, ((prompt_len + (depth + 2) * (warmup + Kb + 8) + verify + 192 + 63) // 64) * 64)
    dec = be.BatchSpecDecoder(base, draft, depth, verify, cache_rows=rows, requests=R,
                              max_out_tokens=(depth + 2) * (warmup + Kb) + 512, max_steps=warmup + Kb + 64)
    dec.warmup(capture=True)
    vocab = min(draft.args.vocab_size, base.args.vocab_size)
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=torch.Generator().manual_seed(4321 + r),
                             dtype=torch.int32).pin_memory() for r in range(R)]
    dec.prefill(prompts)
    for _ in range(warmup):
        dec.replay()
    torch.cuda.synchronize()
    ctl0 = dec.ctl.clone()
    y0 = [s.y.clone() for s in dec.slots]
    secs, produced = [], None
    while len(secs) < 3 or (sum(secs) < min_seconds / 2 and len(secs) < 200):
        dec.ctl.copy_(ctl0)
        for s, y in zip(dec.slots, y0):
            s.y.copy_(y)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(Kb):
            dec.replay()
        e1.record()
        torch.cuda.synchronize()
        secs.append(e0.elapsed_time(e1) / 1e3)
        produced = int((dec.ctl[:, 3] - ctl0[:, 3]).sum())
    sec = statistics.median(secs)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = dec.generate(prompts, max_tokens=Kb, N=Kb)
    torch.cuda.synchronize()
    e2e_sec = time.perf_counter() - t0
    e2e_tokens = sum(r["produced"] for r in res)
    mt = (R * (verify + 1) + 7) // 8
    target = roofline_block(torch, base, dec.slots[0].base_cache, min(32, R * (verify + 1)), prompt_len,
                            f"forward_kernel<{mt},{base.args.head_dim}> at the rows of {R} requests (one cache: timing only)", reps=10)
    out = {"requests_per_gpu": R, "tokens_per_second": produced / sec, "ms_per_step": 1e3 * sec / Kb, "steps": Kb,
           "blocks": len(secs), "tokens_per_step": produced / Kb,
           "e2e_tokens_per_second": e2e_tokens / e2e_sec,
           "gpu_launches_per_step": dec.kernel_launches_per_step,
           "target_pass_us_at_these_rows": target["us_per_launch"], "target_pass_frac_of_measured_peak": target["frac"],
           "what": "BatchSpecDecoder: the requests share every draft and target pass (row groups of one launch, a KV slab "
                   "and a committed length each); tree kernels, acceptance and compaction run per request; every request's "
                   "tokens equal its single-request run (tests/test_batch_gpu.py)"}
    del dec
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the operator sweep, the parity pre-flight, the tensor-parallel attachment and the CPU baseline "
                         "(profiling runs)")
    ap.add_argument("--roofline-only", action="store_true",
                    help="only one model's forward kernel (small profiling case with --layers): the target at 16 rows, or "
                         "with --draft the draft at 8 rows")
    ap.add_argument("--draft", action="store_true", help="with --roofline-only: the draft model's pass instead of the target's")
    ap.add_argument("--layers", type=int, default=0, help="with --roofline-only: number of decoder layers (0 = all)")
    ap.add_argument("--operator-sweep", action="store_true",
                    help="only time the two matmul operators (mma.sync streaming kernel, tcgen05 kernel) at big layer shapes")
    ap.add_argument("--qmm-sweep", action="store_true", help="only the 8192 x 2048 operator sweep at 1..32 rows")
    ap.add_argument("--rows", type=int, default=0, help="with --qmm-sweep: only this row count (profiling)")
    ap.add_argument("--launches", type=int, default=100, help="with --qmm-sweep: timed launches per kernel and row count")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the block of --steps steps until this much time has been measured (0: three blocks; profiling)")
    ap.add_argument("--workload", default="c3", choices=["streams"] + sorted(STREAM_WORKLOADS) + sorted(TP_WORKLOADS),
                    help="c3 (= streams, the default): one independent request stream per GPU; c2: draft-only tree build; c4: "
                         "Llama-3-8B/3.2-1B shapes, prompt 1024; tp70b / tp7b: one stream with the target cut across all ranks")
    args = ap.parse_args()
    if args.workload == "streams":
        args.workload = "c3"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import b200_eagle as be

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.workload in TP_WORKLOADS:
        run_tensor_parallel(args, rank, world, local_rank)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.operator_sweep:
        print(json.dumps({"operator_sweep": operator_sweep(torch, be, dev, reps=max(1, min(args.steps, 20)))}))
        return
    if args.qmm_sweep:
        print(json.dumps({"qmm_sweep": qmm_sweep(torch, be, dev, launches=args.launches,
                                                 rows=(args.rows,) if args.rows else (1, 8, 16, 24, 32))}))
        return
    tname, dname, PROMPT, DEPTH, VERIFY, metric = STREAM_WORKLOADS[args.workload]
    warmup = max(args.warmup, 3)
    K = args.steps

    if args.roofline_only:
        import dataclasses
        shape = be.shape_preset(dname if (args.draft or tname is None) else tname)
        if args.layers:
            shape = dataclasses.replace(shape, num_hidden_layers=args.layers)
        m = be.Model.random_init(shape, seed=2000, device=dev).relayout()
        rows = 8 if (args.draft or tname is None) else VERIFY + 1
        cache = m.make_cache(((PROMPT + 128 + 63) // 64) * 64)
        m(torch.randint(0, shape.vocab_size, (1, PROMPT)), cache=cache, logits_last_only=True)
        blk = roofline_block(torch, m, cache, rows, PROMPT, "forward kernel", reps=max(1, min(args.steps, 20)))
        blk.update({"roofline_only": True, "layers": shape.num_hidden_layers})
        print(json.dumps(blk))
        return

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    draft = be.Model.random_init(be.shape_preset(dname), seed=1000 + rank, device=dev).relayout()
    # c2 has no target: the draft stands in wherever the decoder wants one (it is never run as the target)
    base = be.Model.random_init(be.shape_preset(tname), seed=2000 + rank, device=dev).relayout() if tname else draft
    extras = not args.no_extras
    parity = None
    if extras and tname is not None:
        parity = parity_check(be, base, draft, DEPTH, VERIFY, PROMPT)      # raises on any mismatch

    rows = ((PROMPT + 8 * (warmup + K + DEPTH + 8) + VERIFY + 128 + 63) // 64) * 64
    dec = be.SpecDecoder(base, draft, DEPTH, VERIFY, cache_rows=rows, max_out_tokens=8 * (warmup + K) + 512,
                         max_steps=warmup + K + 64)
    if tname is None:
        dec.step = dec.draft_tree_step                     # the step (and its graph) is the tree build alone
        dec.kernel_launches_per_step = (DEPTH + 1) * (draft.launches_per_forward + 4) + 2
    dec.warmup(capture=True)
    g = torch.Generator().manual_seed(1234 + rank)
    vocab = min(draft.args.vocab_size, base.args.vocab_size)
    prompt_host = torch.randint(0, vocab, (PROMPT,), generator=g, dtype=torch.int32).pin_memory()

    # ---- time to the first token: pinned host prompt -> both models ingest it -> first greedy token on the host
    dec.prefill(prompt_host)            # untimed: records the CUDA graphs of the 128-row prompt passes for these caches
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dec.prefill(prompt_host)
    torch.cuda.synchronize()
    ttft = time.perf_counter() - t0

    # ---- device-resident number: blocks of K graph replays after W warm-up steps ----------------
    for _ in range(warmup):
        dec.replay()
    torch.cuda.synchronize()
    snapshot = (dec.ctl.clone(), dec.y.clone())
    sampler = ClockSampler(local_rank)
    sampler.start()
    torch.cuda.nvtx.range_push("timed_steps")
    secs, produced = timed_blocks(torch, dist, world, dec, K, snapshot, args.min_seconds)
    torch.cuda.nvtx.range_pop()
    if not sampler.rows:
        for _ in range(K):                                  # keep the GPU busy while one direct query runs
            dec.replay()
        sampler.sample_once()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    sec = statistics.median(secs)
    if tname is None:
        produced = K                                        # one tree per step
    log = dec.step_log[2 * warmup: 2 * (warmup + K)].cpu().view(-1, 2)
    mean_accept = float(log[:, 0].float().mean()) if tname else None

    # ---- end to end through the public call, pinned host prompt in, tokens out ----------------
    if tname is not None:
        n_e2e = min(K, 300)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = dec.generate(prompt_host, max_tokens=n_e2e, N=n_e2e)
        torch.cuda.synchronize()
        e2e_sec = time.perf_counter() - t0
        e2e_tokens, e2e_steps = res["produced"], max(res["steps_launched"], 1)
        h2d, d2h = res["h2d_bytes"] / e2e_steps, res["d2h_bytes"] / e2e_steps
        region = ("SpecDecoder.generate: pinned-host prompt copy, prompt ingestion, decode loop with a pinned read-back of the "
                  "counters every step, token read-back")
    else:
        # draft-only: pinned host prompt in, K tree builds, the selected tree (tokens, parents, positions) back to the host
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dec.prefill(prompt_host)
        for _ in range(K):
            dec.replay()
            tree = (dec.draft_tokens[:VERIFY + 1].cpu(), dec.mask_index[:VERIFY].cpu(), dec.tree_position_ids[:VERIFY + 1].cpu())
        torch.cuda.synchronize()
        e2e_sec = time.perf_counter() - t0
        e2e_tokens, e2e_steps = K, K
        h2d, d2h = PROMPT * 4 / K, sum(t.numel() * 4 for t in tree)
        region = "prompt copy from pinned host memory, draft prompt ingestion, K tree builds each followed by a read-back of the tree"

    produced_all, sec_all, e2e_tokens_all, e2e_sec_all = reduce_counters(dist, torch, world, produced, sec, e2e_tokens,
                                                                         e2e_sec, dev)

    line = None
    if rank == 0:
        peak, _ = _peaks()
        prefix_now = int(dec.ctl[0]) if tname else PROMPT
        step_bytes = (base.linear_weight_bytes() if tname else 0) + (DEPTH + 1) * draft.linear_weight_bytes()
        unit = UNIT if tname else "trees/s"
        line = {
            "metric": metric, "value": produced_all / sec_all, "unit": unit, "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": 1e3 * sec_all / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_text(args.workload), "requests": world,
                       "parallelism": f"{world} independent request stream(s)",
                       "l2": f"inputs larger than L2 ({step_bytes / 1e9:.2f} GB of weights streamed per step)",
                       "mean_accept_length": mean_accept, "weight_bytes_per_step": step_bytes,
                       "step_weight_stream_frac_of_peak": step_bytes / (sec_all / K) / 1e9 / peak,
                       "timed_blocks": {"blocks": len(secs), "steps_per_block": K, "seconds_timed": sum(secs),
                                        "ms_per_step_median": 1e3 * sec / K, "ms_per_step_min": 1e3 * min(secs) / K,
                                        "ms_per_step_max": 1e3 * max(secs) / K,
                                        "note": "every block replays the same K steps from the same decode state"},
                       "time_to_first_token_ms": 1e3 * ttft,
                       "parity_checked": parity},
            "clocks": clocks,
            "e2e": {"value": e2e_tokens_all / e2e_sec_all, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "region": region},
            "gpu_launches": dec.kernel_launches_per_step * K * len(secs),
        }
        if tname is not None:
            mt = (VERIFY + 1 + 7) // 8
            line["roofline"] = roofline_block(torch, base, dec.base_cache, VERIFY + 1, prefix_now,
                                              f"forward_kernel<{mt},{base.args.head_dim}> (target pass)")
        dblk = roofline_block(torch, draft, dec.draft_cache, 8, prefix_now,
                              f"draft pass of {draft.launches_per_forward} launch(es), {dname} shape")
        if tname is None:
            line["roofline"] = dblk
        else:
            line["roofline_draft"] = dblk
            step_ms = 1e3 * sec / K
            line["config"]["step_time_shares"] = {
                "target_pass_ms": line["roofline"]["us_per_launch"] / 1e3,
                "draft_passes_ms": (DEPTH + 1) * dblk["us_per_launch"] / 1e3,
                "rest_ms": step_ms - line["roofline"]["us_per_launch"] / 1e3 - (DEPTH + 1) * dblk["us_per_launch"] / 1e3}
        if extras:
            line["qmm_sweep"] = qmm_sweep(torch, be, dev)
        if extras and tname is not None and world == 1:
            try:
                line["config"]["batched_requests"] = batched_requests_numbers(
                    torch, be, base, draft, DEPTH, VERIFY, PROMPT, K, warmup, dev, args.min_seconds)
            except Exception as e:                         # the attachment must not take the headline down with it
                line["config"]["batched_requests"] = {"error": f"{type(e).__name__}: {e}"}
            try:
                line["config"]["accept_length_sensitivity"] = accept_length_numbers(torch, be, draft, dname, DEPTH, VERIFY,
                                                                                    PROMPT, dev)
            except Exception as e:
                line["config"]["accept_length_sensitivity"] = {"error": f"{type(e).__name__}: {e}"}
    # ---- at N > 1: the tensor-parallel target on the same ranks (collective), attached to the line
    if world > 1 and extras and args.workload == "c3":
        tp = None
        try:
            del dec
            torch.cuda.empty_cache()
            r = tensor_parallel_numbers(torch, dist, be, "tp70b", rank, world, dev, K=20, warmup=3, with_e2e=False)
            tp = {"workload": f"{r['tname']}-shape target cut over {world} GPUs + replicated {r['dname']}-shape draft, prompt "
                              f"{r['prompt_len']}, depth {r['depth']}, verify {r['verify']}",
                  "tokens_per_second": r["produced"] / r["sec"], "ms_per_step": 1e3 * r["sec"] / 20, "steps": 20,
                  "mean_accept_length": r["mean_accept"],
                  "target_pass_ms": {"persistent_kernel_peer_memory_allreduce": 1e3 * r["fsec"],
                                     "persistent_kernel_pull_form_of_the_exchange": 1e3 * r["pull_sec"],
                                     "per_op_kernels_nccl_allreduce_eager": 1e3 * r["nccl_sec"]},
                  "draft_pass_ms": 1e3 * r["dsec"], "draft": r["draft_mode"]}
        except Exception as e:                             # the attachment must not take the headline down with it
            tp = {"error": f"{type(e).__name__}: {e}"}
        if line is not None:
            line["config"]["tensor_parallel"] = tp
    if rank == 0:
        if extras and not args.no_cpu_baseline and world == 1:
            n_cpu, cpu_sec, cores = cpu_sample(2, warm=1, workload=args.workload)
            line["cpu_baseline"] = {"value": n_cpu / cpu_sec, "unit": line["unit"], "cores": cores, "kind": "port",
                                    "sample": f"2 steps (after 1 untimed) at the full shapes, weights drawn directly in packed "
                                              f"4-bit form, {PROMPT} committed KV rows pre-filled"}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
