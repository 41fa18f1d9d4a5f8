"""Benchmark of the tree speculative decoding hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (N = 1 and every rank at N > 1): full speculative decode steps, greedy, Qwen2-7B-shape
4-bit target + Qwen2-0.5B-shape 4-bit draft (random-init weights, seeded), 256-token seeded random
prompt, depth 3, 15 verify tokens; one "step" is one speculative step (draft catch-up pass, 3 draft
tree passes, tree finalisation, one target pass on 16 tokens, acceptance, KV compaction).
Metric: accepted tokens per second (tokens produced by the timed steps / device time).

The JSON line also carries: the end-to-end number through ``SpecDecoder.generate`` with a pinned
host prompt (``e2e``), the roofline of the dominant kernel (the 4-bit quantised matmul, timed on a
sweep over all target-model linears at 16 rows), and a CPU baseline (the CPU restatement of the
reference's path, timed on a bounded sample on this host's cores).

``--impl reference`` times the CPU restatement only (the reference itself is MLX/Metal and cannot
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

METRIC = "accepted tokens/s (7B-shape 4-bit target + 0.5B draft, 15-node tree)"
UNIT = "tokens/s"
WORKLOAD = "spec-decode qwen2-7b-shape target + qwen2-0.5b-shape draft, prompt 256, depth 3, verify 15, greedy"
DEPTH, VERIFY, PROMPT = 3, 15, 256


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _qmm_bytes(m, n, k, bias=False):
    return n * k // 2 + 4 * n * k // 64 + 2 * m * k + 2 * m * n + (2 * n if bias else 0)


def qmm_roofline(be, torch, model, rows, reps):
    """Time the quantised-matmul launches of one target pass (all layers + head) as one CUDA graph."""
    qk = be.qmm_kernel
    a = model.args
    H, I = a.hidden_size, a.intermediate_size
    nqkv = model.nq + 2 * model.nkv

    def sweep():
        for lw in model.layers:
            model._linear(model.xn, lw["qkv"], model.qkv, rows, qk.EPI_NONE)
            model._linear(model.attn, lw["o"], model.h, rows, qk.EPI_RESIDUAL, extra=model.h)
            model._linear(model.xn, lw["gate"], model.act, rows, qk.EPI_SILU_MUL, lin2=lw["up"])
            model._linear(model.act, lw["down"], model.h, rows, qk.EPI_RESIDUAL, extra=model.h)
        model._linear(model.xn, model.lm_head, model.logits, rows, qk.EPI_NONE)

    nl = len(model.layers)
    resid = 2 * rows * H                                         # residual rows read by the epilogue
    per_layer = (_qmm_bytes(rows, nqkv, H, a.attention_bias)       # q|k|v with bias
                 + _qmm_bytes(rows, H, model.nq) + resid           # o_proj + residual
                 + 2 * _qmm_bytes(rows, I, H) - 2 * rows * H - 2 * rows * I   # gate & up share x, one output
                 + _qmm_bytes(rows, H, I) + resid)                 # down_proj + residual
    alg = nl * per_layer + _qmm_bytes(rows, a.vocab_size, H)
    launches = 4 * nl + 1
    model.h.zero_()
    model.xn.normal_(0, 1)
    model.attn.normal_(0, 1)
    model.act.normal_(0, 1)
    sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / reps
    return alg, launches, sec


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
    """Time the persistent forward kernel alone (one launch = one pass of `rows` tokens over a `prefix`-row
    cache) as a CUDA graph, with CUDA events on the launching stream."""
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


# dram__bytes_read.sum + dram__bytes_write.sum of one forward_kernel<2,128> launch over its algorithmic bytes,
# from one ncu capture of a 4-layer model of the same layer shape (842.4 MB against 846.8 MB; the 28-layer
# launch holds 4.3 GB, too much to capture).  Traffic grows with the layers streamed, so the ratio carries
# over to the launch timed here.
FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC = 0.995


def cpu_sample(steps, warm=0, seed=0):
    """The CPU restatement on a bounded sample: `warm` untimed + `steps` timed speculative steps at the
    full shapes, with the 256 committed KV rows pre-filled (prompt ingestion is outside the metric's
    timer).  Returns (tokens produced by the timed steps, their seconds, host threads used)."""
    import numpy as np
    import b200_eagle as be
    from oracle import eagle_ref, model_ref, qmm_c

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

    da, ba = be.shape_preset("qwen2-0.5b"), be.shape_preset("qwen2-7b")
    draft = model_ref.OracleModel(da, state(da))
    base = model_ref.OracleModel(ba, state(ba))
    rows = PROMPT + 8 * (steps + DEPTH + 2) + VERIFY + 64
    bc, dc = model_ref.make_prompt_cache(base, rows), model_ref.make_prompt_cache(draft, rows)
    for caches in (bc, dc):
        for c in caches:
            c.keys[:, :, :PROMPT] = (rng.standard_normal(c.keys[:, :, :PROMPT].shape) * 0.5).astype(np.float16)
            c.values[:, :, :PROMPT] = (rng.standard_normal(c.values[:, :, :PROMPT].shape) * 0.5).astype(np.float16)
            c.offset = PROMPT
    from oracle import tree_ref as tr
    y, a, n, sec = np.array([1]), 0, 0, 0.0
    for it in range(warm + steps):
        tic = time.perf_counter()
        tpi, mi, dt, logits, bo, do = eagle_ref.spec_step(y, base, draft, bc, dc, a, 8, DEPTH, VERIFY)
        retrieve = tr.post_process_draft_tree(tpi, VERIFY, mi)
        cand = dt[0][retrieve]
        best, a, sample = tr.evaluate_posterior_greedy(logits[retrieve], cand)
        idx, acc = retrieve[best, 1:1 + a], cand[best, 1:1 + a]
        tr.accept_candidate([c.keys for c in bc], [c.values for c in bc], idx, a, bo)
        for c in bc:
            c.offset = bo + a + 1
        for c in dc:
            c.offset = do
        y = np.concatenate([acc.astype(np.int64), [min(int(sample.argmax()), da.vocab_size - 1)]])
        if it >= warm:
            n += 1 + a
            sec += time.perf_counter() - tic
    return n, sec, qmm_c.num_threads()


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


def run_tensor_parallel(args, rank, world, local_rank):
    """One request stream with a tensor-parallel target: column/row-parallel shards, the all-reduce of the
    row-parallel partial products inside the persistent kernel over peer memory, vocabulary-parallel argmax.
    Also times one target pass both ways: the persistent kernel, and the per-op kernels with NCCL all-reduces."""
    import torch
    import torch.distributed as dist
    import b200_eagle as be

    tname, dname, prompt_len, depth, verify = TP_WORKLOADS[args.workload]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world < 2:
        raise SystemExit("--workload tp*: launch under torch.distributed.run with 2, 4 or 8 ranks")
    dist.init_process_group("nccl", device_id=dev)
    warmup, K = max(args.warmup, 3), args.steps
    tshape, dshape = be.shape_preset(tname), be.shape_preset(dname)
    draft = be.Model.random_init(dshape, seed=1000, device=dev).relayout()          # same weights on every rank
    base = be.Model.random_init_shard(tshape, 2000, dev, rank, world).relayout()
    base.tp.open_exchange(tshape.hidden_size)
    assert base.can_fuse()
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
    sampler = ClockSampler(local_rank)
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

    n_e2e = min(K, 300)
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    res = dec.generate(prompt_host, max_tokens=n_e2e, N=n_e2e)
    torch.cuda.synchronize()
    e2e_sec = time.perf_counter() - t0
    e2e_steps = max(res["steps_launched"], 1)

    # one target pass alone, both ways (collective: every rank runs it)
    prefix_now = int(dec.ctl[0])
    alg, fsec = forward_roofline(torch, base, dec.base_cache, verify + 1, prefix_now, reps=20)
    base.fused = False                                # per-op kernels + NCCL all-reduce, launched eagerly
    f = base.fwd
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

    t = torch.tensor([sec, e2e_sec, fsec, nccl_sec], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec, e2e_sec, fsec, nccl_sec = (float(v) for v in t)
    if rank == 0:
        peak, peak_src = _peaks()
        achieved = alg / fsec / 1e9
        step_bytes = base.linear_weight_bytes() + (depth + 1) * draft.linear_weight_bytes()
        mt = (verify + 1 + 7) // 8
        line = {
            "metric": "accepted tokens/s (one request stream, tensor-parallel target)", "value": produced / sec,
            "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup, "ms_per_step": 1e3 * sec / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic (random-init weights drawn at shard shapes from one seed on every rank)",
            "config": {"workload": f"spec-decode {tname}-shape target cut over {world} GPUs + replicated {dname}-shape "
                                   f"draft, prompt {prompt_len}, depth {depth}, verify {verify}, greedy",
                       "parallelism": f"tp{world} target (all-reduce inside the persistent kernel over peer memory), "
                                      "replicated draft and tree logic",
                       "l2": "inputs larger than L2 (weights streamed every step)", "mean_accept_length": mean_accept,
                       "weight_bytes_per_step_per_gpu": step_bytes,
                       "step_weight_stream_frac_of_peak": step_bytes / (sec / K) / 1e9 / peak,
                       "target_pass_ms": {"persistent_kernel_peer_memory_allreduce": 1e3 * fsec,
                                          "per_op_kernels_nccl_allreduce_eager": 1e3 * nccl_sec}},
            "clocks": clocks,
            "e2e": {"value": res["produced"] / e2e_sec, "unit": UNIT,
                    "h2d_bytes_per_step": res["h2d_bytes"] / e2e_steps, "d2h_bytes_per_step": res["d2h_bytes"] / e2e_steps,
                    "region": "SpecDecoder.generate on every rank: pinned-host prompt copy, prompt ingestion, decode loop "
                              "with a pinned read-back of the counters every step, token read-back"},
            "gpu_launches": dec.kernel_launches_per_step * K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src,
                         "kernel": f"forward_kernel<{mt},{tshape.head_dim}>: one target pass of {verify + 1} rows over a "
                                   f"{prefix_now}-row cache on one shard of {world}, exchanges with the peers included",
                         "algorithmic_bytes_per_launch": alg, "us_per_launch": 1e6 * fsec},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    base.tp.close_exchange()
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
    if rank != 0:
        return
    steps = max(1, min(args.steps, 4))
    warm = 1 if args.warmup > 0 else 0
    n, sec, cores = cpu_sample(steps, warm)
    value = n / sec
    sample = (f"{steps} of the requested {args.steps} steps at the full shapes on {cores} host threads; weights drawn "
              "directly in packed 4-bit form, 256 committed KV rows pre-filled (prompt ingestion untimed)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sec / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (MLX/Metal cannot run "
                       "on Linux)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--roofline-only", action="store_true",
                    help="only the target model's forward kernel at 16 rows (small profiling case with --layers)")
    ap.add_argument("--layers", type=int, default=0, help="with --roofline-only: number of decoder layers (0 = all 28)")
    ap.add_argument("--operator-sweep", action="store_true",
                    help="only time the two matmul operators (mma.sync streaming kernel, tcgen05 kernel) at big layer shapes")
    ap.add_argument("--workload", default="streams", choices=["streams"] + sorted(TP_WORKLOADS),
                    help="streams: one independent request stream per GPU (the default, what --gpus N scales); "
                         "tp70b / tp7b: one stream with the target cut across all ranks (needs 2+ ranks)")
    args = ap.parse_args()
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"        # NCCL writes its version banner to stdout, which carries the JSON line
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
    if args.workload != "streams":
        run_tensor_parallel(args, rank, world, local_rank)
        return
    if args.operator_sweep:
        torch.cuda.set_device(local_rank)
        print(json.dumps({"operator_sweep": operator_sweep(torch, be, torch.device("cuda", local_rank),
                                                           reps=max(1, min(args.steps, 20)))}))
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    K = args.steps

    if args.roofline_only:
        import dataclasses
        shape = be.shape_preset("qwen2-7b")
        if args.layers:
            shape = dataclasses.replace(shape, num_hidden_layers=args.layers)
        base = be.Model.random_init(shape, seed=2000, device=dev).relayout()
        peak, peak_src = _peaks()
        reps = max(1, min(args.steps, 20))
        if base.can_fuse():
            cache = base.make_cache(512)
            base(torch.randint(0, shape.vocab_size, (1, PROMPT)), cache=cache, logits_last_only=True)
            alg, qsec = forward_roofline(torch, base, cache, VERIFY + 1, PROMPT, reps)
            launches = 1
        else:
            alg, launches, qsec = qmm_roofline(be, torch, base, VERIFY + 1, reps=reps)
        print(json.dumps({"roofline_only": True, "layers": shape.num_hidden_layers, "achieved_gbs": alg / qsec / 1e9,
                          "peak": peak, "frac": alg / qsec / 1e9 / peak, "launches": launches,
                          "algorithmic_bytes": alg, "us_per_launch": 1e6 * qsec / launches}))
        return
    draft = be.Model.random_init(be.shape_preset("qwen2-0.5b"), seed=1000 + rank, device=dev).relayout()
    base = be.Model.random_init(be.shape_preset("qwen2-7b"), seed=2000 + rank, device=dev).relayout()
    rows = ((PROMPT + 8 * (warmup + K + DEPTH + 8) + VERIFY + 128 + 63) // 64) * 64
    dec = be.SpecDecoder(base, draft, DEPTH, VERIFY, cache_rows=rows, max_out_tokens=8 * (warmup + K) + 512,
                         max_steps=warmup + K + 64)
    dec.warmup(capture=True)
    g = torch.Generator().manual_seed(1234 + rank)
    prompt_host = torch.randint(0, draft.args.vocab_size, (PROMPT,), generator=g, dtype=torch.int32).pin_memory()

    # ---- device-resident number: K graph replays after W warm-up steps -------------------------
    dec.prefill(prompt_host)
    for _ in range(warmup):
        dec.replay()
    torch.cuda.synchronize()
    n0 = int(dec.ctl[3])
    sampler = ClockSampler(local_rank)
    sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.nvtx.range_push("timed_steps")
    e0.record()
    for _ in range(K):
        dec.replay()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    if world > 1:
        dist.barrier()
    sec = e0.elapsed_time(e1) / 1e3
    clocks = sampler.stop()
    produced = int(dec.ctl[3]) - n0
    log = dec.step_log[2 * warmup: 2 * (warmup + K)].cpu().view(-1, 2)
    mean_accept = float(log[:, 0].float().mean())

    # ---- end to end through the public call, pinned host prompt in, tokens out ----------------
    n_e2e = min(K, 300)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = dec.generate(prompt_host, max_tokens=n_e2e, N=n_e2e)
    torch.cuda.synchronize()
    e2e_sec = time.perf_counter() - t0
    e2e_tokens, e2e_steps = res["produced"], max(res["steps_launched"], 1)

    produced_all, sec_all, e2e_tokens_all, e2e_sec_all = reduce_counters(dist, torch, world, produced, sec, e2e_tokens,
                                                                         e2e_sec, dev)

    line = None
    if rank == 0:
        peak, peak_src = _peaks()
        if base.can_fuse():
            prefix_now = int(dec.ctl[0])
            alg, qsec = forward_roofline(torch, base, dec.base_cache, VERIFY + 1, prefix_now, reps=20)
            qmm_launches, traffic = 1, FORWARD_KERNEL_DRAM_OVER_ALGORITHMIC * alg
            kernel_name = (f"forward_kernel<2,128>: one target pass of {VERIFY + 1} rows over a {prefix_now}-row cache "
                           "(embedding, 28 layers, vocabulary projection) in one persistent launch")
        else:
            alg, qmm_launches, qsec = qmm_roofline(be, torch, base, VERIFY + 1, reps=20)
            traffic = None
            kernel_name = f"qmm_tiled_kernel, {qmm_launches} launches of one target pass at {VERIFY + 1} rows"
        achieved = alg / qsec / 1e9
        step_bytes = base.linear_weight_bytes() + (DEPTH + 1) * draft.linear_weight_bytes()
        line = {
            "metric": METRIC, "value": produced_all / sec_all, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": 1e3 * sec_all / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests": world, "parallelism": f"{world} independent request stream(s)",
                       "l2": "inputs larger than L2 (4.26 GB of weights streamed per step)",
                       "mean_accept_length": mean_accept, "weight_bytes_per_step": step_bytes,
                       "step_weight_stream_frac_of_peak": step_bytes / (sec_all / K) / 1e9 / peak},
            "clocks": clocks,
            "e2e": {"value": e2e_tokens_all / e2e_sec_all, "unit": UNIT,
                    "h2d_bytes_per_step": res["h2d_bytes"] / e2e_steps, "d2h_bytes_per_step": res["d2h_bytes"] / e2e_steps,
                    "region": "SpecDecoder.generate: pinned-host prompt copy, prompt ingestion, decode loop with a "
                              "pinned read-back of the counters every step, token read-back"},
            "gpu_launches": dec.kernel_launches_per_step * K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_src,
                         "kernel": kernel_name,
                         "algorithmic_bytes_per_launch": alg / qmm_launches, "us_per_launch": 1e6 * qsec / qmm_launches},
        }
        if not args.no_cpu_baseline and world == 1:
            n_cpu, cpu_sec, cores = cpu_sample(2, warm=1)
            line["cpu_baseline"] = {"value": n_cpu / cpu_sec, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": "2 speculative steps (after 1 untimed) at the full shapes, weights drawn "
                                              "directly in packed 4-bit form, 256 committed KV rows pre-filled"}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
