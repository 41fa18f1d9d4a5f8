"""Parity at the benchmark shapes, against the CPU oracle (not against the product's own other kernels).

(1) The persistent forward kernel at full layer widths (two layers, the whole vocabulary head) on tree passes over
    a 1024-row cache prefix: logits and the new K/V rows against ``oracle.model_ref.OracleModel`` within the
    logits tolerance of this library, ``|d| <= 2^-6 |want| + 2e-2``.  The prefix rows are seeded random values
    written into both caches (a CPU prompt pass of 1024 tokens at these widths would take minutes).
(2) Lock-step integer parity of whole speculative steps on the full models of the benchmark configurations:
    the oracle's tree logic runs on the GPU's logits after every kernel, everything integer must be bit-equal.
"""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import model_ref
from oracle.lockstep import lockstep

pytestmark = pytest.mark.gpu
f64 = np.float64
PREFIX = 1024


def _close(got, want, rel, abs_):
    got, want = np.asarray(got).astype(f64), np.asarray(want).astype(f64)
    err = np.abs(got - want)
    assert np.all(err <= rel * np.abs(want) + abs_), f"max err {err.max()} (want scale {np.abs(want).max()})"


def _random_tree(rng, rows):
    """Ancestor mask (bool, rows x rows) and depths of a random tree whose node 0 is the root."""
    tm = np.eye(rows, dtype=bool)
    for i in range(1, rows):
        tm[i] |= tm[rng.integers(max(0, i - 6), i)]
    return tm, tm.sum(1) - 1


@pytest.mark.parametrize("name,rows", [("qwen2-7b", 16), ("qwen2-7b", 32), ("llama3-8b", 32), ("llama3-8b", 16),
                                       ("qwen2-0.5b", 8), ("llama3.2-1b", 8)])
def test_tree_pass_at_full_layer_widths_matches_the_oracle(be, cuda, name, rows):
    args = dataclasses.replace(be.shape_preset(name), num_hidden_layers=2)
    m = be.Model.random_init(args, seed=31, device=cuda)
    om = model_ref.OracleModel(args, m.state_numpy())
    m.relayout()
    assert m.can_fuse()
    rng = np.random.default_rng(rows)
    cache = m.make_cache(PREFIX + 64)
    oc = model_ref.make_prompt_cache(om, PREFIX + 64)
    for li, c in enumerate(oc):
        c.keys[:, :, :PREFIX] = (rng.standard_normal(c.keys[:, :, :PREFIX].shape) * 0.5).astype(np.float16)
        c.values[:, :, :PREFIX] = (rng.standard_normal(c.values[:, :, :PREFIX].shape) * 0.5).astype(np.float16)
        c.offset = PREFIX
        cache.data[li, 0, :, :PREFIX].copy_(torch.from_numpy(c.keys[0, :, :PREFIX]))
        cache.data[li, 1, :, :PREFIX].copy_(torch.from_numpy(c.values[0, :, :PREFIX]))
    cache.offset = PREFIX
    tokens = rng.integers(0, args.vocab_size, rows)
    tm, depth = _random_tree(rng, rows)
    add = np.where(tm, 0.0, -np.inf).astype(np.float32)
    mask = np.concatenate([np.zeros((rows, PREFIX), np.float32), add], axis=1)
    got = m(torch.from_numpy(tokens)[None], cache=cache, mask=torch.from_numpy(mask)[None, None],
            position_ids=torch.from_numpy(depth + PREFIX)[None])[0].cpu().numpy()
    m.check_fused_error()
    want = om(tokens, oc, mask=mask, position_ids=(depth + PREFIX).astype(np.int64))
    _close(got, want, 2.0 ** -6, 2e-2)
    # the token the GPU would pick is, for the oracle, within the tolerance of its own best one
    wf = want.astype(f64)
    picked = wf[np.arange(rows), got.argmax(-1)]
    assert np.all(picked >= wf.max(-1) - 2 * (2.0 ** -6 * np.abs(wf.max(-1)) + 2e-2))
    for li, c in enumerate(oc):
        _close(cache.data[li, 0, :, PREFIX:PREFIX + rows].cpu().numpy(), c.keys[0, :, PREFIX:PREFIX + rows], 2.0 ** -6, 2e-2)
        _close(cache.data[li, 1, :, PREFIX:PREFIX + rows].cpu().numpy(), c.values[0, :, PREFIX:PREFIX + rows], 2.0 ** -6, 2e-2)


@pytest.mark.parametrize("target,draft,prompt,depth,T", [("qwen2-7b", "qwen2-0.5b", 256, 3, 15),
                                                          ("llama3-8b", "llama3.2-1b", 1024, 4, 31)])
def test_full_models_of_the_benchmark_configurations_in_lockstep(be, cuda, target, draft, prompt, depth, T):
    d = be.Model.random_init(be.shape_preset(draft), seed=1000, device=cuda).relayout()
    b = be.Model.random_init(be.shape_preset(target), seed=2000, device=cuda).relayout()
    rows = ((prompt + 8 * (depth + 12) + T + 128 + 63) // 64) * 64
    hist = lockstep(be, b, d, depth, T, steps=3, prompt_len=prompt, seed=17, cache_rows=rows, check_kv=False)
    assert len(hist) == 3
    b.check_fused_error()
    d.check_fused_error()
