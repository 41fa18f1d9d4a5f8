"""Lock-step parity of the on-device tree logic: after every kernel of a decode step the CPU oracle's
integer logic is run on the GPU-produced logits, and every index / token / mask / length must be
bit-identical (scores are fp32 and compared exactly too)."""
import numpy as np
import pytest
import torch

from oracle import detmath, tree_ref as tr

pytestmark = pytest.mark.gpu
K = 8


@pytest.fixture(scope="module")
def models(be, cuda):
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=cuda, gen_device="cpu")
    base.norm.mul_(8.0)      # sharper distributions: deep trees, long accepted paths
    draft.norm.mul_(8.0)
    draft.relayout()         # draft on the streaming weight layout, target on the row-major one
    return args, base, draft


def _lockstep(be, base, draft, depth, T, steps, prompt_len, seed, **kw):
    from oracle.lockstep import lockstep
    return lockstep(be, base, draft, depth, T, steps, prompt_len, seed, **kw)


@pytest.mark.parametrize("depth,T,self_draft", [(3, 15, False), (3, 15, True), (4, 31, True), (1, 7, False),
                                                 (0, 7, True), (6, 23, True), (2, 23, False)])
def test_decode_steps_in_lockstep_with_the_oracle(be, models, depth, T, self_draft):
    _, base, draft = models
    hist = _lockstep(be, base, base if self_draft else draft, depth, T, steps=5, prompt_len=37, seed=depth * 10 + T)
    if self_draft and depth >= 1:
        assert max(hist) >= 2          # drafting with the target itself must get deep paths accepted


def test_rowstats_and_argmax_keys_are_exact(be, cuda):
    from b200_eagle import _lib
    L, p = _lib.lib(), _lib.ptr
    rng = np.random.default_rng(0)
    R, V = 8, 151936
    lg = (rng.standard_normal((R, V)) * 2).astype(np.float16)
    lg[3, 100] = lg[3, 90000] = 9.0           # tie: lower index must win
    lg[5, :] = 0.0
    lg[5, 7] = -0.0
    d = torch.from_numpy(lg).to(cuda)
    rmax = torch.zeros(32, dtype=torch.int32, device=cuda)
    rsum = torch.zeros(32, dtype=torch.int64, device=cuda)
    key = torch.zeros(32, dtype=torch.int64, device=cuda)
    st = _lib.stream_ptr(cuda)
    assert L.b200_logits_rowstats(p(d), R, V, p(rmax), p(rsum), st) == 0
    assert L.b200_logits_argmax(p(d), R, V, p(key), st) == 0
    x = lg.astype(np.float64)
    want_sum = detmath.exp_fixed(x - x.max(-1, keepdims=True)).sum(-1)
    assert rsum[:R].cpu().tolist() == want_sum.tolist()
    idx = [0xFFFFFFFF - (int(k) & 0xFFFFFFFF) for k in key[:R].cpu().tolist()]
    assert idx == lg.astype(np.float32).argmax(-1).tolist() and idx[3] == 100 and idx[5] == 0
