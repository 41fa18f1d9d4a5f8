"""Per-layer kernels and the whole forward pass (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import eagle_ref, model_ref, qmm_ref, tree_ref as tr

pytestmark = pytest.mark.gpu
f64 = np.float64


def _close(got, want, rel, abs_):
    got, want = got.astype(f64), want.astype(f64)
    err = np.abs(got - want)
    assert np.all(err <= rel * np.abs(want) + abs_), f"max err {err.max()} (want scale {np.abs(want).max()})"


@pytest.fixture(scope="module", params=["tiny-qwen2", "tiny-llama"])
def pair(request, be, cuda):
    args = be.shape_preset(request.param)
    m = be.Model.random_init(args, seed=5, device=cuda, gen_device="cpu")
    return args, m, model_ref.OracleModel(args, m.state_numpy())


def test_rms_norm(be, cuda):
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(5, 896, generator=g) * 3).half()
    w = (1 + 0.1 * torch.randn(896, generator=g)).half()
    y = torch.empty_like(x, device=cuda)
    xd, wd = x.to(cuda), w.to(cuda)
    rc = be._lib.lib().b200_rms_norm(be._lib.ptr(xd), be._lib.ptr(wd), be._lib.ptr(y), None, 5, 896,
                                     1e-6, be._lib.stream_ptr(cuda))
    assert rc == 0
    torch.cuda.synchronize()
    _close(y.cpu().numpy(), model_ref.rms_norm(x.numpy(), w.numpy(), 1e-6), 2.0 ** -10, 1e-4)


def test_rope_positions_operator_and_permutation_property(be, cuda):
    # mlx_arrayed_rope_kernel.py:155-236: B=34, L=249, H=37, D=64, offset 467 in the reference's self-check
    rng = np.random.default_rng(0)
    B, H, L, D, off = 3, 5, 33, 64, 467
    x = rng.standard_normal((B, H, L, D)).astype(np.float16)
    inv = (2.0 ** (-np.log2(1e6) * np.arange(0, D, 2) / D)).astype(np.float32)
    perm = np.stack([rng.permutation(L) for _ in range(B)])
    xd, invd = torch.from_numpy(x).to(cuda), torch.from_numpy(inv).to(cuda)
    got = be.rope_positions(xd, torch.from_numpy(perm + off).to(cuda), invd, 1.0)
    _close(got.cpu().numpy(), model_ref.rope_positions(x, perm + off, inv, 1.0), 2.0 ** -9, 2e-3)
    # array-position RoPE == contiguous RoPE of the reordered input, gathered back: bit-equal on one device
    reordered = torch.gather(xd, 2, torch.from_numpy(np.argsort(perm, 1)).to(cuda)[:, None, :, None].expand(B, H, L, D))
    contiguous = be.rope_positions(reordered, torch.arange(L, device=cuda)[None].repeat(B, 1) + off, invd, 1.0)
    back = torch.gather(contiguous, 2, torch.from_numpy(perm).to(cuda)[:, None, :, None].expand(B, H, L, D))
    assert torch.equal(got, back)


def test_embedding_gather(pair, cuda):
    args, m, om = pair
    ids = [0, 5, args.vocab_size - 1, 17]
    m.fwd.tokens[:4].copy_(torch.tensor(ids, dtype=torch.int32))
    from b200_eagle import _lib
    rc = _lib.lib().b200_embed_gather(_lib.ptr(m.fwd.tokens), _lib.ptr(m.embed.weight), _lib.ptr(m.embed.scales),
                                      _lib.ptr(m.embed.biases), _lib.ptr(m.h), 4, args.hidden_size, args.vocab_size,
                                      _lib.stream_ptr(cuda))
    assert rc == 0
    assert np.array_equal(m.h[:4].cpu().numpy(), om.embed_tokens(ids))


def test_causal_forward_matches_oracle_logits_and_cache(pair):
    args, m, om = pair
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, args.vocab_size, 45)          # 2 passes of the 32-row kernel path
    cache = m.make_cache(128)
    logits = m(torch.from_numpy(prompt)[None], cache=cache)[0].cpu().numpy()
    oc = model_ref.make_prompt_cache(om, 128)
    want = om(prompt, oc)
    assert cache.offset == 45 == oc[0].offset
    # logits: stated tolerance |d| <= 2^-6 |want| + 2e-2 (fp16 activations through 2 layers)
    _close(logits, want, 2.0 ** -6, 2e-2)
    assert np.mean(logits.argmax(-1) == want.argmax(-1)) >= 0.9
    for li, c in enumerate(oc):
        _close(cache.data[li, 0, :, :45].cpu().numpy(), c.keys[0, :, :45], 2.0 ** -6, 2e-2)
        _close(cache.data[li, 1, :, :45].cpu().numpy(), c.values[0, :, :45], 2.0 ** -6, 2e-2)


def test_tree_decoding_with_golden_mask_matches_oracle(be, pair):
    args, m, om = pair
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, args.vocab_size, 70)          # prefix longer than one key block
    tokens = rng.integers(0, args.vocab_size, 8)
    mask_index = np.array([0, 1, 2, 2, 3, 4, 5])
    tm = np.eye(8, dtype=bool)
    for i in range(7):
        tm[i + 1] |= tm[mask_index[i]]
    pos = tm.sum(1) - 1
    cache = m.make_cache(192)
    m(torch.from_numpy(prompt)[None], cache=cache, logits_last_only=True)
    got = be.eagle.tree_decoding(torch.from_numpy(tokens)[None], torch.from_numpy(tm), torch.from_numpy(pos), m, cache)
    oc = model_ref.make_prompt_cache(om, 192)
    om(prompt, oc)
    want = eagle_ref.tree_decoding(tokens[None], tm, pos, om, oc)
    _close(got[0].cpu().numpy(), want, 2.0 ** -6, 2e-2)
    assert cache.offset == 78


def test_flat_rope_draft_level_call_matches_oracle(pair):
    """The draft-level call of generate_draft_tree: 8 tokens, one shared position, eye-block mask."""
    args, m, om = pair
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, args.vocab_size, 20)
    cache = m.make_cache(128)
    m(torch.from_numpy(prompt)[None], cache=cache, logits_last_only=True)
    oc = model_ref.make_prompt_cache(om, 128)
    om(prompt, oc)
    off = 20
    mask = np.full((8, off + 16), -np.inf, dtype=np.float32)
    mask[:, :off] = 0
    eye = np.where(np.eye(8, dtype=bool), 0, -np.inf)
    rows = None
    for i in range(2):
        toks = rng.integers(0, args.vocab_size, 8)
        mask[:, off + 8 * i: off + 8 * (i + 1)] = eye
        mm = mask[:, : off + 8 * (i + 1)]
        got = m(torch.from_numpy(toks)[None], cache=cache, mask=torch.from_numpy(mm)[None, None],
                position_ids=off + i, flat_rope=True)[0].cpu().numpy()
        want = om(toks, oc, mask=mm, position_ids=off + i, flat_rope=True)
        _close(got, want, 2.0 ** -6, 2e-2)
        out_ids = rng.integers(0, 8, 8)
        mask = mask[out_ids]


def test_call_rejects_what_it_cannot_do(be, pair):
    args, m, _ = pair
    cache = m.make_cache(64)
    with pytest.raises(be._lib.B200Error):
        m(torch.zeros(1, 4, dtype=torch.int64))                       # no cache
    with pytest.raises(be._lib.B200Error):
        m(torch.zeros(1, 80, dtype=torch.int64), cache=cache)         # cache too small
