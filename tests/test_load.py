"""Checkpoint ingestion (the counterpart of mlx_utils.py:59-181): an MLX-format 4-bit checkpoint written locally
is read back into an identical model; malformed checkpoints are refused."""
import json
import os

import numpy as np
import pytest
import torch


def _same(a, b):
    assert a.args == b.args
    for la, lb in zip(a.layers, b.layers):
        for k in ("qkv", "o", "gate", "up", "down"):
            for f in ("weight", "scales", "biases", "bias"):
                x, y = getattr(la[k], f), getattr(lb[k], f)
                assert (x is None) == (y is None)
                if x is not None:
                    assert torch.equal(x.cpu(), y.cpu())
        assert torch.equal(la["input_norm"].cpu(), lb["input_norm"].cpu())
        assert torch.equal(la["post_norm"].cpu(), lb["post_norm"].cpu())
    assert torch.equal(a.embed.weight.cpu(), b.embed.weight.cpu()) and torch.equal(a.norm.cpu(), b.norm.cpu())
    assert (a.lm_head is a.embed) == (b.lm_head is b.embed)
    if a.lm_head is not a.embed:
        assert torch.equal(a.lm_head.weight.cpu(), b.lm_head.weight.cpu())


@pytest.mark.parametrize("preset", ["tiny-qwen2", "tiny-llama"])
def test_checkpoint_round_trip_on_cpu(be, tmp_path, preset):
    args = be.shape_preset(preset)
    m = be.Model.random_init(args, seed=3, device="cpu")
    path = str(tmp_path / preset)
    be.load.save_mlx_checkpoint(m, path)
    cfg = json.load(open(os.path.join(path, "config.json")))
    assert cfg["quantization"] == {"group_size": 64, "bits": 4} and cfg["model_type"] == args.model_type
    names = be.load.read_safetensors(os.path.join(path, "model.safetensors"))
    assert names["model.layers.0.self_attn.q_proj.weight"].shape == (args.num_attention_heads * args.head_dim, args.hidden_size // 8)
    assert ("model.layers.0.self_attn.q_proj.bias" in names) == (preset == "tiny-qwen2")      # Qwen2 q/k/v biases
    assert ("lm_head.weight" in names) == (not args.tie_word_embeddings)
    m2, tok = be.load.load(path, "cpu")
    assert tok is None                                    # no tokenizer files in the directory
    _same(m, m2)


def test_bf16_scales_are_converted_and_bad_checkpoints_are_refused(be, tmp_path):
    args = be.shape_preset("tiny-llama")
    m = be.Model.random_init(args, seed=4, device="cpu")
    path = str(tmp_path / "bf16")
    be.load.save_mlx_checkpoint(m, path, dtype=torch.bfloat16)
    m2 = be.load.load_model(path, "cpu")
    want = m.layers[0]["qkv"].scales.to(torch.bfloat16).to(torch.float16)
    assert torch.equal(m2.layers[0]["qkv"].scales, want) and m2.layers[0]["qkv"].scales.dtype == torch.float16
    cfg = json.load(open(os.path.join(path, "config.json")))
    cfg["quantization"]["bits"] = 8
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    with pytest.raises(be._lib.B200Error):
        be.load.load_model(path, "cpu")
    cfg["quantization"]["bits"] = 4
    cfg["hidden_size"] = args.hidden_size * 2             # shapes no longer match the tensors
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    with pytest.raises(be._lib.B200Error):
        be.load.load_model(path, "cpu")
    with pytest.raises(FileNotFoundError):
        be.load.load(str(tmp_path / "missing"), "cpu")


@pytest.mark.gpu
def test_loaded_checkpoint_generates_like_the_model_it_was_written_from(be, cuda, tmp_path):
    args = be.shape_preset("tiny-qwen2")
    base = be.Model.random_init(args, seed=11, device=cuda, gen_device="cpu")
    draft = be.Model.random_init(args, seed=12, device=cuda, gen_device="cpu")
    for m in (base, draft):
        m.norm.mul_(8.0)
    be.load.save_mlx_checkpoint(base, str(tmp_path / "base"))
    be.load.save_mlx_checkpoint(draft, str(tmp_path / "draft"))
    base2, _ = be.load.load(str(tmp_path / "base"), cuda)
    draft2, _ = be.load.load(str(tmp_path / "draft"), cuda)
    prompt = torch.from_numpy(np.random.default_rng(5).integers(0, args.vocab_size, 25))
    want = be.generate_step(prompt, base.relayout(), draft.relayout(), depth=3, verify_num_tokens=15, max_tokens=24, N=24,
                            verbose=False)
    got = be.generate_step(prompt, base2.relayout(), draft2.relayout(), depth=3, verify_num_tokens=15, max_tokens=24, N=24,
                           verbose=False)
    assert got["tokens"] == want["tokens"] and got["accept_lengths"] == want["accept_lengths"]
