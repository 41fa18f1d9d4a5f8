"""Checkpoint ingestion: MLX-format 4-bit checkpoints -> ``llama.Model``.

The counterpart of the reference's ``mlx_utils.py:59-181`` (``load_model`` / ``load``): a directory with
``config.json`` (Hugging Face keys plus ``"quantization": {"group_size": 64, "bits": 4}``) and
``model*.safetensors`` (``weight*.safetensors`` for old exports, ``mlx_utils.py:90-96``) whose quantised
linear layers and the embedding are stored the way ``mx.quantize`` / ``nn.QuantizedLinear`` lay them out:

    <name>.weight   uint32 [N, K/8]    element j of a pack in bits 4j..4j+3
    <name>.scales   fp16/bf16 [N, K/64]
    <name>.biases   fp16/bf16 [N, K/64]
    <name>.bias     fp16/bf16 [N]       (Qwen2 q/k/v projections)

with the Hugging Face module names (``model.embed_tokens``, ``model.layers.<i>.self_attn.{q,k,v,o}_proj``,
``model.layers.<i>.mlp.{gate,up,down}_proj``, ``model.layers.<i>.{input,post_attention}_layernorm``,
``model.norm``, ``lm_head``).  q, k and v become one fused matrix here.  Everything is checked against the
configuration before it is used; an unsupported checkpoint raises instead of loading wrongly.  The kernels of
this library are fp16: bf16 scales, biases and norm weights are converted (rounded) to fp16.

There is no network access where this was written, so the tests write a checkpoint in this layout themselves
(``save_mlx_checkpoint``) and read it back.  The safetensors container is parsed here directly (8-byte
little-endian header length, JSON header, raw little-endian tensor data), so no extra package is needed.
"""
from __future__ import annotations

import glob
import json
import os
import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib
from .llama import Model, ModelArgs, QLinear

_DTYPES = {"U32": (np.uint32, 4), "I32": (np.int32, 4), "F16": (np.float16, 2), "F32": (np.float32, 4),
           "BF16": (np.uint16, 2), "U8": (np.uint8, 1), "I64": (np.int64, 8)}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one ``.safetensors`` file as CPU torch tensors (uint32 packs come back as int32 bit
    patterns, bf16 as torch.bfloat16)."""
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise _lib.B200Error(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or n > (1 << 30):
            raise _lib.B200Error(f"{path}: implausible safetensors header length {n}")
        header = json.loads(f.read(n).decode("utf-8"))
        base = 8 + n
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = meta["dtype"]
            if dt not in _DTYPES:
                raise _lib.B200Error(f"{path}: tensor {name} has unsupported dtype {dt}")
            npdt, size = _DTYPES[dt]
            lo, hi = meta["data_offsets"]
            shape = tuple(meta["shape"])
            count = int(np.prod(shape)) if shape else 1
            if hi - lo != count * size:
                raise _lib.B200Error(f"{path}: tensor {name}: {hi - lo} bytes for shape {shape} of {dt}")
            f.seek(base + lo)
            arr = np.frombuffer(f.read(hi - lo), dtype=npdt).reshape(shape).copy()
            if dt == "BF16":
                t = torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
            elif dt == "U32":
                t = torch.from_numpy(arr.view(np.int32))
            else:
                t = torch.from_numpy(arr)
            out[name] = t
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Writes CPU tensors (int32 is stored as U32: the packed weights) in the safetensors container."""
    names = {torch.int32: "U32", torch.float16: "F16", torch.float32: "F32", torch.bfloat16: "BF16"}
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in names:
            raise _lib.B200Error(f"cannot write {name} of dtype {t.dtype}")
        raw = t.view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for raw in blobs:
            f.write(raw)


def _args_from_config(config: dict) -> ModelArgs:
    known = {f for f in ModelArgs.__dataclass_fields__}
    args = ModelArgs(**{k: v for k, v in config.items() if k in known})          # ModelArgs.from_dict of the reference
    if config.get("model_type") == "qwen2":
        args.attention_bias = True                                               # mlx_utils.py:116-117
    return args


def _f16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).contiguous()


def load_model(model_path: str, device, model_config: Optional[dict] = None) -> Model:
    """``mlx_utils.load_model`` (``:59-141``) for this library: reads ``config.json`` and every weight file of
    the directory and returns a ``Model`` on ``device`` (row-major packed weights; call ``relayout()`` for the
    persistent-kernel path)."""
    with open(os.path.join(model_path, "config.json")) as f:
        config = json.load(f)
    config.update(model_config or {})
    q = config.get("quantization")
    if not q or int(q.get("bits", 0)) != 4 or int(q.get("group_size", 0)) != 64:
        raise _lib.B200Error("only 4-bit / group-64 quantised checkpoints are supported (config.json: quantization)")
    if config.get("model_type") not in ("llama", "qwen2"):
        raise _lib.B200Error(f"no implementation for model architecture {config.get('model_type')!r}")
    files = sorted(glob.glob(os.path.join(model_path, "model*.safetensors"))) or \
        sorted(glob.glob(os.path.join(model_path, "weight*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors found in {model_path}")
    w: Dict[str, torch.Tensor] = {}
    for wf in files:
        w.update(read_safetensors(wf))
    w = {k: v for k, v in w.items() if "rotary_emb.inv_freq" not in k}            # Model.sanitize of the reference
    args = _args_from_config(config)
    dev = torch.device(device)
    H, I, hd = args.hidden_size, args.intermediate_size, args.head_dim
    nq, nkv = args.num_attention_heads * hd, args.num_key_value_heads * hd

    def lin(prefix: str, n: int, k: int, bias: bool = False) -> Tuple[torch.Tensor, ...]:
        for part in ("weight", "scales", "biases"):
            if f"{prefix}.{part}" not in w:
                raise _lib.B200Error(f"checkpoint has no {prefix}.{part} (is the layer quantised?)")
        wq, s, b = w[f"{prefix}.weight"], w[f"{prefix}.scales"], w[f"{prefix}.biases"]
        if wq.dtype != torch.int32 or tuple(wq.shape) != (n, k // 8) or tuple(s.shape) != (n, k // 64) or s.shape != b.shape:
            raise _lib.B200Error(f"{prefix}: expected packed [{n}, {k // 8}] with scales [{n}, {k // 64}], "
                                 f"found {tuple(wq.shape)} / {tuple(s.shape)}")
        bv = None
        if bias:
            if f"{prefix}.bias" not in w:
                raise _lib.B200Error(f"checkpoint has no {prefix}.bias")
            bv = _f16(w[f"{prefix}.bias"])
        return wq.contiguous(), _f16(s), _f16(b), bv

    def qlinear(parts) -> QLinear:
        wq = torch.cat([p[0] for p in parts]).to(dev)
        s = torch.cat([p[1] for p in parts]).to(dev)
        b = torch.cat([p[2] for p in parts]).to(dev)
        bias = torch.cat([p[3] for p in parts]).to(dev) if parts[0][3] is not None else None
        return QLinear(wq, s, b, bias)

    layers = []
    for i in range(args.num_hidden_layers):
        pre = f"model.layers.{i}"
        ab = args.attention_bias
        layers.append(dict(
            qkv=qlinear([lin(f"{pre}.self_attn.q_proj", nq, H, ab), lin(f"{pre}.self_attn.k_proj", nkv, H, ab),
                         lin(f"{pre}.self_attn.v_proj", nkv, H, ab)]),
            o=qlinear([lin(f"{pre}.self_attn.o_proj", H, nq)]),
            gate=qlinear([lin(f"{pre}.mlp.gate_proj", I, H)]), up=qlinear([lin(f"{pre}.mlp.up_proj", I, H)]),
            down=qlinear([lin(f"{pre}.mlp.down_proj", H, I)]),
            input_norm=_f16(w[f"{pre}.input_layernorm.weight"]).to(dev),
            post_norm=_f16(w[f"{pre}.post_attention_layernorm.weight"]).to(dev)))
    embed = qlinear([lin("model.embed_tokens", args.vocab_size, H)])
    lm_head = None if args.tie_word_embeddings else qlinear([lin("lm_head", args.vocab_size, H)])
    return Model(args, layers, embed, _f16(w["model.norm.weight"]).to(dev), lm_head, dev)


def load(path: str, device, tokenizer_config: Optional[dict] = None, model_config: Optional[dict] = None):
    """``mlx_utils.load`` (``:144-181``): ``(model, tokenizer)``.  ``path`` must be a local directory (nothing is
    downloaded).  The tokenizer comes from ``transformers`` when the directory holds tokenizer files, else None."""
    if not os.path.isdir(path):
        raise FileNotFoundError(f"{path}: not a local checkpoint directory (downloads are not supported here)")
    model = load_model(path, device, model_config)
    tokenizer = None
    if any(os.path.exists(os.path.join(path, n)) for n in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(path, **(tokenizer_config or {}))
    return model, tokenizer


def save_mlx_checkpoint(model: Model, path: str, dtype: torch.dtype = torch.float16) -> None:
    """Writes ``model`` (row-major weights still present) as an MLX-format checkpoint directory; the inverse of
    ``load_model``.  ``dtype`` is the type of scales, biases and norm weights in the file (fp16 or bf16)."""
    a = model.args
    os.makedirs(path, exist_ok=True)
    hd = a.head_dim
    nq, nkv = a.num_attention_heads * hd, a.num_key_value_heads * hd
    t: Dict[str, torch.Tensor] = {}

    def put(prefix: str, lin: QLinear, r0: int = 0, r1: Optional[int] = None):
        if lin.weight is None:
            raise _lib.B200Error("save_mlx_checkpoint needs the row-major weights (call it before relayout())")
        r1 = lin.out_features if r1 is None else r1
        t[f"{prefix}.weight"] = lin.weight[r0:r1].cpu()
        t[f"{prefix}.scales"] = lin.scales[r0:r1].cpu().to(dtype)
        t[f"{prefix}.biases"] = lin.biases[r0:r1].cpu().to(dtype)
        if lin.bias is not None:
            t[f"{prefix}.bias"] = lin.bias[r0:r1].cpu().to(dtype)

    for i, lw in enumerate(model.layers):
        pre = f"model.layers.{i}"
        put(f"{pre}.self_attn.q_proj", lw["qkv"], 0, nq)
        put(f"{pre}.self_attn.k_proj", lw["qkv"], nq, nq + nkv)
        put(f"{pre}.self_attn.v_proj", lw["qkv"], nq + nkv, nq + 2 * nkv)
        put(f"{pre}.self_attn.o_proj", lw["o"])
        put(f"{pre}.mlp.gate_proj", lw["gate"])
        put(f"{pre}.mlp.up_proj", lw["up"])
        put(f"{pre}.mlp.down_proj", lw["down"])
        t[f"{pre}.input_layernorm.weight"] = lw["input_norm"].cpu().to(dtype)
        t[f"{pre}.post_attention_layernorm.weight"] = lw["post_norm"].cpu().to(dtype)
    put("model.embed_tokens", model.embed)
    if model.lm_head is not model.embed:
        put("lm_head", model.lm_head)
    t["model.norm.weight"] = model.norm.cpu().to(dtype)
    write_safetensors(os.path.join(path, "model.safetensors"), t)
    config = {k: getattr(a, k) for k in ModelArgs.__dataclass_fields__}
    config["quantization"] = {"group_size": 64, "bits": 4}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
