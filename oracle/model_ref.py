"""CPU restatement (numpy + the C matmul) of the reference's Llama/Qwen2 forward with tree hooks.

Test infrastructure.  Follows ``mlx_llama.py``:

* ``Attention.__call__`` (``:121-196``): q/k/v projections (+bias for Qwen2), reshape to heads, RoPE
  either at per-token array positions (``rope_positions``, ``mlx_arrayed_rope_kernel.py:60-123``) or
  at an integer offset, with ``flat_rope`` giving every token the same position (``:141-143``),
  cache append (``:178``), softmax(q k^T * scale + mask) v with grouped KV heads (``:185-192``),
  output projection;
* ``MLP`` (``:214-215``), ``TransformerBlock`` (``:231-249``), ``LlamaModel`` (``:265-286``),
  ``Model`` (``:298-313``, tied head = the quantised embedding used as a linear layer).

Numerics (MLX's own are unavailable): every op result is rounded to fp16, as in an fp16 MLX
graph; inside an op the math is fp32 (RMSNorm, RoPE, attention scores/softmax, matmul
accumulation).  Token ids beyond the embedding table are clamped to the last row.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np

from . import qmm_c, qmm_ref

f16, f32, f64 = np.float16, np.float32, np.float64


class OracleKVCache:
    """One layer's ``(1, Hkv, rows, hd)`` keys / values and the number of rows in use."""

    def __init__(self, n_kv: int, hd: int, rows: int):
        self.keys = np.zeros((1, n_kv, rows, hd), dtype=f16)
        self.values = np.zeros((1, n_kv, rows, hd), dtype=f16)
        self.offset = 0

    def update_and_fetch(self, k, v):
        L = k.shape[2]
        self.keys[:, :, self.offset:self.offset + L] = k
        self.values[:, :, self.offset:self.offset + L] = v
        self.offset += L
        return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]


def make_prompt_cache(model: "OracleModel", rows: int) -> List[OracleKVCache]:
    a = model.args
    return [OracleKVCache(a.num_key_value_heads, a.head_dim, rows) for _ in range(a.num_hidden_layers)]


def rms_norm(x, w, eps):
    xf = x.astype(f32)
    inv = f32(1.0) / np.sqrt((xf * xf).mean(axis=-1, keepdims=True, dtype=f32) + f32(eps))
    return ((xf * inv) * w.astype(f32)).astype(f16)


def rope_positions(x, positions, inv_freqs, scaling_factor):
    """x ``(B,H,L,D)`` fp16, positions ``(B,L)`` int; half-split layout, fp32 math."""
    D = x.shape[-1]
    theta = (f32(scaling_factor) * inv_freqs.astype(f32))[None, None, None, :] * \
        positions.astype(f32)[:, None, :, None]
    c, s = np.cos(theta, dtype=f32), np.sin(theta, dtype=f32)
    x1, x2 = x[..., : D // 2].astype(f32), x[..., D // 2:].astype(f32)
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1).astype(f16)


def half_add(a, b):
    return (a.astype(f64) + b.astype(f64)).astype(f16)


def half_mul(a, b):
    return (a.astype(f64) * b.astype(f64)).astype(f16)


def silu_mul(gate, up):
    sig = (f32(1.0) / (f32(1.0) + np.exp(-gate.astype(f32)))).astype(f16)
    return half_mul(half_mul(gate, sig), up)


class OracleLinear:
    def __init__(self, d):
        self.w, self.s, self.b, self.bias = d["weight"], d["scales"], d["biases"], d.get("bias")

    def __call__(self, x):
        return qmm_c.qmm(x, self.w, self.s, self.b, 64, bias=self.bias)


class OracleModel:
    """Built from ``Model.state_numpy()`` of the product so both sides hold identical weights."""

    def __init__(self, args, state: dict):
        self.args = args
        self.embed = state["embed"]
        self.layers = []
        for L in state["layers"]:
            self.layers.append(dict(qkv=OracleLinear(L["qkv"]), o=OracleLinear(L["o"]), gate=OracleLinear(L["gate"]),
                                    up=OracleLinear(L["up"]), down=OracleLinear(L["down"]),
                                    input_norm=L["input_norm"], post_norm=L["post_norm"]))
        self.norm = state["norm"]
        self.lm_head = OracleLinear(state["lm_head"] if state["lm_head"] is not None else state["embed"])
        self.inv_freqs = state["inv_freqs"]
        self.scaling = state["rope_scaling_factor"]

    def embed_tokens(self, ids):
        e = self.embed
        ids = np.clip(np.asarray(ids).reshape(-1), 0, e["weight"].shape[0] - 1)
        return qmm_ref.dequantize(e["weight"][ids], e["scales"][ids], e["biases"][ids])

    def _attention(self, lw, x, mask, cache, position_ids, flat_rope):
        a = self.args
        L = x.shape[0]
        Hq, Hkv, hd = a.num_attention_heads, a.num_key_value_heads, a.head_dim
        qkv = lw["qkv"](x)
        q = qkv[:, : Hq * hd].reshape(1, L, Hq, hd).transpose(0, 2, 1, 3)
        k = qkv[:, Hq * hd: (Hq + Hkv) * hd].reshape(1, L, Hkv, hd).transpose(0, 2, 1, 3)
        v = qkv[:, (Hq + Hkv) * hd:].reshape(1, L, Hkv, hd).transpose(0, 2, 1, 3)
        if isinstance(position_ids, np.ndarray):
            pos = position_ids.reshape(1, L)
        else:
            base = cache.offset if position_ids is None else int(position_ids)
            pos = (np.full((1, L), base) if flat_rope else base + np.arange(L)[None]).astype(np.int64)
        q = rope_positions(q, pos, self.inv_freqs, self.scaling)
        k = rope_positions(k, pos, self.inv_freqs, self.scaling)
        keys, values = cache.update_and_fetch(k, v)
        G = Hq // Hkv
        out = np.zeros((L, Hq, hd), dtype=f16)
        scale = f32(hd ** -0.5)
        for h in range(Hq):
            kk = keys[0, h // G].astype(f32)
            vv = values[0, h // G].astype(f32)
            s = (q[0, h].astype(f32) @ kk.T) * scale + mask
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p = p / p.sum(axis=-1, keepdims=True, dtype=f32)
            out[:, h] = (p.astype(f32) @ vv).astype(f16)
        return lw["o"](out.reshape(L, Hq * hd))

    def __call__(self, inputs, cache: List[OracleKVCache], mask: Optional[np.ndarray] = None,
                 position_ids=None, flat_rope: bool = False) -> np.ndarray:
        """``inputs (L,)`` -> logits ``(L, V)`` fp16; ``mask`` additive ``(L, cache.offset + L)`` or None
        (causal, what ``create_attention_mask`` gives with a cache)."""
        ids = np.asarray(inputs).reshape(-1)
        L = ids.shape[0]
        h = self.embed_tokens(ids)
        off = cache[0].offset
        if mask is None:
            m = np.zeros((L, off + L), dtype=f32)
            m[:, off:] = np.where(np.tril(np.ones((L, L), dtype=bool)), 0.0, -np.inf)
            mask = m
        mask = mask.astype(f16).astype(f32)          # mask.astype(h.dtype), mlx_llama.py:278
        for lw, c in zip(self.layers, cache):
            r = self._attention(lw, rms_norm(h, lw["input_norm"], self.args.rms_norm_eps), mask, c,
                                position_ids, flat_rope)
            h = half_add(h, r)
            x = rms_norm(h, lw["post_norm"], self.args.rms_norm_eps)
            r = lw["down"](silu_mul(lw["gate"](x), lw["up"](x)))
            h = half_add(h, r)
        return self.lm_head(rms_norm(h, self.norm, self.args.rms_norm_eps))
