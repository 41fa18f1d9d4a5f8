"""Tree-position RoPE operator with the reference's call signature.

``rope_positions(inp, offsets, inv_freqs, scaling_factor)`` follows
``mlx_arrayed_rope_kernel.py:46-152``: ``inp`` is ``(B, H, L, D)``, ``offsets`` holds
one integer position per (batch, token), ``inv_freqs`` is ``(D/2,)`` fp32; layout is
non-traditional (element i pairs with i + D/2), math in fp32, output in the input
dtype.  Inside the decode loop the same rotation runs fused with the KV-cache
append (``b200_rope_kv_append``); this stand-alone form is the drop-in operator.
"""
from __future__ import annotations

import torch

from . import _lib


def rope_positions(inp: torch.Tensor, offsets: torch.Tensor, inv_freqs: torch.Tensor, scaling_factor: float = 1.0,
                   verbose: bool = False) -> torch.Tensor:
    _lib.require_cuda(inp, offsets, inv_freqs)
    if inp.dtype != torch.float16 or inp.dim() != 4:
        raise _lib.B200Error("rope_positions expects a float16 (B, H, L, D) tensor")
    B, H, L, D = inp.shape
    if offsets.numel() != B * L or inv_freqs.numel() != D // 2:
        raise _lib.B200Error("offsets must be (B, L) and inv_freqs (D/2,)")
    x = inp.contiguous()
    out = torch.empty_like(x)
    rc = _lib.lib().b200_rope_positions(_lib.ptr(x), _lib.ptr(offsets.to(torch.int32).contiguous()),
                                        _lib.ptr(inv_freqs.float().contiguous()), float(scaling_factor),
                                        _lib.ptr(out), B, H, L, D, _lib.stream_ptr(inp.device))
    _lib.check(rc, "b200_rope_positions")
    return out
