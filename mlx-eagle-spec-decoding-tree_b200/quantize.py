"""4-bit affine group quantisation in the MLX layout (torch, any device).

Produces what ``mx.quantize(w, group_size=64, bits=4)`` produces and what the
reference's kernels consume (``qmm_kernel.py:219-229``,
``kernels/progression/simd_no_swizzle_cast.metal:82-124``): ``uint32`` packs of
eight 4-bit codes (element j in bits 4j..4j+3), one fp16 scale and one fp16 bias
per 64 consecutive ``k`` of a row.  The packed tensor is returned as ``int32``
(same bits) because torch has no arithmetic on ``uint32``.
"""
from __future__ import annotations

import torch

GROUP_SIZE = 64
BITS = 4


def quantize(w: torch.Tensor, group_size: int = GROUP_SIZE, bits: int = BITS):
    if bits != 4 or group_size != 64:
        raise ValueError("only bits=4, group_size=64 is implemented")
    n, k = w.shape
    if k % group_size:
        raise ValueError("K must be a multiple of the group size")
    g = w.float().reshape(n, k // group_size, group_size)
    w_max = g.amax(-1)
    w_min = g.amin(-1)
    n_bins = float((1 << bits) - 1)
    mask = w_min.abs() > w_max.abs()
    scales = ((w_max - w_min) / n_bins).clamp_min(1e-7)
    scales = torch.where(mask, scales, -scales)
    edge = torch.where(mask, w_min, w_max)
    q0 = torch.round(edge / scales)
    scales = torch.where(q0 != 0, edge / torch.where(q0 != 0, q0, torch.ones_like(q0)), scales)
    biases = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    scales16 = scales.half()
    biases16 = biases.half()
    s = scales16.float().unsqueeze(-1)
    s = torch.where(s == 0, torch.full_like(s, 1e-7), s)
    q = torch.round((g - biases16.float().unsqueeze(-1)) / s).clamp_(0, n_bins).to(torch.int32)
    q = q.reshape(n, k // 8, 8)
    shifts = (4 * torch.arange(8, device=w.device, dtype=torch.int32)).view(1, 1, 8)
    packed = (q << shifts).sum(-1, dtype=torch.int64)          # disjoint bit fields: sum == or
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed.contiguous(), scales16.contiguous(), biases16.contiguous()


def dequantize(wq: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
               group_size: int = GROUP_SIZE) -> torch.Tensor:
    """fp16 weights ``(N, K)``; for building test inputs, not used by the decode path."""
    n = wq.shape[0]
    shifts = (4 * torch.arange(8, device=wq.device, dtype=torch.int32)).view(1, 1, 8)
    q = ((wq.to(torch.int32).unsqueeze(-1) >> shifts) & 0xF).reshape(n, -1).double()
    s = scales.double().repeat_interleave(group_size, dim=1)
    b = biases.double().repeat_interleave(group_size, dim=1)
    return (q * s + b).half()
