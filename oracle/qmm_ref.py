"""CPU restatement of the reference's batched 4-bit affine quantised matmul.

Test infrastructure: only tests, the smoke check and the CPU-baseline legs of
the benchmark may import this file.

Follows ``kernels/progression/simd_no_swizzle_cast.metal``:

* packing (``:82,96,110,124``): one ``uint32`` holds 8 consecutive ``k``
  values of one weight row, element ``j`` in bits ``4j .. 4j+3``;
* one fp16 scale and one fp16 bias per 64 consecutive ``k`` of a row
  (``:63-64,76-77,154-155``);
* dequantisation in half precision, ``half(q) * s + b`` (``:83,97,111,125``) -
  restated as a single rounding of the exact value to fp16 (the shader is built
  with Metal's default fast-math, where the multiply-add contracts);
* fp16 x fp16 products accumulated in fp32 (``:66-68,93``), result cast to fp16
  (``:236-241``).  The shader's k-order (a permutation of K shared by both
  operands) only changes the fp32 summation order, which the tolerance covers.

``qmm_gold`` accumulates the same products in fp64 and is what tolerances are
stated against.
"""
from __future__ import annotations

import numpy as np

GROUP_SIZE = 64
PACK = 8  # 4-bit values per uint32


def unpack_nibbles(wq: np.ndarray) -> np.ndarray:
    """``(N, K/8) uint32 -> (N, K) uint8`` with element j of a pack in bits 4j..4j+3."""
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    shifts = (4 * np.arange(PACK, dtype=np.uint32))[None, None, :]
    q = (wq[:, :, None] >> shifts) & np.uint32(0xF)
    return q.reshape(wq.shape[0], wq.shape[1] * PACK).astype(np.uint8)


def dequantize(wq: np.ndarray, scales: np.ndarray, biases: np.ndarray,
               group_size: int = GROUP_SIZE, dtype=np.float16) -> np.ndarray:
    """Dequantised weights ``(N, K)`` rounded once to ``dtype`` (exact q*s+b in fp64 first)."""
    q = unpack_nibbles(wq).astype(np.float64)
    s = np.repeat(scales.astype(np.float64), group_size, axis=1)
    b = np.repeat(biases.astype(np.float64), group_size, axis=1)
    return (q * s + b).astype(dtype)


def qmm(x: np.ndarray, wq: np.ndarray, scales: np.ndarray, biases: np.ndarray,
        group_size: int = GROUP_SIZE, bias: np.ndarray | None = None) -> np.ndarray:
    """``y = x @ dequant(W).T`` with fp32 accumulation, fp16 result; ``+ bias`` afterwards in fp16.

    The bias add after the kernel follows ``mlx_model_fwd_bench.py:69-71``.
    """
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    w = dequantize(wq, scales, biases, group_size).astype(np.float32)
    y = (x2.astype(np.float32) @ w.T).astype(np.float16)
    if bias is not None:
        y = (y.astype(np.float64) + bias.astype(np.float64)[None, :]).astype(np.float16)
    return y.reshape(*lead, wq.shape[0])


def qmm_gold(x: np.ndarray, wq: np.ndarray, scales: np.ndarray, biases: np.ndarray,
             group_size: int = GROUP_SIZE) -> np.ndarray:
    """Same products summed in fp64 (no final rounding): the yardstick for tolerances."""
    x2 = x.reshape(-1, x.shape[-1])
    w = dequantize(wq, scales, biases, group_size).astype(np.float64)
    return x2.astype(np.float64) @ w.T


def quantize(w: np.ndarray, group_size: int = GROUP_SIZE, bits: int = 4):
    """Affine 4-bit quantiser producing the layout above (min/max per group, MLX's edge rule).

    Not on the parity path: oracle and GPU always consume the same packed
    tensors.  The edge rule (scale sign chosen so that the group's
    larger-magnitude end is represented exactly) is the published MLX
    ``quantize`` recipe that ``qmm_kernel.py:219-229`` calls.
    """
    assert bits == 4
    n, k = w.shape
    assert k % group_size == 0
    g = w.astype(np.float32).reshape(n, k // group_size, group_size)
    w_max = g.max(-1)
    w_min = g.min(-1)
    n_bins = float((1 << bits) - 1)
    mask = np.abs(w_min) > np.abs(w_max)
    scales = np.maximum((w_max - w_min) / n_bins, 1e-7)
    scales = np.where(mask, scales, -scales)
    edge = np.where(mask, w_min, w_max)
    q0 = np.rint(edge / scales)
    scales = np.where(q0 != 0, edge / np.where(q0 != 0, q0, 1.0), scales)
    biases = np.where(q0 == 0, 0.0, edge)
    scales16 = scales.astype(np.float16)
    biases16 = biases.astype(np.float16)
    s = scales16.astype(np.float32)[..., None]
    b = biases16.astype(np.float32)[..., None]
    s = np.where(s == 0, np.float32(1e-7), s)
    q = np.clip(np.rint((g - b) / s), 0, n_bins).astype(np.uint32).reshape(n, k // PACK, PACK)
    shifts = (4 * np.arange(PACK, dtype=np.uint32))[None, None, :]
    wq = np.bitwise_or.reduce(q << shifts, axis=-1).astype(np.uint32)
    return wq, scales16, biases16
