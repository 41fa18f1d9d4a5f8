"""Deterministic exp / log / log-sum-exp used for the draft tree's log-probabilities.

Test infrastructure (CPU oracle).  The reference computes
``softmax(logits).log()`` (``mlx_eagle.py:104``) and ``logits - logsumexp``
(``mlx_eagle.py:410-412``) with MLX ops whose rounding is not specified.  The
tree decisions (top-k, rescoring, node selection) depend on these values, so the
restatement fixes an arithmetic that a CPU and a GPU reproduce bit for bit:

* ``exp_det`` / ``log_det`` use only IEEE-754 double add, multiply, divide,
  round-to-nearest-even, ``frexp`` and ``ldexp`` - every one rounded separately
  (no fused multiply-add) - so any conforming machine gets identical bits;
* the sum of exponentials is taken in 2^-40 fixed point with integer addition,
  which is associative: the order in which a parallel machine adds does not matter.

``log_probs(logits)`` returns ``float32(logit - lse)`` per element.
"""
from __future__ import annotations

import numpy as np

LOG2E = 1.4426950408889634
LN2_HI = 6.93147180369123816490e-01   # ln 2 with the low 21 bits zero: k*LN2_HI is exact for |k| < 2^20
LN2_LO = 1.90821492927058770002e-10
FIX_BITS = 40
EXP_CUTOFF = -40.0                      # exp(d) * 2^40 < 0.5 below this; contributes 0
_EXP_COEF = [1.0 / float(np.prod(np.arange(1, n + 1, dtype=np.float64))) for n in range(0, 14)]
_LOG_COEF = [1.0 / (2 * n + 1) for n in range(0, 12)]


def exp_det(d: np.ndarray) -> np.ndarray:
    """exp(d) for d <= 0 (float64 in, float64 out), identical on CPU and GPU; 0 for d < -40."""
    d = np.asarray(d, dtype=np.float64)
    dd = np.maximum(d, EXP_CUTOFF)
    kf = np.rint(dd * LOG2E)
    r = (dd - kf * LN2_HI) - kf * LN2_LO
    p = np.full_like(r, _EXP_COEF[13])
    for c in _EXP_COEF[12::-1]:
        p = p * r + c
    out = np.ldexp(p, kf.astype(np.int32))
    return np.where(d < EXP_CUTOFF, 0.0, out)


def exp_fixed(d: np.ndarray) -> np.ndarray:
    """round-to-nearest-even(exp_det(d) * 2^40) as int64."""
    return np.rint(np.ldexp(exp_det(d), FIX_BITS)).astype(np.int64)


def log_det(total: np.ndarray) -> np.ndarray:
    """ln(total * 2^-40) for positive integer ``total`` (sum of ``exp_fixed``)."""
    sd = np.asarray(total).astype(np.uint64).astype(np.float64)
    f, e = np.frexp(sd)
    small = f < 0.70710678118654752440
    f = np.where(small, f * 2.0, f)
    e = np.where(small, e - 1, e).astype(np.float64) - float(FIX_BITS)
    s = (f - 1.0) / (f + 1.0)
    z = s * s
    q = np.full_like(z, _LOG_COEF[11])
    for c in _LOG_COEF[10::-1]:
        q = q * z + c
    lnf = (2.0 * s) * q
    return e * LN2_HI + (e * LN2_LO + lnf)


def logsumexp(logits: np.ndarray) -> np.ndarray:
    """Row-wise log-sum-exp (float64) of fp16 logits, last axis."""
    x = np.asarray(logits).astype(np.float64)
    m = x.max(axis=-1, keepdims=True)
    total = exp_fixed(x - m).sum(axis=-1, keepdims=True, dtype=np.int64)
    return (m + log_det(total))[..., 0]


def log_probs(logits: np.ndarray) -> np.ndarray:
    """``float32(logit - lse)``: the log-softmax the tree scores are built from."""
    x = np.asarray(logits).astype(np.float64)
    lse = logsumexp(logits)[..., None]
    return (x - lse).astype(np.float32)
