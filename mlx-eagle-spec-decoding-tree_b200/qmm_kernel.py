"""Batched 4-bit quantised matmul operator: same call as the reference's ``qmm_kernel.matmul``.

``matmul(x, w, s, b, group_size)`` (``qmm_kernel.py:84-98``) returns a list with
one array, which ``mlx_eagle.py:704-705`` unwraps as ``qmm(*args)[0]``; the same
convention is kept so a maintainer can swap the import.  Unlike the Metal
kernel this one takes any row count (1..32 in one pass, more in passes of 32),
not just 8/16/24/32.
"""
from __future__ import annotations

import ctypes
from functools import reduce

import torch

from . import _lib

EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_F32 = 0, 1, 2, 3
_WORKSPACE_BYTES = 32 << 20
_workspaces: dict = {}


def workspace(device) -> torch.Tensor:
    """Per-device scratch for split-K partial sums (zero-initialised once; the kernel re-zeroes
    the counters it uses).  Launches that share it must be ordered on one stream."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_WORKSPACE_BYTES, dtype=torch.uint8, device=f"cuda:{key}")
        _workspaces[key] = ws
    return ws


def _check_operands(x, w, s, b, group_size):
    _lib.require_cuda(x, w, s, b)
    if x.dtype != torch.float16 or s.dtype != torch.float16 or b.dtype != torch.float16:
        raise _lib.B200Error("x, scales and biases must be float16 (the reference kernel is fp16-only, "
                             "simd_no_swizzle_cast.metal:55-64)")
    if w.dtype not in (torch.int32, torch.uint32):
        raise _lib.B200Error("packed weights must be int32/uint32")
    k = x.shape[-1]
    # the reference asserts this at mlx_model_fwd_bench.py:68
    assert (k % 128) == 0, "K must be a multiple of 128"
    if w.shape[1] * 8 != k or s.shape != (w.shape[0], k // group_size) or b.shape != s.shape:
        raise _lib.B200Error("weight / scale / bias shapes do not match x")


def matmul(x, w, s, b, group_size=64, d_dtype=torch.float16, bias=None, **_ignored):
    """``[x @ dequant(w, s, b).T]`` with x ``(*B, K)`` fp16 and w ``(N, K/8)`` packed 4-bit."""
    _check_operands(x, w, s, b, group_size)
    if d_dtype != torch.float16:
        raise _lib.B200Error("only float16 output is implemented")
    *lead, k = x.shape
    m = reduce(lambda a, c: a * c, lead, 1)
    n = w.shape[0]
    x2 = x.reshape(m, k).contiguous()
    y = torch.empty((m, n), dtype=torch.float16, device=x.device)
    ws = workspace(x.device)
    rc = _lib.lib().b200_qmm(_lib.ptr(x2), _lib.ptr(w), _lib.ptr(s), _lib.ptr(b), _lib.ptr(bias),
                             _lib.ptr(y), m, n, k, group_size, 0, _lib.ptr(ws), ws.numel(),
                             _lib.stream_ptr(x.device))
    _lib.check(rc, "b200_qmm")
    return [y.reshape(*lead, n)]


def matmul_fused(x, w, s, b, *, epilogue=EPI_NONE, w2=None, s2=None, b2=None, bias=None,
                 extra=None, out=None, group_size=64):
    """Product plus the element-wise op that follows it in the model (bias, residual add, or
    SiLU(gate)*up with ``(w, s, b)`` = gate_proj and ``(w2, s2, b2)`` = up_proj).  At most 32 rows."""
    _check_operands(x, w, s, b, group_size)
    m, k = x.shape
    n = w.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    ws = workspace(x.device)
    rc = _lib.lib().b200_qmm_fused(_lib.ptr(x), _lib.ptr(w), _lib.ptr(s), _lib.ptr(b), _lib.ptr(w2),
                                   _lib.ptr(s2), _lib.ptr(b2), _lib.ptr(bias), _lib.ptr(extra),
                                   _lib.ptr(y), m, n, k, group_size, 0, epilogue, _lib.ptr(ws),
                                   ws.numel(), _lib.stream_ptr(x.device))
    _lib.check(rc, "b200_qmm_fused")
    return y


def workspace_bytes(m: int, n: int, k: int) -> int:
    return int(_lib.lib().b200_qmm_workspace_bytes(m, n, k))


def relayout(w, s, b) -> torch.Tensor:
    """One-off re-layout of MLX-format 4-bit weights into the streaming ("tiled") layout the fast
    kernel reads: records of 16 rows x 128 k, lane-ordered packs followed by {scale, bias} pairs.
    The counterpart of the reference's offline ``swizzle`` (``swizzle.py:41-57``).  Returns a uint8
    tensor; ``matmul_tiled`` consumes it."""
    _lib.require_cuda(w, s, b)
    n, k = w.shape[0], w.shape[1] * 8
    out = torch.empty(_lib.lib().b200_qmm_tiled_bytes(n, k), dtype=torch.uint8, device=w.device)
    rc = _lib.lib().b200_qmm_relayout(_lib.ptr(w), _lib.ptr(s), _lib.ptr(b), _lib.ptr(out), n, k,
                                      _lib.stream_ptr(w.device))
    _lib.check(rc, "b200_qmm_relayout")
    return out


def matmul_tiled(x, wt, n, *, epilogue=EPI_NONE, wt2=None, bias=None, extra=None, out=None):
    """``x (M<=32, K) @ W.T`` on re-laid-out weights ``wt`` (from ``relayout``) of ``n`` output rows."""
    _lib.require_cuda(x, wt)
    m, k = x.shape
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    ws = workspace(x.device)
    rc = _lib.lib().b200_qmm_tiled(_lib.ptr(x), _lib.ptr(wt), _lib.ptr(wt2), _lib.ptr(bias), _lib.ptr(extra),
                                   _lib.ptr(y), m, n, k, epilogue, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device))
    _lib.check(rc, "b200_qmm_tiled")
    return y


def stream_error(device) -> int:
    """Non-zero if a bounded wait inside the tiled kernel ever gave up on this device (reads the flag)."""
    return int(workspace(device)[4092:4096].view(torch.int32).item())


_umma_ws = {}


def matmul_umma(x, wt, n, *, bias=None, out=None):
    """``x (M<=128, K) @ W.T`` on re-laid-out weights ``wt`` through the tcgen05 tensor cores
    (``b200_qmm_umma``; ``n`` and K multiples of 128, plain epilogue)."""
    _lib.require_cuda(x, wt)
    m, k = x.shape
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    need = _lib.lib().b200_qmm_umma_workspace_bytes(m, k)
    if need == 0:
        raise _lib.B200Error("b200_qmm_umma: need 1 <= M <= 128 and K a multiple of 128")
    key = (x.device, torch.cuda.current_stream(x.device).cuda_stream)
    ws = _umma_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=x.device)
        _umma_ws[key] = ws
    rc = _lib.lib().b200_qmm_umma(_lib.ptr(x), _lib.ptr(wt), _lib.ptr(bias), _lib.ptr(y), m, n, k, _lib.ptr(ws),
                                  ws.numel(), _lib.stream_ptr(x.device))
    _lib.check(rc, "b200_qmm_umma")
    return y


def umma_error(device) -> int:
    """Non-zero if a bounded wait inside the tcgen05 kernel ever gave up on this device's current stream."""
    ws = _umma_ws.get((device, torch.cuda.current_stream(device).cuda_stream))
    return 0 if ws is None else int(ws[:4].view(torch.int32).item())
