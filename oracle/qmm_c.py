"""ctypes binding of the C oracle (``qmm_cpu.c``); test infrastructure only."""
from __future__ import annotations

import ctypes

import numpy as np

from .build import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_oracle())
        _lib.oracle_qmm_f16.restype = ctypes.c_int
        _lib.oracle_qmm_f16.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 5
        _lib.oracle_f64_to_f16.restype = ctypes.c_uint16
        _lib.oracle_f64_to_f16.argtypes = [ctypes.c_double]
        _lib.oracle_num_threads.restype = ctypes.c_int
        _lib.oracle_set_num_threads.restype = None
        _lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def qmm(x, wq, scales, biases, group_size=64, bias=None, nthreads=0):
    """``y = x @ dequant(W).T`` (fp16 in/out, fp32 accumulate) on the host cores."""
    lead = x.shape[:-1]
    x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]), dtype=np.float16)
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    biases = np.ascontiguousarray(biases, dtype=np.float16)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float16)
    m, k = x2.shape
    n = wq.shape[0]
    y = np.empty((m, n), dtype=np.float16)
    rc = lib().oracle_qmm_f16(_p(x2), _p(wq), _p(scales), _p(biases), _p(bias), _p(y),
                              m, n, k, group_size, nthreads)
    if rc != 0:
        raise ValueError(f"oracle_qmm_f16 rejected the shape (rc={rc})")
    return y.reshape(*lead, n)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Run later matmuls on every core this process may use, even when a launcher exported
    ``OMP_NUM_THREADS=1``; returns the thread count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(n)
    return num_threads()
