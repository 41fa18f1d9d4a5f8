"""ctypes loader of ``libb200eagle.so``.

There is no fallback: if the library has not been built (``python -m`` of
``build.py`` in this directory, or ``__graft_entry__.build()``), importing an
operator raises.  All tensors handed to the library are CUDA tensors owned by
torch; the library only sees raw device pointers and the current CUDA stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200eagle.so")

E_NAMES = {-1: "EINVAL (bad shape/size/flags)", -2: "EALIGN (pointer not 16-byte aligned)",
           -3: "EUNSUPPORTED (dtype/group size)", -4: "EWORKSPACE (workspace too small)",
           -5: "ECUDA (CUDA runtime error)", -6: "ELIMIT (size beyond a fixed maximum)"}

_lib = None


class B200Error(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(
                f"{LIB_PATH} is missing: build it first (python {os.path.join(_HERE, 'build.py')}). "
                "There is no CPU or PyTorch fallback for this path.")
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
        if os.environ.get("B200_PDL", "1") == "0":
            _lib.b200_set_pdl(0)
    return _lib


def _declare(l: ctypes.CDLL) -> None:
    vp, i32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    l.b200_version.restype = i32
    l.b200_last_cuda_error.restype = i32
    l.b200_set_pdl.restype = None
    l.b200_set_pdl.argtypes = [i32]
    l.b200_set_wait_limit.restype = None
    l.b200_set_wait_limit.argtypes = [ctypes.c_uint]
    l.b200_qmm_workspace_bytes.restype = sz
    l.b200_qmm_workspace_bytes.argtypes = [i32, i32, i32]
    l.b200_qmm.restype = i32
    l.b200_qmm.argtypes = [vp] * 6 + [i32] * 5 + [vp, sz, vp]
    l.b200_qmm_fused.restype = i32
    l.b200_qmm_fused.argtypes = [vp] * 10 + [i32] * 6 + [vp, sz, vp]
    f32, u64 = ctypes.c_float, ctypes.c_ulonglong
    l.b200_qmm_noalloc_max_scratch_bytes.restype = sz
    l.b200_qmm_noalloc.restype = i32
    l.b200_qmm_noalloc.argtypes = [vp] * 6 + [i32] * 5 + [vp]
    l.b200_qmm_tiled_bytes.restype = sz
    l.b200_qmm_tiled_bytes.argtypes = [i32, i32]
    l.b200_qmm_relayout.restype = i32
    l.b200_qmm_relayout.argtypes = [vp, vp, vp, vp, i32, i32, vp]
    l.b200_qmm_tiled_workspace_bytes.restype = sz
    l.b200_qmm_tiled_workspace_bytes.argtypes = [i32, i32, i32]
    l.b200_qmm_tiled.restype = i32
    l.b200_qmm_tiled.argtypes = [vp] * 6 + [i32] * 4 + [vp, sz, vp]
    l.b200_qmm_umma_workspace_bytes.restype = sz
    l.b200_qmm_umma_workspace_bytes.argtypes = [i32, i32]
    l.b200_qmm_umma.restype = i32
    l.b200_qmm_umma.argtypes = [vp] * 4 + [i32] * 3 + [vp, sz, vp]
    l.b200_embed_gather.restype = i32
    l.b200_embed_gather.argtypes = [vp] * 5 + [i32] * 3 + [vp]
    l.b200_rms_norm.restype = i32
    l.b200_rms_norm.argtypes = [vp] * 4 + [i32, i32, f32, vp]
    l.b200_rope_kv_append.restype = i32
    l.b200_rope_kv_append.argtypes = [vp, vp, vp, f32, vp, vp, vp] + [i32] * 6 + [vp]
    l.b200_rope_positions.restype = i32
    l.b200_rope_positions.argtypes = [vp, vp, vp, f32, vp] + [i32] * 4 + [vp]
    l.b200_tree_attention_workspace_bytes.restype = sz
    l.b200_tree_attention_workspace_bytes.argtypes = [i32] * 5
    l.b200_tree_attention.restype = i32
    l.b200_tree_attention.argtypes = [vp, i32, vp, vp, vp, vp, i32, vp] + [i32] * 6 + [f32, vp, sz, vp]
    l.b200_topk_blocks.restype = i32
    l.b200_topk_blocks.argtypes = [i32]
    l.b200_logits_rowstats.restype = i32
    l.b200_logits_rowstats.argtypes = [vp, i32, i32, vp, vp, vp]
    l.b200_logits_topk_candidates.restype = i32
    l.b200_logits_topk_candidates.argtypes = [vp, i32, i32, vp, vp, i32, vp, vp]
    l.b200_tree_expand.restype = i32
    l.b200_tree_expand.argtypes = [vp, i32, i32] + [vp] * 14
    l.b200_prep_catchup.restype = i32
    l.b200_prep_catchup.argtypes = [vp] * 8
    l.b200_tree_finalize.restype = i32
    l.b200_tree_finalize.argtypes = [i32, i32] + [vp] * 15
    l.b200_logits_argmax.restype = i32
    l.b200_logits_argmax.argtypes = [vp, i32, i32, vp, vp]
    l.b200_tree_accept.restype = i32
    l.b200_tree_accept.argtypes = [i32] + [vp] * 10
    l.b200_tree_accept_sample_workspace_bytes.restype = sz
    l.b200_tree_accept_sample_workspace_bytes.argtypes = [i32]
    l.b200_tree_accept_sample.restype = i32
    l.b200_tree_accept_sample.argtypes = [i32, i32, vp, vp, vp, vp, vp, ctypes.c_double, vp, vp, vp, vp, vp, vp, sz, vp]
    l.b200_sample_token.restype = i32
    l.b200_sample_token.argtypes = [vp, i32, ctypes.c_double, ctypes.c_uint, ctypes.c_uint, vp, vp, vp, sz, vp, vp]
    l.b200_logits_rowstats_temp.restype = i32
    l.b200_logits_rowstats_temp.argtypes = [vp, i32, i32, vp, vp, ctypes.c_double, vp]
    l.b200_forward_plan_hint.restype = None
    l.b200_forward_plan_hint.argtypes = [ctypes.c_char_p]
    l.b200_forward_workspace_bytes.restype = sz
    l.b200_forward_workspace_bytes.argtypes = [ctypes.POINTER(ForwardDesc)]
    l.b200_forward_tp_buffer_bytes.restype = sz
    l.b200_forward_tp_buffer_bytes.argtypes = [i32]
    l.b200_tp_exchange_alloc.restype = i32
    l.b200_tp_exchange_alloc.argtypes = [sz, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
    l.b200_tp_exchange_open.restype = i32
    l.b200_tp_exchange_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    l.b200_tp_exchange_close.restype = i32
    l.b200_tp_exchange_close.argtypes = [vp]
    l.b200_tp_exchange_free.restype = i32
    l.b200_tp_exchange_free.argtypes = [vp]
    l.b200_tp_exchange_reset.restype = i32
    l.b200_tp_exchange_reset.argtypes = [vp, sz]
    l.b200_tp_exchange_error.restype = i32
    l.b200_tp_exchange_error.argtypes = [vp]
    l.b200_tp_argmax_combine.restype = i32
    l.b200_tp_argmax_combine.argtypes = [vp, i32, ctypes.c_uint, i32, i32, ctypes.POINTER(ctypes.c_void_p), vp]
    l.b200_forward.restype = i32
    l.b200_forward.argtypes = [ctypes.POINTER(ForwardDesc), vp]
    l.b200_add_f16.restype = i32
    l.b200_add_f16.argtypes = [vp, vp, sz, vp]
    l.b200_silu_mul_f16.restype = i32
    l.b200_silu_mul_f16.argtypes = [vp, vp, vp, sz, vp]
    l.b200_residual_add_f32.restype = i32
    l.b200_residual_add_f32.argtypes = [vp, vp, i32, i32, vp]
    l.b200_argmax_key_shift.restype = i32
    l.b200_argmax_key_shift.argtypes = [vp, i32, ctypes.c_uint, vp]
    l.b200_kv_compact.restype = i32
    l.b200_kv_compact.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp]


class ForwardDesc(ctypes.Structure):
    """Mirror of ``b200_forward_desc`` (include/b200_eagle.h): host struct of sizes and device pointers."""
    _fields_ = ([(n, ctypes.c_int) for n in (
        "M", "rows_out", "hidden", "intermediate", "n_heads", "n_kv_heads", "head_dim", "vocab", "n_layers",
        "cache_rows", "write_off", "tail")]
        + [(n, ctypes.c_float) for n in ("rms_eps", "rope_scaling", "attn_scale")]
        + [("attn_split_blocks", ctypes.c_int)]
        + [(n, ctypes.c_void_p) for n in (
            "tokens", "pos", "mask", "prefix", "row_index", "inv_freq", "embed_wq", "embed_scales", "embed_biases",
            "final_norm", "lm_head_tiled", "layer_table", "h", "hw", "qkv", "attn", "act", "logits", "kv_cache",
            "workspace")]
        + [("workspace_bytes", ctypes.c_size_t), ("timeline", ctypes.c_void_p), ("timeline_pitch", ctypes.c_int),
           ("phase_mask", ctypes.c_int), ("tp_world", ctypes.c_int), ("tp_rank", ctypes.c_int),
           ("head_rows", ctypes.c_int), ("grid_ctas", ctypes.c_int), ("tp_peers", ctypes.c_void_p * 8),
           ("scales_in_fast_range", ctypes.c_int), ("tp_two_shot", ctypes.c_int), ("requests", ctypes.c_int)])


def check(rc: int, what: str) -> None:
    if rc != 0:
        extra = ""
        if rc == -5:
            extra = f" (cudaError {lib().b200_last_cuda_error()})"
        raise B200Error(f"{what} failed: {E_NAMES.get(rc, rc)}{extra}")


def ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise B200Error("this operator only runs on CUDA tensors (no CPU path is provided)")
