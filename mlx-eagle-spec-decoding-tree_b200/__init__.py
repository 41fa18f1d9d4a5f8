"""B200-native (sm_100a) kernels and host loop for EAGLE-2-style tree speculative decoding.

Drop-in for the hot path of 0seba/mlx-eagle-spec-decoding-tree: the operator
modules keep the reference's names and call signatures, the work is done by
``libb200eagle.so`` (hand-written CUDA behind a C ABI, see ``include/b200_eagle.h``).
"""
from . import _lib, quantize, qmm_kernel, llama, eagle, rope, load  # noqa: F401
from .qmm_kernel import matmul  # noqa: F401
from .rope import rope_positions  # noqa: F401
from .llama import Model, ModelArgs, KVCache, BatchKVCache, shape_preset  # noqa: F401
from .eagle import SpecDecoder, BatchSpecDecoder, generate_step, spec_step  # noqa: F401

__all__ = ["matmul", "rope_positions", "Model", "ModelArgs", "KVCache", "shape_preset", "SpecDecoder", "BatchSpecDecoder", "BatchKVCache",
           "generate_step", "spec_step", "qmm_kernel", "quantize", "llama", "eagle", "rope", "load"]
