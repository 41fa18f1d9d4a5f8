"""CPU oracle for the tree speculative decoding path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / ``--impl reference`` legs of ``bench.py`` as the checker and the
timed CPU baseline, never as the product path.

Parity status: **parity unpinned against MLX itself.**  The reference's
arithmetic lives in ``mlx`` / ``mlx_lm`` (no version pinned by the reference,
not installable here) and in Metal shaders; neither can be executed on Linux.
What is pinned: the structural known-answer vectors of the reference's own test
(``mlx_eagle_tests.py:80,97-113``: tree mask, position ids, retrieve indices)
and the algebraic properties it asserts (array-position RoPE equals contiguous
RoPE under permutation, ``mlx_arrayed_rope_kernel.py:211-236``; the compacted
speculative cache equals the sequentially built cache,
``mlx_eagle_tests.py:135-170``).

Modules
-------
qmm_ref     4-bit affine dequantise + matmul  (``kernels/progression/simd_no_swizzle_cast.metal``)
detmath     deterministic exp/log used for log-probabilities
tree_ref    tree build / finalise / accept / compaction  (``mlx_eagle.py``)
model_ref   Llama/Qwen2 forward with tree hooks  (``mlx_llama.py``)
"""
