"""Importable alias of the ``mlx-eagle-spec-decoding-tree_b200`` package.

The package directory carries the reference's name (with hyphens), which the
``import`` statement cannot spell; ``import b200_eagle`` returns that package.
Use ``b200_eagle.<submodule>`` attributes (all submodules are imported eagerly),
not ``import b200_eagle.<submodule>``.
"""
import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
sys.modules[__name__] = importlib.import_module("mlx-eagle-spec-decoding-tree_b200")
