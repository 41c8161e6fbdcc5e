"""Loads the operator library and registers the shape-only ("fake") implementations.

Mirrors mindiesd/layers/register_ops.py:24-128 of MindIE-SD: the library is
`<package>/plugin/libPTAExtensionOPS.so`, the namespace is `mindiesd`, and a fake implementation
can only be registered for an operator the library defines.  Unlike the reference the library is
loaded whether or not a device is present (the schemas are needed to trace on CPU); calling an
operator still needs a CUDA device, and a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

from pathlib import Path
from typing import Callable

import torch

from ..utils.exception import ParametersInvalid

MINDIE_NS = "mindiesd"
_LIB = Path(__file__).resolve().parents[1] / "plugin" / "libPTAExtensionOPS.so"
_loaded = False


def _load_mindie_ops_library() -> None:
    global _loaded
    if _loaded:
        return
    if not _LIB.exists():
        raise FileNotFoundError(
            f"{_LIB} not found: build it with `python mindie-sd_b200/csrc/build.py`. "
            "The attention operators have no other implementation.")
    torch.ops.load_library(str(_LIB))
    _loaded = True


_load_mindie_ops_library()


def check_mindie_operator_exists(op_name: str) -> bool:
    try:
        getattr(torch.ops.mindiesd, op_name)
        return True
    except AttributeError:
        return False


def register_mindie_fake_op(op_name: str) -> Callable:
    """Decorator: registers `fn` as the fake (meta) implementation of mindiesd::<op_name>."""
    if not isinstance(op_name, str) or not op_name:
        raise ParametersInvalid("op_name must be a non-empty string")
    if not check_mindie_operator_exists(op_name):
        raise RuntimeError(
            f"MindIE operator {MINDIE_NS}::{op_name} not found! "
            "Ensure the SO library is loaded and the operator is registered with TORCH_LIBRARY.")
    return torch.library.register_fake(f"{MINDIE_NS}::{op_name}")
