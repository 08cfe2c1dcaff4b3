"""Shared pytest plumbing: the ``gpu`` marker, import path, golden-vector loader."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"
TOKEN_NAMES = ("r", "decay_logits", "k", "v", "a", "b")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    """Load one committed golden case as CPU torch tensors (16-bit tensors are
    stored as raw bit patterns; see tests/golden/make_golden.py)."""
    blob = np.load(GOLDEN / f"{name}.npz")
    dtype = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[str(blob["dtype"])]
    case = {"dtype": dtype, "scale": float(blob["scale"])}
    for key in blob.files:
        if key in ("dtype", "scale"):
            continue
        arr = blob[key]
        if arr.dtype == np.uint16:
            case[key] = torch.from_numpy(arr.view(np.int16).copy()).view(dtype)
        else:
            case[key] = torch.from_numpy(arr.copy())
    case.setdefault("decay_bias", None)
    return case


GOLDEN_CASES = ("recurrent_bf16", "recurrent_bf16_bias", "recurrent_fp16_bias",
                "recurrent_bf16_long", "recurrent_bf16_unit", "rl_infctx_fp16")


def load_testhooks():
    """The test build of the C-ABI library (same sources, -DFRWKV_TEST_HOOKS): the product's entry points plus
    frwkv_sm100_test_skip_commit() and frwkv_sm100_test_recurrent_parts().  Built on demand (nvcc, cached)."""
    import ctypes

    from flashrwkv2_b200 import _lib
    from flashrwkv2_b200.build import build_testhooks

    lib = ctypes.CDLL(str(build_testhooks()))
    _lib.declare(lib)
    lib.frwkv_sm100_test_skip_commit.restype = None
    lib.frwkv_sm100_test_skip_commit.argtypes = [ctypes.c_int]
    lib.frwkv_sm100_test_recurrent_parts.restype = None
    lib.frwkv_sm100_test_recurrent_parts.argtypes = [ctypes.c_int]
    return lib
