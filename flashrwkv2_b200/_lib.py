"""ctypes binding of libfrwkv_sm100.so (the C ABI declared in include/frwkv_sm100.h).

There is no CPU fallback: if the library has not been built, loading raises.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfrwkv_sm100.so"

IO_BF16, IO_FP16, IO_FP32 = 0, 1, 2
DECAY_LOGITS, DECAY_RETENTION = 0, 1
PREFILL_AUTO, PREFILL_RECURRENT, PREFILL_CHUNK_TC = 0, 1, 2
ABI_VERSION = 2
STATIC_POOL_SLOTS = 65536

# every symbol include/frwkv_sm100.h declares
SYMBOLS = (
    "frwkv_sm100_abi_version",
    "frwkv_sm100_last_error",
    "frwkv_sm100_wkv7_validate_metadata",
    "frwkv_sm100_wkv7_validate_metadata_static",
    "frwkv_sm100_wkv7_recurrent",
    "frwkv_sm100_wkv7_recurrent_fp16_state",
    "frwkv_sm100_wkv7_prefill",
    "frwkv_sm100_wkv7_prefill_workspace_bytes",
    "frwkv_sm100_wkv7_recurrent_fused_gate",
    "frwkv_sm100_wkv7_prefill_fused_gate",
    "frwkv_sm100_wkv7_recurrent_readout",
    "frwkv_sm100_wkv7_prefill_readout",
    "frwkv_sm100_wkv7_pretrain_forward",
    "frwkv_sm100_wkv7_pretrain_backward",
)

_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryMissing(
            f"{LIB_PATH} is not built; run `python -m flashrwkv2_b200.build` "
            "(there is no CPU or PyTorch fallback for the WKV7 operator)")
    lib = declare(ctypes.CDLL(str(LIB_PATH)))
    if lib.frwkv_sm100_abi_version() != ABI_VERSION:
        raise RuntimeError("libfrwkv_sm100.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def declare(lib: ctypes.CDLL) -> ctypes.CDLL:
    """Attach the argument and result types of every entry point include/frwkv_sm100.h declares."""
    vp, ci, cf, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    lib.frwkv_sm100_abi_version.restype = ci
    lib.frwkv_sm100_abi_version.argtypes = []
    lib.frwkv_sm100_last_error.restype = ctypes.c_char_p
    lib.frwkv_sm100_last_error.argtypes = []
    lib.frwkv_sm100_wkv7_validate_metadata.restype = ci
    lib.frwkv_sm100_wkv7_validate_metadata.argtypes = [vp, vp, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp]
    lib.frwkv_sm100_wkv7_validate_metadata_static.restype = ci
    lib.frwkv_sm100_wkv7_validate_metadata_static.argtypes = [vp, vp, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]
    lib.frwkv_sm100_wkv7_recurrent.restype = ci
    lib.frwkv_sm100_wkv7_recurrent.argtypes = [vp] * 13 + [ci, ci, ci, ci, ci, cf, ci, vp]
    lib.frwkv_sm100_wkv7_recurrent_fp16_state.restype = ci
    lib.frwkv_sm100_wkv7_recurrent_fp16_state.argtypes = [vp] * 5 + [ci] + [vp] * 8 + [ci, ci, ci, ci, cf, ci, vp, vp]
    lib.frwkv_sm100_wkv7_prefill.restype = ci
    lib.frwkv_sm100_wkv7_prefill.argtypes = [vp] * 13 + [ci, ci, ci, ci, ci, cf, ci, ci, vp, sz, vp, vp]
    lib.frwkv_sm100_wkv7_prefill_workspace_bytes.restype = sz
    lib.frwkv_sm100_wkv7_prefill_workspace_bytes.argtypes = [ci, ci, ci]
    lib.frwkv_sm100_wkv7_recurrent_fused_gate.restype = ci
    lib.frwkv_sm100_wkv7_recurrent_fused_gate.argtypes = [vp] * 15 + [ci, ci, ci, ci, ci, cf, ci, vp]
    lib.frwkv_sm100_wkv7_prefill_fused_gate.restype = ci
    lib.frwkv_sm100_wkv7_prefill_fused_gate.argtypes = [vp] * 15 + [ci, ci, ci, ci, ci, cf, ci, ci, vp, sz, vp, vp]
    lib.frwkv_sm100_wkv7_recurrent_readout.restype = ci
    lib.frwkv_sm100_wkv7_recurrent_readout.argtypes = [vp] * 21 + [ci, ci, ci, ci, ci, cf, ci, vp]
    lib.frwkv_sm100_wkv7_prefill_readout.restype = ci
    lib.frwkv_sm100_wkv7_prefill_readout.argtypes = [vp] * 21 + [ci, ci, ci, ci, ci, cf, ci, ci, vp, sz, vp, vp]
    lib.frwkv_sm100_wkv7_pretrain_forward.restype = ci
    lib.frwkv_sm100_wkv7_pretrain_forward.argtypes = [vp] * 9 + [ci, ci, ci, vp]
    lib.frwkv_sm100_wkv7_pretrain_backward.restype = ci
    lib.frwkv_sm100_wkv7_pretrain_backward.argtypes = [vp] * 15 + [ci, ci, ci, vp]
    return lib


def last_error() -> str:
    return load().frwkv_sm100_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Raise the reference's native error type (RuntimeError) for a rejected call."""
    if rc != 0:
        raise RuntimeError(last_error() or f"libfrwkv_sm100 call failed with code {rc}")
