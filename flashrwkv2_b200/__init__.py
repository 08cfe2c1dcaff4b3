"""B200-native (sm_100a) WKV7 time-mix recurrence behind FlashRWKV2's operator contract.

Backend selection mirrors rwkv-rs/FlashRWKV2 flashrwkv2/__init__.py:12-55: the private
native module is chosen by compute capability and published as ``flashrwkv2_b200._C``.
The only backend is ``_C_sm100`` (capability 10.0 exactly: an sm_100a cubin); there is no Triton/TileLang path,
no multi-backend dispatch and no CPU fallback.
"""

import importlib as _importlib
import sys as _sys

import torch as _torch

_NATIVE_BACKENDS = (
    ((10, 0), "_C_sm100"),
)


def _backend_module_name(capability: tuple[int, int]) -> str:
    major, minor = capability
    # the backend is an sm_100a cubin ("a" = architecture-specific features: tcgen05, TMEM): it runs on
    # capability 10.0 exactly, not on later 10.x parts
    matches = [(target, name) for target, name in _NATIVE_BACKENDS if target == (major, minor)]
    if not matches:
        have = ", ".join(f"sm{t[0]}{t[1]}" for t, _ in _NATIVE_BACKENDS)
        raise RuntimeError(
            f"flashrwkv2_b200 has no binary-compatible native backend for sm{major}{minor}; "
            f"available cubin backends are {have}")
    return max(matches, key=lambda item: item[0])[1]


def _load_native_backend():
    if not _torch.cuda.is_available():
        return None
    capability = tuple(_torch.cuda.get_device_capability())
    module_name = _backend_module_name(capability)
    try:
        module = _importlib.import_module(f"{__name__}.{module_name}")
    except ImportError as error:
        raise RuntimeError(
            f"flashrwkv2_b200 selected backend {module_name} for sm{capability[0]}{capability[1]}, "
            "but that private extension is not built or cannot be loaded") from error
    _sys.modules[f"{__name__}._C"] = module
    return module


_C = _load_native_backend()

from .tmix.wkv7 import (  # noqa: E402
    infer_tmix_wkv7_fused_gate_fp32io16_forward_varlen,
    infer_tmix_wkv7_prefill_fp32io16_forward_varlen,
    infer_tmix_wkv7_readout_fp32io16_forward_varlen,
    infer_tmix_wkv7_recurrent_fp16_forward_varlen,
    infer_tmix_wkv7_recurrent_fp32io16_forward_varlen,
    prepare_tmix_wkv7_recurrent_metadata,
    pretrain_tmix_wkv7_recurrent_bf16,
    rl_infctx_tmix_wkv7_chunk_fp32io16,
)

__all__ = [
    "infer_tmix_wkv7_fused_gate_fp32io16_forward_varlen",
    "infer_tmix_wkv7_prefill_fp32io16_forward_varlen",
    "infer_tmix_wkv7_readout_fp32io16_forward_varlen",
    "infer_tmix_wkv7_recurrent_fp16_forward_varlen",
    "infer_tmix_wkv7_recurrent_fp32io16_forward_varlen",
    "prepare_tmix_wkv7_recurrent_metadata",
    "pretrain_tmix_wkv7_recurrent_bf16",
    "rl_infctx_tmix_wkv7_chunk_fp32io16",
]
