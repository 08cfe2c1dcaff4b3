"""Argument checks shared by the WKV7 operator wrappers.

The wrappers keep the reference's error contract (rwkv-rs/FlashRWKV2
flashrwkv2/tmix/wkv7/__init__.py:20-88, rl_infctx.py:12-38): ``TypeError`` for wrong Python or
tensor types, ``ValueError`` for wrong ranks, shapes, layouts or values, both raised before
anything is launched.  Each check is one call to :func:`need`.
"""

from __future__ import annotations

import torch

TOKEN_NAMES = ("r", "decay_logits", "k", "v", "a", "b")


def need(condition: bool, error: type[Exception], message: str) -> None:
    if not condition:
        raise error(message)


def tensor(value, name: str) -> None:
    need(isinstance(value, torch.Tensor), TypeError, f"{name} must be a torch.Tensor")


def packed_tokens(tokens) -> None:
    """Six packed [total_tokens, H, D] tensors, contiguous."""
    for name, value in zip(TOKEN_NAMES, tokens):
        tensor(value, name)
        need(value.ndim == 3, ValueError, f"{name} must have packed shape [total_tokens,H,D]")
        need(value.is_contiguous(), ValueError, f"{name} must be contiguous")


def fp32_pool(pool) -> None:
    tensor(pool, "state_pool")
    need(pool.is_contiguous(), ValueError, "state_pool must be contiguous")
    need(pool.dtype == torch.float32, TypeError, "state_pool must have dtype float32")


def metadata(cu_seqlens, state_indices) -> None:
    tensor(cu_seqlens, "cu_seqlens")
    need(cu_seqlens.ndim == 1, ValueError, "cu_seqlens must be one-dimensional")
    tensor(state_indices, "state_indices")


def cuda_contiguous(value, name: str, dtype: torch.dtype | None = None) -> None:
    tensor(value, name)
    need(value.is_cuda and value.is_contiguous(), ValueError, f"{name} must be contiguous CUDA")
    need(dtype is None or value.dtype == dtype, TypeError, f"{name} must have dtype {dtype}")


def positive_int(value, name: str) -> None:
    need(isinstance(value, int) and not isinstance(value, bool) and value > 0, ValueError,
         f"{name} must be a positive integer")


def device_scalar(value, name: str, device) -> None:
    ok = (isinstance(value, torch.Tensor) and value.dtype == torch.int32 and value.is_cuda
          and value.is_contiguous() and value.numel() == 1 and value.device == device)
    need(ok, ValueError, f"{name} must be a one-element contiguous CUDA int32 tensor")
