"""WKV7 training operator (forward with state checkpoints + backward) on B200.

Same public contract as rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/pretrain.py:13-133: six contiguous CUDA bfloat16
tensors ``[B, T, C]``, ``C`` a multiple of the head size, ``T`` a multiple of 16, zero initial state, decay logits
``w`` (retention ``exp(-e^{-1/2} * sigmoid(w))``); returns ``[B, T, C]`` bfloat16 and is differentiable in all six
inputs.  ``TypeError`` for wrong types and dtypes, ``ValueError`` for wrong shapes and layouts, before any launch.
This backend builds head size 64.
"""

from __future__ import annotations

import torch

from . import _checks as check

CHUNK_LEN = 16
NAMES = ("r", "w", "k", "v", "a", "b")


def _extension():
    import flashrwkv2_b200

    if flashrwkv2_b200._C is None:
        raise RuntimeError("flashrwkv2_b200 native backend is not loaded (needs a CUDA device of capability 10.0)")
    return flashrwkv2_b200._C


def _validate(tensors, head_size: int) -> tuple[int, int, int]:
    check.need(head_size in (64, 128, 256), ValueError, "head_size must be one of 64, 128, or 256")
    check.need(head_size == 64, ValueError, "this backend builds the WKV7 training operator for head_size 64 only")
    check.need(len(tensors) == 6, ValueError, "the operator takes r, w, k, v, a and b")
    r = tensors[0]
    check.tensor(r, "r")
    check.need(r.ndim == 3 and min(r.shape) > 0, ValueError, "r must have shape [B,T,C] with nonzero dimensions")
    for name, value in zip(NAMES, tensors):
        check.tensor(value, name)
        check.need(value.dtype == torch.bfloat16, TypeError, f"{name} must be bfloat16")
        check.need(value.is_cuda and value.is_contiguous(), ValueError, f"{name} must be contiguous CUDA")
        check.need(value.shape == r.shape, ValueError, f"{name} must match r shape")
        check.need(value.device == r.device, ValueError, f"{name} must share the r device")
    batch, tokens, channels = r.shape
    check.need(channels % head_size == 0, ValueError, "C must be divisible by head_size")
    check.need(tokens % CHUNK_LEN == 0, ValueError, "T must be divisible by the chunk length 16")
    return batch, tokens, channels


class _Recurrence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, head_size):
        batch, tokens, channels = _validate((r, w, k, v, a, b), head_size)
        heads = channels // head_size
        rows = tuple(x.view(batch, tokens, heads, head_size) for x in (r, w, k, v, a, b))
        y = torch.empty_like(rows[3])
        boundary = torch.empty((batch, heads, tokens // CHUNK_LEN, head_size, head_size), device=r.device,
                               dtype=torch.float32)
        state_dot_a = torch.empty((batch, tokens, heads, head_size), device=r.device, dtype=torch.float32)
        _extension().pretrain_tmix_wkv7_recurrent_forward(*rows, y, boundary, state_dot_a, head_size)
        ctx.save_for_backward(*rows, boundary, state_dot_a)
        ctx.dense_shape = (batch, tokens, channels)
        ctx.head_size = head_size
        return y.view(batch, tokens, channels)

    @staticmethod
    def backward(ctx, grad_output):
        *rows, boundary, state_dot_a = ctx.saved_tensors
        batch, tokens, channels = ctx.dense_shape
        dy = grad_output.contiguous().view(batch, tokens, channels // ctx.head_size, ctx.head_size)
        grads = tuple(torch.empty_like(x) for x in rows)
        _extension().pretrain_tmix_wkv7_recurrent_backward(*rows, dy, boundary, state_dot_a, *grads, ctx.head_size)
        return tuple(g.view(batch, tokens, channels) for g in grads) + (None,)


def pretrain_tmix_wkv7_recurrent_bf16(r: torch.Tensor, w: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                      a: torch.Tensor, b: torch.Tensor, *, head_size: int = 64) -> torch.Tensor:
    """The differentiable WKV7 recurrence over dense ``[B, T, C]`` bfloat16 tensors (see the module docstring)."""
    _validate((r, w, k, v, a, b), head_size)
    return _Recurrence.apply(r, w, k, v, a, b, head_size)


__all__ = ["pretrain_tmix_wkv7_recurrent_bf16"]
