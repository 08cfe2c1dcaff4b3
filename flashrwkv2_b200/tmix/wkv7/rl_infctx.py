"""Chunk-forward operator that returns the final state pool (caller's pool untouched).

Contract of rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/rl_infctx.py:66-152.  Differences in
mechanism, not in results: sequence boundaries are validated on the device by the metadata
kernel (one host read of the 3-word status instead of three ``.item()`` syncs, a host list
of slots and a Python loop over chunks), no per-chunk metadata is built, and the work is
one fused kernel that always uses 64-row chunks.  ``chunk_size`` and ``strategy`` are
validated and otherwise ignored: every choice gives the same result.
"""

from __future__ import annotations

import math

import torch


def _check_tensor(tensor, name, dtype=None):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous CUDA")
    if dtype is not None and tensor.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}")


_META_MESSAGES = (
    (1 << 0, "cu_seqlens must start at zero and end at total_tokens"),
    (1 << 1, "each RL/Infctx sequence must be non-empty"),
    (1 << 2, "state_indices must be within state_pool"),
    (1 << 3, "state_indices must not contain duplicates"),
)


def rl_infctx_tmix_wkv7_chunk_fp32io16(
    r,
    decay_logits,
    k,
    v,
    a,
    b,
    *,
    state_pool=None,
    cu_seqlens,
    state_indices=None,
    chunk_size: int = 16,
    strategy: str = "recompute",
    scale: float = 1.0,
    decay_bias=None,
    decay_mode: str = "logits",
):
    """Returns ``(output, final_pool)``; ``state_pool`` (zeros if None) is not modified."""
    from . import _extension

    if chunk_size not in {16, 32, 64}:
        raise ValueError("chunk_size must be one of 16, 32, or 64")
    if strategy not in {"materialized", "recompute"}:
        raise ValueError("strategy must be 'materialized' or 'recompute'")
    if not math.isfinite(float(scale)):
        raise ValueError("scale must be finite")
    tensors = {"r": r, "decay_logits": decay_logits, "k": k, "v": v, "a": a, "b": b}
    for name, tensor in tensors.items():
        _check_tensor(tensor, name)
        if tensor.dtype not in {torch.float16, torch.bfloat16}:
            raise TypeError(f"{name} must be float16 or bfloat16")
    if r.ndim != 3 or r.shape[0] <= 0 or r.shape[1] <= 0 or r.shape[2] not in {64, 128, 256}:
        raise ValueError("RL/Infctx token tensors must have shape [N,H,D]")
    if r.shape[2] != 64:
        raise ValueError("the sm_100a backend implements head size 64 only")
    if any(t.shape != r.shape or t.device != r.device for t in tensors.values()):
        raise ValueError("RL/Infctx token tensors must match r and share a device")
    if decay_bias is not None:
        _check_tensor(decay_bias, "decay_bias")
        if decay_bias.dtype != r.dtype or decay_bias.device != r.device:
            raise TypeError("decay_bias must match token dtype and device")
        if tuple(decay_bias.shape) not in {(r.shape[1] * r.shape[2],), (r.shape[1], r.shape[2])}:
            raise ValueError("decay_bias must have shape [H*D] or [H,D]")
    _check_tensor(cu_seqlens, "cu_seqlens", torch.int32)
    if cu_seqlens.device != r.device:
        raise ValueError("cu_seqlens must share the token device")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must have shape [B+1]")
    batch = cu_seqlens.numel() - 1
    if state_indices is None:
        state_indices = torch.arange(batch, device=r.device, dtype=torch.int32)
    _check_tensor(state_indices, "state_indices", torch.int32)
    if state_indices.ndim != 1 or state_indices.numel() != batch:
        raise ValueError("state_indices must have shape [B]")
    if state_indices.device != r.device:
        raise ValueError("state_indices must share the token device")
    if state_pool is None:
        state_pool = torch.zeros(batch, r.shape[1], 64, 64, device=r.device, dtype=torch.float32)
    _check_tensor(state_pool, "state_pool", torch.float32)
    if state_pool.ndim != 4 or tuple(state_pool.shape[1:]) != (r.shape[1], 64, 64):
        raise ValueError("state_pool must have shape [slots,H,D,D]")

    ext = _extension()
    # device-side validation of the boundaries and slots; the reference raises ValueError for
    # bad metadata, so read the status back once (12 bytes) before launching the recurrence
    ticket = ext.prepare_tmix_wkv7_recurrent_graph_metadata(
        cu_seqlens, state_indices,
        torch.tensor([r.shape[0]], dtype=torch.int32, device=r.device),
        torch.tensor([batch], dtype=torch.int32, device=r.device),
        int(r.shape[0]), int(batch), int(state_pool.shape[0]), int(r.shape[0]))
    error = int(ticket._status()[0].item())
    for bit, message in _META_MESSAGES:
        if error & bit:
            raise ValueError(message)
    if error:
        raise ValueError(f"invalid RL/Infctx metadata (status {error})")
    final_pool = state_pool.clone()
    output = torch.empty_like(v)
    ext.tmix_wkv7_prefill_fp32(cu_seqlens, state_indices, final_pool, r, decay_logits, k, v, a, b, output,
                               float(scale), decay_bias, ticket, -1, decay_mode, "auto")
    return output, final_pool


def rl_infctx_tmix_wkv7_chunk_fp32io16_factor_recompute(*args, **kwargs):
    """Explicit recompute entry of the reference's operator family (same result)."""
    kwargs["strategy"] = "recompute"
    return rl_infctx_tmix_wkv7_chunk_fp32io16(*args, **kwargs)


__all__ = ["rl_infctx_tmix_wkv7_chunk_fp32io16", "rl_infctx_tmix_wkv7_chunk_fp32io16_factor_recompute"]
