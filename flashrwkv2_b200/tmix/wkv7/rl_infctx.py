"""Chunk-forward operator that returns the final state pool and leaves the caller's pool alone.

Contract of rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/rl_infctx.py:66-152 (same keywords, same error
types).  The mechanism differs: sequence boundaries and slots are validated by the device kernel
(one 12-byte status read-back instead of three ``.item()`` syncs, a host list of slots and a Python
loop over chunks), no per-chunk metadata is built, and one fused kernel does the work.
``chunk_size`` and ``strategy`` are validated and otherwise ignored: every choice gives the same
result.
"""

from __future__ import annotations

import math

import torch

from . import _checks as check

# device status bit -> the reference wrapper's complaint
_STATUS_MESSAGES = {
    1 << 0: "cu_seqlens must start at zero and end at total_tokens",
    1 << 1: "each RL/Infctx sequence must be non-empty",
    1 << 2: "state_indices must be within state_pool",
    1 << 3: "state_indices must not contain duplicates",
}


def rl_infctx_tmix_wkv7_chunk_fp32io16(r, decay_logits, k, v, a, b, *, state_pool=None, cu_seqlens,
                                       state_indices=None, chunk_size: int = 16, strategy: str = "recompute",
                                       scale: float = 1.0, decay_bias=None, decay_mode: str = "logits"):
    """Returns ``(output, final_pool)``; ``state_pool`` (zeros when None) is never modified."""
    from . import _extension

    check.need(chunk_size in (16, 32, 64), ValueError, "chunk_size must be one of 16, 32, or 64")
    check.need(strategy in ("materialized", "recompute"), ValueError,
               "strategy must be 'materialized' or 'recompute'")
    check.need(math.isfinite(float(scale)), ValueError, "scale must be finite")
    tokens = (r, decay_logits, k, v, a, b)
    for name, value in zip(check.TOKEN_NAMES, tokens):
        check.cuda_contiguous(value, name)
        check.need(value.dtype in (torch.float16, torch.bfloat16), TypeError, f"{name} must be float16 or bfloat16")
    check.need(r.ndim == 3 and min(r.shape[:2]) > 0 and r.shape[2] in (64, 128, 256), ValueError,
               "RL/Infctx token tensors must have shape [N,H,D]")
    check.need(r.shape[2] == 64, ValueError, "the sm_100a backend implements head size 64 only")
    check.need(all(t.shape == r.shape and t.device == r.device for t in tokens), ValueError,
               "RL/Infctx token tensors must match r and share a device")
    total, heads, dim = r.shape
    if decay_bias is not None:
        check.cuda_contiguous(decay_bias, "decay_bias")
        check.need(decay_bias.dtype == r.dtype and decay_bias.device == r.device, TypeError,
                   "decay_bias must match token dtype and device")
        check.need(tuple(decay_bias.shape) in ((heads * dim,), (heads, dim)), ValueError,
                   "decay_bias must have shape [H*D] or [H,D]")
    check.cuda_contiguous(cu_seqlens, "cu_seqlens", torch.int32)
    check.need(cu_seqlens.device == r.device, ValueError, "cu_seqlens must share the token device")
    check.need(cu_seqlens.ndim == 1 and cu_seqlens.numel() >= 2, ValueError, "cu_seqlens must have shape [B+1]")
    batch = cu_seqlens.numel() - 1
    if state_indices is None:
        state_indices = torch.arange(batch, device=r.device, dtype=torch.int32)
    check.cuda_contiguous(state_indices, "state_indices", torch.int32)
    check.need(state_indices.ndim == 1 and state_indices.numel() == batch, ValueError,
               "state_indices must have shape [B]")
    check.need(state_indices.device == r.device, ValueError, "state_indices must share the token device")
    if state_pool is None:
        state_pool = torch.zeros(batch, heads, dim, dim, device=r.device, dtype=torch.float32)
    check.cuda_contiguous(state_pool, "state_pool", torch.float32)
    check.need(state_pool.ndim == 4 and tuple(state_pool.shape[1:]) == (heads, dim, dim), ValueError,
               "state_pool must have shape [slots,H,D,D]")

    native = _extension()
    counts = torch.tensor([total, batch], dtype=torch.int32, device=r.device)
    ticket = native.prepare_tmix_wkv7_recurrent_graph_metadata(
        cu_seqlens, state_indices, counts[0:1], counts[1:2], int(total), int(batch), int(state_pool.shape[0]),
        int(total))
    status = int(ticket._status()[0].item())  # the reference raises for bad metadata, so look before launching
    for bit, message in _STATUS_MESSAGES.items():
        check.need(not status & bit, ValueError, message)
    check.need(status == 0, ValueError, f"invalid RL/Infctx metadata (status {status})")
    final_pool = state_pool.clone()
    output = torch.empty_like(v)
    native.tmix_wkv7_prefill_fp32(cu_seqlens, state_indices, final_pool, r, decay_logits, k, v, a, b, output,
                                  float(scale), decay_bias, ticket, -1, decay_mode, "auto")
    return output, final_pool


def rl_infctx_tmix_wkv7_chunk_fp32io16_factor_recompute(*args, **kwargs):
    """The reference's explicit "recompute" entry; same result as any other strategy here."""
    return rl_infctx_tmix_wkv7_chunk_fp32io16(*args, **{**kwargs, "strategy": "recompute"})


__all__ = ["rl_infctx_tmix_wkv7_chunk_fp32io16", "rl_infctx_tmix_wkv7_chunk_fp32io16_factor_recompute"]
