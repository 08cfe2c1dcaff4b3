"""Public WKV7 operators: the reference's ``flashrwkv2.tmix.wkv7`` contract on B200.

Same names, keyword arguments and error types as rwkv-rs/FlashRWKV2
flashrwkv2/tmix/wkv7/__init__.py:20-256 (``TypeError`` / ``ValueError`` from these
wrappers before any launch, ``RuntimeError`` from the native layer).  Extra keyword
arguments, all optional: ``decay_mode`` ("logits" as in the reference, or "retention"
when ``w`` already is the per-channel retention), ``output_f32`` (fp32 copy of the
output before rounding) and, for prefill, ``strategy``.
"""

from __future__ import annotations

import torch


def _extension():
    import flashrwkv2_b200

    extension = getattr(flashrwkv2_b200, "_C", None)
    if extension is None:
        raise RuntimeError(
            "flashrwkv2_b200 CUDA backend is not loaded (no CUDA device, or libfrwkv_sm100.so not "
            "built); the WKV7 operators have no CPU fallback")
    return extension


def _validate_packed_inputs(*tensors: torch.Tensor) -> tuple[torch.Tensor, ...]:
    for name, tensor in zip(("r", "decay_logits", "k", "v", "a", "b"), tensors):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.ndim != 3:
            raise ValueError(f"{name} must have packed shape [total_tokens,H,D]")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    return tensors


def _validate_state(state: torch.Tensor) -> None:
    if not isinstance(state, torch.Tensor):
        raise TypeError("state_pool must be a torch.Tensor")
    if not state.is_contiguous():
        raise ValueError("state_pool must be contiguous")
    if state.dtype != torch.float32:
        raise TypeError("state_pool must have dtype float32")


def _check_metadata_inputs(cu_seqlens, state_indices) -> None:
    if not isinstance(cu_seqlens, torch.Tensor):
        raise TypeError("cu_seqlens must be a torch.Tensor")
    if cu_seqlens.ndim != 1:
        raise ValueError("cu_seqlens must be one-dimensional")
    if not isinstance(state_indices, torch.Tensor):
        raise TypeError("state_indices must be a torch.Tensor")


def prepare_tmix_wkv7_recurrent_metadata(
    cu_seqlens: torch.Tensor,
    state_indices: torch.Tensor,
    *,
    state_pool_size: int,
    total_tokens: int | None = None,
    max_seqlen: int | None = None,
    token_capacity: int | None = None,
    sequence_capacity: int | None = None,
    max_seqlen_capacity: int | None = None,
    num_active_tokens: torch.Tensor | None = None,
    num_active_sequences: torch.Tensor | None = None,
) -> object:
    """Create a static ticket (``total_tokens`` form: snapshot + validation, one host sync)
    or a live capacity ticket (capacity form: metadata buffers and the two active-count
    scalars stay live; no host sync, usable for warm-up with zero active counts and
    inside CUDA-graph capture).  Reference: flashrwkv2/tmix/wkv7/__init__.py:91-176."""
    _check_metadata_inputs(cu_seqlens, state_indices)
    graph_values = (token_capacity, sequence_capacity, max_seqlen_capacity, num_active_tokens,
                    num_active_sequences)
    if any(value is not None for value in graph_values):
        if total_tokens is not None or max_seqlen is not None:
            raise ValueError("graph metadata uses capacity arguments, not total_tokens/max_seqlen")
        if any(value is None for value in graph_values):
            raise ValueError("all graph metadata capacity and active-count arguments are required")
        for name, value in (("token_capacity", token_capacity), ("sequence_capacity", sequence_capacity),
                            ("state_pool_size", state_pool_size), ("max_seqlen_capacity", max_seqlen_capacity)):
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        for name, value in (("num_active_tokens", num_active_tokens),
                            ("num_active_sequences", num_active_sequences)):
            if (not isinstance(value, torch.Tensor) or value.dtype != torch.int32 or not value.is_cuda
                    or not value.is_contiguous() or value.numel() != 1 or value.device != cu_seqlens.device):
                raise ValueError(f"{name} must be a one-element contiguous CUDA int32 tensor")
        return _extension().prepare_tmix_wkv7_recurrent_graph_metadata(
            cu_seqlens, state_indices, num_active_tokens, num_active_sequences, token_capacity,
            sequence_capacity, state_pool_size, max_seqlen_capacity)
    if total_tokens is None:
        raise ValueError("total_tokens is required for static recurrent metadata")
    return _extension().prepare_tmix_wkv7_recurrent_metadata(
        cu_seqlens, state_indices, total_tokens, state_pool_size, -1 if max_seqlen is None else int(max_seqlen))


def _ticket_for(r, state, cu_seqlens, state_indices, max_seqlen, validated_metadata):
    if validated_metadata is not None:
        return validated_metadata
    return prepare_tmix_wkv7_recurrent_metadata(
        cu_seqlens, state_indices, total_tokens=r.shape[0], state_pool_size=state.shape[0],
        max_seqlen=max_seqlen)


def infer_tmix_wkv7_recurrent_fp32io16_forward_varlen(
    r: torch.Tensor,
    decay_logits: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    state_pool: torch.Tensor,
    cu_seqlens: torch.Tensor,
    state_indices: torch.Tensor,
    scale: float = 1.0,
    decay_bias: torch.Tensor | None = None,
    max_seqlen: int | None = None,
    validated_metadata: object | None = None,
    decay_mode: str = "logits",
    output_f32: torch.Tensor | None = None,
) -> torch.Tensor:
    """Run the packed RWKV-7 recurrence in place on ``state_pool`` and return y.
    Reference: flashrwkv2/tmix/wkv7/__init__.py:179-256."""
    packed = _validate_packed_inputs(r, decay_logits, k, v, a, b)
    _validate_state(state_pool)
    _check_metadata_inputs(cu_seqlens, state_indices)
    ticket = _ticket_for(r, state_pool, cu_seqlens, state_indices, max_seqlen, validated_metadata)
    output = torch.empty_like(packed[3])
    _extension().tmix_wkv7_recurrent_fp32_from_decay_logits(
        cu_seqlens, state_indices, state_pool, *packed, output, float(scale), decay_bias, ticket,
        -1 if max_seqlen is None else int(max_seqlen), decay_mode, output_f32)
    return output


def infer_tmix_wkv7_prefill_fp32io16_forward_varlen(
    r: torch.Tensor,
    decay_logits: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    state_pool: torch.Tensor,
    cu_seqlens: torch.Tensor,
    state_indices: torch.Tensor,
    scale: float = 1.0,
    decay_bias: torch.Tensor | None = None,
    max_seqlen: int | None = None,
    validated_metadata: object | None = None,
    decay_mode: str = "logits",
    strategy: str = "auto",
    output_f32: torch.Tensor | None = None,
    error_flag: torch.Tensor | None = None,
) -> torch.Tensor:
    """Same contract as :func:`infer_tmix_wkv7_recurrent_fp32io16_forward_varlen` (in place on
    ``state_pool``, returns y) for long and ragged rows: 64-row chunks on the tensor cores with
    the state carried in fp32.  No counterpart with this signature exists in the reference (its
    chunk operator takes host-built per-chunk metadata); see
    :func:`flashrwkv2_b200.tmix.wkv7.rl_infctx.rl_infctx_tmix_wkv7_chunk_fp32io16` for that one."""
    packed = _validate_packed_inputs(r, decay_logits, k, v, a, b)
    _validate_state(state_pool)
    _check_metadata_inputs(cu_seqlens, state_indices)
    ticket = _ticket_for(r, state_pool, cu_seqlens, state_indices, max_seqlen, validated_metadata)
    output = torch.empty_like(packed[3])
    _extension().tmix_wkv7_prefill_fp32(
        cu_seqlens, state_indices, state_pool, *packed, output, float(scale), decay_bias, ticket,
        -1 if max_seqlen is None else int(max_seqlen), decay_mode, strategy, output_f32, error_flag)
    return output


from .rl_infctx import rl_infctx_tmix_wkv7_chunk_fp32io16  # noqa: E402

__all__ = [
    "infer_tmix_wkv7_prefill_fp32io16_forward_varlen",
    "infer_tmix_wkv7_recurrent_fp32io16_forward_varlen",
    "prepare_tmix_wkv7_recurrent_metadata",
    "rl_infctx_tmix_wkv7_chunk_fp32io16",
]
