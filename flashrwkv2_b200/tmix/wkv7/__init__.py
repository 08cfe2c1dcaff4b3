"""Public WKV7 operators: the reference's ``flashrwkv2.tmix.wkv7`` contract on B200.

Names, keyword arguments and error types are those of rwkv-rs/FlashRWKV2
flashrwkv2/tmix/wkv7/__init__.py:91-256: ``TypeError`` / ``ValueError`` from these wrappers before
any launch, ``RuntimeError`` from the native layer.  Extra optional keywords: ``decay_mode``
("logits" as in the reference, or "retention" when ``w`` already is the per-channel retention),
``output_f32`` (fp32 copy of the output before rounding) and, for prefill, ``strategy`` and
``error_flag``.
"""

from __future__ import annotations

import torch

from . import _checks as check


def _extension():
    """The loaded native module; there is nothing to fall back to when it is absent."""
    import flashrwkv2_b200

    native = getattr(flashrwkv2_b200, "_C", None)
    if native is None:
        raise RuntimeError(
            "flashrwkv2_b200 CUDA backend is not loaded (no CUDA device, or the extension is not "
            "built); the WKV7 operators have no CPU fallback")
    return native


_CAPACITY_KEYS = ("token_capacity", "sequence_capacity", "max_seqlen_capacity", "num_active_tokens",
                  "num_active_sequences")


def prepare_tmix_wkv7_recurrent_metadata(cu_seqlens: torch.Tensor, state_indices: torch.Tensor, *,
                                         state_pool_size: int, total_tokens: int | None = None,
                                         max_seqlen: int | None = None, **capacity) -> object:
    """Validate packed-sequence metadata once and return a ticket for later calls on the same stream.

    Two forms, as in the reference (flashrwkv2/tmix/wkv7/__init__.py:91-176):

    * static -- pass ``total_tokens`` (and optionally ``max_seqlen``): the metadata is snapshotted and
      checked on the host and on the device; invalid metadata raises here (one host sync);
    * capacity -- pass all of ``token_capacity``, ``sequence_capacity``, ``max_seqlen_capacity``,
      ``num_active_tokens``, ``num_active_sequences``: buffers and the two active-count scalars stay
      live, validation runs on the device only, nothing synchronises, so the call can be made with
      zero active counts for warm-up and again inside CUDA-graph capture.
    """
    unknown = set(capacity) - set(_CAPACITY_KEYS)
    if unknown:
        raise TypeError(f"prepare_tmix_wkv7_recurrent_metadata() got an unexpected keyword argument "
                        f"'{sorted(unknown)[0]}'")
    check.metadata(cu_seqlens, state_indices)
    given = {key: capacity.get(key) for key in _CAPACITY_KEYS}
    if all(value is None for value in given.values()):
        check.need(total_tokens is not None, ValueError, "total_tokens is required for static recurrent metadata")
        return _extension().prepare_tmix_wkv7_recurrent_metadata(
            cu_seqlens, state_indices, total_tokens, state_pool_size, -1 if max_seqlen is None else int(max_seqlen))
    check.need(total_tokens is None and max_seqlen is None, ValueError,
               "graph metadata uses capacity arguments, not total_tokens/max_seqlen")
    check.need(all(value is not None for value in given.values()), ValueError,
               "all graph metadata capacity and active-count arguments are required")
    for key in ("token_capacity", "sequence_capacity", "max_seqlen_capacity"):
        check.positive_int(given[key], key)
    check.positive_int(state_pool_size, "state_pool_size")
    for key in ("num_active_tokens", "num_active_sequences"):
        check.device_scalar(given[key], key, cu_seqlens.device)
    return _extension().prepare_tmix_wkv7_recurrent_graph_metadata(
        cu_seqlens, state_indices, given["num_active_tokens"], given["num_active_sequences"],
        given["token_capacity"], given["sequence_capacity"], state_pool_size, given["max_seqlen_capacity"])


def _launch(native_name: str, tokens, *, state_pool, cu_seqlens, state_indices, scale, decay_bias, max_seqlen,
            validated_metadata, extra):
    """Shared body of the two in-place operators: check, obtain a ticket, allocate y, call native."""
    check.packed_tokens(tokens)
    check.fp32_pool(state_pool)
    check.metadata(cu_seqlens, state_indices)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_tmix_wkv7_recurrent_metadata(
            cu_seqlens, state_indices, total_tokens=tokens[0].shape[0], state_pool_size=state_pool.shape[0],
            max_seqlen=max_seqlen)
    y = torch.empty_like(tokens[3])
    getattr(_extension(), native_name)(
        cu_seqlens, state_indices, state_pool, *tokens, y, float(scale), decay_bias, ticket,
        -1 if max_seqlen is None else int(max_seqlen), *extra)
    return y


def infer_tmix_wkv7_recurrent_fp32io16_forward_varlen(
        r: torch.Tensor, decay_logits: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
        b: torch.Tensor, *, state_pool: torch.Tensor, cu_seqlens: torch.Tensor, state_indices: torch.Tensor,
        scale: float = 1.0, decay_bias: torch.Tensor | None = None, max_seqlen: int | None = None,
        validated_metadata: object | None = None, decay_mode: str = "logits",
        output_f32: torch.Tensor | None = None) -> torch.Tensor:
    """Packed RWKV-7 recurrence, in place on ``state_pool`` at ``state_indices``; returns y.
    Decode steps and short rows (register-streaming kernel).  Reference:
    flashrwkv2/tmix/wkv7/__init__.py:179-256."""
    return _launch("tmix_wkv7_recurrent_fp32_from_decay_logits", (r, decay_logits, k, v, a, b),
                   state_pool=state_pool, cu_seqlens=cu_seqlens, state_indices=state_indices, scale=scale,
                   decay_bias=decay_bias, max_seqlen=max_seqlen, validated_metadata=validated_metadata,
                   extra=(decay_mode, output_f32))


def infer_tmix_wkv7_prefill_fp32io16_forward_varlen(
        r: torch.Tensor, decay_logits: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
        b: torch.Tensor, *, state_pool: torch.Tensor, cu_seqlens: torch.Tensor, state_indices: torch.Tensor,
        scale: float = 1.0, decay_bias: torch.Tensor | None = None, max_seqlen: int | None = None,
        validated_metadata: object | None = None, decay_mode: str = "logits", strategy: str = "auto",
        output_f32: torch.Tensor | None = None, error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """Same contract for long and ragged rows: chunks on the tensor cores, state carried in fp32, in
    place on ``state_pool``.  The reference has no operator with this signature (its chunk operator
    takes host-built per-chunk metadata and returns a new pool: see
    :func:`flashrwkv2_b200.tmix.wkv7.rl_infctx.rl_infctx_tmix_wkv7_chunk_fp32io16`).

    ``strategy``: "auto" (tensor-core chunk kernel for 16-bit tokens and rows of 16 tokens or more, the recurrence
    for the rest), "chunk_tc" or "recurrent".  Limits of the chunk kernel: it agrees with the fp32 recurrence to
    1-2.5e-3 of the output's RMS (5e-3 is the stated gate); in ``decay_mode="retention"`` the product of the
    retentions over a 32-row chunk must stay above 1e-36 (any retention RWKV-7 can produce, >= 0.545 per token, does).
    ``error_flag`` (one int32 on the device, zeroed by the caller) receives bit 1 when that range is left (the
    output is then invalid) and bit 0 when a bounded device wait gave up (that (sequence, head)'s rows are NaN and its
    state slot keeps its old value)."""
    return _launch("tmix_wkv7_prefill_fp32", (r, decay_logits, k, v, a, b), state_pool=state_pool,
                   cu_seqlens=cu_seqlens, state_indices=state_indices, scale=scale, decay_bias=decay_bias,
                   max_seqlen=max_seqlen, validated_metadata=validated_metadata,
                   extra=(decay_mode, strategy, output_f32, error_flag))


def infer_tmix_wkv7_recurrent_fp16_forward_varlen(
        r: torch.Tensor, decay_logits: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
        b: torch.Tensor, *, state_pool: torch.Tensor, elapsed_state_pool: torch.Tensor, cu_seqlens: torch.Tensor,
        state_indices: torch.Tensor, scale: float = 1.0, decay_bias: torch.Tensor | None = None,
        max_seqlen: int | None = None, validated_metadata: object | None = None) -> torch.Tensor:
    """Packed recurrence with an fp16 state pool (half the state traffic of the fp32 contract): fp16 tokens, decay
    applied as ``state + state * delta`` with a dithered fp16 delta, state rounded to fp16 after every token, in
    place on ``state_pool``; ``elapsed_state_pool`` (int32 ``[slots]``) supplies the dither phase and advances by
    each sequence's token count.  Reference: flashrwkv2/tmix/wkv7/__init__.py:259-318 (same signature, checks
    and error types)."""
    tokens = (r, decay_logits, k, v, a, b)
    check.packed_tokens(tokens)
    check.tensor(state_pool, "state_pool")
    check.need(state_pool.is_contiguous(), ValueError, "state_pool must be contiguous")
    check.need(state_pool.dtype == torch.float16, TypeError, "FP16-state state_pool must have dtype float16")
    check.tensor(elapsed_state_pool, "elapsed_state_pool")
    check.need(elapsed_state_pool.dtype == torch.int32, TypeError, "elapsed_state_pool must have dtype torch.int32")
    check.need(elapsed_state_pool.is_cuda and elapsed_state_pool.is_contiguous(), ValueError,
               "elapsed_state_pool must be contiguous CUDA int32")
    check.need(elapsed_state_pool.device == state_pool.device, ValueError,
               "elapsed_state_pool must share state_pool's device")
    check.need(elapsed_state_pool.ndim == 1 and elapsed_state_pool.shape[0] == state_pool.shape[0], ValueError,
               "elapsed_state_pool must have shape [state_pool_slots]")
    check.metadata(cu_seqlens, state_indices)
    if max_seqlen is not None:
        check.positive_int(max_seqlen, "max_seqlen")
    launch_max_seqlen = -1 if max_seqlen is None else int(max_seqlen)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_tmix_wkv7_recurrent_metadata(
            cu_seqlens, state_indices, total_tokens=r.shape[0], state_pool_size=state_pool.shape[0],
            max_seqlen=max_seqlen)
    y = torch.empty_like(v)
    _extension().tmix_wkv7_recurrent_fp16_from_decay_logits(
        cu_seqlens, state_indices, elapsed_state_pool, state_pool, *tokens, y, float(scale), decay_bias, ticket,
        launch_max_seqlen)
    return y


def infer_tmix_wkv7_fused_gate_fp32io16_forward_varlen(
        r: torch.Tensor, decay_logits: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a12: torch.Tensor, *,
        k_k: torch.Tensor, a0: torch.Tensor, k_a: torch.Tensor, state_pool: torch.Tensor, cu_seqlens: torch.Tensor,
        state_indices: torch.Tensor, scale: float = 1.0, decay_bias: torch.Tensor | None = None,
        max_seqlen: int | None = None, validated_metadata: object | None = None, decay_mode: str = "logits",
        strategy: str = "auto", output_f32: torch.Tensor | None = None,
        error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """The in-place WKV7 operators with the kk / a-gate producer fused into their load stage.

    The reference runs a separate kernel between the projections and WKV7 that writes three packed tensors
    (flashrwkv2 wkv_prepare, csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/infer_fp16_forward_varlen.cu:52-106):
    ``kk = normalize(k * k_k)`` per head, ``g = sigmoid(a0 + a12)``, ``a = -kk``, ``b = kk * g`` and the gated key
    ``k * (1 + (g - 1) * k_a)``.  Here ``k`` is the raw key projection and ``a12`` the per-token gate logits; the
    kernels form the three tensors in registers (rounded to the token dtype where the reference stores them), so they
    are never written to or read from HBM.  ``strategy="decode"`` uses the register-streaming recurrence (decode
    steps and short rows); "auto", "recurrent" and "chunk_tc" are the prefill strategies."""
    tokens = (r, decay_logits, k, v, a12, a12)
    check.packed_tokens(tokens)
    check.fp32_pool(state_pool)
    check.metadata(cu_seqlens, state_indices)
    for name, value in (("k_k", k_k), ("a0", a0), ("k_a", k_a)):
        check.tensor(value, name)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_tmix_wkv7_recurrent_metadata(
            cu_seqlens, state_indices, total_tokens=r.shape[0], state_pool_size=state_pool.shape[0],
            max_seqlen=max_seqlen)
    y = torch.empty_like(v)
    _extension().tmix_wkv7_fused_gate_fp32(
        cu_seqlens, state_indices, state_pool, r, decay_logits, k, v, a12, k_k, a0, k_a, y, float(scale), decay_bias,
        ticket, -1 if max_seqlen is None else int(max_seqlen), decay_mode, strategy, output_f32, error_flag)
    return y


def infer_tmix_wkv7_readout_fp32io16_forward_varlen(
        r: torch.Tensor, decay_logits: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor,
        b: torch.Tensor | None, *, gate: torch.Tensor, r_k: torch.Tensor, ln_weight: torch.Tensor,
        ln_bias: torch.Tensor, state_pool: torch.Tensor, cu_seqlens: torch.Tensor, state_indices: torch.Tensor,
        scale: float = 1.0, k_k: torch.Tensor | None = None, a0: torch.Tensor | None = None,
        k_a: torch.Tensor | None = None, decay_bias: torch.Tensor | None = None, max_seqlen: int | None = None,
        validated_metadata: object | None = None, decay_mode: str = "logits",
        wkv_output: torch.Tensor | None = None, output_f32: torch.Tensor | None = None,
        output_weight: torch.Tensor | None = None, strategy: str = "decode",
        error_flag: torch.Tensor | None = None) -> torch.Tensor:
    """The in-place WKV7 recurrence followed, in the same kernel, by the elementwise stage of the reference's readout
    (flashrwkv2/tmix/readout/__init__.py:10-77: head normalisation with eps 64e-5, ``sum(r*k*r_k) * v`` residual,
    output gate): the recurrence's y never makes the round trip through HBM and r, k, v are not read a second time.

    Returns the gated tensor ``[T, H, 64]`` that feeds the output projection, or, when ``output_weight`` ``[C, C]`` is
    given, the projected ``[T, C]`` result (a plain library GEMM, as in the reference).  ``wkv_output`` and
    ``output_f32``, when given, also receive the recurrence's own y.  With ``k_k``, ``a0`` and ``k_a`` the kk / a-gate
    producer is fused in as well (``k`` raw, ``a`` = gate logits a12, ``b`` ignored).  ``strategy="decode"`` (decode
    steps and short rows) runs the stage as the epilogue of the register-streaming kernel; "auto", "chunk_tc" and
    "recurrent" are the prefill strategies, behind which the stage is a second, HBM-bound launch over the stored y
    rows (the tensor-core chunk kernel is bound by CUDA-core instructions, so it carries no epilogue)."""
    fused = k_k is not None or a0 is not None or k_a is not None
    if fused and (k_k is None or a0 is None or k_a is None):
        raise ValueError("k_k, a0 and k_a must be given together")
    if not fused and b is None:
        raise ValueError("b is required unless the kk / a-gate parameters are given")
    check.packed_tokens((r, decay_logits, k, v, a, a if fused else b))
    check.fp32_pool(state_pool)
    check.metadata(cu_seqlens, state_indices)
    for name, value in (("gate", gate), ("r_k", r_k), ("ln_weight", ln_weight), ("ln_bias", ln_bias)):
        check.tensor(value, name)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_tmix_wkv7_recurrent_metadata(
            cu_seqlens, state_indices, total_tokens=r.shape[0], state_pool_size=state_pool.shape[0],
            max_seqlen=max_seqlen)
    out = torch.empty_like(v)
    _extension().tmix_wkv7_readout_fp32(
        cu_seqlens, state_indices, state_pool, r, decay_logits, k, v, a, None if fused else b, gate, r_k, ln_weight,
        ln_bias, out, float(scale), k_k, a0, k_a, decay_bias, ticket, -1 if max_seqlen is None else int(max_seqlen),
        decay_mode, wkv_output, output_f32, strategy, error_flag)
    if output_weight is not None:
        return torch.nn.functional.linear(out.reshape(out.shape[0], -1), output_weight)
    return out


from .pretrain import pretrain_tmix_wkv7_recurrent_bf16  # noqa: E402
from .rl_infctx import rl_infctx_tmix_wkv7_chunk_fp32io16  # noqa: E402

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
