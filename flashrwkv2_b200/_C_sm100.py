"""The sm_100a native backend module: FlashRWKV2's private-extension surface over the C ABI.

It exports the names, argument order, defaults and error behaviour of the reference's
pybind module for the WKV7 path (rwkv-rs/FlashRWKV2
csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cpp:227-458 and
csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cpp:158-241), so the reference's
Python wrappers work against it unchanged; argument errors are ``RuntimeError`` with the
reference's message fragments (csrc/validation.cpp:27-129).  All arithmetic happens in
libfrwkv_sm100.so; this module validates, builds tickets and passes raw device pointers
and the current CUDA stream through ctypes.  Additions over the reference surface:
``decay_mode`` ("logits" | "retention"), an optional fp32 ``output_f32`` (the output before
rounding), and ``tmix_wkv7_prefill_fp32`` which takes ``cu_seqlens`` directly.
"""

from __future__ import annotations

import math

import torch

from . import _lib

_IO = {torch.bfloat16: _lib.IO_BF16, torch.float16: _lib.IO_FP16}
_IO_WITH_FP32 = {**_IO, torch.float32: _lib.IO_FP32}
_DECAY = {"logits": _lib.DECAY_LOGITS, "retention": _lib.DECAY_RETENTION}
_STRATEGY = {"auto": _lib.PREFILL_AUTO, "recurrent": _lib.PREFILL_RECURRENT, "chunk_tc": _lib.PREFILL_CHUNK_TC}
_INT32_MAX = 2**31 - 1
HEAD_SIZE = 64

_lib.load()  # fail at import when the library is missing: there is nothing to fall back to


def _check(cond: bool, message: str) -> None:
    if not cond:
        raise RuntimeError(message)


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def _check_cuda_contiguous(t, name: str) -> None:
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be CUDA")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _check_recurrent_layout(query_start_loc, state_indices, state, r, w, k, v, a, b, output, scale,
                            allow_fp32_tokens: bool = False):
    """Host argument contract; csrc/validation.cpp:27-129 of the reference (D = 64 only here)."""
    named = (("query_start_loc", query_start_loc), ("state_indices", state_indices), ("state", state),
             ("r", r), ("decay_logits", w), ("k", k), ("v", v), ("a", a), ("b", b), ("output", output))
    for name, t in named:
        _check_cuda_contiguous(t, name)
    _check(query_start_loc.dtype == torch.int32, "query_start_loc must be int32")
    _check(state_indices.dtype == torch.int32, "state_indices must be int32")
    _check(math.isfinite(float(scale)), "scale must be finite")
    n = state_indices.numel()
    _check(0 < n <= 65535, "state_indices must contain 1..65535 sequences")
    _check(state_indices.dim() == 1, "state_indices must have shape [N]")
    _check(query_start_loc.dim() == 1 and query_start_loc.shape[0] == n + 1,
           "query_start_loc must have shape [N+1]")
    _check(state.dim() == 4 and state.shape[0] > 0 and state.shape[1] > 0 and state.shape[2] == state.shape[3],
           "state must have square shape [slots,H,D,D]")
    _check(state.dtype == torch.float32, "state must be float32")
    d = state.shape[2]
    _check(d in (64, 128, 256), f"recurrent head size must be 64, 128, or 256, got {d}")
    _check(d == HEAD_SIZE, f"the sm_100a backend implements head size 64 only, got {d}")
    _check(state.shape[0] <= _INT32_MAX, "state slot count must fit in int32")
    h = state.shape[1]
    _check(r.dim() == 3 and r.shape[0] > 0 and r.shape[1] == h and r.shape[2] == d,
           "r must have shape [total_tokens,H,D] matching state")
    _check(r.shape[0] <= _INT32_MAX, "token count must fit in int32")
    _check(all(t.shape == r.shape for t in (w, k, v, a, b, output)),
           "r,decay_logits,k,v,a,b,output shape mismatch")
    allowed = _IO_WITH_FP32 if allow_fp32_tokens else _IO
    _check(r.dtype in allowed, "token tensors must be float16 or bfloat16")
    _check(all(t.dtype == r.dtype for t in (w, k, v, a, b, output)),
           "r,decay_logits,k,v,a,b,output dtype mismatch")
    for name, t in named:
        _check(t.device == state.device, f"{name} must be on the same device as state")
    return n, h, d


def _check_decay_bias(decay_bias, state, r) -> None:
    if decay_bias is None:
        return
    _check_cuda_contiguous(decay_bias, "decay_bias")
    _check(decay_bias.device == state.device, "decay_bias must be on the same device as state")
    _check(decay_bias.dtype == r.dtype, "decay_bias must match the token tensor dtype")
    h, d = state.shape[1], state.shape[2]
    _check((decay_bias.dim() == 1 and decay_bias.numel() == h * d)
           or (decay_bias.dim() == 2 and tuple(decay_bias.shape) == (h, d)),
           "decay_bias must have shape [H*D] or [H,D]")


def _version(t: torch.Tensor):
    return None if t.is_inference() else t._version


class _RecurrentMetadataTicket:
    """Validated packed-sequence metadata bound to one stream; the counterpart of
    RecurrentMetadataTicket (infer_recurrent_fp32io16_forward_varlen.cpp:89-225)."""

    def __init__(self, query_start_loc, state_indices, cu_snapshot, slots_snapshot, status, workspace,
                 num_active_tokens, num_active_sequences, total_tokens, state_pool_size, max_seqlen,
                 graph_mode, stream):
        self._cu, self._slots = query_start_loc, state_indices
        self._cu_snap, self._slots_snap = cu_snapshot, slots_snapshot
        self._status_t, self._workspace = status, workspace
        self._n_tok, self._n_seq = num_active_tokens, num_active_sequences
        self._cu_version, self._slots_version = _version(query_start_loc), _version(state_indices)
        self._cu_ptr, self._slots_ptr = query_start_loc.data_ptr(), state_indices.data_ptr()
        self._cu_geom = (tuple(query_start_loc.shape), tuple(query_start_loc.stride()))
        self._slots_geom = (tuple(state_indices.shape), tuple(state_indices.stride()))
        self._total_tokens, self._pool_size, self._max = int(total_tokens), int(state_pool_size), int(max_seqlen)
        self._graph, self._device, self._stream_handle = bool(graph_mode), query_start_loc.device, stream

    def _check_compatible(self, query_start_loc, state_indices, total_tokens, state_pool_size, max_seqlen):
        _check(query_start_loc is self._cu, "validated_metadata query_start_loc identity mismatch")
        _check(state_indices is self._slots, "validated_metadata state_indices identity mismatch")
        _check(query_start_loc.data_ptr() == self._cu_ptr and state_indices.data_ptr() == self._slots_ptr,
               "validated_metadata metadata data_ptr mismatch")
        _check((tuple(query_start_loc.shape), tuple(query_start_loc.stride())) == self._cu_geom
               and (tuple(state_indices.shape), tuple(state_indices.stride())) == self._slots_geom,
               "validated_metadata metadata shape or stride mismatch")
        if not self._graph and self._cu_version is not None:
            _check(_version(query_start_loc) == self._cu_version,
                   "validated_metadata query_start_loc version mismatch")
        if not self._graph and self._slots_version is not None:
            _check(_version(state_indices) == self._slots_version,
                   "validated_metadata state_indices version mismatch")
        _check(query_start_loc.device == self._device and state_indices.device == self._device,
               "validated_metadata device mismatch")
        _check(int(total_tokens) == self._total_tokens, "validated_metadata total_tokens mismatch")
        _check(int(state_pool_size) == self._pool_size, "validated_metadata state_pool_size mismatch")
        if max_seqlen > 0:
            _check(int(max_seqlen) == self._max, "validated_metadata max_seqlen mismatch")
        _check(_stream(self._device) == self._stream_handle,
               "validated_metadata stream mismatch; prepare and consume the ticket on the same CUDA stream")

    def _query_start_loc_snapshot(self):
        return self._cu_snap

    def _state_indices_snapshot(self):
        return self._slots_snap

    def _status(self):
        return self._status_t

    def _max_seqlen(self):
        return self._max

    def _is_graph(self):
        return self._graph

    def _num_active_tokens(self):
        return self._n_tok

    def _num_active_sequences(self):
        return self._n_seq


def _check_metadata_tensors(query_start_loc, state_indices) -> None:
    _check_cuda_contiguous(query_start_loc, "query_start_loc")
    _check_cuda_contiguous(state_indices, "state_indices")
    _check(state_indices.device == query_start_loc.device, "state_indices must be on the same device as state")
    _check(query_start_loc.dtype == torch.int32 and state_indices.dtype == torch.int32,
           "recurrent metadata must be int32")


def _host_check_metadata(query_start_loc, state_indices, total_tokens, state_pool_size) -> int:
    """Static tickets validate on the host too and raise, like the reference
    (infer_recurrent_fp32io16_forward_varlen.cpp:45-80); one D2H copy, vectorised."""
    cu = query_start_loc.cpu().numpy()
    slots = state_indices.cpu().numpy()
    n = slots.shape[0]
    _check(int(cu[0]) == 0, "query_start_loc must start at 0")
    _check(int(cu[n]) == total_tokens, "the final query_start_loc offset must equal total_tokens")
    lo, hi = cu[:-1].astype("int64"), cu[1:].astype("int64")
    _check(bool(((lo >= 0) & (hi > lo) & (hi <= total_tokens)).all()),
           "query_start_loc must be strictly increasing with non-empty sequences")
    _check(bool(((slots >= 0) & (slots < state_pool_size)).all()),
           "state_indices entries must be within the state pool")
    import numpy as np

    _check(np.unique(slots).shape[0] == n, "state_indices must be unique within one call")
    return int((hi - lo).max())


def _launch_validation(query_start_loc, state_indices, n_tok, n_seq, token_capacity, seq_capacity,
                       state_pool_size, max_seqlen, snapshot: bool):
    device = query_start_loc.device
    with torch.cuda.device(device):
        status = torch.empty(3, dtype=torch.int32, device=device)
        seen = torch.empty(state_pool_size, dtype=torch.int32, device=device)
        cu_snap = torch.empty_like(query_start_loc) if snapshot else query_start_loc
        slots_snap = torch.empty_like(state_indices) if snapshot else state_indices
        _lib.check(_lib.load().frwkv_sm100_wkv7_validate_metadata(
            query_start_loc.data_ptr(), state_indices.data_ptr(), int(seq_capacity), int(token_capacity),
            int(state_pool_size), int(max_seqlen), _ptr(n_tok), _ptr(n_seq), status.data_ptr(),
            seen.data_ptr(), cu_snap.data_ptr() if snapshot else 0, slots_snap.data_ptr() if snapshot else 0,
            _stream(device)))
    return cu_snap, slots_snap, status, seen


def prepare_tmix_wkv7_recurrent_metadata(query_start_loc, state_indices, total_tokens, state_pool_size,
                                         max_seqlen=-1):
    """Static ticket: host + device validation, snapshots; one host sync."""
    _check_metadata_tensors(query_start_loc, state_indices)
    _check(query_start_loc.dim() == 1 and state_indices.dim() == 1 and state_indices.numel() > 0
           and query_start_loc.numel() == state_indices.numel() + 1,
           "query_start_loc must have shape [B+1] and state_indices shape [B]")
    _check(state_indices.numel() <= 65535, "state_indices must contain at most 65535 sequences")
    _check(0 < total_tokens <= _INT32_MAX, "total_tokens must be positive and fit in int32")
    _check(0 < state_pool_size <= _INT32_MAX, "state_pool_size must be positive and fit in int32")
    inferred = _host_check_metadata(query_start_loc, state_indices, int(total_tokens), int(state_pool_size))
    if max_seqlen <= 0:
        max_seqlen = inferred
    else:
        _check(int(max_seqlen) == inferred, "max_seqlen must equal the largest packed sequence length")
    cu_snap, slots_snap, status, seen = _launch_validation(
        query_start_loc, state_indices, None, None, total_tokens, state_indices.numel(), state_pool_size,
        total_tokens, snapshot=True)
    return _RecurrentMetadataTicket(query_start_loc, state_indices, cu_snap, slots_snap, status, seen, None, None,
                                    total_tokens, state_pool_size, max_seqlen, False,
                                    _stream(query_start_loc.device))


def _check_graph_scalar(t, ref, name: str) -> None:
    _check(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")
    _check(t.device == ref.device, f"{name} must share the metadata CUDA device")
    _check(t.dtype == torch.int32, f"{name} must have dtype int32")
    _check(t.numel() == 1, f"{name} must contain one element")


def prepare_tmix_wkv7_recurrent_graph_metadata(query_start_loc, state_indices, num_active_tokens,
                                               num_active_sequences, token_capacity, sequence_capacity,
                                               state_pool_size, max_seqlen_capacity):
    """Capacity ticket: live metadata and live active counts, device validation only, no host
    sync -- usable for same-stream warm-up and inside CUDA-graph capture."""
    _check_metadata_tensors(query_start_loc, state_indices)
    _check(0 < sequence_capacity <= 65535 and state_indices.dim() == 1
           and state_indices.numel() == sequence_capacity and query_start_loc.dim() == 1
           and query_start_loc.numel() == sequence_capacity + 1,
           "graph metadata shapes must match sequence_capacity")
    _check(0 < token_capacity <= _INT32_MAX, "token_capacity must be positive and fit in int32")
    _check(0 < state_pool_size <= _INT32_MAX, "state_pool_size must be positive and fit in int32")
    _check(0 < max_seqlen_capacity <= token_capacity,
           "max_seqlen_capacity must be positive and not exceed token_capacity")
    _check_graph_scalar(num_active_tokens, query_start_loc, "num_active_tokens")
    _check_graph_scalar(num_active_sequences, query_start_loc, "num_active_sequences")
    cu_snap, slots_snap, status, seen = _launch_validation(
        query_start_loc, state_indices, num_active_tokens, num_active_sequences, token_capacity,
        sequence_capacity, state_pool_size, max_seqlen_capacity, snapshot=False)
    return _RecurrentMetadataTicket(query_start_loc, state_indices, cu_snap, slots_snap, status, seen,
                                    num_active_tokens, num_active_sequences, token_capacity, state_pool_size,
                                    max_seqlen_capacity, True, _stream(query_start_loc.device))


def _resolve_metadata(query_start_loc, state_indices, state, r, validated_metadata, max_seqlen):
    if validated_metadata is not None:
        validated_metadata._check_compatible(query_start_loc, state_indices, r.shape[0], state.shape[0],
                                             max_seqlen)
        return (validated_metadata._query_start_loc_snapshot(), validated_metadata._state_indices_snapshot(),
                validated_metadata._status(), validated_metadata._max_seqlen(), validated_metadata)
    # un-ticketed native call: device validation only (the host-raising check lives in the
    # static prepare entry, as in the reference binding :375-381)
    cu_snap, slots_snap, status, seen = _launch_validation(
        query_start_loc, state_indices, None, None, r.shape[0], state_indices.numel(), state.shape[0],
        r.shape[0], snapshot=True)
    return cu_snap, slots_snap, status, int(max_seqlen), (cu_snap, slots_snap, status, seen)


def _check_output_f32(output_f32, output) -> None:
    if output_f32 is None:
        return
    _check_cuda_contiguous(output_f32, "output_f32")
    _check(output_f32.dtype == torch.float32 and output_f32.shape == output.shape
           and output_f32.device == output.device, "output_f32 must be a float32 tensor shaped like output")


def tmix_wkv7_recurrent_fp32_from_decay_logits(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b,
                                               output, scale, decay_bias=None, validated_metadata=None,
                                               max_seqlen=-1, decay_mode="logits", output_f32=None):
    """In-place recurrence on ``state`` (register-streaming kernel).  Reference entry:
    infer_recurrent_fp32io16_forward_varlen.cpp:330-387."""
    _check(decay_mode in _DECAY, "decay_mode must be 'logits' or 'retention'")
    n, h, _ = _check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b, output,
                                      scale, allow_fp32_tokens=True)
    _check_decay_bias(decay_bias, state, r)
    _check(decay_bias is None or decay_mode == "logits", "decay_bias only applies to decay logits")
    _check_output_f32(output_f32, output)
    cu, slots, status, max_seqlen, keep = _resolve_metadata(query_start_loc, state_indices, state, r,
                                                            validated_metadata, max_seqlen)
    with torch.cuda.device(state.device):
        _lib.check(_lib.load().frwkv_sm100_wkv7_recurrent(
            cu.data_ptr(), slots.data_ptr(), status.data_ptr(), state.data_ptr(), r.data_ptr(),
            decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(), _ptr(decay_bias),
            output.data_ptr(), _ptr(output_f32), n, r.shape[0], h, _IO_WITH_FP32[r.dtype], _DECAY[decay_mode],
            float(scale), int(max_seqlen), _stream(state.device)))
    del keep


def tmix_wkv7_prefill_fp32(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b, output, scale,
                           decay_bias=None, validated_metadata=None, max_seqlen=-1, decay_mode="logits",
                           strategy="auto", output_f32=None, error_flag=None):
    """In-place prefill on ``state`` taking ``cu_seqlens`` directly (no host chunk metadata).
    ``strategy``: "auto" | "recurrent" | "chunk_tc"."""
    _check(decay_mode in _DECAY, "decay_mode must be 'logits' or 'retention'")
    _check(strategy in _STRATEGY, "strategy must be 'auto', 'recurrent' or 'chunk_tc'")
    n, h, _ = _check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b, output,
                                      scale, allow_fp32_tokens=True)
    _check_decay_bias(decay_bias, state, r)
    _check(decay_bias is None or decay_mode == "logits", "decay_bias only applies to decay logits")
    _check_output_f32(output_f32, output)
    if error_flag is not None:
        _check(error_flag.is_cuda and error_flag.dtype == torch.int32 and error_flag.numel() >= 1,
               "error_flag must be a CUDA int32 tensor")
    cu, slots, status, max_seqlen, keep = _resolve_metadata(query_start_loc, state_indices, state, r,
                                                            validated_metadata, max_seqlen)
    lib = _lib.load()
    with torch.cuda.device(state.device):
        need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n, r.shape[0], h)
        workspace = torch.empty(need, dtype=torch.uint8, device=state.device) if need else None
        _lib.check(lib.frwkv_sm100_wkv7_prefill(
            cu.data_ptr(), slots.data_ptr(), status.data_ptr(), state.data_ptr(), r.data_ptr(),
            decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(), _ptr(decay_bias),
            output.data_ptr(), _ptr(output_f32), n, r.shape[0], h, _IO_WITH_FP32[r.dtype], _DECAY[decay_mode],
            float(scale), int(max_seqlen), _STRATEGY[strategy], _ptr(workspace), int(need), _ptr(error_flag),
            _stream(state.device)))
    del keep


def rl_infctx_tmix_wkv7_chunk_fp32io16_forward(sequence_chunk_offsets, chunk_token_starts, chunk_token_ends, state,
                                               r, decay_logits, k, v, a, b, strategy=1, scale=1.0,
                                               decay_bias=None, decay_mode="logits"):
    """Reference-shaped chunk forward: ``state`` is [B,H,D,D] gathered working state; returns
    ``(output, final_state)`` and leaves ``state`` untouched
    (rl_infctx_chunk_fp32io16_forward.cpp:158-230).  The reference's per-chunk host metadata is
    accepted for signature compatibility; only the sequence boundaries it encodes are used (the
    kernel always works in 64-row chunks), and they are recovered on the device without a sync.
    ``strategy`` 0 ("materialized") and 1 ("recompute") both map to the single fused kernel."""
    _check(strategy in (0, 1), "strategy must be 0 (materialized) or 1 (recompute)")
    _check(isinstance(state, torch.Tensor) and state.is_cuda and state.is_contiguous()
           and state.dtype == torch.float32, "RL/Infctx state must be contiguous CUDA float32")
    _check(state.dim() == 4 and state.shape[0] > 0 and state.shape[1] > 0 and state.shape[2] == state.shape[3]
           and state.shape[2] in (64, 128, 256), "RL/Infctx state must have shape [B,H,D,D], D in {64,128,256}")
    for name, t in (("sequence_chunk_offsets", sequence_chunk_offsets), ("chunk_token_starts", chunk_token_starts),
                    ("chunk_token_ends", chunk_token_ends)):
        _check_cuda_contiguous(t, name)
        _check(t.dtype == torch.int32 and t.dim() == 1, f"{name} must be a one-dimensional int32 tensor")
    _check(chunk_token_starts.shape == chunk_token_ends.shape and chunk_token_starts.numel() > 0,
           "chunk token metadata must have matching shape [C]")
    _check(sequence_chunk_offsets.numel() == state.shape[0] + 1, "query_start_loc must have shape [N+1]")
    working = state.clone()
    output = torch.empty_like(v)
    slots = torch.arange(state.shape[0], dtype=torch.int32, device=state.device)
    starts_ext = torch.cat((chunk_token_starts, chunk_token_ends[-1:]))
    cu = starts_ext.index_select(0, sequence_chunk_offsets.to(torch.int64)).contiguous()
    tmix_wkv7_prefill_fp32(cu, slots, working, r, decay_logits, k, v, a, b, output, scale, decay_bias, None, -1,
                           decay_mode, "auto")
    return output, working
