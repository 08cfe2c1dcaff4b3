"""Metadata validation, tickets, fail-closed behaviour and CUDA-graph use on the GPU.

Shaped after rwkv-rs/FlashRWKV2 tests/tmix/wkv7/test.py:239-373 (graph capture with a
zero-active warm-up), :526-602 (rejection matrix, state unchanged), :692-766 (ticket
identity / version / stream) and :769-792 (low-level fail-closed).  Failures are injected
on the host (bad metadata); nothing here faults the device.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
NAMES = ("r", "decay_logits", "k", "v", "a", "b")


def _ops():
    import flashrwkv2_b200.tmix.wkv7 as mod

    return mod


def _case(lengths=(1, 15, 16, 17, 65), dtype=torch.bfloat16, heads=2, pool_slots=9, seed=20260804):
    g = torch.Generator().manual_seed(seed)
    total = sum(lengths)
    scales = (0.12, 3.5, 0.06, 0.06, 0.06, 0.06)
    case = {n: (torch.randn(total, heads, 64, generator=g) * s).to(dtype).to(DEV) for n, s in zip(NAMES, scales)}
    cu = [0]
    for length in lengths:
        cu.append(cu[-1] + length)
    case["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32, device=DEV)
    case["state_indices"] = torch.tensor([5, 0, 7, 2, 4][: len(lengths)], dtype=torch.int32, device=DEV)
    case["state_pool"] = (torch.randn(pool_slots, heads, 64, 64, generator=g) * 0.03).to(DEV)
    return case


def _args(case):
    return tuple(case[n] for n in NAMES)


KINDS = ["wrong_rank", "wrong_length", "wrong_dtype", "wrong_start", "wrong_end", "non_increasing",
         "empty_sequence", "wrong_slot_length", "duplicate_slot", "negative_slot", "out_of_range_slot"]


@pytest.mark.parametrize("kind", KINDS)
def test_public_rejects_invalid_metadata_and_preserves_state(kind):
    case = _case()
    cu, slots, pool = case["cu_seqlens"], case["state_indices"], case["state_pool"]
    bad_cu, bad_slots = cu, slots
    if kind == "wrong_rank":
        bad_cu = cu.reshape(1, -1)
    elif kind == "wrong_length":
        bad_cu = cu[:-1]
    elif kind == "wrong_dtype":
        bad_cu = cu.to(torch.int64)
    elif kind == "wrong_start":
        bad_cu = cu + 1
    elif kind == "wrong_end":
        bad_cu = cu.clone()
        bad_cu[-1] -= 1
    elif kind == "non_increasing":
        bad_cu = cu.clone()
        bad_cu[2] = bad_cu[1] - 1
    elif kind == "empty_sequence":
        bad_cu = cu.clone()
        bad_cu[2] = bad_cu[1]
    elif kind == "wrong_slot_length":
        bad_slots = slots[:-1]
    elif kind == "duplicate_slot":
        bad_slots = slots.clone()
        bad_slots[1] = bad_slots[0]
    elif kind == "negative_slot":
        bad_slots = slots.clone()
        bad_slots[0] = -1
    else:
        bad_slots = slots.clone()
        bad_slots[0] = pool.shape[0]
    before = pool.clone()
    with pytest.raises((TypeError, ValueError, RuntimeError)):
        _ops().infer_tmix_wkv7_recurrent_fp32io16_forward_varlen(
            *_args(case), state_pool=pool, cu_seqlens=bad_cu, state_indices=bad_slots)
    torch.cuda.synchronize()
    assert torch.equal(pool, before)


DEVICE_KINDS = {
    "wrong_start": 1 << 0, "wrong_end": 1 << 0, "non_increasing": 1 << 1, "empty_sequence": 1 << 1,
    "duplicate_slot": 1 << 3, "negative_slot": 1 << 2, "out_of_range_slot": 1 << 2, "too_long": 1 << 5,
    "bad_active": 1 << 4,
}


@pytest.mark.parametrize("kind", sorted(DEVICE_KINDS))
def test_device_validation_status_bits(kind):
    """The validation kernel alone, through the C ABI: status word per error kind."""
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    cu = torch.tensor([0, 1, 16, 32, 49, 114], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 0, 7, 2, 4], dtype=torch.int32, device=DEV)
    n_tok = torch.tensor([114], dtype=torch.int32, device=DEV)
    n_seq = torch.tensor([5], dtype=torch.int32, device=DEV)
    max_seqlen = 114
    if kind == "wrong_start":
        cu += 1
    elif kind == "wrong_end":
        cu[-1] -= 1
    elif kind == "non_increasing":
        cu[2] = cu[1] - 1
    elif kind == "empty_sequence":
        cu[2] = cu[1]
    elif kind == "duplicate_slot":
        slots[1] = slots[0]
    elif kind == "negative_slot":
        slots[0] = -1
    elif kind == "out_of_range_slot":
        slots[0] = 9
    elif kind == "too_long":
        max_seqlen = 64
    elif kind == "bad_active":
        n_seq.fill_(0)
    status = torch.full((3,), 77, dtype=torch.int32, device=DEV)
    seen = torch.empty(9, dtype=torch.int32, device=DEV)
    rc = lib.frwkv_sm100_wkv7_validate_metadata(cu.data_ptr(), slots.data_ptr(), 5, 114, 9, max_seqlen,
                                                n_tok.data_ptr(), n_seq.data_ptr(), status.data_ptr(),
                                                seen.data_ptr(), 0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    got = status.cpu().tolist()
    assert got[0] & DEVICE_KINDS[kind], got
    assert got[1] == 0 and got[2] == 0


def test_endpoint_bit_beside_range_errors_is_deterministic():
    """More than 32 sequences (so warps other than the first take part), a wrong end point and a broken range at
    once: as in the reference (csrc/validation/recurrent_metadata.cu:83-93) the end-point test is finished before
    any range error is recorded, so both bits are always reported, by the ordinary and by the static entry."""
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    n = 100
    cu_list = list(range(0, 2 * n + 1, 2))
    cu_list[-1] += 1          # wrong end point (the declared token count is 2n)
    cu_list[70] = cu_list[69]  # empty sequence 69 in a later warp
    cu = torch.tensor(cu_list, dtype=torch.int32, device=DEV)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(20):
        status = torch.full((3,), 77, dtype=torch.int32, device=DEV)
        seen = torch.empty(n, dtype=torch.int32, device=DEV)
        assert lib.frwkv_sm100_wkv7_validate_metadata(cu.data_ptr(), slots.data_ptr(), n, 2 * n, n, 2 * n, 0, 0,
                                                      status.data_ptr(), seen.data_ptr(), 0, 0, stream) == 0
        static = torch.full((3,), 77, dtype=torch.int32, device=DEV)
        assert lib.frwkv_sm100_wkv7_validate_metadata_static(cu.data_ptr(), slots.data_ptr(), n, 2 * n, n, 2 * n, 0, 0,
                                                             static.data_ptr(), 0, 0, stream) == 0
        assert status.cpu().tolist() == [1 | 2, 0, 0] and static.cpu().tolist() == [1 | 2, 0, 0]


def test_device_validation_accepts_valid_and_snapshots():
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    cu = torch.tensor([0, 1, 16, 32, 49, 114], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 0, 7, 2, 4], dtype=torch.int32, device=DEV)
    status = torch.full((3,), 77, dtype=torch.int32, device=DEV)
    seen = torch.empty(9, dtype=torch.int32, device=DEV)
    cu_snap, slots_snap = torch.zeros_like(cu), torch.zeros_like(slots)
    rc = lib.frwkv_sm100_wkv7_validate_metadata(cu.data_ptr(), slots.data_ptr(), 5, 114, 9, 114, 0, 0,
                                                status.data_ptr(), seen.data_ptr(), cu_snap.data_ptr(),
                                                slots_snap.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    assert status.cpu().tolist() == [0, 114, 5]
    assert torch.equal(cu_snap, cu) and torch.equal(slots_snap, slots)
    # rejected arguments launch nothing and say why
    rc = lib.frwkv_sm100_wkv7_validate_metadata(cu.data_ptr(), slots.data_ptr(), 70000, 114, 9, 114, 0, 0,
                                                status.data_ptr(), seen.data_ptr(), 0, 0, 0)
    assert rc != 0 and "65535" in _lib.last_error()


def test_ticket_rejects_identity_version_and_stream_mismatches():
    ops = _ops()
    case = _case(lengths=(4, 5))
    args = _args(case)
    cu, slots, pool = case["cu_seqlens"], case["state_indices"], case["state_pool"]
    ticket = ops.prepare_tmix_wkv7_recurrent_metadata(cu, slots, total_tokens=9, state_pool_size=pool.shape[0])
    assert not ticket._is_graph() and ticket._max_seqlen() == 5
    assert ticket._status().cpu().tolist() == [0, 9, 2]
    run = ops.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen
    with pytest.raises(RuntimeError, match="identity"):
        run(*args, state_pool=pool.clone(), cu_seqlens=cu.clone(), state_indices=slots, validated_metadata=ticket)
    short = tuple(t[:-1].contiguous() for t in args)
    with pytest.raises(RuntimeError, match="total_tokens"):
        run(*short, state_pool=pool.clone(), cu_seqlens=cu, state_indices=slots, validated_metadata=ticket)
    with pytest.raises(RuntimeError, match="state_pool_size"):
        run(*args, state_pool=torch.cat((pool, torch.zeros_like(pool[:1]))), cu_seqlens=cu, state_indices=slots,
            validated_metadata=ticket)
    cu[1] += 1
    with pytest.raises(RuntimeError, match="version"):
        run(*args, state_pool=pool.clone(), cu_seqlens=cu, state_indices=slots, validated_metadata=ticket)
    cu[1] -= 1
    ticket2 = ops.prepare_tmix_wkv7_recurrent_metadata(cu, slots, total_tokens=9, state_pool_size=pool.shape[0])
    other = torch.cuda.Stream()
    with torch.cuda.stream(other), pytest.raises(RuntimeError, match="stream"):
        run(*args, state_pool=pool.clone(), cu_seqlens=cu, state_indices=slots, validated_metadata=ticket2)
    other.synchronize()
    with pytest.raises(RuntimeError, match="max_seqlen"):
        ops.prepare_tmix_wkv7_recurrent_metadata(cu, slots, total_tokens=9, state_pool_size=pool.shape[0],
                                                 max_seqlen=4)
    # a valid ticket reused twice gives bit-identical results
    p1, p2 = pool.clone(), pool.clone()
    y1 = run(*args, state_pool=p1, cu_seqlens=cu, state_indices=slots, validated_metadata=ticket2)
    y2 = run(*args, state_pool=p2, cu_seqlens=cu, state_indices=slots, validated_metadata=ticket2)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(p1, p2)


@pytest.mark.parametrize("entry", ("recurrent", "prefill_recurrent", "prefill_auto"))
def test_low_level_invalid_metadata_fails_closed_without_state_write(entry):
    import flashrwkv2_b200

    case = _case(lengths=(40,), dtype=torch.float16)
    pool = case["state_pool"]
    bad_cu = torch.tensor([1, 40], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0], dtype=torch.int32, device=DEV)
    out = torch.zeros_like(case["v"])
    before = pool.clone()
    ext = flashrwkv2_b200._C
    if entry == "recurrent":
        ext.tmix_wkv7_recurrent_fp32_from_decay_logits(bad_cu, slots, pool, *_args(case), out, 1.0, None, None)
    else:
        ext.tmix_wkv7_prefill_fp32(bad_cu, slots, pool, *_args(case), out, 1.0, None, None, -1, "logits",
                                   "recurrent" if entry == "prefill_recurrent" else "auto")
    torch.cuda.synchronize()
    assert torch.isnan(out).all()
    assert torch.equal(pool, before)


def test_zero_active_warmup_then_graph_replay():
    ops = _ops()
    g = torch.Generator().manual_seed(20260809)
    tok_cap, seq_cap, n_slots, heads = 4, 4, 2, 1
    packed = tuple((torch.randn(tok_cap, heads, 64, generator=g) * s).half().to(DEV)
                   for s in (0.1, 2.0, 0.05, 0.05, 0.05, 0.05))
    initial = (torch.randn(n_slots, heads, 64, 64, generator=g) * 0.02).to(DEV)
    state = initial.clone()
    cu = torch.tensor([0, -1, -1, -1, -1], dtype=torch.int32, device=DEV)
    slots = torch.full((seq_cap,), 99, dtype=torch.int32, device=DEV)
    n_tok = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.Stream()

    def ticket():
        return ops.prepare_tmix_wkv7_recurrent_metadata(
            cu, slots, state_pool_size=n_slots, token_capacity=tok_cap, sequence_capacity=seq_cap,
            max_seqlen_capacity=3, num_active_tokens=n_tok, num_active_sequences=n_seq)

    def run(pool, tk):
        return ops.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen(
            *packed, state_pool=pool, cu_seqlens=cu, state_indices=slots, validated_metadata=tk)

    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        warm = ticket()
        run(state, warm)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    assert warm._is_graph() and torch.equal(state, initial)

    cu.copy_(torch.tensor([0, 1, 4, -1, -1], dtype=torch.int32))
    slots.copy_(torch.tensor([1, 0, 99, 99], dtype=torch.int32))
    n_tok.fill_(4)
    n_seq.fill_(2)
    expected_state = initial.clone()
    expected = run(expected_state, ticket())
    torch.cuda.synchronize()
    assert not torch.equal(expected_state, initial)

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        captured = run(state, ticket())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, expected) and torch.equal(state, expected_state)
    # ... and the replay is right, not merely equal to the eager launch: the CPU oracle on the same metadata
    from oracle.wkv7_oracle import max_err_over_rms, wkv7_oracle

    y_ref, pool_ref = wkv7_oracle(*(x.cpu() for x in packed), state_pool=initial.cpu(), cu_seqlens=[0, 1, 4],
                                  state_indices=[1, 0])
    assert max_err_over_rms(captured.float().cpu(), y_ref) <= 5e-3  # fp16 rounding of y
    assert max_err_over_rms(state.cpu(), pool_ref) <= 1e-5

    # live metadata rewrite: one active sequence on slot 0
    state.copy_(initial)
    cu.copy_(torch.tensor([0, 2, -1, -1, -1], dtype=torch.int32))
    slots.copy_(torch.tensor([0, 99, 99, 99], dtype=torch.int32))
    n_tok.fill_(2)
    n_seq.fill_(1)
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.equal(state[0], initial[0]) and torch.equal(state[1], initial[1])

    # duplicate slots under replay: fail closed, state untouched
    state.copy_(initial)
    cu.copy_(torch.tensor([0, 1, 2, -1, -1], dtype=torch.int32))
    slots.copy_(torch.tensor([1, 1, 99, 99], dtype=torch.int32))
    n_tok.fill_(2)
    n_seq.fill_(2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(state, initial)


def test_native_layer_rejects_bad_tensors():
    """Native-layer contract (RuntimeError with the reference's message fragments)."""
    import flashrwkv2_b200

    ext = flashrwkv2_b200._C
    case = _case(lengths=(4, 5))
    cu, slots, pool = case["cu_seqlens"], case["state_indices"], case["state_pool"]
    out = torch.empty_like(case["v"])
    a = list(_args(case))

    def call(**over):
        kw = dict(cu=cu, slots=slots, pool=pool, toks=a, out=out, scale=1.0, bias=None)
        kw.update(over)
        ext.tmix_wkv7_recurrent_fp32_from_decay_logits(kw["cu"], kw["slots"], kw["pool"], *kw["toks"], kw["out"],
                                                       kw["scale"], kw["bias"], None)

    with pytest.raises(RuntimeError, match="contiguous"):
        call(toks=[a[0].transpose(0, 1)] + a[1:])
    with pytest.raises(RuntimeError, match="shape"):
        call(toks=[a[0][:-1].contiguous()] + a[1:])
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        call(toks=[t.to(torch.float64) for t in a], out=out.double())
    with pytest.raises(RuntimeError, match="dtype mismatch"):
        call(toks=[a[0].half()] + a[1:])
    with pytest.raises(RuntimeError, match="square"):
        call(pool=pool[:, :, :, :32].contiguous())
    with pytest.raises(RuntimeError, match="64, 128, or 256"):
        call(pool=torch.zeros(9, 2, 32, 32, device=DEV))
    with pytest.raises(RuntimeError, match="head size 64 only"):
        call(pool=torch.zeros(9, 2, 128, 128, device=DEV))
    with pytest.raises(RuntimeError, match="finite"):
        call(scale=float("inf"))
    with pytest.raises(RuntimeError, match="decay_bias"):
        call(bias=torch.zeros(3, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError, match="CUDA"):
        call(toks=[a[0].cpu()] + a[1:])
    torch.cuda.synchronize()
