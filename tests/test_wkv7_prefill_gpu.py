"""GPU parity of the tensor-core chunked prefill against the CPU oracle.

Gate (bf16 / fp16 tokens): max|d|/RMS <= 5e-3 on the fp32 y (`output_f32`, the output
before rounding) and on the final state; the rounded y is exactly the rounding of that fp32
y and within the reference's relative-RMSE gate for its chunk operator (7e-3 on y, 8e-3 on
the state: rwkv-rs/FlashRWKV2 tests/fixtures/tolerances-v1.json:13-17).  The kernel's operand
precision (bf16 hi/lo for the one product with unbounded operands, fp16 with one or two terms for the
rest) is chosen to stay a factor of two inside the gate: it measures 1.2e-3 .. 2.2e-3, and TIGHT
(3e-3) is what the small cases here are held to.
"""

from __future__ import annotations

import pytest
import torch
from conftest import TOKEN_NAMES, load_golden
from test_wkv7_recurrent_gpu import _oracle, _random_case, _run_op, _to_dev

from oracle.wkv7_oracle import max_err_over_rms, relative_rmse

pytestmark = pytest.mark.gpu

GATE = 5e-3
TIGHT = 3e-3
DEV = "cuda"


def _check(case, y, y32, pool, err=None, gate=TIGHT):
    y_ref, pool_ref = _oracle(case, f64=True)
    touched = case["state_indices"].tolist()
    ey = max_err_over_rms(y32, y_ref)
    es = max_err_over_rms(pool[touched], pool_ref[touched])
    assert ey <= gate and es <= gate, (ey, es)
    assert torch.equal(y, y32.to(y.dtype))
    assert relative_rmse(y, y_ref) <= 7e-3 and relative_rmse(pool[touched], pool_ref[touched]) <= 8e-3
    for slot in range(pool.shape[0]):
        if slot not in touched:
            assert torch.equal(pool[slot], case["state_pool"][slot])
    if err is not None:
        assert int(err.item()) == 0, "a bounded wait in the kernel gave up"


def _run_tc(case):
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, y32, pool = _run_op(case, op="prefill", strategy="chunk_tc", error_flag=err)
    return y, y32, pool, err


@pytest.mark.parametrize("lengths", [(64,), (1,), (63,), (65,), (128,), (1, 15, 16, 17, 65), (200, 3, 129)])
def test_chunk_lengths_and_ragged_tails(lengths):
    slots = list(reversed(range(len(lengths))))
    case = _random_case(lengths, 2, torch.bfloat16, seed=sum(lengths), slots=slots, pool_slots=len(lengths) + 2)
    _check(case, *_run_tc(case))


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_logits_mode_with_bias_and_scale(dtype):
    case = _random_case((70, 130, 5), 3, dtype, seed=21, retention=False, bias=True)
    case["scale"] = 0.5
    _check(case, *_run_tc(case))


def test_fp16_retention():
    case = _random_case((100, 64), 2, torch.float16, seed=22)
    _check(case, *_run_tc(case))


@pytest.mark.parametrize("name", ("recurrent_bf16", "recurrent_bf16_bias", "recurrent_fp16_bias",
                                  "recurrent_bf16_long", "recurrent_bf16_unit"))
def test_golden_reference_cases_through_chunk_kernel(name):
    case = load_golden(name)
    y, y32, pool, err = _run_tc(case)
    touched = case["state_indices"].tolist()
    assert max_err_over_rms(y32, case["y"]) <= TIGHT
    assert max_err_over_rms(pool[touched], case["final_pool"][touched]) <= TIGHT
    assert int(err.item()) == 0


def test_zero_state_and_many_heads():
    case = _random_case((192,), 40, torch.bfloat16, seed=23)
    case["state_pool"].zero_()
    _check(case, *_run_tc(case))


def test_long_rows_dense_prefill_shape():
    """Dense prefill shape reduced to 2 x 4096 tokens x 8 heads, against the C oracle."""
    from flashrwkv2_b200.workloads import make_workload

    wl = make_workload("c2", n_seq=2, heads=8)
    t = wl.tensors
    case = {"r": t["r"], "decay_logits": t["w"], "k": t["k"], "v": t["v"], "a": t["a"], "b": t["b"],
            "cu_seqlens": t["cu_seqlens"], "state_indices": t["state_indices"], "state_pool": t["state_pool"],
            "decay_bias": None, "scale": 1.0, "decay_mode": "retention"}
    y, y32, pool, err = _run_tc(case)
    _check(case, y, y32, pool, err, gate=GATE)
    ey = max_err_over_rms(y32, _oracle(case, f64=True)[0])
    assert ey <= TIGHT, ey


def test_varlen_shape_reduced():
    """Ragged packed prefill: 16 sequences of U[1,600] tokens, 40 heads."""
    from flashrwkv2_b200.workloads import make_workload

    wl = make_workload("c3", n_seq=16, seq_len=600)
    t = wl.tensors
    case = {"r": t["r"], "decay_logits": t["w"], "k": t["k"], "v": t["v"], "a": t["a"], "b": t["b"],
            "cu_seqlens": t["cu_seqlens"], "state_indices": t["state_indices"], "state_pool": t["state_pool"],
            "decay_bias": None, "scale": 1.0, "decay_mode": "retention"}
    _check(case, *_run_tc(case))


def test_split_call_equals_single_call_and_recurrent_path():
    """Size-independent properties: running the first 256 tokens and then the rest with the carried
    state equals one call; and the tensor-core path agrees with the CUDA-core recurrence."""
    import flashrwkv2_b200.tmix.wkv7 as ops

    case = _random_case((700,), 4, torch.bfloat16, seed=31)
    y_one, y32_one, pool_one, _ = _run_tc(case)
    d = _to_dev(case)
    pool = d["state_pool"].clone()
    outs = []
    for lo, hi in ((0, 256), (256, 700)):
        toks = [d[n][lo:hi].contiguous() for n in TOKEN_NAMES]
        cu = torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV)
        y32 = torch.empty(toks[0].shape, dtype=torch.float32, device=DEV)
        ops.infer_tmix_wkv7_prefill_fp32io16_forward_varlen(
            *toks, state_pool=pool, cu_seqlens=cu, state_indices=d["state_indices"], decay_mode="retention",
            strategy="chunk_tc", output_f32=y32)
        outs.append(y32)
    torch.cuda.synchronize()
    assert max_err_over_rms(torch.cat(outs).cpu(), y32_one) <= 1e-5  # chunk boundaries fall on the same rows
    assert max_err_over_rms(pool.cpu(), pool_one) <= 1e-5
    y_rec, y32_rec, pool_rec = _run_op(case, op="prefill", strategy="recurrent")
    assert max_err_over_rms(y32_one, y32_rec) <= TIGHT and max_err_over_rms(pool_one, pool_rec) <= TIGHT


def test_run_to_run_bit_identical():
    case = _random_case((130, 64, 9), 3, torch.bfloat16, seed=33)
    first = _run_tc(case)
    second = _run_tc(case)
    for x, y in zip(first[:3], second[:3]):
        assert torch.equal(x, y)


def test_rl_infctx_wrapper_matches_reference_case():
    """The reference's own rl_infctx cases: golden fp16 (2,5) with slots [3,1]; bf16 T=65 over every
    chunk_size / strategy choice (tests/tmix/wkv7/rl_infctx/test.py:60-116,187-241)."""
    from flashrwkv2_b200.tmix.wkv7.rl_infctx import rl_infctx_tmix_wkv7_chunk_fp32io16 as chunk

    case = load_golden("rl_infctx_fp16")
    d = _to_dev(case)
    before = d["state_pool"].clone()
    y, final = chunk(*(d[n] for n in TOKEN_NAMES), state_pool=d["state_pool"], cu_seqlens=d["cu_seqlens"],
                     state_indices=d["state_indices"], chunk_size=16, strategy="materialized",
                     decay_bias=d["decay_bias"])
    torch.cuda.synchronize()
    assert y.dtype == torch.float16 and torch.equal(d["state_pool"], before)
    assert torch.allclose(y.float().cpu(), case["y"].float(), rtol=0, atol=2e-3)
    assert torch.allclose(final.cpu(), case["final_pool"], rtol=0, atol=2e-3)
    assert torch.equal(final[[0, 2]], before[[0, 2]])

    big = _random_case((65,), 2, torch.bfloat16, seed=43, retention=False)
    y_ref, pool_ref = _oracle(big, f64=True)
    db = _to_dev(big)
    results = []
    for chunk_size in (16, 32, 64):
        for strategy in ("materialized", "recompute"):
            y, final = chunk(*(db[n] for n in TOKEN_NAMES), state_pool=db["state_pool"],
                             cu_seqlens=db["cu_seqlens"], state_indices=db["state_indices"],
                             chunk_size=chunk_size, strategy=strategy)
            torch.cuda.synchronize()
            assert relative_rmse(y.cpu(), y_ref) <= 7e-3 and relative_rmse(final.cpu(), pool_ref) <= 8e-3
            results.append((y, final))
    assert all(torch.equal(results[0][0], r[0]) and torch.equal(results[0][1], r[1]) for r in results)
    # metadata errors raise ValueError, like the reference wrapper
    with pytest.raises(ValueError, match="duplicates"):
        two = _to_dev(_random_case((4, 5), 1, torch.bfloat16, seed=44))
        chunk(*(two[n] for n in TOKEN_NAMES), state_pool=two["state_pool"], cu_seqlens=two["cu_seqlens"],
              state_indices=torch.tensor([1, 1], dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError, match="non-empty|start at zero"):
        chunk(*(two[n] for n in TOKEN_NAMES), state_pool=two["state_pool"],
              cu_seqlens=torch.tensor([0, 4, 4], dtype=torch.int32, device=DEV))


def test_native_rl_infctx_symbol_with_host_chunk_metadata():
    """The reference-shaped native entry (per-chunk host metadata) gives the same answer."""
    import flashrwkv2_b200

    case = _random_case((40, 100), 2, torch.bfloat16, seed=45, retention=False)
    d = _to_dev(case)
    seq_off = torch.tensor([0, 3, 10], dtype=torch.int32, device=DEV)  # 16-row chunks: 3 + 7
    starts = torch.tensor([0, 16, 32] + [40 + 16 * i for i in range(7)], dtype=torch.int32, device=DEV)
    ends = torch.tensor([16, 32, 40] + [min(140, 56 + 16 * i) for i in range(7)], dtype=torch.int32, device=DEV)
    working = d["state_pool"].clone()
    y, final = flashrwkv2_b200._C.rl_infctx_tmix_wkv7_chunk_fp32io16_forward(
        seq_off, starts, ends, working, *(d[n] for n in TOKEN_NAMES), 1, 1.0, None)
    torch.cuda.synchronize()
    y_ref, pool_ref = _oracle(case, f64=True)
    assert torch.equal(working, d["state_pool"])
    assert relative_rmse(y.cpu(), y_ref) <= 7e-3 and relative_rmse(final.cpu(), pool_ref) <= 8e-3


def test_longest_first_order_changes_schedule_not_results():
    """Through the C ABI: with scratch for the longest-first ranking and without it (natural order) the
    outputs are bit-identical, and scratch that is too small is refused without launching."""
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    case = _random_case((5, 200, 33, 64, 1, 97), 2, torch.bfloat16, seed=51, slots=[3, 0, 5, 1, 4, 2])
    d = _to_dev(case)
    n, total, heads = 6, sum((5, 200, 33, 64, 1, 97)), 2
    need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n, total, heads)
    assert need == n * 4 and lib.frwkv_sm100_wkv7_prefill_workspace_bytes(1, 64, 2) == 0
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for ws_bytes in (0, need):
        pool = d["state_pool"].clone()
        y = torch.empty_like(d["v"])
        ws = torch.full((max(ws_bytes, 4),), 255, dtype=torch.uint8, device=DEV)
        rc = lib.frwkv_sm100_wkv7_prefill(
            d["cu_seqlens"].data_ptr(), d["state_indices"].data_ptr(), 0, pool.data_ptr(),
            *(d[n_].data_ptr() for n_ in TOKEN_NAMES), 0, y.data_ptr(), 0, n, total, heads, _lib.IO_BF16,
            _lib.DECAY_RETENTION, 1.0, 200, _lib.PREFILL_CHUNK_TC, ws.data_ptr() if ws_bytes else 0, ws_bytes, 0, stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        if ws_bytes:
            assert ws[:need].view(torch.int32).cpu().tolist() == [1, 5, 3, 2, 0, 4]  # lengths 200,97,64,33,5,1
        results.append((y.clone(), pool))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    y_ref, pool_ref = _oracle(case, f64=True)
    assert relative_rmse(results[1][0].cpu(), y_ref) <= 7e-3
    rc = lib.frwkv_sm100_wkv7_prefill(
        d["cu_seqlens"].data_ptr(), d["state_indices"].data_ptr(), 0, d["state_pool"].data_ptr(),
        *(d[n_].data_ptr() for n_ in TOKEN_NAMES), 0, y.data_ptr(), 0, n, total, heads, _lib.IO_BF16,
        _lib.DECAY_RETENTION, 1.0, 200, _lib.PREFILL_CHUNK_TC, ws.data_ptr(), 8, 0, stream)
    assert rc != 0 and "workspace" in _lib.last_error()


def test_auto_strategy_splits_a_mixed_batch_by_length():
    """Decode-like rows next to prompts (continuous batching): under "auto" rows shorter than 16 tokens go to
    the recurrence kernel and the rest to the tensor-core kernel, in one call; every row must be right."""
    lengths = (1, 1, 40, 1, 200, 3, 15, 16, 1, 33)
    case = _random_case(lengths, 3, torch.bfloat16, seed=61, slots=[9, 0, 8, 1, 7, 2, 6, 3, 5, 4], pool_slots=11)
    y, y32, pool = _run_op(case, op="prefill", strategy="auto")
    _check(case, y, y32, pool)
    # the short rows are computed in fp32 by the recurrence kernel: they meet its 1e-5 gate
    y_ref, _ = _oracle(case, f64=True)
    cu = case["cu_seqlens"].tolist()
    short_rows = torch.cat([torch.arange(cu[i], cu[i + 1]) for i, n in enumerate(lengths) if n < 16])
    assert max_err_over_rms(y32[short_rows], y_ref[short_rows]) <= 1e-5


def _run_tc_c_abi(lib, case):
    """The tensor-core prefill through the C ABI of `lib` (the product library or its test build)."""
    from flashrwkv2_b200 import _lib

    d = _to_dev(case)
    pool = d["state_pool"].clone()
    y = torch.empty_like(d["v"])
    y32 = torch.empty(d["v"].shape, dtype=torch.float32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_seq, (total, heads, _) = d["state_indices"].numel(), d["v"].shape
    io = _lib.IO_BF16 if d["v"].dtype == torch.bfloat16 else _lib.IO_FP16
    mode = _lib.DECAY_RETENTION if case.get("decay_mode") == "retention" else _lib.DECAY_LOGITS
    rc = lib.frwkv_sm100_wkv7_prefill(
        d["cu_seqlens"].data_ptr(), d["state_indices"].data_ptr(), 0, pool.data_ptr(),
        *(d[n].data_ptr() for n in TOKEN_NAMES), 0, y.data_ptr(), y32.data_ptr(), n_seq, total, heads, io, mode,
        float(case["scale"]), 0, _lib.PREFILL_CHUNK_TC, 0, 0, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    return y.cpu(), y32.cpu(), pool.cpu(), err


def test_bounded_wait_reports_instead_of_hanging():
    """A tcgen05.commit that never comes: the waiting warps give up after about a second, the CTA raises the error
    flag and leaves in order (every warp, the MMA-issuing one included), and the device stays usable for the next
    call.  The commit is left out by a hook that exists only in the test build of the library
    (tests/lib/libfrwkv_sm100_testhooks.so, the same sources with -DFRWKV_TEST_HOOKS); no GPU fault is involved,
    the wait simply runs out."""
    from conftest import load_testhooks

    hooks = load_testhooks()
    case = _random_case((96, 40), 2, torch.bfloat16, seed=31)
    hooks.frwkv_sm100_test_skip_commit(1)
    try:
        _, _, _, err = _run_tc_c_abi(hooks, case)
    finally:
        hooks.frwkv_sm100_test_skip_commit(-1)
    assert int(err.item()) & 1 == 1
    _check(case, *_run_tc_c_abi(hooks, case))
    _check(case, *_run_tc(case))


def test_decay_product_out_of_range_raises_the_error_flag():
    """Retention mode accepts any rho, but the chunk kernel divides by the product of rho over a chunk: a caller whose
    retentions are far below what RWKV-7 can produce (rho >= 0.545) gets bit 1 of the error flag, not a silent
    inf/NaN; the same batch through the recurrence kernel is exact."""
    case = _random_case((64,), 2, torch.bfloat16, seed=77)
    case["decay_logits"] = torch.full_like(case["decay_logits"], 0.05)  # 0.05^32 is far below 2^-120
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    _run_op(case, op="prefill", strategy="chunk_tc", error_flag=err)
    assert int(err.item()) & 2 == 2
    y, y32, pool = _run_op(case, op="prefill", strategy="recurrent")
    y_ref, pool_ref = _oracle(case, f64=True)
    assert max_err_over_rms(pool, pool_ref) <= 1e-5


@pytest.mark.parametrize("seed", range(32))
def test_random_shapes_against_the_oracle(seed):
    """Seeded random batches: ragged lengths around the chunk boundaries, odd head counts, both token types, both
    decay modes, bias, scale, permuted slots in a larger pool.  Each case goes through the tensor-core kernel alone
    and through the length-splitting default, and must agree with the CPU oracle."""
    import random

    rng = random.Random(1000 + seed)
    n_seq = rng.randint(1, 6)
    special = (1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 95, 96, 97, 127, 128, 129, 160, 257)
    lengths = tuple(rng.choice(special) if rng.random() < 0.6 else rng.randint(1, 300) for _ in range(n_seq))
    heads = rng.choice((1, 2, 3, 5))
    dtype = rng.choice((torch.bfloat16, torch.float16))
    retention = rng.random() < 0.5
    pool_slots = n_seq + rng.randint(0, 3)
    slots = rng.sample(range(pool_slots), n_seq)
    case = _random_case(lengths, heads, dtype, seed=2000 + seed, slots=slots, pool_slots=pool_slots,
                        retention=retention, bias=(not retention) and rng.random() < 0.5)
    case["scale"] = rng.choice((1.0, 0.37))
    _check(case, *_run_tc(case))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    _check(case, *_run_op(case, op="prefill", strategy="auto", error_flag=err), err)


def _workload_case(wl):
    t = wl.tensors
    return {"r": t["r"], "decay_logits": t["w"], "k": t["k"], "v": t["v"], "a": t["a"], "b": t["b"],
            "cu_seqlens": t["cu_seqlens"], "state_indices": t["state_indices"], "state_pool": t["state_pool"],
            "decay_bias": None, "scale": 1.0, "decay_mode": "retention"}


def test_retention_mode_8192_tokens_against_the_c_oracle():
    """One sequence of 8192 tokens (the row length of the 7B-width prefill workload), two heads, retention mode,
    through the default strategy: 256 chunks of state carry against the float64 token loop."""
    from flashrwkv2_b200.workloads import make_workload

    case = _workload_case(make_workload("c4_prefill", n_seq=1, heads=2))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, y32, pool = _run_op(case, op="prefill", strategy="auto", error_flag=err)
    _check(case, y, y32, pool, err, gate=TIGHT)


def test_ragged_workload_exact_lengths_one_head():
    """The 64 sequence lengths of the ragged prefill workload (1 .. 8192 tokens, about 300 k rows), one head,
    retention mode, default strategy (rows under 16 tokens take the recurrence kernel in the same call)."""
    from flashrwkv2_b200.workloads import make_workload

    wl = make_workload("c3", heads=1)
    assert wl.n_seq == 64 and wl.total_tokens > 200_000
    case = _workload_case(wl)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, y32, pool = _run_op(case, op="prefill", strategy="auto", error_flag=err)
    _check(case, y, y32, pool, err, gate=TIGHT)


def test_prefill_operator_under_cuda_graph_capture():
    """The prefill operator (length ranking, recurrence for short rows, chunk kernel; tensor maps encoded on the
    host) captured in a CUDA graph with a capacity ticket, replayed after the metadata was rewritten in place, and
    compared with the oracle (shaped after rwkv-rs/FlashRWKV2 tests/tmix/wkv7/test.py:239-373)."""
    import flashrwkv2_b200.tmix.wkv7 as ops

    lengths_a, lengths_b = (40, 70, 3), (100, 13)
    cap_tok, cap_seq, heads, n_slots = 128, 4, 2, 5
    case = _random_case((cap_tok,), heads, torch.bfloat16, seed=91, pool_slots=n_slots)
    tokens = tuple(case[n].to(DEV) for n in TOKEN_NAMES)
    initial = case["state_pool"].to(DEV)
    state = initial.clone()
    cu = torch.full((cap_seq + 1,), -1, dtype=torch.int32, device=DEV)
    slots = torch.full((cap_seq,), 99, dtype=torch.int32, device=DEV)
    n_tok = torch.zeros(1, dtype=torch.int32, device=DEV)
    n_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    cu[0] = 0
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.Stream()

    def set_meta(lengths, use_slots):
        ends = torch.tensor(lengths).cumsum(0).tolist()
        cu.copy_(torch.tensor([0] + ends + [-1] * (cap_seq - len(lengths)), dtype=torch.int32))
        slots.copy_(torch.tensor(list(use_slots) + [99] * (cap_seq - len(lengths)), dtype=torch.int32))
        n_tok.fill_(ends[-1])
        n_seq.fill_(len(lengths))

    def run(pool):
        ticket = ops.prepare_tmix_wkv7_recurrent_metadata(
            cu, slots, state_pool_size=n_slots, token_capacity=cap_tok, sequence_capacity=cap_seq,
            max_seqlen_capacity=cap_tok, num_active_tokens=n_tok, num_active_sequences=n_seq)
        return ops.infer_tmix_wkv7_prefill_fp32io16_forward_varlen(
            *tokens, state_pool=pool, cu_seqlens=cu, state_indices=slots, validated_metadata=ticket,
            decay_mode="retention", error_flag=err)

    def expect(lengths, use_slots):
        total = sum(lengths)
        ref_case = dict(case, cu_seqlens=torch.tensor([0] + torch.tensor(lengths).cumsum(0).tolist(), dtype=torch.int32),
                        state_indices=torch.tensor(use_slots, dtype=torch.int32))
        for n in TOKEN_NAMES:
            ref_case[n] = case[n][:total]
        return _oracle(ref_case, f64=True)

    set_meta(lengths_a, (4, 0, 2))
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        run(state.clone())  # warm-up outside capture: kernel attributes, tensor-map cache, allocator pools
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        y = run(state)
    for lengths, use_slots in ((lengths_a, (4, 0, 2)), (lengths_b, (1, 3))):
        state.copy_(initial)
        set_meta(lengths, use_slots)
        graph.replay()
        torch.cuda.synchronize()
        y_ref, pool_ref = expect(lengths, use_slots)
        total = sum(lengths)
        assert max_err_over_rms(y[:total].float().cpu(), y_ref) <= 3e-2  # bf16 rounding of y on top of the gate
        assert relative_rmse(y[:total].cpu(), y_ref) <= 7e-3
        touched = list(use_slots)
        assert max_err_over_rms(state.cpu()[touched], pool_ref[touched]) <= TIGHT
        for slot in range(n_slots):
            if slot not in touched:
                assert torch.equal(state[slot], initial[slot])
        assert int(err.item()) == 0


@pytest.mark.parametrize("lengths", [(2048,) * 10, (2047,) * 10, (4200, 2049, 2048, 2047, 64, 6200, 1, 33, 2112, 100)])
def test_work_queue_hands_the_state_from_segment_to_segment(lengths):
    """More streams than the GPU has CTA slots (10 sequences x 30 heads = 300 > 296): the chunk kernel runs with
    persistent CTAs that take (stream, segment) tasks.  Equal lengths are cut into several segments (300 streams on
    296 slots would otherwise take two rounds) whose state passes through the pool slot; the ragged batch is left to
    the longest-first order with one CTA per stream.  Against the C oracle, and bit-identical to the same call without
    scratch (one CTA per stream, natural order, no queue)."""
    from flashrwkv2_b200 import _lib

    case = _random_case(lengths, 30, torch.bfloat16, seed=404, slots=[3, 9, 0, 7, 1, 8, 2, 6, 4, 5], pool_slots=11)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, y32, pool = _run_op(case, op="prefill", strategy="chunk_tc", error_flag=err)
    _check(case, y, y32, pool, err, gate=TIGHT)
    lib = _lib.load()
    assert lib.frwkv_sm100_wkv7_prefill_workspace_bytes(10, sum(lengths), 30) > 10 * 30 * 4  # queue scratch asked for
    y_direct, y32_direct, pool_direct, err_direct = _run_tc_c_abi(lib, case)  # passes no workspace
    assert int(err_direct.item()) == 0
    assert torch.equal(y, y_direct) and torch.equal(pool, pool_direct)


@pytest.mark.parametrize("n_seq,heads,length", [(5, 64, 1056), (7, 48, 1500), (11, 32, 800), (20, 30, 331), (4, 128, 2048)])
def test_queue_and_whole_stream_launches_agree_bit_for_bit(n_seq, heads, length):
    """Uniform batches a little above one round of CTA slots, where the launcher's estimate sends some to the work
    queue (several segment counts) and keeps others on one CTA per stream: whatever it picks must reproduce the call
    without scratch (natural order, one CTA per stream) bit for bit, with no error bit."""
    from flashrwkv2_b200 import _lib

    case = _random_case((length,) * n_seq, heads, torch.bfloat16, seed=n_seq * heads)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    y, y32, pool = _run_op(case, op="prefill", strategy="chunk_tc", error_flag=err)
    assert int(err.item()) == 0 and not torch.isnan(y32).any()
    y_direct, y32_direct, pool_direct, err_direct = _run_tc_c_abi(_lib.load(), case)
    assert int(err_direct.item()) == 0
    assert torch.equal(y, y_direct) and torch.equal(y32, y32_direct) and torch.equal(pool, pool_direct)
