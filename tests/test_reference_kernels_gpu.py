"""Drop-in check on a GPU: the product module and a build of the reference project's own CUDA kernels are called
through the SAME pybind symbols with the SAME device tensors, and must agree.

`oracle/_ref/_C_ref.so` is the reference's unmodified recurrent and rl_infctx chunk-forward sources compiled for
sm_100 (oracle/build_ref.py; rwkv-rs/FlashRWKV2 csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.{cpp,cu},
rl_infctx_chunk_fp32io16_forward.{cpp,cu}).  It exists only where a reference checkout was present at build time, so
every test here skips without it.  Gates: 1e-5 max|d|/RMS between the two fp32 recurrences (same arithmetic, other
summation order), the 16-bit y within one unit in the last place; 5e-3 max|d|/RMS for the tensor-core chunk kernel.
"""

from __future__ import annotations

import pytest
import torch
from conftest import TOKEN_NAMES
from test_wkv7_recurrent_gpu import _random_case, _to_dev

from oracle.build_ref import load_ref
from oracle.wkv7_oracle import max_err_over_rms

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    try:
        module = load_ref()
    except (ImportError, OSError) as error:  # built against another torch / CUDA runtime than the one present
        pytest.skip(f"oracle/_ref/_C_ref.so does not load here: {error}")
    if module is None:
        pytest.skip("oracle/_ref/_C_ref.so was not built (no reference checkout at build time)")
    return module


@pytest.fixture(scope="module")
def ours():
    import flashrwkv2_b200

    assert flashrwkv2_b200._C is not None and flashrwkv2_b200._C.__file__.endswith(".so")
    return flashrwkv2_b200._C


def _recurrent(module, d, *, ticket: bool, max_seqlen: int):
    pool = d["state_pool"].clone()
    y = torch.empty_like(d["v"])
    validated = None
    if ticket:
        validated = module.prepare_tmix_wkv7_recurrent_metadata(d["cu_seqlens"], d["state_indices"],
                                                                d["r"].shape[0], pool.shape[0], max_seqlen)
    module.tmix_wkv7_recurrent_fp32_from_decay_logits(d["cu_seqlens"], d["state_indices"], pool,
                                                      *(d[n] for n in TOKEN_NAMES), y, float(d["scale"]),
                                                      d["decay_bias"], validated, max_seqlen)
    torch.cuda.synchronize()
    return y.float().cpu(), pool.cpu()


def _one_ulp(y_a, y_b, dtype):
    """16-bit outputs of two fp32 computations may round to neighbouring values."""
    eps = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    tol = eps * torch.maximum(y_a.abs(), y_b.abs()) + 1e-6
    return bool(((y_a - y_b).abs() <= tol).all())


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("bias", (False, True))
def test_decode_step_matches_the_reference_kernel(ref, ours, dtype, bias):
    case = _random_case((1,) * 48, 4, dtype, seed=71, retention=False, bias=bias,
                        slots=list(reversed(range(48))), pool_slots=50)
    case["scale"] = 0.75
    d = _to_dev(case)
    d["scale"] = case["scale"]
    y_ref, pool_ref = _recurrent(ref, d, ticket=True, max_seqlen=1)
    y, pool = _recurrent(ours, d, ticket=True, max_seqlen=1)
    assert max_err_over_rms(pool, pool_ref) <= 1e-5
    assert _one_ulp(y, y_ref, dtype)
    assert torch.equal(pool[48:], pool_ref[48:])  # slots outside state_indices: untouched by both


@pytest.mark.parametrize("ticket", (False, True))
def test_ragged_recurrence_matches_the_reference_kernel(ref, ours, ticket):
    lengths = (5, 1, 33, 64, 2, 17)
    case = _random_case(lengths, 3, torch.bfloat16, seed=72, retention=False, bias=True)
    d = _to_dev(case)
    d["scale"] = 1.0
    y_ref, pool_ref = _recurrent(ref, d, ticket=ticket, max_seqlen=max(lengths))
    y, pool = _recurrent(ours, d, ticket=ticket, max_seqlen=max(lengths))
    assert max_err_over_rms(pool, pool_ref) <= 1e-5
    assert _one_ulp(y, y_ref, torch.bfloat16)


def test_invalid_metadata_is_rejected_like_the_reference(ref, ours):
    """Duplicate slots: preparing a ticket raises ("unique"); the un-ticketed native call validates on the
    device and fails closed, i.e. y is all NaN and the pool is untouched, in both modules."""
    case = _random_case((2, 2), 2, torch.bfloat16, seed=73, retention=False)
    d = _to_dev(case)
    d["scale"] = 1.0
    d["state_indices"] = torch.tensor([1, 1], dtype=torch.int32, device=DEV)
    for module in (ref, ours):
        with pytest.raises(RuntimeError, match="unique"):
            module.prepare_tmix_wkv7_recurrent_metadata(d["cu_seqlens"], d["state_indices"], 4, 2, 2)
        y, pool = _recurrent(module, d, ticket=False, max_seqlen=2)
        assert bool(torch.isnan(y).all())
        assert torch.equal(pool, case["state_pool"])


def _chunk_metadata(lengths, chunk):
    offsets, starts, ends, begin = [0], [], [], 0
    for length in lengths:
        for s in range(begin, begin + length, chunk):
            starts.append(s)
            ends.append(min(s + chunk, begin + length))
        offsets.append(len(starts))
        begin += length
    return tuple(torch.tensor(x, dtype=torch.int32, device=DEV) for x in (offsets, starts, ends))


@pytest.mark.parametrize("strategy", (0, 1))
@pytest.mark.parametrize("chunk", (16, 64))
def test_chunk_forward_matches_the_reference_kernels(ref, ours, strategy, chunk):
    lengths = (130, 64, 37, 256)
    case = _random_case(lengths, 2, torch.bfloat16, seed=74 + chunk, retention=False, bias=True)
    d = _to_dev(case)
    meta = _chunk_metadata(lengths, chunk)
    results = []
    for module in (ref, ours):
        state = d["state_pool"].clone()
        y, final = module.rl_infctx_tmix_wkv7_chunk_fp32io16_forward(*meta, state, *(d[n] for n in TOKEN_NAMES),
                                                                     strategy, 1.0, d["decay_bias"])
        torch.cuda.synchronize()
        assert torch.equal(state, d["state_pool"]), "the caller's state must not be modified"
        results.append((y.float().cpu(), final.cpu()))
    (y_ref, s_ref), (y, s) = results
    assert max_err_over_rms(s, s_ref) <= 5e-3
    rms = float((y_ref ** 2).mean().sqrt())
    # both y are bf16: the 5e-3 gate plus one rounding step of the larger value
    assert bool(((y - y_ref).abs() <= 5e-3 * rms + 2.0 ** -7 * torch.maximum(y.abs(), y_ref.abs())).all())
    assert float(((y - y_ref) ** 2).mean().sqrt() / (y_ref ** 2).mean().sqrt()) <= 7e-3


def _device_rms(x):
    return float(x.float().pow(2).mean().sqrt())


@pytest.mark.parametrize("name", ("c1", "c2", "c3", "c4_decode", "c4_prefill"))
def test_full_size_configurations_match_the_reference_kernels(ref, ours, name):
    """Every benchmark configuration at its full size (the CPU oracle cannot reach these): the product's operator
    (decode kernel for T=1, tensor-core chunk kernel otherwise) against the reference's recurrent kernel, logits
    decay mode, inputs generated on the device with the benchmark's distributions."""
    from flashrwkv2_b200.workloads import make_workload

    shape = make_workload(name, with_tensors=False)
    token_bytes = shape.total_tokens * shape.heads * 64 * 2
    state_bytes = shape.n_seq * shape.heads * 64 * 64 * 4
    need = 9 * token_bytes + 3 * state_bytes + (2 << 30)  # six inputs, logits, two outputs; three pools; slack
    free, _ = torch.cuda.mem_get_info()
    if free < need:
        pytest.skip(f"needs {need >> 30} GiB of device memory, {free >> 30} GiB free")
    wl = make_workload(name, device=DEV)
    t = wl.tensors
    g = torch.Generator(device=DEV).manual_seed(wl.seed + 100)
    logits = torch.empty_like(t["w"])
    for lo in range(0, wl.total_tokens, 65536):  # bounded temporaries
        hi = min(wl.total_tokens, lo + 65536)
        logits[lo:hi] = (torch.randn((hi - lo, wl.heads, 64), generator=g, device=DEV) * 3.5).to(logits.dtype)
    tokens = (t["r"], logits, t["k"], t["v"], t["a"], t["b"])
    max_len = max(wl.lengths)
    outs = []
    for module in (ref, ours):
        pool = t["state_pool"].clone()
        y = torch.empty_like(t["v"])
        ticket = module.prepare_tmix_wkv7_recurrent_metadata(t["cu_seqlens"], t["state_indices"], wl.total_tokens,
                                                             pool.shape[0], max_len)
        if module is ours and max_len > 1:
            module.tmix_wkv7_prefill_fp32(t["cu_seqlens"], t["state_indices"], pool, *tokens, y, 1.0, None, ticket,
                                          max_len, "logits", "auto")
        else:
            module.tmix_wkv7_recurrent_fp32_from_decay_logits(t["cu_seqlens"], t["state_indices"], pool, *tokens, y,
                                                              1.0, None, ticket, max_len)
        torch.cuda.synchronize()
        outs.append((y, pool))
    (y_ref, s_ref), (y, s) = outs
    gate = 1e-5 if max_len == 1 else 5e-3
    assert float((s - s_ref).abs().max()) <= gate * _device_rms(s_ref)
    rms = _device_rms(y_ref[: 1 << 16])
    for lo in range(0, wl.total_tokens, 1 << 16):
        a, b = y[lo:lo + (1 << 16)].float(), y_ref[lo:lo + (1 << 16)].float()
        tol = gate * rms + 2.0 ** -7 * torch.maximum(a.abs(), b.abs())  # one bf16 rounding step on top of the gate
        assert bool(((a - b).abs() <= tol).all()), (name, lo)


def test_fp16_state_family_against_the_reference_kernels(ref):
    """The fp16-state decode contract: the reference's own kernels (csrc/sm120/tmix/wkv7/
    infer_recurrent_fp16_forward_varlen.{cpp,cu}, half2 arithmetic) and this library's through the same pybind symbol on
    the same tensors.  Gate: the reference's relative RMSE for the family (3e-3, tests/fixtures/tolerances-v1.json:27-29);
    elapsed counters equal; untouched slots bit-identical."""
    import flashrwkv2_b200
    from test_wkv7_fp16_state_gpu import _case

    from oracle.wkv7_oracle import relative_rmse

    if not hasattr(ref, "tmix_wkv7_recurrent_fp16_from_decay_logits"):
        pytest.skip("oracle/_ref/_C_ref.so was built without the fp16-state family")
    for lengths, heads in (((1,) * 64, 64), ((1, 2, 4, 9, 33), 2), ((8, 8), 3)):
        case = _case(lengths, heads=heads, seed=31 + len(lengths))
        d = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
        outs = []
        for module in (ref, flashrwkv2_b200._C):
            pool, elapsed = d["state_pool"].clone(), d["elapsed_state_pool"].clone()
            y = torch.empty_like(d["v"])
            module.tmix_wkv7_recurrent_fp16_from_decay_logits(
                d["cu_seqlens"], d["state_indices"], elapsed, pool, *(d[n] for n in TOKEN_NAMES), y, float(case["scale"]),
                d["decay_bias"], None, -1)
            torch.cuda.synchronize()
            outs.append((y.cpu(), pool.cpu(), elapsed.cpu()))
        (y_r, pool_r, el_r), (y_o, pool_o, el_o) = outs
        touched = case["state_indices"].tolist()
        assert relative_rmse(y_o, y_r) <= 3e-3 and relative_rmse(pool_o[touched], pool_r[touched]) <= 3e-3
        assert torch.equal(el_o, el_r)
        for slot in range(pool_o.shape[0]):
            if slot not in touched:
                assert torch.equal(pool_o[slot], case["state_pool"][slot])
