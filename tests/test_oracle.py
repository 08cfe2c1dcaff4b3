"""Pins the CPU oracle (Python and C) to the committed outputs of the reference's
own fp32 recurrence, and pins the chunked WY/UT algebra to the token loop."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from conftest import GOLDEN_CASES, TOKEN_NAMES, load_golden

from oracle import c_oracle
from oracle.wkv7_oracle import (chunked_wy_f64, logits_from_retention, max_err_over_rms,
                                relative_rmse, retention_from_logits, wkv7_oracle, wkv7_oracle_f64)


def _run(fn, case, **kw):
    return fn(*(case[n] for n in TOKEN_NAMES), state_pool=case["state_pool"],
              cu_seqlens=case["cu_seqlens"], state_indices=case["state_indices"],
              scale=case["scale"], decay_bias=case["decay_bias"], **kw)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_python_oracle_matches_reference_outputs(name):
    case = load_golden(name)
    y, pool = _run(wkv7_oracle, case)
    # same fp32 arithmetic, possibly a different summation order inside the matmul
    assert max_err_over_rms(y, case["y"].float()) < (2e-3 if name == "rl_infctx_fp16" else 2e-5)
    assert max_err_over_rms(pool, case["final_pool"]) < 2e-5
    touched = set(case["state_indices"].tolist())
    for slot in range(case["state_pool"].shape[0]):
        if slot not in touched:
            assert torch.equal(pool[slot], case["state_pool"][slot])


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_c_oracle_matches_reference_outputs(name):
    case = load_golden(name)
    for f64 in (False, True):
        y, pool = _run(c_oracle.wkv7_oracle_c, case, f64=f64)
        assert max_err_over_rms(y, case["y"].float()) < (2e-3 if name == "rl_infctx_fp16" else 2e-5)
        assert max_err_over_rms(pool, case["final_pool"]) < 2e-5


def test_rl_infctx_output_rounding():
    # that reference variant rounds y to the token dtype (rl_infctx/test.py:52-55)
    case = load_golden("rl_infctx_fp16")
    y, _ = _run(wkv7_oracle, case)
    assert relative_rmse(y.half(), case["y"]) < 1e-3


def test_retention_mode_equals_logits_mode():
    torch.manual_seed(3)
    T, H = 40, 2
    logits = torch.randn(T, H, 64) * 2
    toks = [torch.randn(T, H, 64) * 0.3 for _ in range(5)]
    r, k, v, a, b = toks
    pool = torch.randn(2, H, 64, 64) * 0.1
    kw = dict(state_pool=pool, cu_seqlens=[0, 25, 40], state_indices=[1, 0])
    y0, p0 = wkv7_oracle_f64(r, logits, k, v, a, b, decay_mode="logits", **kw)
    w = retention_from_logits(logits.double())
    y1, p1 = wkv7_oracle_f64(r, w, k, v, a, b, decay_mode="retention", **kw)
    assert max_err_over_rms(y1, y0) < 1e-12 and max_err_over_rms(p1, p0) < 1e-12
    back = logits_from_retention(w)
    assert (back - logits.double()).abs().max() < 1e-9


def test_c_oracle_threads_and_modes_agree():
    torch.manual_seed(5)
    T, H = 70, 3
    x = torch.rand(T, H, 64) * 4.5 - 5
    w = torch.exp(-torch.exp(x))
    r, k, v = (torch.randn(T, H, 64) for _ in range(3))
    kk = torch.nn.functional.normalize(torch.randn(T, H, 64), dim=-1)
    a, b = -kk, kk * torch.sigmoid(torch.randn(T, H, 64))
    pool = torch.randn(3, H, 64, 64) * 0.1
    kw = dict(state_pool=pool, cu_seqlens=[0, 1, 6, 70], state_indices=[2, 0, 1], decay_mode="retention")
    y_py, p_py = wkv7_oracle(r, w, k, v, a, b, **kw)
    y1, p1 = c_oracle.wkv7_oracle_c(r, w, k, v, a, b, n_threads=1, **kw)
    y4, p4 = c_oracle.wkv7_oracle_c(r, w, k, v, a, b, n_threads=4, **kw)
    assert torch.equal(y1, y4) and torch.equal(p1, p4)
    assert max_err_over_rms(y1, y_py) < 2e-5 and max_err_over_rms(p1, p_py) < 2e-5


@pytest.mark.parametrize("T", (1, 17, 64, 65, 200))
def test_chunked_wy_form_equals_token_loop(T):
    rng = np.random.default_rng(T)
    w = np.exp(-np.exp(rng.uniform(-5, -0.5, (T, 64))))
    r, k, v = (rng.standard_normal((T, 64)) for _ in range(3))
    kk = rng.standard_normal((T, 64))
    kk /= np.linalg.norm(kk, axis=-1, keepdims=True)
    a, b = -kk, kk / (1 + np.exp(-rng.standard_normal((T, 64))))
    S0 = rng.standard_normal((64, 64)) * 0.1
    y, S = chunked_wy_f64(r, w, k, v, a, b, S0, scale=0.7)
    tt = lambda x: torch.from_numpy(x).unsqueeze(1)
    y_ref, p_ref = wkv7_oracle_f64(tt(r), tt(w), tt(k), tt(v), tt(a), tt(b),
                                   state_pool=torch.from_numpy(S0)[None, None], cu_seqlens=[0, T],
                                   state_indices=[0], scale=0.7, decay_mode="retention")
    assert max_err_over_rms(torch.from_numpy(y), y_ref[:, 0]) < 1e-9
    assert max_err_over_rms(torch.from_numpy(S), p_ref[0, 0]) < 1e-9


def test_fp16_state_oracle_reproduces_the_reference_function_exactly():
    """The fp16-state decode contract: the restatement against the committed output of the reference's own
    rwkv7_fp16_reference (tests/golden/make_golden.py): fp16 rounding after every token makes this bit-exact."""
    from oracle.wkv7_oracle import wkv7_fp16_state_oracle

    case = load_golden("recurrent_fp16_state")
    y, pool, elapsed = wkv7_fp16_state_oracle(
        *(case[n] for n in TOKEN_NAMES), state_pool=case["state_pool"], elapsed_state_pool=case["elapsed_state_pool"],
        cu_seqlens=case["cu_seqlens"], state_indices=case["state_indices"], scale=case["scale"],
        decay_bias=case["decay_bias"])
    assert y.dtype == torch.float16 and pool.dtype == torch.float16
    assert torch.equal(y, case["y"]) and torch.equal(pool, case["final_pool"])
    lengths = (case["cu_seqlens"][1:] - case["cu_seqlens"][:-1]).tolist()
    expected = case["elapsed_state_pool"].clone()
    for slot, n in zip(case["state_indices"].tolist(), lengths):
        expected[slot] += n
    assert torch.equal(elapsed, expected)


def test_readout_oracle_is_group_norm_plus_residual_times_gate():
    """The readout restatement against an independent formulation: torch's group norm with one group per head
    (eps 64e-5, as rwkv-rs/FlashRWKV2 csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:25 sets it)."""
    from oracle.wkv7_oracle import readout_prelinear_oracle

    g = torch.Generator().manual_seed(12)
    tokens, heads = 9, 5
    y, r, k, v, gate = (torch.randn(tokens, heads, 64, generator=g) for _ in range(5))
    r_k, ln_w, ln_b = (torch.randn(heads * 64, generator=g) for _ in range(3))
    got = readout_prelinear_oracle(y, r, k, v, r_k, ln_w, ln_b, gate)
    normed = torch.nn.functional.group_norm(y.reshape(tokens, heads * 64), heads, ln_w, ln_b, eps=64.0e-5)
    residual = (r * k * r_k.reshape(1, heads, 64)).sum(-1, keepdim=True) * v
    want = (normed.reshape(tokens, heads, 64) + residual) * gate
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
