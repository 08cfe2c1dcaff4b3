"""GPU parity of the WKV7 training operator (forward with checkpoints, backward).

Expectation: oracle.wkv7_oracle.wkv7_pretrain_oracle, the restatement of rwkv-rs/FlashRWKV2
tests/tmix/wkv7/pretrain/test.py:44-65, evaluated in float64 on the CPU; its torch.autograd gradients are the
expectation for the backward pass (the reference's own test does the same in fp32 with atol 0.03 / rtol 0.05,
:103-124).  Outputs and gradients are bfloat16, so a value may differ from the float64 expectation by half a unit in
the last place; beyond that the gates are 1e-4 of the tensor's RMS for y and 2e-3 for the gradients (the backward
pass rebuilds every state from the next one in fp32, up to 16 steps from a checkpoint).  The reference's own
kernels (built into oracle/_ref) pin the restatement.
"""

from __future__ import annotations

import inspect

import pytest
import torch

from oracle.wkv7_oracle import wkv7_pretrain_oracle

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _case(batch, tokens, heads, seed, magnitude=0.05):
    """magnitude 0.05: six independent small tensors, as the reference's test draws them (tests/tmix/wkv7/pretrain/
    test.py:25-41).  Larger magnitudes use the structure the model gives a and b (a = -kk, b = kk * gate with kk a
    unit vector per head), without which the recurrence is not contractive and the gradients overflow."""
    g = torch.Generator().manual_seed(seed)
    shape = (batch, tokens, heads * 64)
    if magnitude <= 0.05:
        return tuple((torch.randn(shape, generator=g) * magnitude).bfloat16() for _ in range(6))
    r, k, v = (torch.randn(shape, generator=g) * magnitude for _ in range(3))
    w = torch.randn(shape, generator=g) * 3.0
    kk = torch.nn.functional.normalize(torch.randn(batch, tokens, heads, 64, generator=g), dim=-1).reshape(shape)
    a, b = -kk, kk * torch.sigmoid(torch.randn(shape, generator=g))
    return tuple(x.bfloat16() for x in (r, w, k, v, a, b))


def _beyond_rounding(got, want):
    """Largest deviation beyond half a bf16 unit in the last place of the expectation, relative to its RMS."""
    want = want.double()
    exponent = torch.floor(torch.log2(want.abs().clamp_min(2.0 ** -126)))
    half_ulp = 0.5 * torch.exp2(exponent - 7)
    excess = (got.double() - want).abs() - 1.01 * half_ulp
    return float(excess.max() / want.square().mean().sqrt())


def _expected(values, grad_output):
    leaves = tuple(x.double().requires_grad_() for x in values)
    y = wkv7_pretrain_oracle(*leaves, dtype=torch.float64)
    y.backward(grad_output.double())
    return y.detach(), [x.grad for x in leaves]


def _run(values, grad_output):
    from flashrwkv2_b200.tmix.wkv7 import pretrain_tmix_wkv7_recurrent_bf16

    leaves = tuple(x.to(DEV).requires_grad_() for x in values)
    y = pretrain_tmix_wkv7_recurrent_bf16(*leaves)
    y.backward(grad_output.to(DEV))
    torch.cuda.synchronize()
    return y.detach().cpu(), [x.grad.cpu() for x in leaves]


def test_public_contract():
    from flashrwkv2_b200.tmix.wkv7 import pretrain_tmix_wkv7_recurrent_bf16

    signature = inspect.signature(pretrain_tmix_wkv7_recurrent_bf16)
    assert tuple(signature.parameters) == ("r", "w", "k", "v", "a", "b", "head_size")
    assert signature.parameters["head_size"].default == 64


@pytest.mark.parametrize("batch,tokens,heads,magnitude", [(1, 16, 1, 0.05), (2, 32, 2, 0.05), (2, 64, 3, 0.5),
                                                          (1, 256, 2, 0.3), (3, 48, 5, 1.0)])
def test_forward_and_backward_match_the_oracle(batch, tokens, heads, magnitude):
    values = _case(batch, tokens, heads, seed=batch + tokens + heads, magnitude=magnitude)
    grad_output = torch.randn(values[0].shape, generator=torch.Generator().manual_seed(7)).bfloat16()
    y, grads = _run(values, grad_output)
    y_ref, grads_ref = _expected(values, grad_output)
    assert y.dtype == torch.bfloat16 and y.shape == values[0].shape
    assert _beyond_rounding(y, y_ref) <= 1e-4
    for name, got, want in zip("rwkvab", grads, grads_ref):
        assert got.dtype == torch.bfloat16 and torch.isfinite(got.float()).all(), name
        assert _beyond_rounding(got, want) <= 2e-3, (name, _beyond_rounding(got, want))


def test_long_sequence_state_reconstruction_does_not_drift():
    """1024 tokens: 64 checkpoints, every state in between rebuilt by up to 15 divisions by rho."""
    values = _case(1, 1024, 1, seed=5, magnitude=0.5)
    grad_output = torch.randn(values[0].shape, generator=torch.Generator().manual_seed(8)).bfloat16()
    y, grads = _run(values, grad_output)
    y_ref, grads_ref = _expected(values, grad_output)
    assert _beyond_rounding(y, y_ref) <= 1e-4
    for name, got, want in zip("rwkvab", grads, grads_ref):
        assert _beyond_rounding(got, want) <= 2e-3, (name, _beyond_rounding(got, want))


def test_run_to_run_bit_identical_and_inputs_untouched():
    values = _case(2, 32, 2, seed=3)
    grad_output = torch.ones(values[0].shape).bfloat16()
    first = _run(values, grad_output)
    second = _run(values, grad_output)
    assert torch.equal(first[0], second[0])
    for x, y in zip(first[1], second[1]):
        assert torch.equal(x, y)


def test_wrapper_rejections_happen_before_any_launch():
    from flashrwkv2_b200.tmix.wkv7 import pretrain_tmix_wkv7_recurrent_bf16 as op

    values = [x.to(DEV) for x in _case(1, 16, 1, seed=1)]
    with pytest.raises(ValueError, match="divisible by the chunk length"):
        op(*(x[:, :8].contiguous() for x in values))
    with pytest.raises(TypeError, match="bfloat16"):
        op(values[0].float(), *values[1:])
    with pytest.raises(ValueError, match="match r shape"):
        op(values[0], values[1][:, :, :32].contiguous(), *values[2:])
    with pytest.raises(ValueError, match="contiguous CUDA"):
        op(values[0].cpu(), *values[1:])
    with pytest.raises(ValueError, match="head_size"):
        op(*values, head_size=32)


def test_against_the_reference_kernels():
    """The reference's own training kernels (forward and backward, unmodified sources built for sm_100 into
    oracle/_ref) on the same tensors: outputs and gradients agree to bf16 rounding of nearly equal fp32 values."""
    import flashrwkv2_b200
    from oracle.build_ref import load_ref

    try:
        ref = load_ref()
    except (ImportError, OSError) as error:
        pytest.skip(f"oracle/_ref/_C_ref.so does not load here: {error}")
    if ref is None or not hasattr(ref, "pretrain_tmix_wkv7_recurrent_forward"):
        pytest.skip("oracle/_ref/_C_ref.so was not built with the reference's training kernels")
    batch, tokens, heads = 2, 64, 4
    rows = [x.to(DEV).view(batch, tokens, heads, 64) for x in _case(batch, tokens, heads, seed=11, magnitude=0.3)]
    dy = torch.randn(batch, tokens, heads, 64, generator=torch.Generator().manual_seed(2)).bfloat16().to(DEV)
    results = []
    for module in (flashrwkv2_b200._C, ref):
        y = torch.empty_like(rows[0])
        boundary = torch.empty(batch, heads, tokens // 16, 64, 64, device=DEV)
        sa = torch.empty(batch, tokens, heads, 64, device=DEV)
        grads = [torch.empty_like(rows[0]) for _ in range(6)]
        module.pretrain_tmix_wkv7_recurrent_forward(*rows, y, boundary, sa, 64)
        module.pretrain_tmix_wkv7_recurrent_backward(*rows, dy, boundary, sa, *grads, 64)
        torch.cuda.synchronize()
        results.append((y.cpu(), boundary.cpu(), sa.cpu(), [g.cpu() for g in grads]))
    (y, boundary, sa, grads), (y_ref, boundary_ref, sa_ref, grads_ref) = results
    rms = lambda t: float(t.float().square().mean().sqrt())
    assert float((boundary - boundary_ref).abs().max()) <= 1e-5 * max(rms(boundary_ref), 1e-6) + 1e-7
    assert float((sa - sa_ref).abs().max()) <= 1e-5 * max(rms(sa_ref), 1e-6) + 1e-7
    assert float((y.float() - y_ref.float()).abs().max()) <= 2.0 ** -7 * float(y_ref.float().abs().max())
    for name, got, want in zip("rwkvab", grads, grads_ref):
        assert float((got.float() - want.float()).abs().max()) <= 2.0 ** -6 * float(want.float().abs().max()), name
