"""Generates tests/golden/*.npz from the REFERENCE's own oracle function.

Run in a container that has the reference checkout (read-only) mounted:

    python tests/golden/make_golden.py /path/to/FlashRWKV2

It imports ``rwkv7_decay_logits_reference`` from the reference's
``tests/tmix/wkv7/test.py`` (lines 29-85) and ``_reference`` from
``tests/tmix/wkv7/rl_infctx/test.py`` (lines 16-57), feeds them seeded CPU
inputs shaped like the reference's own test cases, and stores inputs and
outputs.  The reference keeps no golden vectors of its own (every case is
generated from a seed), so these files are the pin for the CPU oracle in
``oracle/``.  16-bit tensors are stored as their raw uint16 bit patterns.
The fixtures travel with the repository; the reference checkout does not.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def _case(seed, lengths, slots, pool_slots, heads, dtype, scales, bias_scale=None, state_scale=0.03):
    """Inputs in the style of the reference's _make_case (tests/tmix/wkv7/test.py:170-230),
    drawn on the CPU generator."""
    torch.manual_seed(seed)
    total = sum(lengths)
    shape = (total, heads, 64)
    names = ("r", "decay_logits", "k", "v", "a", "b")
    case = {n: (torch.randn(shape) * s).to(dtype) for n, s in zip(names, scales)}
    cu = [0]
    for length in lengths:
        cu.append(cu[-1] + length)
    case["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32)
    case["state_indices"] = torch.tensor(slots, dtype=torch.int32)
    case["state_pool"] = torch.randn(pool_slots, heads, 64, 64) * state_scale
    case["decay_bias"] = None if bias_scale is None else (torch.randn(heads, 64) * bias_scale).to(dtype)
    return case


def fp16_state(ref) -> None:
    """The fp16-state decode contract: the reference's rwkv7_fp16_reference (tests/tmix/wkv7/test.py:88-149) on a
    ragged fp16 case with bias, scale, permuted slots and nonzero elapsed counters."""
    std = (0.12, 3.5, 0.06, 0.06, 0.06, 0.06)
    case = _case(20260804 + 66, (1, 2, 4, 9, 33), [5, 0, 7, 2, 4], 9, 2, torch.float16, std, bias_scale=0.2)
    state = case["state_pool"].half()
    elapsed = torch.tensor([17, 0, 123456, 3, 99, 1 << 20, 7, 65535, 5], dtype=torch.int32)
    y, final = ref.rwkv7_fp16_reference(
        case["r"], case["decay_logits"], case["k"], case["v"], case["a"], case["b"], state_pool=state,
        elapsed_state_pool=elapsed, cu_seqlens=case["cu_seqlens"], state_indices=case["state_indices"], scale=0.5,
        decay_bias=case["decay_bias"])
    blob = {k: _bits(v) for k, v in case.items() if v is not None and k != "state_pool"}
    blob.update(state_pool=_bits(state), elapsed_state_pool=elapsed.numpy(), y=_bits(y), final_pool=_bits(final),
                scale=np.float64(0.5), dtype=np.array("torch.float16"))
    np.savez_compressed(OUT / "recurrent_fp16_state.npz", **blob)
    print("recurrent_fp16_state", tuple(y.shape), float(y.float().abs().max()))


def main(ref_root: str, only: str | None = None) -> None:
    root = Path(ref_root)
    sys.path[:0] = [str(root), str(root / "tests")]
    ref = _load(root / "tests/tmix/wkv7/test.py", "ref_wkv7_test")
    if only == "fp16_state":
        fp16_state(ref)
        return
    ref_chunk = _load(root / "tests/tmix/wkv7/rl_infctx/test.py", "ref_rl_infctx_test")
    std = (0.12, 3.5, 0.06, 0.06, 0.06, 0.06)
    cases = {
        # the reference's ragged precision case: lengths, permuted slots, scales (test.py:170-230)
        "recurrent_bf16": _case(20260804 + 64, (1, 15, 16, 17, 65), [5, 0, 7, 2, 4], 9, 2, torch.bfloat16, std),
        "recurrent_bf16_bias": _case(20260804 + 65, (1, 15, 16, 17, 65), [5, 0, 7, 2, 4], 9, 2,
                                     torch.bfloat16, std, bias_scale=0.2),
        "recurrent_fp16_bias": _case(20260804 + 65, (1, 15, 16, 17, 65), [5, 0, 7, 2, 4], 9, 2,
                                     torch.float16, std, bias_scale=0.2),
        # a longer sequence so the chunked path crosses several 64-row chunks
        "recurrent_bf16_long": _case(7, (200, 3, 129), [2, 0, 1], 3, 2, torch.bfloat16, std),
        # benchmark-style magnitudes (r,k,v ~ N(0,1)) on one head
        "recurrent_bf16_unit": _case(11, (96, 64), [1, 0], 2, 1, torch.bfloat16,
                                     (1.0, 3.5, 1.0, 1.0, 0.125, 0.125), state_scale=0.1),
    }
    for name, case in cases.items():
        y, pool = ref.rwkv7_decay_logits_reference(
            case["r"], case["decay_logits"], case["k"], case["v"], case["a"], case["b"],
            state_pool=case["state_pool"], cu_seqlens=case["cu_seqlens"],
            state_indices=case["state_indices"], scale=0.5 if "bias" in name else 1.0,
            decay_bias=case["decay_bias"])
        blob = {k: _bits(v) for k, v in case.items() if v is not None}
        blob.update(y=y.numpy(), final_pool=pool.numpy(), scale=np.float64(0.5 if "bias" in name else 1.0),
                    dtype=np.array(str(case["r"].dtype)))
        np.savez_compressed(OUT / f"{name}.npz", **blob)
        print(name, tuple(y.shape), float(y.abs().max()))

    # rl_infctx ragged case (tests/tmix/wkv7/rl_infctx/test.py:60-116): fp16, lengths (2,5), slots [3,1]
    torch.manual_seed(37)
    inputs = [(torch.randn(7, 1, 64) * 0.01).to(torch.float16) for _ in range(6)]
    pool = torch.randn(4, 1, 64, 64) * 0.01
    cu = torch.tensor([0, 2, 7], dtype=torch.int32)
    slots = torch.tensor([3, 1], dtype=torch.int32)
    bias = (torch.randn(1, 64) * 0.01).to(torch.float16)
    y, final = ref_chunk._reference(*inputs, state_pool=pool, cu_seqlens=cu, state_indices=slots, decay_bias=bias)
    blob = {n: _bits(t) for n, t in zip(("r", "decay_logits", "k", "v", "a", "b"), inputs)}
    blob.update(cu_seqlens=cu.numpy(), state_indices=slots.numpy(), state_pool=pool.numpy(),
                decay_bias=_bits(bias), y=_bits(y), final_pool=final.numpy(), scale=np.float64(1.0),
                dtype=np.array("torch.float16"))
    np.savez_compressed(OUT / "rl_infctx_fp16.npz", **blob)
    print("rl_infctx_fp16", tuple(y.shape))
    fp16_state(ref)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/FlashRWKV2 [fp16_state]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
