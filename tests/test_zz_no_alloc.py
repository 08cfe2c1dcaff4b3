"""The allocation-free metadata validation entry, through the C ABI.

`frwkv_sm100_wkv7_validate_metadata_static` is for hosts that have no device memory to offer
as scratch (a binding that owns no allocator, a loop that must never call cudaMalloc): its
duplicate-slot scratch is an array built into the library.  Being integer work, its results
must equal the ordinary entry's exactly.  Two calls are made back to back, the second with
metadata chosen so that anything the first call left in the shared array would show up as a
false duplicate if it were not reset.  This file sorts last so a run that stops at the first
failure has already executed every other test.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _both(lib, cu, slots, pool_size, max_seqlen, n_tok=None, n_seq=None):
    """Run the ordinary entry (caller scratch) and the static entry; return both results."""
    stream = torch.cuda.current_stream().cuda_stream
    n, tokens = slots.numel(), 114
    out = []
    for static in (False, True):
        status = torch.full((3,), -5, dtype=torch.int32, device=DEV)
        cu_snap, slots_snap = torch.full_like(cu, -9), torch.full_like(slots, -9)
        tok_p = 0 if n_tok is None else n_tok.data_ptr()
        seq_p = 0 if n_seq is None else n_seq.data_ptr()
        if static:
            rc = lib.frwkv_sm100_wkv7_validate_metadata_static(
                cu.data_ptr(), slots.data_ptr(), n, tokens, pool_size, max_seqlen, tok_p, seq_p, status.data_ptr(),
                cu_snap.data_ptr(), slots_snap.data_ptr(), stream)
        else:
            seen = torch.empty(pool_size, dtype=torch.int32, device=DEV)
            rc = lib.frwkv_sm100_wkv7_validate_metadata(
                cu.data_ptr(), slots.data_ptr(), n, tokens, pool_size, max_seqlen, tok_p, seq_p, status.data_ptr(),
                seen.data_ptr(), cu_snap.data_ptr(), slots_snap.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        out.append((status.cpu().tolist(), cu_snap.cpu().tolist(), slots_snap.cpu().tolist()))
    return out


def test_static_entry_matches_ordinary_entry_on_consecutive_calls():
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    cu = torch.tensor([0, 1, 16, 32, 49, 114], dtype=torch.int32, device=DEV)
    # call 1: valid metadata, slots 5,0,7,2,4 of a 9-slot pool
    slots = torch.tensor([5, 0, 7, 2, 4], dtype=torch.int32, device=DEV)
    ordinary, static = _both(lib, cu, slots, 9, 114)
    assert static == ordinary and static[0] == [0, 114, 5]
    # call 2, straight after: the same slots in another order, plus the largest pool the entry takes.
    # Stale "seen" marks from call 1 would make every slot look like a duplicate.
    slots2 = torch.tensor([4, 2, 7, 0, 5], dtype=torch.int32, device=DEV)
    ordinary, static = _both(lib, cu, slots2, _lib.STATIC_POOL_SLOTS, 114)
    assert static == ordinary and static[0] == [0, 114, 5]
    # call 3: a real duplicate and a too-long sequence are still reported, identically
    slots3 = torch.tensor([4, 2, 4, 0, 5], dtype=torch.int32, device=DEV)
    ordinary, static = _both(lib, cu, slots3, 9, 64)
    assert static == ordinary and static[0][0] == (1 << 3) | (1 << 5) and static[0][1:] == [0, 0]
    # live active counts (the capacity form) behave the same
    n_tok = torch.tensor([16], dtype=torch.int32, device=DEV)
    n_seq = torch.tensor([2], dtype=torch.int32, device=DEV)
    ordinary, static = _both(lib, cu, slots, 9, 114, n_tok, n_seq)
    assert static == ordinary and static[0] == [0, 16, 2]


def test_static_entry_rejects_pools_beyond_its_scratch():
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    cu = torch.tensor([0, 4], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0], dtype=torch.int32, device=DEV)
    status = torch.full((3,), -5, dtype=torch.int32, device=DEV)
    rc = lib.frwkv_sm100_wkv7_validate_metadata_static(
        cu.data_ptr(), slots.data_ptr(), 1, 4, _lib.STATIC_POOL_SLOTS + 1, 4, 0, 0, status.data_ptr(), 0, 0,
        torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "exceeds the built-in scratch" in _lib.last_error()
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [-5, -5, -5]  # nothing was launched
