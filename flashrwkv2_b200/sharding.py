"""Sequence sharding across the GPUs of one box: no collective on the data path.

The WKV7 recurrence is independent per (sequence, head); the reference already
expresses a batch as independent packed sequences with per-sequence state slots
(rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/__init__.py:224-256).  Whole sequences
are therefore assigned to ranks, longest-processing-time-first on token count;
each rank gets its own re-based ``cu_seqlens``, its rows and its state slots.
A sequence is never split (its state is a serial dependency) and heads are not
split (that would multiply launches without reducing state traffic per token).
"""

from __future__ import annotations

import heapq

import torch


def shard_sequences(lengths, world: int) -> list[list[int]]:
    """LPT assignment: returns, per rank, the sorted list of sequence indices.
    Deterministic (ties broken by sequence index, then by rank)."""
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    heap = [(0, rank) for rank in range(world)]
    heapq.heapify(heap)
    bins: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        load, rank = heapq.heappop(heap)
        bins[rank].append(i)
        heapq.heappush(heap, (load + int(lengths[i]), rank))
    return [sorted(b) for b in bins]


def shard_packed(tensors: dict, cu_seqlens: torch.Tensor, state_indices: torch.Tensor,
                 world: int, rank: int) -> dict:
    """Slice a packed batch for ``rank``: token tensors (any key holding a
    [T_tot, ...] tensor among r,w,k,v,a,b), a re-based ``cu_seqlens`` and the
    rank's ``state_indices`` (which keep addressing the caller's global pool), plus
    ``rows`` -- the global row index of every local row, for scattering y back."""
    cu = [int(x) for x in cu_seqlens.cpu().tolist()]
    lengths = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
    mine = shard_sequences(lengths, world)[rank]
    rows = [torch.arange(cu[i], cu[i + 1]) for i in mine]
    rows_t = torch.cat(rows) if rows else torch.zeros(0, dtype=torch.int64)
    out = {"sequences": mine, "rows": rows_t}
    for name in ("r", "w", "k", "v", "a", "b"):
        if name in tensors:
            out[name] = tensors[name].index_select(0, rows_t.to(tensors[name].device)).contiguous()
    local_cu = torch.zeros(len(mine) + 1, dtype=torch.int64)
    if mine:
        local_cu[1:] = torch.tensor([lengths[i] for i in mine]).cumsum(0)
    out["cu_seqlens"] = local_cu.to(torch.int32).to(cu_seqlens.device)
    idx = torch.tensor(mine, dtype=torch.int64, device=state_indices.device)
    out["state_indices"] = state_indices.index_select(0, idx).contiguous()
    return out
