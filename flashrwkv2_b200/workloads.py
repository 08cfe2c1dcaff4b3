"""Seeded synthetic WKV7 workloads: the five benchmark configurations.

No public dataset is involved; the reference's own benchmarks are synthetic too
(rwkv-rs/FlashRWKV2 benchmarks/tmix/wkv7/bench.py:238-300).  Distributions, for
every configuration: r, k, v ~ N(0,1); retention w = exp(-exp(x)), x ~ U(-5,-0.5);
kk = L2-normalised N(0,1) over the head dimension; a = -kk; b = kk * sigmoid(N(0,1)).
w is the retention itself (``decay_mode="retention"``), scale = 1, no decay bias,
``state_indices = arange(N)``.

Tensors are generated with ``torch.manual_seed(seed)`` on ``device`` (CPU by
default, so a GPU run and the CPU oracle see identical values after a copy).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class Workload:
    name: str
    lengths: list[int]
    heads: int
    dtype: torch.dtype
    seed: int
    state_std: float  # 0 => zero initial state
    kind: str  # "decode" | "prefill" | "cpu"
    tensors: dict = field(default_factory=dict)
    sequences: list = field(default_factory=list)  # indices of these sequences in the whole (unsharded) batch

    @property
    def total_tokens(self) -> int:
        return int(sum(self.lengths))

    @property
    def n_seq(self) -> int:
        return len(self.lengths)


def token_tensors(total: int, heads: int, *, generator: torch.Generator, device, dtype,
                  block_tokens: int = 1 << 15, keep: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
    """r, w (retention), k, v, a, b of shape [total, heads, 64] in ``dtype``.
    Generated in blocks of tokens so that the fp32 intermediates stay small.  With ``keep`` (a bool
    mask over the ``total`` rows) the whole batch is still drawn, block by block, from the one
    generator, but only the marked rows are stored: a shard is a slice of the one seeded batch."""
    kept = total if keep is None else int(keep.sum().item())
    out = {n: torch.empty((kept, heads, 64), device=device, dtype=dtype) for n in "rwkvab"}
    at = 0
    for lo in range(0, total, block_tokens):
        hi = min(total, lo + block_tokens)
        shape = (hi - lo, heads, 64)
        rows = None if keep is None else keep[lo:hi].nonzero().squeeze(1)
        count = hi - lo if rows is None else int(rows.numel())

        def randn():
            return torch.randn(shape, generator=generator, device=device, dtype=torch.float32)

        def put(name, block):
            if count:
                out[name][at:at + count] = (block if rows is None else block.index_select(0, rows)).to(dtype)

        put("r", randn())
        put("k", randn())
        put("v", randn())
        x = torch.rand(shape, generator=generator, device=device, dtype=torch.float32) * 4.5 - 5.0
        put("w", torch.exp(-torch.exp(x)))
        kk = torch.nn.functional.normalize(randn(), dim=-1)
        put("a", -kk)
        put("b", kk * torch.sigmoid(randn()))
        at += count
    return out


def _lengths(name: str, seed: int, n_seq: int | None, seq_len: int | None) -> list[int]:
    if name == "c3":
        g = torch.Generator().manual_seed(seed)
        n = 64 if n_seq is None else n_seq
        top = 8192 if seq_len is None else seq_len
        return [int(x) for x in torch.randint(1, top + 1, (n,), generator=g).tolist()]
    raise KeyError(name)


_SPECS = {
    # name: (n_seq, seq_len, heads, dtype, seed, state_std, kind)
    "c0": (1, 64, 32, torch.float32, 0, 0.0, "cpu"),
    "c1": (256, 1, 32, torch.bfloat16, 1, 0.1, "decode"),
    "c2": (8, 4096, 32, torch.bfloat16, 2, 0.1, "prefill"),
    "c3": (64, None, 40, torch.bfloat16, 3, 0.1, "prefill"),
    "c4_decode": (2048, 1, 64, torch.bfloat16, 4, 0.1, "decode"),
    "c4_prefill": (64, 8192, 64, torch.bfloat16, 4, 0.1, "prefill"),
}


def describe(name: str) -> str:
    n, t, h, dt, seed, std, kind = _SPECS[name]
    t_txt = "U[1,8192]" if t is None else str(t)
    return f"{name}: {kind} N={n} T={t_txt} H={h} D=64 {str(dt).split('.')[-1]} seed={seed}"


def make_workload(name: str, *, device="cpu", n_seq: int | None = None, seq_len: int | None = None,
                  heads: int | None = None, rank: int = 0, world: int = 1,
                  with_tensors: bool = True) -> Workload:
    """Build one of c0, c1, c2, c3, c4_decode, c4_prefill.  ``n_seq`` / ``seq_len`` /
    ``heads`` shrink a configuration for parity tests.  With ``world > 1`` the rank keeps the
    sequences :func:`flashrwkv2_b200.sharding.shard_sequences` assigns to it: every rank draws
    the whole batch from the same seed, block by block, and stores only its own rows and state
    slots, so the union of the shards is exactly the single-GPU batch."""
    base_n, base_t, base_h, dtype, seed, std, kind = _SPECS[name]
    h = base_h if heads is None else heads
    if name == "c3":
        all_lengths = _lengths(name, seed, n_seq, seq_len)
    else:
        all_lengths = [base_t if seq_len is None else seq_len] * (base_n if n_seq is None else n_seq)
    mine = list(range(len(all_lengths)))
    if world > 1:
        from .sharding import shard_sequences

        mine = shard_sequences(all_lengths, world)[rank]
    lengths = [all_lengths[i] for i in mine]
    wl = Workload(name, lengths, h, dtype, seed, std, kind)
    wl.sequences = mine
    if not with_tensors:
        return wl
    g = torch.Generator(device=device).manual_seed(seed)
    total = int(sum(all_lengths))
    keep = None
    if world > 1:
        starts = [0]
        for length in all_lengths:
            starts.append(starts[-1] + length)
        keep = torch.zeros(total, dtype=torch.bool, device=device)
        for i in mine:
            keep[starts[i]:starts[i + 1]] = True
    wl.tensors = token_tensors(total, h, generator=g, device=device, dtype=dtype, keep=keep)
    n = wl.n_seq
    if std > 0:
        pool = torch.empty((n, h, 64, 64), device=device, dtype=torch.float32)
        local = {seq: j for j, seq in enumerate(mine)}
        for lo in range(0, len(all_lengths), 64):
            hi = min(len(all_lengths), lo + 64)
            block = torch.randn((hi - lo, h, 64, 64), generator=g, device=device) * std
            for seq in range(lo, hi):
                if seq in local:
                    pool[local[seq]] = block[seq - lo]
    else:
        pool = torch.zeros((n, h, 64, 64), device=device, dtype=torch.float32)
    cu = torch.zeros(n + 1, dtype=torch.int64)
    cu[1:] = torch.tensor(lengths, dtype=torch.int64).cumsum(0)
    wl.tensors["state_pool"] = pool
    wl.tensors["cu_seqlens"] = cu.to(torch.int32).to(device)
    wl.tensors["state_indices"] = torch.arange(n, dtype=torch.int32, device=device)
    return wl
