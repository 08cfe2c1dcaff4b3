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

    @property
    def total_tokens(self) -> int:
        return int(sum(self.lengths))

    @property
    def n_seq(self) -> int:
        return len(self.lengths)


def token_tensors(total: int, heads: int, *, generator: torch.Generator, device, dtype,
                  block_tokens: int = 1 << 15) -> dict[str, torch.Tensor]:
    """r, w (retention), k, v, a, b of shape [total, heads, 64] in ``dtype``.
    Generated in blocks of tokens so that the fp32 intermediates stay small."""
    out = {n: torch.empty((total, heads, 64), device=device, dtype=dtype) for n in "rwkvab"}
    for lo in range(0, total, block_tokens):
        hi = min(total, lo + block_tokens)
        shape = (hi - lo, heads, 64)

        def randn():
            return torch.randn(shape, generator=generator, device=device, dtype=torch.float32)

        out["r"][lo:hi] = randn().to(dtype)
        out["k"][lo:hi] = randn().to(dtype)
        out["v"][lo:hi] = randn().to(dtype)
        x = torch.rand(shape, generator=generator, device=device, dtype=torch.float32) * 4.5 - 5.0
        out["w"][lo:hi] = torch.exp(-torch.exp(x)).to(dtype)
        kk = torch.nn.functional.normalize(randn(), dim=-1)
        out["a"][lo:hi] = (-kk).to(dtype)
        out["b"][lo:hi] = (kk * torch.sigmoid(randn())).to(dtype)
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
    ``heads`` shrink a configuration for parity tests.  With ``world > 1`` only the
    sequences :func:`flashrwkv2_b200.sharding.shard_sequences` assigns to ``rank`` are
    generated (each rank seeds with ``seed * 1000 + rank``)."""
    base_n, base_t, base_h, dtype, seed, std, kind = _SPECS[name]
    h = base_h if heads is None else heads
    if name == "c3":
        lengths = _lengths(name, seed, n_seq, seq_len)
    else:
        lengths = [base_t if seq_len is None else seq_len] * (base_n if n_seq is None else n_seq)
    if world > 1:
        from .sharding import shard_sequences

        mine = shard_sequences(lengths, world)[rank]
        lengths = [lengths[i] for i in mine]
        seed = seed * 1000 + rank
    wl = Workload(name, lengths, h, dtype, seed, std, kind)
    if not with_tensors:
        return wl
    g = torch.Generator(device=device).manual_seed(seed)
    total = wl.total_tokens
    wl.tensors = token_tensors(total, h, generator=g, device=device, dtype=dtype)
    n = wl.n_seq
    if std > 0:
        pool = torch.empty((n, h, 64, 64), device=device, dtype=torch.float32)
        for lo in range(0, n, 64):
            hi = min(n, lo + 64)
            pool[lo:hi] = torch.randn((hi - lo, h, 64, 64), generator=g, device=device) * std
    else:
        pool = torch.zeros((n, h, 64, 64), device=device, dtype=torch.float32)
    cu = torch.zeros(n + 1, dtype=torch.int64)
    cu[1:] = torch.tensor(lengths, dtype=torch.int64).cumsum(0)
    wl.tensors["state_pool"] = pool
    wl.tensors["cu_seqlens"] = cu.to(torch.int32).to(device)
    wl.tensors["state_indices"] = torch.arange(n, dtype=torch.int32, device=device)
    return wl
