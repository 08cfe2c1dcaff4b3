"""World-size-2 gloo test of the sharded path on CPU: every rank takes the sequences the
LPT sharder gives it, computes them independently (the oracle stands in for the kernel --
this test is about the host logic), and the union equals the unsharded result; timing
reduction is a max over ranks and the token count a sum."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, str(ROOT))
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from flashrwkv2_b200 import dist as fdist
    from flashrwkv2_b200.sharding import shard_packed
    from flashrwkv2_b200.workloads import make_workload
    from oracle.c_oracle import wkv7_oracle_c

    r, _, w = fdist.init(backend="gloo")
    assert (r, w) == (rank, world)
    wl = make_workload("c3", n_seq=6, seq_len=40, heads=2)
    t = wl.tensors
    shard = shard_packed(t, t["cu_seqlens"], t["state_indices"], world, rank)
    y, pool = wkv7_oracle_c(*(shard[n] for n in "rwkvab"), state_pool=t["state_pool"],
                            cu_seqlens=shard["cu_seqlens"], state_indices=shard["state_indices"],
                            decay_mode="retention", n_threads=1)
    fdist.barrier()
    slowest = fdist.reduce_max(1.0 + rank)
    tokens = fdist.reduce_sum(float(shard["r"].shape[0]))
    everyone = fdist.gather_objects(shard["sequences"])
    torch.save({"rows": shard["rows"], "y": y, "pool": pool, "slots": shard["state_indices"], "slowest": slowest,
                "tokens": tokens, "everyone": everyone}, os.path.join(out_dir, f"rank{rank}.pt"))
    fdist.barrier()
    fdist.shutdown()


def test_two_rank_sharded_run_equals_unsharded(tmp_path):
    from flashrwkv2_b200.workloads import make_workload
    from oracle.c_oracle import wkv7_oracle_c

    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    wl = make_workload("c3", n_seq=6, seq_len=40, heads=2)
    t = wl.tensors
    y_ref, pool_ref = wkv7_oracle_c(*(t[n] for n in "rwkvab"), state_pool=t["state_pool"],
                                    cu_seqlens=t["cu_seqlens"], state_indices=t["state_indices"],
                                    decay_mode="retention", n_threads=1)
    y = torch.zeros_like(y_ref)
    pool = t["state_pool"].clone()
    seen = []
    for rank in range(world):
        blob = torch.load(tmp_path / f"rank{rank}.pt")
        y[blob["rows"]] = blob["y"]
        idx = blob["slots"].long()
        pool[idx] = blob["pool"][idx]
        assert blob["slowest"] == 2.0 and blob["tokens"] == float(wl.total_tokens)
        seen += blob["everyone"][rank]
    assert sorted(seen) == list(range(6))
    assert torch.equal(y, y_ref) and torch.equal(pool, pool_ref)
