"""WKV7 benchmark: tokens/s and fraction of roofline on 1/2/4/8 B200, next to the CPU recurrence.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c4|c1|c2|c3|c4_decode|c4_prefill] [--no-extras] [--no-e2e]
                    [--extra fp16_state|fused_gate|readout|pretrain|gpu_baseline] [--min-region-s S]

Default workload ``c4``: the 7B-width batch sharded by sequence over the N GPUs of one box (strong scaling: the
total work is fixed, every rank keeps the sequences the longest-first sharder gives it, all sliced from the one
seeded batch; no collective on the data path).  It has two parts:

  * headline -- decode step, 2048 sequences x 1 token, H=64, D=64, bf16 tokens, fp32 state updated in place
    (``value``, ``ms_per_step``, ``roofline`` against HBM, ``e2e``, ``clocks``);
  * ``prefill`` -- 64 sequences x 8192 tokens, H=64, through the tensor-core chunk kernel, a block of the same
    shape (its own ``value``, ``ms_per_step``, ``roofline`` with the HBM and the tensor fraction, ``clocks``).

A step is one pass of the operator over the batch (one decode launch; one prefill call).  The timed region is K
steps times R back-to-back repeats, R chosen from the warm-up so that the region lasts at least half a second;
``ms_per_step`` is per step.  Times are CUDA events, maximum over ranks.  With ``--workload`` one of the single
configurations is measured instead (also sharded when N > 1).  On one GPU the smaller configurations (c1 decode
256 x H32, c2 dense prefill 8 x 4096 x H32, c3 ragged prefill) are appended under ``extras`` together with the
reference's own CUDA kernels on the same GPU.

Keys of the JSON line:
  value      tokens/s with inputs resident in HBM, through the C ABI;
  e2e        tokens/s through the public Python operator with the six token tensors copied from pinned host
             memory and y copied back to the host inside the timed region (the state pool is device-resident by
             contract), plus the host time one operator call takes;
  roofline   algorithmic bytes per launch / average duration against the measured HBM copy bandwidth
             (prefill: also counted flop against the measured bf16 peak);
  cpu_baseline  the port of the reference's fp32 PyTorch recurrence on the host cores, bounded sample.

``--impl reference`` times the reference's CPU implementation of the path (its fp32 PyTorch token loop, restated
in oracle/wkv7_oracle.py: its package refuses to import on capability 10.x and its CPU path is that loop) on the
same workload.  That process hides the GPUs before torch is imported, so the product's libraries are never loaded
into it.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "WKV7 tokens/s & % roofline (decode HBM, prefill TC) at 1/2/4/8 B200"
ALGO_BYTES_DECODE_PAIR = 16384 + 16384 + 6 * 128 + 128  # state in + out, six bf16 rows, one bf16 y row
ALGO_BYTES_DECODE_FP16_STATE_PAIR = 8192 + 8192 + 6 * 128 + 128  # the fp16-state contract: half the state bytes
ALGO_FLOP_PREFILL_TOKEN_HEAD = 98304  # 12 GEMMs of 64^3 per 64 rows
ALGO_BYTES_PREFILL_TOKEN_HEAD = 7 * 128
ALGO_BYTES_PREFILL_PAIR = 32768
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# DRAM bytes of one launch (read + written) from ncu captures (profiles/): decode from captures of the c4_decode
# launch itself (131,072 pairs) and of the c1 launch (8,192 pairs); the other forms per (sequence, head) of their
# c4-sized captures; prefill per (token, head), from a capture of the c2 launch (traffic grows in proportion to the
# units).  Reads equal the algorithmic bytes; the state written by the last CTAs is still dirty in L2 when a kernel
# ends, so the totals are a little below them.
DECODE_DIRTY_IN_L2_BYTES = 58.0e6  # 4.412 GB algorithmic - 4.354 GB measured (c4); 275.8 MB - 217.2 MB (c1)
DECODE_FP16_STATE_TRAFFIC_PER_PAIR = 2.211e9 / 131072
DECODE_READOUT_TRAFFIC_PER_PAIR = 4.383e9 / 131072
PREFILL_TRAFFIC_PER_TOKEN_HEAD = (809.58e6 + 127.15e6) / (32768 * 32)
MIN_REGION_S = 0.5

DECODE_WORKLOADS = ("c1", "c4_decode")


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def workload_config(name: str, world: int) -> dict:
    """The ``config`` object: identical in both arms for the same command line."""
    from flashrwkv2_b200.workloads import describe

    parts = {"c4": ["c4_decode", "c4_prefill"]}.get(name, [name])
    return {
        "workload": " + ".join(describe(p) for p in parts),
        "headline": describe(parts[0]),
        "sharding": (f"by sequence over {world} GPU(s), longest first, every shard a slice of the one seeded batch; "
                     "no collective"),
        "decay_mode": "retention", "io_dtype": "bf16", "state_dtype": "fp32",
        "l2": ("decode: state pools in rotation, at least 1 GiB per GPU and every launch's own state larger than "
               "L2; prefill: inputs of one step larger than L2"),
        "timed_region": f"K steps x R repeats back to back, R such that the region lasts >= {MIN_REGION_S} s",
    }


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed regions run."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(", ") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
        os.unlink(self.file.name)
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            if len(row) < 9:
                continue
            try:
                sm.append(float(row[1]))
                sm_max.append(float(row[2]))
                power.append(float(row[3]))
            except ValueError:
                continue
            for name, flag in zip(names, row[5:9]):
                if flag.strip().lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        cut = statistics.median(power)  # "under load": the samples in the upper half of the power readings
        loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def _event_time_ms(fn, count, finish=None):
    import torch

    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(count):
        fn(i)
    if finish is not None:
        finish()
    end.record()
    end.synchronize()
    return start.elapsed_time(end)


def _timed_region(step, steps, warmup, fdist):
    """Warm up, pick the repeat count from the warm-up, time steps x repeats; returns (ms per step, repeats)."""
    import torch

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    probe = max(3, min(warmup, 10))
    estimate_ms = fdist.reduce_max(_event_time_ms(step, probe) / probe)
    repeats = max(1, math.ceil(MIN_REGION_S * 1e3 / max(estimate_ms * steps, 1e-6)))
    repeats = int(fdist.reduce_max(repeats))
    fdist.barrier()
    elapsed_ms = _event_time_ms(step, steps * repeats)
    fdist.barrier()
    return fdist.reduce_max(elapsed_ms) / (steps * repeats), repeats


def _roofline(name, kind, peaks, peak_kind, ms_per_step, pairs, token_heads):
    if kind == "decode":
        algo = pairs * ALGO_BYTES_DECODE_PAIR
        # reads are counted in full; of the state a launch writes, what is still dirty in L2 when the kernel ends
        # (about 58 MB in both captures: the 8,192-pair c1 launch and the 131,072-pair c4 launch) is not
        traffic = int(max(pairs * (16384 + 6 * 128), pairs * ALGO_BYTES_DECODE_PAIR - DECODE_DIRTY_IN_L2_BYTES))
        kernel = "wkv7_recurrent_stream_kernel"
    else:
        algo = token_heads * ALGO_BYTES_PREFILL_TOKEN_HEAD + pairs * ALGO_BYTES_PREFILL_PAIR
        traffic = int(token_heads * PREFILL_TRAFFIC_PER_TOKEN_HEAD)
        kernel = "wkv7_chunk32_tc_kernel"
    achieved = algo / (ms_per_step * 1e-3) / 1e9
    out = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
           "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": traffic, "peak_kind": f"of {peak_kind}",
           "algorithmic_bytes_per_launch": algo, "kernel": kernel, "per": "launch on the slowest rank's GPU"}
    if kind != "decode":
        tflops = token_heads * ALGO_FLOP_PREFILL_TOKEN_HEAD / (ms_per_step * 1e-3) / 1e12
        out["tensor_tflops"] = round(tflops, 2)
        out["tensor_frac_of_bf16_peak"] = round(tflops / peaks["bf16_tflops"], 4)
        # for reference: the flop the recurrence itself needs, 9 D^2 per (token, head), at the same time
        out["recurrence_minimal_tflops"] = round(token_heads * 9 * 64 * 64 / (ms_per_step * 1e-3) / 1e12, 2)
    return out


def measure(name, args, rank, local_rank, world, *, with_e2e=True, steps=None, warmup=None):
    """One workload on this rank's shard: device-resident timing, roofline, clocks and (optionally) end to end."""
    import torch

    from flashrwkv2_b200 import _lib, dist as fdist
    from flashrwkv2_b200.tmix import wkv7 as ops
    from flashrwkv2_b200.workloads import describe, make_workload

    device = torch.device("cuda", local_rank)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()
    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    is_decode = name in DECODE_WORKLOADS
    stream = torch.cuda.current_stream().cuda_stream
    wl = make_workload(name, device=device, rank=rank, world=world)
    t = wl.tensors
    n_seq, heads, tokens = wl.n_seq, wl.heads, wl.total_tokens
    sampler = ClockSampler(local_rank).start()

    if is_decode:
        # rotating state pools: every launch streams its state from HBM (no pool is still in L2 when it comes round)
        state_bytes = n_seq * heads * 16384
        n_sets = max(2, math.ceil(2**30 / state_bytes))
        if state_bytes >= 2**30:
            n_sets = 1
        pools = [t["state_pool"]] + [t["state_pool"].clone() for _ in range(n_sets - 1)]
        ys = [torch.empty_like(t["v"]) for _ in range(n_sets)]

        def step(i):
            j = i % n_sets
            rc = lib.frwkv_sm100_wkv7_recurrent(
                t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, pools[j].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
                t["b"].data_ptr(), 0, ys[j].data_ptr(), 0, n_seq, tokens, heads, _lib.IO_BF16,
                _lib.DECAY_RETENTION, 1.0, 1, stream)
            if rc:
                raise RuntimeError(_lib.last_error())

        launches_per_step = 1
        l2_note = f"{n_sets} state pool(s) of {state_bytes / 2**20:.0f} MiB in rotation"
    else:
        y = torch.empty_like(t["v"])
        need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n_seq, tokens, heads)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        err = torch.zeros(1, dtype=torch.int32, device=device)
        max_len = max(wl.lengths)

        def step(i):
            rc = lib.frwkv_sm100_wkv7_prefill(
                t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
                t["b"].data_ptr(), 0, y.data_ptr(), 0, n_seq, tokens, heads, _lib.IO_BF16,
                _lib.DECAY_RETENTION, 1.0, max_len, _lib.PREFILL_AUTO, ws.data_ptr(), need, err.data_ptr(), stream)
            if rc:
                raise RuntimeError(_lib.last_error())

        # length ranking (2..2048 sequences), recurrence kernel for rows under 16 tokens, chunk kernel
        launches_per_step = 3 if 1 < n_seq <= 2048 else 2
        l2_note = f"inputs of one step {tokens * heads * 896 / 2**20:.0f} MiB"

    ms_per_step, repeats = _timed_region(step, steps, warmup, fdist)
    total_tokens = fdist.reduce_sum(tokens)
    clocks = sampler.stop()
    max_pairs = int(fdist.reduce_max(n_seq * heads))
    max_token_heads = int(fdist.reduce_max(tokens * heads))
    block = {
        "workload": describe(name), "value": round(total_tokens / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
        "ms_per_step": round(ms_per_step, 6), "steps": steps, "repeats": repeats,
        "tokens_per_step": int(total_tokens), "l2": l2_note,
        "gpu_launches": steps * repeats * launches_per_step,
        "roofline": _roofline(name, "decode" if is_decode else "prefill", peaks, peak_kind, ms_per_step, max_pairs,
                              max_token_heads),
        "clocks": clocks,
    }
    if not is_decode:
        block["error_flag"] = int(err.item())

    h2d = sum(t[n].numel() * t[n].element_size() for n in "rwkvab")
    d2h = t["v"].numel() * t["v"].element_size()
    if with_e2e and not args.no_e2e and h2d <= 8 * 2**30:  # bound pinned host memory on shared boxes
        # the caller's six token tensors live in one pinned host block -> one host->device copy per step.
        # Two streams, as a serving loop would run it: step i+1's upload overlaps step i's kernel and the
        # download of its y (PCIe is full duplex); every step still uploads its inputs and downloads its result.
        host = torch.stack([t[n].cpu() for n in "rwkvab"]).pin_memory()
        dev_in = [torch.empty_like(host, device=device) for _ in range(2)]
        y_host = [torch.empty(t["v"].shape, dtype=t["v"].dtype).pin_memory() for _ in range(2)]
        pool, cu, slots = t["state_pool"], t["cu_seqlens"], t["state_indices"]
        ticket = ops.prepare_tmix_wkv7_recurrent_metadata(cu, slots, total_tokens=tokens,
                                                          state_pool_size=pool.shape[0])
        op = (ops.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen if is_decode
              else ops.infer_tmix_wkv7_prefill_fp32io16_forward_varlen)
        main_stream = torch.cuda.current_stream()
        up_stream = torch.cuda.Stream()
        uploaded = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        for ev in consumed:
            ev.record(main_stream)
        host_s = [0.0, 0]

        def e2e_step(i):
            j = i % 2
            up_stream.wait_event(consumed[j])  # the kernel that last read this input buffer has finished
            with torch.cuda.stream(up_stream):
                dev_in[j].copy_(host, non_blocking=True)
                uploaded[j].record(up_stream)
            main_stream.wait_event(uploaded[j])
            d = dev_in[j]
            begin = time.perf_counter()
            out = op(d[0], d[1], d[2], d[3], d[4], d[5], state_pool=pool, cu_seqlens=cu, state_indices=slots,
                     validated_metadata=ticket, decay_mode="retention")
            host_s[0] += time.perf_counter() - begin
            host_s[1] += 1
            consumed[j].record(main_stream)
            y_host[j].copy_(out, non_blocking=True)

        def e2e_finish():
            main_stream.wait_stream(up_stream)

        for i in range(5):
            e2e_step(i)
        torch.cuda.synchronize()
        probe_ms = fdist.reduce_max(_event_time_ms(e2e_step, 5, e2e_finish) / 5)
        e2e_steps = int(fdist.reduce_max(max(2000 if probe_ms < 0.25 else 3, math.ceil(MIN_REGION_S * 1e3 / probe_ms))))
        host_s[0], host_s[1] = 0.0, 0
        fdist.barrier()
        e2e_ms = _event_time_ms(e2e_step, e2e_steps, e2e_finish)
        fdist.barrier()
        e2e_ms = fdist.reduce_max(e2e_ms)
        block["e2e"] = {"value": round(total_tokens / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "tokens/s",
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                        "ms_per_step": round(e2e_ms / e2e_steps, 6),
                        "host_us_per_operator_call": round(host_s[0] / max(1, host_s[1]) * 1e6, 2)}
    else:
        block["e2e"] = None
    block["_workload_object"] = wl
    return block


def measure_fp16_state_decode(args, local_rank):
    """The fp16-state decode contract on the 7B-width decode batch (2048 sequences, H=64, fp16 tokens, decay
    logits, fp16 state pool): same kernel, half the state traffic.  One GPU, device-resident."""
    import torch

    from flashrwkv2_b200 import _lib, dist as fdist
    from flashrwkv2_b200.workloads import make_workload

    device = torch.device("cuda", local_rank)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()
    wl = make_workload("c4_decode", device=device)
    t = wl.tensors
    n_seq, heads, tokens = wl.n_seq, wl.heads, wl.total_tokens
    tok = {n: t[n].half() for n in "rkvab"}
    sig = (-torch.log(t["w"].float()) / 0.6065306597126334).clamp(1e-4, 1 - 1e-4)
    tok["w"] = torch.log(sig / (1 - sig)).half()  # the decay logits whose retention is w
    pool = t["state_pool"].half()  # 1 GiB: every launch streams it from HBM
    err = torch.zeros(1, dtype=torch.int32, device=device)
    elapsed = torch.zeros(n_seq, dtype=torch.int32, device=device)
    y = torch.empty_like(tok["v"])
    stream = torch.cuda.current_stream().cuda_stream
    sampler = ClockSampler(local_rank).start()

    def step(i):
        rc = lib.frwkv_sm100_wkv7_recurrent_fp16_state(
            t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, elapsed.data_ptr(), pool.data_ptr(), n_seq,
            tok["r"].data_ptr(), tok["w"].data_ptr(), tok["k"].data_ptr(), tok["v"].data_ptr(), tok["a"].data_ptr(),
            tok["b"].data_ptr(), 0, y.data_ptr(), n_seq, tokens, heads, _lib.DECAY_LOGITS, 1.0, 1, err.data_ptr(),
            stream)
        if rc:
            raise RuntimeError(_lib.last_error())

    ms_per_step, repeats = _timed_region(step, args.steps, args.warmup, fdist)
    algo = n_seq * heads * ALGO_BYTES_DECODE_FP16_STATE_PAIR
    achieved = algo / (ms_per_step * 1e-3) / 1e9
    return {"workload": "c4_decode shapes, fp16 tokens (decay logits), fp16 state pool, elapsed-phase dither",
            "value": round(tokens / (ms_per_step * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms_per_step, 6),
            "steps": args.steps, "repeats": repeats, "gpu_launches": 2 * args.steps * repeats,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": int(n_seq * heads * DECODE_FP16_STATE_TRAFFIC_PER_PAIR),
                         "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo,
                         "kernel": "wkv7_decode_fp16_state_kernel + advance_elapsed_kernel"},
            "error_flag": int(err.item()), "clocks": sampler.stop()}


def measure_fused_gate(args, local_rank):
    """The fused kk / a-gate input form (five token tensors instead of six; a, b and the gated key formed in
    registers): decode step at the c4_decode shapes and dense prefill at the c2 shapes, one GPU, device-resident."""
    import torch

    from flashrwkv2_b200 import _lib, dist as fdist
    from flashrwkv2_b200.workloads import make_workload

    device = torch.device("cuda", local_rank)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for name in ("c4_decode", "c2"):
        wl = make_workload(name, device=device)
        t = wl.tensors
        n_seq, heads, tokens = wl.n_seq, wl.heads, wl.total_tokens
        g = torch.Generator(device=device).manual_seed(17)
        a12 = (torch.randn(t["k"].shape, generator=g, device=device) * 1.5).to(t["k"].dtype)
        k_k = (1.0 + 0.3 * torch.randn(heads * 64, generator=g, device=device)).to(t["k"].dtype)
        a0 = (0.5 * torch.randn(heads * 64, generator=g, device=device)).to(t["k"].dtype)
        k_a = torch.rand(heads * 64, generator=g, device=device).to(t["k"].dtype)
        y = torch.empty_like(t["v"])
        err = torch.zeros(1, dtype=torch.int32, device=device)
        need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n_seq, tokens, heads)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        decode = name == "c4_decode"
        head = (t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), a12.data_ptr(),
                k_k.data_ptr(), a0.data_ptr(), k_a.data_ptr(), 0, y.data_ptr(), 0, n_seq, tokens, heads, _lib.IO_BF16,
                _lib.DECAY_RETENTION, 1.0, max(wl.lengths))

        def step(i):
            if decode:
                rc = lib.frwkv_sm100_wkv7_recurrent_fused_gate(*head, stream)
            else:
                rc = lib.frwkv_sm100_wkv7_prefill_fused_gate(*head, _lib.PREFILL_AUTO, ws.data_ptr(), need, err.data_ptr(),
                                                             stream)
            if rc:
                raise RuntimeError(_lib.last_error())

        ms_per_step, repeats = _timed_region(step, args.steps, args.warmup, fdist)
        pairs, token_heads = n_seq * heads, tokens * heads
        algo = pairs * (32768 + 5 * 128 + 128) if decode else token_heads * (5 * 128 + 128) + pairs * 32768
        achieved = algo / (ms_per_step * 1e-3) / 1e9
        out[name] = {"value": round(tokens / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
                     "ms_per_step": round(ms_per_step, 6), "repeats": repeats,
                     "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                                  "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": None,
                                  "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo},
                     "error_flag": int(err.item())}
        del wl, t
        torch.cuda.empty_cache()
    out["workload"] = "five token tensors (r, w, raw k, v, a12) + per-channel k_k, a0, k_a; 640 B in + 128 B out per (token, head)"
    return out


def measure_readout(args, local_rank):
    """The recurrence kernel with the readout's elementwise stage (head norm, r.k residual, output gate) as its
    epilogue, decode step at the c4_decode shapes, one GPU, device-resident: the plain input form (six token
    tensors + the output gate in, the gated result out; y is not stored) and the form with the kk / a-gate
    producer fused in as well (five token tensors + the gate)."""
    import torch

    from flashrwkv2_b200 import _lib, dist as fdist
    from flashrwkv2_b200.workloads import make_workload

    device = torch.device("cuda", local_rank)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    wl = make_workload("c4_decode", device=device)
    t = wl.tensors
    n_seq, heads, tokens = wl.n_seq, wl.heads, wl.total_tokens
    dtype = t["k"].dtype
    g = torch.Generator(device=device).manual_seed(23)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=device)
    gate = rnd(*t["k"].shape).to(dtype)
    a12 = (rnd(*t["k"].shape) * 1.5).to(dtype)
    r_k, ln_w, ln_b = (0.2 * rnd(heads * 64)).to(dtype), (1.0 + 0.2 * rnd(heads * 64)).to(dtype), (0.1 * rnd(heads * 64)).to(dtype)
    k_k, a0, k_a = (1.0 + 0.3 * rnd(heads * 64)).to(dtype), (0.5 * rnd(heads * 64)).to(dtype), torch.rand(heads * 64, generator=g, device=device).to(dtype)
    x = torch.empty_like(t["v"])
    out = {}
    for label, fused in (("plain_inputs", False), ("fused_gate_inputs", True)):
        call = (t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(),
                a12.data_ptr() if fused else t["a"].data_ptr(), 0 if fused else t["b"].data_ptr(),
                k_k.data_ptr() if fused else 0, a0.data_ptr() if fused else 0, k_a.data_ptr() if fused else 0, 0,
                gate.data_ptr(), r_k.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), x.data_ptr(), 0, 0, n_seq, tokens,
                heads, _lib.IO_BF16, _lib.DECAY_RETENTION, 1.0, 1, stream)

        def step(i):
            rc = lib.frwkv_sm100_wkv7_recurrent_readout(*call)
            if rc:
                raise RuntimeError(_lib.last_error())

        ms_per_step, repeats = _timed_region(step, args.steps, args.warmup, fdist)
        pairs = n_seq * heads
        algo = pairs * (32768 + (6 if fused else 7) * 128 + 128)
        achieved = algo / (ms_per_step * 1e-3) / 1e9
        out[label] = {"value": round(tokens / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
                      "ms_per_step": round(ms_per_step, 6), "repeats": repeats,
                      "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": None if fused else int(pairs * DECODE_READOUT_TRAFFIC_PER_PAIR),
                                   "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo}}
    out["workload"] = ("c4_decode shapes; the token tensors + the output gate in, the gated readout result out "
                       "(y not stored); the two-operator pipeline moves 768 B more per (token, head)")
    del wl, t, gate, a12, x
    torch.cuda.empty_cache()
    # prefill rows (c2 shapes): chunk kernel, then the readout stage as a second, HBM-bound launch over the stored y
    wl = make_workload("c2", device=device)
    t = wl.tensors
    n_seq, heads, tokens = wl.n_seq, wl.heads, wl.total_tokens
    gate = rnd(*t["k"].shape).to(dtype)
    r_k, ln_w, ln_b = (0.2 * rnd(heads * 64)).to(dtype), (1.0 + 0.2 * rnd(heads * 64)).to(dtype), (0.1 * rnd(heads * 64)).to(dtype)
    x, y = torch.empty_like(t["v"]), torch.empty_like(t["v"])
    err = torch.zeros(1, dtype=torch.int32, device=device)
    need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n_seq, tokens, heads)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
    call = (t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
            t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
            t["b"].data_ptr(), 0, 0, 0, 0, gate.data_ptr(), r_k.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(),
            x.data_ptr(), y.data_ptr(), 0, n_seq, tokens, heads, _lib.IO_BF16, _lib.DECAY_RETENTION, 1.0,
            max(wl.lengths), _lib.PREFILL_AUTO, ws.data_ptr(), need, err.data_ptr(), stream)

    def prefill_step(i):
        rc = lib.frwkv_sm100_wkv7_prefill_readout(*call)
        if rc:
            raise RuntimeError(_lib.last_error())

    ms_per_step, repeats = _timed_region(prefill_step, args.steps, args.warmup, fdist)
    token_heads = tokens * heads
    algo = token_heads * (7 * 128 + 6 * 128) + n_seq * heads * 32768
    achieved = algo / (ms_per_step * 1e-3) / 1e9
    out["prefill_c2"] = {"value": round(tokens / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
                         "ms_per_step": round(ms_per_step, 6), "repeats": repeats,
                         "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                                      "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": None,
                                      "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo},
                         "kernels": "wkv7_chunk32_tc_kernel + wkv7_readout_rows_kernel (two launches; y round trip)",
                         "error_flag": int(err.item())}
    del wl, t
    torch.cuda.empty_cache()
    return out


def measure_pretrain(args, local_rank):
    """The WKV7 training operator (forward with checkpoints + backward) on a dense 8 x 4096 x H32 bf16 batch, next to
    the reference's own training kernels on the same tensors when oracle/_ref holds them.  CUDA-core kernels bound by
    the per-token chain; reported for completeness of the operator family."""
    import torch

    import flashrwkv2_b200
    from oracle.build_ref import load_ref

    device = torch.device("cuda", local_rank)
    batch, tokens, heads = 8, 4096, 32
    g = torch.Generator(device=device).manual_seed(29)
    shape = (batch, tokens, heads, 64)
    rnd = lambda: torch.randn(shape, generator=g, device=device)
    r, k, v = (rnd().mul_(0.5).bfloat16() for _ in range(3))
    w = rnd().mul_(3.0).bfloat16()
    kk = torch.nn.functional.normalize(rnd(), dim=-1)
    a, b = (-kk).bfloat16(), (kk * torch.sigmoid(rnd())).bfloat16()
    dy = rnd().bfloat16()
    out = {"workload": f"dense B={batch} T={tokens} H={heads} D=64 bf16, zero initial state"}
    modules = [("this_build", flashrwkv2_b200._C)]
    try:
        ref = load_ref()
    except (ImportError, OSError):
        ref = None
    if ref is not None and hasattr(ref, "pretrain_tmix_wkv7_recurrent_forward"):
        modules.append(("reference_kernels", ref))
    for label, module in modules:
        y = torch.empty_like(r)
        boundary = torch.empty(batch, heads, tokens // 16, 64, 64, device=device)
        sa = torch.empty(shape, device=device)
        grads = [torch.empty_like(r) for _ in range(6)]
        forward = lambda i: module.pretrain_tmix_wkv7_recurrent_forward(r, w, k, v, a, b, y, boundary, sa, 64)
        backward = lambda i: module.pretrain_tmix_wkv7_recurrent_backward(r, w, k, v, a, b, dy, boundary, sa, *grads, 64)
        times = []
        for fn in (forward, backward):
            fn(0)
            times.append(_event_time_ms(fn, 5) / 5)
        out[label] = {"forward_ms": round(times[0], 3), "backward_ms": round(times[1], 3),
                      "tokens_per_s_forward_backward": round(batch * tokens / (sum(times) * 1e-3), 1)}
    return out


def run_ours(args, rank, local_rank, world):
    import torch

    torch.cuda.set_device(local_rank)
    name = args.workload
    head_name = "c4_decode" if name == "c4" else name
    head = measure(head_name, args, rank, local_rank, world)
    wl = head.pop("_workload_object")
    line = {
        "metric": METRIC, "value": head["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(name, world),
        "repeats": head["repeats"], "tokens_per_step": head["tokens_per_step"], "clocks": head["clocks"],
        "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "roofline": head["roofline"],
    }
    if rank == 0 and world == 1 and not args.no_extras:
        line["cpu_baseline"] = cpu_baseline(head_name, wl)
    del wl
    torch.cuda.empty_cache()
    if name == "c4":
        prefill = measure("c4_prefill", args, rank, local_rank, world, with_e2e=False)
        prefill.pop("_workload_object")
        line["prefill"] = prefill
        line["gpu_launches"] += prefill["gpu_launches"]
        torch.cuda.empty_cache()
    if world == 1 and not args.no_extras and name == "c4":
        extras = {}
        for extra in ("c1", "c2", "c3"):
            try:
                block = measure(extra, args, rank, local_rank, world, with_e2e=extra == "c1")
                block.pop("_workload_object")
                extras[extra] = block
            except RuntimeError as error:  # reported, not hidden
                extras[extra] = {"error": str(error)}
            torch.cuda.empty_cache()
        try:
            extras["c4_decode_fp16_state"] = measure_fp16_state_decode(args, local_rank)
        except RuntimeError as error:
            extras["c4_decode_fp16_state"] = {"error": str(error)}
        torch.cuda.empty_cache()
        try:
            extras["fused_gate"] = measure_fused_gate(args, local_rank)
        except RuntimeError as error:
            extras["fused_gate"] = {"error": str(error)}
        try:
            extras["readout_epilogue"] = measure_readout(args, local_rank)
        except Exception as error:  # noqa: BLE001
            extras["readout_epilogue"] = {"error": str(error)}
        try:
            extras["pretrain"] = measure_pretrain(args, local_rank)
        except Exception as error:  # noqa: BLE001
            extras["pretrain"] = {"error": str(error)}
        torch.cuda.empty_cache()
        torch.cuda.empty_cache()
        try:
            extras["gpu_baseline"] = gpu_baseline(torch.device("cuda", local_rank))
        except Exception as error:  # a baseline that cannot load or run must not take the bench line with it
            extras["gpu_baseline"] = {"error": f"{type(error).__name__}: {error}"}
        line["extras"] = extras
    return line


def _cpu_sample(name, wl, limit_s=10.0, use_c=False):
    """Time the CPU recurrence on a bounded sample of the workload; returns (tokens/s, cores, text)."""
    import torch

    from oracle import c_oracle
    from oracle.wkv7_oracle import wkv7_oracle

    t = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in wl.tensors.items()}
    lengths = wl.lengths
    prefix = 1 if max(lengths) == 1 else min(max(lengths), 16)
    # first `prefix` tokens of every sequence, all heads
    rows, cu = [], [0]
    base = 0
    for length in lengths:
        take = min(length, prefix)
        rows.append(torch.arange(base, base + take))
        cu.append(cu[-1] + take)
        base += length
    rows = torch.cat(rows)
    toks = [t[n].index_select(0, rows).contiguous() for n in "rwkvab"]
    kw = dict(state_pool=t["state_pool"], cu_seqlens=torch.tensor(cu, dtype=torch.int32),
              state_indices=t["state_indices"], decay_mode="retention")
    fn = (lambda: c_oracle.wkv7_oracle_c(*toks, **kw)) if use_c else (lambda: wkv7_oracle(*toks, **kw))
    fn()  # warm
    done, reps = 0.0, 0
    begin = time.perf_counter()
    while done < limit_s and reps < 2000:
        fn()
        reps += 1
        done = time.perf_counter() - begin
    tokens = int(rows.numel()) * reps
    cores = c_oracle.max_threads() if use_c else torch.get_num_threads()
    sample = (f"first {prefix} token(s) of each of {len(lengths)} sequences, all {wl.heads} heads, "
              f"{reps} repetition(s), {done:.1f} s")
    return tokens / done, cores, sample


def cpu_baseline(name, wl):
    value, cores, sample = _cpu_sample(name, wl, use_c=False)
    c_value, c_cores, _ = _cpu_sample(name, wl, limit_s=3.0, use_c=True)
    return {"value": round(value, 1), "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": sample + " (fp32 PyTorch token loop, the reference's CPU path restated)",
            "c_openmp_port": {"value": round(c_value, 1), "cores": c_cores}, "host_cpus": os.cpu_count()}


def gpu_baseline(device):
    """The reference project's own CUDA kernels on this GPU (a baseline, like cpu_baseline): its unmodified
    recurrent and rl_infctx chunk-forward sources built for sm_100 (oracle/build_ref.py), called through the
    reference's native symbols.  Decode: 256 x H32, ticket prepared once, rotating state pools.  Prefill: the dense
    8 x 4096 workload through the recurrent operator (what the reference's inference path runs for T > 1) and
    through the rl_infctx chunk operator (chunk 64; clones and workspaces included, as its API does).  The
    reference has only the logits decay mode; kernel time does not depend on the values.  A missing build is
    reported here, in the bench line, not skipped silently."""
    import torch

    from flashrwkv2_b200.workloads import make_workload
    from oracle.build_ref import load_ref

    ref = load_ref()
    if ref is None:
        return {"unavailable": "oracle/_ref/_C_ref.so not built (needs a reference checkout at build time)"}
    out = {"kind": "reference kernels, unmodified sources compiled for sm_100"}
    names = ("r", "w", "k", "v", "a", "b")
    wl = make_workload("c1", device=device)
    t = wl.tensors
    pools = [t["state_pool"]] + [t["state_pool"].clone() for _ in range(7)]
    ticket = ref.prepare_tmix_wkv7_recurrent_metadata(t["cu_seqlens"], t["state_indices"], wl.total_tokens,
                                                      t["state_pool"].shape[0], 1)
    y = torch.empty_like(t["v"])

    def decode_step(i):
        ref.tmix_wkv7_recurrent_fp32_from_decay_logits(t["cu_seqlens"], t["state_indices"], pools[i % 8],
                                                       *(t[n] for n in names), y, 1.0, None, ticket, 1)

    for i in range(5):
        decode_step(i)
    steps = 200
    ms = _event_time_ms(decode_step, steps) / steps
    out["decode"] = {"workload": "c1", "kernel": "wkv_fp32_v2_small_warp_kernel",
                     "tokens_per_s": round(wl.total_tokens / (ms * 1e-3), 1), "us_per_step": round(ms * 1e3, 2)}
    del pools
    wl = make_workload("c2", device=device)
    t = wl.tensors
    y = torch.empty_like(t["v"])
    ticket = ref.prepare_tmix_wkv7_recurrent_metadata(t["cu_seqlens"], t["state_indices"], wl.total_tokens,
                                                      t["state_pool"].shape[0], 4096)

    def recurrent_step(i):
        ref.tmix_wkv7_recurrent_fp32_from_decay_logits(t["cu_seqlens"], t["state_indices"], t["state_pool"],
                                                       *(t[n] for n in names), y, 1.0, None, ticket, 4096)

    starts = torch.arange(0, wl.total_tokens, 64, dtype=torch.int32, device=device)
    meta = (torch.arange(0, wl.n_seq + 1, dtype=torch.int32, device=device) * (4096 // 64), starts, starts + 64)

    def chunk_step(strategy):
        def step(i):
            ref.rl_infctx_tmix_wkv7_chunk_fp32io16_forward(*meta, t["state_pool"], *(t[n] for n in names), strategy,
                                                           1.0, None)
        return step

    if hasattr(ref, "tmix_wkv7_recurrent_fp16_from_decay_logits"):
        # the reference's fp16-state decode family on the c1 shapes (fp16 tokens, decay logits)
        wl16 = make_workload("c1", device=device)
        t16 = wl16.tensors
        tok = [t16[n].half() for n in names]
        pool16 = t16["state_pool"].half()
        elapsed = torch.zeros(pool16.shape[0], dtype=torch.int32, device=device)
        y16 = torch.empty_like(tok[3])
        tk = ref.prepare_tmix_wkv7_recurrent_metadata(t16["cu_seqlens"], t16["state_indices"], wl16.total_tokens,
                                                      pool16.shape[0], 1)

        def f16_step(i):
            ref.tmix_wkv7_recurrent_fp16_from_decay_logits(t16["cu_seqlens"], t16["state_indices"], elapsed, pool16,
                                                           *tok, y16, 1.0, None, tk, 1)

        for i in range(5):
            f16_step(i)
        ms = _event_time_ms(f16_step, 200) / 200
        out["decode_fp16_state"] = {"workload": "c1 shapes, fp16 state", "tokens_per_s": round(wl16.total_tokens / (ms * 1e-3), 1),
                                    "us_per_step": round(ms * 1e3, 2)}
        del wl16, t16, tok, pool16
    if hasattr(ref, "tmix_lnx_rkvres_xg_forward_varlen"):
        # the reference's elementwise readout kernel (consumer of y) on the c4_decode shapes: 2048 tokens x 64 heads.
        # Timing only: its fp16 tensors are filled with small random values, kernel time does not depend on them.
        rows, channels = 2048, 64 * 64
        packed = [torch.randn(rows, channels, device=device).half() for _ in range(5)]
        vectors = [torch.randn(channels, device=device).half() for _ in range(3)]
        result = torch.empty(rows, channels, dtype=torch.float16, device=device)

        def readout_step(i):
            ref.tmix_lnx_rkvres_xg_forward_varlen(rows, 1, rows, channels, 64, 64, *packed[:4], *vectors, packed[4],
                                                  result)

        for i in range(5):
            readout_step(i)
        ms = _event_time_ms(readout_step, 200) / 200
        out["readout_elementwise"] = {"workload": "c4_decode shapes (2048 x 64 heads), fp16; inputs may sit in L2",
                                      "us_per_step": round(ms * 1e3, 2)}
        del packed, result
    out["prefill"] = {"workload": "c2"}
    for label, fn in (("recurrent (wkv_fp32_v2_kernel)", recurrent_step),
                      ("rl_infctx chunk 64, recompute", chunk_step(1)),
                      ("rl_infctx chunk 64, materialized", chunk_step(0))):
        for i in range(2):
            fn(i)
        ms = _event_time_ms(fn, 5) / 5
        out["prefill"][label] = {"tokens_per_s": round(wl.total_tokens / (ms * 1e-3), 1), "ms_per_step": round(ms, 4)}
    return out


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path on the host cores (rank 0 only)."""
    import torch

    from flashrwkv2_b200.workloads import make_workload

    if rank != 0:
        return None
    # torchrun pins OMP_NUM_THREADS=1; the CPU path gets every host thread it can use
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    name = "c4_decode" if args.workload == "c4" else args.workload
    if name in DECODE_WORKLOADS:
        wl = make_workload(name)
    else:  # a prefix of every sequence is what a step times: generate no more than that
        wl = make_workload(name, n_seq=8 if name != "c3" else None, seq_len=256)
    per_step_limit = max(1.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    sample, values, steps_ms = "", [], []
    for i in range(args.warmup + args.steps):
        begin = time.perf_counter()
        value, cores, sample = _cpu_sample(name, wl, limit_s=per_step_limit, use_c=False)
        if i >= args.warmup:
            values.append(value)
            steps_ms.append((time.perf_counter() - begin) * 1e3)
    value = statistics.mean(values)
    return {
        "impl": "reference", "metric": METRIC,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(statistics.mean(steps_ms), 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.workload, world),
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "each step: " + sample},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": ("the reference ships no sm_100 kernel and its import rejects capability 10.x; its CPU "
                 "implementation of this path is the fp32 PyTorch token loop of its test-suite, restated in "
                 "oracle/wkv7_oracle.py; the GPUs are hidden from this process"),
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--workload", default="c4", choices=("c4", "c1", "c2", "c3", "c4_decode", "c4_prefill"))
    parser.add_argument("--no-extras", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--extra", default=None, choices=("fp16_state", "fused_gate", "readout", "pretrain", "gpu_baseline"),
                        help="one GPU: measure only this block of the default run's extras and print it")
    parser.add_argument("--min-region-s", type=float, default=MIN_REGION_S,
                        help="shortest timed region (default 0.5 s); 0 for a profiler capture of a few launches")
    args = parser.parse_args()
    globals()["MIN_REGION_S"] = max(0.0, args.min_region_s)
    if args.impl == "reference":
        # the reference arm is CPU code: hide the GPUs before torch (and the package) are imported, so that
        # none of the product's shared libraries is loaded into this process
        os.environ["CUDA_VISIBLE_DEVICES"] = ""
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
    else:
        args.steps = 20 if args.steps is None else args.steps
        args.warmup = 5 if args.warmup is None else max(3, args.warmup)

    import torch

    from flashrwkv2_b200 import dist as fdist

    if args.impl == "reference":
        rank, _, world = fdist.world_from_env()
        line = run_reference(args, rank, max(world, args.gpus))
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the WKV7 operator has no CPU fallback")
    rank, local_rank, world = fdist.init()
    if world == 1 and args.gpus > 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nnodes=1 "
                         f"--nproc-per-node {args.gpus} --master-addr 127.0.0.1 bench.py --gpus {args.gpus}")
    if args.extra is not None:
        if world != 1:
            raise SystemExit("--extra runs on one GPU")
        torch.cuda.set_device(local_rank)
        block = {"fp16_state": lambda: measure_fp16_state_decode(args, local_rank),
                 "fused_gate": lambda: measure_fused_gate(args, local_rank),
                 "readout": lambda: measure_readout(args, local_rank),
                 "pretrain": lambda: measure_pretrain(args, local_rank),
                 "gpu_baseline": lambda: gpu_baseline(torch.device("cuda", local_rank))}[args.extra]()
        print(json.dumps({"extra": args.extra, **block}), flush=True)
        fdist.shutdown()
        return
    line = run_ours(args, rank, local_rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    fdist.shutdown()


if __name__ == "__main__":
    main()
