"""WKV7 benchmark: tokens/s and fraction of roofline on B200, next to the CPU recurrence.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c1|c2|c3|c4_decode|c4_prefill] [--no-extras]

A step is one pass of the hot path over one batch.  The headline workload is the decode
step (N=256 sequences per GPU, T=1, H=32, D=64, bf16 tokens, fp32 state updated in place).
With N GPUs every rank runs the same amount of work on its own sequences (weak scaling, no
collective on the data path); the time is the maximum over ranks, measured with CUDA events.

Keys of the JSON line:
  value      tokens/s with inputs resident in HBM, through the C ABI;
  e2e        tokens/s through the public Python operator with the six token tensors copied
             from pinned host memory and y copied back to the host inside the timed region
             (the state pool is device-resident by contract);
  roofline   the decode kernel's algorithmic bytes per launch / its average duration, against
             the measured HBM copy bandwidth;
  cpu_baseline  the port of the reference's fp32 PyTorch recurrence on the host cores;
  gpu_baseline  (extra) the reference's own CUDA kernels, built unmodified for sm_100, on this GPU;
  prefill    (extra) the same figures for the dense prefill workload (8 x 4096 tokens, H=32).

``--impl reference`` times the reference's CPU implementation of the path (its fp32 PyTorch
token loop, restated in oracle/wkv7_oracle.py: its package refuses to import on capability
10.x and its CPU path is that loop) on the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ALGO_BYTES_DECODE_PAIR = 16384 + 16384 + 6 * 128 + 128  # state in + out, six bf16 rows, one bf16 y row
ALGO_FLOP_PREFILL_TOKEN_HEAD = 98304  # 12 GEMMs of 64^3 per 64-row chunk
ALGO_BYTES_PREFILL_TOKEN_HEAD = 7 * 128
ALGO_BYTES_PREFILL_PAIR = 32768
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode kernel at the headline
# workload (N=256, H=32), from the ncu capture summarised in profiles/decode_c1_wkv7_recurrent_stream_kernel.md.
# It is below the algorithmic bytes because part of the written state is still dirty in L2 when the kernel ends.
DECODE_TRAFFIC_BYTES = 140538368 + 77164544


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


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
        # "under load": the samples in the upper half of the power readings
        cut = statistics.median(power)
        loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def _event_time_ms(fn, steps, finish=None):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        fn(i)
    if finish is not None:
        finish()
    end.record()
    end.synchronize()
    return start.elapsed_time(end)


def _decode_sets(wl_name, n_sets, rank, world, device, n_seq=None, heads=None):
    """Rotating input/state sets whose total footprint exceeds L2 several times over."""
    from flashrwkv2_b200.workloads import make_workload

    sets = []
    for i in range(n_sets):
        wl = make_workload(wl_name, device=device, n_seq=n_seq, heads=heads)
        if i:  # distinct data per set without re-seeding cost: perturb cheaply
            for name in "rkv":
                wl.tensors[name] = wl.tensors[name].roll(i, 0)
        sets.append(wl)
    return sets


def run_ours(args, rank, local_rank, world):
    from flashrwkv2_b200 import _lib, dist as fdist
    from flashrwkv2_b200.tmix import wkv7 as ops
    from flashrwkv2_b200.workloads import describe, make_workload

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()
    name = args.workload
    is_decode = name in ("c1", "c4_decode")
    sampler = ClockSampler(local_rank)

    per_rank_n = None
    if name == "c4_decode":
        per_rank_n = 2048 // world if args.scaling == "strong" else 2048
    wl0 = make_workload(name, with_tensors=False, n_seq=per_rank_n)
    heads = wl0.heads
    stream = torch.cuda.current_stream().cuda_stream

    if is_decode:
        n_seq = wl0.n_seq
        state_bytes = n_seq * heads * 16384
        n_sets = max(2, min(8, int(2 * 2**30 // state_bytes)))  # >= 1 GiB of state in rotation when it fits
        if state_bytes * n_sets < 3 * 126e6:
            n_sets = int(3 * 126e6 // state_bytes) + 1
        sets = _decode_sets(name, n_sets, rank, world, device, n_seq=per_rank_n)
        ys = [torch.empty_like(s.tensors["v"]) for s in sets]
        tokens_per_step = wl0.total_tokens

        def step(i):
            t = sets[i % n_sets].tensors
            rc = lib.frwkv_sm100_wkv7_recurrent(
                t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
                t["b"].data_ptr(), 0, ys[i % n_sets].data_ptr(), 0, n_seq, tokens_per_step, heads, _lib.IO_BF16,
                _lib.DECAY_RETENTION, 1.0, 1, stream)
            if rc:
                raise RuntimeError(_lib.last_error())

        algo_bytes = n_seq * heads * ALGO_BYTES_DECODE_PAIR
        l2_note = f"rotating {n_sets} state pools ({state_bytes * n_sets / 2**20:.0f} MiB) > L2"
    else:
        sets = [make_workload(name, device=device, rank=rank if args.scaling == "strong" else 0,
                              world=world if args.scaling == "strong" else 1)]
        t = sets[0].tensors
        wl0 = sets[0]
        tokens_per_step = wl0.total_tokens
        n_seq = wl0.n_seq
        y = torch.empty_like(t["v"])
        pristine = t["state_pool"].clone()
        need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n_seq, tokens_per_step, heads)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        err = torch.zeros(1, dtype=torch.int32, device=device)
        max_len = max(wl0.lengths)

        def step(i):
            rc = lib.frwkv_sm100_wkv7_prefill(
                t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
                t["b"].data_ptr(), 0, y.data_ptr(), 0, n_seq, tokens_per_step, heads, _lib.IO_BF16,
                _lib.DECAY_RETENTION, 1.0, max_len, _lib.PREFILL_AUTO, ws.data_ptr(), need, err.data_ptr(), stream)
            if rc:
                raise RuntimeError(_lib.last_error())

        algo_bytes = tokens_per_step * heads * ALGO_BYTES_PREFILL_TOKEN_HEAD + n_seq * heads * ALGO_BYTES_PREFILL_PAIR
        l2_note = f"inputs {tokens_per_step * heads * 896 / 2**20:.0f} MiB per step > L2"

    # ---- device-resident timing -------------------------------------------------------
    sampler.start()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    fdist.barrier()
    elapsed_ms = _event_time_ms(step, args.steps)
    fdist.barrier()
    elapsed_ms = fdist.reduce_max(elapsed_ms)
    total_tokens = fdist.reduce_sum(tokens_per_step)
    ms_per_step = elapsed_ms / args.steps
    value = total_tokens / (ms_per_step * 1e-3)
    # decode: one kernel per step; prefill (auto): length ranking (2..2048 sequences), recurrence for short rows, chunk kernel
    launches = args.steps * (1 if is_decode else (3 if 1 < n_seq <= 2048 else 2))

    # ---- end to end through the public operator, host buffers ---------------------------
    src = sets[0].tensors
    h2d = sum(src[n].numel() * src[n].element_size() for n in "rwkvab")
    d2h = src["v"].numel() * src["v"].element_size()
    e2e = None
    if args.no_e2e or h2d > 8 * 2**30:  # bound pinned host memory on shared boxes
        clocks = sampler.stop()
    else:
        # the caller's six token tensors live in one pinned host block -> one host->device copy per step.
        # Two streams, as a serving loop would run it: step i+1's upload overlaps step i's kernel and the
        # download of its y (PCIe is full duplex); every step still uploads its inputs and downloads its result.
        host = torch.stack([src[n].cpu() for n in "rwkvab"]).pin_memory()
        dev_in = [torch.empty_like(host, device=device) for _ in range(2)]
        y_host = [torch.empty(src["v"].shape, dtype=src["v"].dtype).pin_memory() for _ in range(2)]
        pool = src["state_pool"]
        cu, slots = src["cu_seqlens"], src["state_indices"]
        ticket = ops.prepare_tmix_wkv7_recurrent_metadata(cu, slots, total_tokens=tokens_per_step,
                                                          state_pool_size=pool.shape[0])
        op = (ops.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen if is_decode
              else ops.infer_tmix_wkv7_prefill_fp32io16_forward_varlen)
        main_stream = torch.cuda.current_stream()
        up_stream = torch.cuda.Stream()
        uploaded = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        for ev in consumed:
            ev.record(main_stream)

        def e2e_step(i):
            j = i % 2
            up_stream.wait_event(consumed[j])  # the kernel that last read this input buffer has finished
            with torch.cuda.stream(up_stream):
                dev_in[j].copy_(host, non_blocking=True)
                uploaded[j].record(up_stream)
            main_stream.wait_event(uploaded[j])
            d = dev_in[j]
            out = op(d[0], d[1], d[2], d[3], d[4], d[5], state_pool=pool, cu_seqlens=cu, state_indices=slots,
                     validated_metadata=ticket, decay_mode="retention")
            consumed[j].record(main_stream)
            y_host[j].copy_(out, non_blocking=True)

        def e2e_finish():
            main_stream.wait_stream(up_stream)

        e2e_steps = max(3, min(args.steps, 2000 if is_decode else 20))
        for i in range(min(args.warmup, 10)):
            e2e_step(i)
        torch.cuda.synchronize()
        fdist.barrier()
        e2e_ms = _event_time_ms(e2e_step, e2e_steps, e2e_finish)
        fdist.barrier()
        e2e_ms = fdist.reduce_max(e2e_ms)
        clocks = sampler.stop()
        e2e = {"value": round(total_tokens / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps}

    achieved = algo_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": DECODE_TRAFFIC_BYTES if name == "c1" else None,
                "peak_kind": f"of {peak_kind}", "algorithmic_bytes_per_launch": algo_bytes,
                "kernel": "wkv7_recurrent_stream_kernel" if is_decode else "wkv7 prefill"}
    if not is_decode:
        flops = tokens_per_step * heads * ALGO_FLOP_PREFILL_TOKEN_HEAD
        roofline["tensor_tflops"] = round(flops / (ms_per_step * 1e-3) / 1e12, 2)
        roofline["tensor_frac_of_bf16_peak"] = round(roofline["tensor_tflops"] / peaks["bf16_tflops"], 4)

    line = {
        "metric": "WKV7 tokens/s & % roofline (decode HBM, prefill TC) at 1/2/4/8 B200",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 6), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(name) + (f"; {n_seq} sequences per GPU" if world > 1 else ""),
                   "tokens_per_step_per_gpu": tokens_per_step, "l2": l2_note, "decay_mode": "retention",
                   "io_dtype": "bf16", "state_dtype": "fp32"},
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": launches,
        "roofline": roofline,
    }

    if rank == 0 and world == 1 and not args.no_extras:
        line["cpu_baseline"] = cpu_baseline(name, sets[0])
        if is_decode:
            try:
                line["prefill"] = prefill_extra(lib, _lib, device, peaks, stream)
            except RuntimeError as error:  # reported, not hidden
                line["prefill"] = {"error": str(error)}
            try:
                line["gpu_baseline"] = gpu_baseline(device, sets)
            except Exception as error:  # a baseline that cannot load or run must not take the bench line with it
                line["gpu_baseline"] = {"error": f"{type(error).__name__}: {error}"}
    return line


def prefill_extra(lib, _lib, device, peaks, stream):
    """Dense prefill (8 x 4096 tokens, H=32) timed in the same run: tokens/s, HBM and tensor fractions."""
    from flashrwkv2_b200.workloads import make_workload

    wl = make_workload("c2", device=device)
    t = wl.tensors
    n_seq, heads, total = wl.n_seq, wl.heads, wl.total_tokens
    y = torch.empty_like(t["v"])
    need = lib.frwkv_sm100_wkv7_prefill_workspace_bytes(n_seq, total, heads)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
    err = torch.zeros(1, dtype=torch.int32, device=device)
    out = {}
    for label, strategy in (("auto", _lib.PREFILL_AUTO), ("recurrent", _lib.PREFILL_RECURRENT)):
        def step(i):
            rc = lib.frwkv_sm100_wkv7_prefill(
                t["cu_seqlens"].data_ptr(), t["state_indices"].data_ptr(), 0, t["state_pool"].data_ptr(),
                t["r"].data_ptr(), t["w"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["a"].data_ptr(),
                t["b"].data_ptr(), 0, y.data_ptr(), 0, n_seq, total, heads, _lib.IO_BF16, _lib.DECAY_RETENTION,
                1.0, 4096, strategy, ws.data_ptr(), need, err.data_ptr(), stream)
            if rc:
                raise RuntimeError(_lib.last_error())
        try:
            for i in range(3):
                step(i)
            ms = _event_time_ms(step, 10) / 10
        except RuntimeError as error:
            out[label] = {"error": str(error)}
            continue
        algo = total * heads * ALGO_BYTES_PREFILL_TOKEN_HEAD + n_seq * heads * ALGO_BYTES_PREFILL_PAIR
        flops = total * heads * ALGO_FLOP_PREFILL_TOKEN_HEAD
        out[label] = {"tokens_per_s": round(total / (ms * 1e-3), 1), "ms_per_step": round(ms, 4),
                      "hbm_frac": round(algo / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                      "tensor_frac_of_bf16_peak": round(flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4),
                      "error_flag": int(err.item())}
    out["workload"] = "c2: prefill N=8 T=4096 H=32 D=64 bf16"
    return out


def _cpu_sample(name, wl, limit_s=10.0, use_c=False):
    """Time the CPU recurrence on a bounded sample of the workload; returns (tokens/s, cores, text)."""
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


def gpu_baseline(device, decode_sets):
    """The reference project's own CUDA kernels on this GPU (a baseline, like cpu_baseline): its unmodified
    recurrent and rl_infctx chunk-forward sources built for sm_100 into oracle/_ref (oracle/build_ref.py), called
    through the reference's native symbols.  Decode: the headline workload, ticket prepared once, rotating sets.
    Prefill: the dense 8 x 4096 workload through the recurrent operator (what the reference's inference path runs
    for T > 1) and through the rl_infctx chunk operator (chunk 64; clones and workspaces included, as its API does).
    The reference has only the logits decay mode; kernel time does not depend on the values."""
    from flashrwkv2_b200.workloads import make_workload
    from oracle.build_ref import load_ref

    ref = load_ref()
    if ref is None:
        return {"unavailable": "oracle/_ref/_C_ref.so not built (needs a reference checkout at build time)"}
    out = {"kind": "reference kernels, unmodified sources compiled for sm_100"}
    names = ("r", "w", "k", "v", "a", "b")
    # decode
    tickets, ys = [], []
    for wl in decode_sets:
        t = wl.tensors
        tickets.append(ref.prepare_tmix_wkv7_recurrent_metadata(t["cu_seqlens"], t["state_indices"], wl.total_tokens,
                                                                 t["state_pool"].shape[0], 1))
        ys.append(torch.empty_like(t["v"]))

    def decode_step(i):
        j = i % len(decode_sets)
        t = decode_sets[j].tensors
        ref.tmix_wkv7_recurrent_fp32_from_decay_logits(t["cu_seqlens"], t["state_indices"], t["state_pool"],
                                                       *(t[n] for n in names), ys[j], 1.0, None, tickets[j], 1)

    for i in range(5):
        decode_step(i)
    steps = 200
    ms = _event_time_ms(decode_step, steps) / steps
    tokens = decode_sets[0].total_tokens
    out["decode"] = {"kernel": "wkv_fp32_v2_small_warp_kernel", "tokens_per_s": round(tokens / (ms * 1e-3), 1),
                     "us_per_step": round(ms * 1e3, 2)}
    # prefill
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

    out["prefill"] = {"workload": "c2: prefill N=8 T=4096 H=32 D=64 bf16"}
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
    from flashrwkv2_b200.workloads import describe, make_workload

    if rank != 0:
        return None
    # torchrun pins OMP_NUM_THREADS=1; the CPU path gets every host thread it can use
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    name = args.workload
    per_rank_n = 2048 if name == "c4_decode" else None
    wl = make_workload(name, n_seq=per_rank_n) if name in ("c1", "c4_decode") else make_workload(
        name, n_seq=8 if name != "c3" else None, seq_len=256)
    steps_ms = []
    per_step_limit = max(1.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    sample = ""
    values = []
    for i in range(args.warmup + args.steps):
        begin = time.perf_counter()
        value, cores, sample = _cpu_sample(name, wl, limit_s=per_step_limit, use_c=False)
        if i >= args.warmup:
            values.append(value)
            steps_ms.append((time.perf_counter() - begin) * 1e3)
    value = statistics.mean(values)
    return {
        "impl": "reference",
        "metric": "WKV7 tokens/s & % roofline (decode HBM, prefill TC) at 1/2/4/8 B200",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(statistics.mean(steps_ms), 3), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(name), "decay_mode": "retention", "io_dtype": "bf16", "state_dtype": "fp32"},
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "each step: " + sample},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": ("the reference ships no sm_100 kernel and its import rejects capability 10.x; its CPU "
                 "implementation of this path is the fp32 PyTorch token loop of its test-suite, restated in "
                 "oracle/wkv7_oracle.py"),
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--workload", default="c1", choices=("c1", "c2", "c3", "c4_decode", "c4_prefill"))
    parser.add_argument("--scaling", default="weak", choices=("weak", "strong"))
    parser.add_argument("--no-extras", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    args = parser.parse_args()
    decode = args.workload in ("c1", "c4_decode")
    if args.impl == "reference":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
    else:
        args.steps = (20000 if decode else 20) if args.steps is None else args.steps
        args.warmup = (200 if decode else 3) if args.warmup is None else max(3, args.warmup)

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
    line = run_ours(args, rank, local_rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    fdist.shutdown()


if __name__ == "__main__":
    main()
