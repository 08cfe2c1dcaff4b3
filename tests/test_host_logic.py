"""CPU-only checks: backend selection, the C-ABI library's exports, wrapper argument
rejection (before any launch), workload generation and sequence sharding."""

from __future__ import annotations

import ctypes
import inspect
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_backend_selection_by_capability():
    import flashrwkv2_b200 as pkg

    assert pkg._backend_module_name((10, 0)) == "_C_sm100"
    for capability in ((9, 0), (12, 0), (8, 0), (10, 3)):  # sm_100a code does not run on later 10.x parts
        with pytest.raises(RuntimeError, match="no binary-compatible native backend"):
            pkg._backend_module_name(capability)


def test_backend_not_loaded_without_cuda(monkeypatch):
    import flashrwkv2_b200 as pkg

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert pkg._load_native_backend() is None


def test_backend_loader_reports_missing_extension(monkeypatch):
    import flashrwkv2_b200 as pkg

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda *a: (10, 0))
    monkeypatch.setattr(pkg, "_NATIVE_BACKENDS", (((10, 0), "_C_missing"),))
    with pytest.raises(RuntimeError, match="not built or cannot be loaded"):
        pkg._load_native_backend()


def test_operators_fail_loudly_without_backend(monkeypatch):
    """No CPU fallback: with no backend loaded the operator raises instead of computing."""
    import flashrwkv2_b200 as pkg
    from flashrwkv2_b200.tmix import wkv7

    monkeypatch.setattr(pkg, "_C", None)
    t = torch.zeros(2, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        wkv7.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen(
            t, t, t, t, t, t, state_pool=torch.zeros(1, 1, 64, 64), cu_seqlens=torch.tensor([0, 2], dtype=torch.int32),
            state_indices=torch.tensor([0], dtype=torch.int32))


def test_library_loads_and_exports_every_declared_symbol():
    from flashrwkv2_b200 import _lib
    from flashrwkv2_b200.build import build, build_extension

    build()
    build_extension()
    header = (ROOT / "include" / "frwkv_sm100.h").read_text()
    declared = set(re.findall(r"\b(frwkv_sm100_\w+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS)
    lib = _lib.load()
    assert isinstance(lib, ctypes.CDLL)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.frwkv_sm100_abi_version() == _lib.ABI_VERSION
    # argument rejection needs no GPU: null pointers are refused before any launch
    rc = lib.frwkv_sm100_wkv7_recurrent(*([0] * 13), 1, 1, 1, 0, 0, 1.0, 1, 0)
    assert rc != 0 and "non-null" in _lib.last_error()
    rc = lib.frwkv_sm100_wkv7_prefill(*([0] * 13), 1, 1, 1, 0, 0, 1.0, 1, 0, 0, 0, 0, 0)
    assert rc != 0
    assert lib.frwkv_sm100_wkv7_prefill_workspace_bytes(1, 64, 1) >= 0


def test_native_module_exports_reference_symbols():
    from flashrwkv2_b200 import _C_sm100 as ext

    for name in ("prepare_tmix_wkv7_recurrent_metadata", "prepare_tmix_wkv7_recurrent_graph_metadata",
                 "tmix_wkv7_recurrent_fp32_from_decay_logits", "rl_infctx_tmix_wkv7_chunk_fp32io16_forward",
                 "_RecurrentMetadataTicket", "tmix_wkv7_prefill_fp32", "tmix_wkv7_recurrent_fp16_from_decay_logits"):
        assert hasattr(ext, name), name
    def arg_names(fn):  # pybind functions carry their signature in the first docstring line
        head = fn.__doc__.splitlines()[0]
        return [piece.split(":")[0].strip() for piece in head[head.index("(") + 1:head.rindex(")")].split(", ")
                if ":" in piece]

    assert arg_names(ext.tmix_wkv7_recurrent_fp32_from_decay_logits)[:14] == [
        "query_start_loc", "state_indices", "state", "r", "decay_logits", "k", "v", "a", "b", "output", "scale",
        "decay_bias", "validated_metadata", "max_seqlen"]
    assert arg_names(ext.rl_infctx_tmix_wkv7_chunk_fp32io16_forward)[:13] == [
        "sequence_chunk_offsets", "chunk_token_starts", "chunk_token_ends", "state", "r", "decay_logits", "k", "v",
        "a", "b", "strategy", "scale", "decay_bias"]
    assert arg_names(ext.tmix_wkv7_recurrent_fp16_from_decay_logits) == [
        "query_start_loc", "state_indices", "elapsed_state_pool", "state", "r", "decay_logits", "k", "v", "a", "b",
        "output", "scale", "decay_bias", "validated_metadata", "max_seqlen"]
    assert arg_names(ext.prepare_tmix_wkv7_recurrent_metadata) == [
        "query_start_loc", "state_indices", "total_tokens", "state_pool_size", "max_seqlen"]
    assert arg_names(ext.prepare_tmix_wkv7_recurrent_graph_metadata) == [
        "query_start_loc", "state_indices", "num_active_tokens", "num_active_sequences", "token_capacity",
        "sequence_capacity", "state_pool_size", "max_seqlen_capacity"]
    assert ext.__file__.endswith(".so"), "the native module must be the compiled extension"
    for method in ("_check_compatible", "_query_start_loc_snapshot", "_state_indices_snapshot", "_status",
                   "_max_seqlen", "_is_graph", "_num_active_tokens", "_num_active_sequences"):
        assert hasattr(ext._RecurrentMetadataTicket, method)


def test_public_signature_matches_reference_contract():
    from flashrwkv2_b200.tmix.wkv7 import infer_tmix_wkv7_recurrent_fp32io16_forward_varlen as op

    params = inspect.signature(op).parameters
    for name in ("r", "decay_logits", "k", "v", "a", "b", "state_pool", "cu_seqlens", "state_indices", "scale",
                 "decay_bias", "max_seqlen", "validated_metadata"):
        assert name in params
    with pytest.raises(TypeError, match="log_decay"):
        op(None, None, None, None, None, None, state_pool=None, cu_seqlens=None, log_decay=None)


def test_fp16_state_signature_matches_reference_contract():
    """rwkv-rs/FlashRWKV2 tests/tmix/wkv7/test.py:883-893: raw decay logits only, no elapsed alias."""
    from flashrwkv2_b200.tmix.wkv7 import infer_tmix_wkv7_recurrent_fp16_forward_varlen as op

    params = inspect.signature(op).parameters
    for name in ("decay_logits", "state_pool", "elapsed_state_pool", "max_seqlen", "validated_metadata"):
        assert name in params
    assert "log_decay" not in params and "elapsed_t" not in params
    t = torch.zeros(2, 1, 64, dtype=torch.float16)
    with pytest.raises(TypeError, match="FP16-state state_pool"):
        op(t, t, t, t, t, t, state_pool=torch.zeros(1, 1, 64, 64), elapsed_state_pool=torch.zeros(1, dtype=torch.int32),
           cu_seqlens=torch.tensor([0, 2], dtype=torch.int32), state_indices=torch.tensor([0], dtype=torch.int32))
    with pytest.raises(TypeError, match="torch.int32"):
        op(t, t, t, t, t, t, state_pool=torch.zeros(1, 1, 64, 64, dtype=torch.float16),
           elapsed_state_pool=torch.zeros(1, dtype=torch.int64), cu_seqlens=torch.tensor([0, 2], dtype=torch.int32),
           state_indices=torch.tensor([0], dtype=torch.int32))


def test_wrapper_rejections_happen_before_any_launch():
    from flashrwkv2_b200.tmix import wkv7
    from flashrwkv2_b200.tmix.wkv7.rl_infctx import rl_infctx_tmix_wkv7_chunk_fp32io16 as chunk

    t = torch.zeros(4, 2, 64, dtype=torch.bfloat16)
    pool = torch.zeros(2, 2, 64, 64)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    slots = torch.tensor([0], dtype=torch.int32)
    op = wkv7.infer_tmix_wkv7_recurrent_fp32io16_forward_varlen
    with pytest.raises(TypeError, match="r must be a torch.Tensor"):
        op(None, t, t, t, t, t, state_pool=pool, cu_seqlens=cu, state_indices=slots)
    with pytest.raises(ValueError, match="packed shape"):
        op(t[0], t, t, t, t, t, state_pool=pool, cu_seqlens=cu, state_indices=slots)
    with pytest.raises(ValueError, match="contiguous"):
        op(t.transpose(0, 1), t, t, t, t, t, state_pool=pool, cu_seqlens=cu, state_indices=slots)
    with pytest.raises(TypeError, match="float32"):
        op(t, t, t, t, t, t, state_pool=pool.half(), cu_seqlens=cu, state_indices=slots)
    with pytest.raises(ValueError, match="one-dimensional"):
        op(t, t, t, t, t, t, state_pool=pool, cu_seqlens=cu.reshape(1, -1), state_indices=slots)
    with pytest.raises(ValueError, match="total_tokens is required"):
        wkv7.prepare_tmix_wkv7_recurrent_metadata(cu, slots, state_pool_size=2)
    with pytest.raises(ValueError, match="capacity arguments"):
        wkv7.prepare_tmix_wkv7_recurrent_metadata(cu, slots, state_pool_size=2, total_tokens=4, token_capacity=4)
    with pytest.raises(ValueError, match="all graph metadata"):
        wkv7.prepare_tmix_wkv7_recurrent_metadata(cu, slots, state_pool_size=2, token_capacity=4)
    with pytest.raises(ValueError, match="chunk_size"):
        chunk(t, t, t, t, t, t, cu_seqlens=cu, chunk_size=48)
    with pytest.raises(ValueError, match="strategy"):
        chunk(t, t, t, t, t, t, cu_seqlens=cu, strategy="fast")
    with pytest.raises(ValueError, match="finite"):
        chunk(t, t, t, t, t, t, cu_seqlens=cu, scale=float("nan"))
    with pytest.raises(ValueError, match="contiguous CUDA"):
        chunk(t, t, t, t, t, t, cu_seqlens=cu)


def test_workloads_are_seeded_and_shaped():
    from flashrwkv2_b200.workloads import describe, make_workload

    c0 = make_workload("c0")
    assert c0.tensors["r"].shape == (64, 32, 64) and c0.tensors["r"].dtype == torch.float32
    assert float(c0.tensors["state_pool"].abs().max()) == 0.0
    again = make_workload("c0")
    assert all(torch.equal(c0.tensors[n], again.tensors[n]) for n in "rwkvab")
    w = c0.tensors["w"]
    assert float(w.min()) > 0.54 and float(w.max()) < 0.9934
    kk = -c0.tensors["a"]
    assert torch.allclose(kk.norm(dim=-1), torch.ones(64, 32), atol=1e-5)
    c1 = make_workload("c1", n_seq=8, heads=2)
    assert c1.tensors["r"].dtype == torch.bfloat16 and c1.tensors["cu_seqlens"].tolist() == list(range(9))
    c3 = make_workload("c3", with_tensors=False)
    assert c3.n_seq == 64 and all(1 <= x <= 8192 for x in c3.lengths)
    assert make_workload("c3", with_tensors=False).lengths == c3.lengths
    assert "N=2048" in describe("c4_decode")


def test_lpt_sharding_properties():
    from flashrwkv2_b200.sharding import shard_packed, shard_sequences
    from flashrwkv2_b200.workloads import make_workload

    lengths = make_workload("c3", with_tensors=False).lengths
    for world in (1, 2, 4, 8):
        bins = shard_sequences(lengths, world)
        assert sorted(i for b in bins for i in b) == list(range(len(lengths)))
        loads = [sum(lengths[i] for i in b) for b in bins]
        assert max(loads) - min(loads) <= max(lengths)  # LPT bound
    assert [len(b) for b in shard_sequences([1] * 2048, 8)] == [256] * 8
    assert [len(b) for b in shard_sequences([8192] * 64, 8)] == [8] * 8
    # packed slicing: rows, re-based cu_seqlens, slots
    cu = torch.tensor([0, 3, 4, 9, 11], dtype=torch.int32)
    slots = torch.tensor([7, 5, 3, 1], dtype=torch.int32)
    toks = {"r": torch.arange(11).float().reshape(11, 1, 1).expand(11, 1, 64).contiguous()}
    parts = [shard_packed(toks, cu, slots, 2, rank) for rank in range(2)]
    assert sorted(torch.cat([p["rows"] for p in parts]).tolist()) == list(range(11))
    for p in parts:
        assert p["cu_seqlens"][0] == 0 and p["cu_seqlens"][-1] == p["r"].shape[0]
        assert p["state_indices"].tolist() == [slots[i].item() for i in p["sequences"]]
        assert torch.equal(p["r"][:, 0, 0], p["rows"].float())


def test_sharded_workload_is_a_slice_of_the_one_seeded_batch():
    """make_workload(rank, world): every rank draws the same batch and keeps its own sequences, so a run on N
    GPUs works on exactly the inputs of the single-GPU run."""
    from flashrwkv2_b200.sharding import shard_sequences
    from flashrwkv2_b200.workloads import make_workload

    full = make_workload("c3", n_seq=7, seq_len=50, heads=2)
    cu = full.tensors["cu_seqlens"].tolist()
    bins = shard_sequences(full.lengths, 3)
    for rank in range(3):
        part = make_workload("c3", n_seq=7, seq_len=50, heads=2, rank=rank, world=3)
        assert part.sequences == bins[rank] and part.lengths == [full.lengths[i] for i in bins[rank]]
        at = 0
        for j, seq in enumerate(part.sequences):
            n = cu[seq + 1] - cu[seq]
            for name in "rwkvab":
                assert torch.equal(part.tensors[name][at:at + n], full.tensors[name][cu[seq]:cu[seq + 1]])
            assert torch.equal(part.tensors["state_pool"][j], full.tensors["state_pool"][seq])
            at += n
        assert part.tensors["cu_seqlens"][-1].item() == at
    decode = [make_workload("c4_decode", n_seq=16, heads=1, rank=r, world=4) for r in range(4)]
    assert [d.n_seq for d in decode] == [4] * 4


def test_c_abi_rejects_misaligned_tensors_before_any_launch():
    """Every tensor is read or written with 16-byte vectors, decay_bias and the fp32 output copy included: a
    contiguous view at an odd offset (say flat_params[1:1+H*64]) must come back as an argument error, not reach
    the kernel.  The pointers here are made-up numbers; a rejected call dereferences and launches nothing."""
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    base = 0x7F0000000000

    def call(entry, bias=0, y32=0, y=base + 0x8000):
        ptrs = [base + 0x1000 * i for i in range(1, 11)]  # cu, slots, (status=0), pool, r, w, k, v, a, b
        head = (ptrs[0], ptrs[1], 0, ptrs[2], *ptrs[3:9], bias, y, y32, 4, 4, 2, _lib.IO_BF16, _lib.DECAY_LOGITS, 1.0, 1)
        if entry == "recurrent":
            return lib.frwkv_sm100_wkv7_recurrent(*head, 0)
        return lib.frwkv_sm100_wkv7_prefill(*head, _lib.PREFILL_AUTO, 0, 0, 0, 0)

    for entry in ("recurrent", "prefill"):
        for kw in (dict(bias=base + 0x9002), dict(y32=base + 0xA004), dict(y=base + 0x8008)):
            assert call(entry, **kw) == 1, (entry, kw)
            assert "16-byte aligned" in _lib.last_error()


def test_readout_entries_reject_bad_arguments_before_any_launch():
    """The entries with the readout stage: missing or misaligned readout tensors, a partial set of gate parameters
    and (prefill) a missing y come back as argument errors.  Made-up pointers: nothing is dereferenced or launched."""
    from flashrwkv2_b200 import _lib

    lib = _lib.load()
    base = 0x7F0000000000
    p = [base + 0x1000 * i for i in range(1, 20)]

    def call(entry, gate=(0, 0, 0), ro=None, y=0, out=None):
        ro = (p[10], p[11], p[12], p[13]) if ro is None else ro
        out = p[14] if out is None else out
        head = (p[0], p[1], 0, p[2], p[3], p[4], p[5], p[6], p[7], p[8], *gate, 0, *ro, out, y, 0, 4, 4, 2, _lib.IO_BF16,
                _lib.DECAY_LOGITS, 1.0, 1)
        if entry == "recurrent":
            return lib.frwkv_sm100_wkv7_recurrent_readout(*head, 0)
        return lib.frwkv_sm100_wkv7_prefill_readout(*head, _lib.PREFILL_AUTO, 0, 0, 0, 0)

    for entry in ("recurrent", "prefill"):
        assert call(entry, gate=(p[15], 0, p[16]), y=p[17]) == 1 and "together" in _lib.last_error()
        assert call(entry, ro=(0, p[11], p[12], p[13]), y=p[17]) == 1 and "non-null" in _lib.last_error()
        assert call(entry, ro=(p[10] + 2, p[11], p[12], p[13]), y=p[17]) == 1 and "aligned" in _lib.last_error()
        assert call(entry, out=p[14] + 8, y=p[17]) == 1 and "aligned" in _lib.last_error()
    assert call("prefill", y=0) == 1 and "y must be non-null" in _lib.last_error()


def test_native_module_exports_the_fused_operators():
    from flashrwkv2_b200 import _C_sm100 as ext

    for name in ("tmix_wkv7_fused_gate_fp32", "tmix_wkv7_readout_fp32"):
        assert hasattr(ext, name), name
    head = ext.tmix_wkv7_readout_fp32.__doc__.splitlines()[0]
    for arg in ("out_gate", "r_k", "ln_weight", "ln_bias", "wkv_output", "strategy", "error_flag"):
        assert arg + ":" in head, arg


def test_training_operator_contract_without_a_gpu():
    """Signature and native argument names of the reference's training operator
    (rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/pretrain.py:117-133, pretrain_recurrent_bf16_forward.cpp:51-62), and the
    wrapper's rejections, which come before the backend is touched."""
    import inspect

    import torch

    from flashrwkv2_b200 import _C_sm100 as ext
    from flashrwkv2_b200.tmix.wkv7.pretrain import pretrain_tmix_wkv7_recurrent_bf16 as op

    assert tuple(inspect.signature(op).parameters) == ("r", "w", "k", "v", "a", "b", "head_size")
    forward = ext.pretrain_tmix_wkv7_recurrent_forward.__doc__.splitlines()[0]
    backward = ext.pretrain_tmix_wkv7_recurrent_backward.__doc__.splitlines()[0]
    for name in ("r", "w", "k", "v", "a", "b", "output", "boundary", "state_dot_a", "head_size"):
        assert f"{name}:" in forward, name
    for name in ("grad_output", "boundary", "state_dot_a", "grad_r", "grad_w", "grad_k", "grad_v", "grad_a", "grad_b"):
        assert f"{name}:" in backward, name
    x = torch.zeros(1, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="bfloat16"):
        op(x.float(), x, x, x, x, x)
    with pytest.raises(ValueError, match="contiguous CUDA"):
        op(x, x, x, x, x, x)
    with pytest.raises(ValueError, match="head_size"):
        op(x, x, x, x, x, x, head_size=48)
    with pytest.raises(ValueError, match="shape"):
        op(x[0], x, x, x, x, x)
