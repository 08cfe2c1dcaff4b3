"""ctypes front-end of oracle/wkv7_oracle.c.  TEST INFRASTRUCTURE ONLY.

Same contract as :func:`oracle.wkv7_oracle.wkv7_oracle`; used where the Python
token loop is too slow (larger parity cases, the benchmark's CPU baseline).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libwkv7_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile wkv7_oracle.c with gcc (a few seconds)."""
    src = _HERE / "wkv7_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libwkv7_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        lib = ctypes.CDLL(str(_LIB_PATH))
        fp, ip, vp = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int), ctypes.c_void_p
        for name in ("wkv7_oracle_f32", "wkv7_oracle_f64"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [vp] * 7 + [vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_double, ctypes.c_int, ctypes.c_int]
        lib.wkv7_oracle_max_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(_load().wkv7_oracle_max_threads())


def wkv7_oracle_c(r, w, k, v, a, b, *, state_pool, cu_seqlens, state_indices, scale=1.0,
                  decay_bias=None, decay_mode="logits", f64=False, n_threads=None):
    """Returns ``(y, new_pool)`` (fp32, or fp64 when ``f64``); inputs untouched."""
    lib = _load()
    toks = [t.detach().cpu().float().contiguous() for t in (r, w, k, v, a, b)]
    total, heads, dim = toks[0].shape
    real = torch.float64 if f64 else torch.float32
    pool = state_pool.detach().cpu().to(real).contiguous().clone()
    y = torch.zeros((total, heads, dim), dtype=real)
    cu = torch.as_tensor(cu_seqlens).detach().cpu().to(torch.int32).contiguous()
    sl = torch.as_tensor(state_indices).detach().cpu().to(torch.int32).contiguous()
    bias = None if decay_bias is None else decay_bias.detach().cpu().float().contiguous()
    mode = {"logits": 0, "retention": 1}[decay_mode]
    if n_threads is None:
        n_threads = min(max_threads(), os.cpu_count() or 1)
    fn = lib.wkv7_oracle_f64 if f64 else lib.wkv7_oracle_f32
    rc = fn(*(t.data_ptr() for t in toks), 0 if bias is None else bias.data_ptr(), y.data_ptr(),
            pool.data_ptr(), cu.data_ptr(), sl.data_ptr(), int(sl.numel()), heads, dim,
            float(scale), mode, int(n_threads))
    if rc != 0:
        raise RuntimeError(f"wkv7 C oracle rejected its arguments (code {rc})")
    return y, pool
