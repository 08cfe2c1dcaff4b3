"""Test infrastructure, not product code.

Builds the reference project's own WKV7 CUDA sources, unmodified and where they lie in a reference
checkout, into oracle/_ref/_C_ref.so for sm_100:

    python oracle/build_ref.py <path to the FlashRWKV2 checkout> [--force]

The sources are arch-neutral CUDA C++ (no inline PTX, no arch guards), so the only changes against the
reference's own build are the target architecture and the module entry (oracle/ref_module.cpp, which
registers the reference's recurrent (fp32- and fp16-state) and rl_infctx chunk bindings and wraps the host launchers
of its kk/a-gate and elementwise readout kernels).  Nothing is copied: nvcc and g++
read the files in place, objects and the module go to oracle/_ref/ (git-ignored).  The module needs a GPU
to do anything; tests and the bench use it as a second checker and as a same-GPU timing comparison.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
MODULE = OUT / "_C_ref.so"

# reference files on the WKV7 recurrent + rl_infctx chunk-forward path (relative to the checkout)
REFERENCE_SOURCES = (
    "csrc/validation.cpp",
    "csrc/validation/recurrent_metadata.cu",
    "csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cpp",
    "csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu",
    "csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cpp",
    "csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cu",
    "csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_backward.cu",  # emit_outputs / replay used by the forward
    "csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cpp",  # the fp16-state decode family
    "csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu",
    "csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/infer_fp16_forward_varlen.cu",  # producer of a, b and the gated key
    "csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu",  # consumer of y: head norm, r.k residual, gate
    "csrc/sm120/tmix/wkv7/pretrain_recurrent_bf16_forward.cpp",  # the training operator: forward + backward
    "csrc/sm120/tmix/wkv7/pretrain_recurrent_bf16_forward.cu",
)


def build_ref(checkout: str | os.PathLike, force: bool = False) -> Path | None:
    """Returns the module path, or None when the checkout lacks the sources."""
    import torch
    from torch.utils import cpp_extension

    root = Path(checkout)
    srcs = [root / s for s in REFERENCE_SOURCES]
    if not all(s.exists() for s in srcs):
        return None
    srcs.append(HERE / "ref_module.cpp")
    h = hashlib.sha256(torch.__version__.encode())
    for s in srcs + sorted((root / "csrc").glob("*.h")) + sorted((root / "csrc/sm120/tmix/wkv7").glob("*.cuh")):
        h.update(s.read_bytes())
    digest = h.hexdigest()
    stamp = OUT / ".digest"
    if MODULE.exists() and stamp.exists() and stamp.read_text() == digest and not force:
        return MODULE
    OUT.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{d}" for d in cpp_extension.include_paths(device_type="cuda")]
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    # -D_N_ / -D_CHUNK_LEN_: the compile-time head size and checkpoint distance of the reference's training kernels
    # (its setup.py passes the same two values)
    defs = ["-DTORCH_EXTENSION_NAME=_C_ref", "-DTORCH_API_INCLUDE_EXTENSION_H", "-DFLASHRWKV_BACKEND_SM120=1",
            "-D_N_=64", "-D_CHUNK_LEN_=16",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(src: Path) -> Path:
        obj = OUT / ((src.parent.name + "_" + src.name).replace(".", "_") + ".o")
        if src.suffix == ".cu":
            cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100", "-lineinfo",
                   "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
                   "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                   "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", *defs, *inc, "-c", str(src),
                   "-o", str(obj)]
        else:
            cmd = ["g++", "-O2", "-fPIC", "-std=c++17", "-Wno-deprecated-declarations", *defs, *inc, "-c", str(src),
                   "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode != 0:
            raise RuntimeError(f"reference source {src} did not compile:\n{res.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as pool:
        objs = list(pool.map(compile_one, srcs))
    libdirs = cpp_extension.library_paths(device_type="cuda")
    cmd = ["g++", "-shared", "-o", str(MODULE), *map(str, objs), *[f"-L{d}" for d in libdirs], "-lc10", "-lc10_cuda",
           "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError(f"link of the reference module failed:\n{res.stderr[-4000:]}")
    for obj in objs:  # only the module travels
        obj.unlink()
    stamp.write_text(digest)
    return MODULE


def load_ref():
    """Imports oracle/_ref/_C_ref.so if it was built; None otherwise.  Needs torch imported first."""
    if not MODULE.exists():
        return None
    import importlib.util

    import torch  # noqa: F401  (libtorch must be loaded before the module)

    spec = importlib.util.spec_from_file_location("_C_ref", MODULE)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    built = build_ref(sys.argv[1], force="--force" in sys.argv[2:])
    print(built if built else "reference sources not found; nothing built")
