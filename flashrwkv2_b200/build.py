"""Builds libfrwkv_sm100.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m flashrwkv2_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library has no torch dependency.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc" / "sm100"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libfrwkv_sm100.so"
OBJ_DIR = PKG / "build" / "obj"

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def sources() -> list[Path]:
    return sorted(CSRC.rglob("*.cu"))


BINDINGS = PKG / "csrc" / "bindings"
EXT = PKG / "_C_sm100.so"


def build_extension(force: bool = False) -> Path:
    """Compile the pybind/torch shim (_C_sm100) with g++ and link it against libfrwkv_sm100.so."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    srcs = sorted(BINDINGS.glob("*.cpp"))
    h = hashlib.sha256(torch.__version__.encode())
    for f in srcs + sorted(BINDINGS.glob("*.h")) + sorted((PKG.parent / "include").glob("*.h")):
        h.update(f.read_bytes())
    stamp = LIB_DIR / ".ext_digest"
    digest = h.hexdigest()
    if EXT.exists() and stamp.exists() and stamp.read_text() == digest and not force:
        return EXT
    inc = [f"-I{d}" for d in cpp_extension.include_paths(device_type="cuda")]
    inc += [f"-I{sysconfig.get_paths()['include']}", f"-I{PKG.parent / 'include'}"]
    flags = ["-O2", "-fPIC", "-std=c++17", "-DTORCH_EXTENSION_NAME=_C_sm100", "-DTORCH_API_INCLUDE_EXTENSION_H",
             "-DFLASHRWKV_BACKEND_SM100=1", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
             "-Wno-deprecated-declarations"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    ext_obj = PKG / "build" / "ext"
    ext_obj.mkdir(parents=True, exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = ext_obj / (src.stem + ".o")
        res = subprocess.run(["g++", *flags, *inc, "-c", str(src), "-o", str(obj)], capture_output=True, text=True,
                             env=env)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed for {src}:\n{res.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as pool:
        objs = list(pool.map(compile_one, srcs))
    libdirs = cpp_extension.library_paths(device_type="cuda")
    cmd = ["g++", "-shared", "-o", str(EXT), *map(str, objs), *[f"-L{d}" for d in libdirs], f"-L{LIB_DIR}",
           "-lfrwkv_sm100", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-lcudart", "-Wl,-rpath,$ORIGIN/lib"]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError(f"link of _C_sm100 failed:\n{res.stderr[-4000:]}")
    stamp.write_text(digest)
    return EXT


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.rglob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(src: Path, verbose: bool, extra: tuple[str, ...] = (), tag: str = "") -> Path:
    stem = src.stem + tag
    obj = OBJ_DIR / (stem + "." + _digest(src) + ".o")
    if obj.exists():
        return obj
    for stale in OBJ_DIR.glob(stem + ".*.o"):
        stale.unlink()
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    log = OBJ_DIR / (stem + ".ptxas.txt")
    log.write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr}")
    if verbose:
        print(res.stderr, file=sys.stderr)
    return obj


def _link(lib: Path, objs: list[Path], stamp: Path, force: bool) -> Path:
    wanted = "\n".join(o.name for o in objs)
    if lib.exists() and stamp.exists() and stamp.read_text() == wanted and not force:
        return lib
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC"]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr}")
    stamp.write_text(wanted)
    return lib


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.o"):
            f.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    return _link(LIB, objs, LIB_DIR / ".objects", force)


# The same sources compiled with -DFRWKV_TEST_HOOKS: a second library that only the tests load.  It adds
# frwkv_sm100_test_skip_commit() and frwkv_sm100_test_recurrent_parts(); the product library has neither.
TEST_LIB = PKG.parent / "tests" / "lib" / "libfrwkv_sm100_testhooks.so"


def build_testhooks(force: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    TEST_LIB.parent.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    # a library built from exactly these sources (it travels with the tree, the objects do not) is used as it is
    stamp = TEST_LIB.parent / ".objects"
    wanted = "\n".join(f"{s.stem}.hooks.{_digest(s)}.o" for s in srcs)
    if TEST_LIB.exists() and stamp.exists() and stamp.read_text() == wanted and not force:
        return TEST_LIB
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, False, ("-DFRWKV_TEST_HOOKS",), ".hooks"), srcs))
    return _link(TEST_LIB, objs, TEST_LIB.parent / ".objects", force)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    print(build_extension(force="--force" in sys.argv))
    print(build_testhooks(force="--force" in sys.argv))
