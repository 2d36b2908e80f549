"""Ahead-of-time build of the native libraries.

Two shared objects are produced inside the package directory (they are git-ignored but travel
with a source snapshot to a GPU machine):

* ``_lib/libogb_cuda.so``    -- every ``csrc/kernels/*.cu`` compiled by ``nvcc`` for sm_100a only
                               (``-gencode arch=compute_100a,code=sm_100a``).  Plain C ABI; no
                               PyTorch headers, so a full rebuild takes seconds.
* ``_lib/libogb_runtime.so`` -- ``csrc/runtime/*.cpp`` + ``csrc/cpu_ref/*.cpp`` + ``csrc/capi/*.cpp``
                               compiled by ``g++``: paged-KV manager, scheduler, ONNX reader, CPU
                               reference kernels and the ``oge_*`` C API.

The reference compiles its CUDA-C strings with NVRTC at first use
(crates/onnx-runtime-ep-cuda/src/runtime.rs:132-138,1112); here everything is compiled before
the process starts and nothing is specialised at run time.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = Path(__file__).resolve().parent
LIB_DIR = PKG / "_lib"
OBJ_DIR = ROOT / "build" / "obj"
CUDA_LIB = LIB_DIR / "libogb_cuda.so"
RUNTIME_LIB = LIB_DIR / "libogb_runtime.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]
# --use_fast_math only affects intrinsics-free float math in glue kernels; numerically sensitive
# paths call exp2f/__expf explicitly.
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-fopenmp", "-mavx2", "-mfma"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set NVCC or add /usr/local/cuda/bin to PATH")


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def cuda_sources() -> list[Path]:
    return sorted((ROOT / "csrc" / "kernels").glob("*.cu"))


def runtime_sources() -> list[Path]:
    out: list[Path] = []
    for sub in ("runtime", "cpu_ref"):
        out += sorted((ROOT / "csrc" / sub).glob("*.cpp"))
    return out


def _stamp_ok(lib: Path, digest: str) -> bool:
    stamp = lib.with_suffix(".stamp")
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == digest


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    srcs = cuda_sources()
    hdrs = sorted((ROOT / "csrc" / "kernels").glob("*.h")) + sorted((ROOT / "csrc" / "kernels").glob("*.cuh"))
    digest = _digest(srcs + hdrs, " ".join(NVCC_FLAGS))
    if not force and _stamp_ok(CUDA_LIB, digest):
        return CUDA_LIB
    nvcc = _nvcc()
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    logs: dict[str, str] = {}

    def one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        logs[src.name] = _run([nvcc, *NVCC_FLAGS, "-I", str(src.parent), "-c", str(src), "-o", str(obj)])
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(one, srcs))
    _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    (ROOT / "build" / "ptxas.log").write_text("\n".join(f"== {k}\n{v}" for k, v in sorted(logs.items())))
    CUDA_LIB.with_suffix(".stamp").write_text(digest)
    if verbose:
        print(f"built {CUDA_LIB}")
    return CUDA_LIB


def cuda_include_dir() -> str:
    """The CUDA toolkit's include directory (CUDA_HOME, else beside nvcc, else the usual place), or '' when there is none."""
    cands = [os.environ.get("CUDA_HOME", ""), os.environ.get("CUDA_PATH", "")]
    nvcc = shutil.which("nvcc")
    if nvcc:
        cands.append(str(Path(nvcc).resolve().parent.parent))
    cands.append("/usr/local/cuda")
    for c in cands:
        if c and (Path(c) / "include" / "cupti.h").exists():
            return str(Path(c) / "include")
    return ""


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    srcs = runtime_sources()
    hdrs: list[Path] = []
    for sub in ("runtime", "cpu_ref", "capi", "abi"):
        hdrs += sorted((ROOT / "csrc" / sub).glob("*.h")) + sorted((ROOT / "csrc" / sub).glob("*.hpp"))
    digest = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    if not force and _stamp_ok(RUNTIME_LIB, digest):
        return RUNTIME_LIB
    if not srcs:
        return RUNTIME_LIB
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("OGB_CXX") or shutil.which("g++") or "g++"
    inc = ["-I", str(ROOT / "csrc"), "-I", str(ROOT / "csrc" / "capi")]
    cuda_inc = cuda_include_dir()            # the GPU activity collector reads record layouts from cupti.h when it is there
    if cuda_inc:
        inc += ["-I", cuda_inc]

    def one(src: Path) -> Path:
        obj = OBJ_DIR / (src.parent.name + "_" + src.stem + ".o")
        _run([cxx, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(one, srcs))
    _run([cxx, "-shared", "-fopenmp", "-o", str(RUNTIME_LIB), *map(str, objs), "-ldl", "-lpthread"])
    RUNTIME_LIB.with_suffix(".stamp").write_text(digest)
    if verbose:
        print(f"built {RUNTIME_LIB}")
    return RUNTIME_LIB


CAPI_LIB = LIB_DIR / "libonnx_genai_b200.so"


def build_capi(force: bool = False, verbose: bool = False) -> Path:
    """The C interface (csrc/capi): a CPython embedding, so it links the interpreter's shared library."""
    import sysconfig

    src = ROOT / "csrc" / "capi" / "capi.cpp"
    hdr = ROOT / "csrc" / "capi" / "onnx_genai_b200.h"
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ldver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    flags = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-I", sysconfig.get_paths()["include"],
             f'-DOGB_DEFAULT_PYTHON="{sys.executable}"', f'-DOGB_DEFAULT_ROOT="{ROOT}"']
    digest = _digest([src, hdr], " ".join(flags) + libdir + ldver)
    if not force and _stamp_ok(CAPI_LIB, digest):
        return CAPI_LIB
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("OGB_CXX") or shutil.which("g++") or "g++"
    _run([cxx, *flags, "-shared", str(src), "-o", str(CAPI_LIB), f"-L{libdir}", f"-lpython{ldver}", f"-Wl,-rpath,{libdir}",
          "-ldl", "-lpthread"])
    CAPI_LIB.with_suffix(".stamp").write_text(digest)
    if verbose:
        print(f"built {CAPI_LIB}")
    return CAPI_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_runtime(force, verbose)
    build_capi(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
