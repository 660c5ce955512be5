"""Builds the native library in-tree: every ``csrc/*.cu`` / ``*.cpp`` is compiled
for sm_100a (``*.cc``: host-only CPU kernels, by the host compiler) and linked into
``mimir_b200/_native/libmimir_b200.so``.

The library has a plain C ABI (no Python or torch headers), so it compiles in
seconds, loads through ``ctypes`` here and through ``purego`` from Go, and the
same symbols serve both.  Run ``python -m mimir_b200._native.build``.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libmimir_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.name + ".o")
    stamp = OBJ / (src.name + ".sha")
    dig = _digest(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    if src.suffix == ".cc":
        # host-only sources (CPU kernels with per-function ISA targets) go straight to the host compiler
        cxx = shutil.which("g++") or shutil.which("c++")
        if cxx is None:
            raise RuntimeError("no C++ compiler found")
        cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if src.suffix == ".cpp":
            cmd.insert(1, "-x")
            cmd.insert(2, "cu")
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ / (src.name + ".log")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src.name} failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"[build] {src.name}\n")
    stamp.write_text(dig)
    return obj


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp")) + sorted(CSRC.glob("*.cc"))


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compiles what changed and links the shared library; returns its path."""
    OBJ.mkdir(exist_ok=True)
    if force:
        for f in OBJ.glob("*.sha"):
            f.unlink()
    srcs = sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if LIB.exists() and LIB.stat().st_mtime >= newest and not force:
        return LIB
    tmp = LIB.with_suffix(".so.tmp")
    cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-lpthread", "-ldl", "-lmvec", "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB)
    if verbose:
        sys.stderr.write(f"[build] linked {LIB}\n")
    return LIB


CAPI_LIB = HERE / "libmimir_capi.so"


def build_capi(verbose: bool = False) -> Path:
    """Builds ``libmimir_capi.so``: the C ABI over framework objects (``csrc/capi/mimir_capi.c``), a
    plain C file that embeds the interpreter, linked against the shared libpython of this Python."""
    import sysconfig
    src = CSRC / "capi" / "mimir_capi.c"
    hdr = CSRC / "capi" / "mimir_capi.h"
    if CAPI_LIB.exists() and CAPI_LIB.stat().st_mtime >= max(src.stat().st_mtime, hdr.stat().st_mtime):
        return CAPI_LIB
    inc = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler found")
    tmp = CAPI_LIB.with_suffix(".so.tmp")
    cmd = [cc, "-shared", "-fPIC", "-O2", "-fvisibility=hidden", "-I", inc, "-I", str(src.parent), str(src), "-o", str(tmp),
           f"-L{libdir}", f"-lpython{ver}", f"-Wl,-rpath,{libdir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the C ABI library failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, CAPI_LIB)
    if verbose:
        sys.stderr.write(f"[build] linked {CAPI_LIB}\n")
    return CAPI_LIB


def ptxas_report() -> str:
    """Concatenates the registers / spills / shared-memory lines of the last build."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        out.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(out)


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    build_capi(verbose=True)
    if "--report" in sys.argv:
        print(ptxas_report())
