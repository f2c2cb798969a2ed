"""In-tree build of the native library.

Every ``.cu`` under ``csrc/`` is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``), every ``.cpp`` by g++, and the objects are linked
into ``fluidmoe_b200/_C*.so`` next to this file.  nvcc cross-compiles, so no GPU is needed to
build.  Objects are cached under ``fluidmoe_b200/build/`` keyed by a hash of the source, the
headers and the flags.
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
CSRC = HERE / "csrc"
BUILD = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
# extra nvcc flags of developer builds, e.g. FLUIDMOE_BUILD_DEFINES=-DFM_FLASH_PROFILE
NVCC_FLAGS += os.environ.get("FLUIDMOE_BUILD_DEFINES", "").split()
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _includes() -> list[str]:
    import pybind11

    return [
        f"-I{CSRC}", f"-I{CSRC / 'include'}", f"-I{_cuda_home()}/include",
        f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
    ]


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")):
        h.update(hdr.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _compile(src: Path, verbose: bool) -> Path:
    is_cu = src.suffix == ".cu"
    flags = NVCC_FLAGS if is_cu else CXX_FLAGS
    obj = BUILD / f"{src.stem}.{_digest(src, flags)}.o"
    if obj.exists():
        return obj
    BUILD.mkdir(exist_ok=True)
    if is_cu:
        cmd = [f"{_cuda_home()}/bin/nvcc", *flags, *_includes(), "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *flags, *_includes(), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = BUILD / f"{src.stem}.log"
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(f"[build] {src.relative_to(HERE)}\n")
    return obj


def target_path() -> Path:
    return HERE / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(verbose: bool = True, force: bool = False) -> Path:
    srcs = sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))
    if force and BUILD.exists():
        for f in BUILD.glob("*.o"):
            f.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    # objects of earlier source versions are of no further use: keep the cache to one object per source
    current = {o.name for o in objs}
    for f in BUILD.glob("*.o"):
        if f.name not in current:
            f.unlink()
    out = target_path()
    stamp = BUILD / "link.stamp"
    key = " ".join(str(o) for o in objs)
    if out.exists() and stamp.exists() and stamp.read_text() == key:
        return out
    cmd = [
        f"{_cuda_home()}/bin/nvcc", "-shared", "-o", str(out), *[str(o) for o in objs],
        "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl", "-lpthread", "-lrt",
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp.write_text(key)
    if verbose:
        sys.stderr.write(f"[build] linked {out.name}\n")
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv)
