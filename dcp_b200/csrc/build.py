"""In-tree native build: CUDA kernels (sm_100a) -> dcp_b200/_kernels.so, C++ planner -> dcp_b200/_planner*.so.

Both libraries are built with plain nvcc / g++ command lines (no JIT cache), so the
resulting shared objects sit next to the Python sources and travel with the tree.
Run as ``python -m dcp_b200.csrc.build`` or through ``__graft_entry__.build()``.
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
PKG = HERE.parent
KERNEL_DIR = HERE / "kernels"
PLANNER_DIR = HERE / "planner"
OBJ_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha1()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, log_path=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        Path(log_path).write_text(" ".join(map(str, cmd)) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))
    return res.stdout


def kernels_lib_path() -> Path:
    return PKG / "_kernels.so"


def planner_lib_path() -> Path:
    return PKG / ("_planner" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sorted(KERNEL_DIR.glob("*.cu"))
    hdrs = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    out = kernels_lib_path()
    stamp = OBJ_DIR / "kernels.stamp"
    digest = _digest(srcs + hdrs)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    hdr_digest = _digest(hdrs)

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        ostamp = OBJ_DIR / (src.stem + ".stamp")
        d = hashlib.sha1((hdr_digest + hashlib.sha1(src.read_bytes()).hexdigest()).encode()).hexdigest()
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        log = _run([_nvcc(), *NVCC_FLAGS, "-I", str(KERNEL_DIR), "-c", str(src), "-o", str(obj)],
                   OBJ_DIR / (src.stem + ".ptxas.log"))
        if verbose:
            print(log)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    stamp.write_text(digest)
    return out


def build_planner(force: bool = False) -> Path:
    import pybind11

    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sorted(PLANNER_DIR.glob("*.cpp"))
    hdrs = sorted(PLANNER_DIR.glob("*.hpp"))
    out = planner_lib_path()
    if not srcs:
        return out
    stamp = OBJ_DIR / "planner.stamp"
    digest = _digest(srcs + hdrs)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + str(PLANNER_DIR)]
    _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", *inc, *map(str, srcs), "-o", str(out)])
    stamp.write_text(digest)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_planner(force)


if __name__ == "__main__":
    k, p = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", k, p)
