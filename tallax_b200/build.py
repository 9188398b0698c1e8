"""Builds the CUDA library in-tree: nvcc, sm_100a only, no other dependency.

    python -m tallax_b200.build            # recompile the sources that changed, then link
    python -m tallax_b200.build --force    # recompile everything
    python -m tallax_b200.build -v         # print ptxas resource usage (registers, spills, shared memory)
    python -m tallax_b200.build --checked  # libtallax_b200_checked.so: the streaming sampler verifies its
                                           # indices (tlx_common.cuh, TLX_IN_BOUNDS); loaded instead of the
                                           # normal library when TLX_LIBRARY=checked is set
    python -m tallax_b200.build --timeline # libtallax_b200_timeline.so: the streaming sampler's kernels
                                           # record global-timer stamps per CTA (sampler.cu, TLX_STAMP)

Every .cu file is compiled to an object of its own (in parallel) under lib/obj, so that a change to one
kernel file does not rebuild the others.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libtallax_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "tallax_b200.h"))
    return hs


def _newer(path, deps):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, checked: bool = False, timeline: bool = False) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = list(NVCC_FLAGS)
    tag = ""
    obj_dir, lib_path = OBJ_DIR, LIB_PATH
    if checked:
        flags += ["-DTLX_CHECKED=1"]
        obj_dir = os.path.join(LIB_DIR, "obj_checked")
        lib_path = os.path.join(LIB_DIR, "libtallax_b200_checked.so")
        os.makedirs(obj_dir, exist_ok=True)
    if timeline:
        flags += ["-DTLX_TIMELINE=1"] + (["-DTLX_TIMELINE_TWICE=1"] if os.environ.get("TLX_TIMELINE_TWICE") else [])
        obj_dir = os.path.join(LIB_DIR, "obj_timeline")
        lib_path = os.path.join(LIB_DIR, "libtallax_b200_timeline.so")
        os.makedirs(obj_dir, exist_ok=True)
    if verbose:
        flags += ["-Xptxas", "-v"]
    # the mode (checked or not) of the objects that are there; a change of mode rebuilds everything
    mode_file = os.path.join(obj_dir, "mode")
    old_mode = open(mode_file).read() if os.path.exists(mode_file) else None
    if old_mode != tag:
        force = True
    headers = _headers()
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or verbose or _newer(obj, [src, *headers]):
            jobs.append([nvcc, *flags, "-c", src, "-o", obj])

    def run(cmd):
        return cmd, subprocess.run(cmd, capture_output=True, text=True)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, res in ex.map(run, jobs):
                if res.returncode != 0:
                    raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + res.stdout + res.stderr)
                if verbose:
                    print(res.stderr)
    if jobs or not os.path.exists(lib_path):
        res = subprocess.run([nvcc, "-shared", "-o", lib_path, *objs, "-lcudart"], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
        with open(mode_file, "w") as f:
            f.write(tag)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv,
                timeline="--timeline" in sys.argv))
