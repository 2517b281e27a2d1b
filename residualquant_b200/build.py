"""Build recipe for the C-ABI kernel library (`librq_b200.so`, in-tree, sm_100a only).

    python -m residualquant_b200.build [--force] [--verbose] [--timeline]

`--timeline` additionally builds `librq_b200_timeline.so`: the same library with the attention kernels' phase timestamps
compiled in (RQ_ATTENTION_TIMELINE=1), for `python -m residualquant_b200.timeline`.

nvcc cross-compiles without a GPU.  The quantizer translation unit is built with -fmad=false because its
packed output has to be reproducible bit for bit; no translation unit uses --use_fast_math.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIBRARY = os.path.join(HERE, "librq_b200.so")
TIMELINE_LIBRARY = os.path.join(HERE, "librq_b200_timeline.so")
TIMELINE_UNITS = ("rq_attention_d128.cu", "rq_attention_d96.cu")   # the units that instantiate the attention kernels

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
UNITS = {
    "rq_quantize.cu": ["-fmad=false"],
    "rq_attention.cu": [],
    "rq_attention_d128.cu": [],
    "rq_attention_d96.cu": [],
    "rq_peer.cu": [],
    "rq_capi.cu": [],
}
HEADERS = ["rq_common.cuh", "rq_kernels.h", "rq_attention_impl.cuh", os.path.join("..", "..", "include", "rq_b200.h")]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the kernels cannot be built")
    return found


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(s) > stamp for s in sources)


def _compile(unit: str, flags, verbose: bool, suffix: str = "") -> str:
    source = os.path.join(CSRC, unit)
    obj = os.path.join(BUILD, unit.replace(".cu", suffix + ".o"))
    deps = [source, os.path.abspath(__file__)] + [os.path.join(CSRC, h) for h in HEADERS]
    if _stale(obj, deps):
        cmd = [nvcc(), *ARCH, *COMMON, *flags, "-c", source, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {unit}:\n{done.stdout}\n{done.stderr}")
        if verbose:
            print(done.stderr, flush=True)
    return obj


def _link(target: str, objects) -> None:
    if _stale(target, objects):
        cmd = [nvcc(), *ARCH, "-shared", "-o", target, *objects]  # static cudart: no runtime search path needed
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    if force:
        for name in os.listdir(BUILD):
            os.remove(os.path.join(BUILD, name))
        for library in (LIBRARY, TIMELINE_LIBRARY):
            if os.path.exists(library):
                os.remove(library)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(UNITS)) as pool:
        objects = list(pool.map(lambda item: _compile(item[0], item[1], verbose), UNITS.items()))
        stamped = {}
        if timeline:
            stamped = dict(zip(TIMELINE_UNITS, pool.map(
                lambda unit: _compile(unit, [*UNITS[unit], "-DRQ_ATTENTION_TIMELINE=1"], verbose, "_timeline"), TIMELINE_UNITS)))
    _link(LIBRARY, objects)
    if timeline:
        swapped = [stamped.get(unit, obj) for unit, obj in zip(UNITS, objects)]
        _link(TIMELINE_LIBRARY, swapped)
    return LIBRARY


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--timeline", action="store_true", help="also build the library with phase timestamps compiled in")
    args = parser.parse_args()
    print(build(args.force, args.verbose, args.timeline))
    sys.exit(0)
