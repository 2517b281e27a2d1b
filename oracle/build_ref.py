"""Build the reference's own CUDA extension for the hot path (TEST INFRASTRUCTURE: a second parity source and the
"kernel to beat" timing; nothing in the shipped package loads it).

The sources are compiled where they lie in a checkout of heejunkim00/ResidualQuant
(plugins/residual_quantization/csrc); nothing is copied.  Only the dispatch translation units named in UNITS are
built (each instantiates every schedule, page size and mean variant of one model/mode/group family and takes many
minutes); `ref_stubs.cpp` supplies empty registration functions for the families that are left out, so that the
reference's own binding.cpp links unchanged.  Output: oracle/_ref/_cuda*.so, importable as module `_cuda` with the
reference's `attention(...)` and `quantize(...)`.

    python oracle/build_ref.py <reference checkout> [family ...]     # default family: ouro_anchor_3_g32
    python oracle/build_ref.py <reference checkout> --python-only    # only the PyTorch statement (seconds)

Besides the extension, `place_python` puts the reference's PyTorch statement of the same maths
(scripts/calibration/{quantization,rotation_math,rotation_training}.py: FP32Chain.reconstruct, probabilities) under
oracle/_ref/py/calibration/, so that the benchmark machine -- which has no checkout -- can time the reference's own CPU
path.  oracle/_ref/ is a build product: git-ignored, never part of the repository's history.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
FAMILIES = [f"{model}_{mode}_{group}" for model in ("ouro", "huginn")
            for mode in ("anchor_0", "anchor_3", "adjacent_0") for group in ("g16", "g32")]


PYTHON_FILES = ("quantization.py", "rotation_math.py", "rotation_training.py")


def place_python(reference: str) -> str:
    """Copy the reference's three calibration modules into oracle/_ref/py/calibration/ (importable as `calibration.*`
    with oracle/_ref/py on sys.path, the package name their own imports use)."""
    source = os.path.join(reference, "scripts", "calibration")
    if not all(os.path.isfile(os.path.join(source, name)) for name in PYTHON_FILES):
        raise SystemExit(f"{source} does not hold {PYTHON_FILES}")
    target = os.path.join(OUT, "py", "calibration")
    os.makedirs(target, exist_ok=True)
    for name in PYTHON_FILES:
        shutil.copyfile(os.path.join(source, name), os.path.join(target, name))
    return target


def main(reference: str, families) -> str:
    import torch
    from torch.utils import cpp_extension

    csrc = os.path.join(reference, "plugins", "residual_quantization", "csrc")
    if not os.path.isdir(csrc):
        raise SystemExit(f"{csrc} not found")
    unknown = [f for f in families if f not in FAMILIES]
    if unknown:
        raise SystemExit(f"unknown families {unknown}; choose from {FAMILIES}")
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(OUT, "_cuda" + suffix)

    stubs = os.path.join(OUT, "obj", "ref_stubs.cpp")
    with open(stubs, "w") as f:
        f.write("// registration functions of the dispatch families that were not compiled\n")
        for family in FAMILIES:
            if family not in families:
                f.write(f"void register_{family}() {{}}\n")

    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    includes = [csrc, *cpp_extension.include_paths(), sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
    defines = ["-DTORCH_EXTENSION_NAME=_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    common = ["-O3", "-std=c++17", *defines, *[f"-I{p}" for p in includes]]
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    jobs = []
    for source in (os.path.join(csrc, "dispatch", "binding.cpp"), os.path.join(csrc, "attention", "api.cpp"),
                   os.path.join(csrc, "quantize", "api.cpp"), stubs):
        obj = os.path.join(OUT, "obj", os.path.basename(os.path.dirname(source)) + "_" + os.path.basename(source) + ".o")
        jobs.append((obj, ["g++", "-fPIC", *common, "-c", source, "-o", obj]))
    for family in families:
        source = os.path.join(csrc, "dispatch", f"decode_{family}.cu")
        obj = os.path.join(OUT, "obj", f"decode_{family}.o")
        # the reference's own nvcc flags (setup.py), for sm_100a only
        jobs.append((obj, [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math",
                           "--extra-device-vectorization", "--restrict", "-Xcompiler", "-fPIC",
                           "--expt-relaxed-constexpr", *common, "-c", source, "-o", obj]))

    def run(job):
        obj, cmd = job
        if os.path.exists(obj) and not obj.endswith("ref_stubs.cpp.o"):
            return obj
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{done.stdout}\n{done.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 2) - 1)) as pool:
        objects = list(pool.map(run, jobs))
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", target, *objects, f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return target


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(place_python(sys.argv[1]))
    if "--python-only" not in sys.argv[2:]:
        print(main(sys.argv[1], [a for a in sys.argv[2:] if not a.startswith("--")] or ["ouro_anchor_3_g32"]))
