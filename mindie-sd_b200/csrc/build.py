"""Builds the native libraries of this package in-tree with nvcc for sm_100a.

    python mindie-sd_b200/csrc/build.py [--force] [--no-torch-ext]
    python mindie-sd_b200/csrc/build.py --variant /tmp/libvariant.so -D SDB_FA_BF16_MODE=5 [-D ...]

Outputs (next to the Python package, where its loader looks for them):
    mindiesd/plugin/libmindiesd_b200.so    the C-ABI library (CUDA only, no torch types)
    mindiesd/plugin/libPTAExtensionOPS.so  the torch operator library registering torch.ops.mindiesd.*
The second keeps the file name the reference's loader opens
(mindiesd/layers/register_ops.py:24-44 of MindIE-SD).

--variant builds one more copy of the C-ABI library with the attention kernel's build-time switches (the -D names at
the top of fa_fwd.cu) set differently, for compare_builds.py; the product libraries are not touched.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent / "mindiesd"
PLUGIN = PKG / "plugin"
OBJ = CSRC / "build"
INCLUDE = CSRC.parent.parent / "include"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

CABI_SOURCES = sorted(p.name for p in CSRC.glob("*.cu"))
CABI_LIB = PLUGIN / "libmindiesd_b200.so"
TORCH_EXT_SOURCES = ["torch_ops.cpp"]
TORCH_EXT_LIB = PLUGIN / "libPTAExtensionOPS.so"


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels of this package cannot be built")
    return exe


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), proc.stdout, proc.stderr))
    return proc.stdout + proc.stderr


def build_cabi(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    PLUGIN.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    sources = sorted(p.name for p in CSRC.glob("*.cu"))
    objs, jobs = [], []
    for src in sources:
        obj = OBJ / (src + ".o")
        objs.append(obj)
        if force or not _newer(obj, [CSRC / src] + headers):
            cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
                  ["-I", str(INCLUDE), "-c", str(CSRC / src), "-o", str(obj)]
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for out in pool.map(_run, jobs):
                if verbose and out.strip():
                    print(out)
    if force or jobs or not _newer(CABI_LIB, objs):
        _run([_nvcc()] + ARCH_FLAGS + ["-shared", "-cudart", "shared", "-o", str(CABI_LIB)] + [str(o) for o in objs] +
             ["-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return CABI_LIB


def build_torch_ext(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    srcs = [CSRC / s for s in TORCH_EXT_SOURCES]
    if not force and _newer(TORCH_EXT_LIB, srcs + [CABI_LIB] + list(INCLUDE.glob("*.h"))):
        return TORCH_EXT_LIB
    inc = []
    for d in cpp_extension.include_paths("cuda"):
        inc += ["-I", d]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
           "-I", str(INCLUDE)] + inc + [str(s) for s in srcs] + \
          ["-o", str(TORCH_EXT_LIB), "-L", str(PLUGIN), "-lmindiesd_b200",
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd)
    return TORCH_EXT_LIB


def build_variant(out: Path, defines, verbose: bool = False) -> Path:
    """The C-ABI library with fa_fwd.cu recompiled under the given -D switches; every other object is the
    product's (built first if needed)."""
    build_cabi(False, False)
    obj = Path(str(out) + ".fa_fwd.o")
    cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-D" + d for d in defines] + \
          ["-I", str(INCLUDE), "-c", str(CSRC / "fa_fwd.cu"), "-o", str(obj)]
    log = _run(cmd)
    if verbose and log.strip():
        print(log)
    others = [str(OBJ / (p.name + ".o")) for p in sorted(CSRC.glob("*.cu")) if p.name != "fa_fwd.cu"]
    _run([_nvcc()] + ARCH_FLAGS + ["-shared", "-cudart", "shared", "-o", str(out), str(obj)] + others +
         ["-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    obj.unlink()
    return out


def build_all(force: bool = False, torch_ext: bool = True, verbose: bool = False):
    libs = [build_cabi(force, verbose)]
    if torch_ext and all((CSRC / s).exists() for s in TORCH_EXT_SOURCES):
        libs.append(build_torch_ext(force))
    return libs


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--no-torch-ext", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--variant", metavar="OUT.so", help="build a copy of the C-ABI library with other switches")
    ap.add_argument("-D", dest="defines", action="append", default=[], metavar="NAME=VALUE")
    a = ap.parse_args()
    if a.variant:
        print(build_variant(Path(a.variant), a.defines, a.verbose))
        sys.exit(0)
    for lib in build_all(a.force, not a.no_torch_ext, a.verbose):
        print(lib)
    sys.exit(0)
