"""In-tree build of the native libraries.

Two artefacts, both placed in ``oneccl_b200/lib`` so that they travel with the
source tree:

* ``libccl_b200.so``   - the collective library itself (C++17 host runtime and
  sm_100a CUDA kernels, static CUDA runtime, no torch dependency); exports the
  ``ccl::`` C++ API of ``csrc/include/oneapi/ccl.hpp`` and a flat C API used by
  the Python bindings.
* ``_ccl_torch.so``    - the torch.distributed backend ("ccl" ProcessGroup),
  built against the installed torch headers.

The build is driven by a generated ninja file: one object per source, rebuilt
only when the source or a header changes.  ``python -m oneccl_b200._build``
builds everything; ``build_native()`` / ``build_torch_backend()`` are what
``__graft_entry__.build`` calls.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "oneccl_b200" / "lib"
BUILD = ROOT / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources(subdirs, exts):
    out = []
    for d in subdirs:
        for ext in exts:
            out += sorted((CSRC / d).rglob(f"*{ext}"))
    return out


def _ninja_escape(p) -> str:
    return str(p).replace(" ", "$ ").replace(":", "$:")


def _write_ninja(path: Path, rules: str, builds: list[str]):
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(rules + "\n" + "\n".join(builds) + "\n")


def build_native(verbose: bool = False, sanitize: str = "") -> Path:
    """Compile csrc/{core,bootstrap,transport,sched,coll,gpu,api,capi} into libccl_b200.so.

    ``sanitize`` = "address" or "thread" builds an instrumented copy of the host code into
    ``build/lib-<sanitizer>/`` (the CUDA translation units stay uninstrumented); the C++ examples can be
    linked against it to run the host runtime under ASan / TSan."""
    assert sanitize in ("", "address", "thread")
    libdir = BUILD / f"lib-{sanitize}" if sanitize else LIBDIR
    libdir.mkdir(parents=True, exist_ok=True)
    bdir = BUILD / (f"native-{sanitize}" if sanitize else "native")
    bdir.mkdir(parents=True, exist_ok=True)
    san_cxx = f" -fsanitize={sanitize} -fno-omit-frame-pointer" if sanitize else ""
    san_link = f" -Xcompiler -fsanitize={sanitize}" if sanitize else ""
    subdirs = ["core", "bootstrap", "transport", "sched", "coll", "comm", "fusion", "topo", "gpu", "api", "capi"]
    cpp = _sources(subdirs, [".cpp"])
    cu = _sources(subdirs, [".cu"])
    inc = f"-I{CSRC} -I{CSRC / 'include'} -I/usr/local/cuda/include"
    cxxflags = f"-std=c++17 -O2 -g1 -fPIC -Wall -Wno-unused-function -pthread {inc}{san_cxx}"
    nvflags = (
        f"-std=c++17 -O3 -lineinfo {' '.join(ARCH_FLAGS)} --expt-relaxed-constexpr --extended-lambda "
        f"-Xcompiler -fPIC -Xcompiler -Wno-unused-function {inc}"
    )
    rules = f"""
ninja_required_version = 1.5
cxx = {CXX}
nvcc = {NVCC}
cxxflags = {cxxflags}
nvflags = {nvflags}

rule cxx
  command = $cxx -MMD -MF $out.d $cxxflags -c $in -o $out
  depfile = $out.d
  deps = gcc
  description = CXX $in

rule nvcc
  command = $nvcc -MD -MF $out.d $nvflags -c $in -o $out
  depfile = $out.d
  deps = gcc
  description = NVCC $in

rule link
  command = $nvcc -shared -o $out $in -cudart static {'' if sanitize else '-Xlinker --no-undefined '}-Xlinker -soname=libccl_b200.so -lpthread -ldl -lrt{san_link}
  description = LINK $out
"""
    builds, objs = [], []
    for s in cpp:
        o = bdir / (str(s.relative_to(CSRC)).replace("/", "_") + ".o")
        builds.append(f"build {_ninja_escape(o)}: cxx {_ninja_escape(s)}")
        objs.append(o)
    for s in cu:
        o = bdir / (str(s.relative_to(CSRC)).replace("/", "_") + ".o")
        builds.append(f"build {_ninja_escape(o)}: nvcc {_ninja_escape(s)}")
        objs.append(o)
    lib = libdir / "libccl_b200.so"
    builds.append(f"build {_ninja_escape(lib)}: link {' '.join(_ninja_escape(o) for o in objs)}")
    builds.append(f"default {_ninja_escape(lib)}")
    _write_ninja(bdir / "build.ninja", rules, builds)
    _run_ninja(bdir, verbose)
    return lib


def build_torch_backend(verbose: bool = False) -> Path:
    """Compile the c10d backend against the installed torch and link it to libccl_b200.so."""
    import torch
    from torch.utils import cpp_extension as ce

    build_native(verbose)
    bdir = BUILD / "torch"
    bdir.mkdir(parents=True, exist_ok=True)
    srcs = sorted((ROOT / "oneccl_b200" / "torch_backend").glob("*.cpp"))
    if not srcs:
        raise RuntimeError("no torch backend sources")
    incs = ce.include_paths() + [str(CSRC), str(CSRC / "include"), "/usr/local/cuda/include",
                                 sysconfig.get_paths()["include"]]
    inc = " ".join(f"-I{p}" for p in incs)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxxflags = (
        f"-std=c++17 -O2 -fPIC -Wall -Wno-unused-function -Wno-sign-compare -pthread {inc} "
        f"-D_GLIBCXX_USE_CXX11_ABI={abi} -DTORCH_EXTENSION_NAME=_ccl_torch -DTORCH_API_INCLUDE_EXTENSION_H -DUSE_C10D_NCCL=0"
    )
    tlib = Path(torch.__file__).parent / "lib"
    ext = LIBDIR / "_ccl_torch.so"
    ldflags = (
        f"-shared -L{tlib} -L{LIBDIR} -Wl,-rpath,{tlib} '-Wl,-rpath,$$ORIGIN' "
        f"-lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda -ltorch -ltorch_python -lccl_b200"
    )
    rules = f"""
ninja_required_version = 1.5
cxx = {CXX}
cxxflags = {cxxflags}
ldflags = {ldflags}

rule cxx
  command = $cxx -MMD -MF $out.d $cxxflags -c $in -o $out
  depfile = $out.d
  deps = gcc
  description = CXX $in

rule link
  command = $cxx -o $out $in $ldflags
  description = LINK $out
"""
    builds, objs = [], []
    for s in srcs:
        o = bdir / (s.name + ".o")
        builds.append(f"build {_ninja_escape(o)}: cxx {_ninja_escape(s)}")
        objs.append(o)
    builds.append(f"build {_ninja_escape(ext)}: link {' '.join(_ninja_escape(o) for o in objs)} | {_ninja_escape(LIBDIR / 'libccl_b200.so')}")
    builds.append(f"default {_ninja_escape(ext)}")
    _write_ninja(bdir / "build.ninja", rules, builds)
    _run_ninja(bdir, verbose)
    return ext


def _run_ninja(bdir: Path, verbose: bool):
    ninja = shutil.which("ninja")
    cmd = [ninja] if ninja else [sys.executable, "-m", "ninja"]
    cmd += ["-C", str(bdir)]
    if verbose:
        cmd.append("-v")
    jobs = os.environ.get("CCL_BUILD_JOBS")
    if jobs:
        cmd += ["-j", jobs]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-20000:])
        raise RuntimeError(f"native build failed in {bdir}")
    if verbose:
        print(r.stdout)


def build_all(verbose: bool = False):
    build_native(verbose)
    if (ROOT / "oneccl_b200" / "torch_backend").exists():
        build_torch_backend(verbose)


if __name__ == "__main__":
    # python -m oneccl_b200._build [-v] [--sanitize address|thread]
    if "--sanitize" in sys.argv:
        kind = sys.argv[sys.argv.index("--sanitize") + 1]
        print(build_native(verbose="-v" in sys.argv, sanitize=kind))  # path for CCL_B200_LIBRARY
    else:
        build_all(verbose="-v" in sys.argv)
