"""In-tree native build: host scheduler (g++), simulator CLI (g++), CUDA runtime + kernels (nvcc sm_100a).

Everything is compiled with explicit commands into the source tree (``fast_b200/*.so``,
``build/fastb-sim``) so that the binaries travel with the tree; nothing is JIT-cached elsewhere.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "fast_b200"
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
EXT = sysconfig.get_config_var("EXT_SUFFIX")

SCHED_SRCS = ["decompose", "plan", "validate", "cost_model", "lower", "workload", "serialize", "host_threads"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _run(cmd, **kw):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _headers(sub):
    return [p for p in (CSRC / sub).rglob("*") if p.suffix in (".h", ".cuh", ".hpp")]


def build_sched(force=False):
    import pybind11

    out = PKG / f"_sched{EXT}"
    srcs = [CSRC / "sched" / f"{s}.cc" for s in SCHED_SRCS] + [CSRC / "sched" / "py_sched.cc"]
    if force or _stale(out, srcs + _headers("sched")):
        inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}"]
        _run(["g++", "-std=c++17", "-O2", "-Wall", "-shared", "-fPIC", "-pthread", *inc, *srcs, "-o", out])
    return out


def build_sim(force=False):
    out = ROOT / "build" / "fastb-sim"
    out.parent.mkdir(exist_ok=True)
    srcs = [CSRC / "sim" / "main.cc"] + [CSRC / "sched" / f"{s}.cc" for s in SCHED_SRCS]
    if force or _stale(out, srcs + _headers("sched")):
        _run(["g++", "-std=c++17", "-O2", "-Wall", "-pthread", *srcs, "-o", out])
    return out


def build_twin_check(force=False, tsan=True, relaxed=False):
    """Threaded host twin of the executor protocol as an executable; with ``tsan`` it is built with
    ThreadSanitizer (build/fastb-twin-tsan), which makes it the protocol's race detector.
    ``relaxed`` builds the deliberately broken variant (signals without release / acquire) that the
    detector must report."""
    out = ROOT / "build" / (("fastb-twin-tsan" if tsan else "fastb-twin") + ("-relaxed" if relaxed else ""))
    out.parent.mkdir(exist_ok=True)
    srcs = [CSRC / "sched" / "twin_check.cc"] + [CSRC / "sched" / f"{s}.cc" for s in SCHED_SRCS]
    if force or _stale(out, srcs + _headers("sched")):
        flags = ["-O1", "-g", "-fsanitize=thread"] if tsan else ["-O2"]
        if relaxed:
            flags.append("-DFASTB_TWIN_RELAXED")
        _run(["g++", "-std=c++17", *flags, "-Wall", "-pthread", *srcs, "-o", out])
    return out


def build_moe_twin(force=False, tsan=True, broken=False):
    """Threaded host twin of the expert-parallel step's synchronisation (csrc/sched/moe_twin.cc);
    with ``tsan`` built with ThreadSanitizer (build/fastb-moe-twin-tsan). ``broken`` drops the wait
    for the owners' ready flags before combine, which the detector must report."""
    out = ROOT / "build" / (("fastb-moe-twin-tsan" if tsan else "fastb-moe-twin") + ("-broken" if broken else ""))
    out.parent.mkdir(exist_ok=True)
    srcs = [CSRC / "sched" / "moe_twin.cc"]
    if force or _stale(out, srcs):
        flags = ["-O1", "-g", "-fsanitize=thread"] if tsan else ["-O2"]
        if broken:
            flags.append("-DFASTB_MOE_TWIN_NO_READY_WAIT")
        _run(["g++", "-std=c++17", *flags, "-Wall", "-pthread", *srcs, "-o", out])
    return out


def build_selfcheck(force=False):
    """Native self-check executable of the scheduler library (build/fastb-selfcheck)."""
    out = ROOT / "build" / "fastb-selfcheck"
    out.parent.mkdir(exist_ok=True)
    srcs = [CSRC / "sched" / "selfcheck.cc"] + [CSRC / "sched" / f"{s}.cc" for s in SCHED_SRCS]
    if force or _stale(out, srcs + _headers("sched") + _headers("runtime") + [CSRC / "kernels" / "tile_walker.h"]):
        _run(["g++", "-std=c++17", "-O2", "-Wall", "-pthread", *srcs, "-o", out])
    return out


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "runtime").glob("*.cu"))


def build_cuda(force=False, verbose=False):
    """Compile every .cu for sm_100a and link them with the torch binding into fast_b200/_C.so."""
    import torch
    from torch.utils import cpp_extension as ce

    out = PKG / f"_C{EXT}"
    OBJ.mkdir(parents=True, exist_ok=True)
    hdrs = _headers("kernels") + _headers("runtime") + _headers("torch")
    cu = cuda_sources()
    cpp = sorted((CSRC / "torch").glob("*.cpp")) + sorted((CSRC / "runtime").glob("*.cc"))
    torch_inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    log = []

    def nvcc(src):
        o = OBJ / (src.stem + ".o")
        if force or _stale(o, [src] + hdrs):
            log.append(_run([f"{cuda_home}/bin/nvcc", *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
                             "-Xcompiler", "-fPIC", "-Xptxas", "-v", f"-I{CSRC}", f"-I{cuda_home}/include", "-c", src, "-o", o]))
        return o

    def gxx(src):
        o = OBJ / (src.stem + ".o")
        if force or _stale(o, [src] + hdrs):
            _run(["g++", "-std=c++17", "-O2", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
                  "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", *torch_inc, f"-I{cuda_home}/include", "-c", src, "-o", o])
        return o

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(nvcc, cu)) + list(ex.map(gxx, cpp))
    if force or _stale(out, objs):
        libs = [f"-L{p}" for p in ce.library_paths()] + [f"-L{cuda_home}/lib64"]
        _run(["g++", "-shared", *objs, "-o", out, *libs, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
              "-lcudart", "-lcuda", f"-Wl,-rpath,{ce.library_paths()[0]}", f"-Wl,-rpath,{cuda_home}/lib64"])
    if verbose:
        print("".join(log))
    (ROOT / "build" / "ptxas.log").write_text("".join(log)) if log else None
    return out


def build_all(force=False, verbose=False):
    build_sched(force)
    build_sim(force)
    build_selfcheck(force)
    if cuda_sources():
        build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built")
