"""In-tree build of every shared library of the package (no CMake: g++ and nvcc directly).

Layout of the outputs mirrors the reference's (CMakeLists.txt:8 puts every extension library into
one `lib/` directory; the infra library is shared so that the registry exists once per process,
infra/pass/CMakeLists.txt:3-14):

    lib/libTritonExtPassInfra.so   registry + loop IR + pass manager
    lib/libloop_split.so           pass extension   (pass/LoopSplit)
    lib/libdot_tile_select.so      pass extension   (pass/DotTileSelect)
    lib/libb200_dot.so             backend extension: sm_100a kernels (tt.dot GEMM, fused attention forward)
                                   + launch C-ABI + lowering pass

Each extension is named by its `triton-ext.conf` and is skipped when TRITON_EXT_NAMES is set and
does not list it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

from . import conf

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
INCLUDE = os.path.join(ROOT, "include")

# (directory under csrc, pass class, sources, needs nvcc)
EXTENSIONS = [
    ("pass/LoopSplit", "LoopBisectPass", ["LoopSplitPass.cpp", "LoopSplitText.cpp"], False),
    ("pass/DotTileSelect", "DotTileSelectPass", ["DotTileSelectPass.cpp"], False),
    ("backend/B200Dot", "B200DotLoweringPass", ["b200_dot.cu", "b200_dot_static.cu", "B200DotLowering.cpp",
                                                   "../B200Attention/b200_attention.cu"], True),
]

CXXFLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _all_sources(d: str) -> list[str]:
    out = []
    for base, _, files in os.walk(d):
        out += [os.path.join(base, f) for f in files]
    return out


def build_all(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> list[str]:
    """Build everything that is missing or older than its sources; returns the library paths."""
    os.makedirs(LIB, exist_ok=True)
    built = []
    common_deps = _all_sources(os.path.join(CSRC, "infra")) + _all_sources(INCLUDE)
    infra = os.path.join(LIB, "libTritonExtPassInfra.so")
    if force or _stale(infra, common_deps):
        _run(["g++", *CXXFLAGS, "-shared", "-I", INCLUDE, "-I", os.path.join(CSRC, "infra"),
              os.path.join(CSRC, "infra", "pass_registry.cpp"), os.path.join(CSRC, "infra", "dot_loop_ir.cpp"),
              "-o", infra], verbose)
    built.append(infra)
    allow = conf.ext_names_filter()
    for rel, cls, sources, cuda in EXTENSIONS:
        d = os.path.join(CSRC, rel)
        if not conf.should_build(d, allow):
            continue
        meta = conf.read_conf(d)
        out = os.path.join(LIB, f"lib{meta.name}.so")
        deps = (common_deps + _all_sources(d) + _all_sources(os.path.join(CSRC, "backend", "B200Dot")) +
                _all_sources(os.path.join(CSRC, "backend", "B200Attention")))
        if force or _stale(out, deps):
            defs = [f"-DTRITON_EXT_NAME={meta.name}", f"-DTRITON_EXT_CLASS={cls}"]
            incs = ["-I", INCLUDE, "-I", os.path.join(CSRC, "infra"), "-I", os.path.join(CSRC, "backend", "B200Dot"),
                    "-I", os.path.join(CSRC, "backend", "B200Attention")]
            link = ["-L", LIB, "-lTritonExtPassInfra"]
            srcs = [os.path.join(d, s) for s in sources]
            if cuda:
                nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
                cmd = [nvcc, *NVCC_ARCH, "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                       *defs, *incs, *srcs, *link, "-Xlinker", "-rpath=$ORIGIN", "-o", out]
                if ptxas_verbose:
                    cmd[1:1] = ["-Xptxas", "-v"]
            else:
                cmd = ["g++", *CXXFLAGS, "-shared", *defs, *incs, *srcs, *link, "-Wl,-rpath,$ORIGIN", "-o", out]
            _run(cmd, verbose or ptxas_verbose)
        built.append(out)
    # The calibration probe of the tile model (a stand-alone program, not a library: nothing loads it).
    probe_src = os.path.join(CSRC, "backend", "B200Dot", "calibrate", "tcgen05_issue_probe.cu")
    probe = os.path.join(LIB, "tcgen05_issue_probe")
    if os.path.exists(probe_src) and (force or _stale(probe, [probe_src])):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, *NVCC_ARCH, "-O3", "-std=c++17", probe_src, "-o", probe], verbose)
    return built


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose=True, ptxas_verbose="--ptxas" in sys.argv):
        print(p)
