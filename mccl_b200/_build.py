"""In-tree build of the native extension for sm_100a.

`build()` compiles every C++ / CUDA source under ``csrc/`` with
``-gencode arch=compute_100a,code=sm_100a`` through ninja
(``torch.utils.cpp_extension``) and leaves ``mccl_b200/_C.so`` beside this
file.  Nothing is compiled at import time: the package loads that file and
fails loudly if it is missing.  nvcc cross-compiles, so the build needs no GPU.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
PKG = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(ROOT, "build", "_C")

# Sources that are programs or tests of their own, not part of the extension.
_EXCLUDE = ("agent_main.cpp", os.sep + "tests" + os.sep)

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-Wall", "-Wno-unused-function", "-Wno-sign-compare"]


def sources() -> list[str]:
    out = []
    for pat in ("**/*.cpp", "**/*.cu"):
        for f in glob.glob(os.path.join(CSRC, pat), recursive=True):
            if any(x in f for x in _EXCLUDE):
                continue
            out.append(f)
    return sorted(out)


def _cutlass_include() -> list[str]:
    """CUTLASS / CuTe headers vendored in site-packages, if any (optional)."""
    import site
    for sp in site.getsitepackages():
        cand = os.path.join(sp, "flashinfer", "data", "cutlass", "include")
        if os.path.isdir(cand):
            return [cand]
    return []


def _stdcxx_ldflags() -> list[str]:
    """Links the shared libstdc++ explicitly.

    Some toolchain wrappers resolve -lstdc++ to the static archive; a second,
    private copy of the C++ runtime inside the extension has uninitialised
    locale state and crashes on the first stream insertion.  Naming the shared
    object first keeps a single C++ runtime in the process.
    """
    for d in ("/usr/lib/x86_64-linux-gnu", "/usr/lib/aarch64-linux-gnu", "/usr/lib64"):
        if os.path.exists(os.path.join(d, "libstdc++.so.6")):
            return [f"-L{d}", "-l:libstdc++.so.6"]
    return []


def build(verbose: bool = False) -> str:
    """Compiles the extension and returns the path of ``_C.so``."""
    from torch.utils.cpp_extension import load

    os.makedirs(BUILD_DIR, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 8))
    load(
        name="_C",
        sources=sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=CUDA_FLAGS,
        extra_include_paths=[CSRC],
        extra_ldflags=_stdcxx_ldflags() + ["-ldl", "-lpthread"],
        build_directory=BUILD_DIR,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    built = os.path.join(BUILD_DIR, "_C.so")
    target = os.path.join(PKG, "_C.so")
    if not os.path.exists(target) or os.path.getmtime(built) > os.path.getmtime(target):
        shutil.copy2(built, target + ".tmp")
        os.replace(target + ".tmp", target)
    build_agent(verbose)
    return target


def build_agent(verbose: bool = False) -> str | None:
    """Builds the stand-alone ``mccl-agent`` daemon (host only)."""
    main = os.path.join(CSRC, "agent", "agent_main.cpp")
    if not os.path.exists(main):
        return None
    out = os.path.join(PKG, "bin", "mccl-agent")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    srcs = [main] + sorted(glob.glob(os.path.join(CSRC, "cluster", "*.cpp")))
    newest = max(os.path.getmtime(s) for s in srcs)
    if os.path.exists(out) and os.path.getmtime(out) >= newest:
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-pthread", "-I", CSRC, "-o", out] + srcs + _stdcxx_ldflags()
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
