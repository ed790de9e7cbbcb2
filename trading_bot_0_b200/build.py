"""Build the CUDA library in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m trading_bot_0_b200.build            # -> trading_bot_0_b200/lib/libssd_b200.so
    python -m trading_bot_0_b200.build --torch    # also -> lib/libssd_b200_torch.so (libtorch autograd node over the C ABI)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libssd_b200.so"
SOURCES = ["ssd_api.cu", "ssd_simt.cu", "ssd_decode.cu", "ssd_tensor.cu", "ssd_noalloc.cu", "ssd_prepost.cu", "ssd_sp.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared"]
LINK_LIBS = ["-ldl"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        [PKG.parent / "include" / "ssd_b200.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "ssd_b200.h", Path(__file__)]


def build(force: bool = False, verbose: bool = False) -> Path:
    """One object per source file (compiled in parallel, rebuilt only when the source or a header is newer), then one
    link step.  No relocatable device code: every kernel is launched from the file that defines it."""
    if not force and not needs_build():
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    LIB.parent.mkdir(parents=True, exist_ok=True)
    objdir = LIB.parent / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_t = max(h.stat().st_mtime for h in _headers())
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: str):
        obj = objdir / (src + ".o")
        if not force and obj.exists() and obj.stat().st_mtime >= max(hdr_t, (CSRC / src).stat().st_mtime):
            return obj, None
        cmd = [nvcc_path(), *flags, "-c", str(CSRC / src), "-o", str(obj)]
        return obj, (cmd, subprocess.run(cmd, capture_output=True, text=True))

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        results = list(ex.map(compile_one, SOURCES))
    for obj, run in results:
        if run is None:
            continue
        cmd, r = run
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cmd = [nvcc_path(), "-shared", "-Xcompiler", "-fPIC", *[str(o) for o, _ in results], "-o", str(LIB), *LINK_LIBS]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed: " + " ".join(cmd))
    return LIB


def host_cxx() -> str:
    """The system g++ first: a toolchain wrapper in $CXX may resolve -lstdc++ to a static archive, and a second copy of the
    C++ runtime inside a library loaded next to libtorch breaks stream formatting (seen as a crash while an error message
    was being built).  --exclude-libs below keeps any archive's symbols out of the dynamic symbol table as well."""
    for cand in ("/usr/bin/g++", os.environ.get("CXX"), shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("no host C++ compiler found")


TORCH_LIB = PKG / "lib" / "libssd_b200_torch.so"
TORCH_SRC = CSRC / "ssd_torch.cpp"


def build_torch(force: bool = False) -> Path:
    """The libtorch autograd node and the libtch-style C entry points (host C++ only: g++ against this image's libtorch,
    linked to libssd_b200.so beside it)."""
    build(force=False)
    deps = [TORCH_SRC, PKG.parent / "include" / "ssd_b200.h", Path(__file__)]
    if not force and TORCH_LIB.exists() and all(d.stat().st_mtime <= TORCH_LIB.stat().st_mtime for d in deps):
        return TORCH_LIB
    import torch
    from torch.utils import cpp_extension as E
    inc = [f"-I{p}" for p in E.include_paths("cuda")]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [host_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wl,--exclude-libs,ALL",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", *inc, str(TORCH_SRC), "-o", str(TORCH_LIB),
           f"-L{LIB.parent}", "-lssd_b200", f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("g++ failed: " + " ".join(cmd))
    return TORCH_LIB


CALLER = PKG / "lib" / "ssd_torch_caller"
CALLER_SRC = PKG.parent / "tests" / "cpp" / "ssd_torch_caller.cpp"


def build_torch_caller(force: bool = False) -> Path:
    """The C++ test program that drives the C entry points of libssd_b200_torch.so the way a tch-rs binding would."""
    build_torch(force=False)
    if not force and CALLER.exists() and CALLER.stat().st_mtime >= max(CALLER_SRC.stat().st_mtime, TORCH_LIB.stat().st_mtime):
        return CALLER
    import torch
    from torch.utils import cpp_extension as E
    inc = [f"-I{p}" for p in E.include_paths("cuda")]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    # the CUDA runtime libtorch was linked against: the pip package beside torch if there is one, else the toolkit's
    rt = Path(tlib).parent.parent / "nvidia" / "cuda_runtime" / "lib"
    cudart = [f"-L{rt}", "-l:libcudart.so.12", f"-Wl,-rpath,{rt}"] if (rt / "libcudart.so.12").exists() else \
        ["-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"]
    cmd = [host_cxx(), "-O1", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, str(CALLER_SRC), "-o", str(CALLER), f"-L{LIB.parent}", "-lssd_b200_torch", "-lssd_b200", f"-L{tlib}",
           "-Wl,--no-as-needed", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", *cudart, "-Wl,-rpath,$ORIGIN",
           f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("g++ failed: " + " ".join(cmd))
    return CALLER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch(force=True))
        print(build_torch_caller(force=True))
