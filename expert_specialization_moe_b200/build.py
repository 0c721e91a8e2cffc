"""In-tree build of libes_b200.so (the C-ABI library holding every CUDA kernel) for sm_100a.

    python -m expert_specialization_moe_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Sources are torch-free, so a full rebuild takes well under a minute.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libes_b200.so"
STAMP = LIBDIR / "libes_b200.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
] + os.environ.get("ES_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; es_b200 has no CPU fallback and cannot be built without the CUDA toolkit")
    return cand


def sources():
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*")) + list(INCLUDE.glob("*.h"))):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    fp = _fingerprint()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == fp:
        return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = LIBDIR / (src.stem + ".o")
        cmd = [nvcc, "-c", str(src), "-o", str(obj), f"-I{INCLUDE}", f"-I{CSRC}"] + NVCC_FLAGS
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(f"== {src.name}\n{out}")
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    (LIBDIR / "build.log").write_text("\n".join(log))
    if verbose:
        print("\n".join(log))
    cmd = [nvcc, "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-lcudart", "-Xlinker", "--no-undefined"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    for o in objs:
        o.unlink()
    STAMP.write_text(fp)
    return LIB


TORCH_SRC = PKG / "csrc_torch" / "es_b200_torch.cpp"
TORCH_LIB = LIBDIR / "libes_b200_torch.so"
TORCH_STAMP = LIBDIR / "libes_b200_torch.stamp"


def build_torch_ops(force: bool = False) -> Path:
    """The torch operator registration (TORCH_LIBRARY(es_b200)): one host-only C++ file compiled with g++ against the
    installed torch headers and linked to libes_b200.so (found beside it through $ORIGIN)."""
    import torch
    build(force=False)
    h = hashlib.sha256()
    h.update(TORCH_SRC.read_bytes())
    h.update((INCLUDE / "es_b200.h").read_bytes())
    h.update(torch.__version__.encode())
    fp = h.hexdigest()
    if not force and TORCH_LIB.exists() and TORCH_STAMP.exists() and TORCH_STAMP.read_text().strip() == fp:
        return TORCH_LIB
    tdir = Path(torch.__file__).resolve().parent
    cuda_home = Path(_nvcc()).resolve().parent.parent
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
           f"-I{cuda_home / 'include'}", f"-I{INCLUDE}", str(TORCH_SRC), "-o", str(TORCH_LIB),
           f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
           f"-L{LIBDIR}", "-les_b200", f"-L{cuda_home / 'lib64'}", "-lcudart",
           "-Wl,-rpath,$ORIGIN", "-Wl,--no-undefined"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the torch operator registration failed:\n{r.stdout}")
    TORCH_STAMP.write_text(fp)
    return TORCH_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    print(build_torch_ops(force="--force" in sys.argv))
