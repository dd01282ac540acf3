"""In-tree build of the CUDA library: one nvcc call, sm_100a only.

    python -m tilert_b200.build

writes ``tilert_b200/libtilert_b200.so`` next to the package (the place ``load_backend`` looks).
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
SRC = PKG / "csrc" / "cabi.cu"
OUT = PKG / "libtilert_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


BIND_SRC = PKG / "csrc" / "torch_binding.cpp"
BIND_OUT = PKG / "libtilert_dsv32.so"


def build_binding(force: bool = False) -> Path:
    """The dispatcher registration library (TORCH_LIBRARY translation unit over the C ABI): g++ against the
    installed torch headers, linked to libtilert_b200.so next to it."""
    import torch

    if not force and BIND_OUT.exists() and BIND_OUT.stat().st_mtime >= max(BIND_SRC.stat().st_mtime, OUT.stat().st_mtime):
        return BIND_OUT
    t = Path(torch.__file__).resolve().parent
    cuda_inc = "/usr/local/cuda/include"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{t / 'include'}", f"-I{t / 'include' / 'torch' / 'csrc' / 'api' / 'include'}", f"-I{cuda_inc}", str(BIND_SRC),
           "-o", str(BIND_OUT), f"-L{t / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", f"-L{PKG}",
           "-l:libtilert_b200.so", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stdout}\n{res.stderr}")
    return BIND_OUT


def needs_build() -> bool:
    if not OUT.exists():
        return True
    newest = max(p.stat().st_mtime for p in list((PKG / "csrc").glob("*")) + [PKG.parent / "include" / "tilert_b200.h"])
    return newest > OUT.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    cmd = ["nvcc", *NVCC_FLAGS, *( ["-Xptxas", "-v"] if verbose else []), "-o", str(OUT), str(SRC)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
    print(build_binding(force=True))
