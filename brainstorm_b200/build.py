"""Builds ``libbrt_b200.so`` (hand-written sm_100a kernels behind the C ABI of
``include/brt_b200.h``) in-tree with nvcc.

    python -m brainstorm_b200.build [--force] [--verbose]

The library has no Python or torch dependency; ``brainstorm_b200._lib`` loads it
with ctypes.  nvcc cross-compiles without a GPU.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libbrt_b200.so"
OBJ_DIR = PKG / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"),
                                                "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return cand


def _host_compiler_flags():
    # the image's default CC points at a wrapper that nvcc cannot drive; prefer the system g++
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def sources():
    return sorted(CSRC.glob("*.cu"))


def _nccl_flags():
    """Link flags for NCCL: the copy bundled with torch's wheels, else the system one."""
    try:
        import nvidia.nccl as n

        for base in n.__path__:
            lib = Path(base) / "lib"
            if (lib / "libnccl.so.2").exists():
                inc = Path(base) / "include"
                return ([f"-I{inc}"] if inc.exists() else []), [f"-L{lib}", "-l:libnccl.so.2",
                                                                 "-Xlinker", f"-rpath={lib}"]
    except Exception:
        pass
    return [], ["-lnccl"]


def _stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in [*sources(), *CSRC.glob("*.cuh"),
                                             *INCLUDE.glob("*.h"), Path(__file__)])
    return LIB.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    nccl_inc, nccl_link = _nccl_flags()
    ptxas = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *_host_compiler_flags(), *ptxas, f"-I{INCLUDE}",
               *nccl_inc, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"$ {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            sys.stderr.write(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    cmd = [nvcc, *ARCH_FLAGS, *_host_compiler_flags(), "-shared", "-o", str(LIB),
           *map(str, objs), *nccl_link]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"$ {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
