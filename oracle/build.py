"""Build recipe for the CPU checker (test infrastructure, not the product).

``python oracle/build.py``           builds ``oracle/liboracle.so`` from ``brt_oracle.c``
``python oracle/build.py --ref``     also builds the reference project's own router and
                                     distributed torch extensions into ``oracle/_ref/``
                                     when the reference tree is available (see
                                     ``build_reference``).

The shared objects are build artefacts: they are git-ignored and rebuilt on demand.
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
SRC = HERE / "brt_oracle.c"
REF_OUT = HERE / "_ref"

_BASE_FLAGS = [
    "-O2", "-fPIC", "-ffp-contract=off", "-Wall", "-Wextra", "-std=gnu11",
    "-fvisibility=hidden", "-shared",
]


def _compilers():
    seen = []
    for c in ("/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc")):
        if c and c not in seen and os.path.exists(c):
            seen.append(c)
    return seen


def build_oracle(force: bool = False) -> Path:
    """Compile the C restatement; OpenMP when the compiler supports it."""
    if not force and LIB.exists() and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    errors = []
    for cc in _compilers():
        for omp in (["-fopenmp"], []):
            cmd = [cc, *_BASE_FLAGS, *omp, "-o", str(LIB), str(SRC), "-lm"]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode == 0:
                return LIB
            errors.append(f"$ {' '.join(cmd)}\n{proc.stderr}")
    raise RuntimeError("could not build liboracle.so:\n" + "\n".join(errors))


def reference_root() -> Path:
    """The reference checkout: BRT_REFERENCE_ROOT, else a directory named ``reference``
    beside this repository."""
    default = Path(__file__).resolve().parents[2] / "reference"
    return Path(os.environ.get("BRT_REFERENCE_ROOT", str(default)))


def build_reference(force: bool = False):
    """Compile the reference's own router/distributed extensions, unmodified.

    Sources are read where they lie under the reference tree; only the two
    extension modules are written, to ``oracle/_ref/brt_ref_router*.so`` and
    ``oracle/_ref/brt_ref_distributed*.so``.  The reference's ``setup.py`` is not
    run: it asks for C++14 and an un-vendored dmlc-core; the few CHECK/LOG macros
    the sources use come from the shim header written next to the objects.
    Returns the output directory, or None when the reference tree is absent.
    """
    ref = reference_root()
    if not (ref / "src" / "router" / "route.cu").exists():
        return None
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    REF_OUT.mkdir(exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    outputs = {
        "brt_ref_router": REF_OUT / f"brt_ref_router{suffix}",
        "brt_ref_distributed": REF_OUT / f"brt_ref_distributed{suffix}",
    }
    if not force and all(p.exists() for p in outputs.values()):
        return REF_OUT

    shim_dir = REF_OUT / "shim" / "dmlc"
    shim_dir.mkdir(parents=True, exist_ok=True)
    # Minimal stand-in for the CHECK*/LOG macros of dmlc-core (an empty git
    # submodule in the reference tree).  A failed check throws instead of
    # aborting the process.
    (shim_dir / "common.h").write_text(_DMLC_SHIM)
    (shim_dir / "logging.h").write_text('#include "common.h"\n')

    torch_inc = cpp_extension.include_paths()
    py_inc = sysconfig.get_paths()["include"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = [f"-I{ref / 'include'}", f"-I{REF_OUT / 'shim'}", f"-I{py_inc}",
            f"-I{cuda_home}/include", *[f"-I{p}" for p in torch_inc]]
    torch_lib = Path(torch.__file__).parent / "lib"
    nccl_lib = None
    try:
        import nvidia.nccl as _n  # noqa: F401

        for base in _n.__path__:
            cand = Path(base) / "lib"
            if (cand / "libnccl.so.2").exists():
                nccl_lib = cand
    except Exception:
        pass
    obj_dir = REF_OUT / "obj"
    obj_dir.mkdir(exist_ok=True)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    nvcc = shutil.which("nvcc") or f"{cuda_home}/bin/nvcc"
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"$ {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")

    def nvcc_obj(src, name):
        out = obj_dir / f"{name}.o"
        run([nvcc, "-std=c++17", "-O3", "-Xcompiler", "-fPIC", "-ccbin", cxx,
             "-gencode", "arch=compute_100a,code=sm_100a", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             *incs, "-c", str(src), "-o", str(out)])
        return out

    def cxx_obj(src, name, ext_name):
        out = obj_dir / f"{name}.o"
        run([cxx, "-std=c++17", "-O2", "-fPIC", "-DUSE_CUDA", "-DUSE_NCCL",
             f"-DTORCH_EXTENSION_NAME={ext_name}", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             "-DTORCH_API_INCLUDE_EXTENSION_H", *incs, "-c", str(src), "-o", str(out)])
        return out

    link_common = [f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-ltorch", "-ltorch_cpu",
                   "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python",
                   f"-L{cuda_home}/lib64", "-lcudart"]

    router_objs = [
        nvcc_obj(ref / "src/router/location.cu", "location"),
        nvcc_obj(ref / "src/router/route.cu", "route"),
        cxx_obj(ref / "src/backend/torch/router.cc", "router_binding", "brt_ref_router"),
    ]
    run([cxx, "-shared", "-o", str(outputs["brt_ref_router"]), *map(str, router_objs),
         *link_common])

    if nccl_lib is not None:
        dist_objs = [
            nvcc_obj(ref / "src/distributed/local_reorder.cu", "local_reorder"),
            cxx_obj(ref / "src/distributed/collective.cc", "collective", "brt_ref_distributed"),
            cxx_obj(ref / "src/backend/torch/nccl_manager.cc", "nccl_manager",
                    "brt_ref_distributed"),
            cxx_obj(ref / "src/backend/torch/distributed.cc", "distributed_binding",
                    "brt_ref_distributed"),
        ]
        run([cxx, "-shared", "-o", str(outputs["brt_ref_distributed"]), *map(str, dist_objs),
             *link_common, f"-L{nccl_lib}", f"-Wl,-rpath,{nccl_lib}", "-l:libnccl.so.2"])
    shutil.rmtree(obj_dir, ignore_errors=True)
    return REF_OUT


_DMLC_SHIM = r"""// Stand-in for the few dmlc-core logging macros the reference sources use.
#pragma once
#include <sstream>
#include <stdexcept>
#include <iostream>
namespace brt_ref_shim {
struct Fatal {
  std::ostringstream s;
  template <typename T> Fatal& operator<<(const T& v) { s << v; return *this; }
  [[noreturn]] ~Fatal() noexcept(false) { throw std::runtime_error(s.str()); }
};
struct Warn {
  template <typename T> Warn& operator<<(const T& v) { std::cerr << v; return *this; }
  ~Warn() { std::cerr << std::endl; }
};
struct Voidify { void operator&(Fatal&) {} void operator&(Warn&) {} };
}  // namespace brt_ref_shim
#ifndef CHECK
#define BRT_REF_CHECK_(cond, text) \
  (cond) ? (void)0 : ::brt_ref_shim::Voidify() & ::brt_ref_shim::Fatal() << "Check failed: " text " "
#define CHECK(x) BRT_REF_CHECK_((x), #x)
#define CHECK_EQ(a, b) BRT_REF_CHECK_((a) == (b), #a " == " #b)
#define CHECK_NE(a, b) BRT_REF_CHECK_((a) != (b), #a " != " #b)
#define CHECK_LE(a, b) BRT_REF_CHECK_((a) <= (b), #a " <= " #b)
#define CHECK_LT(a, b) BRT_REF_CHECK_((a) < (b), #a " < " #b)
#define CHECK_GE(a, b) BRT_REF_CHECK_((a) >= (b), #a " >= " #b)
#define CHECK_GT(a, b) BRT_REF_CHECK_((a) > (b), #a " > " #b)
#endif
#ifndef LOG
#define LOG_FATAL ::brt_ref_shim::Fatal()
#define LOG_WARNING ::brt_ref_shim::Warn()
#define LOG_INFO ::brt_ref_shim::Warn()
#define LOG_ERROR ::brt_ref_shim::Warn()
#define LOG(sev) LOG_##sev
#endif
"""


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference(force="--force" in sys.argv))
