"""In-tree build of the sm_100a extension.

Kernels (`*.cu`) are compiled with nvcc for `compute_100a/sm_100a` only and see no torch
headers, so each file builds in seconds; the torch-facing glue (`*bindings.cpp`) is compiled
with g++. Everything links into `halite_b200/_C.so`, next to the package, so the binary
travels with the source tree. A content hash of sources and flags beside the `.so` decides
whether a rebuild is needed; a stale or missing binary on a machine without nvcc is an error,
never a silent fallback.
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
SO_PATH = os.path.join(PKG, "_C.so")
HASH_PATH = os.path.join(PKG, "_C.hash")
OBJ_DIR = os.path.join(CSRC, "build")
EXT_NAME = "_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wno-deprecated-declarations",
             f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-D_GLIBCXX_USE_CXX11_ABI=1"]


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    hdr = sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh")))
    return cu, cpp, hdr


def source_hash() -> str:
    cu, cpp, hdr = _sources()
    h = hashlib.sha256()
    for name in cu + cpp + hdr:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(SO_PATH) and os.path.exists(HASH_PATH)):
        return False
    with open(HASH_PATH) as f:
        return f.read().strip() == source_hash()


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return cand
    nvcc = shutil.which("nvcc")
    if nvcc:
        return os.path.dirname(os.path.dirname(nvcc))
    raise RuntimeError("nvcc not found: cannot build the halite_b200 sm_100a extension")


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link `_C.so`. Returns the path."""
    if not force and is_current():
        return SO_PATH
    import torch
    from torch.utils import cpp_extension

    cuda = _cuda_home()
    nvcc = os.path.join(cuda, "bin", "nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    cu, cpp, _ = _sources()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx_flags = [f for f in CXX_FLAGS if not f.startswith("-D_GLIBCXX")] + [f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [
        f"-I{os.path.join(cuda, 'include')}",
        f"-I{sysconfig.get_paths()['include']}",
        f"-I{CSRC}",
    ]
    jobs = []
    objs = []
    for name in cu:
        obj = os.path.join(OBJ_DIR, name + ".o")
        objs.append(obj)
        extra = ["-Xptxas", "-v"] if verbose else []
        jobs.append([nvcc, *NVCC_FLAGS, *extra, f"-I{CSRC}", "-c", os.path.join(CSRC, name), "-o", obj])
    for name in cpp:
        obj = os.path.join(OBJ_DIR, name + ".o")
        objs.append(obj)
        jobs.append(["g++", *cxx_flags, *inc, "-c", os.path.join(CSRC, name), "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        outs = list(pool.map(_run, jobs))
    if verbose:
        for o in outs:
            sys.stderr.write(o)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = [
        "g++", "-shared", *objs, "-o", SO_PATH,
        f"-L{torch_lib}", f"-L{os.path.join(cuda, 'lib64')}",
        "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
        "-lcudart", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}",
    ]
    _run(link)
    with open(HASH_PATH, "w") as f:
        f.write(source_hash())
    return SO_PATH


_module = None


def load():
    """Import the built extension (building it first when the sources changed and nvcc exists)."""
    global _module
    if _module is not None:
        return _module
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    if not is_current():
        if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
            build()
        elif not os.path.exists(SO_PATH):
            raise RuntimeError("halite_b200/_C.so is missing and nvcc is not available to build it")
    spec = importlib.util.spec_from_file_location(EXT_NAME, SO_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _module = mod
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
