"""Build the native extension ``opacus_b200/_C*.so`` in-tree.

``python -m opacus_b200.build`` compiles every ``csrc/*.cu`` with

    nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3

(sm_100a only; there is no other target) and the host-side bindings with the
host compiler, then links them against the installed torch.  No GPU is needed to
build.  Objects are cached under ``csrc/.build`` keyed by source hash, so a
rebuild only recompiles what changed.
"""
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
SRC = ROOT / "csrc"
OBJ = SRC / ".build"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _ext_path() -> Path:
    return ROOT / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(SRC.glob("*.h")) + sorted(SRC.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr)


def build(verbose: bool = False, force: bool = False, ptxas_verbose: bool = False) -> Path:
    """Compile what is stale and return the path of the shared object."""
    import torch
    from torch.utils import cpp_extension

    OBJ.mkdir(exist_ok=True)
    objects, changed = [], False
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")

    for cu in sorted(SRC.glob("*.cu")):
        flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_verbose else [])
        tag = _digest(cu, " ".join(flags))
        obj = OBJ / f"{cu.stem}.{tag}.o"
        if force or not obj.exists():
            for old in OBJ.glob(f"{cu.stem}.*.o"):
                old.unlink()
            _run([_nvcc(), *flags, "-I", SRC, "-c", cu, "-o", obj], verbose or ptxas_verbose)
            changed = True
        objects.append(obj)

    cxx = os.environ.get("CXX", "g++")
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{cuda_inc}", f"-I{SRC}",
                                                               f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    host_flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
                  "-DTORCH_API_INCLUDE_EXTENSION_H", "-w"]
    cpp = SRC / "bindings.cpp"
    tag = _digest(cpp, " ".join(host_flags) + torch.__version__)
    bobj = OBJ / f"bindings.{tag}.o"
    if force or not bobj.exists():
        for old in OBJ.glob("bindings.*.o"):
            old.unlink()
        _run([cxx, *host_flags, *inc, "-c", cpp, "-o", bobj], verbose)
        changed = True
    objects.append(bobj)

    out = _ext_path()
    if changed or not out.exists():
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
        _run([cxx, "-shared", *objects, "-o", out, f"-L{torch_lib}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda",
              "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart_static", "-lrt", "-ldl", "-lpthread",
              f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"], verbose)
    return out


def extension_path() -> Path:
    return _ext_path()


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_verbose="--ptxas" in sys.argv)
    print(path)
