"""Builds the native libraries in-tree with nvcc / g++ (no JIT cache, so the
built files travel with the source tree).

    python -m byteir_b200.build [--force]
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OUT = PKG / "_lib"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
HOSTCXX = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd):
    print(" ".join(str(c) for c in cmd), flush=True)
    subprocess.check_call([str(c) for c in cmd])


def build_kernels(force=False, verbose_ptxas=False):
    """libb200_kernels.so: the sm_100a kernels behind include/b200_kernels.h"""
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    deps = srcs + sorted((CSRC / "kernels").glob("*.cuh")) + [ROOT / "include" / "b200_kernels.h"]
    target = OUT / "libb200_kernels.so"
    if not force and not _newer(target, deps):
        return target
    OUT.mkdir(exist_ok=True)
    objs = []
    obj_dir = PKG / "_build"
    obj_dir.mkdir(exist_ok=True)
    procs = []
    for s in srcs:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if not force and not _newer(o, [s] + deps[len(srcs):]):
            continue
        cmd = [NVCC, "-std=c++17", "-O3", *ARCH, "-lineinfo", "-Xcompiler", "-fPIC",
               "-ccbin", HOSTCXX, "--expt-relaxed-constexpr",
               "-I", ROOT / "include", "-I", CSRC / "kernels", "-c", s, "-o", o]
        if verbose_ptxas:
            cmd += ["-Xptxas", "-v"]
        print(" ".join(str(c) for c in cmd), flush=True)
        procs.append((s, subprocess.Popen([str(c) for c in cmd])))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    _run([NVCC, "-shared", *ARCH, "-ccbin", HOSTCXX, "-o", target, *objs, "-lcudart"])
    return target


CUDA_INC = Path(NVCC).resolve().parent.parent / "include"
CUDA_LIB = Path(NVCC).resolve().parent.parent / "lib64"


def _gxx(srcs, target, extra, deps, force):
    if not force and not _newer(target, list(srcs) + list(deps)):
        return target
    OUT.mkdir(exist_ok=True)
    _run([HOSTCXX, "-std=c++17", "-O2", "-g", "-fPIC", "-shared", "-Wall", "-Wno-unused-function",
          "-I", ROOT / "include", "-I", CUDA_INC, *srcs, "-o", target,
          f"-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{CUDA_LIB}", *extra])
    return target


def build_flash_attn(force=False):
    """libflash_attn.so: the byre.custom entry points (run_flash_attn_fwd / _bwd), over libb200_kernels.so"""
    src = CSRC / "flash_attn" / "flash_api.cc"
    return _gxx([src], OUT / "libflash_attn.so",
                ["-L", OUT, "-lb200_kernels", "-L", CUDA_LIB, "-lcudart"],
                [ROOT / "include" / "b200_kernels.h", OUT / "libb200_kernels.so"], force)


def build_brt(force=False):
    """libbrt_b200.so: the MLIR-free brt host runtime, its CUDA provider and the C API"""
    srcs = sorted((CSRC / "brt").glob("*.cc"))
    hdrs = [p for p in (ROOT / "include").rglob("*.h")]
    return _gxx(srcs, OUT / "libbrt_b200.so",
                ["-L", OUT, "-lb200_kernels", "-L", CUDA_LIB, "-lcudart", "-ldl", "-lpthread"],
                hdrs + [OUT / "libb200_kernels.so"], force)


def build_all(force=False):
    libs = [build_kernels(force), build_flash_attn(force), build_brt(force)]
    return libs


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
