"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host engines.

The kernels are plain ``extern "C"`` launchers (raw pointers + a ``cudaStream_t``) compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into ``recsdk_b200/_C_cuda.so`` and called through
``ctypes``; the host engines are a pybind11 module ``recsdk_b200/_C_host*.so``.  Neither depends on
libtorch headers, so a full rebuild takes well under a minute and needs no GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import List

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC_CUDA = ROOT / "csrc" / "cuda"
CSRC_HOST = ROOT / "csrc" / "host"
BUILD_DIR = ROOT / "build"

CUDA_SO = PKG_DIR / "_C_cuda.so"
HOST_SO = PKG_DIR / ("_C_host" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fopenmp", "-Wall", "-Wno-sign-compare"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: Path, sources: List[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("native build failed:\n  %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def _digest(flags: List[str]) -> str:
    return hashlib.sha1(" ".join(flags).encode()).hexdigest()[:8]


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/cuda/*.cu`` for sm_100a and link ``_C_cuda.so``."""
    srcs = sorted(CSRC_CUDA.glob("*.cu"))
    hdrs = sorted(CSRC_CUDA.glob("*.cuh")) + sorted(CSRC_CUDA.glob("*.h"))
    BUILD_DIR.mkdir(exist_ok=True)
    tag = _digest(NVCC_FLAGS)
    objs, jobs = [], []
    for s in srcs:
        o = BUILD_DIR / ("%s.%s.o" % (s.stem, tag))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append([_nvcc()] + NVCC_FLAGS + ["-I", str(CSRC_CUDA), "-c", str(s), "-o", str(o)])
    if jobs:
        if verbose:
            print("[recsdk_b200] nvcc: %d translation units" % len(jobs), file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or _stale(CUDA_SO, objs):
        _run([_nvcc(), "-shared", "-o", str(CUDA_SO)] + [str(o) for o in objs] + ["-lcudart"])
    return CUDA_SO


def build_host(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/host/*.cpp`` into the pybind11 module ``_C_host``."""
    import pybind11

    srcs = sorted(CSRC_HOST.glob("*.cpp"))
    hdrs = sorted(CSRC_HOST.glob("*.h")) + sorted(CSRC_HOST.glob("*.hpp"))
    BUILD_DIR.mkdir(exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC_HOST)]
    cuda_inc = Path("/usr/local/cuda/include")
    if cuda_inc.exists():
        inc += ["-I", str(cuda_inc)]
    tag = _digest(CXX_FLAGS)
    objs, jobs = [], []
    for s in srcs:
        o = BUILD_DIR / ("host_%s.%s.o" % (s.stem, tag))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(["g++"] + CXX_FLAGS + inc + ["-c", str(s), "-o", str(o)])
    if jobs:
        if verbose:
            print("[recsdk_b200] g++: %d translation units" % len(jobs), file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or _stale(HOST_SO, objs):
        libs = ["-fopenmp", "-lpthread", "-ldl"]
        _run(["g++", "-shared", "-o", str(HOST_SO)] + [str(o) for o in objs] + libs)
    return HOST_SO


_API_RE = None


def scan_signatures() -> dict:
    """Parse the ``RB_API`` declarations of ``csrc/cuda/*.cu`` into ctypes signature codes
    (``p`` pointer / stream, ``i`` int, ``l`` long long, ``f`` float; first letter = return type)."""
    import re

    out = {}
    rx = re.compile(r"RB_API\s+(int|long long|void)\s+(rb_\w+)\s*\(([^)]*)\)", re.S)
    for src in sorted(CSRC_CUDA.glob("*.cu")):
        for ret, name, args in rx.findall(src.read_text()):
            code = {"int": "i", "long long": "l", "void": "v"}[ret]
            args = args.strip()
            if args and args != "void":
                for a in args.split(","):
                    a = " ".join(a.split())
                    if "*" in a or a.startswith("cudaStream_t"):
                        code += "p"
                    elif a.startswith("long long") or a.startswith("unsigned long long") or a.startswith("int64_t") \
                            or a.startswith("uint64_t") or a.startswith("size_t"):
                        code += "l"
                    elif a.startswith("float"):
                        code += "f"
                    elif a.startswith("double"):
                        code += "d"
                    elif a.startswith("int") or a.startswith("unsigned") or a.startswith("uint32_t"):
                        code += "i"
                    else:
                        raise RuntimeError("cannot map C argument %r of %s" % (a, name))
            out[name] = code
    return out


def write_signatures() -> Path:
    sigs = scan_signatures()
    target = PKG_DIR / "ops" / "_signatures.py"
    body = ['"""Generated by recsdk_b200._build.write_signatures() from csrc/cuda/*.cu; do not edit."""',
            "SIGNATURES = {"]
    for k in sorted(sigs):
        body.append('    "%s": "%s",' % (k, sigs[k]))
    body.append("}")
    text = "\n".join(body) + "\n"
    if not target.exists() or target.read_text() != text:
        target.write_text(text)
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    write_signatures()
    build_host(force=force, verbose=verbose)
    build_cuda(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built:", CUDA_SO, HOST_SO)
