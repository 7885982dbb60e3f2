"""Builds the reference's own host-side id-processing library, UNMODIFIED, from its source tree into ``baseline/_ref``.

The reference's device code needs an Ascend NPU and cannot run here, but its host engines
(``training/torch_rec_v1/hybrid_torchrec/src``: ``IdsMapper``, ``unique``, ``block_bucketize_sparse_features_cpu``) are plain
C++ over libtorch + OpenMP.  This script compiles exactly those sources (no copy into this repository, no edits) with
the flags of the reference's own ``CMakeLists.txt`` that matter for speed (``-O3 -fopenmp -std=c++17``) and links them into
``baseline/_ref/libhybrid_cpp.so``, which ``python -m recsdk_b200.utils.microbench host_engines`` loads with
``torch.ops.load_library`` to time the reference's engines beside this package's on the same ids.

    python baseline/build_ref_host.py [/path/to/reference]        # or RECSDK_REFERENCE_ROOT=/path/to/reference
"""
import os
import subprocess
import sys
import sysconfig


def default_reference_root() -> str:
    """The reference checkout: ``RECSDK_REFERENCE_ROOT``, else a ``reference`` directory beside this repository."""
    env = os.environ.get("RECSDK_REFERENCE_ROOT")
    if env:
        return env
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.path.join(os.path.dirname(repo), "reference")


def build(ref_root: str = "", verbose: bool = True) -> str:
    import torch

    ref_root = ref_root or default_reference_root()
    if not os.path.isdir(os.path.join(ref_root, "training")):
        raise FileNotFoundError("no reference checkout at %r: set RECSDK_REFERENCE_ROOT" % ref_root)
    from torch.utils import cpp_extension as ce

    here = os.path.dirname(os.path.abspath(__file__))
    out_dir = os.path.join(here, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    so = os.path.join(out_dir, "libhybrid_cpp.so")
    src_dir = os.path.join(ref_root, "training", "torch_rec_v1", "hybrid_torchrec", "src")
    srcs = [os.path.join(src_dir, "bind_torch_lib.cpp")] + sorted(
        os.path.join(src_dir, "ids_process", f) for f in os.listdir(os.path.join(src_dir, "ids_process")) if f.endswith(".cpp"))
    if os.path.exists(so) and all(os.path.getmtime(so) >= os.path.getmtime(s) for s in srcs):
        return so
    inc = ["-I" + p for p in ce.include_paths()] + ["-I" + os.path.join(src_dir, "ids_process"), "-I" + src_dir,
                                                     "-I" + sysconfig.get_paths()["include"]]
    abi = "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(out_dir, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-fopenmp", "-DNDEBUG", abi] + inc + ["-c", s, "-o", o]
        if verbose:
            print("[ref host build]", os.path.basename(s), file=sys.stderr)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    for s, p in procs:
        _out, err = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("reference host source %s did not compile:\n%s" % (s, err[-4000:]))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", so] + objs + ["-L" + libdir, "-ltorch", "-ltorch_cpu", "-lc10", "-fopenmp",
                                                   "-Wl,-rpath," + libdir]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return so


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else ""))
