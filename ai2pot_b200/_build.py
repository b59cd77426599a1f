"""In-tree build of the native libraries (no JIT cache: the built files travel with the tree).

  ai2pot_b200/_lib/libai2pot_b200.so   CUDA kernels + C ABI, sm_100a only

Run ``python -m ai2pot_b200._build`` (or call build()). Needs nvcc; no GPU.
"""
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    objs = []
    procs = []
    for src in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
            log = open(obj + ".log", "w")
            procs.append((src, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), log, obj))
    for src, p, log, obj in procs:
        rc = p.wait()
        log.close()
        out = open(obj + ".log").read()
        if verbose or rc != 0:
            sys.stderr.write(out)
        if rc != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    lib = os.path.join(LIBDIR, "libai2pot_b200.so")
    if force or procs or _stale(lib, objs):
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", lib] + objs + ["-lcudart"])
    return lib


def build_bench(force=False):
    """libai2b_fma_peak.so: the FMA-pipe microbenchmark bench.py uses for its roofline denominator (not linked
    into the product library)."""
    src = os.path.join(CSRC, "bench", "fma_peak.cu")
    out = os.path.join(LIBDIR, "libai2b_fma_peak.so")
    if force or _stale(out, [src]):
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-shared", "-Xcompiler",
                               "-fPIC", "-o", out, src, "-lcudart"])
    return out


GLUE = {"libmtpr_bind.so": ["mtpr_bind.cpp"], "libnep_bind.so": ["nep_bind.cpp"], "libfvt_sr_op_bind.so": ["fvt_sr_op_bind.cpp"],
        "libfitutils_bind.so": ["fitutils_bind.cpp"]}


def build_glue(force=False, verbose=False):
    """Torch-op libraries with the reference's file names (what ai2pot.fromcc loads and what the
    LAMMPS interface links: -lmtpr_bind -lnep_bind). Plain g++ against the installed torch."""
    import torch
    from torch.utils import cpp_extension
    gdir = os.path.join(CSRC, "torch_glue")
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    headers = glob.glob(os.path.join(gdir, "*.h")) + glob.glob(os.path.join(gdir, "*.inc")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    procs, outs = [], []
    for lib, srcs in GLUE.items():
        out = os.path.join(LIBDIR, lib)
        outs.append(out)
        paths = [os.path.join(gdir, s) for s in srcs]
        if force or _stale(out, paths + headers + [os.path.join(LIBDIR, "libai2pot_b200.so")]):
            cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-w"] + inc + paths + \
                  ["-o", out, "-L" + LIBDIR, "-lai2pot_b200", "-L" + tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda",
                   "-lc10_cuda", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
            log = open(out + ".log", "w")
            procs.append((lib, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), log, out))
    for lib, p, log, out in procs:
        rc = p.wait()
        log.close()
        if rc != 0 or verbose:
            sys.stderr.write(open(out + ".log").read())
        if rc != 0:
            raise RuntimeError(f"g++ failed on {lib}")
    return outs


def install_python_modules():
    """Python modules the reference's loader expects to find beside the libraries: ``nblist`` (it does
    ``sys.path.append(lib_dir); import nblist``, ai2pot/fromcc/__init__.py:52-58)."""
    shutil.copyfile(os.path.join(HERE, "fromcc", "nblist_toplevel.py"), os.path.join(LIBDIR, "nblist.py"))


def build(force=False, verbose=False):
    lib = build_cuda(force, verbose)
    build_glue(force, verbose)
    build_bench(force)
    install_python_modules()
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
