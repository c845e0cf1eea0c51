"""Compile the CUDA library in-tree for sm_100a with nvcc (cross-compiles without a GPU).

    python -m skywalker_b200.build [--force] [--verbose]

Produces skywalker_b200/libskywalker_b200.so (the C ABI of include/skywalker_b200.h) and
skywalker_b200/skywalker (the command-line driver).  Objects go to skywalker_b200/csrc/_obj/.
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libskywalker_b200.so")
CLI = os.path.join(PKG, "skywalker")

CU_SOURCES = ["skw_ctx.cu", "skw_alias_build.cu", "skw_walk.cu", "skw_walk_direct.cu", "skw_khop.cu", "skw_gen.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "--expt-relaxed-constexpr"]


def nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def host_cxx():
    # the system compiler carries libgomp; some images export CXX to a wrapper without it
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    cli = os.path.join(CSRC, "cli")
    if os.path.isdir(cli):
        hs += [os.path.join(cli, f) for f in os.listdir(cli) if f.endswith(".h")]
    hs.append(os.path.join(ROOT, "include", "skywalker_b200.h"))
    return hs


def _compile(src, force, verbose):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if not force and not _newer(obj, [path] + _headers()):
        return obj, ""
    cmd = [nvcc(), "-ccbin", host_cxx()] + ARCH + NVCC_FLAGS + ["-c", path, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, p.stdout, p.stderr))
    return obj, p.stderr if verbose else ""


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=min(8, len(CU_SOURCES))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), CU_SOURCES))
    objs = [o for o, _ in results]
    for _, log in results:
        if log:
            sys.stderr.write(log)
    if force or _newer(LIB, objs):
        cmd = [nvcc(), "-ccbin", host_cxx()] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode:
            raise RuntimeError("link failed:\n%s\n%s" % (p.stdout, p.stderr))
    cli_src = os.path.join(CSRC, "cli", "main.cpp")
    if os.path.exists(cli_src) and (force or _newer(CLI, [cli_src, LIB] + _headers())):
        cmd = [host_cxx(), "-O2", "-std=c++17", "-pthread", "-I", os.path.join(ROOT, "include"),
               "-I", "/usr/local/cuda/include", cli_src, "-o", CLI, "-L", PKG, "-lskywalker_b200",
               "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"]
        if os.path.exists("/usr/include/nccl.h"):
            cmd += ["-DSKW_HAVE_NCCL", "-lnccl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode:
            raise RuntimeError("CLI build failed:\n%s\n%s" % (p.stdout, p.stderr))
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
