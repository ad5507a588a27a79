"""Build the CUDA libraries (sm_100a) in-tree with nvcc.  No torch dependency: each library is a plain C-ABI shared
object.  Two targets, built independently so that a model only compiles what it runs:
    core  lib/libao_b200.so      csrc/*.cu      weight-only quantized linears, the Llama decode kernels (include/ao_b200.h)
    lm    lib/libao_b200_lm.so   csrc/lm/*.cu   sequence-model mechanisms on an fp32 residual stream (include/ao_b200_lm.h)
Usage: python -m torchao_fork_b200.build [core|lm|all] [-v] [-f]"""
import fcntl
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libao_b200.so")
LIB_LM = os.path.join(LIBDIR, "libao_b200_lm.so")
TARGETS = {"core": (CSRC, LIB), "lm": (os.path.join(CSRC, "lm"), LIB_LM)}

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-DAO_B200_BUILD",
]


def sources(target="core"):
    return sorted(f for f in os.listdir(TARGETS[target][0]) if f.endswith(".cu"))


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, target="core"):
    """Compiles what is stale of `target` ("core", "lm" or "all") and links it; returns the library's path (the core
    library's for "all").  Safe to call from several processes at once (a lock file serialises them)."""
    if target == "all":
        build(verbose, force, "lm")
        return build(verbose, force, "core")
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    with open(os.path.join(OBJDIR, f".{target}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        return _build_locked(verbose, force, target)


def _build_locked(verbose, force, target):
    src_dir, lib_path = TARGETS[target]
    headers = [os.path.join(src_dir, f) for f in os.listdir(src_dir) if f.endswith((".cuh", ".h"))]
    inc = os.path.join(HERE, "..", "include")
    headers += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    jobs = []
    objs = []
    for src in sources(target):
        s = os.path.join(src_dir, src)
        o = os.path.join(OBJDIR, ("" if target == "core" else target + "_") + src[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [NVCC, *FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=8) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed: " + " ".join(cmd))
    if jobs or force or _stale(lib_path, objs):
        tmp = lib_path + f".{os.getpid()}.tmp"
        cmd = [NVCC, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
        os.replace(tmp, lib_path)
    return lib_path


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if not a.startswith("-")] or ["all"]
    for name in names:
        print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, target=name))
