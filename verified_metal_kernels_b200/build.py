"""Builds libvmk_b200.so from csrc/*.cu with nvcc for sm_100a, in-tree."""
import fcntl
import glob
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, os.environ.get("VMK_LIB_NAME", "libvmk_b200.so"))   # a debug build may use another name
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def deps():
    return sources() + sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(HERE, "..", "include", "vmk_b200.h")]


def fingerprint():
    """Hash of every source, header and flag that goes into the library.  File times are not used: a copy of
    the tree to another machine does not keep them."""
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + os.environ.get("VMK_EXTRA_NVCC_FLAGS", "").split()).encode())
    for d in deps():
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def needs_build():
    if not os.path.exists(LIB) or not os.path.exists(LIB + ".stamp"):
        return True
    with open(LIB + ".stamp") as f:
        return f.read().strip() != fingerprint()


def build(force=False, verbose=False):
    """Compile every .cu to an object and link the shared library.  Returns the library path.  Safe to call
    from several processes at once (one rank per GPU): a file lock lets one of them build, the library appears
    under its name only when complete, and the others then find it up to date."""
    if not force and not needs_build():
        return LIB
    with open(os.path.join(HERE, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or needs_build():
                _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


def _build_locked(verbose):
    nvcc = os.environ.get("NVCC", "nvcc")
    extra = os.environ.get("VMK_EXTRA_NVCC_FLAGS", "").split()      # e.g. -DVMK_TC_TIMING for device-side phase timers
    objdir = os.path.join(HERE, "build" + ("_" + os.path.basename(LIB) if extra else ""))
    os.makedirs(objdir, exist_ok=True)
    stamp = fingerprint()
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for cmd, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        objs.append(obj)
    tmp = LIB + ".tmp.%d" % os.getpid()
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", tmp] + objs + ["-lcudart"])
    os.replace(tmp, LIB)
    with open(LIB + ".stamp.tmp", "w") as f:
        f.write(stamp + "\n")
    os.replace(LIB + ".stamp.tmp", LIB + ".stamp")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
