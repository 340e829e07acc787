"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The reference builds one shared library ``TFFInfer`` with CMake for the arch of the
local GPU (CMakeLists.txt:1-118, cmake/detect_cuda_arch.cmake).  Here the target is
fixed (sm_100a) and the build is a few ``nvcc`` calls, so that a fresh checkout can
compile what it needs at its first call, as an ordinary user, without network.

The library goes to ``csrc/_build/`` inside the package when that is writable, else
to a per-user folder under the system's temporary directory.  A stamp records the
hash of the sources and flags; the library is rebuilt when they change.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libtffinfer_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def extra_flags_from_env() -> List[str]:
    """More flags for nvcc from TFFINFER_NVCC_FLAGS (for instance -DTFF_DEC_STAGES=2 to try another depth of
    the decode attention's ring); they enter the stamp, so changing them rebuilds the library."""
    return os.environ.get("TFFINFER_NVCC_FLAGS", "").split()


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise RuntimeError("nvcc not found (looked at CUDA_HOME, PATH and /usr/local/cuda/bin): "
                       "the CUDA kernels of tffinfer_b200 cannot be compiled")


def _source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + headers():
        h.update(f.encode())
        with open(os.path.join(CSRC_DIR, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra_flags_from_env()).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("TFFINFER_BUILD_DIR")
    if env and _writable_dir(env):
        return env
    intree = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(intree):
        return intree
    alt = os.path.join(tempfile.gettempdir(), f"tffinfer_b200_build_{os.getuid()}")
    if _writable_dir(alt):
        return alt
    raise RuntimeError(f"no writable folder for the kernel library (tried {intree} and {alt})")


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[tffinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library; compiles it first if needed."""
    bdir = build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "stamp.txt")
    want = _source_hash()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build:
        raise RuntimeError(f"{lib} is missing or out of date")
    compile_all(bdir, verbose=verbose)
    with open(stamp, "w") as f:
        f.write(want + "\n")
    return lib


def _heartbeat(stop: threading.Event, t0: float, verbose: bool, what: str) -> None:
    while not stop.wait(10.0):
        _say(f"still compiling {what} ... {time.time() - t0:.0f} s", verbose)


def compile_all(bdir: str, verbose: bool = True, extra_flags: Optional[List[str]] = None) -> str:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} into {bdir}", verbose)
    flags = ARCH_FLAGS + NVCC_FLAGS + extra_flags_from_env() + (extra_flags or [])
    stop = threading.Event()
    hb = threading.Thread(target=_heartbeat, args=(stop, t0, verbose, "kernels"), daemon=True)
    hb.start()

    def one(src: str) -> str:
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [nvcc] + flags + ["-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{p.stdout}")
        _say(f"  {src} done ({time.time() - t0:.0f} s)", verbose)
        return obj

    try:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            objs = list(ex.map(one, srcs))
        tmp = os.path.join(bdir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs + ["-lcudart"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{p.stdout}")
        os.replace(tmp, os.path.join(bdir, LIB_NAME))
    finally:
        stop.set()
    _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s", verbose)
    return os.path.join(bdir, LIB_NAME)


# ------------------------------------------------------------------ host runtime (no CUDA)
HOST_DIR = os.path.join(CSRC_DIR, "host")
HOST_LIB_NAME = "libtffinfer_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def find_cxx() -> str:
    for c in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        w = shutil.which(c) if c else None
        if w:
            return w
    raise RuntimeError("no C++ compiler found (looked at CXX, g++, c++, clang++): "
                       "the host runtime of tffinfer_b200 cannot be compiled")


def host_library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date host-runtime library (page pools, block tables, step packing; csrc/host/),
    compiled with the host compiler alone, so it also builds where there is no CUDA toolkit."""
    bdir = build_dir()
    lib = os.path.join(bdir, HOST_LIB_NAME)
    stamp = os.path.join(bdir, "host_stamp.txt")
    files = sorted(f for f in os.listdir(HOST_DIR) if f.endswith((".cpp", ".h")))
    h = hashlib.sha256()
    for f in files:
        h.update(f.encode())
        with open(os.path.join(HOST_DIR, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(HOST_FLAGS).encode())
    want = h.hexdigest()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build:
        raise RuntimeError(f"{lib} is missing or out of date")
    cxx = find_cxx()
    tmp = os.path.join(bdir, f".{HOST_LIB_NAME}.{os.getpid()}")
    srcs = [os.path.join(HOST_DIR, f) for f in files if f.endswith(".cpp")]
    p = subprocess.run([cxx] + HOST_FLAGS + ["-I", HOST_DIR] + srcs + ["-o", tmp],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"compiling the host runtime failed:\n{p.stdout}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(want + "\n")
    _say(f"built {HOST_LIB_NAME}", verbose)
    return lib


if __name__ == "__main__":
    print(host_library_path(build=True, verbose=True))
    print(library_path(build=True, verbose=True))
