"""Builds the CUDA sources of this folder into one shared library for sm_100a.

Plain `nvcc`, one object per source file (compiled in parallel), linked into
`_build/libmynah_slm_b200.so` beside the sources. The sources include no
PyTorch header, so a cold build takes seconds per file rather than minutes. A
stamp of the sources' contents and the flags decides whether anything has to
be rebuilt, so the library that travels with the tree is used as it is.

When the folder is not writable (a checkout that belongs to someone else) the
build goes to a per-user folder under the system's temporary directory.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libmynah_slm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]
# further flags for an experiment (e.g. -DMYNAH_PDL_LATE); they are part of the stamp, so a change rebuilds
NVCC_FLAGS += os.environ.get("MYNAH_NVCC_EXTRA", "").split()


class BuildError(RuntimeError):
    pass


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    inc = os.path.join(os.pardir, "include")
    return (sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))
            + sorted(os.path.join(inc, f) for f in os.listdir(os.path.join(HERE, inc)) if f.endswith(".h")))


def _stamp() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    local = os.path.join(HERE, "_build")
    if _writable(local):
        return local
    alt = os.path.join(tempfile.gettempdir(), f"mynah_slm_b200_build_{os.getuid()}")
    if _writable(alt):
        return alt
    raise BuildError(f"neither {local} nor {alt} is writable")


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of mynah_slm_b200 cannot be built")


def library_path(verbose: bool = False) -> str:
    """Path of an up-to-date library, building it first if need be."""
    out = build_dir()
    lib = os.path.join(out, LIB_NAME)
    stamp_file = os.path.join(out, "stamp")
    stamp = _stamp()
    if os.path.isfile(lib) and os.path.isfile(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    _build(out, lib, verbose)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return lib


def _say(msg: str) -> None:
    if os.environ.get("MYNAH_QUIET", "0") in ("", "0"):          # the C interface sets it: that library never prints
        print(f"[mynah_slm_b200] {msg}", file=sys.stderr, flush=True)


def _build(out: str, lib: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    _say(f"building {len(srcs)} CUDA sources for sm_100a into {out} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f}s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()

    def compile_one(src: str) -> str:
        obj = os.path.join(out, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr:
            _say(f"{src}:\n{r.stderr}")
        _say(f"compiled {src} ({time.time() - t0:.0f}s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
    finally:
        done.set()
    _say(f"built {LIB_NAME} in {time.time() - t0:.0f}s")


# ---------------------------------------------------------------- the host-side runtime (no CUDA)
HOST_LIB_NAME = "libmynah_slm_b200_host.so"
HOST_SOURCES = [os.path.join("host", "runtime.cpp")]
HOST_HEADERS = [os.path.join(os.pardir, "include", "mynah_slm_b200_host.h"),
                os.path.join(os.pardir, "include", "mynah_random_normal.h")]
# -ffp-contract=off: the random-weights arithmetic must round every operation on its own, as the device does
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-ffp-contract=off", "-pthread"]


def _find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++): the host runtime of "
                     "mynah_slm_b200 cannot be built")


def host_library_path() -> str:
    """Path of the up-to-date host runtime (page books, step packing), building it first if need be.
    It needs a C++ compiler only, no GPU and no nvcc."""
    out = build_dir()
    lib = os.path.join(out, HOST_LIB_NAME)
    stamp_file = os.path.join(out, "host_stamp")
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    for f in HOST_SOURCES + HOST_HEADERS:
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    stamp = h.hexdigest()
    if os.path.isfile(lib) and os.path.isfile(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [_find_cxx(), *HOST_FLAGS, "-o", tmp, *[os.path.join(HERE, f) for f in HOST_SOURCES]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"compiling the host runtime failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return lib


# ---------------------------------------------------------------- the C interface (hosts a Python interpreter)
CAPI_LIB_NAME = "libmynah_slm_b200_capi.so"
CAPI_SOURCES = [os.path.join("host", "capi.c")]
CAPI_HEADERS = [os.path.join(os.pardir, "include", "mynah_slm_b200.h"), os.path.join(os.pardir, "include", "mynah_slm_b200_host.h")]


def capi_library_path() -> str:
    """Path of the up-to-date library behind `include/mynah_slm_b200.h`, building it first if need be. It links
    the Python library of the interpreter that builds it and remembers that interpreter and this checkout as the
    defaults it starts with (MYNAH_PYTHON and MYNAH_SLM_B200_ROOT override them)."""
    import sysconfig
    out = build_dir()
    lib = os.path.join(out, CAPI_LIB_NAME)
    stamp_file = os.path.join(out, "capi_stamp")
    root = os.path.dirname(os.path.dirname(HERE))
    inc, libdir = sysconfig.get_paths()["include"], sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    if not os.path.isfile(os.path.join(inc, "Python.h")):
        raise BuildError(f"Python.h is not under {inc}: the C interface of mynah_slm_b200 needs Python's headers")
    flags = ["-O2", "-std=c11", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", f"-I{inc}",
             f'-DMYNAH_DEFAULT_PYTHON="{sys.executable}"', f'-DMYNAH_DEFAULT_ROOT="{root}"']
    link = [f"-Wl,-soname,{CAPI_LIB_NAME}"] + ([f"-L{libdir}", f"-Wl,-rpath,{libdir}"] if libdir else []) + [f"-lpython{ver}"]
    h = hashlib.sha256(" ".join(flags + link).encode())
    for f in CAPI_SOURCES + CAPI_HEADERS:
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    stamp = h.hexdigest()
    if os.path.isfile(lib) and os.path.isfile(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    cc = next((c for c in (os.environ.get("CC"), shutil.which("gcc"), shutil.which("cc"), shutil.which("clang")) if c and os.path.isfile(c)), None)
    if cc is None:
        raise BuildError("no C compiler found (looked at $CC, gcc, cc, clang): the C interface cannot be built")
    tmp = lib + f".tmp{os.getpid()}"
    r = subprocess.run([cc, *flags, "-o", tmp, *[os.path.join(HERE, f) for f in CAPI_SOURCES], *link], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"compiling the C interface failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return lib


if __name__ == "__main__":
    print(host_library_path())
    print(capi_library_path())
    print(library_path(verbose="-v" in sys.argv))
