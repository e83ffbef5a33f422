"""Compiling and loading the CUDA libraries of the package.

Each library is a set of ``.cu`` files of this folder compiled by ``nvcc`` for
sm_100a into one shared object with plain C entry points, loaded with
``ctypes``.  A library is compiled the first time something needs it, so a run
in float32 never builds the bfloat16 kernels and the other way round.  The
object's file name carries a hash of its sources and flags: an edited source
gets a new file, a fresh checkout builds once, and a built file that travels
with the tree is used as it is.

Built files go to ``_build/`` beside the sources; where that folder cannot be
written they go to a per-user folder under the system's temporary directory.
While ``nvcc`` runs, a line is printed to standard error every few seconds.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden"]

_CORE_SOURCES = ["elementwise.cu", "qk_rope_store.cu", "attention_generic.cu", "gemm_simt.cu", "sampling.cu",
                 "sample_select.cu", "attention_mma.cu", "attention_tcgen05.cu",
                 "attention_pair_tcgen05.cu", "attention_decode.cu"]

# name -> (sources, extra flags, extra link flags)
LIBRARIES: Dict[str, dict] = {
    "core_f32": {"sources": _CORE_SOURCES, "flags": ["-DIB_ACT_BF16=0"], "link": []},
    "core_bf16": {"sources": _CORE_SOURCES, "flags": ["-DIB_ACT_BF16=1"], "link": []},
    "gemm_bf16": {"sources": ["gemm_tcgen05.cu", "gemm_chain.cu"], "flags": ["-DIB_ACT_BF16=1"], "link": []},
    # host code only (the cache's book-keeping and the step description): the C++ compiler alone builds it
    "host_runtime": {"sources": ["host_runtime.cpp"], "flags": [], "link": [], "host": True},
}

HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return shutil.which(cand) or cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); the host runtime of "
                     "inferrs_b200 cannot be built and there is no other implementation")


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the CUDA kernels of inferrs_b200 cannot be built and there is no other implementation")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def library_hash(name: str) -> str:
    lib = LIBRARIES[name]
    h = hashlib.sha256()
    for f in list(lib["sources"]) + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    flags = HOST_FLAGS if lib.get("host") else ARCH_FLAGS + COMMON_FLAGS
    h.update(" ".join(flags + lib["flags"] + lib["link"]).encode())
    return h.hexdigest()[:16]


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


def build_dirs() -> List[str]:
    """Folders where a built library may be found; the first writable one receives new builds."""
    dirs = [os.path.join(HERE, "_build")]
    if os.environ.get("INFERRS_B200_BUILD_DIR"):
        dirs.insert(0, os.environ["INFERRS_B200_BUILD_DIR"])
    dirs.append(os.path.join(tempfile.gettempdir(), f"inferrs_b200_build_{os.getuid()}"))
    return dirs


def library_path(name: str) -> Optional[str]:
    fname = f"{name}.{library_hash(name)}.so"
    for d in build_dirs():
        p = os.path.join(d, fname)
        if os.path.isfile(p):
            return p
    return None


def _run_with_heartbeat(cmds: Sequence[Sequence[str]], what: str, verbose_flags: bool):
    """Run the commands in parallel; print a line every few seconds until all are done."""
    start = time.time()
    done = threading.Event()

    def beat():
        while not done.wait(5.0):
            print(f"[inferrs_b200] still compiling {what} ({time.time() - start:.0f} s)", file=sys.stderr, flush=True)

    t = threading.Thread(target=beat, daemon=True)
    t.start()

    def run(cmd):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return cmd, r.returncode, r.stdout

    try:
        with ThreadPoolExecutor(max_workers=min(len(cmds), os.cpu_count() or 2)) as ex:
            results = list(ex.map(run, cmds))
    finally:
        done.set()
    for cmd, rc, out in results:
        if rc != 0:
            raise BuildError(f"the compiler failed ({rc}) for: {' '.join(cmd)}\n{out}")
        if verbose_flags and out.strip():
            print(out, file=sys.stderr, flush=True)


def build_library(name: str, force: bool = False, ptxas_verbose: bool = False) -> str:
    """Compile library ``name`` if it is not there yet; return the path of the shared object."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'; known: {sorted(LIBRARIES)}")
    if not force:
        p = library_path(name)
        if p:
            return p
    lib = LIBRARIES[name]
    host = bool(lib.get("host"))
    compiler = find_cxx() if host else find_nvcc()
    out_dir = next((d for d in build_dirs() if _writable_dir(d)), None)
    if out_dir is None:
        raise BuildError(f"no writable folder for built kernels among {build_dirs()}")
    tag = library_hash(name)
    what = "host library" if host else "kernel library"
    print(f"[inferrs_b200] compiling {what} {name}{'' if host else ' for sm_100a'} ({len(lib['sources'])} files) "
          f"into {out_dir}", file=sys.stderr, flush=True)
    t0 = time.time()
    objs, cmds = [], []
    for src in lib["sources"]:
        obj = os.path.join(out_dir, f"{name}.{tag}.{os.path.splitext(src)[0]}.o")
        objs.append(obj)
        flags = HOST_FLAGS if host else ARCH_FLAGS + COMMON_FLAGS
        cmd = [compiler] + flags + lib["flags"] + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        if ptxas_verbose and not host:
            cmd += ["-Xptxas", "-v"]
        cmds.append(cmd)
    _run_with_heartbeat(cmds, name, ptxas_verbose)
    final = os.path.join(out_dir, f"{name}.{tag}.so")
    tmp = final + f".tmp{os.getpid()}"
    link = [compiler, "-shared"] + ([] if host else ARCH_FLAGS) + ["-o", tmp] + objs + lib["link"]
    _run_with_heartbeat([link], f"{name} (link)", False)
    os.replace(tmp, final)
    for old in os.listdir(out_dir):   # builds of earlier source states of this library
        if old.startswith(name + ".") and old.endswith(".so") and old != os.path.basename(final):
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    print(f"[inferrs_b200] built {os.path.basename(final)} in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return final


_LOADED: Dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, built first if need be.  Raises BuildError; there is no other path."""
    with _LOCK:
        if name not in _LOADED:
            _LOADED[name] = ctypes.CDLL(build_library(name))
        return _LOADED[name]


def build_all(ptxas_verbose: bool = False) -> List[str]:
    return [build_library(n, ptxas_verbose=ptxas_verbose) for n in LIBRARIES]


if __name__ == "__main__":
    for p in build_all(ptxas_verbose="-v" in sys.argv):
        print(p)
