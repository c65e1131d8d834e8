"""Builds the CUDA kernels of this package with nvcc for sm_100a, in the tree.

``ensure_library(name)`` compiles what is stale and returns the path of the
shared library; it is called at the first use of a kernel, so a fresh checkout
needs no separate build step.  Objects and libraries live beside the sources
(``_build/`` and ``lib*.so``); when the package folder is read-only they go to a
per-user folder under the system's temporary directory.  Staleness is decided by
a hash of the source, the shared header and the flags, not by time stamps.  A
line is printed to stderr for every file compiled.

Libraries:
  slb_core            every kernel that takes sizes at run time
  slb_attn_d<D>       the tensor-core attention kernels for head size D, built
                      when a model with that head size is first loaded
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--compiler-options", "-fPIC",
              "-Xcudafe", "--diag_suppress=177"]

CORE_SOURCES = ["elementwise.cu", "rope_cache.cu", "attention_generic.cu", "gemm_simt.cu",
                "sampling.cu", "gemm_tcgen05.cu"]
HEADERS = ["common.cuh", "no_alloc.h", "mma_util.cuh", "tma_util.cuh"]

_lock = threading.Lock()
_done: Dict[str, str] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[servelab_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("SLB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of servelab_b200 cannot be built "
                     "(set SLB_NVCC or put nvcc on PATH)")


def _out_root() -> str:
    if os.access(HERE, os.W_OK):
        return HERE
    root = os.path.join(tempfile.gettempdir(), f"servelab_b200_{os.getuid()}")
    os.makedirs(root, exist_ok=True)
    return root


def _digest(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        if os.path.isfile(p):
            with open(p, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _compile_one(nvcc: str, src: str, obj: str, flags: List[str], stamp: str, digest: str,
                 label: str) -> None:
    _say(f"compiling {label}")
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + flags + ["-I", HERE, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed for {label}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)


def ensure_library(name: str = "slb_core", sources: Optional[List[str]] = None,
                   defines: Optional[Dict[str, object]] = None) -> str:
    """Compile (if stale) and return the path of ``lib<name>.so``."""
    with _lock:
        if name in _done:
            return _done[name]
        sources = [s for s in (sources or CORE_SOURCES) if os.path.isfile(os.path.join(HERE, s))]
        flags = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
        root = _out_root()
        bdir = os.path.join(root, "_build", name)
        os.makedirs(bdir, exist_ok=True)
        lib = os.path.join(root, f"lib{name}.so")
        headers = [os.path.join(HERE, h) for h in HEADERS]
        flagstr = " ".join(ARCH_FLAGS + NVCC_FLAGS + flags)
        jobs, objs, digests = [], [], []
        nvcc = None
        for s in sources:
            src = os.path.join(HERE, s)
            obj = os.path.join(bdir, s + ".o")
            stamp = obj + ".sha"
            dg = _digest([src] + headers, flagstr)
            digests.append(dg)
            objs.append(obj)
            old = open(stamp).read() if os.path.isfile(stamp) and os.path.isfile(obj) else ""
            if old != dg:
                nvcc = nvcc or find_nvcc()
                jobs.append((nvcc, src, obj, flags, stamp, dg, f"{s} for {name}"))
        lib_digest = hashlib.sha256("".join(digests).encode()).hexdigest()
        lib_stamp = os.path.join(bdir, "lib.sha")
        lib_old = open(lib_stamp).read() if os.path.isfile(lib_stamp) and os.path.isfile(lib) else ""
        if jobs:
            _say(f"building lib{name}.so: {len(jobs)} of {len(sources)} files to compile "
                 f"(first use; later starts reuse them)")
            with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
                for f in [ex.submit(_compile_one, *j) for j in jobs]:
                    f.result()
        if jobs or lib_old != lib_digest:
            nvcc = nvcc or find_nvcc()
            tmp = lib + f".{os.getpid()}.tmp"
            cmd = [nvcc] + ARCH_FLAGS + ["-shared", "--cudart", "static", "-o", tmp] + objs
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"linking lib{name}.so failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, lib)
            with open(lib_stamp, "w") as f:
                f.write(lib_digest)
            _say(f"built {lib}")
        _done[name] = lib
        return lib


def attention_library(head_dim: int) -> str:
    """The tensor-core attention kernels specialised for one head size."""
    return ensure_library(f"slb_attn_d{head_dim}", ["attention_mma.cu", "attention_tc.cu", "attention_decode.cu"],
                          {"SLB_HEAD_DIM": head_dim})


def build_all(head_dims=(16, 32, 64, 128)) -> List[str]:
    libs = [ensure_library()]
    if os.path.isfile(os.path.join(HERE, "attention_mma.cu")):
        libs += [attention_library(d) for d in head_dims]
    return libs


if __name__ == "__main__":
    for p in build_all():
        print(p)
