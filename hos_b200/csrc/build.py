"""Compiling and loading the CUDA libraries.

Each library is a set of `.cu` files of this folder compiled by nvcc for sm_100a
into one shared object, loaded with ctypes; its functions are plain `extern "C"`.
A library is built at its first use and kept under `_build/` beside the sources
(or, where that folder cannot be written, under the temporary directory), named
by a hash of its sources, headers and flags, so that an edited source is rebuilt
and an unchanged one is not.  While nvcc runs, a line is printed to stderr for
every file and then every few seconds.  A library that cannot be built raises
`ExtensionMissingError`: there is no other path.

Libraries and what needs them:
  core        every model: embedding, norms, rotary + cache write, plain matrix
              product and plain attention (32-bit and bfloat16), sampling, the
              per-slot record
  attn_hdN    bfloat16 models with head_dim N: tensor-core attention for prompts
              and for decoding over the paged cache
  gemm_tc     bfloat16 models: the tcgen05/TMA matrix product
  gemm_skinny bfloat16 models: the matrix product for up to 16 rows (decoding)
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
from typing import Dict, List, Sequence, Tuple

from ..errors import ExtensionMissingError

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]

# library name -> (sources, extra flags)
_STATIC_LIBS: Dict[str, Tuple[List[str], List[str]]] = {
    "core": (["elementwise.cu", "gemm_plain.cu", "attention_plain.cu", "sampling.cu", "slot_state.cu"], []),
    "gemm_tc": (["gemm_tc.cu"], []),
    "gemm_skinny": (["gemm_skinny.cu"], []),
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def library_spec(name: str) -> Tuple[List[str], List[str]]:
    if name in _STATIC_LIBS:
        return _STATIC_LIBS[name]
    if name.startswith("attn_hd"):
        hd = int(name[len("attn_hd"):])
        return ["attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc.cu"], [f"-DHOS_HEAD_DIM={hd}"]
    raise ExtensionMissingError(f"no CUDA library named {name!r}")


def _nvcc() -> str:
    for cand in (os.environ.get("HOS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise ExtensionMissingError("nvcc was not found (looked at $HOS_NVCC, PATH and /usr/local/cuda/bin); "
                                "the CUDA kernels cannot be built and there is no other path")


def _flags(extra: Sequence[str]) -> List[str]:
    return ARCH_FLAGS + BASE_FLAGS + list(extra)


def _digest(sources: Sequence[str], extra: Sequence[str]) -> str:
    h = hashlib.sha1()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".cuh") or f.endswith(".h") or f in sources:
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(_flags(extra)).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[str]:
    dirs = [os.path.join(HERE, "_build")]
    dirs.append(os.path.join(tempfile.gettempdir(), f"hos_b200_build_{os.getuid()}"))
    return dirs


def _say(msg: str) -> None:
    print(f"[hos] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmd: List[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=HERE)
    done = threading.Event()

    def beat():
        while not done.wait(5.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f}s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise ExtensionMissingError(f"nvcc failed on {what}:\n{out.decode(errors='replace')[-4000:]}")


def _compile(name: str, path: str, verbose_ptxas: bool = False) -> None:
    sources, extra = library_spec(name)
    nvcc = _nvcc()
    workdir = tempfile.mkdtemp(prefix="hos_nvcc_", dir=os.path.dirname(path))
    try:
        objs = []

        def one(src: str) -> str:
            obj = os.path.join(workdir, src.replace(".cu", ".o"))
            _say(f"compiling {src} for sm_100a ({name})")
            cmd = [nvcc] + _flags(extra) + (["-Xptxas", "-v"] if verbose_ptxas else []) + \
                  ["-c", os.path.join(HERE, src), "-o", obj]
            _run_with_heartbeat(cmd, src)
            return obj
        with ThreadPoolExecutor(max_workers=min(4, len(sources))) as pool:
            objs = list(pool.map(one, sources))
        tmp_so = os.path.join(workdir, "lib.so")
        _run_with_heartbeat([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_so] + objs,
                            f"link {name}")
        os.replace(tmp_so, path)     # atomic: a concurrent builder sees all or nothing
        _say(f"built {os.path.basename(path)}")
        for old in os.listdir(os.path.dirname(path)):     # builds of earlier sources of this library
            if old.startswith(f"hos_{name}-") and old.endswith(".so") and old != os.path.basename(path):
                try:
                    os.remove(os.path.join(os.path.dirname(path), old))
                except OSError:
                    pass
    finally:
        shutil.rmtree(workdir, ignore_errors=True)


def library_path(name: str, build: bool = True) -> str:
    sources, extra = library_spec(name)
    fname = f"hos_{name}-{_digest(sources, extra)}.so"
    for d in _build_dirs():
        p = os.path.join(d, fname)
        if os.path.exists(p):
            return p
    if not build:
        raise ExtensionMissingError(f"CUDA library {fname} has not been built")
    last_err = None
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = tempfile.mkdtemp(prefix="w_", dir=d)
            os.rmdir(probe)
        except OSError as e:
            last_err = e
            continue
        p = os.path.join(d, fname)
        _compile(name, p)
        return p
    raise ExtensionMissingError(f"no writable folder to build {fname} in ({last_err})")


def load(name: str) -> ctypes.CDLL:
    """The loaded library, built first if need be.  Raises ExtensionMissingError."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = library_path(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionMissingError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def build_all(head_dims: Sequence[int] = (16, 32, 48, 64, 80, 128, 256)) -> List[str]:
    """Build every library (the attention library once per head size: the sizes of the Gemma-2 checkpoints, 128
    and 256, and the ones that the tests' small configurations have; any other multiple of 16 is built when a
    model with it is first loaded)."""
    names = list(_STATIC_LIBS) + [f"attn_hd{h}" for h in head_dims]
    return [library_path(n) for n in names]
