"""Compile-once loader for generated functor modules.

A generated kernel is a small CUDA translation unit that includes the hand-written
templates (``csrc/ixb/gen.cuh``) and defines one functor ``Body`` plus an ``extern "C"``
launcher.  It is compiled with nvcc for sm_100a the first time it is seen, cached on disk
by content hash and called through ctypes.  This replaces ``NPUCachingAutotuner.precompile``
/ ``_precompile_config`` and the launcher closure they build
(``inductor_x/npu_triton_heuristics.py:53-266``), and ``cached_autotune``'s on-disk cache
(``:302-435``).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import subprocess
import threading
import time

import torch

from .. import config

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
_NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
               "-Xcompiler", "-fPIC", "-shared", "-Xcudafe", "--diag_suppress=177"]
_lock = threading.Lock()
_loaded: dict = {}


class GeneratedKernel:
    """Callable handle of one compiled functor module."""

    def __init__(self, key: str, path: str, meta: dict):
        self.key = key
        self.path = path
        self.meta = dict(meta)
        self.lib = ctypes.CDLL(path)
        self.fn = self.lib.ixb_gen_launch
        self.fn.restype = ctypes.c_int
        self.fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_longlong),
                            ctypes.c_void_p]
        self.launches = 0

    def run(self, *args, stream=None):
        ptrs, ints = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                ptrs.append(a.data_ptr())
            else:
                ints.append(int(a))
        if config.dry_run:
            return
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        pa = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
        ia = (ctypes.c_longlong * max(len(ints), 1))(*ints)
        if config.profile_bandwidth:
            return self._run_profiled(pa, ia, stream, args)
        rc = self.fn(pa, ia, stream)
        self.launches += 1
        if rc != 0:
            raise RuntimeError(f"generated kernel {self.meta.get('name', self.key)} failed to launch: "
                               f"cudaError {rc}")

    def _run_profiled(self, pa, ia, stream, args):
        """ms / GB / GB/s per launch, from the bytes of the tensor arguments
        (inductor_x/npu_triton_heuristics.py:274-299)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = self.fn(pa, ia, stream)
        e1.record()
        e1.synchronize()
        if rc != 0:
            raise RuntimeError(f"generated kernel failed to launch: cudaError {rc}")
        ms = e0.elapsed_time(e1)
        gb = sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor)) / 1e9
        print(f"{self.meta.get('name', self.key)}: {ms:.3f}ms    {gb:.3f}GB    {gb / (ms / 1e3):.2f}GB/s")


_headers_digest = None


def _template_digest() -> bytes:
    """Digest of the template headers a generated module includes: editing a header must
    not resurrect modules compiled against the old one from the on-disk cache."""
    global _headers_digest
    if _headers_digest is None:
        h = hashlib.sha256()
        inc = os.path.join(_CSRC, "ixb")
        for name in sorted(os.listdir(inc)):
            if name.endswith((".cuh", ".h")):
                with open(os.path.join(inc, name), "rb") as f:
                    h.update(name.encode() + b"\0" + f.read())
        _headers_digest = h.digest()
    return _headers_digest


def source_key(src: str) -> str:
    return hashlib.sha256(_template_digest() + src.encode()).hexdigest()[:24]


def compile_source(src: str, verbose: bool = False) -> str:
    """Compile ``src`` into the cache directory (if not already there); returns the .so path."""
    key = source_key(src)
    os.makedirs(config.cache_dir, exist_ok=True)
    so = os.path.join(config.cache_dir, f"ixbgen_{key}.so")
    if os.path.exists(so):
        return so
    cu = os.path.join(config.cache_dir, f"ixbgen_{key}.cu")
    with open(cu, "w") as f:
        f.write(src)
    tmp = f"{so}.{os.getpid()}.tmp"
    t0 = time.time()
    # A row module states how many CTAs per SM its registers are bounded for.  If ptxas had
    # to spill under that bound the module is rebuilt with a looser one.
    m = re.search(r"#define IXB_GEN_MIN_CTAS (\d+)", src)
    bounds = [None]
    if m:
        n = int(m.group(1))
        bounds = [n] + [b for b in (6, 4, 3, 2, 1) if b < n]
    for bound in bounds:
        extra = [] if bound is None else [f"-DIXB_GEN_MIN_CTAS={bound}"]
        cmd = ["nvcc", *_NVCC_FLAGS, "-Xptxas", "-v", *extra, "-I", _CSRC, "-o", tmp, cu]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for generated kernel {cu}:\n{proc.stderr[-4000:]}")
        spills = [int(x) for x in re.findall(r"(\d+) bytes spill stores", proc.stderr)]
        if bound in (None, 1) or not any(spills):
            break
    os.replace(tmp, so)
    if verbose:
        print(f"compiled {so} in {time.time() - t0:.1f}s")
    return so


def load_kernel(src: str, **meta) -> GeneratedKernel:
    """Entry point named in generated wrapper code."""
    key = source_key(src)
    with _lock:
        k = _loaded.get(key)
        if k is None:
            k = GeneratedKernel(key, compile_source(src), meta)
            _loaded[key] = k
    return k
