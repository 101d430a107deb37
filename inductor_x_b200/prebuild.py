"""Prepare generated modules on a machine without a GPU.

``torch.compile`` builds a kernel the first time a graph runs, with nvcc, on the machine that
runs it.  Where that machine should not spend its first minutes compiling (a benchmark box, a
serving start-up), the same modules can be produced ahead of time: the graphs are compiled
here for CPU tensors of the same shapes with the backend in dry-run mode, which emits and
builds exactly the source the GPU run will ask for (plus the launch-shape candidates the
first call measures) into ``config.cache_dir``.  Nothing is launched.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Iterable, Sequence, Tuple


@contextlib.contextmanager
def _dry_cpu_backend(candidates: bool):
    import torch
    from torch._inductor.codegen.common import (get_scheduling_for_device, get_wrapper_codegen_for_device,
                                                init_backend_registration, register_backend_for_device)

    from . import config
    from .codegen import B200Scheduling, B200WrapperCodeGen

    init_backend_registration()
    old = (get_scheduling_for_device("cpu"), get_wrapper_codegen_for_device("cpu"))
    saved = (config.dry_run, config.prebuild_candidates, torch._inductor.config.fx_graph_cache,
             torch._inductor.config.cpu_backend)
    config.dry_run, config.prebuild_candidates = True, candidates
    torch._inductor.config.fx_graph_cache = False
    # the op handlers ask which backend family is current (it decides how the result type of a
    # masked sub-block is found): answer as on the GPU
    torch._inductor.config.cpu_backend = "triton"
    register_backend_for_device("cpu", B200Scheduling, B200WrapperCodeGen)
    try:
        yield
    finally:
        register_backend_for_device("cpu", *old)
        (config.dry_run, config.prebuild_candidates, torch._inductor.config.fx_graph_cache,
         torch._inductor.config.cpu_backend) = saved


def prebuild(graphs: Iterable[Tuple[str, Callable, Sequence]], candidates: bool = True, verbose: bool = True):
    """Compile each ``(name, fn, example CPU tensors)``; returns {name: number of modules}."""
    import torch
    from torch._inductor.utils import run_and_get_code

    built = {}
    with _dry_cpu_backend(candidates):
        for name, fn, args in graphs:
            torch._dynamo.reset()
            _, code = run_and_get_code(torch.compile(fn), *args)
            built[name] = sum(c.count("ixb_load_kernel('''") for c in code)
            if verbose:
                print(f"prebuilt {name}: {built[name]} generated module(s)", flush=True)
    torch._dynamo.reset()
    return built
