"""Scheduling for the B200 backend: one fused node group -> one template instantiation.

Counterpart of ``NPUTritonScheduling`` (``inductor_x/codegen/schduling.py:24-163``).  The
reference overrides ``codegen_node_schedule`` to un-flatten the indexing of every node into
true axes before picking split/tiling axes (``decide_codegen_dims_in_kernel``); here the
stock SIMD flow is kept and the un-flattening questions are answered per access by
``codegen/ir.py`` while the kernel is emitted.  Tiling is always the flat
``(numel, rnumel)`` pair, as in the reference's ``select_tiling`` patch
(``inductor_x/codegen/triton.py:175-177``).
"""
from __future__ import annotations

import sympy
from torch._inductor.codegen.common import BackendFeature
from torch._inductor.codegen.simd import SIMDScheduling
from torch._inductor.utils import get_kernel_metadata
from torch._inductor.virtualized import V
from torch.utils._ordered_set import OrderedSet

from .kernel import B200Kernel

HEADER = "from inductor_x_b200.codegen.jit import load_kernel as ixb_load_kernel"


class B200Scheduling(SIMDScheduling):
    kernel_type = B200Kernel  # type: ignore[assignment]

    def __init__(self, scheduler) -> None:
        super().__init__(scheduler)
        wrapper = V.graph.wrapper_code
        if wrapper is not None:
            wrapper.header.splice(HEADER)

    @classmethod
    def get_backend_features(cls, device):
        # no tuple reductions: var_mean is lowered to the two-pass form, as the reference
        # does (inductor_x/lowering.py:270-325); scans only in the form the lowering lets
        # through (a sum along a stride-1 row held on chip); no sorts / foreach
        return OrderedSet([BackendFeature.INPLACE_BUFFERS, BackendFeature.REDUCE_TO_SINGLE_ELEMENT,
                           BackendFeature.SCAN])

    @classmethod
    def get_tiling_and_scores(cls, node_schedule, numel, reduction_numel=sympy.S.One,
                              coalesce_analysis=None):
        # always the flat (numel, rnumel) pair; pointwise groups carry rnumel == 1, which is
        # also what lets the scheduler fuse them into a reduction of the same rows
        return {"x": numel, "r0_": reduction_numel}, None

    @classmethod
    def select_tiling(cls, node_schedule, numel, reduction_numel=sympy.S.One, coalesce_analysis=None):
        return cls.get_tiling_and_scores(node_schedule, numel, reduction_numel)[0]

    def define_kernel(self, src_code, node_schedule, kernel) -> str:
        wrapper = V.graph.wrapper_code
        if src_code in wrapper.src_to_kernel:
            return wrapper.src_to_kernel[src_code]
        family = getattr(kernel, "mapping", "row" if kernel.is_row else "pointwise")
        kernel_name = f"ixb_{family}_{wrapper.next_kernel_suffix()}"
        wrapper.src_to_kernel[src_code] = kernel_name
        origins, detailed = get_kernel_metadata(node_schedule, wrapper)
        wrapper.define_kernel(kernel_name, src_code, f"{origins}\n{detailed}", gpu=False)
        return kernel_name

    def codegen_sync(self) -> None:
        V.graph.wrapper_code.writeline(V.graph.device_ops.synchronize())

    def can_fuse_multi_outputs_template(self, node1, node2) -> bool:
        return False
