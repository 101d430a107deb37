"""Decomposition-table edits of the B200 backend.

Surface kept from ``inductor_x/decomposition.py:18-47``
(``_register_npu_inductor_decompositons``).  The reference *deletes* the decompositions of
``gelu``, ``_log_softmax``, ``nll_loss_*`` and friends so that those ops reach vendor
kernels; that is exactly what stops it from fusing ``sum(gelu(x*w+b))`` into one kernel.
Here they are left in place - the pointwise and row templates instantiate the decomposed
bodies - and the three decompositions the reference adds are either correct in stock
Inductor already (``expm1``) or wrong in the reference and therefore not copied
(``erfc`` as ``1 - exp(x)``, ``:44-47``; ``scatter.src`` as a one-hot product, ``:27-37``).
The function exists so that code written against the reference's surface keeps working; it
only verifies the table is in the state the templates rely on.
"""
from __future__ import annotations

import torch
from torch._inductor.decomposition import decompositions

aten = torch.ops.aten

# ops whose decomposition the fused templates rely on (the reference removes these)
DECOMPOSITION_KEEP_OP = [aten.gelu, aten._log_softmax, aten._softmax, aten.native_layer_norm,
                         aten.silu]


def _register_b200_inductor_decompositions():
    """Check that the decompositions the templates fuse through are present; returns the
    list of (op, present) pairs for logging / tests.  No decomposition is deleted."""
    report = []
    for packet in DECOMPOSITION_KEEP_OP:
        for name in packet.overloads():
            op = getattr(packet, name)
            report.append((op, op in decompositions))
    return report
