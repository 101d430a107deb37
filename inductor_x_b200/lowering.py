"""Lowering policy of the B200 backend.

Surface kept from ``inductor_x/lowering.py``: ``make_reduction`` (tags every realised
reduction with the axes it keeps / reduces, ``:16-45``), ``_init_set`` (``:150-171``) and
``_register_b200_inductor_fallbacks`` (the reference's ``_register_npu_inductor_fallbacks``,
``:173-339``).

What changed underneath.  The reference whitelists ~50 aten ops (``GENERATE_LIST``,
``:80-148``) and turns *everything else* into an extern call, so e.g. ``gelu``, ``sigmoid``,
``pow``, ``sin/cos`` and ``index_select`` break fusion.  Here the templates instantiate any
pointwise / reduction / indexing body, so the policy is inverted: only the op families no
template exists for (sorts, random numbers, scatter with a reduction other than add, and every
scan except a ``cumsum`` / ``cumprod`` along the last axis, which the row template scans on chip)
are forced to extern kernels; accumulating scatters (``index_put(accumulate=True)``,
``scatter_add``, ``index_add``) are generated with atomic adds.  The reference's special lowerings are not carried over where they encode
bugs or NPU workarounds: ``sum_`` always returning fp32 (``:204-215``), the hard-coded
``[32768, 2]`` fallback (``:211-212``), ``embedding`` ignoring ``padding_idx``
(``:327-330``).  fp32 accumulation for half inputs and the two-pass variance
(``var_mean_helper_``, ``:270-325``) are what stock Inductor already does for a backend
without tuple reductions, which is how ``B200Scheduling`` declares itself.
"""
from __future__ import annotations

import torch
from torch._inductor import ir, lowering
from torch._inductor.lowering import (_make_reduction_inner, _validate_reduction_axis, fallbacks,
                                      lowerings, make_fallback)

aten = torch.ops.aten
prims = torch.ops.prims

# op families without a B200 template: they stay extern (ATen) kernels
FALLBACK_LIST = [
    aten.cummax, aten.cummin, aten.logcumsumexp,
    aten.sort, aten.topk, aten.scatter_reduce, aten.bernoulli, aten.rand, aten.randn, aten.randint, aten.randperm,
    aten.native_dropout, aten.multinomial, aten.bucketize, aten.searchsorted, aten.histc,
]


def _special_function_ops():
    """The special functions Inductor's Triton and C++ backends carry their own
    implementations of (Bessel and gamma families, orthogonal polynomials, ``digamma``,
    ``zeta``, ``ndtri`` ...): no template implements them, so they stay extern kernels."""
    from torch._inductor.codegen.common import pointwise_overrides_data

    out = []
    for name, data in pointwise_overrides_data.items():
        if name in ("fma", "mul_rn"):
            continue
        for ns in (aten, prims):
            op = getattr(ns, data.name, None)
            if op is not None:
                out.append(op)
    out.append(aten.frexp)
    return out


def make_reduction(reduction_type: str, override_return_dtype=None):
    """``Reduction.create`` wrapper that records which axes a reduction keeps and reduces
    on the IR node (``kept_idx`` / ``reduced_idx``) and realises it, as
    ``inductor_x/lowering.py:16-45`` does; the kernel emitter reads the tags to tell inner
    from outer reductions."""

    def inner(x, axis=None, keepdims=False, *, dtype=None):
        kwargs = _make_reduction_inner(x, axis=axis, keepdims=keepdims, dtype=dtype,
                                       override_return_dtype=override_return_dtype)
        result = ir.Reduction.create(reduction_type=reduction_type, input_node=x, **kwargs)
        data = getattr(getattr(result, "data", None), "data", None)
        if isinstance(data, ir.Reduction):
            size = x.get_size()
            axes = set(_validate_reduction_axis(x, axis))
            # IR nodes are frozen dataclasses: the tags are set past the freeze
            object.__setattr__(data, "kept_idx", [i for i in range(len(size)) if i not in axes])
            object.__setattr__(data, "reduced_idx", [i for i in range(len(size)) if i in axes])
            result.realize()
        return result

    return inner


def _init_set(input_list, output_set):
    """Expand OpOverloadPackets into their overloads (``inductor_x/lowering.py:150-171``)."""
    for fn in input_list:
        output_set.add(fn)
        if isinstance(fn, torch._ops.OpOverloadPacket):
            for overload in fn.overloads():
                other = getattr(fn, overload)
                output_set.add(other)


#: longest row a scan keeps on chip (elements); longer rows stay with the extern kernel
MAX_SCAN_ROW = 16384


def _row_scan_ok(x, axis, dtype) -> bool:
    """cumsum / cumprod cases the row template scans: a floating sum (fp32 accumulation) or an exact
    64-bit integer sum along the last axis of a row that a team holds on chip.  Everything else
    - other axes (the MoE gating graph scans along the token axis), a requested output dtype
    other than the natural one, very long or dynamic rows - stays an extern kernel, which is
    all the reference does for cumsum (``inductor_x/lowering.py:235-245``)."""
    size = x.get_size()
    if len(size) == 0:
        return False
    if x.get_dtype() in (torch.float32, torch.float16, torch.bfloat16):
        if dtype is not None and dtype != x.get_dtype():
            return False
    elif x.get_dtype() in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        if dtype not in (None, torch.int64):      # integer rows are summed exactly in 64 bits
            return False
    else:
        return False
    if axis is None or axis % len(size) != len(size) - 1:
        return False
    try:
        n = int(size[-1])
    except (TypeError, ValueError):
        return False
    return 2 <= n <= MAX_SCAN_ROW


def _install_scan_lowerings():
    """Stock scan lowering for the supported form of cumsum / cumprod, extern kernel otherwise."""
    for op in (aten.cumsum.default, aten.cumprod.default):
        stock = lowerings.get(op)
        if stock is None or getattr(stock, "_ixb_guarded", False):
            continue
        extern = lowering.fallback_handler(op, add_to_fallback_set=False)

        def guarded(x, axis=None, *, dim=None, dtype=None, _stock=stock, _extern=extern):
            axis = dim if axis is None else axis      # aten names the argument `dim`
            if _row_scan_ok(x, axis, dtype):
                return _stock(x, axis, dtype=dtype)
            return _extern(x, axis, dtype=dtype)

        guarded._ixb_guarded = True
        lowerings[op] = guarded
    # scans with other operators (running maximum / minimum with their indices, log-sum-exp):
    # their stock lowerings build a Scan node whenever the backend declares scans, so they are
    # pinned to the extern kernel here
    for op in (aten.logcumsumexp.default, aten.cummax.default, aten.cummin.default):
        stock = lowerings.get(op)
        if stock is None or getattr(stock, "_ixb_guarded", False):
            continue
        extern = lowering.fallback_handler(op, add_to_fallback_set=False)
        extern._ixb_guarded = True
        lowerings[op] = extern


def _register_b200_inductor_fallbacks():
    """Force the op families in ``FALLBACK_LIST`` to extern kernels.  Returns the overloads
    that were switched."""
    _install_scan_lowerings()
    targets = set()
    _init_set(FALLBACK_LIST + _special_function_ops(), targets)
    switched = []
    for op in targets:
        if isinstance(op, torch._ops.OpOverloadPacket):
            continue
        if op in lowerings and op not in fallbacks:
            try:
                del lowerings[op]
                make_fallback(op, warn=False)
                switched.append(op)
            except Exception:
                pass
    return switched
