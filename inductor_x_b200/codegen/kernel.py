"""Template instantiator: turns one fused node group into a CUDA functor body.

This is the replacement for the reference's Triton emitter ``NPUIndexTritonKernel``
(``inductor_x/codegen/triton.py:345-1789``).  Where that class prints an Ascend-flavoured
Triton kernel (range-tree entries with ``loop1/loop2`` tile loops, ``_prime`` index
variables, ``.permute(1,0)``), this one prints a small ``Body`` struct whose single method is
straight-line C++ over per-thread vector values, and instantiates one of the hand-written
templates of ``csrc/ixb/gen.cuh`` with it:

* no reduction            -> ``pointwise_gen_kernel``  (``tile(xbase, nvalid)``)
* reduction that fits     -> ``row_gen_kernel``        (``row(ctx, xindex)``), the row lives
                             in the registers of a team; chained reductions with pointwise
                             stages between them stay in one kernel.

Loads and stores are classified by ``codegen/ir.py``: contiguous along the thread's vector
(or along the reduced row) -> 128-bit access, anything else -> per-element gather/scatter.
"""
from __future__ import annotations

import contextlib
from typing import Any, Optional

import sympy
import torch
from torch._inductor import config as inductor_config
from torch._inductor.codegen.common import (CSEVariable, DeferredLine, IndentedBuffer, SizeArg,
                                            TensorArg)
from torch._inductor.codegen.simd import IterationRangesEntry, SIMDKernel
from torch._inductor.utils import sympy_subs
from torch._inductor.virtualized import V
from torch.utils._sympy.printers import PythonPrinter

from .. import config as ixb_config
from . import ir as index_ir
from . import split_tiling
from .overrides import (B200Overrides, CPP_TYPE, FLOAT_DTYPES, INT_DTYPES, IxbExprPrinter,
                        constant_literal)

G = "ixb::gen::"

REDUCTION_OPS = {
    "sum": "ixb::SumOp", "max": "ixb::MaxOp", "min": "ixb::MinOp", "prod": "ixb::ProdOp",
}


class UnsupportedByTemplates(NotImplementedError):
    """The fused group needs something no B200 template provides yet."""


class B200Kernel(SIMDKernel):
    overrides = B200Overrides  # type: ignore[assignment]
    suffix = ";"
    newvar_prefix = "const auto "
    pexpr = PythonPrinter().doprint
    sexpr = IxbExprPrinter().doprint
    kexpr = sexpr
    allow_block_ptr = False

    def __init__(self, tiling, **kwargs: Any) -> None:
        self._row_cfg: Optional[split_tiling.RowConfig] = None
        self._buffer_dtypes: list = []
        super().__init__(tiling, **kwargs)
        self.is_row = self.features.is_reduction()
        if self.is_row:
            rnumel = self._static_numel("r0_")
            dt = self._narrowest_node_dtype()
            self._row_cfg = split_tiling.choose_row_config(rnumel, dt)
            if self._row_cfg is None:
                raise UnsupportedByTemplates(
                    f"reduced extent {rnumel} does not fit the persistent row template")
            if any(p.startswith("r") and p != "r0_" for p in self.numels):
                raise UnsupportedByTemplates("multi-axis reduction tilings")
        else:
            self.vec = split_tiling.choose_pointwise_vec(self._node_dtypes())

    # ------------------------------------------------------------------ policy hooks
    def should_use_persistent_reduction(self) -> bool:
        return True  # the row is always held on chip; oversize rows are rejected above

    def should_use_cooperative_reduction(self) -> bool:
        return False

    def want_no_x_dim(self) -> bool:
        return False

    def dtype_to_str(self, dtype: torch.dtype) -> str:
        return CPP_TYPE[dtype]

    @property
    def index_dtype(self) -> str:
        return "long long"

    def _static_numel(self, prefix: str) -> int:
        n = self.numels.get(prefix, sympy.S.One)
        try:
            return int(n)
        except TypeError as e:
            raise UnsupportedByTemplates(f"dynamic extent {n} for '{prefix}'") from e

    def _node_dtypes(self):
        out = []
        for node in self.features.scheduler_nodes():
            for dep in list(node.read_writes.reads) + list(node.read_writes.writes):
                try:
                    out.append(V.graph.get_dtype(dep.name))
                except Exception:
                    pass
        return out

    def _narrowest_node_dtype(self) -> torch.dtype:
        floats = [d for d in self._node_dtypes() if d in FLOAT_DTYPES]
        return split_tiling.narrowest_dtype(floats or self._node_dtypes())

    # ------------------------------------------------------------------ index helpers
    def _root(self, prefix: str):
        for t in self.range_trees:
            if t.prefix == prefix:
                return t
        return None

    def _expanded(self, index: sympy.Expr) -> sympy.Expr:
        return index_ir.expand_to_roots(index, self.range_tree_nodes)

    def _has_reduction_var(self, index: sympy.Expr) -> bool:
        rt = self._root("r0_")
        if rt is None:
            return False
        exp = self._expanded(index)
        return rt.symbol() in exp.free_symbols

    def _is_indirect(self, index: sympy.Expr) -> bool:
        return any(str(s).startswith(("tmp", "indirect")) for s in index.free_symbols)

    def codegen_iteration_ranges_entry(self, entry: IterationRangesEntry) -> None:
        expr = self.rename_indexing(entry.expr)
        self.indexing_code.writeline(f"const auto {entry.name} = {self.sexpr(expr)};")

    # ------------------------------------------------------------------ masks
    def _base_mask(self, vector: bool) -> str:
        if self.is_row:
            return "rmask" if vector else "(c.lane == 0)"
        return "xmask"

    def _load_mask_expr(self, vector: bool, for_store: bool) -> str:
        m = self._base_mask(vector) if (for_store or vector or not self.is_row) else "true"
        if not for_store and self._load_mask is not None:
            m = f"ixb::gen::op::logical_and({m}, {self._load_mask})"
        return m

    # ------------------------------------------------------------------ loads
    def load(self, name: str, index: sympy.Expr) -> CSEVariable:
        var = self.args.input(name)
        index = self.prepare_indexing(index)
        dtype = V.graph.get_dtype(name)
        ctype = self.dtype_to_str(dtype)
        idx = self.index_to_str(index)
        indirect = self._is_indirect(index)
        val_dtype = torch.float32 if dtype in FLOAT_DTYPES else (torch.bool if dtype == torch.bool else torch.int64)
        other = "0" if self._load_other is None else constant_literal(self._load_other, val_dtype)
        other = {torch.float32: f"(float)({other})", torch.int64: f"(long long)({other})",
                 torch.bool: f"(bool)({other})"}[val_dtype]
        masked = self._load_mask is not None

        line = None
        if not indirect and not masked:
            exp = self._expanded(index)
            if self.is_row:
                xr, rr = self._root("x"), self._root("r0_")
                if self.inside_reduction and rr is not None and rr.symbol() in exp.free_symbols:
                    stride = index_ir.reduction_stride(exp, xr.symbol(), rr.symbol(),
                                                       self._static_numel("x"), self._static_numel("r0_"))
                    if stride == 1:
                        # row-contiguous: 128-bit loads from the start of this row
                        line = (f"c.load_row(({var}) + ({G}lane0({idx}) - {G}lane0(r0_index)))")
            else:
                xr = self._root("x")
                if index_ir.is_vector_contiguous(exp, xr.symbol(), self.vec, self._static_numel("x")):
                    line = f"{G}ldvec<{ctype}, kVec>(({var}) + {G}lane0({idx}), nvalid)"
        if line is None:
            vector = (not self.is_row) or self._has_reduction_var(index) or indirect
            mask = self._load_mask_expr(vector, for_store=False)
            line = f"{G}gather({var}, {idx}, {mask}, {other})"
        return self.cse.generate(self.compute, line, dtype=val_dtype)

    # ------------------------------------------------------------------ stores
    def store(self, name: str, index: sympy.Expr, value: CSEVariable, mode=None) -> None:
        var = self.args.output(name)
        index = self.prepare_indexing(index)
        dtype = V.graph.get_dtype(name)
        ctype = self.dtype_to_str(dtype)
        idx = self.index_to_str(index)
        if mode is not None:
            raise UnsupportedByTemplates(f"store mode {mode}")
        line = None
        if not self._is_indirect(index):
            exp = self._expanded(index)
            if self.is_row:
                xr, rr = self._root("x"), self._root("r0_")
                if self.inside_reduction and rr is not None and rr.symbol() in exp.free_symbols:
                    stride = index_ir.reduction_stride(exp, xr.symbol(), rr.symbol(),
                                                       self._static_numel("x"), self._static_numel("r0_"))
                    if stride == 1:
                        line = (f"c.store_row(({var}) + ({G}lane0({idx}) - {G}lane0(r0_index)), {value});")
            else:
                xr = self._root("x")
                if index_ir.is_vector_contiguous(exp, xr.symbol(), self.vec, self._static_numel("x")):
                    line = f"{G}stvec<{ctype}, kVec>(({var}) + {G}lane0({idx}), nvalid, {value});"
        if line is None:
            vector = (not self.is_row) or self._has_reduction_var(index) or self._is_indirect(index)
            mask = self._base_mask(vector)
            line = f"{G}scatter({var}, {idx}, {mask}, {value});"
        # dropped at print time if the buffer turns out to be internal to the kernel
        self.compute.writeline(DeferredLine(name, line))

    def store_reduction(self, name: str, index: sympy.Expr, value: CSEVariable) -> None:
        var = self.args.output(name)
        index = self.prepare_indexing(index)
        idx = self.index_to_str(index)
        # one thread of the team writes the per-row result
        self.compute.writeline(DeferredLine(name, f"{G}scatter({var}, {idx}, (c.lane == 0), {value});"))

    # ------------------------------------------------------------------ reductions
    def reduction(self, dtype, src_dtype, reduction_type, value):
        assert self.inside_reduction and self.is_row
        key = (src_dtype, reduction_type, value)
        if key in self.cse.reduction_cache:
            return self.cse.reduction_cache[key]
        if reduction_type == "welford_reduce":
            result = self.welford_reduce_fallback(dtype, value)
        elif reduction_type == "online_softmax_reduce":
            # (row max, sum of exp(value - max)): the row is in registers, so the two-pass
            # form costs no extra memory traffic
            result = self.prepare_softmax_twopass_fallback(dtype, value)
        elif reduction_type in ("argmax", "argmin"):
            is_max = "true" if reduction_type == "argmax" else "false"
            result = self.cse.generate(self.compute, f"c.template reduce_arg<{is_max}>({value})",
                                       dtype=torch.int64)
        elif reduction_type == "any":
            result = self.cse.generate(self.compute, f"c.reduce_any({value})", dtype=torch.bool)
        elif reduction_type in REDUCTION_OPS:
            text = f"c.template reduce<{REDUCTION_OPS[reduction_type]}>({value})"
            if src_dtype in INT_DTYPES or src_dtype == torch.bool:
                # exact up to 2^24; integer reductions beyond that need an integer team exchange
                text = f"ixb::gen::op::to_int({text})"
                result = self.cse.generate(self.compute, text, dtype=torch.int64)
            else:
                result = self.cse.generate(self.compute, text, dtype=torch.float32)
        else:
            raise UnsupportedByTemplates(f"reduction type {reduction_type}")
        self.cse.reduction_cache[key] = result
        return result

    # ------------------------------------------------------------------ bounds checks
    def check_bounds(self, expr, size, lower, upper) -> None:
        # indirect indices are wrapped by Inductor's lowering; out-of-range indices are the
        # caller's error as in eager mode, they are not trapped on the device
        return

    # ------------------------------------------------------------------ assembling
    def codegen_body(self) -> None:
        self.body.splice(self.loads)
        self.body.splice(self.compute)
        self.body.splice(self.stores)
        self.loads.clear()
        self.compute.clear()
        self.stores.clear()

    def _kernel_args(self):
        """(c declaration, assignment from the launcher's arrays) per argument, in the
        order ``call_kernel`` passes them."""
        _, call_args, precompile_args, _ = self.args.python_argdefs()
        decls, assigns = [], []
        pi = ii = 0
        outputs = set(self.args.output_buffers.values()) | {
            getattr(v, "inner_name", None) for v in self.args.inplace_buffers.values()}
        for arg in precompile_args:
            if isinstance(arg, TensorArg):
                ctype = self.dtype_to_str(arg.dtype)
                const = "" if arg.name in outputs or arg.name.startswith(("out_ptr", "in_out_ptr")) else "const "
                decls.append(f"{const}{ctype}* {arg.name};")
                assigns.append(f"b.{arg.name} = ({const}{ctype}*)ptrs[{pi}];")
                pi += 1
            elif isinstance(arg, SizeArg):
                decls.append(f"long long {arg.name};")
                assigns.append(f"b.{arg.name} = ints[{ii}];")
                ii += 1
            else:
                raise UnsupportedByTemplates(f"kernel argument {arg!r}")
        return decls, assigns, call_args

    def codegen_kernel(self, name: Optional[str] = None) -> str:
        self.codegen_body()
        decls, assigns, _ = self._kernel_args()
        xnumel = self._static_numel("x")
        src = IndentedBuffer()
        src.writeline('#include "ixb/gen.cuh"')
        src.writeline("namespace {")
        src.writeline("using namespace ixb;")
        src.writeline("struct Body {")
        with src.indent():
            for d in decls:
                src.writeline(d)
            if self.is_row:
                cfg = self._row_cfg
                src.writeline("template <class Ctx>")
                src.writeline("__device__ __forceinline__ void row(Ctx& c, const long long xindex) const {")
                with src.indent():
                    src.writeline("const auto r0_index = c.rindex();")
                    src.writeline("const auto rmask = c.rmask();")
                    src.splice(self.indexing_code)
                    src.splice(self.body)
                src.writeline("}")
            else:
                src.writeline(f"static constexpr int kVec = {self.vec};")
                src.writeline("__device__ __forceinline__ void tile(const long long xbase, const int nvalid) const {")
                with src.indent():
                    src.writeline(f"const auto xindex = {G}iota<kVec>(xbase);")
                    src.writeline(f"const auto xmask = xindex < (xbase + nvalid);")
                    src.splice(self.indexing_code)
                    src.splice(self.body)
                src.writeline("}")
        src.writeline("};")
        src.writeline("}  // namespace")
        src.writeline('extern "C" int ixb_gen_launch(void** ptrs, const long long* ints, void* stream) {')
        with src.indent():
            src.writeline("Body b;")
            for a in assigns:
                src.writeline(a)
            if self.is_row:
                cfg = self._row_cfg
                rnumel = self._static_numel("r0_")
                rt = self.dtype_to_str(self._narrowest_node_dtype())
                if cfg.vec * {"float": 4, "double": 8}.get(rt, 2) != 16:
                    rt = {4: "float", 8: "ixb::bf16"}[cfg.vec]
                src.writeline(f"return {G}launch_row_gen<Body, {rt}, {cfg.team}, {cfg.teams}, {cfg.vpt}>"
                              f"(b, {xnumel}LL, {rnumel}, stream);")
            else:
                src.writeline(f"return {G}launch_pointwise<Body>(b, {xnumel}LL, stream);")
        src.writeline("}")
        text = src.getvalue()
        family = "row" if self.is_row else "pointwise"
        return f"ixb_load_kernel('''\n{text}''', family={family!r})"

    def call_kernel(self, name: str, node: Any = None, deallocate_ws: bool = True) -> None:
        wrapper = V.graph.wrapper_code
        for v in self.args.sizevars:
            wrapper.ensure_size_computed(v)
        _, call_args, _, _ = self.args.python_argdefs()
        device = V.graph.get_current_device_or_throw()
        if device.type == "cuda":
            stream = wrapper.write_get_raw_stream(device.index, V.graph.name)
            wrapper.writeline(f"{name}.run({', '.join(map(str, call_args))}, stream={stream})")
        else:
            wrapper.writeline(f"{name}.run({', '.join(map(str, call_args))}, stream=None)")

    def codegen_nan_check(self) -> None:
        return
