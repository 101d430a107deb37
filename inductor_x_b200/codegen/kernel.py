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
import math
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


def config_bytes(dtype: torch.dtype) -> int:
    return ixb_config.BYTES_PER_ELEMENT.get(dtype, 8)

G = "ixb::gen::"

REDUCTION_OPS = {
    "sum": "ixb::SumOp", "max": "ixb::MaxOp", "min": "ixb::MinOp", "prod": "ixb::ProdOp",
}


INT_REDUCTION_OPS = {"sum": "ISum", "prod": "IProd", "max": "IMax", "min": "IMin"}

#: registers a thread may spend on operands that are the same for every row; operands beyond
#: that budget (the least used ones) live in a shared-memory table
MAX_CONST_REGS = 64
#: per-column operands hoisted out of the row loop at most (registers + shared memory)
MAX_CONSTS = 6
#: streamed operands fetched one row ahead as raw 128-bit vectors
MAX_STAGED = 2


class UnsupportedByTemplates(NotImplementedError):
    """The fused group needs something no B200 template provides yet."""


class B200CSEVariable(CSEVariable):
    """Records the op and operands every value came from: the emitter's peephole rewrites
    (fused multiply-add, folded scalar factors, reuse of the online-softmax exponentials,
    sums carried by an earlier exchange) look operands up in that table."""

    #: the integer type the value has in the graph (integers are carried in 64 bits whatever
    #: that type is; ops whose result can leave its range wrap it back), None for other kinds
    int_type: Optional[torch.dtype] = None

    def update_on_args(self, name, args, kwargs):
        V.kernel.note_op(self, name, args, kwargs)
        self.int_type = graph_int_type(self, name, args, kwargs or {})


_COMPARISONS = ("eq", "ne", "lt", "le", "gt", "ge", "isnan", "isinf", "signbit", "logical_and", "logical_or",
                "logical_xor", "logical_not", "and_", "or_")


def graph_int_type(var, name, args, kwargs) -> Optional[torch.dtype]:
    """Integer type of an op's result as eager mode would compute it: the conversion target,
    else the promoted type of the integer operands (Python scalars do not take part)."""
    if getattr(var, "dtype", None) != torch.int64 or name in _COMPARISONS:
        return None
    if name in ("to_dtype", "constant", "index_expr"):
        dt = kwargs.get("dtype", args[1] if len(args) > 1 else None)
        return dt if dt in INT_DTYPES else None
    if name in ("bitwise_left_shift", "bitwise_right_shift"):
        args = args[:1]                     # the result has the type of the shifted value
    out = None
    for a in args:
        if not isinstance(a, CSEVariable) or a.dtype == torch.bool:
            continue
        t = getattr(a, "int_type", None) or (a.dtype if a.dtype in INT_DTYPES else None)
        if t is None:
            return None
        out = t if out is None else torch.promote_types(out, t)
    return out


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
        self._ph: dict = {}
        self._ph_by_key: dict = {}
        self._row_prefetch: list = []
        self.dag: dict = {}          # value name -> (op name, operands)
        self.scalars: set = set()    # values that do not vary along the reduced row
        self.consts: list = []       # hoisted row-invariant operands: (member, pointer text, element count)
        self.staged: list = []       # operands fetched a row ahead: (member, ctype, pointer text)
        self.const_of: dict = {}     # value name -> Consts member text
        self.online: dict = {}       # name of a softmax input -> its online-softmax exchange
        self.online_exp: dict = {}   # name of exp(input - max) -> exchange
        self.checked_indices = 0     # data-dependent indices checked on the device (debug builds)
        self.x_indexing = IndentedBuffer()
        self.r_indexing = IndentedBuffer()
        self.looped = False                      # rows walked in chunks (decided before the range trees exist)
        self.post_loop_combine = IndentedBuffer()
        self.post_loop_store = IndentedBuffer()
        self.outside_loop_vars: set = set()
        self.n_acc = 0
        super().__init__(tiling, **kwargs)
        self.is_row = self.features.is_reduction()
        if self.is_row:
            # a symbolic reduced extent is served up to the capacity of the launch shape chosen
            # for the extent seen at trace time (the launcher refuses longer rows)
            rnumel = self._numel_hint("r0_")
            dt = self._narrowest_node_dtype()
            if self.looped:
                self._row_cfg = split_tiling.choose_loop_config(dt)
            else:
                self._row_cfg = split_tiling.choose_row_config(rnumel, dt, rows=self._numel_hint("x"))
                if self._row_cfg is None and self._reads_are_strided():
                    # an outer reduction of any length: the outer mapping loops over the reduced
                    # axis itself; the row text is never used
                    self._row_cfg = split_tiling.choose_loop_config(dt)
            if self._row_cfg is None:
                raise UnsupportedByTemplates(
                    f"reduced extent {rnumel} does not fit the persistent row template")
            if any(p.startswith("r") and p != "r0_" for p in self.numels):
                raise UnsupportedByTemplates("multi-axis reduction tilings")
            self._outer_vec = split_tiling.choose_pointwise_vec(self._node_dtypes())
        else:
            self.vec = split_tiling.choose_pointwise_vec(self._node_dtypes())

    def create_cse_var(self, *args, **kwargs):
        return B200CSEVariable(*args, **kwargs)

    # ------------------------------------------------------------------ value table
    def note_op(self, var, name, args, kwargs=None) -> None:
        # a peephole that replaced the op by a different one says so (pending_dag)
        entry = getattr(self, "pending_dag", None) or (name, args, kwargs or {})
        self.pending_dag = None
        self.dag.setdefault(var.name, entry)
        if name == "exp" and getattr(self, "pending_online_exp", None) is not None:
            self.online_exp[var.name] = self.pending_online_exp
        self.pending_online_exp = None
        if name in ("load", "reduction"):
            return
        if name == "index_expr":
            if self.is_row and not self._has_reduction_var(self.prepare_indexing(args[0])):
                self.scalars.add(var.name)
            return
        if not self.is_row:
            return
        if all(str(a) in self.scalars for a in args if isinstance(a, CSEVariable)):
            self.scalars.add(var.name)

    def resolve(self, v):
        """The value ``v`` names, seen through casts between floating types (all floating
        values are fp32 inside a kernel)."""
        for _ in range(8):
            d = self.dag.get(str(v))
            if d is None or d[0] != "to_dtype":
                break
            src = d[1][0]
            dst = d[1][1] if len(d[1]) > 1 else d[2].get("dtype")
            if not isinstance(src, CSEVariable) or src.dtype not in FLOAT_DTYPES or dst not in FLOAT_DTYPES:
                break
            v = src
        return v

    def op_of(self, v, name: str):
        """Operands of ``v`` if it was produced by op ``name`` (through float casts)."""
        d = self.dag.get(str(self.resolve(v)))
        return d[1] if d is not None and d[0] == name else None

    def const_value(self, v):
        d = self.dag.get(str(self.resolve(v)))
        if d is not None and d[0] == "constant":
            return d[1][0]
        return v if isinstance(v, (int, float)) and not isinstance(v, bool) else None

    def is_scalar(self, v) -> bool:
        return not isinstance(v, CSEVariable) or str(v) in self.scalars

    def is_float(self, v) -> bool:
        return isinstance(v, CSEVariable) and v.dtype in FLOAT_DTYPES

    def half_group(self) -> bool:
        """True when the group reads or writes a 16-bit floating type (its results are
        compared at that precision)."""
        return self._narrowest_node_dtype() in (torch.float16, torch.bfloat16)

    # ------------------------------------------------------------------ policy hooks
    def should_use_persistent_reduction(self) -> bool:
        """The row is held on chip by one team when it fits comfortably (up to
        ``split_tiling.MAX_PERSISTENT_VPT`` vectors per thread at the widest team); a longer
        stride-1 row is walked in chunks - one loop per reduction, the reference's looped inner
        reduction (``inductor_x/codegen/triton.py:1208-1253``).  Outer (strided) reductions
        always use the outer mapping, whose body loops over the reduced axis anyway."""
        if not self.features.is_reduction():
            return True
        vec = min(max(ixb_config.get_aligned_numel(self._narrowest_node_dtype()), 1), 8)
        try:
            rnumel = int(self.features.reduction_numel)
        except TypeError:
            # run-time extent: persistent up to the compiled capacity; where the extent seen at
            # trace time is beyond what any launch shape holds, the row is walked in chunks, whose
            # count the launcher derives from the run-time extent (any length is served)
            hint = int(V.graph.sizevars.size_hint(self.features.reduction_numel))
            self.looped = -(-hint // vec) > split_tiling.MAX_TEAM * split_tiling.MAX_VPT
            return not self.looped
        nvec = -(-rnumel // vec)
        long_row = nvec > split_tiling.MAX_TEAM * split_tiling.MAX_PERSISTENT_VPT
        try:
            kept = int(self.features.numel)
        except TypeError:
            kept = vec
        # a strided (outer) reduction is served by the outer mapping, which needs at least one
        # vector of kept elements; anything else that long is walked in chunks
        self.looped = long_row and not (kept >= vec and self._reads_are_strided())
        return not self.looped

    def _reads_are_strided(self) -> bool:
        """True when no read of a reduction node walks a reduced variable with stride 1: an
        outer reduction (decided from the scheduler nodes, before any code is emitted).  The
        reduced variables of a dependency are its trailing loop variables whose extents
        multiply to the reduced extent."""
        from torch._inductor.dependencies import MemoryDep

        try:
            rnumel = int(self.features.reduction_numel)
        except TypeError:
            return False
        saw = False
        for node in self.features.scheduler_nodes():
            if not node.is_reduction():
                continue
            for dep in node.read_writes.reads:
                if not isinstance(dep, MemoryDep) or not dep.var_names:
                    continue
                prod, rvars = 1, []
                for v, size in zip(reversed(dep.var_names), reversed(dep.size)):
                    if prod >= rnumel:
                        break
                    try:
                        prod *= int(size)
                    except TypeError:
                        return False
                    rvars.append(v)
                if prod != rnumel:
                    continue             # this dependency does not span the reduced axis in its loop nest
                rvars = [v for v in rvars if v in dep.index.free_symbols]
                if not rvars:
                    continue             # broadcast along the reduced axis
                saw = True
                strides = V.graph.sizevars.stride_vars(dep.index, rvars)
                if any(st == 1 for st in strides):
                    return False
        return saw

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

    def _numel_hint(self, prefix: str) -> int:
        """The extent if it is static, else the value it had when the graph was traced.  The
        kept extent may be symbolic (the launcher receives it at run time); the hint only
        steers choices - launch shape, whether a kernel is worth tuning - never addresses."""
        n = self.numels.get(prefix, sympy.S.One)
        try:
            return int(n)
        except TypeError:
            return max(int(V.graph.sizevars.size_hint(n)), 1)

    def _is_dynamic(self, prefix: str = "x") -> bool:
        return not self.numels.get(prefix, sympy.S.One).is_Integer

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
        line = f"const auto {entry.name} = {self.sexpr(expr)};"
        # reduced-axis variables live inside the reduction loop of the outer mapping
        (self.r_indexing if entry.is_reduction else self.x_indexing).writeline(line)

    # ------------------------------------------------------------------ two mappings
    # A reduction group can be laid out in two ways and the choice is only known once the
    # whole group has been seen:
    #   row    - the reduced axis is held by a team (xindex scalar, r0_index a vector)
    #   outer  - threads map along the kept axis (xindex a vector, r0_index the scalar loop
    #            variable of a loop emitted around everything before the reduction)
    # Expression text is rank-agnostic (auto + overloads), so only loads, stores and the
    # reduction itself differ.  Those are emitted as placeholders that carry both texts
    # and are substituted in codegen_kernel.
    def _placeholder(self, kind: str, key, row_text: str, outer_text: str, **info) -> str:
        table = self._ph_by_key
        if key is not None and key in table:
            return table[key]
        tag = f"@{kind}{len(self._ph)}@"
        self._ph[tag] = dict(kind=kind, row=row_text, outer=outer_text, **info)
        if key is not None:
            table[key] = tag
        return tag

    def _fast_flag(self, exp: sympy.Expr, vec: int) -> str:
        """Template argument that makes a vector access unconditional in full tiles: the
        index is proven a multiple of the vector width, so with 16-byte aligned base
        pointers (checked by the launcher) the address is aligned."""
        aligned = index_ir.vector_access(exp, self._root("x").symbol(), vec)[1]
        return "FAST" if aligned else "false"

    def _xr_roots(self):
        return self._root("x"), self._root("r0_")

    def _outer_x_contiguous(self, exp: sympy.Expr) -> bool:
        """x-vector contiguity of an access for every value of the reduced index, decided
        from the structure of the index (no term may mix the kept and the reduced index)."""
        xr, rr = self._xr_roots()
        if self._numel_hint("x") < self._outer_vec:
            return False
        if rr is None or rr.symbol() not in exp.free_symbols:
            return index_ir.is_vector_contiguous(exp, xr.symbol(), self._outer_vec, self._numel_hint("x"))
        return index_ir.x_contiguous_for_all_r(exp, xr.symbol(), rr.symbol(), self._outer_vec)

    # ------------------------------------------------------------------ loads
    def _refuse_fp64(self, name: str, dtype: torch.dtype) -> None:
        if dtype == torch.float64 and not ixb_config.fp64_as_fp32:
            raise UnsupportedByTemplates(
                f"buffer {name} is float64: the B200 templates compute floating values in fp32 "
                "(set IXB_FP64_AS_FP32=1 to accept that)")

    def load(self, name: str, index: sympy.Expr) -> CSEVariable:
        out = self._load_value(name, index)
        dtype = V.graph.get_dtype(name)
        if dtype in INT_DTYPES and isinstance(out, B200CSEVariable):
            out.int_type = dtype
        return out

    def _load_value(self, name: str, index: sympy.Expr) -> CSEVariable:
        var = self.args.input(name)
        index = self.prepare_indexing(index)
        dtype = V.graph.get_dtype(name)
        self._refuse_fp64(name, dtype)
        ctype = self.dtype_to_str(dtype)
        idx = self.index_to_str(index)
        indirect = self._is_indirect(index)
        val_dtype = torch.float32 if dtype in FLOAT_DTYPES else (torch.bool if dtype == torch.bool else torch.int64)
        fill = self._load_other
        if isinstance(fill, float) and val_dtype != torch.float32 and not math.isfinite(fill):
            # a pad value of the converted result (max-pooling integers pads with -inf): the select
            # after the masked sub-block supplies it, the load only needs some in-range value
            fill = 0
        other = "0" if fill is None else constant_literal(fill, val_dtype)
        other = {torch.float32: f"(float)({other})", torch.int64: f"(long long)({other})",
                 torch.bool: f"(bool)({other})"}[val_dtype]
        masked = self._load_mask is not None
        lm = f"ixb::gen::op::logical_and(@M@, {self._load_mask})" if masked else "@M@"
        gather = f"{G}gather({var}, {idx}, {lm}, {other})"

        if not self.is_row:
            line = gather.replace("@M@", "xmask")
            xsym = self._root("x").symbol()
            if not indirect and not masked:
                exp0 = self._expanded(index)
                if xsym in exp0.free_symbols and not index_ir.is_vector_constant(exp0, xsym, self.vec) and \
                        not index_ir.vector_access(exp0, xsym, self.vec)[0]:
                    # strided along the flat index: a transpose candidate; the text is settled
                    # when the whole group has been seen (register tile or per-element gather)
                    loads = self.__dict__.setdefault("_gather_loads", [])
                    loads.append(exp0)
                    tag = f"@T{len(loads) - 1}@"
                    self.__dict__.setdefault("_tile_loads", {})[tag] = dict(
                        ctype=ctype, dtype=dtype, var=var, idx=idx, exp=exp0, gather=line)
                    return self.cse.generate(self.compute, tag, dtype=val_dtype)
            if indirect and not masked:
                # direct part contiguous along the vector: one 128-bit access whenever the
                # indirect operands are per-vector scalars (decided by their C++ type)
                exp = self._expanded(index)
                ind = sorted(str(s) for s in exp.free_symbols if str(s).startswith(("tmp", "indirect")))
                contig, aligned = index_ir.vector_access(exp, xsym, self.vec)
                if contig and not (exp.free_symbols - {xsym} - {s for s in exp.free_symbols if str(s) in ind}):
                    al = "FAST" if aligned else "false"
                    line = (f"{G}igather<{ctype}, kVec, {al}>({var}, {idx}, xmask, {other}, nvalid, "
                            f"{', '.join(ind)})")
            if not indirect and not masked:
                exp = self._expanded(index)
                if xsym in exp.free_symbols and index_ir.is_vector_constant(exp, xsym, self.vec):
                    line = f"{G}ld_uniform({var}, {G}lane0({idx}), nvalid > 0, {other})"
                if index_ir.is_vector_contiguous(exp, self._root("x").symbol(), self.vec, self._numel_hint("x")):
                    al = self._fast_flag(exp, self.vec)
                    line = f"{G}ldvec<{ctype}, kVec, {al}>(({var}) + {G}lane0({idx}), nvalid)"
            return self.cse.generate(self.compute, line, dtype=val_dtype)

        # reduction group: text for both mappings
        exp = self._expanded(index)
        xr, rr = self._xr_roots()
        has_r = rr is not None and rr.symbol() in exp.free_symbols
        stride = None
        if not indirect and has_r and self.inside_reduction:
            stride = index_ir.reduction_stride(exp, xr.symbol(), rr.symbol(), self._numel_hint("x"),
                                               self._numel_hint("r0_"))
        vector_row = has_r or indirect
        row_text = gather.replace("@M@", "rmask" if vector_row else "true")
        const_member = None
        if stride == 1 and not masked:
            row_ptr = f"({var}) + ({G}lane0({idx}) - {G}lane0(r0_index))"
            row_text = f"c.load_row({row_ptr})"
            cfg = self._row_cfg
            n = cfg.elems_per_thread
            narrow_ok = dtype in (torch.float32, torch.float16, torch.bfloat16) and \
                config_bytes(dtype) >= config_bytes(self._narrowest_node_dtype())
            if xr.symbol() not in exp.free_symbols:
                # the same for every row (a per-column scale or shift): loaded and widened
                # once per thread while registers allow
                const_member = next((m for m, ptr, _ in self.consts if ptr == row_ptr), None)
                if const_member is None and narrow_ok and len(self.consts) < MAX_CONSTS and \
                        cfg.team >= 32 and cfg.vec % 4 == 0 and not self.looped:
                    const_member = f"@K{len(self.consts)}@"      # final slot and home decided at print time
                    self.consts.append((const_member, row_ptr, n))
                if const_member is not None:
                    row_text = const_member
            else:
                if row_ptr not in self._row_prefetch:
                    self._row_prefetch.append(row_ptr)     # streamed once per row: worth prefetching
                aligned = index_ir.row_starts_aligned(exp, xr.symbol(), rr.symbol(), cfg.vec) and \
                    not self._is_dynamic("r0_") and self._numel_hint("r0_") % cfg.vec == 0
                if narrow_ok and aligned and not self.looped:
                    member = next((m for m, _, ptr in self.staged if ptr == row_ptr), None)
                    if member is None and len(self.staged) < MAX_STAGED:
                        member = f"raw.s{len(self.staged)}"
                        self.staged.append((member, ctype, row_ptr))
                    if member is not None:
                        row_text = f"c.template operand<STAGED, {ctype}>({member}, {row_ptr})"
        outer_text = gather.replace("@M@", "xmask")
        x_contig = False
        if not indirect and not masked and xr.symbol() in exp.free_symbols:
            x_contig = self._outer_x_contiguous(exp)
            if x_contig:
                al = self._fast_flag(exp, self._outer_vec)
                outer_text = f"{G}ldvec<{ctype}, kVec, {al}>(({var}) + {G}lane0({idx}), nvalid)"
        tag = self._placeholder("L", (name, idx, str(self._load_mask), other), row_text, outer_text,
                                stride=stride, has_r=has_r, x_contig=x_contig, indirect=indirect, exp=exp,
                                in_reduction=self.inside_reduction)
        out = self.cse.generate(self.compute, tag, dtype=val_dtype)
        self.dag.setdefault(out.name, ("load", (name, index), {}))
        if not vector_row:
            self.scalars.add(out.name)
        if const_member is not None:
            self.const_of[out.name] = const_member
        return out

    # ------------------------------------------------------------------ stores
    def store(self, name: str, index: sympy.Expr, value: CSEVariable, mode=None) -> None:
        var = self.args.output(name)
        index = self.prepare_indexing(index)
        dtype = V.graph.get_dtype(name)
        self._refuse_fp64(name, dtype)
        ctype = self.dtype_to_str(dtype)
        idx = self.index_to_str(index)
        if mode not in (None, "atomic_add"):
            raise UnsupportedByTemplates(f"store mode {mode}")
        indirect = self._is_indirect(index)
        exp = self._expanded(index)
        if mode == "atomic_add":
            if dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32):
                raise UnsupportedByTemplates(f"atomic add into {dtype}")
            # accumulating scatter: one atomic per element, whatever the mapping
            if not self.is_row:
                self.compute.writeline(DeferredLine(name, f"{G}scatter_add({var}, {idx}, xmask, {value});"))
                return
            xr, rr = self._xr_roots()
            has_r = (rr is not None and rr.symbol() in exp.free_symbols) or indirect
            row_text = f"{G}scatter_add({var}, {idx}, {'rmask' if has_r else 'c.leader()'}, {value});"
            outer_text = f"{G}scatter_add({var}, {idx}, ixb::gen::op::logical_and(xmask, c.writer()), {value});"
            tag = self._placeholder("S", None, row_text, outer_text, has_r=has_r, in_reduction=self.inside_reduction)
            self.compute.writeline(DeferredLine(name, tag))
            return
        if not self.is_row:
            line = f"{G}scatter({var}, {idx}, xmask, {value});"
            if not indirect and index_ir.is_vector_contiguous(exp, self._root("x").symbol(), self.vec,
                                                              self._numel_hint("x")):
                al = self._fast_flag(exp, self.vec)
                line = f"{G}stvec<{ctype}, kVec, {al}>(({var}) + {G}lane0({idx}), nvalid, {value});"
            self.compute.writeline(DeferredLine(name, line))
            return
        xr, rr = self._xr_roots()
        has_r = rr is not None and rr.symbol() in exp.free_symbols
        vector_row = has_r or indirect
        row_text = f"{G}scatter({var}, {idx}, {'rmask' if vector_row else 'c.leader()'}, {value});"
        if not indirect and has_r and self.inside_reduction:
            stride = index_ir.reduction_stride(exp, xr.symbol(), rr.symbol(), self._numel_hint("x"),
                                               self._numel_hint("r0_"))
            if stride == 1:
                row_ptr = f"({var}) + ({G}lane0({idx}) - {G}lane0(r0_index))"
                row_text = f"c.store_row({row_ptr}, {value});"
                cfg = self._row_cfg
                if not self.looped and index_ir.row_starts_aligned(exp, xr.symbol(), rr.symbol(), cfg.vec) and \
                        not self._is_dynamic("r0_") and self._numel_hint("r0_") % cfg.vec == 0 and \
                        dtype in FLOAT_DTYPES and \
                        config_bytes(dtype) >= config_bytes(self._narrowest_node_dtype()):
                    row_text = f"c.template put_row<STAGED>({row_ptr}, {value});"
        outer_text = f"{G}scatter({var}, {idx}, ixb::gen::op::logical_and(xmask, c.writer()), {value});"
        if not indirect and not has_r and self._outer_x_contiguous(exp):
            outer_text = (f"{G}stvec<{ctype}, kVec>(({var}) + {G}lane0({idx}), c.writer() ? nvalid : 0, "
                          f"{value});")
        tag = self._placeholder("S", None, row_text, outer_text, has_r=has_r,
                                in_reduction=self.inside_reduction)
        # dropped at print time if the buffer turns out to be internal to the kernel
        self.compute.writeline(DeferredLine(name, tag))

    def store_reduction(self, name: str, index: sympy.Expr, value: CSEVariable) -> None:
        prior = self.inside_reduction
        self.inside_reduction = False
        compute = self.compute
        if self.looped:
            self.compute = self.post_loop_store      # after the chunk loop that produced the value
        try:
            self.store(name, index, value)
        finally:
            self.inside_reduction = prior
            self.compute = compute

    # ------------------------------------------------------------------ scans
    def scan(self, dtypes, combine_fn, values):
        """Inclusive prefix sum / product along a stride-1 row held by a team (``cumsum`` and
        ``cumprod`` over the last axis; the reference keeps them extern kernels,
        ``inductor_x/lowering.py:235-245``).  Other combine functions, several values, looped or
        strided rows are refused; the lowering only sends the supported form here."""
        assert self.inside_reduction and self.is_row
        if len(values) != 1 or self.looped or self._is_dynamic("r0_"):
            raise UnsupportedByTemplates("scan: one value over a static row held on chip only")
        is_int = dtypes[0] in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool)
        if not is_int and dtypes[0] not in (torch.float32, torch.float16, torch.bfloat16):
            raise UnsupportedByTemplates(f"scan of {dtypes[0]}")
        # which combine function is it?  run it on two probes and read the op off the value table
        probe_dtype = torch.int64 if is_int else torch.float32
        a = self.cse.newvar(dtype=probe_dtype)
        b = self.cse.newvar(dtype=probe_dtype)
        probe = IndentedBuffer()
        saved = self.compute
        self.compute = probe
        try:
            (res,) = combine_fn((a,), (b,))
        finally:
            self.compute = saved
        which = None
        for name in ("add", "mul"):
            operands = self.op_of(res, name)
            if operands is not None and {str(o) for o in operands} == {str(a), str(b)}:
                which = name
        if which is None:
            raise UnsupportedByTemplates("scan: only sums and products are scanned by the row template")
        self._has_scan = True
        if is_int:      # exact 64-bit integers
            iop = "ISum" if which == "add" else "IProd"
            out = self.cse.generate(self.compute, f"c.template scan_int<typename Ctx::{iop}>({values[0]})",
                                    dtype=torch.int64)
        else:
            op = "ixb::SumOp" if which == "add" else "ixb::ProdOp"
            out = self.cse.generate(self.compute, f"c.template scan<{op}>({values[0]})", dtype=torch.float32)
        return (out,)

    # ------------------------------------------------------------------ reductions
    def _reduction_marker(self, tag: str) -> None:
        self.compute.writeline(f"@B{tag[2:]}")  # marks where the reduction loop of the outer mapping ends

    def reduction(self, dtype, src_dtype, reduction_type, value):
        assert self.inside_reduction and self.is_row
        key = (src_dtype, reduction_type, value)
        if key in self.cse.reduction_cache:
            return self.cse.reduction_cache[key]
        if self.looped:
            result = self._looped_reduction(src_dtype, reduction_type, value)
        elif reduction_type == "welford_reduce" and not ixb_config.merged_welford:
            result = self.welford_reduce_fallback(dtype, value)
        elif reduction_type == "online_softmax_reduce" and not (ixb_config.merged_online_softmax
                                                                and src_dtype in FLOAT_DTYPES):
            result = self.prepare_softmax_twopass_fallback(dtype, value)
        elif reduction_type == "welford_reduce":
            # (mean, m2, weight) from one exchange of merged partial statistics
            tag = self._placeholder("R", None, f"c.welford({value})", "", outer_ok=False)
            self._reduction_marker(tag)
            w = self.cse.generate(self.compute, tag, dtype=torch.float32)
            result = tuple(self.cse.generate(self.compute, f"{w}.{field}", dtype=torch.float32)
                           for field in ("mean", "m2", "weight"))
        elif reduction_type == "online_softmax_reduce":
            # (row max, sum of exp(value - max)) from one exchange of rescaled partial sums;
            # the thread keeps its exponentials, and later row sums that are linear in them
            # join the same exchange as riders (the text is completed in _substitute)
            n = self._row_cfg.elems_per_thread
            tag = self._placeholder("R", None, "", "", outer_ok=False, online=True, value=str(value),
                                    riders_s=[], riders_p=[], n=n)
            self._reduction_marker(tag)
            ex = self.cse.generate(self.compute, tag, dtype=torch.float32)
            self.dag.setdefault(ex.name, ("reduction", (reduction_type, value), {}))
            result = tuple(self.cse.generate(self.compute, f"{ex}.{field}", dtype=torch.float32)
                           for field in ("max", "sum"))
            info = dict(tag=tag, var=str(ex), max=str(result[0]), sum=str(result[1]), value=str(self.resolve(value)))
            self.online[info["value"]] = info
        elif reduction_type in ("argmax", "argmin"):
            is_max = "true" if reduction_type == "argmax" else "false"
            # 32- and 64-bit integers are compared as integers (a float merges neighbours beyond 2^24)
            form = "reduce_arg_int" if src_dtype in (torch.int32, torch.int64) else "reduce_arg"
            tag = self._placeholder("R", None, f"c.template {form}<{is_max}>({value})", "", outer_ok=False)
            self._reduction_marker(tag)
            result = self.cse.generate(self.compute, tag, dtype=torch.int64)
        elif reduction_type == "any":
            tag = self._placeholder("R", None, f"c.reduce_any({value})", "", outer_ok=False)
            self._reduction_marker(tag)
            result = self.cse.generate(self.compute, tag, dtype=torch.bool)
        elif reduction_type in REDUCTION_OPS:
            op = REDUCTION_OPS[reduction_type]
            is_int = src_dtype in INT_DTYPES or src_dtype == torch.bool
            hoisted = None if is_int or reduction_type != "sum" else self._sum_from_earlier_exchange(value)
            if hoisted is not None:
                result = self.cse.generate(self.compute, hoisted, dtype=torch.float32)
            else:
                row_text = f"c.template reduce<{op}>({value})"
                outer_text = f"c.template combine<{op}>(acc)"
                if reduction_type == "sum" and not is_int:
                    factors = self.op_of(value, "mul")
                    if factors is not None and all(self.is_float(f) for f in factors):
                        row_text = f"c.reduce_dot({factors[0]}, {factors[1]})"
                if is_int:
                    # 64-bit integer accumulation and exchange: exact (the float path would
                    # round sums beyond 2^24)
                    iop = INT_REDUCTION_OPS[reduction_type]
                    row_text = f"c.template reduce_int<typename Ctx::{iop}>({value})"
                    outer_text = f"c.template combine_int<typename Ctx::{iop}>(acc)"
                tag = self._placeholder("R", None, row_text, outer_text, outer_ok=True, op=op,
                                        value=str(value), rtype=reduction_type, is_int=is_int)
                self._reduction_marker(tag)
                result = self.cse.generate(self.compute, tag,
                                           dtype=torch.int64 if is_int else torch.float32)
        else:
            raise UnsupportedByTemplates(f"reduction type {reduction_type}")
        for r in (result if isinstance(result, tuple) else (result,)):
            if isinstance(r, CSEVariable):
                self.scalars.add(r.name)
                self.dag.setdefault(r.name, ("reduction", (reduction_type, value), {}))
        self.cse.reduction_cache[key] = result
        return result

    def _looped_reduction(self, src_dtype, reduction_type, value):
        """One reduction of a row walked in chunks: a per-thread accumulator declared ahead of
        the loop, folded with the chunk's elements inside it, and one team exchange after it."""
        n = self.n_acc
        self.n_acc += 1
        acc = f"_acc{n}"
        is_int = src_dtype in INT_DTYPES or src_dtype == torch.bool
        if reduction_type == "welford_reduce":
            # running (mean, m2, weight) of the thread, merged chunk by chunk, one exchange at the end
            self.body.writeline(f"typename Ctx::Welford {acc}{{0.f, 0.f, 0.f}};")
            self.compute.writeline(f"{acc} = Ctx::merge({acc}, c.local_welford({value}));")
            w = self.cse.generate(self.post_loop_combine, f"c.xwelford({acc})", dtype=torch.float32)
            result = tuple(self.cse.generate(self.post_loop_combine, f"{w}.{field}", dtype=torch.float32)
                           for field in ("mean", "m2", "weight"))
            self.outside_loop_vars.update([w, *result])
            return result
        if reduction_type == "online_softmax_reduce":
            self.body.writeline(f"typename Ctx::MaxSum {acc}{{-INFINITY, 0.f}};")
            self.compute.writeline(f"c.online_chunk({acc}, {value});")
            ms = self.cse.generate(self.post_loop_combine, f"c.online_finish({acc})", dtype=torch.float32)
            result = tuple(self.cse.generate(self.post_loop_combine, f"{ms}.{field}", dtype=torch.float32)
                           for field in ("max", "sum"))
            self.outside_loop_vars.update([ms, *result])
            return result
        if reduction_type in ("argmax", "argmin"):
            is_max = "true" if reduction_type == "argmax" else "false"
            if src_dtype in (torch.int32, torch.int64):
                self.body.writeline(f"typename Ctx::ArgPairI {acc} = Ctx::template arg_identity_int<{is_max}>();")
                self.compute.writeline(f"{acc} = Ctx::template arg_better<{is_max}>({acc}, "
                                       f"c.template local_arg_int<{is_max}>({value}));")
                text, out_dtype = f"c.template xreduce_arg_int<{is_max}>({acc})", torch.int64
            else:
                self.body.writeline(f"ixb::ArgPair {acc} = ixb::ArgOp<{is_max}>::identity();")
                self.compute.writeline(f"{acc} = ixb::ArgOp<{is_max}>::combine({acc}, "
                                       f"c.template local_arg<{is_max}>({value}));")
                text, out_dtype = f"c.template xreduce_arg<{is_max}>({acc})", torch.int64
        elif reduction_type == "any":
            self.body.writeline(f"float {acc} = 0.f;")
            self.compute.writeline(f"{acc} = fmaxf({acc}, c.template local_fold<ixb::MaxOp>("
                                   f"ixb::gen::op::where({value}, 1.f, 0.f)));")
            text, out_dtype = f"(c.template xreduce<ixb::MaxOp>({acc}) != 0.f)", torch.bool
        elif reduction_type in REDUCTION_OPS and is_int:
            iop = INT_REDUCTION_OPS[reduction_type]
            self.body.writeline(f"long long {acc} = Ctx::{iop}::id();")
            self.compute.writeline(f"{acc} = Ctx::{iop}::f({acc}, c.template local_fold_int<typename Ctx::{iop}>({value}));")
            text, out_dtype = f"c.template xreduce_int<typename Ctx::{iop}>({acc})", torch.int64
        elif reduction_type in REDUCTION_OPS:
            op = REDUCTION_OPS[reduction_type]
            self.body.writeline(f"float {acc} = {op}::identity();")
            self.compute.writeline(f"{acc} = {op}::combine({acc}, c.template local_fold<{op}>({value}));")
            text, out_dtype = f"c.template xreduce<{op}>({acc})", torch.float32
        else:
            raise UnsupportedByTemplates(f"reduction type {reduction_type} over a row walked in chunks")
        result = self.cse.generate(self.post_loop_combine, text, dtype=out_dtype)
        self.outside_loop_vars.add(result)
        return result

    # ---- sums that ride in the online-softmax exchange -----------------------------------
    # With e = exp(v - max(v)) and S = sum(e) coming out of one exchange, a later
    #   sum(e / S * g + v)  ==  sum(e * g) / S + sum(v)
    # needs no exchange of its own: sum(e * g) and sum(v) can be accumulated per thread before
    # the maximum is known and folded together with S.  A value qualifies when it is a linear
    # combination, with row-scalar coefficients, of (a) e times a vector that does not depend
    # on the exchange and (b) vectors that do not depend on it.
    def _depends_on(self, v, ex, seen=None) -> bool:
        if not isinstance(v, CSEVariable):
            return False
        name = str(v)
        if name in (ex["max"], ex["sum"], ex["var"]) or name in self.online_exp:
            return True
        d = self.dag.get(name)
        if d is None:
            return True          # unknown origin: assume the worst
        if d[0] in ("load", "constant", "index_expr"):
            return False
        if d[0] == "reduction":
            return True
        return any(self._depends_on(a, ex) for a in d[1])

    def _early_text(self, v, ex):
        """Text that names the float vector ``v`` at the point of the exchange ``ex``, or None
        if ``v`` is only defined later."""
        v = self.resolve(v)
        name = str(v)
        if name in self.const_of:
            return self.const_of[name]
        order = list(self.dag)
        if name in self.dag and ex["var"] in self.dag and order.index(name) < order.index(ex["var"]):
            return name if not self.is_scalar(v) else None
        return None

    def _linear_form(self, v, ex, depth=0):
        """[(coefficient text or None, 'e' | 'p', vector text or None)] or None."""
        OPN = "ixb::gen::op::"
        v = self.resolve(v)
        name = str(v)
        if depth > 12 or not self.is_float(v):
            return None
        if self.online_exp.get(name) is ex:
            return [(None, "e", None)]
        if not self._depends_on(v, ex):
            if self.is_scalar(v):
                return None
            t = self._early_text(v, ex)
            return [(None, "p", t)] if t is not None else None
        d = self.dag.get(name)
        if d is None:
            return None
        opn, args = d[0], d[1]

        def scaled(form, factor, divide=False):
            out = []
            for coef, kind, w in form:
                if divide:
                    c = f"{OPN}truediv({coef if coef is not None else '1.0f'}, {factor})"
                else:
                    c = str(factor) if coef is None else f"{OPN}mul({coef}, {factor})"
                out.append((c, kind, w))
            return out

        if opn == "mul" and len(args) == 2:
            for a, b in ((args[0], args[1]), (args[1], args[0])):
                fa = self._linear_form(a, ex, depth + 1)
                if fa is None:
                    continue
                if self.is_scalar(b) and (isinstance(b, CSEVariable) or isinstance(b, (int, float))):
                    return scaled(fa, b)
                if self.is_float(b) and not self._depends_on(b, ex):
                    wt = self._early_text(b, ex)
                    if wt is None:
                        return None
                    return [(coef, kind, wt if w is None else f"{OPN}mul({w}, {wt})") for coef, kind, w in fa]
            return None
        if opn == "truediv" and len(args) == 2 and self.is_scalar(args[1]):
            fa = self._linear_form(args[0], ex, depth + 1)
            return None if fa is None else scaled(fa, args[1], divide=True)
        if opn in ("add", "sub") and len(args) == 2:
            fa = self._linear_form(args[0], ex, depth + 1)
            fb = self._linear_form(args[1], ex, depth + 1)
            if fa is None or fb is None:
                return None
            if opn == "sub":
                fb = [(f"{OPN}neg({c if c is not None else '1.0f'})", kind, w) for c, kind, w in fb]
            return fa + fb
        return None

    def _sum_from_earlier_exchange(self, value):
        if not self.online or not ixb_config.merged_online_softmax:
            return None
        ex = list(self.online.values())[-1]
        form = self._linear_form(value, ex)
        if form is None:
            return None
        ph = self._ph[ex["tag"]]
        rs, rp = list(ph["riders_s"]), list(ph["riders_p"])
        terms = []
        for coef, kind, w in form:
            if kind == "e" and w is None:
                total = ex["sum"]
            elif kind == "e":
                if w not in rs:
                    rs.append(w)
                total = f"{ex['var']}.scaled[{rs.index(w)}]"
            else:
                if w is None:
                    return None
                if w not in rp:
                    rp.append(w)
                total = f"{ex['var']}.plain[{rp.index(w)}]"
            terms.append(total if coef is None else f"ixb::gen::op::mul({coef}, {total})")
        if len(rs) + len(rp) > 2:
            return None
        ph["riders_s"], ph["riders_p"] = rs, rp
        text = terms[0]
        for t in terms[1:]:
            text = f"ixb::gen::op::add({text}, {t})"
        return text

    # ------------------------------------------------------------------ bounds checks
    def check_bounds(self, expr, size, lower, upper) -> None:
        # Negative indices are wrapped by Inductor's lowering.  Range checks are made where the
        # index is formed (B200Overrides.indirect_indexing) in modules generated with
        # config.debug_bounds; otherwise an out-of-range index is the caller's error, as in
        # eager mode.  Nothing is trapped on the device either way.
        return

    # ------------------------------------------------------------------ assembling
    def codegen_body(self) -> None:
        if self.looped and self.inside_reduction:
            if not (self.loads or self.compute or self.stores or self.post_loop_combine or self.post_loop_store):
                return
            # one pass over the row in chunks; everything the pass needs is (re)loaded inside
            self.body.writeline("for (int chunk = 0; chunk < c.nchunks(); ++chunk) {")
            with self.body.indent():
                self.body.writeline("c.set_chunk(chunk);")
                self.body.writeline("const auto r0_index = c.rindex();")
                self.body.writeline("const auto rmask = c.rmask();")
                self.body.splice(self.r_indexing.getvalue())
                self.body.splice(self.loads)
                self.body.splice(self.compute)
                self.body.splice(self.stores)
            self.body.writeline("}")
            self.body.splice(self.post_loop_combine)
            self.body.splice(self.post_loop_store)
            # values from inside the loop are out of scope now: later passes reload
            self.cse.invalidate(self.outside_loop_vars)
            self._ph_by_key.clear()
        else:
            self.body.splice(self.loads)
            self.body.splice(self.compute)
            self.body.splice(self.stores)
            self.body.splice(self.post_loop_combine)
            self.body.splice(self.post_loop_store)
        self.loads.clear()
        self.compute.clear()
        self.stores.clear()
        self.post_loop_combine.clear()
        self.post_loop_store.clear()

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

    # ------------------------------------------------------------------ mapping choice
    def _choose_outer(self, body_text: str) -> bool:
        """Outer mapping iff the group is one ordinary reduction whose reduced axis is not
        stride-1 in any load, at least one load is contiguous along the kept axis, nothing
        r-dependent is stored, and nothing computed inside the reduction loop is used after
        it except the reduction result."""
        import re

        reds = [v for v in self._ph.values() if v["kind"] == "R"]
        if len(reds) != 1 or not reds[0].get("outer_ok"):
            return False
        loads = [v for v in self._ph.values() if v["kind"] == "L" and v["has_r"]]
        if not loads or any(v["indirect"] or v["stride"] in (None, 1) for v in loads):
            return False
        if not any(v["x_contig"] for v in loads):
            return False
        if any(v["kind"] == "S" and v["has_r"] for v in self._ph.values()):
            return False
        marker = next(t for t, v in self._ph.items() if v["kind"] == "R").replace("@R", "@B")
        head, _, tail = body_text.partition(marker)
        defined = set(re.findall(r"const auto (tmp\d+) =", head))
        used_after = set(re.findall(r"\b(tmp\d+)\b", tail))
        return not (defined & used_after)

    def _outer_tx(self) -> int:
        """Threads along the kept axis in the outer mapping: as many as the shortest
        contiguous run among the x-contiguous loads of the reduction holds vectors (so that
        the remaining lanes of a warp walk the reduced axis), at most a warp."""
        xsym = self._root("x").symbol()
        loads = [v for v in self._ph.values() if v["kind"] == "L" and v["has_r"] and v["x_contig"]]
        tx = 32
        while tx > 1:
            span = tx * self._outer_vec
            if span <= self._numel_hint("x") and all(
                    index_ir.vector_access(v["exp"], xsym, span)[0] for v in loads):
                break
            tx //= 2
        return tx

    def _outer_split(self):
        """(threads along the kept axis, cluster size) of the outer mapping.  With fewer tiles
        than SMs and a long reduced axis the tile narrows (down to 64-byte runs) and a cluster
        of up to 8 CTAs shares each tile, combining through distributed shared memory - the
        reference's outer split (inductor_x/codegen/split_tiling.py:159-165) without the trip
        through global memory.  Integer reductions and run-time extents keep one CTA per tile."""
        tx = self._outer_tx()
        red = next(v for v in self._ph.values() if v["kind"] == "R")
        if red.get("is_int") or self._is_dynamic("r0_") or self._is_dynamic("x"):
            return tx, 1
        x, r, vec = self._numel_hint("x"), self._static_numel("r0_"), self._outer_vec
        sms = ixb_config.num_sms
        tiles = lambda t: -(-x // (t * vec))
        elsize = config_bytes(self._narrowest_node_dtype())
        while tx > 1 and tx * vec * elsize > 64 and tiles(tx) * 8 < sms:
            tx //= 2
        cs = 1
        ty = 256 // tx
        while cs < 8 and tiles(tx) * cs * 2 <= 2 * sms and r // (ty * cs * 2) >= 8:
            cs *= 2
        return (tx, cs) if cs > 1 else (self._outer_tx(), 1)

    def _transposing_order(self):
        """Constants of the lane order for a pointwise kernel whose stores are contiguous along
        the flat index but whose strided loads are contiguous along another digit C of it (a
        transpose): consecutive lanes of a warp then step along C, so that each of the V scalar
        loads of a thread is one coalesced request across the warp, while every thread still
        stores one 128-bit vector along the flat index.  This is the job of the reference's
        second set of index variables and ``.permute(1, 0)`` on the tile
        (``inductor_x/codegen/triton.py:856-888, 1303-1332``), done here by the walking order
        alone - the sectors a warp touches on both sides are fully used, without a shared-memory
        tile.  Returns (LB, dC, LC) or None."""
        if self.is_row or self._is_dynamic("x") or not getattr(self, "_gather_loads", None):
            return None
        xsym = self._root("x").symbol()
        xnumel = self._numel_hint("x")
        found = None
        for exp in self._gather_loads:
            split = index_ir._axis_pieces(exp, xsym)
            if split is None or split[0].free_symbols:
                return None
            unit = [(c, d, m) for c, d, m in split[1] if c == 1 and d > 1]
            low = [(c, d, m) for c, d, m in split[1] if d == 1]
            if len(unit) != 1 or len(low) != 1 or low[0][2] is None:
                return None
            lb, (_, dc, lc) = low[0][2], unit[0]
            if lc is None:
                lc = xnumel // dc
            if dc % lb or xnumel % (dc * lc) or lc % 32 or lb % self.vec:
                return None
            if found is not None and found != (lb, dc, lc):
                return None
            found = (lb, dc, lc)
        return found

    def _register_tile(self, order):
        """kC (elements per 128-bit load along C) when every strided load of the group can be
        staged as a register tile under the transposing order ``order``: one storage width, rows
        of the tile 16-byte aligned by construction, extents that the 4 x 8 lane arrangement
        divides.  None keeps the per-element gathers."""
        tl = getattr(self, "_tile_loads", None)
        if order is None or not tl:
            return None
        lb, dc, lc = order
        sizes = {config_bytes(v["dtype"]) for v in tl.values()}
        if len(sizes) != 1 or not all(v["dtype"] in (torch.float32, torch.float16, torch.bfloat16) for v in tl.values()):
            return None
        kc = 16 // sizes.pop()
        xsym = self._root("x").symbol()
        nbv = lb // self.vec
        if lc % (kc * 8) or nbv % 4:
            return None
        for v in tl.values():
            _, pieces = index_ir._axis_pieces(v["exp"], xsym)
            rest = index_ir._axis_pieces(v["exp"], xsym)[0]
            if not rest.is_Integer or int(rest) % kc:
                return None
            if any(c % kc for c, d, m in pieces if not (c == 1 and d == dc)):
                return None
        return kc

    def _short_row_tiling(self):
        """(LB, LC) when the kept index of a short-row kernel should be walked in tiles: the
        kept space is [..][LC][LB] with LB fastest (the output's order), every streamed row
        operand has rows adjacent in memory along the LC digit and far apart along LB, and the
        per-row results are contiguous along LB.  None otherwise."""
        if self.looped or self._is_dynamic("x") or self._is_dynamic("r0_"):
            return None
        xr, rr = self._xr_roots()
        rnumel = self._static_numel("r0_")
        if rnumel * config_bytes(self._narrowest_node_dtype()) > 512:
            return None
        loads = [v for v in self._ph.values() if v["kind"] == "L" and v["has_r"] and not v["indirect"]]
        if not loads or any(v["stride"] != 1 for v in loads):
            return None
        found = None
        for v in loads:
            split = index_ir._axis_pieces(v["exp"].subs({rr.symbol(): 0}), xr.symbol())
            if split is None:
                return None
            pieces = {d: (c, m) for c, d, m in split[1]}
            if 1 not in pieces or pieces[1][1] is None:
                return None
            lb = pieces[1][1]
            if lb not in pieces:
                return None
            coef_c, lc = pieces[lb]
            if lc is None:
                lc = self._numel_hint("x") // lb       # the outermost digit: FloorDiv without modulus
                if self._numel_hint("x") != lb * lc:
                    return None
            if coef_c != rnumel or pieces[1][0] < coef_c * lc or lb % 16 or lc % 16:
                return None
            if found is not None and found != (lb, lc):
                return None
            found = (lb, lc)
        return found

    def _substitute(self, text: str, outer: bool) -> str:
        for tag, v in self._ph.items():
            if v.get("online") and not outer:
                rs, rp = v["riders_s"], v["riders_p"]
                v["row"] = (f"c.template online_softmax<{len(rs)}, {len(rp)}>({v['value']}, "
                            f"{G}refs<kN>({', '.join(rs)}), {G}refs<kN>({', '.join(rp)}))")
            text = text.replace(tag, v["outer"] if outer else v["row"])
        return text

    def codegen_kernel(self, name: Optional[str] = None) -> str:
        self.codegen_body()
        decls, assigns, _ = self._kernel_args()
        xnumel_hint = self._numel_hint("x")
        body_text = self.body.getvalue()
        x_idx, r_idx = self.x_indexing.getvalue(), self.r_indexing.getvalue()
        outer = self.is_row and self._choose_outer(body_text)
        self.mapping = "outer" if outer else ("row" if self.is_row else "pointwise")
        if self.mapping == "row" and not self.looped and not self._is_dynamic("r0_") and \
                self._static_numel("r0_") > self._row_cfg.capacity:
            raise UnsupportedByTemplates(
                f"a strided reduction over {self._static_numel('r0_')} elements that the outer template cannot "
                "take (several reductions or values shared across the reduction loop)")

        src = IndentedBuffer()
        if self.checked_indices:
            src.writeline("#define IXB_DEBUG_BOUNDS 1")
        src.writeline('#include "ixb/gen.cuh"')
        if self.is_row and not outer:
            # The launch shape is a set of macros so that the module loader can build the
            # same body in other shapes (-D...) and keep the one that measures fastest;
            # IXB_GEN_MIN_CTAS bounds the registers and is relaxed by the loader on spills.
            cfg = self._row_cfg
            kregs = min(len(self.consts), MAX_CONST_REGS // max(cfg.elems_per_thread, 1))
            for macro, val in (("IXB_GEN_MIN_CTAS", cfg.min_ctas), ("IXB_ROW_TEAM", cfg.team),
                               ("IXB_ROW_TEAMS", cfg.teams), ("IXB_ROW_VPT", cfg.vpt),
                               ("IXB_ROW_PF", cfg.prefetch), ("IXB_ROW_KREGS", kregs)):
                src.writeline(f"#ifndef {macro}")
                src.writeline(f"#define {macro} {val}")
                src.writeline("#endif")
        src.writeline("namespace {")
        src.writeline("using namespace ixb;")
        src.writeline("struct Body {")
        with src.indent():
            for d in decls:
                src.writeline(d)
            if self.is_row and self._is_dynamic("r0_"):
                src.writeline("long long r_extent;   // reduced extent, known at run time")
            if outer:
                red_tag, red = next((t, v) for t, v in self._ph.items() if v["kind"] == "R")
                marker = red_tag.replace("@R", "@B")
                head, _, tail = body_text.partition(marker)
                rnumel = "r_extent" if self._is_dynamic("r0_") else f"{self._static_numel('r0_')}LL"
                conv = "to_int" if red.get("is_int") else "to_float"
                acc_line = {
                    "sum": "acc = ixb::gen::op::add(acc, ixb::gen::op::{c}({v}));",
                    "prod": "acc = ixb::gen::op::mul(acc, ixb::gen::op::{c}({v}));",
                    "max": "acc = ixb::gen::op::maximum(acc, ixb::gen::op::{c}({v}));",
                    "min": "acc = ixb::gen::op::minimum(acc, ixb::gen::op::{c}({v}));",
                }[red["rtype"]].format(v=red["value"], c=conv)
                src.writeline(f"static constexpr int kVec = {self._outer_vec};")
                src.writeline("template <bool FAST, class Ctx>")
                src.writeline("__device__ __forceinline__ void tile(Ctx& c, const long long xbase, const int nvalid) const {")
                with src.indent():
                    src.writeline(f"const auto xindex = {G}iota<kVec>(xbase);")
                    src.writeline("const auto xmask = xindex < (xbase + nvalid);")
                    src.splice(x_idx)
                    if red.get("is_int"):
                        iop = INT_REDUCTION_OPS[red["rtype"]]
                        src.writeline(f"auto acc = Ctx::template splat_int<kVec>(Ctx::{iop}::id());")
                    else:
                        src.writeline(f"auto acc = Ctx::template splat<kVec>({red['op']}::identity());")
                    import re

                    head_text = self._substitute(head, True)
                    # Full aligned tiles: the plain vector loads of eight reduced steps are issued
                    # as raw 128-bit loads into an array before any of them is widened or used, so
                    # that eight requests per thread are in flight whatever registers the compiler
                    # would have spent on hoisting them itself (it keeps four to five).
                    load_re = re.compile(r"^\s*const auto (tmp\d+) = ixb::gen::ldvec<(ixb::f16|ixb::bf16|float), kVec, FAST>"
                                         r"\((.*), nvalid\);\s*$")
                    loads, rest = [], []
                    for line in head_text.splitlines():
                        m = load_re.match(line)
                        if m and not re.search(r"\btmp\d+\b", m.group(3)):
                            loads.append(m.groups())
                        else:
                            rest.append(line)

                    def plain_loop(start):
                        src.writeline("#pragma unroll 8")
                        src.writeline(f"for (long long r0_index = {start}; r0_index < {rnumel}; r0_index += c.rstep()) {{")
                        with src.indent():
                            src.splice(r_idx)
                            src.splice(head_text)
                            src.writeline(acc_line)
                        src.writeline("}")

                    if loads:
                        src.writeline("if constexpr (FAST) {")
                        with src.indent():
                            src.writeline("long long rb = c.rbegin();")
                            src.writeline(f"for (; rb + 7 * c.rstep() < {rnumel}; rb += 8 * c.rstep()) {{")
                            with src.indent():
                                for name, ctype, _ in loads:
                                    src.writeline(f"{G}RawVec<{ctype}, kVec> raw_{name}[8];")
                                src.writeline("#pragma unroll")
                                src.writeline("for (int u = 0; u < 8; ++u) {")
                                with src.indent():
                                    src.writeline("const long long r0_index = rb + u * c.rstep();")
                                    src.splice(r_idx)
                                    for name, ctype, ptr in loads:
                                        src.writeline(f"raw_{name}[u] = {G}ldraw<{ctype}, kVec>({ptr});")
                                src.writeline("}")
                                src.writeline("#pragma unroll")
                                src.writeline("for (int u = 0; u < 8; ++u) {")
                                with src.indent():
                                    for name, _, _ in loads:
                                        src.writeline(f"{G}pin(raw_{name}[u]);")
                                src.writeline("}")
                                src.writeline("#pragma unroll")
                                src.writeline("for (int u = 0; u < 8; ++u) {")
                                with src.indent():
                                    src.writeline("const long long r0_index = rb + u * c.rstep();")
                                    src.splice(r_idx)
                                    for name, ctype, _ in loads:
                                        src.writeline(f"const auto {name} = {G}widen_raw(raw_{name}[u]);")
                                    src.splice("\n".join(rest))
                                    src.writeline(acc_line)
                                src.writeline("}")
                            src.writeline("}")
                            plain_loop("rb")
                        src.writeline("} else {")
                        with src.indent():
                            plain_loop("c.rbegin()")
                        src.writeline("}")
                    else:
                        plain_loop("c.rbegin()")
                    src.splice(self._substitute(tail, True))
                src.writeline("}")
            elif self.is_row:
                import re

                cfg = self._row_cfg
                tiling = self._short_row_tiling()
                # rows of a whole 128-byte line or more: the output digit runs fastest inside a tile
                b_first = tiling is not None and \
                    self._static_numel("r0_") * config_bytes(self._narrowest_node_dtype()) >= 128
                slot_line = ("const long long xindex = xslot;" if tiling is None else
                             f"const long long xindex = {G}tile_order<{tiling[0]}, {tiling[1]}, 16, 16, "
                             f"{'true' if b_first else 'false'}>(xslot);")
                row_body = re.sub(r"@B\d+@\n?", "", self._substitute(body_text, False))
                # per-column operands, most used first: the first IXB_ROW_KREGS of them are
                # registers, the others are read from the shared-memory table
                order = sorted(range(len(self.consts)), key=lambda j: -row_body.count(self.consts[j][0]))
                for new, old in enumerate(order):
                    row_body = row_body.replace(self.consts[old][0], f"{G}kget<{new}, IXB_ROW_KREGS>(c, k.k{new})")
                src.writeline(f"static constexpr int kN = IXB_ROW_VPT * {cfg.vec};   // elements per thread")
                src.writeline(f"static constexpr bool kLooped = {'true' if self.looped else 'false'};   // row walked in chunks")
                src.writeline(f"static constexpr int kConsts = {len(self.consts)};")
                src.writeline("static constexpr int kSmemConsts = kConsts > IXB_ROW_KREGS ? kConsts - IXB_ROW_KREGS : 0;")
                src.writeline("struct Consts {")
                with src.indent():
                    for new in range(len(order)):
                        src.writeline(f"{G}vf<kN> k{new};")
                src.writeline("};")
                src.writeline("struct Raw {")
                with src.indent():
                    for member, ctype, _ in self.staged:
                        src.writeline(f"{G}RawRow<{ctype}, IXB_ROW_VPT, {cfg.vec}> {member[4:]};")
                src.writeline("};")
                # operands that are the same for every row: once per thread
                src.writeline("template <class Ctx>")
                src.writeline("__device__ __forceinline__ void init(Ctx& c, Consts& k) const {")
                with src.indent():
                    if self.consts:
                        src.writeline("const long long xindex = 0;")
                        src.writeline("const auto r0_index = c.rindex();")
                        src.splice(x_idx)
                        src.splice(r_idx)
                        for new, old in enumerate(order):
                            src.writeline(f"{G}kinit<{new}, IXB_ROW_KREGS>(c, k.k{new}, {self.consts[old][1]});")
                src.writeline("}")
                # raw vectors of the streamed operands of one row (requested a row ahead)
                src.writeline("template <class Ctx>")
                src.writeline("__device__ __forceinline__ void fetch(Ctx& c, const long long xslot, Raw& raw) const {")
                with src.indent():
                    if self.staged:
                        src.writeline(slot_line)
                        src.writeline("const auto r0_index = c.rindex();")
                        src.splice(x_idx)
                        src.splice(r_idx)
                        for member, _, ptr in self.staged:
                            src.writeline(f"c.fetch_row({ptr}, {member});")
                src.writeline("}")
                src.writeline("template <bool STAGED, class Ctx>")
                src.writeline("__device__ __forceinline__ void row(Ctx& c, const Consts& k, const long long xslot, "
                              "const Raw& raw) const {")
                with src.indent():
                    src.writeline(slot_line)
                    if self.looped:
                        src.splice(x_idx)        # the reduced index is defined inside each chunk loop
                    else:
                        src.writeline("const auto r0_index = c.rindex();")
                        src.writeline("const auto rmask = c.rmask();")
                        src.splice(x_idx)
                        src.splice(r_idx)
                    src.splice(row_body)
                src.writeline("}")
                # L2 prefetch of the streamed operands of a later row
                src.writeline("template <class Ctx>")
                src.writeline("__device__ __forceinline__ void prefetch(Ctx& c, const long long xslot) const {")
                with src.indent():
                    if self._row_prefetch:
                        src.writeline(slot_line)
                        src.writeline("const auto r0_index = c.rindex();")
                        src.splice(x_idx)
                        src.splice(r_idx)
                        for ptr in self._row_prefetch:
                            src.writeline(f"c.prefetch_row({ptr});")
                src.writeline("}")
            else:
                src.writeline(f"static constexpr int kVec = {self.vec};")
                order = self._transposing_order()
                kc = self._register_tile(order)
                tile_loads = getattr(self, "_tile_loads", {})
                for n, (tag, v) in enumerate(tile_loads.items()):
                    text = v["gather"] if kc is None else f"(STAGED ? {G}take(raw.t{n}, ci) : {v['gather']})"
                    body_text = body_text.replace(tag, text)
                if kc is not None:
                    lb, dc, lc = order
                    nbv = lb // self.vec
                    src.writeline(f"static constexpr int kTileC = {kc};          // elements per 128-bit load along the loads' axis")
                    src.writeline(f"static constexpr long long kStepC = {dc}LL;   // flat-index distance between output vectors of a tile")
                    src.writeline("struct Tile {")
                    with src.indent():
                        for n, v in enumerate(tile_loads.values()):
                            src.writeline(f"{G}TileRaw<{v['ctype']}, kVec> t{n};")
                    src.writeline("};")
                    src.writeline("__device__ __forceinline__ long long first_of_tile(long long slot) const {")
                    with src.indent():
                        src.writeline("// lanes: 4 vectors along the flat index by 8 tiles along the loads' axis")
                        src.writeline("const long long bv_lo = slot % 4; long long t = slot / 4;")
                        src.writeline("const long long c_lo = t % 8; t /= 8;")
                        src.writeline(f"const long long bv_hi = t % {nbv // 4}; t /= {nbv // 4};")
                        src.writeline(f"const long long mid = t % {dc // lb}; t /= {dc // lb};")
                        src.writeline(f"const long long c_hi = t % {lc // (kc * 8)}; t /= {lc // (kc * 8)};")
                        src.writeline(f"return (bv_hi * 4 + bv_lo) * kVec + mid * {lb}LL + (c_hi * 8 + c_lo) * {kc * dc}LL "
                                      f"+ t * {dc * lc}LL;")
                    src.writeline("}")
                    src.writeline("__device__ __forceinline__ void fetch_tile(const long long xbase, Tile& raw) const {")
                    with src.indent():
                        src.writeline(f"const auto xindex = {G}iota<kVec>(xbase);")
                        src.splice(x_idx)
                        for n, v in enumerate(tile_loads.values()):
                            src.writeline(f"{G}fetch_tile(raw.t{n}, {v['var']}, {v['idx']});")
                    src.writeline("}")
                else:
                    src.writeline("struct Tile {};")
                src.writeline("__device__ __forceinline__ long long first_of(long long slot) const {")
                with src.indent():
                    if order is None:
                        src.writeline("return slot * kVec;")
                    else:
                        lb, dc, lc = order
                        nbv = lb // self.vec
                        tbv = next(t for t in (8, 4, 2, 1) if nbv % t == 0)
                        src.writeline("// lanes along the digit the loads are contiguous in, vectors along the flat index")
                        src.writeline("const long long c_lo = slot % 32; long long t = slot / 32;")
                        src.writeline(f"const long long bv_lo = t % {tbv}; t /= {tbv};")
                        src.writeline(f"const long long bv_hi = t % {nbv // tbv}; t /= {nbv // tbv};")
                        src.writeline(f"const long long mid = t % {dc // lb}; t /= {dc // lb};")
                        src.writeline(f"const long long c_hi = t % {lc // 32}; t /= {lc // 32};")
                        src.writeline(f"return (bv_hi * {tbv} + bv_lo) * kVec + mid * {lb}LL + (c_hi * 32 + c_lo) * {dc}LL "
                                      f"+ t * {dc * lc}LL;")
                src.writeline("}")
                src.writeline("template <bool FAST, bool STAGED = false>")
                src.writeline("__device__ __forceinline__ void tile(const long long xbase, const int nvalid, "
                              "const Tile& raw = Tile(), const int ci = 0) const {")
                with src.indent():
                    src.writeline(f"const auto xindex = {G}iota<kVec>(xbase);")
                    src.writeline("const auto xmask = xindex < (xbase + nvalid);")
                    src.splice(x_idx)
                    src.splice(body_text)
                src.writeline("}")
        src.writeline("};")
        src.writeline("}  // namespace")
        src.writeline('extern "C" int ixb_gen_launch(void** ptrs, const long long* ints, void* stream) {')
        with src.indent():
            src.writeline("Body b;")
            for a in assigns:
                src.writeline(a)
            # the kept extent is always the last integer argument: a literal in the wrapper for a
            # static graph, an expression over the wrapper's size symbols for a dynamic one
            n_int = len([a for a in assigns if 'ints[' in a])
            src.writeline(f"const long long xnumel = ints[{n_int}];")
            if self.is_row and self._is_dynamic("r0_"):
                src.writeline(f"const long long r_extent = ints[{n_int + 1}];")
                src.writeline("b.r_extent = r_extent;")
            if outer:
                tx, cs = self._outer_split()
                launch = f"launch_outer_gen<Body, {tx}>" if cs == 1 else f"launch_outer_split_gen<Body, {tx}, {cs}>"
                src.writeline(f"return {G}{launch}(b, xnumel, stream, "
                              f"{G}pointers_aligned(ptrs, {len([a for a in assigns if 'ptrs[' in a])}));")
            elif self.is_row:
                cfg = self._row_cfg
                dyn_r = self._is_dynamic("r0_")
                rnumel = "(int)r_extent" if dyn_r else str(self._static_numel("r0_"))
                # the type that fixes how many elements one 128-bit vector of the row holds
                narrow = self._narrowest_node_dtype()
                rt = {torch.float32: "float", torch.bfloat16: "ixb::bf16", torch.float16: "ixb::f16"}.get(
                    narrow, f"ixb::Lanes<{cfg.vec}>")
                nptr = len([a for a in assigns if 'ptrs[' in a])
                # FULL: the row fills every vector of the team, no ragged tail to test for
                full = "false" if dyn_r or self.looped else f"IXB_ROW_TEAM * IXB_ROW_VPT * {cfg.vec} == {rnumel}"
                src.writeline(f"constexpr bool kFull = {full};")
                src.writeline(f"return {G}launch_row_gen<Body, {rt}, IXB_ROW_TEAM, IXB_ROW_TEAMS, IXB_ROW_VPT, "
                              f"IXB_GEN_MIN_CTAS, IXB_ROW_PF, kFull>(b, xnumel, {rnumel}, stream, "
                              f"{G}pointers_aligned(ptrs, {nptr}));")
            else:
                launcher = "launch_pointwise_tile" if self._register_tile(self._transposing_order()) else "launch_pointwise"
                src.writeline(f"return {G}{launcher}<Body>(b, xnumel, stream, "
                              f"{G}pointers_aligned(ptrs, {len([a for a in assigns if 'ptrs[' in a])}));")
        src.writeline("}")
        if self.checked_indices:
            src.writeline('extern "C" int ixb_gen_bounds(unsigned long long* out) { '
                          'return ixb::gen::read_bounds_status(out); }')
        text = src.getvalue()
        meta = f"family={self.mapping!r}"
        if self.checked_indices:
            meta += ", bounds=True"
        if self.mapping == "row" and not self._is_dynamic("r0_") and not self.looped:
            cfg = self._row_cfg
            inplace = bool(self.args.inplace_buffers)
            kregs = min(len(self.consts), MAX_CONST_REGS // max(cfg.elems_per_thread, 1))
            shapes = split_tiling.row_candidates(self._static_numel("r0_"), cfg, rows=xnumel_hint,
                                                 n_consts=len(self.consts), kregs=kregs)
            meta += (f", tune=dict(default={(cfg.team, cfg.teams, cfg.vpt, cfg.min_ctas, cfg.prefetch, kregs)!r}, "
                     f"candidates={shapes!r}, rows={xnumel_hint}, row_bytes={self._static_numel('r0_') * config_bytes(self._narrowest_node_dtype())}, "
                     f"idempotent={not inplace!r})")
        return f"ixb_load_kernel('''\n{text}''', {meta})"

    def call_kernel(self, name: str, node: Any = None, deallocate_ws: bool = True) -> None:
        wrapper = V.graph.wrapper_code
        for v in self.args.sizevars:
            wrapper.ensure_size_computed(v)
        _, call_args, _, _ = self.args.python_argdefs()
        numel = V.graph.sizevars.simplify(self.numels.get("x", sympy.S.One))
        for sym in sorted(numel.free_symbols, key=str):
            wrapper.ensure_size_computed(sym)
        call_args = [*call_args, self.pexpr(numel)]
        if self.is_row and self._is_dynamic("r0_"):
            rn = V.graph.sizevars.simplify(self.numels["r0_"])
            for sym in sorted(rn.free_symbols, key=str):
                wrapper.ensure_size_computed(sym)
            call_args.append(self.pexpr(rn))
        device = V.graph.get_current_device_or_throw()
        if device.type == "cuda":
            stream = wrapper.write_get_raw_stream(device.index, V.graph.name)
            wrapper.writeline(f"{name}.run({', '.join(map(str, call_args))}, stream={stream})")
        else:
            wrapper.writeline(f"{name}.run({', '.join(map(str, call_args))}, stream=None)")

    def codegen_nan_check(self) -> None:
        return
