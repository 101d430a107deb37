"""Index-expression analysis for the template instantiator.

Inductor hands a kernel flattened iteration ranges and index expressions written with
``FloorDiv`` / ``ModularIndexing`` of those flat variables.  The reference recovers the
true axes by rewriting such pairs into real loop variables
(``inductor_x/codegen/ir.py:26-146``: ``detect_flattened_dims``, ``rebuild_flattened_dims``,
``substituted_dims_in_indexing``) and then looks for the axes that are stride-1 in some
access (``find_lowest_dimension``, ``inductor_x/codegen/split_tiling.py:188-239``).  The
CUDA templates need the same two facts in a different form:

* is an access *contiguous along the flat vector a thread owns* (128-bit access), and
* is an access *contiguous along the reduced row* (row template) - and if not, what is the
  stride of the reduced variable (outer reduction).

Both are answered on the expression expanded back to the root index variables.  The
vector questions are decided structurally (``vector_access``): the expression must be a sum
of integer multiples of ``root``, ``ModularIndexing(root, d, m)`` and ``FloorDiv(root, d)``
whose break points all fall on vector boundaries, which makes it affine inside every
aligned vector; exact evaluation at sample points then cross-checks that decision.
"""
from __future__ import annotations

import random
from typing import Dict, Iterable, Optional, Sequence

import sympy


def num_splits(*args, **kwargs):
    """Replacement of ``torch._inductor.ir.Reduction.num_splits``
    (``inductor_x/codegen/ir.py:13-24`` forces one split everywhere).  Inductor cuts a long
    reduction with few outputs into two kernels through a scratch tensor.  The outer template
    covers that case on chip - a cluster of CTAs per tile, partials combined through
    distributed shared memory - so the cut is kept only where the kept extent is too small to
    spread over the GPU even with clusters (a handful of outputs), or when
    ``config.allow_multilayer_reduction`` asks for the stock behaviour."""
    from torch._inductor.virtualized import V

    from .. import config

    hint, split = _stock_num_splits(*args, **kwargs)
    if config.allow_multilayer_reduction or kwargs.get("reduction_type", args[6] if len(args) > 6 else None) == "scan":
        return hint, split
    try:
        ranges = kwargs.get("ranges", args[4] if len(args) > 4 else ())
        device = kwargs.get("device", args[0] if args else None)
        kept = 1
        for r in ranges:
            kept *= int(V.graph.sizevars.size_hint(r))
        if getattr(device, "type", None) == "cuda" and int(split) > 1 and kept >= config.min_kept_for_single_kernel:
            return hint, 1
    except Exception:
        pass
    return hint, split


_stock_num_splits = None


def install_num_splits():
    """Patch ``Reduction.num_splits`` once (kept callable as a static method)."""
    global _stock_num_splits
    from torch._inductor import ir as inductor_ir

    if _stock_num_splits is None:
        _stock_num_splits = inductor_ir.Reduction.num_splits
        inductor_ir.Reduction.num_splits = staticmethod(num_splits)


def expand_to_roots(index: sympy.Expr, range_tree_nodes: Dict[sympy.Symbol, object]) -> sympy.Expr:
    """Rewrite ``index`` so that only root index symbols (``xindex``, ``r0_index`` ...) and
    non-range symbols remain.  ``range_tree_nodes`` maps entry symbols to entries whose
    ``.expr`` is written in terms of their root symbol."""
    for _ in range(8):
        syms = [s for s in index.free_symbols if s in range_tree_nodes]
        if not syms:
            break
        index = index.subs({s: range_tree_nodes[s].expr for s in syms})
    return index


def _eval(expr: sympy.Expr, env: Dict[sympy.Symbol, int]) -> Optional[int]:
    try:
        v = expr.subs(env)
        return int(v) if v.is_Integer else None
    except Exception:
        return None


def _sample_bases(numel: int, group: int, n: int = 12) -> Iterable[int]:
    groups = max(numel // group, 1)
    rnd = random.Random(1234)
    picks = {0, 1, 2, groups - 1, groups // 2, groups // 3}
    while len(picks) < min(n, groups):
        picks.add(rnd.randrange(groups))
    return [g * group for g in sorted(picks) if 0 <= g < groups]


def vector_access(expr: sympy.Expr, root: sympy.Symbol, vec: int):
    """(contiguous, aligned) of the ``vec`` elements ``root = b .. b + vec - 1`` for every
    ``b`` that is a multiple of ``vec``, decided from the structure of ``expr``; (False,
    False) when the structure is not one this analysis understands.

    contiguous: ``expr(b + k) == expr(b) + k``; aligned: ``expr(b)`` is a multiple of
    ``vec``.  Symbols other than ``root`` (the reduced index of an outer reduction) may
    appear in terms that do not involve ``root``; such terms must carry a coefficient that
    is a multiple of ``vec`` for the access to count as aligned."""
    from torch.utils._sympy.functions import FloorDiv, ModularIndexing

    unit = 0          # total coefficient of the terms that advance by one per element
    aligned = True
    for term in sympy.Add.make_args(sympy.expand(expr)):
        coeff, atom = term.as_coeff_Mul()
        if not coeff.is_Integer:
            return False, False
        coeff = int(coeff)
        if atom == 1:
            aligned &= coeff % vec == 0
        elif root not in atom.free_symbols:
            aligned &= coeff % vec == 0           # any integer-valued function of other symbols
        elif atom == root:
            unit += coeff
        elif isinstance(atom, ModularIndexing) and atom.args[0] == root and all(a.is_Integer for a in atom.args[1:]):
            d, m = int(atom.args[1]), int(atom.args[2])
            if d % vec == 0:
                aligned &= coeff % vec == 0       # constant inside a vector
            elif d == 1 and m % vec == 0:
                unit += coeff                     # advances without wrapping inside a vector
            else:
                return False, False
        elif isinstance(atom, FloorDiv) and atom.args[0] == root and atom.args[1].is_Integer:
            if int(atom.args[1]) % vec != 0:
                return False, False
            aligned &= coeff % vec == 0
        else:
            return False, False
    return unit == 1, bool(aligned and unit == 1)


def is_vector_constant(expr: sympy.Expr, root: sympy.Symbol, vec: int) -> bool:
    """True when ``expr`` takes one value over every aligned group of ``vec`` consecutive
    values of ``root`` (for instance ``FloorDiv(root, 128)`` with ``vec`` 8)."""
    from torch.utils._sympy.functions import FloorDiv, ModularIndexing

    if expr.free_symbols - {root}:
        return False
    for term in sympy.Add.make_args(sympy.expand(expr)):
        coeff, atom = term.as_coeff_Mul()
        if not coeff.is_Integer:
            return False
        if atom == 1:
            continue
        if isinstance(atom, ModularIndexing) and atom.args[0] == root and all(a.is_Integer for a in atom.args[1:]):
            if int(atom.args[1]) % vec != 0:
                return False
        elif isinstance(atom, FloorDiv) and atom.args[0] == root and atom.args[1].is_Integer:
            if int(atom.args[1]) % vec != 0:
                return False
        else:
            return False
    return True


def is_vector_contiguous(expr: sympy.Expr, root: sympy.Symbol, vec: int, numel: int) -> bool:
    """True when, for every flat position b that is a multiple of ``vec``,
    ``expr(b + k) == expr(b) + k`` for k < vec: the ``vec`` elements a thread owns are
    adjacent in memory.  ``expr`` must contain no symbol other than ``root``."""
    if expr.free_symbols - {root}:
        return False
    if numel < vec:
        return False
    if not vector_access(expr, root, vec)[0]:
        return False
    for b in _sample_bases(numel, vec):
        if b + vec > numel:
            continue
        base = _eval(expr, {root: b})
        if base is None:
            return False
        for k in range(1, vec):
            if _eval(expr, {root: b + k}) != base + k:
                return False
    return True


def _axis_pieces(expr: sympy.Expr, root: sympy.Symbol):
    """Split ``expr`` into (rest, pieces): ``pieces`` lists ``(coeff, divisor, modulus)`` for
    every term that is an integer multiple of ``root``, ``FloorDiv(root, d)`` or
    ``ModularIndexing(root, d, m)`` (modulus None when absent); ``rest`` is the sum of the
    terms free of ``root``.  None when ``root`` occurs in any other shape."""
    from torch.utils._sympy.functions import FloorDiv, ModularIndexing

    rest = sympy.S.Zero
    pieces = []
    for term in sympy.Add.make_args(sympy.expand(expr)):
        if root not in term.free_symbols:
            rest += term
            continue
        coeff, atom = term.as_coeff_Mul()
        if not coeff.is_Integer:
            return None
        if atom == root:
            pieces.append((int(coeff), 1, None))
        elif isinstance(atom, ModularIndexing) and atom.args[0] == root and all(a.is_Integer for a in atom.args[1:]):
            pieces.append((int(coeff), int(atom.args[1]), int(atom.args[2])))
        elif isinstance(atom, FloorDiv) and atom.args[0] == root and atom.args[1].is_Integer:
            pieces.append((int(coeff), int(atom.args[1]), None))
        else:
            return None
    return rest, pieces


def reduction_stride(expr: sympy.Expr, x_root: sympy.Symbol, r_root: sympy.Symbol, xnumel: int,
                     rnumel: int) -> Optional[int]:
    """Stride of the flat reduction variable in ``expr`` if it is one constant over the
    whole range (``expr(x, r) == expr(x, 0) + stride * r``), else None.  Stride 1 means the
    access walks the row contiguously (row template); a larger constant stride means an
    outer reduction; None means the reduced range is itself a flattening of several axes
    with different strides, or has a shape this analysis does not understand.

    Decided from the structure of the expression: the terms in ``r`` must be digits of a
    mixed-radix split of ``r`` - ``ModularIndexing(r, d_i, m_i)`` with ``d_0 == 1`` and
    ``d_{i+1} == d_i * m_i``, the last one reaching the end of the range - and digit ``i``
    must carry the coefficient ``stride * d_i``.  Then the sum is ``stride * r`` exactly."""
    if expr.free_symbols - {x_root, r_root}:
        return None
    if r_root not in expr.free_symbols:
        return 0
    if rnumel == 1:
        return 1
    split = _axis_pieces(expr, r_root)
    if split is None:
        return None
    _, pieces = split
    merged: Dict[tuple, int] = {}
    for coeff, d, m in pieces:
        if m is not None and d * m >= rnumel:
            m = None                       # the modulus never wraps inside the range
        merged[(d, m)] = merged.get((d, m), 0) + coeff
    digits = sorted(merged.items(), key=lambda kv: kv[0][0])
    if not digits or digits[0][0][0] != 1:
        return None
    stride = digits[0][1]
    reach = 1
    for (d, m), coeff in digits:
        if d != reach or coeff != stride * d:
            return None
        if m is None:
            reach = None
            break
        reach = d * m
    if reach is not None and reach < rnumel:
        return None
    if digits[-1][0][1] is not None and reach is not None:
        return None
    # nothing may follow the digit that reaches the end of the range
    last_open = [i for i, ((d, m), _) in enumerate(digits) if m is None]
    if last_open and last_open[0] != len(digits) - 1:
        return None
    return stride


def row_starts_aligned(expr: sympy.Expr, x_root: sympy.Symbol, r_root: sympy.Symbol, vec: int) -> bool:
    """True when the element offset of every row start (``r == 0``) is a multiple of
    ``vec``: every term in the kept index carries a coefficient that is a multiple of
    ``vec``, and so does the constant.  With a 16-byte aligned base pointer each row then
    starts on a 16-byte boundary."""
    if expr.free_symbols - {x_root, r_root}:
        return False
    at0 = expr.subs({r_root: 0}) if r_root in expr.free_symbols else expr
    split = _axis_pieces(at0, x_root)
    if split is None:
        return False
    rest, pieces = split
    if rest.free_symbols or not rest.is_Integer or int(rest) % vec != 0:
        return False
    return all(coeff % vec == 0 for coeff, _, _ in pieces)


def x_contiguous_for_all_r(expr: sympy.Expr, x_root: sympy.Symbol, r_root: sympy.Symbol, vec: int) -> bool:
    """Vector contiguity along the kept index for every value of the reduced index: the
    terms in ``x`` must be vector-contiguous by structure (``vector_access``) and no term
    may mix the two indices."""
    if expr.free_symbols - {x_root, r_root}:
        return False
    split = _axis_pieces(expr, r_root)
    if split is None:
        return False
    rest, _ = split
    if r_root in rest.free_symbols or x_root not in rest.free_symbols:
        return False
    return vector_access(rest, x_root, vec)[0]


def x_stride_at_row_start(expr: sympy.Expr, x_root: sympy.Symbol, r_root: sympy.Symbol,
                          xnumel: int) -> Optional[int]:
    """For a row-contiguous access: distance between the starts of consecutive rows, if it
    is constant (it is ``rnumel`` for a dense operand, 0 for a broadcast row vector)."""
    if xnumel <= 1:
        return 0
    env0 = {r_root: 0}
    base = _eval(expr, {**env0, x_root: 0})
    if base is None:
        return None
    s = None
    for x in sorted({1, 2, xnumel - 1, xnumel // 2} & set(range(1, xnumel))):
        v = _eval(expr, {**env0, x_root: x})
        if v is None or (v - base) % x != 0:
            return None
        cur = (v - base) // x
        if s is None:
            s = cur
        elif cur != s:
            return None
    return s
