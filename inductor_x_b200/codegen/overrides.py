"""Op -> C++ text for generated functor bodies, and the sympy printer for index math.

Every op prints as a call into ``ixb::gen::op`` (``csrc/ixb/gen_ops.cuh``), which is
overloaded for scalars and per-thread vectors, so the text is the same whichever rank the
operands turn out to have.  Counterpart of ``NPUTritonKernelOverrides``
(``inductor_x/codegen/triton.py:99-112``) and of the Ascend libdevice shims
(``inductor_x/npu_triton_helpers.py:4-18``).
"""
from __future__ import annotations

import math

import sympy
import torch
from torch._inductor.codegen.common import OpOverrides
from torch._inductor.virtualized import V, ops
from torch.utils._sympy.printers import ExprPrinter

OP = "ixb::gen::op::"

FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)

CPP_TYPE = {
    torch.float32: "float", torch.float16: "ixb::f16", torch.bfloat16: "ixb::bf16",
    torch.float64: "double", torch.int64: "long long", torch.int32: "int", torch.int16: "short",
    torch.int8: "signed char", torch.uint8: "unsigned char", torch.bool: "bool",
}


def float_literal(val: float) -> str:
    if math.isnan(val):
        return "NAN"
    if math.isinf(val):
        return "INFINITY" if val > 0 else "(-INFINITY)"
    r = repr(float(val))
    if "e" not in r and "." not in r:
        r += ".0"
    return f"{r}f"


def constant_literal(val, dtype: torch.dtype) -> str:
    if dtype == torch.bool:
        return "true" if val else "false"
    if dtype in INT_DTYPES:
        if int(val) <= -(1 << 63):
            return "(-9223372036854775807LL - 1)"      # the literal 9223372036854775808 has no signed type
        return f"{int(val)}LL"
    return float_literal(float(val))


class IxbExprPrinter(ExprPrinter):
    """Index expressions as C++ over scalars or ``vi<N>`` (operators + ixb::gen::op calls)."""

    def _print_Integer(self, expr):
        return f"{int(expr)}LL"

    def _print_Float(self, expr):
        return float_literal(float(expr))

    def _print_FloorDiv(self, expr):
        x, d = expr.args
        return f"{OP}idiv({self.doprint(x)}, {self.doprint(d)})"

    def _print_ModularIndexing(self, expr):
        x, d, m = expr.args
        xs = self.doprint(x)
        if d != 1:
            xs = f"{OP}idiv({xs}, {self.doprint(d)})"
        return f"{OP}imod({xs}, {self.doprint(m)})"

    def _print_Min(self, expr):
        out = self.doprint(expr.args[0])
        for a in expr.args[1:]:
            out = f"{OP}minimum({out}, {self.doprint(a)})"
        return out

    def _print_Max(self, expr):
        out = self.doprint(expr.args[0])
        for a in expr.args[1:]:
            out = f"{OP}maximum({out}, {self.doprint(a)})"
        return out

    def _print_Abs(self, expr):
        return f"{OP}abs({self.doprint(expr.args[0])})"

    def _print_Where(self, expr):
        c, a, b = (self.doprint(x) for x in expr.args)
        return f"{OP}where({c}, {a}, {b})"

    def _print_PowByNatural(self, expr):
        base, exp = expr.args
        b = self.doprint(base)
        return "(" + " * ".join([f"({b})"] * int(exp)) + ")" if int(exp) > 0 else "1LL"

    def _print_Pow(self, expr):
        base, exp = expr.args
        if exp.is_Integer and int(exp) > 0:
            b = self.doprint(base)
            return "(" + " * ".join([f"({b})"] * int(exp)) + ")"
        raise NotImplementedError(f"index power {expr}")

    def _print_ToFloat(self, expr):
        return f"{OP}to_float({self.doprint(expr.args[0])})"

    def _print_TruncToInt(self, expr):
        return f"{OP}to_int({self.doprint(expr.args[0])})"

    def _print_FloorToInt(self, expr):
        return f"{OP}to_int({OP}floor({self.doprint(expr.args[0])}))"

    def _print_Identity(self, expr):
        return self.doprint(expr.args[0])

    # ---- forms that appear with run-time extents (symbolic sizes) -----------------------
    def _fn(self, name, expr):
        return f"{OP}{name}({', '.join(self.doprint(a) for a in expr.args)})"

    def _print_Mod(self, expr):                     # operands known non-negative
        return self._fn("imod", expr)

    def _print_PythonMod(self, expr):               # sign of the divisor, as Python's %
        return self._fn("remainder", expr)

    def _print_IntTrueDiv(self, expr):
        a, b = (self.doprint(x) for x in expr.args)
        return f"{OP}truediv({OP}to_float({a}), {OP}to_float({b}))"

    def _print_FloatTrueDiv(self, expr):
        return self._fn("truediv", expr)

    def _print_FloatPow(self, expr):
        return self._fn("pow", expr)

    def _print_Rational(self, expr):
        return float_literal(float(expr.p) / float(expr.q))

    def _print_CeilToInt(self, expr):
        return f"{OP}to_int({OP}ceil({self.doprint(expr.args[0])}))"

    def _print_RoundToInt(self, expr):
        return f"{OP}to_int({OP}round({self.doprint(expr.args[0])}))"

    def _print_TruncToFloat(self, expr):
        return self._fn("trunc", expr)

    def _print_floor(self, expr):
        return f"{OP}to_int({OP}floor({self.doprint(expr.args[0])}))"

    def _print_ceiling(self, expr):
        return f"{OP}to_int({OP}ceil({self.doprint(expr.args[0])}))"

    def _print_Not(self, expr):
        return self._fn("logical_not", expr)

    def _print_BooleanTrue(self, expr):
        return "true"

    def _print_BooleanFalse(self, expr):
        return "false"

    def _print_Infinity(self, expr):
        return "INFINITY"

    def _print_NegativeInfinity(self, expr):
        return "(-INFINITY)"


for _fn_name in ("sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh", "asin", "acos", "atan", "log2"):
    setattr(IxbExprPrinter, f"_print_OpaqueUnaryFn_{_fn_name}",
            (lambda name: lambda self, expr: self._fn(name, expr))(_fn_name))


def _call(name):
    def fn(*args):
        return f"{OP}{name}({', '.join(str(a) for a in args)})"

    return staticmethod(fn)


# Integers are carried in 64 bits whatever their storage type.  A value that can leave the
# range of its type (a narrowing conversion, a left shift, the complement of an unsigned byte)
# is wrapped back, so that what is computed from it next matches the stored value.
_INT_RANGE = {torch.bool: (1, False), torch.uint8: (8, False), torch.int8: (8, True), torch.int16: (16, True),
              torch.int32: (32, True), torch.int64: (64, True)}


def _fits(src, dst) -> bool:
    """Whether every value of integer type ``src`` is a value of integer type ``dst``."""
    if src not in _INT_RANGE or dst not in _INT_RANGE:
        return False
    (sb, ss), (db, ds) = _INT_RANGE[src], _INT_RANGE[dst]
    return src == dst or (sb < db and (ds or not ss))


def _wrap(expr: str, dtype) -> str:
    bits, signed = _INT_RANGE.get(dtype, (64, True))
    if bits >= 64 or dtype == torch.bool:
        return expr
    return f"{OP}wrap_int<{bits}, {'true' if signed else 'false'}>({expr})"


def _dtype_of(v):
    if isinstance(v, bool):
        return torch.bool
    if isinstance(v, int):
        return torch.int64
    if isinstance(v, float):
        return torch.float32
    return getattr(v, "int_type", None) or getattr(v, "dtype", None)


def _narrow_int_result(*vals):
    """The integer type narrower than 64 bits that eager mode gives the result of an
    arithmetic op on ``vals`` (None when the result is not such an integer)."""
    out = None
    for v in vals:
        if isinstance(v, (bool, int)):
            continue                       # Python scalars do not take part in the promotion
        t = _dtype_of(v)
        if t == torch.bool:
            continue
        if t not in INT_DTYPES:
            return None
        out = t if out is None else torch.promote_types(out, t)
    return out if out in _INT_RANGE and _INT_RANGE[out][0] < 64 else None


def _bitwise(logical: str, bitwise: str):
    """and / or / xor: the logical form for booleans, the bit pattern for integers."""

    def fn(a, b):
        da, db = _dtype_of(a), _dtype_of(b)
        if da in FLOAT_DTYPES or db in FLOAT_DTYPES:
            raise NotImplementedError(f"{bitwise} of floating operands")
        if da in (torch.bool, None) and db in (torch.bool, None):
            return f"{OP}{logical}({a}, {b})"
        return f"{OP}{bitwise}({a}, {b})"

    return staticmethod(fn)


class B200Overrides(OpOverrides):
    """Text of each pointwise op.  Floating math is fp32 whatever the storage type."""

    @staticmethod
    def to_dtype(x, dtype, src_dtype=None, use_compute_types=True):
        if dtype == torch.bool:
            return f"{OP}to_bool({x})"
        if dtype in INT_DTYPES:
            src = src_dtype if src_dtype is not None else _dtype_of(x)
            if src in FLOAT_DTYPES or _fits(src, dtype):
                return f"{OP}to_int({x})"     # (a float outside the range is undefined in eager mode too)
            return _wrap(f"{OP}to_int({x})", dtype)
        return f"{OP}to_float({x})"

    @staticmethod
    def to_dtype_bitcast(x, dtype, src_dtype):
        raise NotImplementedError("to_dtype_bitcast is not instantiable from the B200 templates")

    @staticmethod
    def constant(val, dtype):
        return constant_literal(val, dtype)

    @staticmethod
    def index_expr(expr, dtype):
        idx = V.kernel.index_to_str(V.kernel.prepare_indexing(expr))
        var = V.kernel.cse.generate(V.kernel.compute, idx, dtype=torch.int64)
        if dtype in FLOAT_DTYPES:
            return f"{OP}to_float({var})"
        return str(var)

    @staticmethod
    def indirect_indexing(var, size, check=True, wrap_neg=True):
        from torch._inductor.utils import sympy_index_symbol

        from .. import config as ixb_config

        if ixb_config.debug_bounds and check and hasattr(V.kernel, "checked_indices"):
            # debug build: count a violation, keep the access inside the buffer
            bound = V.kernel.sexpr(V.kernel.rename_indexing(sympy.sympify(size)))
            var = V.kernel.cse.generate(V.kernel.compute, f"ixb::gen::checked_index({var}, {bound})",
                                        dtype=torch.int64)
            V.kernel.checked_indices += 1
        return sympy_index_symbol(str(var))

    @staticmethod
    def masked(mask, body, other):
        with V.kernel.mask_loads(mask, other) as new_mask:
            result = body()
        if isinstance(other, (int, float, bool)):
            dtype = getattr(result, "dtype", None) or torch.float32
            other = V.ops.constant(other, dtype)
        # the raw handler (not the OpsValue wrapper): callers read .dtype of the result
        return V.ops.where(new_mask, result, other)

    bitwise_and = _bitwise("logical_and", "bit_and")
    bitwise_or = _bitwise("logical_or", "bit_or")
    bitwise_xor = _bitwise("logical_xor", "bit_xor")

    @staticmethod
    def bitwise_not(a):
        da = _dtype_of(a)
        if da in (torch.bool, None):
            return f"{OP}logical_not({a})"
        if da in FLOAT_DTYPES:
            raise NotImplementedError("bitwise_not of a floating operand")
        return _wrap(f"{OP}bit_not({a})", da if da == torch.uint8 else torch.int64)

    @staticmethod
    def bitwise_left_shift(a, b):
        return _wrap(f"{OP}lshift({a}, {b})", _narrow_int_result(a))

    @staticmethod
    def bitwise_right_shift(a, b):
        return f"{OP}rshift({a}, {b})"

    @staticmethod
    def and_(a, b):
        return f"{OP}logical_and({a}, {b})"

    @staticmethod
    def or_(a, b):
        return f"{OP}logical_or({a}, {b})"

    @staticmethod
    def load_seed(name, offset):
        raise NotImplementedError("random number ops are not instantiable from the B200 templates")


def _kernel():
    k = V.kernel
    return k if hasattr(k, "dag") else None


def _floats(k, *vals) -> bool:
    return all(k.is_float(v) or isinstance(v, float) for v in vals) and any(k.is_float(v) for v in vals)


class _Peephole:
    """Rewrites applied while the op text is printed.  They do what a compiler does for
    scalar code but cannot do across the packed-pair instructions the vector ops are made
    of: contraction of a*b+c into one fused multiply-add, folding of row-scalar factors into
    one scalar so that a vector is multiplied once, exp(a - rowmax) from the exponentials the
    online-softmax exchange already holds, and the decomposed exact GELU as one call."""

    @staticmethod
    def add(a, b):
        k = _kernel()
        if k is not None and _floats(k, a, b):
            for p, q in ((a, b), (b, a)):
                m = k.op_of(p, "mul")
                if m is not None and _floats(k, *m):
                    return f"{OP}fma({m[0]}, {m[1]}, {q})"
        return _wrap(f"{OP}add({a}, {b})", _narrow_int_result(a, b))

    @staticmethod
    def sub(a, b):
        k = _kernel()
        if k is not None and _floats(k, a, b):
            m = k.op_of(a, "mul")
            if m is not None and _floats(k, *m) and k.is_scalar(b):
                return f"{OP}fma({m[0]}, {m[1]}, {OP}neg({b}))"
        return _wrap(f"{OP}sub({a}, {b})", _narrow_int_result(a, b))

    @staticmethod
    def _gelu(k, a, b):
        """a == v * 0.5 and b == erf(v * sqrt(1/2)) + 1  ->  v"""
        ma, sb = k.op_of(a, "mul"), k.op_of(b, "add")
        if ma is None or sb is None:
            return None
        for v, half in ((ma[0], ma[1]), (ma[1], ma[0])):
            if k.const_value(half) != 0.5:
                continue
            for e, one in ((sb[0], sb[1]), (sb[1], sb[0])):
                if k.const_value(one) != 1.0:
                    continue
                inner = k.op_of(e, "erf")
                me = k.op_of(inner[0], "mul") if inner is not None else None
                if me is None:
                    continue
                for v2, c in ((me[0], me[1]), (me[1], me[0])):
                    cv = k.const_value(c)
                    if cv is not None and abs(cv - 0.7071067811865476) < 1e-12 and \
                            str(k.resolve(v2)) == str(k.resolve(v)):
                        return v
        return None

    @staticmethod
    def mul(a, b):
        k = _kernel()
        if k is not None and _floats(k, a, b):
            for p, q in ((a, b), (b, a)):
                v = _Peephole._gelu(k, p, q)
                if v is not None:
                    k.pending_dag = ("gelu_erf", (v,), {})
                    return f"{OP}gelu_erf({v})"
            # (vector * s1) * s2 -> vector * (s1 * s2); (vector / s1) * s2 -> vector * (s2 / s1)
            for p, q in ((a, b), (b, a)):
                if not k.is_scalar(q) or k.is_scalar(p):
                    continue
                m = k.op_of(p, "mul")
                if m is not None and _floats(k, *m):
                    for v, s1 in ((m[0], m[1]), (m[1], m[0])):
                        if k.is_scalar(s1) and not k.is_scalar(v):
                            return f"{OP}mul({v}, {OP}mul({s1}, {q}))"
                d = k.op_of(p, "truediv")
                if d is not None and _floats(k, *d) and k.is_scalar(d[1]) and not k.is_scalar(d[0]):
                    return f"{OP}mul({d[0]}, {OP}truediv({q}, {d[1]}))"
        return _wrap(f"{OP}mul({a}, {b})", _narrow_int_result(a, b))

    @staticmethod
    def truediv(a, b):
        k = _kernel()
        if k is not None and _floats(k, a, b) and k.is_scalar(b) and not k.is_scalar(a):
            ex = k.online_exp.get(str(k.resolve(a)))
            if ex is not None:
                # exp(v - max) / s: the thread's exponentials times one scalar
                return f"{OP}mul({ex['var']}.e, {OP}truediv({ex['var']}.r, {b}))"
            m = k.op_of(a, "mul")
            if m is not None and _floats(k, *m):
                for v, s1 in ((m[0], m[1]), (m[1], m[0])):
                    if k.is_scalar(s1) and not k.is_scalar(v):
                        return f"{OP}mul({v}, {OP}truediv({s1}, {b}))"
        return f"{OP}truediv({a}, {b})"

    @staticmethod
    def exp(a):
        k = _kernel()
        if k is not None and k.is_float(a):
            s = k.op_of(a, "sub")
            if s is not None and _floats(k, *s):
                ex = k.online.get(str(k.resolve(s[0])))
                if ex is not None and str(s[1]) == ex["max"]:
                    k.pending_online_exp = ex
                    return f"{OP}mul({ex['var']}.e, {ex['var']}.r)"
                if k.is_scalar(s[1]) and not k.is_scalar(s[0]) and k.half_group():
                    return f"{OP}exp_sub({s[0]}, {s[1]})"
        return f"{OP}exp({a})"


for _name in ["exp", "exp2", "expm1", "log", "log2", "log10", "log1p", "sqrt", "rsqrt", "sin", "cos",
              "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh", "asinh", "acosh", "atanh", "erf", "erfc",
              "erfinv", "nextafter", "ldexp", "lgamma", "floor",
              "ceil", "trunc", "round", "reciprocal", "sigmoid", "abs", "neg", "square", "relu",
              "sign", "isnan", "isinf", "signbit", "truediv", "pow", "fmod", "atan2", "copysign",
              "hypot", "add", "sub", "mul", "maximum", "minimum", "floordiv", "truncdiv",
              "remainder", "logical_and", "logical_or", "logical_xor", "logical_not", "eq", "ne",
              "lt", "le", "gt", "ge", "where"]:
    setattr(B200Overrides, _name, _call(_name))
for _name in ["add", "sub", "mul", "truediv", "exp"]:
    setattr(B200Overrides, _name, staticmethod(getattr(_Peephole, _name)))
for _name in ("neg", "abs", "square"):        # -x, |x| and x * x of the most negative value leave the range too
    setattr(B200Overrides, _name,
            staticmethod((lambda n: lambda a: _wrap(f"{OP}{n}({a})", _narrow_int_result(a)))(_name)))
B200Overrides.mod = _call("mod")
B200Overrides.fma = _call("fma")
B200Overrides.mul_rn = _call("mul")       # a product that is never contracted: its name keeps it out of the fma peephole
B200Overrides.int_truediv = _call("truediv")
B200Overrides.libdevice_exp = staticmethod(_Peephole.exp)
B200Overrides.libdevice_sqrt = _call("sqrt")
B200Overrides.libdevice_log = _call("log")
B200Overrides.libdevice_sigmoid = _call("sigmoid")
B200Overrides.libdevice_abs = _call("abs")
