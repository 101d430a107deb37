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


def _call(name):
    def fn(*args):
        return f"{OP}{name}({', '.join(str(a) for a in args)})"

    return staticmethod(fn)


class B200Overrides(OpOverrides):
    """Text of each pointwise op.  Floating math is fp32 whatever the storage type."""

    @staticmethod
    def to_dtype(x, dtype, src_dtype=None, use_compute_types=True):
        if dtype == torch.bool:
            return f"{OP}to_bool({x})"
        if dtype in INT_DTYPES:
            return f"{OP}to_int({x})"
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
    def masked(mask, body, other):
        with V.kernel.mask_loads(mask, other) as new_mask:
            result = body()
        if isinstance(other, (int, float, bool)):
            dtype = getattr(result, "dtype", None) or torch.float32
            other = V.ops.constant(other, dtype)
        # the raw handler (not the OpsValue wrapper): callers read .dtype of the result
        return V.ops.where(new_mask, result, other)

    @staticmethod
    def bitwise_and(a, b):
        return f"{OP}logical_and({a}, {b})"

    @staticmethod
    def bitwise_or(a, b):
        return f"{OP}logical_or({a}, {b})"

    @staticmethod
    def bitwise_xor(a, b):
        return f"{OP}logical_xor({a}, {b})"

    @staticmethod
    def bitwise_not(a):
        return f"{OP}logical_not({a})"

    @staticmethod
    def and_(a, b):
        return f"{OP}logical_and({a}, {b})"

    @staticmethod
    def or_(a, b):
        return f"{OP}logical_or({a}, {b})"

    @staticmethod
    def load_seed(name, offset):
        raise NotImplementedError("random number ops are not instantiable from the B200 templates")


for _name in ["exp", "exp2", "expm1", "log", "log2", "log10", "log1p", "sqrt", "rsqrt", "sin", "cos",
              "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh", "erf", "erfc", "lgamma", "floor",
              "ceil", "trunc", "round", "reciprocal", "sigmoid", "abs", "neg", "square", "relu",
              "sign", "isnan", "isinf", "signbit", "truediv", "pow", "fmod", "atan2", "copysign",
              "hypot", "add", "sub", "mul", "maximum", "minimum", "floordiv", "truncdiv",
              "remainder", "logical_and", "logical_or", "logical_xor", "logical_not", "eq", "ne",
              "lt", "le", "gt", "ge", "where"]:
    setattr(B200Overrides, _name, _call(_name))
B200Overrides.mod = _call("mod")
B200Overrides.int_truediv = _call("truediv")
B200Overrides.libdevice_exp = _call("exp")
B200Overrides.libdevice_sqrt = _call("sqrt")
B200Overrides.libdevice_log = _call("log")
B200Overrides.libdevice_sigmoid = _call("sigmoid")
B200Overrides.libdevice_abs = _call("abs")
