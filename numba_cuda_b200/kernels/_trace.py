"""Turn a Python binary functor into a C++ expression by symbolic tracing.

The reference JIT-compiles the user's function (``cuda.jit(device=True)(fn)``,
numba/cuda/kernels/reduction.py:18).  Here the function is *called* with two
symbolic operands that record every arithmetic / bitwise / comparison operation
applied to them; data-dependent control flow (``a if a > b else b``,
``max(a, b)``, ``if`` statements) is handled by re-running the function once per
outcome of each comparison and joining the results with ``?:``.  The resulting
expression over ``a`` and ``b`` is compiled into the reduce kernel at run time
(``b2k_reduce_expr``).  Anything the tracer cannot follow (calls into ``math``,
loops over the operands, more than 64 paths) raises ``NotImplementedError``.

Arithmetic follows numba's typing of the same function: integer operands are
widened to 64 bits for the whole expression and truncated when the result is
stored -- unsigned items to ``uint64``, signed items and integer constants to
``int64``, and an operation that mixes the two is done in ``int64`` (numba's
integer rule: 64 bits, signed if either side is); float32 stays float32 unless it
meets a Python float (a double); ``//`` and ``%`` have Python's floor semantics.
"""
from __future__ import annotations

import numbers

import numpy as np

_MAX_PATHS = 64


#: comparisons between an unsigned and a signed 64-bit value (helpers of the kernel source)
_MIXED_COMPARE = {
    "({a} < {b})": "b2k_lt({a}, {b})", "({a} <= {b})": "b2k_le({a}, {b})",
    "({a} > {b})": "b2k_lt({b}, {a})", "({a} >= {b})": "b2k_le({b}, {a})",
    "({a} == {b})": "b2k_eq({a}, {b})", "({a} != {b})": "(!b2k_eq({a}, {b}))",
}


class _Tracer:
    def __init__(self, operand_sign=None):
        self.forced = []       # outcomes imposed on the first comparisons
        self.taken = []        # (condition code, outcome) met during this run
        self.operand_sign = operand_sign          # 'u', 's' or None (floating point)
        self.integers = operand_sign is not None

    def decide(self, cond_code: str) -> bool:
        k = len(self.taken)
        outcome = self.forced[k] if k < len(self.forced) else True
        self.taken.append((cond_code, outcome))
        return outcome


class Sym:
    """A traced value: ``code`` is a C++ expression, ``kind`` is 'v' (value) or 'b'
    (bool), ``sign`` is 'u' (uint64), 's' (int64) or None (floating point / unknown)."""

    __slots__ = ("code", "kind", "tr", "sign")
    __array_priority__ = 1000  # keep NumPy scalars from taking over mixed operations

    def __init__(self, code, tr, kind="v", sign=None):
        self.code, self.tr, self.kind, self.sign = code, tr, kind, sign

    # -- helpers
    def _lit(self, other):
        if isinstance(other, Sym):
            return other.code
        if isinstance(other, (bool, np.bool_)):
            return "1" if other else "0"
        if isinstance(other, (numbers.Integral, np.integer)):
            v = int(other)
            if not -(2 ** 63) <= v < 2 ** 64:
                raise NotImplementedError("integer constant out of 64-bit range")
            # B2K_ILIT: the wide integer type for integer arrays, double for float arrays
            # (numba promotes float32 <op> integer to float64)
            if v >= 2 ** 63:       # only uint64 holds it
                return f"{v}ULL" if self.tr.integers else f"B2K_ILIT({v}ULL)"
            return f"B2K_ILIT({v}LL)"
        if isinstance(other, (numbers.Real, np.floating)):
            return repr(float(other)) if np.isfinite(other) else \
                ("B2K_NAN" if np.isnan(other) else ("B2K_INF" if other > 0 else "(-B2K_INF)"))
        raise NotImplementedError(f"cannot use a {type(other).__name__} in a reduce functor")

    def _sign_of(self, other):
        if isinstance(other, Sym):
            return other.sign
        if isinstance(other, (bool, np.bool_)):
            return "s"
        if isinstance(other, (numbers.Integral, np.integer)):
            return "u" if int(other) >= 2 ** 63 else "s"
        return None

    def _meet(self, left, lsign, right, rsign, fmt, kind):
        """One binary operation under the integer rule: unsigned only if both sides are."""
        if self.tr.integers and kind == "v" and "b2k_truediv" in fmt:
            sign = None
        elif lsign is None or rsign is None or not self.tr.integers:
            sign = None
        elif lsign == rsign:
            sign = lsign
        elif kind == "b":
            # an unsigned value against a signed one: compared as the numbers they are
            fmt, sign = _MIXED_COMPARE[fmt], None
        else:
            left, right, sign = f"((long long){left})", f"((long long){right})", "s"
        return Sym(fmt.format(a=left, b=right), self.tr, kind, sign if kind == "v" else None)

    def _bin(self, other, fmt, kind="v"):
        return self._meet(self.code, self.sign, self._lit(other), self._sign_of(other), fmt, kind)

    def _rbin(self, other, fmt, kind="v"):
        return self._meet(self._lit(other), self._sign_of(other), self.code, self.sign, fmt, kind)

    # -- arithmetic
    def __add__(self, o): return self._bin(o, "({a} + {b})")
    def __radd__(self, o): return self._rbin(o, "({a} + {b})")
    def __sub__(self, o): return self._bin(o, "({a} - {b})")
    def __rsub__(self, o): return self._rbin(o, "({a} - {b})")
    def __mul__(self, o): return self._bin(o, "({a} * {b})")
    def __rmul__(self, o): return self._rbin(o, "({a} * {b})")
    def __truediv__(self, o): return self._bin(o, "b2k_truediv({a}, {b})")
    def __rtruediv__(self, o): return self._rbin(o, "b2k_truediv({a}, {b})")
    def __floordiv__(self, o): return self._bin(o, "b2k_floordiv({a}, {b})")
    def __rfloordiv__(self, o): return self._rbin(o, "b2k_floordiv({a}, {b})")
    def __mod__(self, o): return self._bin(o, "b2k_mod({a}, {b})")
    def __rmod__(self, o): return self._rbin(o, "b2k_mod({a}, {b})")
    def __and__(self, o): return self._bin(o, "({a} & {b})")
    def __rand__(self, o): return self._rbin(o, "({a} & {b})")
    def __or__(self, o): return self._bin(o, "({a} | {b})")
    def __ror__(self, o): return self._rbin(o, "({a} | {b})")
    def __xor__(self, o): return self._bin(o, "({a} ^ {b})")
    def __rxor__(self, o): return self._rbin(o, "({a} ^ {b})")
    def __lshift__(self, o): return Sym("({a} << {b})".format(a=self.code, b=self._lit(o)), self.tr, "v", self.sign)
    def __rshift__(self, o): return Sym("({a} >> {b})".format(a=self.code, b=self._lit(o)), self.tr, "v", self.sign)

    def __neg__(self):
        if self.sign == "u":      # the negative of an unsigned value is a signed one
            return Sym(f"(-(long long){self.code})", self.tr, "v", "s")
        return Sym(f"(-{self.code})", self.tr, "v", self.sign)

    def __pos__(self): return self
    def __invert__(self): return Sym(f"(~{self.code})", self.tr, "v", self.sign)
    def __abs__(self): return Sym(f"b2k_abs({self.code})", self.tr, "v", self.sign)

    def __pow__(self, o):
        if isinstance(o, (numbers.Integral, np.integer)) and 0 <= int(o) <= 8:
            if int(o) == 0:
                return Sym("B2K_ILIT(1LL)", self.tr, "v", "s" if self.tr.integers else None)
            return Sym("(" + " * ".join([self.code] * int(o)) + ")", self.tr, "v", self.sign)
        raise NotImplementedError("only small constant integer powers are supported")

    # -- comparisons
    def __lt__(self, o): return self._bin(o, "({a} < {b})", "b")
    def __le__(self, o): return self._bin(o, "({a} <= {b})", "b")
    def __gt__(self, o): return self._bin(o, "({a} > {b})", "b")
    def __ge__(self, o): return self._bin(o, "({a} >= {b})", "b")
    def __eq__(self, o): return self._bin(o, "({a} == {b})", "b")
    def __ne__(self, o): return self._bin(o, "({a} != {b})", "b")
    __hash__ = None

    def __bool__(self):
        code = self.code if self.kind == "b" else f"({self.code} != 0)"
        return self.tr.decide(code)

    def __index__(self):
        raise NotImplementedError("a reduce operand cannot be used as an index")

    def __float__(self):
        raise NotImplementedError("calls that need a concrete number (math.*, float()) cannot be traced")

    __int__ = __float__


def _run(functor, forced, operand_sign):
    tr = _Tracer(operand_sign)
    tr.forced = list(forced)
    res = functor(Sym("a", tr, "v", operand_sign), Sym("b", tr, "v", operand_sign))
    if isinstance(res, Sym):
        code = res.code if res.kind == "v" else f"({res.code} ? 1 : 0)"
    else:
        code = Sym("a", tr)._lit(res)
    return code, tr.taken


def trace_functor(functor, dtype=None) -> str:
    """C++ expression over ``a`` and ``b`` equivalent to ``functor(a, b)`` for items of
    ``dtype`` (its kind decides how integers widen; None = signed)."""
    kind = np.dtype(dtype).kind if dtype is not None else "i"
    operand_sign = {"u": "u", "f": None}.get(kind, "s")
    paths = [0]

    def explore(forced):
        paths[0] += 1
        if paths[0] > _MAX_PATHS:
            raise NotImplementedError("reduce functor has too many data-dependent branches")
        try:
            code, taken = _run(functor, forced, operand_sign)
        except NotImplementedError:
            raise
        except Exception as exc:
            raise NotImplementedError(f"cannot trace the reduce functor: {exc!r}") from exc
        if len(taken) <= len(forced):
            return code
        cond = taken[len(forced)][0]
        yes = explore(forced + [True])
        no = explore(forced + [False])
        return yes if yes == no else f"({cond} ? {yes} : {no})"

    return explore([])
