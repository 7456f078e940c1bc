"""Scalar-expression IR (`AluExp`), `Kernel`, `Reduction` and their wire format.

This is the host-side mirror of the reference's kernel IR (src/alu.ts:133
`AluExp`, :1365 `AluOp`, :1479 `Kernel`, :1544 `Reduction`).  A `Kernel` is the
unit of work a backend receives: ``out[gidx] = exp(gidx)`` or
``out[gidx] = epilogue(acc = REDUCE_{ridx<K} exp(gidx, ridx), gidx)``.

Only what crosses the backend boundary is restated here: node construction,
dtype rules the backend relies on, the lowering of views to flat indices
(src/tuner.ts:219-240 `tuneNullopt`) and a binary serialisation that
`libjaxcuda.so` and the CPU oracle both parse (layout in include/jaxcuda_ir.h).
"""
from __future__ import annotations

import math
import struct
from enum import IntEnum
from typing import Any, Iterable, Sequence


class DType(IntEnum):
    """src/alu.ts:6-13.  Bool is stored as a 4-byte 0/1 (alu.ts:23-29, :95)."""
    Float32 = 0
    Int32 = 1
    Uint32 = 2
    Bool = 3
    Float16 = 4
    Float64 = 5


_NP_NAMES = {
    DType.Float32: "float32", DType.Int32: "int32", DType.Uint32: "uint32",
    DType.Bool: "int32", DType.Float16: "float16", DType.Float64: "float64",
}


def byte_width(dtype: DType) -> int:
    """src/alu.ts:23-37."""
    return {DType.Float16: 2, DType.Float64: 8}.get(dtype, 4)


def np_dtype(dtype: DType) -> str:
    """numpy dtype name used to view a slot's bytes (alu.ts:87-108 `dtypedArray`)."""
    return _NP_NAMES[dtype]


def is_float(dtype: DType) -> bool:
    return dtype in (DType.Float32, DType.Float16, DType.Float64)


class AluOp(IntEnum):
    """src/alu.ts:1365-1407.  GlobalView never crosses the wire: it is lowered
    to Where(valid, GlobalIndex, 0) first (alu.ts:1664-1679)."""
    Add = 0
    Sub = 1
    Mul = 2
    Idiv = 3
    Mod = 4
    Min = 5
    Max = 6
    Sin = 7
    Cos = 8
    Asin = 9
    Atan = 10
    Exp = 11
    Log = 12
    Erf = 13
    Erfc = 14
    Sqrt = 15
    Floor = 16
    Ceil = 17
    Reciprocal = 18
    Cast = 19
    Bitcast = 20
    BitCombine = 21
    BitInvert = 22
    BitShift = 23
    Cmplt = 24
    Cmpne = 25
    Where = 26
    Threefry2x32 = 27
    Const = 28
    Special = 29
    Variable = 30
    GlobalIndex = 31


_BINARY = {AluOp.Add, AluOp.Sub, AluOp.Mul, AluOp.Idiv, AluOp.Mod, AluOp.Min,
           AluOp.Max, AluOp.BitCombine, AluOp.BitShift}
_REQUIRED_FLOAT = {AluOp.Sin, AluOp.Cos, AluOp.Asin, AluOp.Atan, AluOp.Exp,
                   AluOp.Log, AluOp.Erf, AluOp.Erfc, AluOp.Sqrt,
                   AluOp.Reciprocal, AluOp.Floor, AluOp.Ceil}
REDUCE_OPS = {AluOp.Add, AluOp.Mul, AluOp.Min, AluOp.Max}

_BITCOMBINE = {"and": 0, "or": 1, "xor": 2}
_BITSHIFT = {"shl": 0, "shr": 1}
_THREEFRY = {"xor": 0, 0: 1, 1: 2}
_SPECIAL = {"gidx": 0, "ridx": 1}


class AluExp:
    """One node of the expression DAG: (op, dtype, src, arg) as in alu.ts:138-143.

    Nodes are interned, so structurally equal sub-expressions are the same
    object and are emitted once (the reference's code generators likewise
    compute a node with several references once, wasm/translation.ts:238-242).
    """
    __slots__ = ("op", "dtype", "src", "arg", "_key")
    _interned: dict = {}

    def __new__(cls, op: AluOp, dtype: DType, src: Sequence["AluExp"] = (), arg: Any = None):
        src = tuple(src)
        if src and op in _FOLDABLE and all(s.op == AluOp.Const for s in src):
            return AluExp(AluOp.Const, dtype, (), _const_arg(DType(dtype), _fold(AluOp(op), DType(dtype), src, arg)))
        key = (int(op), int(dtype), tuple(id(s) for s in src), _arg_key(arg))
        hit = cls._interned.get(key)
        if hit is not None:
            return hit
        self = object.__new__(cls)
        self.op, self.dtype, self.src, self.arg, self._key = AluOp(op), DType(dtype), src, arg, key
        _typecheck(self)
        cls._interned[key] = self
        return self

    # ---- constructors, named as in alu.ts:189-330 --------------------------
    @staticmethod
    def add(a, b): return _binary(AluOp.Add, a, b)
    @staticmethod
    def sub(a, b): return _binary(AluOp.Sub, a, b)
    @staticmethod
    def mul(a, b): return _binary(AluOp.Mul, a, b)
    @staticmethod
    def idiv(a, b): return _binary(AluOp.Idiv, a, b)
    @staticmethod
    def mod(a, b): return _binary(AluOp.Mod, a, b)
    @staticmethod
    def min(a, b): return _binary(AluOp.Min, a, b)
    @staticmethod
    def max(a, b): return _binary(AluOp.Max, a, b)
    @staticmethod
    def sin(a): return AluExp(AluOp.Sin, a.dtype, [a])
    @staticmethod
    def cos(a): return AluExp(AluOp.Cos, a.dtype, [a])
    @staticmethod
    def asin(a): return AluExp(AluOp.Asin, a.dtype, [a])
    @staticmethod
    def atan(a): return AluExp(AluOp.Atan, a.dtype, [a])
    @staticmethod
    def exp(a): return AluExp(AluOp.Exp, a.dtype, [a])
    @staticmethod
    def log(a): return AluExp(AluOp.Log, a.dtype, [a])
    @staticmethod
    def erf(a): return AluExp(AluOp.Erf, a.dtype, [a])
    @staticmethod
    def erfc(a): return AluExp(AluOp.Erfc, a.dtype, [a])
    @staticmethod
    def sqrt(a): return AluExp(AluOp.Sqrt, a.dtype, [a])
    @staticmethod
    def floor(a): return AluExp(AluOp.Floor, a.dtype, [a])
    @staticmethod
    def ceil(a): return AluExp(AluOp.Ceil, a.dtype, [a])
    @staticmethod
    def reciprocal(a): return AluExp(AluOp.Reciprocal, a.dtype, [a])

    @staticmethod
    def cast(dtype: DType, a: "AluExp") -> "AluExp":
        if a.dtype == dtype:
            return a
        return AluExp(AluOp.Cast, dtype, [a])

    @staticmethod
    def bitcast(dtype: DType, a: "AluExp") -> "AluExp":
        if a.dtype == dtype:
            return a
        return AluExp(AluOp.Bitcast, dtype, [a])

    @staticmethod
    def bit_combine(a, b, kind: str): return AluExp(AluOp.BitCombine, a.dtype, [a, b], kind)
    @staticmethod
    def bit_invert(a): return AluExp(AluOp.BitInvert, a.dtype, [a])
    @staticmethod
    def bit_shift(a, b, kind: str): return AluExp(AluOp.BitShift, a.dtype, [a, b], kind)
    @staticmethod
    def cmplt(a, b): return AluExp(AluOp.Cmplt, DType.Bool, [a, b])
    @staticmethod
    def cmpne(a, b): return AluExp(AluOp.Cmpne, DType.Bool, [a, b])
    @staticmethod
    def where(cond, a, b): return AluExp(AluOp.Where, a.dtype, [cond, a, b])

    @staticmethod
    def threefry2x32(k0, k1, c0, c1, mode: Any = "xor"):
        return AluExp(AluOp.Threefry2x32, DType.Uint32, [k0, k1, c0, c1], mode)

    @staticmethod
    def const(dtype: DType, value) -> "AluExp":
        # alu.ts:280-293: integers are truncated and wrapped, Bool is 0/1.
        if dtype == DType.Bool:
            value = int(bool(value))
        elif dtype == DType.Int32:
            value = _wrap_i32(int(math.trunc(value)))
        elif dtype == DType.Uint32:
            value = int(math.trunc(value)) & 0xFFFFFFFF
        else:
            value = float(value)
        return AluExp(AluOp.Const, dtype, [], value)

    @staticmethod
    def special(dtype: DType, name: str, n: int): return AluExp(AluOp.Special, dtype, [], (name, int(n)))
    @staticmethod
    def variable(dtype: DType, name: str): return AluExp(AluOp.Variable, dtype, [], name)

    @staticmethod
    def global_index(dtype: DType, gid: int, length: int, bufidx: "AluExp") -> "AluExp":
        return AluExp(AluOp.GlobalIndex, dtype, [bufidx], (int(gid), int(length)))

    @staticmethod
    def f32(v): return AluExp.const(DType.Float32, v)
    @staticmethod
    def i32(v): return AluExp.const(DType.Int32, v)
    @staticmethod
    def u32(v): return AluExp.const(DType.Uint32, v)
    @staticmethod
    def bool(v): return AluExp.const(DType.Bool, v)
    @staticmethod
    def f16(v): return AluExp.const(DType.Float16, v)
    @staticmethod
    def f64(v): return AluExp.const(DType.Float64, v)

    def not_(self) -> "AluExp":
        """alu.ts:337-342."""
        if self.dtype != DType.Bool:
            raise TypeError("not() can only be called on boolean expressions")
        return AluExp.cmpne(self, AluExp.bool(True))

    # ---- traversal ----------------------------------------------------------
    def substitute(self, variables: dict) -> "AluExp":
        """Replace Variable/Special leaves by name (alu.ts `substitute`)."""
        memo: dict = {}

        def go(e: AluExp) -> AluExp:
            if id(e) in memo:
                return memo[id(e)]
            if e.op == AluOp.Variable and e.arg in variables:
                r = variables[e.arg]
            elif e.op == AluOp.Special and e.arg[0] in variables:
                r = variables[e.arg[0]]
            elif not e.src:
                r = e
            else:
                r = _rebuild(e, [go(s) for s in e.src])
            memo[id(e)] = r
            return r
        return go(self)

    def toposort(self) -> list:
        order, seen = [], set()
        stack = [(self, False)]
        while stack:
            e, done = stack.pop()
            if done:
                order.append(e)
                continue
            if id(e) in seen:
                continue
            seen.add(id(e))
            stack.append((e, True))
            for s in reversed(e.src):
                if id(s) not in seen:
                    stack.append((s, False))
        return order

    def __repr__(self) -> str:
        if self.op == AluOp.Const:
            return f"{self.arg}"
        if self.op in (AluOp.Special, AluOp.Variable):
            return self.arg[0] if isinstance(self.arg, tuple) else str(self.arg)
        if self.op == AluOp.GlobalIndex:
            return f"G_{self.arg[0]}[{self.src[0]!r}]"
        inner = ", ".join(repr(s) for s in self.src)
        tag = f"<{self.dtype.name}>" if self.op in (AluOp.Cast, AluOp.Bitcast) else ""
        return f"{self.op.name}{tag}({inner})"


def _fold(op: AluOp, dtype: DType, src, arg):
    """Value of an operation on constants, in the double arithmetic of `evaluate`
    (src/alu.ts:1059-1213): the reference folds such nodes when a Kernel is simplified
    (alu.ts:672-676), so e.g. log(0.999) reaches a backend as a constant."""
    v = [s.arg for s in src]
    flt = is_float(dtype)

    def wrap(r):
        if dtype == DType.Int32:
            return _wrap_i32(int(r))
        if dtype == DType.Uint32:
            return int(r) & 0xFFFFFFFF
        return r
    if op == AluOp.Add:
        return int(bool(v[0] or v[1])) if dtype == DType.Bool else wrap(v[0] + v[1])
    if op == AluOp.Sub:
        return wrap(v[0] - v[1])
    if op == AluOp.Mul:
        return int(bool(v[0] and v[1])) if dtype == DType.Bool else wrap(v[0] * v[1])
    if op == AluOp.Idiv:
        if v[1] == 0:
            return (math.copysign(math.inf, v[0]) if v[0] else math.nan) if flt else 0
        q = v[0] / v[1]
        return float(math.trunc(q)) if flt and math.isfinite(q) else (q if flt else wrap(math.trunc(q)))
    if op == AluOp.Mod:
        if v[1] == 0:
            return math.nan if flt else 0
        return math.fmod(v[0], v[1]) if flt else wrap(int(math.fmod(v[0], v[1])))
    if op in (AluOp.Min, AluOp.Max):
        if flt and (math.isnan(v[0]) or math.isnan(v[1])):
            return math.nan
        return min(v) if op == AluOp.Min else max(v)
    if op == AluOp.Cmplt:
        return int(v[0] < v[1])
    if op == AluOp.Cmpne:
        return int(v[0] != v[1])
    if op == AluOp.Where:
        return v[1] if v[0] else v[2]
    x = v[0]
    try:
        if op == AluOp.Sin: return math.sin(x)
        if op == AluOp.Cos: return math.cos(x)
        if op == AluOp.Asin: return math.asin(x)
        if op == AluOp.Atan: return math.atan(x)
        if op == AluOp.Exp: return math.exp(x)
        if op == AluOp.Log: return math.log(x) if x > 0 else (-math.inf if x == 0 else math.nan)
        if op == AluOp.Sqrt: return math.sqrt(x)
        if op == AluOp.Floor: return float(math.floor(x)) if math.isfinite(x) else x
        if op == AluOp.Ceil: return float(math.ceil(x)) if math.isfinite(x) else x
        if op == AluOp.Reciprocal: return 1.0 / x if x else math.copysign(math.inf, x)
    except (ValueError, OverflowError):
        return math.nan if op != AluOp.Exp else math.inf
    if op == AluOp.Cast:
        was_float = is_float(src[0].dtype)
        if dtype == DType.Int32:
            if was_float:
                x = 0 if math.isnan(x) else builtins_max(-2147483648, builtins_min(2147483647, x))
            return _wrap_i32(int(x))
        if dtype == DType.Uint32:
            if was_float:
                x = 0 if math.isnan(x) else builtins_max(0, builtins_min(4294967295, x))
            return int(x) & 0xFFFFFFFF
        if dtype == DType.Bool:
            return int(bool(x))
        return float(x)
    raise AssertionError(op)


def _const_arg(dtype: DType, value):
    return float(value) if is_float(dtype) else int(value)


builtins_max, builtins_min = max, min
_FOLDABLE = {AluOp.Add, AluOp.Sub, AluOp.Mul, AluOp.Idiv, AluOp.Mod, AluOp.Min, AluOp.Max, AluOp.Cmplt,
             AluOp.Cmpne, AluOp.Where, AluOp.Sin, AluOp.Cos, AluOp.Asin, AluOp.Atan, AluOp.Exp, AluOp.Log,
             AluOp.Sqrt, AluOp.Floor, AluOp.Ceil, AluOp.Reciprocal, AluOp.Cast}


def _arg_key(arg):
    if isinstance(arg, float):
        return ("f", struct.pack("<d", arg))
    return arg


def _wrap_i32(v: int) -> int:
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v & 0x80000000 else v


def _typecheck(e: AluExp) -> None:
    """Guards of the AluExp constructor, alu.ts:144-186."""
    if e.op in _REQUIRED_FLOAT and not is_float(e.dtype):
        raise TypeError(f"Unsupported dtype for {e.op.name}: {e.dtype.name}")
    if e.op == AluOp.Bitcast:
        s = e.src[0].dtype
        if e.dtype == DType.Bool or s == DType.Bool or byte_width(e.dtype) != byte_width(s):
            raise TypeError(f"Bitcast from {s.name} -> {e.dtype.name}")
    elif e.op == AluOp.Threefry2x32:
        if e.dtype != DType.Uint32 or any(s.dtype != DType.Uint32 for s in e.src):
            raise TypeError("Threefry2x32 requires uint32 types")
    elif e.op == AluOp.BitCombine:
        if e.src[0].dtype != e.src[1].dtype or is_float(e.src[0].dtype):
            raise TypeError("BitCombine requires matching integral dtype")
    elif e.op == AluOp.BitShift:
        if any(s.dtype == DType.Bool or is_float(s.dtype) for s in e.src):
            raise TypeError("BitShift requires two integral, non-bool dtypes")
    elif e.op == AluOp.BitInvert:
        if is_float(e.src[0].dtype):
            raise TypeError("BitInvert requires an integral dtype")


def _is_const(e: AluExp, v=None) -> bool:
    return e.op == AluOp.Const and (v is None or e.arg == v)


def _binary(op: AluOp, a: AluExp, b: AluExp) -> AluExp:
    """Binary node with the few index-algebra identities that keep lowered
    index expressions in the affine form the backend's classifier reads
    (a small subset of alu.ts:642-1042 `simplify`)."""
    if a.dtype != b.dtype:
        raise TypeError(f"{op.name}: dtype mismatch {a.dtype.name} vs {b.dtype.name}")
    dt = a.dtype
    if dt in (DType.Int32, DType.Uint32):
        if op == AluOp.Add:
            if _is_const(a, 0): return b
            if _is_const(b, 0): return a
            if _is_const(a) and _is_const(b): return AluExp.const(dt, a.arg + b.arg)
            # digits of one index put back together (the "shape tracking" rules of alu.ts:765-791):
            # (x/A)*A + x%A => x   and   ((x/A)%B)*A + x%A => x % (A*B)
            if (a.op == AluOp.Mul and _is_const(a.src[1]) and b.op == AluOp.Mod and _is_const(b.src[1])
                    and a.src[1].arg == b.src[1].arg and a.src[1].arg > 0):
                x, A = b.src[0], b.src[1].arg
                hi = a.src[0]
                def is_x_over_a(e):
                    return e.op == AluOp.Idiv and _is_const(e.src[1], A) and e.src[0] is x
                if is_x_over_a(hi):
                    return x
                if hi.op == AluOp.Mod and _is_const(hi.src[1]) and is_x_over_a(hi.src[0]):
                    return _binary(AluOp.Mod, x, AluExp.const(dt, A * hi.src[1].arg))
        elif op == AluOp.Sub:
            if _is_const(b, 0): return a
        elif op == AluOp.Mul:
            if _is_const(a, 1): return b
            if _is_const(b, 1): return a
            if _is_const(a, 0) or _is_const(b, 0): return AluExp.const(dt, 0)
            if _is_const(a) and _is_const(b): return AluExp.const(dt, a.arg * b.arg)
        elif op == AluOp.Idiv:
            if _is_const(b, 1): return a
        elif op == AluOp.Mod:
            if _is_const(b, 1): return AluExp.const(dt, 0)
            if a.op == AluOp.Special and _is_const(b) and b.arg >= a.arg[1] > 0: return a
            if (a.op == AluOp.Idiv and a.src[0].op == AluOp.Special and _is_const(a.src[1])
                    and _is_const(b) and a.src[1].arg > 0
                    and -(-a.src[0].arg[1] // a.src[1].arg) <= b.arg):
                return a
    if dt == DType.Bool and op == AluOp.Mul:
        if _is_const(a, 1): return b
        if _is_const(b, 1): return a
    return AluExp(op, dt, [a, b])


def _rebuild(e: AluExp, src: list) -> AluExp:
    if all(s is t for s, t in zip(src, e.src)):
        return e
    if e.op in _BINARY and e.op not in (AluOp.BitCombine, AluOp.BitShift):
        return _binary(e.op, src[0], src[1])
    return AluExp(e.op, e.dtype, src, e.arg)


class AluVar:
    """src/alu.ts:1462-1470."""
    gidx = AluExp.variable(DType.Int32, "gidx")
    ridx = AluExp.variable(DType.Int32, "ridx")

    @staticmethod
    def acc(dtype: DType) -> AluExp:
        return AluExp.variable(dtype, "acc")


class Reduction:
    """src/alu.ts:1544-1604.  f16 Add accumulates in f32 and the epilogue casts
    back (alu.ts:1560-1568)."""

    def __init__(self, dtype: DType, op: AluOp, size: int, epilogue: AluExp | None = None):
        if op not in REDUCE_OPS:
            raise TypeError(f"Unsupported reduction: {op.name}")
        self.dtype, self.op, self.size = DType(dtype), AluOp(op), int(size)
        self.epilogue = epilogue if epilogue is not None else AluVar.acc(self.dtype)
        if self.dtype == DType.Float16 and self.op == AluOp.Add:
            self.epilogue = self.epilogue.substitute(
                {"acc": AluExp.cast(DType.Float16, AluVar.acc(DType.Float32))})
            self.dtype = DType.Float32

    def __repr__(self):
        return f"{self.op.name}{{{self.size}}} -> {self.epilogue!r}"


class Kernel:
    """src/alu.ts:1479-1527."""

    def __init__(self, nargs: int, size: int, exp: AluExp, reduction: Reduction | None = None):
        self.nargs, self.size, self.exp, self.reduction = int(nargs), int(size), exp, reduction

    @property
    def dtype(self) -> DType:
        return self.reduction.epilogue.dtype if self.reduction else self.exp.dtype

    @property
    def bytes(self) -> int:
        return self.size * byte_width(self.dtype)

    def algorithmic_bytes(self) -> int:
        """Distinct input bytes addressed plus output bytes: the traffic a perfect
        implementation moves, and the numerator of every bandwidth figure reported."""
        spans: dict = {}
        roots = [self.exp] + ([self.reduction.epilogue] if self.reduction else [])
        for root in roots:
            for e in root.toposort():
                if e.op == AluOp.GlobalIndex:
                    gid, length = e.arg
                    spans[gid] = max(spans.get(gid, 0), length * byte_width(e.dtype))
        return self.bytes + sum(spans.values())

    def lowered(self):
        """`tuneNullopt` (src/tuner.ts:219-240): bind gidx/ridx to ranged
        Specials and cast the body to the accumulator dtype."""
        exp = self.exp
        variables = {"gidx": AluExp.special(DType.Int32, "gidx", self.size)}
        epilogue = None
        if self.reduction:
            variables["ridx"] = AluExp.special(DType.Int32, "ridx", self.reduction.size)
            if exp.dtype != self.reduction.dtype:
                exp = AluExp.cast(self.reduction.dtype, exp)
            epilogue = self.reduction.epilogue.substitute({"gidx": variables["gidx"]})
        return exp.substitute(variables), epilogue

    def serialize(self) -> bytes:
        """Wire image parsed by `jaxcuda_prepare_kernel` and by the oracle."""
        exp, epilogue = self.lowered()
        words = [WIRE_MAGIC, self.nargs, self.size & 0xFFFFFFFF, self.size >> 32,
                 1 if self.reduction else 0,
                 int(self.reduction.dtype) if self.reduction else 0,
                 int(self.reduction.op) if self.reduction else 0,
                 self.reduction.size if self.reduction else 0]
        exp_nodes = _encode_dag(exp, self.nargs)
        epi_nodes = _encode_dag(epilogue, self.nargs) if epilogue is not None else []
        words += [len(exp_nodes), len(epi_nodes)]
        out = struct.pack(f"<{len(words)}I", *words)
        return out + b"".join(exp_nodes) + b"".join(epi_nodes)

    def fingerprint(self) -> int:
        """64-bit FNV-1a of the wire image: the compile-cache key, standing in
        for `FpHash.hash(kernel)` (src/utils.ts:377-435; wasm.ts:126)."""
        h = 0xCBF29CE484222325
        for b in self.serialize():
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        return h

    def __repr__(self):
        r = f", reduction = {self.reduction!r}" if self.reduction else ""
        return f"Kernel{{nargs = {self.nargs}, size = {self.size}, exp = {self.exp!r}{r}}}"


WIRE_MAGIC = 0x314B584A  # "JXK1"
NODE_WORDS = 10


def _encode_dag(root: AluExp, nargs: int) -> list:
    order = root.toposort()
    index = {id(e): i for i, e in enumerate(order)}
    out = []
    for e in order:
        arg0, arg1 = 0, 0
        if e.op == AluOp.Const:
            if is_float(e.dtype):
                arg0 = struct.unpack("<Q", struct.pack("<d", float(e.arg)))[0]
            else:
                arg0 = int(e.arg) & 0xFFFFFFFFFFFFFFFF
        elif e.op == AluOp.Special:
            if e.arg[0] not in _SPECIAL:
                raise ValueError(f"unlowered special {e.arg[0]!r}")
            arg0, arg1 = _SPECIAL[e.arg[0]], e.arg[1]
        elif e.op == AluOp.Variable:
            if e.arg != "acc":
                raise ValueError(f"unbound variable {e.arg!r} (kernel was not lowered)")
        elif e.op == AluOp.GlobalIndex:
            arg0, arg1 = e.arg
            if not 0 <= arg0 < nargs:
                raise ValueError(f"GlobalIndex gid {arg0} out of range for nargs={nargs}")
        elif e.op == AluOp.BitCombine:
            arg0 = _BITCOMBINE[e.arg]
        elif e.op == AluOp.BitShift:
            arg0 = _BITSHIFT[e.arg]
        elif e.op == AluOp.Threefry2x32:
            arg0 = _THREEFRY[e.arg]
        src = [index[id(s)] for s in e.src] + [0] * (4 - len(e.src))
        out.append(struct.pack("<7IQI", int(e.op), int(e.dtype), len(e.src), *src,
                               arg0, arg1 & 0xFFFFFFFF))
    return out
