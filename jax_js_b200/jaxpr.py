"""A Jaxpr and the rules by which `jit` cuts it into Kernels.

The reference's tracing frontend produces, for every `jit`-ed function, a flat list of
primitive equations (`Jaxpr`, src/frontend/jaxpr.ts) and compiles it to the static step list
a backend replays (`jitCompile`, src/frontend/jit.ts:266-465).  Which values are materialised
as a Kernel's output and which are fused into their consumer is decided there, by
`splitGraphDataflow` (src/frontend/jit.ts:791-1098), not by the backend.  The benchmark
programs of this package are therefore written as Jaxprs and cut by a restatement of those
rules, so that the Kernel lists the cuda backend is measured on are the lists the reference's
frontend would hand it:

  * `Builder`: equations with shape inference for the primitives the programs use;
  * `Jaxpr.simplify`: literal folding, no-op movement removal, dead-code elimination
    (src/frontend/jaxpr.ts:252-361);
  * `split_graph_dataflow`: reduction epilogues, values materialised in front of a dot-style
    reduction, black nodes, the argument-count limit;
  * `jit_compile`: the per-primitive expression rules (src/frontend/jit.ts:572-779) over
    `ShapeTracker` views, Kernel construction and the placement of free steps
    (jit.ts:225-249).

Tracing itself (`jvp`, partial evaluation, transposition) is not restated: the Jaxprs are
written out by the callers with the rule each equation comes from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

from .alu import AluExp, AluOp, AluVar, DType, Kernel, Reduction, byte_width, is_float
from .programs import JitProgram, Step
from .shape import ShapeTracker, accessor_global, unravel_alu

MAX_ARGS = 64   # Backend.maxArgs of the cuda backend (the Wasm backend's value, src/backend/wasm.ts:38)


# ---- atoms and equations ----------------------------------------------------------------------

class Var:
    __slots__ = ("shape", "dtype", "name")

    def __init__(self, shape: Sequence[int], dtype: DType, name: str):
        self.shape, self.dtype, self.name = tuple(int(d) for d in shape), DType(dtype), name

    @property
    def size(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def __repr__(self):
        return f"{self.name}:{self.dtype.name}{list(self.shape)}"


class Lit:
    """A scalar literal; weakly typed (src/frontend/jaxpr.ts `Lit`, core.ts:700-737)."""
    __slots__ = ("value", "dtype")
    shape = ()

    def __init__(self, value, dtype: DType = DType.Float32):
        self.value, self.dtype = value, DType(dtype)

    def __repr__(self):
        return repr(self.value)


@dataclass
class Eqn:
    prim: str
    inputs: list
    params: dict
    out: Var


def general_broadcast(a: Sequence[int], b: Sequence[int]) -> tuple:
    """src/utils.ts:322-346."""
    out = []
    a, b = list(a), list(b)
    while a or b:
        x = a.pop() if a else 1
        y = b.pop() if b else 1
        if x != y and x != 1 and y != 1:
            raise TypeError(f"Incompatible array broadcast shapes: {a + [x]} vs {b + [y]}")
        out.append(y if x == 1 else x)
    return tuple(reversed(out))


def _promote(atoms: Sequence) -> DType:
    """Result dtype of a broadcasting primitive: literals are weak and take the arrays' dtype
    (`promoteAvals`, src/frontend/core.ts:716-737).  Arrays of different dtypes are not mixed by
    the programs here."""
    strong = [a.dtype for a in atoms if isinstance(a, Var)]
    if not strong:
        return atoms[0].dtype
    if any(d != strong[0] for d in strong):
        raise TypeError(f"mixed dtypes {strong}")
    return strong[0]


VIEW_PRIMS = ("transpose", "broadcast", "reshape")
UNARY_FUSABLE = ("neg", "reciprocal", "stop_gradient", "cast", "exp", "log", "sqrt")
BINARY_FUSABLE = ("add", "mul", "idiv", "mod", "max", "min")
REDUCE_PRIMS = ("reduce", "dot")
HETEROGENEOUS = ("gather",)


class Builder:
    """Appends equations and infers shapes; the methods are named after the primitives of
    src/frontend/core.ts:60-130."""

    def __init__(self, prefix: str = "t"):
        self.inputs: list = []
        self.eqns: list = []
        self._n = 0
        self._prefix = prefix   # of the names given to unnamed results

    def input(self, name: str, shape: Sequence[int], dtype: DType = DType.Float32) -> Var:
        v = Var(shape, dtype, name)
        self.inputs.append(v)
        return v

    def _emit(self, prim: str, inputs: list, params: dict, shape, dtype, name: str | None) -> Var:
        self._n += 1
        out = Var(shape, dtype, name or f"{self._prefix}{self._n}")
        self.eqns.append(Eqn(prim, list(inputs), params, out))
        return out

    def _binary(self, prim, x, y, name):
        return self._emit(prim, [x, y], {}, general_broadcast(x.shape, y.shape), _promote([x, y]), name)

    def add(self, x, y, name=None): return self._binary("add", x, y, name)
    def mul(self, x, y, name=None): return self._binary("mul", x, y, name)
    def max(self, x, y, name=None): return self._binary("max", x, y, name)
    def min(self, x, y, name=None): return self._binary("min", x, y, name)
    def idiv(self, x, y, name=None): return self._binary("idiv", x, y, name)
    def mod(self, x, y, name=None): return self._binary("mod", x, y, name)

    def _unary(self, prim, x, name, params=None, dtype=None):
        return self._emit(prim, [x], params or {}, x.shape, x.dtype if dtype is None else dtype, name)

    def neg(self, x, name=None): return self._unary("neg", x, name)
    def exp(self, x, name=None): return self._unary("exp", x, name)
    def log(self, x, name=None): return self._unary("log", x, name)
    def sqrt(self, x, name=None): return self._unary("sqrt", x, name)
    def reciprocal(self, x, name=None): return self._unary("reciprocal", x, name)
    def stop_gradient(self, x, name=None): return self._unary("stop_gradient", x, name)
    def cast(self, x, dtype, name=None): return self._unary("cast", x, name, {"dtype": DType(dtype)}, DType(dtype))

    def compare(self, x, y, op: str, name=None):
        return self._emit("compare", [x, y], {"op": op}, general_broadcast(x.shape, y.shape), DType.Bool, name)

    def where(self, cond, x, y, name=None):
        shape = general_broadcast(general_broadcast(cond.shape, x.shape), y.shape)
        return self._emit("where", [cond, x, y], {}, shape, _promote([x, y]), name)

    def reduce(self, x, op: AluOp, axis: Sequence[int], name=None):
        axis = sorted(a % len(x.shape) for a in axis)
        shape = [d for i, d in enumerate(x.shape) if i not in axis]
        return self._emit("reduce", [x], {"op": AluOp(op), "axis": axis}, shape, x.dtype, name)

    def dot(self, x, y, name=None):
        """Contracts the last axis of both operands, broadcasting the others (core.ts `dot`)."""
        if x.shape[-1] != y.shape[-1]:
            raise TypeError(f"dot: contracted axes differ, {x.shape} vs {y.shape}")
        return self._emit("dot", [x, y], {}, general_broadcast(x.shape[:-1], y.shape[:-1]), _promote([x, y]), name)

    def transpose(self, x, perm: Sequence[int], name=None):
        perm = [p % len(x.shape) for p in perm]
        return self._emit("transpose", [x], {"perm": perm}, [x.shape[p] for p in perm], x.dtype, name)

    def broadcast(self, x, shape: Sequence[int], axis: Sequence[int], name=None):
        """Inserts the axes `axis` of the result, then expands to `shape` (core.ts:448-451)."""
        axis = sorted(a % len(shape) for a in axis)
        return self._emit("broadcast", [x], {"shape": tuple(shape), "axis": axis}, shape, x.dtype, name)

    def reshape(self, x, shape: Sequence[int], name=None):
        return self._emit("reshape", [x], {"shape": tuple(shape)}, shape, x.dtype, name)

    def gather(self, x, indices: Sequence[Var], axis: Sequence[int], out_dim: int, name=None):
        idx_shape = ()
        for i in indices:
            idx_shape = general_broadcast(idx_shape, i.shape)
        shape = [d for i, d in enumerate(x.shape) if i not in axis]
        shape[out_dim:out_dim] = idx_shape
        return self._emit("gather", [x] + list(indices), {"axis": list(axis), "out_dim": out_dim}, shape, x.dtype, name)

    def build(self, outs: Sequence[Var]) -> "Jaxpr":
        return Jaxpr(list(self.inputs), list(self.eqns), list(outs))


@dataclass
class Jaxpr:
    in_binders: list
    eqns: list
    outs: list

    def simplify(self) -> "Jaxpr":
        """src/frontend/jaxpr.ts:252-361: fold +0, *1 and literal-literal arithmetic, drop
        movement equations that change nothing, drop equations whose result is unused."""
        ctx: dict = {}
        kept = []

        def is_lit(a, v=None):
            return isinstance(a, Lit) and (v is None or a.value == v)

        for e in self.eqns:
            ins = [ctx.get(id(a), a) for a in e.inputs]
            eq = Eqn(e.prim, ins, e.params, e.out)
            if e.prim == "add":
                a, b = ins
                if is_lit(a, 0): ctx[id(e.out)] = b
                elif is_lit(b, 0): ctx[id(e.out)] = a
                elif is_lit(a) and is_lit(b): ctx[id(e.out)] = Lit(a.value + b.value, a.dtype)
                else: kept.append(eq)
            elif e.prim == "neg":
                if is_lit(ins[0]): ctx[id(e.out)] = Lit(-ins[0].value, ins[0].dtype)
                else: kept.append(eq)
            elif e.prim == "mul":
                a, b = ins
                if is_lit(a, 1): ctx[id(e.out)] = b
                elif is_lit(b, 1): ctx[id(e.out)] = a
                elif is_lit(a) and is_lit(b): ctx[id(e.out)] = Lit(a.value * b.value, a.dtype)
                else: kept.append(eq)
            elif ((e.prim in ("broadcast", "reshape") and tuple(e.params["shape"]) == tuple(ins[0].shape))
                  or (e.prim == "transpose" and all(p == i for i, p in enumerate(e.params["perm"])))):
                ctx[id(e.out)] = ins[0]
            else:
                kept.append(eq)
        outs = [ctx.get(id(o), o) for o in self.outs]
        used = {id(o) for o in outs if isinstance(o, Var)}
        live = []
        for e in reversed(kept):
            if id(e.out) in used:
                live.append(e)
                used.update(id(a) for a in e.inputs if isinstance(a, Var))
        return Jaxpr(self.in_binders, list(reversed(live)), outs)

    def __str__(self):
        lines = ["{ lambda " + ", ".join(map(repr, self.in_binders)) + " ."]
        for e in self.eqns:
            p = " [" + ", ".join(f"{k}={v}" for k, v in e.params.items()) + "]" if e.params else ""
            lines.append(f"    {e.out!r} = {e.prim}{p} " + " ".join(a.name if isinstance(a, Var) else repr(a) for a in e.inputs))
        lines.append("  in ( " + ", ".join(o.name if isinstance(o, Var) else repr(o) for o in self.outs) + " ) }")
        return "\n".join(lines)


# ---- where to cut -----------------------------------------------------------------------------

def split_graph_dataflow(jaxpr: Jaxpr, max_args: int = MAX_ARGS) -> set:
    """ids of the Vars that are dispatched as a Kernel's output ("black" nodes):
    src/frontend/jit.ts:791-1098."""
    eqns = jaxpr.eqns
    defn, usages = {}, {}
    for i, e in enumerate(eqns):
        defn[id(e.out)] = i
        for a in e.inputs:
            if isinstance(a, Var):
                usages.setdefault(id(a), []).append(i)
    out_ids = {id(o) for o in jaxpr.outs if isinstance(o, Var)}

    # reduction epilogues (jit.ts:811-885)
    epilogue_eqns, endpoint_eqns = set(), set()
    for i, e in enumerate(eqns):
        if e.prim not in REDUCE_PRIMS:
            continue
        head = i
        while True:
            epilogue_eqns.add(head)
            out = eqns[head].out
            use = usages.get(id(out), [])
            if id(out) in out_ids or len(use) != 1:
                break
            if use[0] in epilogue_eqns:
                break
            nxt = eqns[use[0]]
            if nxt.prim in UNARY_FUSABLE:
                head = use[0]
                continue
            if nxt.prim in BINARY_FUSABLE:
                other = next(a for a in nxt.inputs if a is not out)
                if isinstance(other, Lit) or general_broadcast(other.shape, out.shape) == tuple(out.shape):
                    head = use[0]
                    continue
            break
        endpoint_eqns.add(head)

    # producers materialised because a dot-style reduction reuses them (jit.ts:887-947)
    materialized = set()

    def has_reuse(shape, promoted):
        off = len(promoted) - len(shape)
        for ax in range(len(promoted) - 1):
            dim = 1 if ax < off else shape[ax - off]
            if dim == 1 and promoted[ax] > 1:
                return True
        return False

    def mark_non_view_producer(v):
        cur = v
        while True:
            d = defn.get(id(cur))
            if d is None:
                return
            e = eqns[d]
            if e.prim not in VIEW_PRIMS:
                break
            nxt = next((a for a in e.inputs if isinstance(a, Var)), None)
            if nxt is None:
                return
            cur = nxt
        materialized.add(id(cur))

    for e in eqns:
        if e.prim != "dot":
            continue
        promoted = general_broadcast(e.inputs[0].shape, e.inputs[1].shape)
        for a in e.inputs:
            if isinstance(a, Var) and has_reuse(a.shape, promoted):
                mark_non_view_producer(a)

    # black nodes, backwards (jit.ts:949-1033)
    black = set(out_ids)
    next_black = {o: o for o in out_ids}
    for i in range(len(eqns) - 1, -1, -1):
        e = eqns[i]
        o = id(e.out)
        if (i in endpoint_eqns or e.prim in HETEROGENEOUS or o in materialized or o in black):
            black.add(o)
            next_black[o] = o
            continue
        reach = set()
        for j in usages.get(o, []):
            u = next_black.get(id(eqns[j].out))
            if u is not None:
                reach.add(u)
        if len(reach) > 1:
            black.add(o)
            next_black[o] = o
        elif len(reach) == 1:
            next_black[o] = next(iter(reach))

    # argument-count limit, forwards with backtracking (jit.ts:1035-1095)
    deps = {id(v): {id(v)} for v in jaxpr.in_binders}
    i = 0
    while i < len(eqns):
        e = eqns[i]
        i += 1
        per_input = []
        for a in e.inputs:
            if isinstance(a, Var):
                per_input.append({id(a)} if id(a) in black else deps[id(a)])
            else:
                per_input.append(set())
        counter: dict = {}
        for s in per_input:
            for d in s:
                counter[d] = counter.get(d, 0) + 1
        if len(counter) > max_args:
            best, pick = 0, -1
            for k, a in enumerate(e.inputs):
                if isinstance(a, Var) and id(a) in defn:
                    uniq = sum(1 for d in per_input[k] if counter[d] == 1)
                    if uniq > best:
                        best, pick = uniq, k
            if pick < 0:
                raise RuntimeError(f"maxArgs: no input to materialise in {e.prim}")
            i = defn[id(e.inputs[pick])]
            black.add(id(eqns[i].out))
            i += 1
        else:
            deps[id(e.out)] = set(counter)
    return black


# ---- lazily fused expressions -----------------------------------------------------------------

class _View:
    """A load of a materialised buffer through a view: the GlobalView leaf (src/alu.ts:1355-1362).
    Its indices are always the unravelled output index of the view's shape (jit.ts:487-506)."""
    __slots__ = ("dtype", "buf", "st")

    def __init__(self, dtype, buf, st):
        self.dtype, self.buf, self.st = dtype, buf, st


class _Node:
    __slots__ = ("fn", "src", "dtype")

    def __init__(self, fn: Callable, src: Sequence, dtype: DType):
        self.fn, self.src, self.dtype = fn, tuple(src), dtype


class _Leaf:
    """A constant or the accumulator variable."""
    __slots__ = ("exp", "dtype")

    def __init__(self, exp: AluExp):
        self.exp, self.dtype = exp, exp.dtype


def _map_views(t, fn):
    if isinstance(t, _View):
        st = fn(t.st)
        return t if st is None else _View(t.dtype, t.buf, st)
    if isinstance(t, _Node):
        return _Node(t.fn, [_map_views(s, fn) for s in t.src], t.dtype)
    return t


def _lower(t, gids: dict, reduce_axis: bool) -> AluExp:
    if isinstance(t, _View):
        shape = t.st.shape
        if reduce_axis:
            idx = unravel_alu(shape[:-1], AluVar.gidx) + [AluVar.ridx]
        else:
            idx = unravel_alu(shape, AluVar.gidx)
        return accessor_global(t.dtype, gids[t.buf], t.st, idx)
    if isinstance(t, _Node):
        return t.fn(*[_lower(s, gids, reduce_axis) for s in t.src])
    return t.exp


def _st_broadcast(st: ShapeTracker, shape: Sequence[int], axis: Sequence[int]) -> ShapeTracker:
    """src/shape.ts:740-752."""
    if axis:
        unsq = list(st.shape)
        for a in sorted(axis):
            unsq.insert(a, 1)
        st = st.reshape(unsq)
    return st.expand(shape)


@dataclass
class _Value:
    kind: str                      # "imm" | "exp" | "red"
    exp: Any = None                # expression tree ("exp", "red")
    args: list = field(default_factory=list)
    buf: str = ""                  # "imm"
    red: tuple | None = None       # (dtype, op, size), "red"
    epilogue: Any = None           # expression tree over `acc`, "red"


def _broadcasted(fn: Callable, out_dtype_of=None, skip_cast=()):
    """`broadcastedJit`, src/frontend/jit.ts:511-546."""
    def rule(exps, atoms, params, out: Var):
        shape = ()
        for a in atoms:
            shape = general_broadcast(shape, a.shape)
        dtype = _promote([a for i, a in enumerate(atoms) if i not in skip_cast])

        def widen(st):
            if tuple(st.shape) != tuple(shape):
                return _st_broadcast(st, shape, list(range(len(shape) - len(st.shape))))
            return None
        new = []
        for i, (x, a) in enumerate(zip(exps, atoms)):
            x = _map_views(x, widen)
            if x.dtype != dtype and i not in skip_cast:
                if isinstance(x, _Leaf) and x.exp.op == AluOp.Const:
                    x = _Leaf(AluExp.const(dtype, x.exp.arg))
                else:
                    x = _Node(lambda v, d=dtype: AluExp.cast(d, v), [x], dtype)
            new.append(x)
        return _Node(lambda *v: fn(*v, **params), new, out.dtype), None
    return rule


def _unop(fn: Callable):
    def rule(exps, atoms, params, out: Var):
        return _Node(lambda v: fn(v, **params), exps, out.dtype), None
    return rule


def _movement(fn: Callable):
    def rule(exps, atoms, params, out: Var):
        return _map_views(exps[0], lambda st: fn(st, **params)), None
    return rule


def _compare(a, b, op):
    """`aluCompare`, src/frontend/array.ts:1786-1800."""
    if op == "less":
        return AluExp.cmplt(a, b)
    if op == "equal":
        return AluExp.cmpne(a, b).not_()
    if op == "not_equal":
        return AluExp.cmpne(a, b)
    if op == "less_equal":
        return AluExp.add(AluExp.cmplt(a, b), AluExp.cmpne(a, b).not_())
    raise ValueError(op)


def _reduce_rule(exps, atoms, params, out: Var):
    """jit.ts:603-622: reduced axes move last and merge into one."""
    shape = atoms[0].shape
    axis = params["axis"]
    kept = [i for i in range(len(shape)) if i not in axis]
    size = 1
    for a in axis:
        size *= shape[a]
    new_shape = [shape[i] for i in kept] + [size]
    perm = kept + list(axis)
    a = _map_views(exps[0], lambda st: st.permute(perm).reshape(new_shape))
    return a, (a.dtype, params["op"], size)


def _dot_rule(exps, atoms, params, out: Var):
    """jit.ts:639-648: Mul then Reduce over the last axis."""
    prod_var = Var(general_broadcast(atoms[0].shape, atoms[1].shape), out.dtype, "")
    c, _ = _RULES["mul"](exps, atoms, {}, prod_var)
    return _reduce_rule([c], [prod_var], {"op": AluOp.Add, "axis": [len(prod_var.shape) - 1]}, out)


def _gather_rule(exps, atoms, params, out: Var):
    """jit.ts:715-763.  The indexed operand is lowered over its own output index, which is then
    replaced by the flat position the index arrays select."""
    axis, out_dim = params["axis"], params["out_dim"]
    xs = atoms[0]
    idx_shape = ()
    for a in atoms[1:]:
        idx_shape = general_broadcast(idx_shape, a.shape)
    final = [d for i, d in enumerate(xs.shape) if i not in axis]
    final[out_dim:out_dim] = idx_shape
    n_idx = len(idx_shape)

    def build(gids):
        idx_all = unravel_alu(final, AluVar.gidx)
        non_axis = idx_all[:out_dim] + idx_all[out_dim + n_idx:]
        src = list(non_axis)
        for i in range(len(xs.shape)):
            if i in axis:
                src.insert(i, None)
        for k, iexp in enumerate(exps[1:]):
            wide = _map_views(iexp, lambda st: _st_broadcast(
                st, final, list(range(out_dim + n_idx - len(st.shape))) + list(range(out_dim + n_idx, len(final)))))
            src[axis[k]] = AluExp.cast(DType.Int32, _lower(wide, gids, False))
        index, _valid = ShapeTracker.from_shape(xs.shape).to_alu_exp(src)
        return _lower(exps[0], gids, False).substitute({"gidx": index})
    return _Deferred(build, out.dtype), None


class _Deferred:
    """An expression that needs the final argument numbering to be built (Gather)."""
    __slots__ = ("build", "dtype")

    def __init__(self, build, dtype):
        self.build, self.dtype = build, dtype


_RULES = {
    "add": _broadcasted(lambda a, b: AluExp.add(a, b)),
    "mul": _broadcasted(lambda a, b: AluExp.mul(a, b)),
    "max": _broadcasted(lambda a, b: AluExp.max(a, b)),
    "min": _broadcasted(lambda a, b: AluExp.min(a, b)),
    "idiv": _broadcasted(lambda a, b: AluExp.idiv(a, b)),
    "mod": _broadcasted(lambda a, b: AluExp.mod(a, b)),
    "compare": _broadcasted(lambda a, b, op: _compare(a, b, op)),
    "where": _broadcasted(lambda c, a, b: AluExp.where(c, a, b), skip_cast=(0,)),
    "neg": _unop(lambda a: AluExp.sub(AluExp.const(a.dtype, 0), a)),
    "reciprocal": _unop(AluExp.reciprocal),
    "exp": _unop(AluExp.exp),
    "log": _unop(AluExp.log),
    "sqrt": _unop(AluExp.sqrt),
    "stop_gradient": _unop(lambda a: a),
    "cast": _unop(lambda a, dtype: AluExp.cast(dtype, a)),
    "reduce": _reduce_rule,
    "dot": _dot_rule,
    "gather": _gather_rule,
    "transpose": _movement(lambda st, perm: st.permute(perm)),
    "broadcast": _movement(lambda st, shape, axis: _st_broadcast(st, shape, axis)),
    "reshape": _movement(lambda st, shape: st.reshape(shape)),
}


def jit_compile(jaxpr: Jaxpr, max_args: int = MAX_ARGS) -> JitProgram:
    """`jitCompile`, src/frontend/jit.ts:266-465.  Buffers are named after the Vars they hold;
    program inputs and outputs are the Jaxpr's, in order."""
    jaxpr = jaxpr.simplify()
    black = split_graph_dataflow(jaxpr, max_args)
    ctx: dict = {id(v): _Value("imm", buf=v.name) for v in jaxpr.in_binders}
    names = [v.name for v in jaxpr.in_binders]
    if len(set(names)) != len(names):
        raise ValueError("duplicate input names")
    prog = JitProgram(inputs=names, outputs=[o.name for o in jaxpr.outs])
    for e in jaxpr.eqns:
        exps, args = [], []
        consumed_red = None

        def add_args(new):
            for a in new:
                if a not in args:
                    args.append(a)

        for a in e.inputs:
            if isinstance(a, Lit):
                exps.append(_Leaf(AluExp.const(a.dtype, a.value)))
                continue
            jv = ctx[id(a)]
            if jv.kind == "imm":
                add_args([jv.buf])
                exps.append(_View(a.dtype, jv.buf, ShapeTracker.from_shape(a.shape)))
            elif jv.kind == "exp":
                add_args(jv.args)
                exps.append(jv.exp)
            else:
                if consumed_red is not None:
                    raise RuntimeError("jit: unexpected, multiple red inputs")
                add_args(jv.args)
                exps.append(jv.epilogue)
                consumed_red = jv
        rule = _RULES[e.prim]
        if consumed_red is not None:
            epilogue, _ = rule(exps, e.inputs, e.params, e.out)
            exp, red = consumed_red.exp, consumed_red.red
            add_args(consumed_red.args)
        else:
            exp, red = rule(exps, e.inputs, e.params, e.out)
            epilogue = _Leaf(AluVar.acc(red[0])) if red else None
        if id(e.out) in black:
            gids = {b: i for i, b in enumerate(args)}
            if isinstance(exp, _Deferred):
                body = exp.build(gids)
            else:
                body = _lower(exp, gids, red is not None)
            reduction = None
            if red:
                reduction = Reduction(red[0], red[1], red[2], _lower(epilogue, gids, False))
            prog.run(e.out.name, Kernel(len(args), e.out.size, body, reduction), list(args))
            ctx[id(e.out)] = _Value("imm", buf=e.out.name)
        elif red:
            ctx[id(e.out)] = _Value("red", exp=exp, args=list(args), red=red, epilogue=epilogue)
        else:
            ctx[id(e.out)] = _Value("exp", exp=exp, args=list(args))
    for o in jaxpr.outs:
        if not isinstance(o, Var) or ctx[id(o)].kind != "imm":
            raise RuntimeError("internal: expected imm, since outs are black nodes")
    _insert_free_steps(prog)
    return prog


def _insert_free_steps(prog: JitProgram) -> None:
    """A free step right after the last use of every intermediate (jit.ts:225-249)."""
    keep = set(prog.outputs) | set(prog.inputs)
    last: dict = {}
    for i, s in enumerate(prog.steps):
        if s.kind == "malloc":
            last[s.name] = i
        elif s.kind == "execute":
            for n in list(s.inputs) + [s.name]:
                if n in last:
                    last[n] = i
    for name, i in sorted(((n, i) for n, i in last.items() if n not in keep), key=lambda t: -t[1]):
        prog.steps.insert(i + 1, Step("free", name))


# ---- vmap over a Jaxpr ------------------------------------------------------------------------

def vmap_jaxpr(jaxpr: Jaxpr, axis_size: int, in_dims: Sequence) -> Jaxpr:
    """The batching rules of src/frontend/vmap.ts:163-470 applied equation by equation, as the
    reference's `BatchTrace` applies them to every primitive a vmapped function executes; mapped
    outputs get their batch axis moved to the front (`vmapFlat`, vmap.ts:519-557)."""
    b = Builder(prefix="v")
    env: dict = {}

    def move(x, src, dst):
        """`moveBatchAxis`, vmap.ts:59-75."""
        if src is None:
            shape = list(x.shape)
            shape.insert(dst, axis_size)
            return b.broadcast(x, shape, [dst])
        if src == dst:
            return x
        perm = list(range(len(x.shape)))
        perm.pop(src)
        perm.insert(dst, src)
        return b.transpose(x, perm)

    for v, d in zip(jaxpr.in_binders, in_dims):
        shape = list(v.shape)
        if d is not None:
            shape.insert(d, axis_size)
        env[id(v)] = (b.input(v.name, shape, v.dtype), d)

    def broadcast_batcher(prim, args, dims, params, name):
        nd = max(len(x.shape) + (1 if d is None else 0) for x, d in zip(args, dims))
        first = next(i for i, d in enumerate(dims) if d is not None)
        first_bdim = dims[first] - len(args[first].shape)
        if all((d is None and len(x.shape) < -first_bdim) or (d is not None and d - len(x.shape) == first_bdim)
               for x, d in zip(args, dims)):
            return args, nd + first_bdim
        new = []
        for x, d in zip(args, dims):
            if d is not None:
                x = move(x, d, 0)
                if len(x.shape) < nd:
                    x = b.reshape(x, [x.shape[0]] + [1] * (nd - len(x.shape)) + list(x.shape[1:]))
            new.append(x)
        return new, 0

    for e in jaxpr.eqns:
        pairs = [env[id(a)] if isinstance(a, Var) else (a, None) for a in e.inputs]
        args, dims = [p[0] for p in pairs], [p[1] for p in pairs]
        name = e.out.name
        if all(d is None for d in dims):
            out = b._emit(e.prim, args, e.params, e.out.shape, e.out.dtype, name)
            env[id(e.out)] = (out, None)
            continue
        p = e.prim
        if p in ("add", "mul", "max", "min", "idiv", "mod", "compare", "where"):
            new, bd = broadcast_batcher(p, args, dims, e.params, name)
            if p == "compare":
                out = b.compare(new[0], new[1], e.params["op"], name)
            elif p == "where":
                out = b.where(*new, name=name)
            else:
                out = b._binary(p, new[0], new[1], name)
        elif p in UNARY_FUSABLE:
            out, bd = b._unary(p, args[0], name, e.params, e.out.dtype), dims[0]
        elif p == "reduce":
            xb = dims[0]
            axis = [ax + (1 if xb <= ax else 0) for ax in e.params["axis"]]
            bd = xb - sum(1 for ax in e.params["axis"] if ax < xb)
            out = b.reduce(args[0], e.params["op"], axis, name)
        elif p == "dot":
            x = move(args[0], dims[0], len(args[0].shape) - (1 if dims[0] is None else 2))
            y = move(args[1], dims[1], len(args[1].shape) - (1 if dims[1] is None else 2))
            out = b.dot(x, y, name)
            bd = len(out.shape) - 1
        elif p == "transpose":
            xb = dims[0]
            perm = [q + (1 if xb <= q else 0) for q in e.params["perm"]]
            perm.insert(xb, xb)
            out, bd = b.transpose(args[0], perm, name), xb
        elif p == "broadcast":
            xb = dims[0]
            shape = list(e.params["shape"])
            shape.insert(xb, axis_size)
            axis = [ax + (1 if xb <= ax else 0) for ax in e.params["axis"]]
            out, bd = b.broadcast(args[0], shape, axis, name), xb
        elif p == "reshape":
            x = move(args[0], dims[0], 0)
            out, bd = b.reshape(x, [axis_size] + list(e.params["shape"]), name), 0
        elif p == "gather":
            if dims[0] is not None or any(d is None for d in dims[1:]) and len(dims) > 2:
                raise NotImplementedError("vmap of gather: only mapped indices over an unmapped operand")
            rank = max(len(i.shape) + (1 if d is None else 0) for i, d in zip(args[1:], dims[1:]))
            idx = []
            for i, d in zip(args[1:], dims[1:]):
                i = move(i, d, 0)
                if len(i.shape) < rank:
                    i = b.reshape(i, [i.shape[0]] + [1] * (rank - len(i.shape)) + list(i.shape[1:]))
                idx.append(i)
            out = b.gather(args[0], idx, e.params["axis"], e.params["out_dim"], name)
            bd = e.params["out_dim"]
        else:
            raise NotImplementedError(f"vmap rule for {p}")
        env[id(e.out)] = (out, bd)

    outs = []
    for o in jaxpr.outs:
        v, d = env[id(o)]
        moved = move(v, d, 0)
        if moved is not v:      # the output keeps its name, the value before the move gets a new one
            v.name, moved.name = moved.name, v.name
        outs.append(moved)
    return b.build(outs)
