"""Kernel sequences that `jit` hands to a backend for the benchmarked programs.

The reference's tracing frontend is device-independent and stays in TypeScript; what the
backend sees per program is a static list of malloc / execute / free steps
(`JitProgram`, src/frontend/jit.ts:111-162).  This module builds those lists directly,
kernel by kernel, in the form the frontend's rules produce them:

  * `np.dot` / `lax.dot`: Mul of two loads under an Add reduction
    (`jitRules[Dot]`, src/frontend/jit.ts:639-648; operand views of src/library/lax.ts:87-128);
  * `nn.softmax` = max, exp(x - max) materialised, sum, mul by reciprocal: four kernels,
    because the keepdims reshape blocks epilogue fusion and exp has two consumers
    (src/library/nn.ts:291-301; src/frontend/jit.ts:833-885, :1015-1028);
  * `nn.logsumexp` (nn.ts:332-345) and `np.argmax` (src/library/numpy.ts:533-556).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from .alu import AluExp, AluOp, AluVar, DType, Kernel, Reduction, byte_width, np_dtype

F32, I32, F16 = DType.Float32, DType.Int32, DType.Float16
_g, _r = AluVar.gidx, AluVar.ridx


def _i(v: int) -> AluExp:
    return AluExp.i32(v)


# ---- single kernels ---------------------------------------------------------------------

def row_reduce_kernel(rows: int, cols: int, op: AluOp, dtype: DType = F32) -> Kernel:
    """K1 / K3: reduce the last axis of a contiguous [rows, cols] array."""
    x = AluExp.global_index(dtype, 0, rows * cols, AluExp.add(AluExp.mul(_g, _i(cols)), _r))
    return Kernel(1, rows, x, Reduction(dtype, op, cols))


def softmax_exp_kernel(rows: int, cols: int) -> Kernel:
    """K2: exp(x + (0 - max[row])), materialised."""
    x = AluExp.global_index(F32, 0, rows * cols, _g)
    m = AluExp.global_index(F32, 1, rows, AluExp.idiv(_g, _i(cols)))
    return Kernel(2, rows * cols, AluExp.exp(AluExp.add(x, AluExp.sub(AluExp.f32(0), m))))


def softmax_scale_kernel(rows: int, cols: int) -> Kernel:
    """K4: u * (1 / sum[row])."""
    u = AluExp.global_index(F32, 0, rows * cols, _g)
    s = AluExp.global_index(F32, 1, rows, AluExp.idiv(_g, _i(cols)))
    return Kernel(2, rows * cols, AluExp.mul(u, AluExp.reciprocal(s)))


def lse_sum_kernel(rows: int, cols: int) -> Kernel:
    """K2': row sum of exp(x - max) with the exponential fused as the reduction body."""
    x = AluExp.global_index(F32, 0, rows * cols, AluExp.add(AluExp.mul(_g, _i(cols)), _r))
    m = AluExp.global_index(F32, 1, rows, _g)
    return Kernel(2, rows, AluExp.exp(AluExp.add(x, AluExp.sub(AluExp.f32(0), m))), Reduction(F32, AluOp.Add, cols))


def lse_finish_kernel(rows: int) -> Kernel:
    """K3': max + log(sum)."""
    s = AluExp.global_index(F32, 0, rows, _g)
    m = AluExp.global_index(F32, 1, rows, _g)
    return Kernel(2, rows, AluExp.add(m, AluExp.log(s)))


def argmax_index_kernel(rows: int, cols: int) -> Kernel:
    """K5: int32 row max of cast(x == max) * (n - ridx) with epilogue n - acc.

    `G_2` is the closed-over constant arange(n, 0, -1) (numpy.ts:533-556); ties resolve to
    the first index because the largest weight wins.
    """
    x = AluExp.global_index(F32, 0, rows * cols, AluExp.add(AluExp.mul(_g, _i(cols)), _r))
    m = AluExp.global_index(F32, 1, rows, _g)
    w = AluExp.global_index(I32, 2, cols, _r)
    eq = AluExp.cmpne(x, m).not_()
    body = AluExp.mul(AluExp.cast(I32, eq), w)
    epilogue = AluExp.add(_i(cols), AluExp.sub(_i(0), AluVar.acc(I32)))
    return Kernel(3, rows, body, Reduction(I32, AluOp.Max, cols, epilogue))


def dot_kernel(M: int, N: int, K: int, dtype: DType = F32, *, a_layout: str = "mk", b_layout: str = "kn",
               batch: int = 1, bias: bool = False, relu: bool = False, swap: bool = False) -> Kernel:
    """C[b, m, n] = sum_k A[b, m, k] * B[b, k, n], optionally + bias[n] and relu, as one Kernel.

    Layouts name the memory order of each operand: "mk" is row-major A, "km" its transpose;
    "kn" is row-major B (the `np.dot` case: read with stride N along k), "nk" its transpose.
    `swap` writes the product as B*A (operand order of src/backend/backend.test.ts:447-458).
    """
    m = AluExp.mod(AluExp.idiv(_g, _i(N)), _i(M))
    n = AluExp.mod(_g, _i(N))
    b = AluExp.idiv(_g, _i(M * N))
    a_ix = AluExp.add(AluExp.mul(m, _i(K)), _r) if a_layout == "mk" else AluExp.add(m, AluExp.mul(_r, _i(M)))
    b_ix = AluExp.add(n, AluExp.mul(_r, _i(N))) if b_layout == "kn" else AluExp.add(AluExp.mul(n, _i(K)), _r)
    if batch > 1:
        a_ix = AluExp.add(AluExp.mul(b, _i(M * K)), a_ix)
        b_ix = AluExp.add(AluExp.mul(b, _i(K * N)), b_ix)
    la = AluExp.global_index(dtype, 0, batch * M * K, a_ix)
    lb = AluExp.global_index(dtype, 1, batch * K * N, b_ix)
    body = AluExp.mul(lb, la) if swap else AluExp.mul(la, lb)
    red = Reduction(dtype, AluOp.Add, K)
    nargs = 2
    if bias or relu:
        acc = red.epilogue  # already Cast<f16>(acc:f32) for float16
        if bias:
            acc = AluExp.add(acc, AluExp.global_index(dtype, 2, N, AluExp.mod(_g, _i(N))))
            nargs = 3
        if relu:
            acc = AluExp.max(acc, AluExp.const(dtype, 0))
        red.epilogue = acc
    return Kernel(nargs, batch * M * N, body, red)


def matvec_kernel(rows: int, cols: int, dtype: DType = F16, *, orientation: str = "xW") -> Kernel:
    """"xW": y[n] = sum_k x[k] W[k, n] for W[rows=K, cols=N] (`np.dot(x, W)`);
    "Wx": y[m] = sum_k W[m, k] x[k] for W[rows=M, cols=K] (`np.dot(W, x)`)."""
    if orientation == "xW":
        x = AluExp.global_index(dtype, 0, rows, _r)
        w = AluExp.global_index(dtype, 1, rows * cols, AluExp.add(_g, AluExp.mul(_r, _i(cols))))
        return Kernel(2, cols, AluExp.mul(x, w), Reduction(dtype, AluOp.Add, rows))
    w = AluExp.global_index(dtype, 0, rows * cols, AluExp.add(AluExp.mul(_g, _i(cols)), _r))
    x = AluExp.global_index(dtype, 1, cols, _r)
    return Kernel(2, rows, AluExp.mul(w, x), Reduction(dtype, AluOp.Add, cols))


def conv2d_kernel(N: int, Ci: int, H: int, W: int, Co: int, KH: int, KW: int, stride: int = 1, pad: int = 0,
                  dtype: DType = F32) -> Kernel:
    """out[n, co, oh, ow] = sum_{ci, kh, kw} x[n, ci, oh*stride + kh - pad, ow*stride + kw - pad] * w[co, ci, kh, kw]
    over NCHW input and OIHW weights, the padded taps read as Where(valid, load, 0): the Kernel
    `jitRules[Conv]` builds from the pooled views of `prepareConv` (src/frontend/jit.ts:649-660,
    src/frontend/convolution.ts)."""
    OH, OW = (H + 2 * pad - KH) // stride + 1, (W + 2 * pad - KW) // stride + 1
    i = _i
    ow, oh = AluExp.mod(_g, i(OW)), AluExp.mod(AluExp.idiv(_g, i(OW)), i(OH))
    co, n = AluExp.mod(AluExp.idiv(_g, i(OW * OH)), i(Co)), AluExp.idiv(_g, i(OW * OH * Co))
    kw, kh, ci = AluExp.mod(_r, i(KW)), AluExp.mod(AluExp.idiv(_r, i(KW)), i(KH)), AluExp.idiv(_r, i(KW * KH))
    ih = AluExp.add(AluExp.add(AluExp.mul(oh, i(stride)), kh), i(-pad))
    iw = AluExp.add(AluExp.add(AluExp.mul(ow, i(stride)), kw), i(-pad))

    def inside(v, hi):
        return AluExp.mul(AluExp.cast(I32, AluExp.cmplt(i(-1), v)), AluExp.cast(I32, AluExp.cmplt(v, i(hi))))
    valid = AluExp.cmpne(AluExp.mul(inside(ih, H), inside(iw, W)), i(0))
    xi = AluExp.add(AluExp.mul(AluExp.add(AluExp.mul(AluExp.add(AluExp.mul(n, i(Ci)), ci), i(H)), ih), i(W)), iw)
    x = AluExp.where(valid, AluExp.global_index(dtype, 0, N * Ci * H * W, xi), AluExp.const(dtype, 0))
    wv = AluExp.global_index(dtype, 1, Co * Ci * KH * KW, AluExp.add(AluExp.mul(co, i(Ci * KH * KW)), _r))
    return Kernel(2, N * Co * OH * OW, AluExp.mul(x, wv), Reduction(dtype, AluOp.Add, Ci * KH * KW))


# ---- step lists ---------------------------------------------------------------------------

@dataclass
class Step:
    kind: str                       # "malloc" | "execute" | "free"
    name: str = ""                  # malloc/free: buffer name; execute: output buffer name
    nbytes: int = 0
    kernel: Kernel | None = None
    inputs: Sequence[str] = ()


@dataclass
class JitProgram:
    """Static step list replayed per call (src/frontend/jit.ts:111-162)."""
    inputs: Sequence[str]
    outputs: Sequence[str]
    steps: list = field(default_factory=list)
    _exes: dict = field(default_factory=dict, repr=False)

    def malloc(self, name: str, nbytes: int) -> None:
        self.steps.append(Step("malloc", name, nbytes))

    def run(self, out: str, kernel: Kernel, inputs: Sequence[str]) -> None:
        self.steps.append(Step("malloc", out, kernel.bytes))
        self.steps.append(Step("execute", out, 0, kernel, tuple(inputs)))

    def free(self, name: str) -> None:
        self.steps.append(Step("free", name))

    def kernels(self):
        return [s.kernel for s in self.steps if s.kind == "execute"]

    def prepare(self, backend) -> None:
        for s in self.steps:
            if s.kind == "execute" and id(s) not in self._exes:
                self._exes[id(s)] = backend.prepare_kernel_sync(s.kernel)

    def execute(self, backend, slots: Sequence[int], on_output=None, out_slots=None, before_step=None) -> list:
        """Replays the steps; `slots` are the input slots (not consumed).  Returns output slots
        with reference count 1, owned by the caller.  `on_output(name, slot)` is called right after
        the kernel that produces a program output has been dispatched.  `out_slots` maps names of
        program outputs to slots the caller already owns: those outputs are written there instead of
        into fresh slots (they must not alias an input of the kernel that writes them).
        `before_step(step)` is called before each kernel is dispatched."""
        self.prepare(backend)
        env = dict(zip(self.inputs, slots))
        owned = set()
        for s in self.steps:
            if s.kind == "malloc":
                if out_slots and s.name in out_slots:
                    env[s.name] = out_slots[s.name]
                    continue
                env[s.name] = backend.malloc(s.nbytes)
                owned.add(s.name)
            elif s.kind == "execute":
                if before_step is not None:
                    before_step(s)
                backend.dispatch(self._exes[id(s)], [env[n] for n in s.inputs], [env[s.name]])
                if on_output is not None and s.name in self.outputs:
                    on_output(s.name, env[s.name])
            elif s.kind == "free" and s.name in owned:
                backend.dec_ref(env.pop(s.name))
                owned.discard(s.name)
        outs = [env[n] for n in self.outputs]
        for n in owned - set(self.outputs):
            backend.dec_ref(env[n])
        return outs

    def capture(self, backend, slots: Sequence[int]):
        """Record the step list as one CUDA graph (jaxcuda_capture_begin/end).  Returns
        (graph, output slots): every `backend.graph_launch(graph)` recomputes the outputs in place
        from whatever the input slots hold then.  The program is dispatched eagerly once first, so
        that every kernel has set up its scratch."""
        for s in self.execute(backend, slots):
            backend.dec_ref(s)
        backend.capture_begin()
        try:
            outs = self.execute(backend, slots)
        except Exception:
            backend.graph_destroy(backend.capture_end())
            raise
        return backend.capture_end(), outs

    def hoisted(self, targets: Sequence[str]) -> "JitProgram":
        """The same Kernels in another order: the Kernel that writes each of `targets`, together with
        the chain of intermediates that only it reads, moves to the earliest point at which its inputs
        exist; everything else keeps its order, and every intermediate is released after its last
        reader in the new order.  Only independent steps change places, so every Kernel sees the
        inputs it saw before and the outputs are the same bits.  (The reference's executor runs its
        list front to back, src/frontend/jit.ts:111-162; a driver that overlaps communication with the
        list wants an output that feeds a long transfer to exist early.)"""
        ex = [s for s in self.steps if s.kind == "execute"]
        nbytes = {s.name: s.nbytes for s in self.steps if s.kind == "malloc"}
        pos = {s.name: i for i, s in enumerate(ex)}
        uses: dict = {}
        for s in ex:
            for n in set(s.inputs):
                uses[n] = uses.get(n, 0) + 1
        after: dict = {}          # position -> chains to run right after it
        moved = set()
        for t in targets:
            if t not in pos:
                raise ValueError(f"{t} is not written by a Kernel of this program")
            chain = [pos[t]]
            while True:
                private = [n for n in ex[chain[0]].inputs if n in pos and uses.get(n) == 1 and n not in self.outputs]
                if len(private) != 1 or pos[private[0]] in moved:
                    break
                chain.insert(0, pos[private[0]])
            ready = max([pos[n] for i in chain for n in ex[i].inputs if n in pos and pos[n] not in chain], default=-1)
            if ready >= chain[0]:
                continue          # already as early as it can be
            moved.update(chain)
            after.setdefault(ready, []).append(chain)
        order = [i for chain in after.get(-1, []) for i in chain]
        for i in range(len(ex)):
            if i in moved:
                continue
            order.append(i)
            for chain in after.get(i, []):
                order.extend(chain)
        last_use = {}
        for rank, i in enumerate(order):
            for n in ex[i].inputs:
                last_use[n] = rank
        out = JitProgram(list(self.inputs), list(self.outputs))
        for rank, i in enumerate(order):
            s = ex[i]
            out.steps.append(Step("malloc", s.name, nbytes[s.name]))
            out.steps.append(Step("execute", s.name, 0, s.kernel, tuple(s.inputs)))
            for n in dict.fromkeys(s.inputs):
                if n in pos and n not in self.outputs and last_use[n] == rank:
                    out.steps.append(Step("free", n))
            if s.name not in last_use and s.name not in self.outputs:
                out.steps.append(Step("free", s.name))
        return out

    def cost(self, backend):
        """Sum of algorithmic bytes, flops and launches over the execute steps."""
        self.prepare(backend)
        tot = [0.0, 0.0, 0]
        for s in self.steps:
            if s.kind == "execute":
                b, f, n = self._exes[id(s)].cost()
                tot[0] += b
                tot[1] += f
                tot[2] += n
        return tuple(tot)


def softmax_lse_argmax_jaxpr(rows: int, cols: int):
    """`(x) => [nn.softmax(x), nn.logsumexp(x, -1), np.argmax(x, -1)]` as the Jaxpr tracing yields:
    src/library/nn.ts:291-301 (softmax), :332-345 (logsumexp), src/library/numpy.ts:533-556 (argmax;
    its `arange(n, 0, -1)` is a closed-over constant, here the second input).  `sub` is `add(neg)`
    and float `div` is `mul(reciprocal)` (src/frontend/core.ts:945-955); a `keepdims` reduction is
    a Reduce followed by a Reshape (core.ts:271-289)."""
    from .jaxpr import Builder, Lit
    b = Builder()
    x = b.input("x", (rows, cols))
    iota = b.input("iota", (cols,), I32)
    keep = (rows, 1)
    # softmax
    m1 = b.stop_gradient(b.reshape(b.reduce(x, AluOp.Max, [1], "m1"), keep))
    u = b.exp(b.add(x, b.neg(m1)), "u")
    s = b.reshape(b.reduce(u, AluOp.Add, [1], "s"), keep)
    softmax = b.mul(u, b.reciprocal(s), "softmax")
    # logsumexp
    m2 = b.stop_gradient(b.reshape(b.reduce(x, AluOp.Max, [1], "m2"), keep), "m2k")
    s2 = b.reshape(b.reduce(b.exp(b.add(x, b.neg(m2))), AluOp.Add, [1], "s2"), keep)
    lse = b.reshape(b.add(m2, b.log(s2)), (rows,), "lse")
    # argmax
    m3 = b.reshape(b.reduce(x, AluOp.Max, [1], "m3"), keep)
    idx = b.mul(b.cast(b.compare(x, m3, "equal"), I32), b.reshape(iota, (cols,)))
    argmax = b.add(Lit(cols, I32), b.neg(b.reduce(idx, AluOp.Max, [1])), "argmax")
    return b.build([softmax, lse, argmax])


def softmax_lse_argmax_program(rows: int, cols: int) -> JitProgram:
    """One jit computing softmax, logsumexp and argmax of x[rows, cols] over the last axis, cut into
    Kernels by the reference's rules (`jaxpr.jit_compile`).

    `Jaxpr.simplify` does no common-subexpression elimination (src/frontend/jaxpr.ts:252-257), so
    the row max is computed three times, once per consumer.  logsumexp uses its stop-gradient row
    max twice (in the shift and in the result), which makes that value reach two dispatched
    Kernels and therefore a Kernel of its own (a copy of `rows` elements; src/frontend/jit.ts:1006-1028).
    Inputs: x and the constant arange(cols, 0, -1); outputs: softmax f32[rows, cols], lse f32[rows],
    argmax i32[rows]; ten Kernels."""
    from .jaxpr import jit_compile
    return jit_compile(softmax_lse_argmax_jaxpr(rows, cols))


def argmax_iota(cols: int) -> np.ndarray:
    return np.arange(cols, 0, -1, dtype=np.int32)
