"""The MLP programs as Jaxprs: `valueAndGrad(loss)` of a ReLU MLP with softmax cross-entropy,
its `vmap` over the batch (per-example gradients), and the `optax.adam` update.

The reference's frontend turns these functions into Jaxprs by tracing (`jvp`, partial evaluation
and transposition, src/frontend/jvp.ts and linearize.ts) and cuts the Jaxprs into Kernels
(`jitCompile`).  The cutting is restated in `jaxpr.py`; the tracing is not, so the equations are
written out here, each group with the rule it comes from:

forward (the known half of the partial evaluation)
  * non-differentiated arguments pass through `stopGradient` (`valueAndGrad`,
    linearize.ts:1126-1128); the copy of x this causes is real: `stop_gradient` is not a view
    primitive, so the producer in front of the first Dot is materialised (jit.ts:887-947);
  * `np.dot(x, W)` = `lax.dot` contracting x's last with W's second-to-last axis: W transposed,
    both reshaped to [B,1,K] and [1,N,K], `core.dot` (numpy.ts:1764-1782, lax.ts:87-128);
  * `nn.relu(z) = max(z, 0)` (nn.ts:47-49); its JVP also evaluates `less(z, 0)` on the
    pre-activation (jvp.ts:205-207), a residual of the backward pass;
  * `nn.logSoftmax` (nn.ts:311-322); the JVP of `log` evaluates `reciprocal(s)` (jvp.ts:262-265);
  * `nn.oneHot(y, C) = eye(C)[y]`, a Gather on a constant (nn.ts:430-435);
  * loss = `logits.mul(oneHot).sum().mul(-1 / batch)`
    (website/src/routes/mnist/+page.svelte:139-150).

backward (`evalJaxprTransposed` over the linear half, linearize.ts:553-634, last equation first)
  * Mul by a known factor: `mul(ct, known)`, un-broadcast to the operand (linearize.ts:722-731,
    `unbroadcast` :637-673); Add: the cotangent to both operands (:736-744); Neg: `neg(ct)`;
    Reduce(add): broadcast back (:745-754); Reshape: reshape back (:902-906);
  * a cotangent that arrives twice is `add(old, new)` (:579-586);
  * `where(less(z, 0), 0, dz)`: `where(cond, 0, ct)` (:838-855), so a pre-activation of exactly
    zero passes its cotangent;
  * Dot: `transposeDot` (:676-701): the cotangent broadcast along the contracted axis, both
    operands permuted so that the target's missing axes are contracted, `core.dot`, reshape to
    the target; the parameter's own reshape and transpose are then undone (:885-906), which is
    why each weight gradient ends in a transposing Kernel;
  * order: the equations of the linear Jaxpr come from a depth-first topological sort
    (`partialEvalGraphToJaxpr`, linearize.ts:464-513; `toposort`, utils.ts:252-290) that follows
    the activation chain before the weight operands, so the pullback visits, per layer from
    the last, bias gradient and input cotangent, and only then the weight gradients, first
    layer first.

Under `vmap` every primitive is batched by `vmap_jaxpr` (the reference's batching rules).
`optax.adam`: packages/optax/src/transform.ts:29-72, treeUtils.ts:29-60, base.ts:74-79,
alias.ts:35-40; `np.power` as in numpy.ts:2982-2999.
"""
from __future__ import annotations

import math
from typing import Sequence

import numpy as np

from .alu import AluOp, DType
from .jaxpr import Builder, Jaxpr, Lit, Var, general_broadcast, jit_compile, vmap_jaxpr
from .programs import JitProgram

F32, I32, U32 = DType.Float32, DType.Int32, DType.Uint32


# ---- library functions over a Builder ---------------------------------------------------------

def np_dot(b: Builder, x: Var, w: Var, name: str | None = None):
    """x[B,K] . w[K,N]; returns (product, x reshaped, w reshaped): the reshaped operands are what
    the backward pass contracts against."""
    B, K = x.shape
    N = w.shape[1]
    xr = b.reshape(x, (B, 1, K))
    wr = b.reshape(b.transpose(w, (1, 0)), (1, N, K))
    return b.dot(xr, wr, name), xr, wr


def unbroadcast(b: Builder, x: Var, shape: Sequence[int]) -> Var:
    """linearize.ts:637-673."""
    shape = tuple(shape)
    extra = list(range(len(x.shape) - len(shape)))
    unsqueeze, kept = [], []
    for i, d in enumerate(shape):
        ix = len(x.shape) - (len(shape) - i)
        if x.shape[ix] > 1 and d == 1:
            unsqueeze.append(i)
            kept.append(ix)
    dims = extra + kept
    if not dims:
        return x
    r = b.reduce(x, AluOp.Add, dims)
    if tuple(r.shape) != shape:
        r = b.broadcast(r, shape, unsqueeze)
    return r


def transpose_dot(b: Builder, ct: Var, known: Var, target_shape: Sequence[int], name: str | None = None) -> Var:
    """linearize.ts:676-701."""
    full = general_broadcast(target_shape, known.shape)
    nd = len(full)
    tshape = [1] * (nd - len(target_shape)) + list(target_shape)
    kshape = [1] * (nd - len(known.shape)) + list(known.shape)
    contracting = [a for a in range(nd) if tshape[a] == 1]
    batch = [a for a in range(nd) if tshape[a] != 1]
    perm = batch + contracting

    def dot_shape(shape):
        return [shape[a] for a in batch] + [math.prod(shape[a] for a in contracting)]
    lhs = b.reshape(b.transpose(b.broadcast(ct, full, [nd - 1]), perm), dot_shape(full))
    rhs = b.reshape(b.transpose(b.reshape(known, kshape), perm), dot_shape(kshape))
    return b.reshape(b.dot(lhs, rhs, name), target_shape)


# ---- valueAndGrad(loss) -----------------------------------------------------------------------

def param_order(n_layers: int) -> list:
    """Leaf order of the parameter pytree: W1, b1, W2, b2, ..."""
    return [n for l in range(1, n_layers + 1) for n in (f"W{l}", f"b{l}")]


def mlp_grad_jaxpr(batch: int | None, dims: Sequence[int], scale: float) -> Jaxpr:
    """`valueAndGrad(loss)(params, x, y)`: inputs x, y, eye, then the parameter leaves; outputs the
    loss and one gradient per leaf.  loss = scale * sum(logSoftmax(mlp(x)) * oneHot(y)).
    `batch=None` is the function of a single example (x[D], y[]), the one `vmap` maps."""
    L, C = len(dims) - 1, dims[-1]
    b = Builder()
    single = batch is None
    B = 1 if single else batch
    x_in = b.input("x", (dims[0],) if single else (B, dims[0]))
    y_in = b.input("y", () if single else (B,), I32)
    eye = b.input("eye", (C, C))
    W = [None] + [None] * L
    bias = list(W)
    for l in range(1, L + 1):
        W[l] = b.input(f"W{l}", (dims[l - 1], dims[l]))
        bias[l] = b.input(f"b{l}", (dims[l],))

    # forward
    x = b.stop_gradient(x_in, "x_sg")
    y = b.stop_gradient(y_in)
    if single:
        x = b.reshape(x, (1, dims[0]))
    a, z, lt, ar, wr = [x], [None], [None], [None], [None]
    for l in range(1, L + 1):
        d, xr, w_r = np_dot(b, a[-1], W[l])
        ar.append(xr)
        wr.append(w_r)
        z.append(b.add(d, bias[l], f"z{l}"))
        if l < L:
            a.append(b.max(z[l], Lit(0.0), f"a{l}"))
            lt.append(b.compare(z[l], Lit(0.0), "less"))
    logits = z[L]
    m = b.stop_gradient(b.reshape(b.reduce(logits, AluOp.Max, [1], "m"), (B, 1)))
    sh = b.add(logits, b.neg(m), "shifted")
    e = b.exp(sh, "e")
    sk = b.reshape(b.reduce(e, AluOp.Add, [1], "s"), (B, 1))
    lg = b.log(sk)
    rs = b.reciprocal(sk)
    logp = b.add(sh, b.neg(lg))
    oh = b.gather(eye, [y], [0], 0, "onehot")
    loss = b.mul(b.reduce(b.mul(logp, oh), AluOp.Add, [0, 1]), Lit(scale), "loss")

    # backward from a cotangent of 1
    ct_tot = b.mul(Lit(1.0), Lit(scale))
    ct_prod = b.broadcast(ct_tot, (B, C), [0, 1])
    g0 = b.mul(ct_prod, oh)                                     # cotangent of logp
    ct_lg = b.neg(unbroadcast(b, g0, (B, 1)))                   # add -> (shifted, neg(log s)); neg
    ct_s = b.reshape(b.mul(rs, ct_lg), (B,))                    # log's tangent is reciprocal(s) * ds; reshape
    ct_e = b.broadcast(ct_s, (B, C), [1])                       # reduce(add)
    dz = b.add(g0, b.mul(e, ct_e), f"dz{L}")                    # exp's tangent is e * dshifted; second arrival
    grads = {}
    pending = []
    for l in range(L, 0, -1):
        grads[f"b{l}"] = unbroadcast_to_bias(b, dz, dims[l], f"db{l}")
        pending.append((l, dz))
        if l > 1:
            ct_ar = transpose_dot(b, dz, wr[l], ar[l].shape)   # cotangent of a_{l-1} reshaped [B,1,K]
            ct_a = b.reshape(ct_ar, (B, dims[l - 1]))
            dz = b.where(lt[l - 1], Lit(0.0), ct_a, f"dz{l - 1}")
    for l, dzl in reversed(pending):
        ct_wr = transpose_dot(b, dzl, ar[l], wr[l].shape, f"dW{l}_nk")
        grads[f"W{l}"] = b.transpose(b.reshape(ct_wr, (dims[l], dims[l - 1])), (1, 0), f"dW{l}")
    return b.build([loss] + [grads[n] for n in param_order(L)])


def unbroadcast_to_bias(b: Builder, ct: Var, n: int, name: str) -> Var:
    r = unbroadcast(b, ct, (n,))
    r.name = name
    return r


def mlp_predict_jaxpr(batch: int, dims: Sequence[int]) -> Jaxpr:
    """`(x, W1, b1, ...) => logSoftmax(mlp(x))`, the forward pass alone (the function jitted in
    test/platform-test/node.test.ts:29-58 and website/src/routes/mnist/+page.svelte:70-79).
    Without a backward pass every pre-activation has one consumer, so bias and ReLU fuse into
    the Dot's epilogue (src/frontend/jit.ts:833-885)."""
    L = len(dims) - 1
    b = Builder()
    a = b.input("x", (batch, dims[0]))
    params = []
    for l in range(1, L + 1):
        params.append((b.input(f"W{l}", (dims[l - 1], dims[l])), b.input(f"b{l}", (dims[l],))))
    for l, (w, bias) in enumerate(params, 1):
        z = b.add(np_dot(b, a, w)[0], bias)
        a = b.max(z, Lit(0.0), f"a{l}") if l < L else z
    m = b.stop_gradient(b.reshape(b.reduce(a, AluOp.Max, [1], "m"), (batch, 1)))
    sh = b.add(a, b.neg(m), "shifted")
    lg = b.log(b.reshape(b.reduce(b.exp(sh), AluOp.Add, [1], "s"), (batch, 1)))
    return b.build([b.add(sh, b.neg(lg), "logp")])


def mlp_grad_program(batch: int, dims: Sequence[int], *, global_batch: int | None = None,
                     per_example: bool = False) -> JitProgram:
    """`jit(valueAndGrad(loss))(params, x, y)` as the backend sees it.

    per_example=False: loss = mean NLL over `global_batch` examples of which this program sees
    `batch` (the data-parallel shard; the gradient sum over shards is then the global mean
    gradient).  Outputs: loss (scalar partial sum) and d<leaf> for every parameter.
    per_example=True: `jit(vmap(valueAndGrad(loss1), [null, 0, 0]))` with loss1 the negative log
    likelihood of one example: per-example loss [batch] and per-example gradients, batch axis
    first.
    Inputs: x f32[batch, dims[0]], y i32[batch], eye f32[C, C], then the parameter leaves.
    """
    L = len(dims) - 1
    if per_example:
        inner = mlp_grad_jaxpr(None, dims, -1.0)
        jaxpr = vmap_jaxpr(inner, batch, [0, 0, None] + [None] * (2 * L))
    else:
        jaxpr = mlp_grad_jaxpr(batch, dims, -1.0 / float(global_batch or batch))
    return jit_compile(jaxpr)


ADAM_B1, ADAM_B2, ADAM_EPS = 0.9, 0.999, 1e-8


def _power(b: Builder, x1, x2: Var) -> Var:
    """`np.power` (numpy.ts:2982-2999) of a literal base and a float32 exponent."""
    x2i = b.idiv(x2, Lit(1.0))                                   # trunc
    should_nan = b.mul(b.compare(x2, x2i, "not_equal"), b.compare(x1, Lit(0.0), "less"))
    sign = b.where(b.compare(b.mod(x2i, Lit(2.0)), Lit(0.0), "not_equal"),
                   b.where(b.compare(x1, Lit(0.0), "less"), Lit(-1.0), Lit(1.0)), Lit(1.0))
    absx = b.where(b.compare(x1, Lit(0.0), "less"), b.mul(x1, Lit(-1.0)), x1)
    return b.where(should_nan, Lit(float("nan")), b.mul(b.exp(b.mul(b.log(absx), x2)), sign))


def adam_jaxpr(sizes: Sequence[int], names: Sequence[str], lr: float = 1e-3, order: Sequence[int] | None = None) -> Jaxpr:
    """One jitted `optax.adam(lr)` update followed by `applyUpdates`.

    Inputs: count u32[], then p, g, mu, nu per leaf.  Outputs: count', then p', mu', nu' per leaf.
    `order` lists the leaves in the order their (mutually independent) equations are written."""
    b = Builder()
    count = b.input("count", (), U32)
    leaves = []
    for n, size in zip(names, sizes):
        leaves.append((b.input(n, (size,)), b.input(f"g_{n}", (size,)), b.input(f"mu_{n}", (size,)), b.input(f"nu_{n}", (size,))))
    count_new = b.add(count, Lit(1, U32), "count_new")

    def correction(decay: float, name: str) -> Var:       # treeBiasCorrection
        t = b.cast(count_new, F32)
        return b.reciprocal(b.add(Lit(1.0), b.neg(_power(b, Lit(decay), t))), name)
    outs = {}
    idx = list(range(len(names))) if order is None else list(order)
    mu_new, nu_new = {}, {}
    for i in idx:                                          # treeUpdateMoment, first then second
        p, g, mu, nu = leaves[i]
        mu_new[i] = b.add(b.mul(g, Lit(1 - ADAM_B1)), b.mul(mu, Lit(ADAM_B1)), f"mu_{names[i]}_new")
    for i in idx:
        p, g, mu, nu = leaves[i]
        nu_new[i] = b.add(b.mul(b.mul(g, g), Lit(1 - ADAM_B2)), b.mul(nu, Lit(ADAM_B2)), f"nu_{names[i]}_new")
    c1 = correction(ADAM_B1, "c1")
    c2 = correction(ADAM_B2, "c2")
    for i in idx:
        p = leaves[i][0]
        mu_hat, nu_hat = b.mul(mu_new[i], c1), b.mul(nu_new[i], c2)
        upd = b.mul(mu_hat, b.reciprocal(b.add(b.sqrt(b.add(nu_hat, Lit(0.0))), Lit(ADAM_EPS))))
        outs[i] = b.add(p, b.mul(upd, Lit(-lr)), f"{names[i]}_new")
    flat = [count_new]
    for i in range(len(names)):
        flat += [outs[i], mu_new[i], nu_new[i]]
    return b.build(flat)


def adam_program(sizes: Sequence[int], names: Sequence[str], lr: float = 1e-3, order: Sequence[int] | None = None) -> JitProgram:
    return jit_compile(adam_jaxpr(sizes, names, lr, order))


def leaf_sizes(dims: Sequence[int]) -> list:
    out = []
    for l in range(1, len(dims)):
        out += [dims[l - 1] * dims[l], dims[l]]
    return out


def init_params(dims: Sequence[int], seed: int = 0) -> list:
    """He-normal weights and zero biases, f32 (the synthetic initial state of the benchmarks)."""
    rng = np.random.default_rng(seed)
    leaves = []
    for l in range(1, len(dims)):
        leaves.append((rng.standard_normal((dims[l - 1], dims[l])) * math.sqrt(2.0 / dims[l - 1])).astype(np.float32))
        leaves.append(np.zeros(dims[l], np.float32))
    return leaves


class MlpTrainer:
    """Data-parallel Adam training of an MLP on one rank: the grad program on this rank's shard of
    the batch, an in-place sum of the gradient leaves (and the loss) over ranks, then the Adam
    program -- identical on every rank, so parameters stay replicated."""

    def __init__(self, backend, dims: Sequence[int], local_batch: int, global_batch: int, lr: float = 1e-3,
                 seed: int = 0, allreduce=None, overlap: bool = True, hoist: bool | None = None):
        self.be, self.dims = backend, list(dims)
        self.names = param_order(len(dims) - 1)
        self.sizes = leaf_sizes(dims)
        self.grad = mlp_grad_program(local_batch, dims, global_batch=global_batch)
        n, L = len(self.names), len(dims) - 1
        # The reference's list yields every weight gradient at its end (dW1 .. dWL), where the sum of
        # the largest has nothing left to run under.  With hoist=True dW2 .. dWL move to where their
        # inputs exist, so each of their sums runs under the back-propagation of the layers below; dW1
        # stays last.  Same Kernels, same bits (JitProgram.hoisted).  Off by default: on eight GPUs the
        # step got slower (1.54 ms against 1.47), because a sum that runs beside the persistent GEMMs
        # of back-propagation takes SMs from their static tile schedule.
        self.hoist = bool(hoist) and L >= 2
        if self.hoist:
            self.grad = self.grad.hoisted([f"dW{l}" for l in range(2, L + 1)])
            # the leaves whose gradients travel with the last sum are updated last
            self.late = ["b2", "b1", "W1"]
        else:
            # the last layer's weights last: their gradient is the last to arrive, and with overlapped
            # sums it is still in flight while the other leaves are updated
            self.late = [f"W{L}"]
        tail = [self.names.index(x) for x in self.late]
        self.adam = adam_program(self.sizes, self.names, lr, order=[i for i in range(n) if i not in tail] + tail)
        self.grad.prepare(backend)
        self.adam.prepare(backend)
        self.allreduce = allreduce if allreduce is not None else backend.allreduce_sum_f32
        # With the backend's own sum, each layer's gradient leaves are summed on a second stream as
        # soon as they exist, under the back-propagation of the layers below.
        self.overlap = overlap and allreduce is None and hasattr(backend, "allreduce_sum_f32_async")
        self.params = [backend.put(a) for a in init_params(dims, seed)]
        self.mu = [backend.put(np.zeros(n, np.float32)) for n in self.sizes]
        self.nu = [backend.put(np.zeros(n, np.float32)) for n in self.sizes]
        self.count = backend.put(np.zeros(1, np.uint32))
        self.eye = backend.put(np.eye(dims[-1], dtype=np.float32))

    def _grads(self, x_slot: int, y_slot: int, world: int, params=None):
        """Gradient program followed by the sum over ranks; returns (loss slot, gradient slots)."""
        be = self.be
        ins = [x_slot, y_slot, self.eye] + list(self.params if params is None else params)
        if world <= 1:
            outs = self.grad.execute(be, ins)
        elif not self.overlap:
            outs = self.grad.execute(be, ins)
            self.allreduce(list(outs[1:]) + [outs[0]])
        else:
            # The program yields the loss and the bias gradients first (last layer first), then the
            # weight gradients from the first layer up (hoisted: dWL .. dW2 each right after the
            # cotangent of its layer, dW1 last).  Every weight gradient goes out as soon as it
            # exists, under the kernels that follow it; the loss and the biases (a few KB) ride with the
            # next of them.  The sums stay in flight into the Adam program: the backend makes every
            # Kernel that reads a gradient wait for that gradient's sum (and for no later one).
            ready = []
            last = "dW1" if self.hoist else f"dW{len(self.dims) - 1}"   # the weight gradient the program yields last

            def on_output(name, slot):
                ready.append(slot)
                if name.startswith("dW"):
                    be.allreduce_sum_f32_async(ready)
                    ready.clear()
                    if name == last:
                        self._tail = True

            self._tail = False
            outs = self.grad.execute(be, ins, on_output)
            if ready:
                be.allreduce_sum_f32_async(ready)
            if not self._tail:
                be.comm_join()
        return outs[0], list(outs[1:])

    def _adam(self, ins, out_slots=None):
        """The Adam program; joins the gradient sum still in flight just before its first reader."""
        be = self.be
        late = {f"g_{x}" for x in self.late}

        def before_step(step):
            if self._tail and late.intersection(step.inputs):
                be.comm_join()
                self._tail = False

        new = self.adam.execute(be, ins, out_slots=out_slots, before_step=before_step if getattr(self, "_tail", False) else None)
        if getattr(self, "_tail", False):
            be.comm_join()
            self._tail = False
        return new

    def _state(self):
        return [self.count] + [s for i in range(len(self.names)) for s in (self.params[i], self.mu[i], self.nu[i])]

    def _set_state(self, flat):
        self.count = flat[0]
        self.params, self.mu, self.nu = list(flat[1::3]), list(flat[2::3]), list(flat[3::3])

    def capture(self, x_slot: int, y_slot: int, world: int = 1) -> None:
        """Record one whole step (gradient program, gradient sum, Adam program) as CUDA graphs and
        replay them from then on: `step` becomes a single graph launch instead of ~44 dispatches.

        A graph reads and writes fixed addresses, so the state (count, parameters, moments) lives in
        two sets of buffers and two graphs are recorded: one steps from set 0 into set 1, the other
        from set 1 into set 0, and `step` alternates between them; nothing is copied back.
        x_slot and y_slot are baked in; refresh a batch by writing into them.  Run at least one eager
        step first (kernels set up their scratch on first dispatch)."""
        be = self.be
        cur = self._state()
        other = [be.malloc(4)] + [be.malloc(4 * n) for n in self.sizes for _ in range(3)]
        out_names = self.adam.outputs
        self.graphs, self.graph_loss = [], []
        for src, dst in ((cur, other), (other, cur)):
            be.capture_begin()
            try:
                loss, grads = self._grads(x_slot, y_slot, world, params=src[1::3])
                ins = [src[0]]
                for i in range(len(self.names)):
                    ins += [src[1 + 3 * i], grads[i], src[2 + 3 * i], src[3 + 3 * i]]
                self._adam(ins, out_slots=dict(zip(out_names, dst)))
                for s in grads:
                    be.dec_ref(s)
            except Exception:
                try:
                    be.graph_destroy(be.capture_end())
                except Exception:
                    pass
                raise
            self.graphs.append(be.capture_end())
            self.graph_loss.append(loss)
        self.graph_sets, self.graph_next, self.graph_io = (cur, other), 0, (x_slot, y_slot, world)

    def step(self, x_slot: int, y_slot: int, world: int = 1) -> int:
        """One training step on resident inputs; returns the slot of the (global) loss."""
        be = self.be
        if getattr(self, "graphs", None):
            if (x_slot, y_slot, world) != self.graph_io:
                raise ValueError("the captured step is bound to the slots it was captured with")
            k = self.graph_next
            be.graph_launch(self.graphs[k])
            self.graph_next = 1 - k
            self._set_state(self.graph_sets[1 - k])
            be.inc_ref(self.graph_loss[k])   # the caller releases the loss slot like an eager one
            return self.graph_loss[k]
        loss, grads = self._grads(x_slot, y_slot, world)
        ins = [self.count]
        for i in range(len(self.names)):
            ins += [self.params[i], grads[i], self.mu[i], self.nu[i]]
        new = self._adam(ins)
        for s in [self.count] + self.params + self.mu + self.nu + grads:
            be.dec_ref(s)
        self.count = new[0]
        self.params, self.mu, self.nu = list(new[1::3]), list(new[2::3]), list(new[3::3])
        return loss

    def wait(self, timeout_ms: int) -> None:
        """Watchdog for the steps issued so far.  A gradient sum whose peer is late or gone never
        finishes, and reading the loss behind it would block for ever; this returns once the steps have
        finished, raises TimeoutError after `timeout_ms` (the caller may wait again or leave the
        communicator with `backend.comm_abort()`), and raises the backend's error when the
        communication library reports a failure (the communicator is then already aborted)."""
        self.be.comm_wait(timeout_ms)

    def close(self):
        if getattr(self, "graphs", None):
            for g, l in zip(self.graphs, self.graph_loss):
                self.be.dec_ref(l)
                self.be.graph_destroy(g)
            # the current state is graph_sets[graph_next]; the other set holds the previous step
            for s in self.graph_sets[1 - self.graph_next]:
                self.be.dec_ref(s)
            self.graphs = None
        for s in [self.count, self.eye] + self.params + self.mu + self.nu:
            self.be.dec_ref(s)
