"""Kernel lists of the MLP programs: per-example gradients under `vmap` and the
data-parallel Adam training step.

What is restated here is only the *output* of the reference's device-independent frontend
for these programs -- the Kernels that `jit(valueAndGrad(loss))` and `optax.adam` hand to
`Backend.dispatch`:

  * forward layer = one Dot kernel with bias and ReLU fused as its epilogue
    (src/frontend/jit.ts:833-885; `nn.relu = maximum(x, 0)`, src/library/nn.ts:47-49);
  * loss = softmax cross-entropy composed as in website/src/routes/mnist/+page.svelte:70-148:
    logSoftmax (src/library/nn.ts:311-322) times `oneHot(y)` = `eye(C)[y]`
    (nn.ts:430-435; a Gather whose index is itself a load, src/frontend/jit.ts:715-763);
  * backward = transposed Dots (`transposeDot`, src/frontend/linearize.ts:676-701): dW is a
    contraction over the batch axis with both operands read with stride = row length,
    dX = dY * W^T with the ReLU mask fused; bias gradients are column sums over a strided axis;
  * `optax.adam`: moments, bias correction from a uint32 step counter and the parameter update
    (packages/optax/src/transform.ts:29-72, treeUtils.ts:29-60, base.ts:74-79), per leaf.

Under `vmap` the batch axis of a per-example gradient ends up last
(src/frontend/vmap.ts:297-303), so per-example dW is an outer-product kernel (K = 1) that
streams out [in, out, batch].
"""
from __future__ import annotations

import math
from typing import Sequence

import numpy as np

from .alu import AluExp, AluOp, AluVar, DType, Kernel, Reduction
from .programs import JitProgram, dot_kernel, row_reduce_kernel, softmax_exp_kernel

F32, I32, U32 = DType.Float32, DType.Int32, DType.Uint32
_g, _r = AluVar.gidx, AluVar.ridx


def _i(v: int) -> AluExp:
    return AluExp.i32(v)


def _f(v: float) -> AluExp:
    return AluExp.f32(v)


def _ld(gid: int, length: int, ix: AluExp, dtype: DType = F32) -> AluExp:
    return AluExp.global_index(dtype, gid, length, ix)


# ---- loss pieces ------------------------------------------------------------------------------

def nll_rows_kernel(batch: int, classes: int, scale: float) -> Kernel:
    """l[b] = scale * sum_j (logits[b,j] - m[b] - log s[b]) * eye[y[b], j]; args logits, m, s, y, eye."""
    logit = _ld(0, batch * classes, AluExp.add(AluExp.mul(_g, _i(classes)), _r))
    m, s = _ld(1, batch, _g), _ld(2, batch, _g)
    y = _ld(3, batch, _g, I32)
    hot = _ld(4, classes * classes, AluExp.add(AluExp.mul(y, _i(classes)), _r))
    logp = AluExp.sub(AluExp.add(logit, AluExp.sub(_f(0), m)), AluExp.log(s))
    epilogue = AluExp.mul(AluVar.acc(F32), _f(scale))
    return Kernel(5, batch, AluExp.mul(logp, hot), Reduction(F32, AluOp.Add, classes, epilogue))


def sum_all_kernel(n: int, scale: float) -> Kernel:
    """Scalar scale * sum(v): the mean over the batch."""
    return Kernel(1, 1, _ld(0, n, _r), Reduction(F32, AluOp.Add, n, AluExp.mul(AluVar.acc(F32), _f(scale))))


def dlogits_kernel(batch: int, classes: int, scale: float) -> Kernel:
    """(softmax - onehot) * scale from e = exp(logits - max), s = sum e; args e, s, y, eye."""
    b = AluExp.idiv(_g, _i(classes))
    e, s = _ld(0, batch * classes, _g), _ld(1, batch, b)
    y = _ld(2, batch, b, I32)
    hot = _ld(3, classes * classes, AluExp.add(AluExp.mul(y, _i(classes)), AluExp.mod(_g, _i(classes))))
    return Kernel(4, batch * classes, AluExp.mul(AluExp.sub(AluExp.mul(e, AluExp.reciprocal(s)), hot), _f(scale)))


def backprop_dot_kernel(batch: int, n_in: int, n_out: int) -> Kernel:
    """dz_prev[b,i] = where(a_prev[b,i] > 0, sum_j dz[b,j] * W[i,j], 0); args dz, W, a_prev."""
    k = dot_kernel(batch, n_in, n_out, F32, a_layout="mk", b_layout="nk")
    act = _ld(2, batch * n_in, _g)
    mask = AluExp.cmplt(_f(0), act)
    k.reduction.epilogue = AluExp.where(mask, AluVar.acc(F32), _f(0))
    return Kernel(3, k.size, k.exp, k.reduction)


def column_sum_kernel(rows: int, cols: int) -> Kernel:
    """db[j] = sum_b dz[b,j]."""
    return Kernel(1, cols, _ld(0, rows * cols, AluExp.add(_g, AluExp.mul(_r, _i(cols)))), Reduction(F32, AluOp.Add, rows))


def outer_product_kernel(n_in: int, n_out: int, batch: int) -> Kernel:
    """Per-example dW[i,j,b] = a[b,i] * dz[b,j] (a Dot with K = 1); args a [batch,n_in], dz [batch,n_out]."""
    b = AluExp.mod(_g, _i(batch))
    j = AluExp.mod(AluExp.idiv(_g, _i(batch)), _i(n_out))
    i = AluExp.idiv(_g, _i(batch * n_out))
    a = _ld(0, batch * n_in, AluExp.add(AluExp.mul(b, _i(n_in)), i))
    dz = _ld(1, batch * n_out, AluExp.add(AluExp.mul(b, _i(n_out)), j))
    return Kernel(2, n_in * n_out * batch, AluExp.mul(a, dz))


def batch_last_kernel(batch: int, n: int) -> Kernel:
    """Per-example db[j,b] = dz[b,j]: the batch axis moved last."""
    ix = AluExp.add(AluExp.mul(AluExp.mod(_g, _i(batch)), _i(n)), AluExp.idiv(_g, _i(batch)))
    return Kernel(1, batch * n, _ld(0, batch * n, ix))


# ---- programs ---------------------------------------------------------------------------------

def _names(n_layers: int):
    return [f"W{l}" for l in range(1, n_layers + 1)], [f"b{l}" for l in range(1, n_layers + 1)]


def param_order(n_layers: int) -> list:
    """Leaf order of the parameter pytree: W1, b1, W2, b2, ..."""
    ws, bs = _names(n_layers)
    return [n for pair in zip(ws, bs) for n in pair]


def mlp_grad_program(batch: int, dims: Sequence[int], *, global_batch: int | None = None,
                     per_example: bool = False) -> JitProgram:
    """`valueAndGrad(loss)(params, x, y)` for an MLP with ReLU hidden layers and softmax
    cross-entropy.

    per_example=False: loss = mean NLL over `global_batch` examples of which this program sees
    `batch` (the data-parallel shard; the gradient sum over shards is then the global mean
    gradient).  Outputs: loss (scalar partial sum) and d<leaf> for every parameter.
    per_example=True: the `vmap`-ed program: per-example loss [batch] and per-example gradients
    with the batch axis last.
    Inputs: x f32[batch, dims[0]], y i32[batch], eye f32[C, C], then the parameter leaves.
    """
    L = len(dims) - 1
    C = dims[-1]
    ws, bs = _names(L)
    leaves = param_order(L)
    p = JitProgram(inputs=["x", "y", "eye"] + leaves, outputs=["loss"] + [f"d{n}" for n in leaves])
    scale = 1.0 if per_example else 1.0 / float(global_batch or batch)
    acts = ["x"]
    for l in range(1, L + 1):
        k = dot_kernel(batch, dims[l], dims[l - 1], F32, bias=True, relu=l < L)
        p.run(f"a{l}", k, [acts[-1], ws[l - 1], bs[l - 1]])
        acts.append(f"a{l}")
    logits = acts[-1]
    p.run("m", row_reduce_kernel(batch, C, AluOp.Max), [logits])
    p.run("e", softmax_exp_kernel(batch, C), [logits, "m"])
    p.run("s", row_reduce_kernel(batch, C, AluOp.Add), ["e"])
    if per_example:
        p.run("loss", nll_rows_kernel(batch, C, -1.0), [logits, "m", "s", "y", "eye"])
    else:
        p.run("nll", nll_rows_kernel(batch, C, 1.0), [logits, "m", "s", "y", "eye"])
        p.run("loss", sum_all_kernel(batch, -scale), ["nll"])
        p.free("nll")
    p.run(f"dz{L}", dlogits_kernel(batch, C, scale), ["e", "s", "y", "eye"])
    for n in ("m", "e", "s"):
        p.free(n)
    for l in range(L, 0, -1):
        dz, a_prev = f"dz{l}", acts[l - 1]
        if per_example:
            p.run(f"dW{l}", outer_product_kernel(dims[l - 1], dims[l], batch), [a_prev, dz])
            p.run(f"db{l}", batch_last_kernel(batch, dims[l]), [dz])
        else:
            p.run(f"dW{l}", dot_kernel(dims[l - 1], dims[l], batch, F32, a_layout="km", b_layout="kn"), [a_prev, dz])
            p.run(f"db{l}", column_sum_kernel(batch, dims[l]), [dz])
        if l > 1:
            p.run(f"dz{l - 1}", backprop_dot_kernel(batch, dims[l - 1], dims[l]), [dz, ws[l - 1], a_prev])
        p.free(dz)
        if l < L:
            p.free(acts[l])
    p.free(acts[L])
    return p


ADAM_B1, ADAM_B2, ADAM_EPS = 0.9, 0.999, 1e-8


def adam_program(sizes: Sequence[int], names: Sequence[str], lr: float = 1e-3, order: Sequence[int] | None = None) -> JitProgram:
    """`optax.adam(lr)` update + `applyUpdates` over the parameter leaves.

    Inputs: count u32[1], then p, g, mu, nu per leaf.  Outputs: count', then p', mu', nu' per leaf.
    `order` lists the leaves in the order their (mutually independent) kernels are dispatched.
    """
    ins, outs = ["count"], ["count_new"]
    for n in names:
        ins += [n, f"g_{n}", f"mu_{n}", f"nu_{n}"]
        outs += [f"{n}_new", f"mu_{n}_new", f"nu_{n}_new"]
    p = JitProgram(inputs=ins, outputs=outs)
    one = AluExp.u32(1)
    p.run("count_new", Kernel(1, 1, AluExp.add(_ld(0, 1, _g, U32), one)), ["count"])

    def correction(decay: float) -> Kernel:   # 1 / (1 - decay**t), t from the uint32 counter
        t = AluExp.cast(F32, _ld(0, 1, _g, U32))
        return Kernel(1, 1, AluExp.reciprocal(AluExp.sub(_f(1), AluExp.exp(AluExp.mul(t, _f(math.log(decay)))))))

    p.run("c1", correction(ADAM_B1), ["count_new"])
    p.run("c2", correction(ADAM_B2), ["count_new"])
    for leaf in (range(len(names)) if order is None else order):
        n, size = names[leaf], sizes[leaf]
        g, mu, nu = _ld(0, size, _g), _ld(1, size, _g), _ld(1, size, _g)
        p.run(f"mu_{n}_new", Kernel(2, size, AluExp.add(AluExp.mul(g, _f(1 - ADAM_B1)), AluExp.mul(mu, _f(ADAM_B1)))),
              [f"g_{n}", f"mu_{n}"])
        p.run(f"nu_{n}_new", Kernel(2, size, AluExp.add(AluExp.mul(AluExp.mul(g, g), _f(1 - ADAM_B2)), AluExp.mul(nu, _f(ADAM_B2)))),
              [f"g_{n}", f"nu_{n}"])
        par, m2, n2 = _ld(0, size, _g), _ld(1, size, _g), _ld(2, size, _g)
        c1, c2 = _ld(3, 1, _i(0)), _ld(4, 1, _i(0))
        denom = AluExp.add(AluExp.sqrt(AluExp.mul(n2, c2)), _f(ADAM_EPS))
        upd = AluExp.mul(AluExp.mul(AluExp.mul(m2, c1), AluExp.reciprocal(denom)), _f(-lr))
        p.run(f"{n}_new", Kernel(5, size, AluExp.add(par, upd)), [n, f"mu_{n}_new", f"nu_{n}_new", "c1", "c2"])
    p.free("c1")
    p.free("c2")
    return p


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
                 seed: int = 0, allreduce=None, overlap: bool = True):
        self.be, self.dims = backend, list(dims)
        self.names = param_order(len(dims) - 1)
        self.sizes = leaf_sizes(dims)
        self.grad = mlp_grad_program(local_batch, dims, global_batch=global_batch)
        # leaves of the last layer first: the first layer's gradients are the last to arrive, and
        # with overlapped sums theirs is still in flight while the other leaves are updated
        self.adam = adam_program(self.sizes, self.names, lr, order=list(reversed(range(len(self.names)))))
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
            ready = []

            def on_output(name, slot):
                ready.append(slot)
                if name.startswith("db"):        # a layer's last leaf: dW and db go out together
                    if name == "db1":
                        # everything summed so far is waited for here; the first layer's own sum, begun
                        # next, is only waited for by the Adam kernels that read it (`_adam`)
                        be.comm_join()
                        self._tail = True
                    be.allreduce_sum_f32_async(ready)
                    ready.clear()

            self._tail = False
            outs = self.grad.execute(be, ins, on_output)
            if ready:
                be.allreduce_sum_f32_async(ready)
            if not self._tail:
                be.comm_join()
        return outs[0], list(outs[1:])

    def _adam(self, ins, out_slots=None):
        """The Adam program; joins a first-layer gradient sum still in flight just before its first reader."""
        be = self.be
        first_layer = {f"g_{self.names[0]}", f"g_{self.names[1]}"}

        def before_step(step):
            if self._tail and first_layer.intersection(step.inputs):
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
