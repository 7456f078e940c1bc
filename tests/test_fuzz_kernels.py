"""Seeded random Kernels.  On CPU: through the planner, the CUDA C emitter and NVRTC (no GPU needed), and
through the oracle: whatever expression the frontend could hand over must either compile for
sm_100a or be refused with the reference's UnsupportedOpError wording, never produce source that
does not compile; and the oracle must evaluate every accepted kernel.  On a GPU: the same kernels
run through the C ABI and are compared with the oracle (integer chains bit-exact, float chains
within the amplified single-op bar)."""
import numpy as np
import pytest

import oracle
from jax_js_b200 import AluExp, AluOp, AluVar, DType, Kernel, Reduction, np_dtype
from jax_js_b200.backend import UnsupportedOpError, check_kernel

F32, I32, U32, BOOL, F16 = DType.Float32, DType.Int32, DType.Uint32, DType.Bool, DType.Float16
g, r = AluVar.gidx, AluVar.ridx


class Gen:
    def __init__(self, rng, size, red):
        self.rng, self.size, self.red, self.args = rng, size, red, []   # args: (dtype, length)

    def pick(self, seq):
        return seq[int(self.rng.integers(len(seq)))]

    def index(self):
        """An int32 index expression over gidx (and ridx under a reduction), with its value range end."""
        i = AluExp.i32
        forms = [(g, self.size), (AluExp.idiv(g, i(3)), (self.size + 2) // 3), (AluExp.mod(g, i(5)), 5), (i(2), 3)]
        if self.red:
            forms += [(AluExp.add(AluExp.mul(g, i(self.red)), r), self.size * self.red), (r, self.red),
                      (AluExp.add(g, AluExp.mul(r, i(self.size))), self.size * self.red)]
        return self.pick(forms)

    def load(self, dtype):
        ix, length = self.index()
        if self.rng.random() < 0.15:
            length = max(1, length // 2)          # some loads may run out of range: they read element 0
        self.args.append((dtype, length))
        return AluExp.global_index(dtype, len(self.args) - 1, length, ix)

    def leaf(self, dtype):
        c = self.rng.random()
        if c < 0.55:
            return self.load(dtype)
        if c < 0.75 and dtype in (I32, U32):
            return AluExp.cast(dtype, g)
        v = {F32: 1.5, F16: 0.5, I32: -3, U32: 7, BOOL: True}[dtype]
        return AluExp.const(dtype, v)

    def exp(self, dtype, depth):
        if depth == 0:
            return self.leaf(dtype)
        sub = lambda dt=dtype: self.exp(dt, depth - 1)
        if dtype == BOOL:
            kind = self.pick(["cmplt", "cmpne", "not", "and", "leaf"])
            src = self.pick([F32, I32, U32])
            if kind == "cmplt":
                return AluExp.cmplt(sub(src), sub(src))
            if kind == "cmpne":
                return AluExp.cmpne(sub(src), sub(src))
            if kind == "not":
                return sub().not_()
            if kind == "and":
                return AluExp.mul(sub(), sub())
            return self.leaf(BOOL)
        ops = ["add", "sub", "mul", "min", "max", "where", "cast", "idiv", "mod", "leaf"]
        if dtype in (F32, F16):
            ops += ["exp", "log", "sin", "cos", "sqrt", "reciprocal", "floor", "erf", "atan"]
        else:
            ops += ["and", "xor", "shl", "shr", "invert", "bitcast"]
        op = self.pick(ops)
        if op in ("add", "sub", "mul", "min", "max", "idiv", "mod"):
            return getattr(AluExp, op)(sub(), sub())
        if op == "where":
            return AluExp.where(self.exp(BOOL, depth - 1), sub(), sub())
        if op == "cast":
            return AluExp.cast(dtype, sub(self.pick([F32, I32, U32, BOOL])))
        if op == "bitcast":
            return AluExp.bitcast(dtype, sub(self.pick([F32, I32, U32])))
        if op in ("and", "xor"):
            return AluExp.bit_combine(sub(), sub(), op)
        if op in ("shl", "shr"):
            return AluExp.bit_shift(sub(), sub(), op)
        if op == "invert":
            return AluExp.bit_invert(sub())
        if op == "leaf":
            return self.leaf(dtype)
        return getattr(AluExp, op)(sub())


def random_kernel(seed):
    rng = np.random.default_rng(seed)
    size = int(rng.choice([1, 7, 64, 1000, 4099, 65536]))
    red = int(rng.choice([0, 0, 3, 10, 64, 513]))
    dtype = [F32, F32, I32, U32, BOOL, F16][int(rng.integers(6))]
    gen = Gen(rng, size, red)
    body = gen.exp(dtype, int(rng.integers(1, 4)))
    reduction = None
    if red:
        op = [AluOp.Add, AluOp.Max, AluOp.Min, AluOp.Mul][int(rng.integers(4))]
        reduction = Reduction(dtype, op, red)
        if rng.random() < 0.5 and dtype != BOOL:
            acc = reduction.epilogue
            reduction.epilogue = AluExp.add(acc, AluExp.cast(acc.dtype, AluExp.mod(g, AluExp.i32(3))))
    return Kernel(len(gen.args), size, body, reduction), gen.args


@pytest.mark.parametrize("seed", range(48))
def test_random_kernel_compiles_or_is_refused_and_the_oracle_runs_it(seed):
    kernel, args = random_kernel(seed)
    rng = np.random.default_rng(1000 + seed)
    arrays = []
    for dtype, length in args:
        if dtype in (F32, F16):
            arrays.append(rng.uniform(-2, 2, length).astype(np_dtype(dtype)))
        elif dtype == BOOL:
            arrays.append(rng.integers(0, 2, length).astype(np.int32))
        else:
            arrays.append(rng.integers(0, 50, length).astype(np_dtype(dtype)))
    try:
        describe, source = check_kernel(kernel, compile=True)
    except UnsupportedOpError as e:
        assert "not supported in cuda backend" in str(e)
        return
    assert describe and 'extern "C" __global__' in source
    out = oracle.run_kernel(kernel, arrays, end=min(kernel.size, 256))
    assert out.shape == (kernel.size,)


def _inputs_for(args, seed):
    rng = np.random.default_rng(1000 + seed)
    arrays = []
    for dtype, length in args:
        if dtype in (F32, F16):
            arrays.append(rng.uniform(-2, 2, length).astype(np_dtype(dtype)))
        elif dtype == BOOL:
            arrays.append(rng.integers(0, 2, length).astype(np.int32))
        else:
            arrays.append(rng.integers(0, 50, length).astype(np_dtype(dtype)))
    return arrays


def _is_exact(kernel):
    """Integer and Bool results that never pass through a float: bit-exact by construction."""
    roots = [kernel.exp] + ([kernel.reduction.epilogue] if kernel.reduction else [])
    return kernel.dtype in (I32, U32, BOOL) and all(e.dtype in (I32, U32, BOOL) for root in roots for e in root.toposort())


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(48))
def test_random_kernel_matches_the_oracle_on_the_gpu(backend, seed):
    from util import run_cuda
    kernel, args = random_kernel(seed)
    arrays = _inputs_for(args, seed)
    got = run_cuda(backend, kernel, arrays)
    want = oracle.run_kernel(kernel, arrays)
    if _is_exact(kernel):
        assert np.array_equal(got, want)
        return
    if kernel.dtype in (I32, U32, BOOL):
        # an integer made from floats (casts, comparisons): a float within rounding of a boundary may
        # land on either side; all but a sliver must agree
        assert (got != want).mean() <= 0.01
        return
    got, want = got.astype(np.float64), want.astype(np.float64)
    tame = np.isfinite(want) & (np.abs(want) < 1e30)
    assert (np.isnan(got) == np.isnan(want))[np.abs(np.nan_to_num(want)) < 1e30].mean() >= 0.99
    # float chains: 1e-4 of max(|want|, 1) (the bar for a single op is 1e-5; three nested ops and a
    # reduction amplify it), for all but a sliver of elements (discontinuities: floor, casts, where)
    tol = (2e-3 if kernel.dtype == F16 else 1e-4) * np.maximum(np.abs(want), 1.0)
    if kernel.reduction is not None:
        tol = tol * np.sqrt(kernel.reduction.size)
    bad = tame & np.isfinite(got) & (np.abs(got - want) > tol)
    assert bad.mean() <= 0.01, (bad.mean(), np.abs(got - want)[bad].max())


def _random_dot(seed):
    from jax_js_b200 import programs as P
    rng = np.random.default_rng(5000 + seed)
    pick = lambda seq: seq[int(rng.integers(len(seq)))]
    M = pick([1, 3, 10, 64, 65, 100, 128, 260, 784, 1000, 2048, 8192])
    N = pick([1, 4, 10, 16, 64, 100, 128, 192, 512, 1028, 2048])
    K = pick([1, 7, 10, 16, 33, 64, 256, 300, 784, 4096])
    dtype = pick([F32, F32, F16])
    kw = dict(a_layout=pick(["mk", "km"]), b_layout=pick(["kn", "nk"]), bias=bool(rng.integers(2)), relu=bool(rng.integers(2)))
    if rng.random() < 0.2:
        kw["batch"] = int(pick([2, 5]))
    if rng.random() < 0.15:
        kw["swap"] = True
    return P.dot_kernel(M, N, K, dtype, **kw), (M, N, K, dtype, kw)


@pytest.mark.parametrize("seed", range(40))
def test_random_dot_shapes_plan_and_compile(seed):
    """Every dot skeleton (tensor-core f16 / 3xTF32 with any tile width and operand majorness, FFMA,
    the three skinny ones, plain reductions) over ragged and degenerate shapes: the generated source
    must compile for sm_100a whatever the route."""
    kernel, what = _random_dot(seed)
    describe, source = check_kernel(kernel, compile=True)
    assert describe.split()[0] in ("gemm-tcgen05", "gemm-ffma", "dot-skinny", "dot-skinny-t", "dot-small-k", "reduce-row", "elementwise",
                                   "reduce-col"), (what, describe)
    assert 'extern "C" __global__' in source
