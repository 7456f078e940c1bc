"""tests/golden/reference_vectors.json (known answers copied from the reference's own tests) replayed
through the CPU oracle and, on a GPU, through the cuda backend: the same vectors pin both."""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from jax_js_b200 import AluExp, DType, Kernel
from jax_js_b200 import programs as P
from jax_js_b200.routine import Routine, Routines, RoutineType

VECTORS = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
DT = {"float32": DType.Float32, "int32": DType.Int32, "uint32": DType.Uint32}
F32, I32 = DType.Float32, DType.Int32


def _arr(v, dtype=np.float32):
    """JSON data -> array; the strings "nan" / "inf" stand for the values JSON cannot spell."""
    def conv(x):
        if isinstance(x, list):
            return [conv(y) for y in x]
        return {"nan": np.nan, "inf": np.inf}.get(x, x) if isinstance(x, str) else x
    return np.array(conv(v), dtype=dtype)


class OracleRunner:
    """Everything through oracle/ (CPU)."""

    def kernel(self, k, args):
        return oracle.run_kernel(k, args)

    def program(self, prog, arrays):
        from oracle_backend import OracleBackend
        be = OracleBackend()
        outs = prog.execute(be, [be.put(a) for a in arrays])
        return [be.slots[s][0] for s in outs]

    def sort(self, x, dt):
        return oracle.sort(x, dt)

    def argsort(self, x, dt):
        return oracle.argsort(x, dt)[1]

    def scatter(self, upd, idx, params):
        return oracle.scatter(upd, [idx], params, F32)

    def lu(self, a):
        return oracle.lu(a)

    def cholesky(self, x):
        return oracle.cholesky(x)

    def jacobi(self, x, params):
        return oracle.jacobi_eigh(x, params["maxSweeps"], params["tolerance"])

    def fft(self, re, im, params):
        return oracle.fft(re, im, params["factors"], params["inverse"])


class CudaRunner:
    """Everything through the C ABI on the GPU."""

    def __init__(self, backend):
        self.be = backend

    def kernel(self, k, args):
        from util import run_cuda
        return run_cuda(self.be, k, args)

    def program(self, prog, arrays):
        slots = [self.be.put(a) for a in arrays]
        outs = prog.execute(self.be, slots)
        res = [self.be.read_sync(o) for o in outs]
        for s in slots + list(outs):
            self.be.dec_ref(s)
        return res

    def _routine(self, name, ins, out_shapes, out_dtypes, params=None):
        np_of = {DType.Float32: np.float32, DType.Int32: np.int32, DType.Uint32: np.uint32}
        code = {np.dtype(np.float32): DType.Float32, np.dtype(np.int32): DType.Int32, np.dtype(np.uint32): DType.Uint32}
        t = RoutineType([list(a.shape) for a in ins], [code[a.dtype] for a in ins], [list(s) for s in out_shapes], out_dtypes)
        exe = self.be.prepare_routine(Routine(name, t, params))
        in_slots = [self.be.put(a) for a in ins]
        outs = [self.be.put(np.full(s, 7, np_of[d])) for s, d in zip(out_shapes, out_dtypes)]
        self.be.dispatch(exe, in_slots, outs)
        res = [self.be.read_sync(o).view(np_of[d]).reshape(s) for o, s, d in zip(outs, out_shapes, out_dtypes)]
        for s in in_slots + outs:
            self.be.dec_ref(s)
        return res

    def sort(self, x, dt):
        return self._routine(Routines.Sort, [x], [x.shape], [dt])[0]

    def argsort(self, x, dt):
        return self._routine(Routines.Argsort, [x], [x.shape, x.shape], [dt, I32])[1]

    def scatter(self, upd, idx, params):
        return self._routine(Routines.Scatter, [upd, idx], [params["shape"]], [F32], params)[0]

    def lu(self, a):
        m, n = a.shape
        return self._routine(Routines.LU, [a], [a.shape, (min(m, n),), (m,)], [F32, I32, I32])

    def cholesky(self, x):
        return self._routine(Routines.Cholesky, [x], [x.shape], [F32])[0]

    def jacobi(self, x, params):
        return self._routine(Routines.JacobiEigh, [x], [x.shape, x.shape], [F32, F32], params)

    def fft(self, re, im, params):
        return self._routine(Routines.Fft, [re, im], [re.shape, im.shape], [F32, F32], params)


def _threefry_kernel(key, counter, mode):
    u = AluExp.u32
    return Kernel(0, 1, AluExp.threefry2x32(u(key[0]), u(key[1]), u(counter[0]), u(counter[1]), mode))


def check(run, v):
    kind = v["kind"]
    if kind == "sort":
        x, want = _arr(v["x"], v["dtype"]), _arr(v["want"], v["dtype"])
        got = run.sort(x, DT[v["dtype"]])
        assert np.array_equal(got, want, equal_nan=True), v["cite"]
    elif kind == "argsort":
        assert run.argsort(_arr(v["x"], v["dtype"]), DT[v["dtype"]]).tolist() == v["want"], v["cite"]
    elif kind == "threefry":
        got = [int(run.kernel(_threefry_kernel(v["key"], v["counter"], m), [])[0]) for m in (0, 1)]
        assert got == v["want"], v["cite"]
    elif kind == "random_bits":
        assert int(run.kernel(_threefry_kernel(v["key"], v["counter"], "xor"), [])[0]) == v["want"], v["cite"]
    elif kind in ("softmax", "logsumexp", "argmax"):
        x = _arr(v["x"])
        rows, cols = x.shape
        sm, lse, am = run.program(P.softmax_lse_argmax_program(rows, cols), [x, P.argmax_iota(cols)])
        if kind == "softmax":
            np.testing.assert_allclose(sm.view(np.float32).reshape(rows, cols), v["want"], rtol=v["rtol"], err_msg=v["cite"])
        elif kind == "logsumexp":
            np.testing.assert_allclose(lse.view(np.float32), v["want"], rtol=0, atol=v["atol"], err_msg=v["cite"])
        else:
            assert am.view(np.int32).tolist() == v["want"], v["cite"]
    elif kind == "matmul":
        a, b = _arr(v["a"]), _arr(v["b"])
        got = run.kernel(P.dot_kernel(a.shape[0], b.shape[1], a.shape[1]), [a, b]).reshape(a.shape[0], b.shape[1])
        assert got.tolist() == v["want"], v["cite"]
    elif kind == "mlp_predict":
        from jax_js_b200 import mlp
        from jax_js_b200.jaxpr import jit_compile
        x = _arr(v["x"])
        prog = jit_compile(mlp.mlp_predict_jaxpr(x.shape[0], v["dims"]))
        (logp,) = run.program(prog, [x] + [_arr(p) for p in v["params"]])
        assert logp.view(np.float32).reshape(x.shape[0], -1).tolist() == v["want"], v["cite"]   # toEqual: exact
    elif kind == "lu":
        lu, piv, perm = run.lu(_arr(v["a"]))
        np.testing.assert_allclose(lu, v["lu"], rtol=v["rtol"], err_msg=v["cite"])
        assert piv.tolist() == v["pivots"] and perm.tolist() == v["permutation"], v["cite"]
    elif kind == "cholesky_reconstructs":
        x = _arr(v["x"])
        L = run.cholesky(x)
        assert (np.triu(L, 1) == 0).all() and L[1, 0] != 0, v["cite"]
        np.testing.assert_allclose(L @ L.T, x, rtol=v["rtol"], err_msg=v["cite"])
    elif kind == "jacobi_eigh":
        x = _arr(v["x"])
        a, vec = run.jacobi(x, {"maxSweeps": max(8, 2 * x.shape[0]), "tolerance": 1e-6})
        assert np.diag(a).tolist() == v["values"] and vec.tolist() == v["vectors"], v["cite"]
    elif kind == "fft":
        n = len(v["real"])
        factors = [4] if n == 4 else None      # factorFftSize(4), src/library/numpy-fft.ts:50-66
        r, i = run.fft(_arr(v["real"]), _arr(v["imag"]), {"factors": factors, "inverse": v["inverse"]})
        np.testing.assert_allclose(r, v["want_real"], rtol=0, atol=v["atol"], err_msg=v["cite"])
        np.testing.assert_allclose(i, v["want_imag"], rtol=0, atol=v["atol"], err_msg=v["cite"])
    elif kind == "scatter":
        params = {"op": v["op"], "shape": v["shape"], "axis": [0], "outDim": 0, "uniqueIndices": True}
        got = run.scatter(_arr(v["updates"]), _arr(v["indices"], np.int32), params)
        assert got.tolist() == v["want"], v["cite"]
    else:
        raise AssertionError(f"unknown vector kind {kind}")


IDS = [f'{i:02d}-{v["kind"]}' for i, v in enumerate(VECTORS)]


@pytest.mark.parametrize("v", VECTORS, ids=IDS)
def test_oracle_reproduces_reference_vector(v):
    check(OracleRunner(), v)


@pytest.mark.gpu
@pytest.mark.parametrize("v", VECTORS, ids=IDS)
def test_cuda_reproduces_reference_vector(backend, v):
    check(CudaRunner(backend), v)
