"""Seeded random step lists: what a capture makes of a list (row programs, producers substituted into
consumers, batches of small Kernels, or nothing) must replay the bits of the same list dispatched
Kernel by Kernel, whatever the wiring: arrays read by several Kernels, arrays released in the middle
(their blocks come back under another name), transposing and broadcasting reads, reductions."""
import numpy as np
import pytest

from jax_js_b200 import AluExp, AluOp, AluVar, DType, Kernel, Reduction

pytestmark = pytest.mark.gpu
F32 = DType.Float32
g, r, i32 = AluVar.gidx, AluVar.ridx, AluExp.i32


def _make_list(rng, rows, cols, n_kernels):
    """Kernels over arrays of shape [rows, cols] ("m"), [rows] ("r") and [cols] ("c").  Returns the
    steps: (kernel, input names, output name, output kind) and the names of the inputs."""
    n = rows * cols
    live = {"x0": "m", "x1": "m", "v0": "r", "w0": "c"}
    steps = []

    def load(arg, kind, out_kind, transposed=False):
        if out_kind == "m":
            row, col = AluExp.idiv(g, i32(cols)), AluExp.mod(g, i32(cols))
            if kind == "m":
                if transposed and rows == cols:
                    return AluExp.global_index(F32, arg, n, AluExp.add(AluExp.mul(col, i32(cols)), row))
                if transposed:
                    return AluExp.global_index(F32, arg, n, AluExp.add(AluExp.mul(g, i32(-1)), i32(n - 1)))   # reversed
                return AluExp.global_index(F32, arg, n, g)
            return AluExp.global_index(F32, arg, rows if kind == "r" else cols, row if kind == "r" else col)
        if out_kind == "r":      # per-row Kernel: reads row vectors (a matrix only under a reduction)
            return AluExp.global_index(F32, arg, rows, g)
        return AluExp.global_index(F32, arg, cols, g)

    for s in range(n_kernels):
        names = sorted(live)
        choice = rng.random()
        out = f"t{s}"
        mats = [nm for nm in names if live[nm] == "m"]
        if choice < 0.2 and mats:                      # row reduction of a matrix (sum or max), optional scale epilogue
            a = mats[int(rng.integers(len(mats)))]
            op = AluOp.Add if rng.random() < 0.5 else AluOp.Max
            body = AluExp.global_index(F32, 0, n, AluExp.add(AluExp.mul(g, i32(cols)), r))
            if rng.random() < 0.5:
                body = AluExp.mul(body, AluExp.f32(0.5))
            steps.append((Kernel(1, rows, body, Reduction(F32, op, cols)), [a], out, "r"))
            live[out] = "r"
        else:
            out_kind = "m" if choice < 0.75 else ("r" if choice < 0.9 else "c")
            cands = [nm for nm in names if live[nm] == out_kind or (out_kind == "m")]
            k_in = int(rng.integers(1, 4))
            ins = [cands[int(rng.integers(len(cands)))] for _ in range(k_in)]
            ins = list(dict.fromkeys(ins))
            terms = [load(j, live[nm], out_kind, transposed=rng.random() < 0.25) for j, nm in enumerate(ins)]
            e = terms[0]
            for t in terms[1:]:
                pick = rng.random()
                e = AluExp.add(e, t) if pick < 0.4 else AluExp.mul(e, t) if pick < 0.7 else AluExp.max(e, t)
            pick = rng.random()
            if pick < 0.2:
                e = AluExp.exp(AluExp.min(e, AluExp.f32(3.0)))
            elif pick < 0.4:
                e = AluExp.where(AluExp.cmplt(e, AluExp.f32(0.0)), AluExp.f32(0.0), e)
            elif pick < 0.6:
                e = AluExp.mul(e, AluExp.f32(0.75))
            size = {"m": n, "r": rows, "c": cols}[out_kind]
            steps.append((Kernel(len(ins), size, e), ins, out, out_kind))
            live[out] = out_kind
    return steps, ["x0", "x1", "v0", "w0"]


@pytest.mark.parametrize("seed,rows,cols", [(1, 16, 16), (2, 64, 10), (3, 32, 128), (4, 300, 8), (5, 1024, 512), (6, 48, 48),
                                            (7, 2048, 64), (8, 40, 12), (9, 32, 128), (10, 128, 256), (11, 8, 1024), (12, 256, 256),
                                            (13, 500, 20), (14, 64, 64), (15, 16, 4096), (16, 1000, 100), (17, 96, 36), (18, 32, 128),
                                            (19, 4096, 16), (20, 24, 24)])
def test_random_step_lists_replay_the_bits_of_their_kernels(backend, seed, rows, cols):
    rng = np.random.default_rng(seed)
    steps, inputs = _make_list(rng, rows, cols, 14)
    last_use = {}
    for idx, (_, ins, out, _) in enumerate(steps):
        for nm in ins:
            last_use[nm] = idx
    keep = {out for _, _, out, _ in steps if rng.random() < 0.35} | {steps[-1][2]}
    sizes = {"m": rows * cols, "r": rows, "c": cols}
    data = {"x0": rng.standard_normal(rows * cols), "x1": rng.uniform(-1, 1, rows * cols), "v0": rng.standard_normal(rows),
            "w0": rng.uniform(0.5, 1.5, cols)}
    exes = [backend.prepare_kernel(k) for k, _, _, _ in steps]

    def run(slots):
        """Dispatches the list; releases every intermediate after its last reader unless it is kept."""
        env = dict(slots)
        for idx, ((k, ins, out, kind), exe) in enumerate(zip(steps, exes)):
            env[out] = backend.malloc(sizes[kind] * 4)
            backend.dispatch(exe, [env[nm] for nm in ins], [env[out]])
            for nm in list(env):
                if nm not in slots and nm not in keep and last_use.get(nm, -1) <= idx and nm != out:
                    backend.dec_ref(env.pop(nm))
            if out not in keep and out not in last_use:
                backend.dec_ref(env.pop(out))
        return {nm: s for nm, s in env.items() if nm not in slots}

    slots = {nm: backend.put(data[nm].astype(np.float32)) for nm in inputs}
    eager = run(slots)
    want = {nm: backend.read_sync(s).copy() for nm, s in eager.items()}
    for s in eager.values():
        backend.dec_ref(s)
    backend.capture_begin()
    outs = run(slots)
    graph = backend.capture_end()
    for _ in range(2):
        backend.graph_launch(graph)
    launches, _, groups = backend.graph_cost(graph)
    assert set(outs) == set(want)
    # a row program adds a row up in another order than the row-reduce kernel: lists with a sum are
    # compared within float32 rounding of the values involved, all others bit for bit
    has_sum = any(k.reduction is not None and k.reduction.op == AluOp.Add for k, _, _, _ in steps)
    for nm, s in outs.items():
        got = backend.read_sync(s)
        if not has_sum:
            assert np.array_equal(got, want[nm]), (nm, launches, groups)
        else:
            a, b = got.view(np.float32).astype(np.float64), want[nm].view(np.float32).astype(np.float64)
            fin = np.isfinite(b)
            assert np.array_equal(np.isfinite(a), fin), nm
            assert np.all(np.abs(a[fin] - b[fin]) <= 1e-4 * (np.abs(b[fin]) + np.abs(b[fin]).mean() + 1e-6)), (nm, launches, groups)
    backend.graph_destroy(graph)
    for s in list(outs.values()) + list(slots.values()):
        backend.dec_ref(s)


def _make_dot_list(rng, M, N, K, n_kernels):
    """Lists around Dot Kernels: operands [M, K] ("a") and [K, N] ("b"), results and other matrices
    [M, N] ("c").  Dots reuse operands (the remainder planes of a captured list are shared), their
    results feed elementwise Kernels once (epilogue fusion) or several times, arrays are rescaled in
    between (a plane must not outlive the values it was made from)."""
    from jax_js_b200 import programs as P
    live = {"a0": "a", "b0": "b", "c0": "c"}
    steps = []
    mn = M * N

    def ew(kind_size, ins, e):
        return Kernel(len(ins), kind_size, e)

    for s in range(n_kernels):
        out = f"t{s}"
        names = sorted(live)
        pick = rng.random()
        a_s = [nm for nm in names if live[nm] == "a"]
        b_s = [nm for nm in names if live[nm] == "b"]
        c_s = [nm for nm in names if live[nm] == "c"]
        if pick < 0.35:
            a, b = a_s[int(rng.integers(len(a_s)))], b_s[int(rng.integers(len(b_s)))]
            steps.append((P.dot_kernel(M, N, K), [a, b], out, "c"))
            live[out] = "c"
        elif pick < 0.5:       # a new operand made from an old one
            kind = "a" if rng.random() < 0.5 else "b"
            src = (a_s if kind == "a" else b_s)
            src = src[int(rng.integers(len(src)))]
            size = M * K if kind == "a" else K * N
            e = AluExp.mul(AluExp.global_index(F32, 0, size, g), AluExp.f32(float(rng.choice([0.5, -1.25, 2.0]))))
            steps.append((ew(size, [src], e), [src], out, kind))
            live[out] = kind
        else:                  # elementwise over [M, N]: gate, sum or product of one or two matrices
            k_in = 1 if rng.random() < 0.4 else 2
            ins = list(dict.fromkeys(c_s[int(rng.integers(len(c_s)))] for _ in range(k_in)))
            terms = [AluExp.global_index(F32, j, mn, g) for j in range(len(ins))]
            if len(terms) == 2:
                e = AluExp.where(AluExp.cmplt(terms[1], AluExp.f32(0.0)), AluExp.f32(0.0), terms[0]) if rng.random() < 0.5 \
                    else AluExp.add(terms[0], terms[1])
            else:
                e = AluExp.max(terms[0], AluExp.f32(0.0)) if rng.random() < 0.5 else AluExp.mul(terms[0], AluExp.f32(0.125))
            steps.append((ew(mn, ins, e), ins, out, "c"))
            live[out] = "c"
    return steps, ["a0", "b0", "c0"]


@pytest.mark.parametrize("seed,M,N,K", [(1, 256, 256, 128), (2, 4096, 1024, 96), (3, 512, 384, 64), (4, 4096, 1024, 160),
                                        (5, 1024, 512, 4096), (6, 2048, 2048, 64)])
def test_random_lists_around_dots_replay_the_bits_of_their_kernels(backend, seed, M, N, K):
    rng = np.random.default_rng(100 + seed)
    steps, inputs = _make_dot_list(rng, M, N, K, 12)
    last_use = {}
    for idx, (_, ins, out, _) in enumerate(steps):
        for nm in ins:
            last_use[nm] = idx
    keep = {out for _, _, out, _ in steps if rng.random() < 0.3} | {steps[-1][2]}
    sizes = {"a": M * K, "b": K * N, "c": M * N}
    data = {"a0": rng.standard_normal(M * K), "b0": rng.uniform(-1, 1, K * N), "c0": rng.standard_normal(M * N)}
    exes = [backend.prepare_kernel(k) for k, _, _, _ in steps]

    def run(slots):
        env = dict(slots)
        for idx, ((k, ins, out, kind), exe) in enumerate(zip(steps, exes)):
            env[out] = backend.malloc(sizes[kind] * 4)
            backend.dispatch(exe, [env[nm] for nm in ins], [env[out]])
            for nm in list(env):
                if nm not in slots and nm not in keep and last_use.get(nm, -1) <= idx and nm != out:
                    backend.dec_ref(env.pop(nm))
            if out not in keep and out not in last_use:
                backend.dec_ref(env.pop(out))
        return {nm: s for nm, s in env.items() if nm not in slots}

    slots = {nm: backend.put(data[nm].astype(np.float32)) for nm in inputs}
    eager = run(slots)
    want = {nm: backend.read_sync(s).copy() for nm, s in eager.items()}
    for s in eager.values():
        backend.dec_ref(s)
    backend.capture_begin()
    outs = run(slots)
    graph = backend.capture_end()
    for _ in range(2):
        backend.graph_launch(graph)
    assert set(outs) == set(want)
    for nm, s in outs.items():
        assert np.array_equal(backend.read_sync(s), want[nm]), (nm, backend.graph_cost(graph))
    backend.graph_destroy(graph)
    for s in list(outs.values()) + list(slots.values()):
        backend.dec_ref(s)
