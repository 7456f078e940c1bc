"""Captured step lists: a training step replayed as one CUDA graph gives the bits of the same step
dispatched kernel by kernel, and calls that cannot be recorded are refused inside a capture."""
import numpy as np
import pytest

from jax_js_b200 import AluExp, AluVar, DType, Kernel, mlp

pytestmark = pytest.mark.gpu


def test_captured_training_step_equals_eager_steps(backend):
    dims, B = [784, 256, 256, 10], 512
    rng = np.random.default_rng(0)
    x, y = rng.uniform(0, 1, (B, 784)).astype(np.float32), rng.integers(0, 10, B).astype(np.int32)
    sx, sy = backend.put(x), backend.put(y)
    eager, graphed = mlp.MlpTrainer(backend, dims, B, B), mlp.MlpTrainer(backend, dims, B, B)
    losses = [[], []]
    for step in range(6):
        if step == 2:
            graphed.capture(sx, sy)            # two eager steps first, then replay
        for i, tr in enumerate((eager, graphed)):
            s = tr.step(sx, sy)
            losses[i].append(backend.get(s, "float32")[0])
            backend.dec_ref(s)
    launches = backend.launch_count()
    s = graphed.step(sx, sy)
    backend.dec_ref(s)
    assert backend.launch_count() - launches >= 40      # a replay still counts its kernels
    assert np.array_equal(np.array(losses[0]).view(np.uint32), np.array(losses[1]).view(np.uint32)), losses
    eager_s = eager.step(sx, sy)
    backend.dec_ref(eager_s)
    for a, b in zip(eager.params, graphed.params):
        assert np.array_equal(backend.read_sync(a), backend.read_sync(b))
    eager.close()
    graphed.close()
    backend.dec_ref(sx)
    backend.dec_ref(sy)
    # memory that belonged to the graph is usable again afterwards
    z = backend.malloc(1 << 20)
    backend.dec_ref(z)


def test_calls_that_cannot_be_recorded_are_refused(backend):
    n = 4096
    k = Kernel(1, n, AluExp.add(AluExp.global_index(DType.Float32, 0, n, AluVar.gidx), AluExp.f32(1)))
    a, b = backend.put(np.zeros(n, np.float32)), backend.malloc(n * 4)
    exe = backend.prepare_kernel(k)
    backend.dispatch(exe, [a], [b])
    backend.capture_begin()
    with pytest.raises(ValueError, match="inside a capture"):
        backend.read_sync(b)
    with pytest.raises(ValueError, match="inside a capture"):
        backend.malloc(16, np.zeros(16, np.uint8))
    backend.dispatch(exe, [a], [b])
    backend.dispatch(exe, [b], [a])
    g = backend.capture_end()
    assert (backend.get(a, "float32") == 0).all()       # recording runs nothing
    for _ in range(3):
        backend.graph_launch(g)
    assert (backend.get(a, "float32") == 6).all()
    backend.graph_destroy(g)
    backend.dec_ref(a)
    backend.dec_ref(b)
