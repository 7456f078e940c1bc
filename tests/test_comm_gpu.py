"""The gradient sum of the data-parallel path on a communicator of one rank: the real NCCL calls,
on the context stream and on the second stream, eagerly and inside a captured step list.  (Sums over
several ranks are covered on CPU by the two-process gloo test and measured by the benchmark.)"""
import numpy as np
import pytest

from jax_js_b200 import DType
from jax_js_b200.alu import AluExp, AluVar, Kernel
from jax_js_b200.backend import CudaBackend

pytestmark = pytest.mark.gpu
F32 = DType.Float32
g = AluVar.gidx


@pytest.fixture()
def solo():
    be = CudaBackend(0)
    try:
        be.comm_init(0, 1, CudaBackend.comm_unique_id())
    except Exception as e:  # no NCCL library on this machine
        be.close()
        pytest.skip(f"NCCL unavailable: {e}")
    yield be
    be.close()


def _inc(be, n):
    return be.prepare_kernel(Kernel(1, n, AluExp.add(AluExp.global_index(F32, 0, n, g), AluExp.f32(1))))


def test_sum_on_second_stream_is_ordered_with_dispatches(solo):
    n = 1 << 20
    inc = _inc(solo, n)
    a, b, c, d = solo.put(np.ones(n, np.float32)), solo.malloc(n * 4), solo.malloc(n * 4), solo.malloc(n * 4)
    solo.dispatch(inc, [a], [b])               # b = 2
    solo.allreduce_sum_f32_async([b])          # after the kernel above, under the kernel below
    solo.dispatch(inc, [a], [c])               # independent of the sum
    solo.comm_join()
    solo.dispatch(inc, [b], [d])               # after the sum: d = 3
    assert (solo.get(d, F32) == 3).all() and (solo.get(c, F32) == 2).all()
    solo.dispatch(inc, [d], [b])               # b = 4
    solo.allreduce_sum_f32_async([b])
    assert (solo.get(b, F32) == 4).all()       # a read joins by itself
    solo.allreduce_sum_f32_async([b, c])
    solo.allreduce_sum_f32([d])                # the plain sum keeps this rank's NCCL calls in order
    solo.sync()
    assert (solo.get(d, F32) == 3).all()
    for s in (a, b, c, d):
        solo.dec_ref(s)


def test_sum_inside_a_captured_step_list(solo):
    n = 1 << 16
    inc = _inc(solo, n)
    a, b = solo.put(np.zeros(n, np.float32)), solo.malloc(n * 4)
    solo.dispatch(inc, [a], [b])
    solo.sync()
    solo.capture_begin()
    solo.dispatch(inc, [a], [b])
    solo.allreduce_sum_f32_async([b])
    solo.comm_join()
    solo.dispatch(inc, [b], [a])               # a += 2 per replay
    graph = solo.capture_end()
    for _ in range(5):
        solo.graph_launch(graph)
    assert (solo.get(a, F32) == 10).all()
    solo.graph_destroy(graph)
    solo.dec_ref(a)
    solo.dec_ref(b)


def test_a_reader_waits_for_the_sum_of_its_operand_only(solo):
    """A Kernel that reads a slot whose sum is still running on the second stream makes the compute
    stream wait for exactly that sum (no join is needed for correctness); sums begun later stay in
    flight.  Eagerly and inside a captured step list."""
    n = 1 << 20
    inc = _inc(solo, n)
    a = solo.put(np.ones(n, np.float32))
    b, c, d, e = (solo.malloc(n * 4) for _ in range(4))

    def run():
        solo.dispatch(inc, [a], [b])               # b = a + 1
        solo.allreduce_sum_f32_async([b])
        solo.dispatch(inc, [a], [c])               # c = a + 1
        solo.allreduce_sum_f32_async([c])
        solo.dispatch(inc, [b], [d])               # reads b: waits for the first sum, not for the second
        solo.dispatch(inc, [c], [e])               # reads c: waits for the second
    w0 = solo.order_waits()
    run()
    assert solo.order_waits() - w0 == 2
    assert (solo.get(d, F32) == 3).all() and (solo.get(e, F32) == 3).all()
    solo.capture_begin()
    run()
    solo.dispatch(inc, [d], [a])                   # a <- a + 3 per replay
    graph = solo.capture_end()
    for _ in range(3):
        solo.graph_launch(graph)
    assert (solo.get(a, F32) == 10).all() and (solo.get(e, F32) == 9).all()
    solo.graph_destroy(graph)
    for s in (a, b, c, d, e):
        solo.dec_ref(s)
