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


def test_comm_wait_returns_when_the_sums_are_done_and_times_out_while_they_run(solo):
    """The watchdog wait on a healthy communicator: with a zero limit it reports work still running
    (and cancels nothing), with a generous one it returns once the queue has drained."""
    n = 1 << 26
    inc = _inc(solo, n)
    a, b = solo.put(np.zeros(n, np.float32)), solo.malloc(n * 4)
    solo.comm_wait(10000)
    for _ in range(50):                         # some milliseconds of queued work, the sum in the middle
        solo.dispatch(inc, [a], [b])
    solo.allreduce_sum_f32_async([b])
    for _ in range(50):
        solo.dispatch(inc, [a], [b])
    with pytest.raises(TimeoutError):
        solo.comm_wait(0)
    solo.comm_wait(10000)
    assert (solo.get(b, F32) == 1).all()
    solo.capture_begin()
    with pytest.raises(ValueError):
        solo.comm_wait(10)
    solo.graph_destroy(solo.capture_end())
    for s in (a, b):
        solo.dec_ref(s)


def test_an_error_reported_by_nccl_aborts_the_communicator(tmp_path):
    """Failure made on the host: a stand-in NCCL library whose asynchronous error state the test
    sets.  comm_wait reports it, the communicator is aborted, later sums are refused and the context
    still runs Kernels."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    lib = tmp_path / "libfakenccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(lib), os.path.join(here, "fake_nccl.c")], check=True)
    script = r"""
import os, sys
import numpy as np
sys.path.insert(0, os.environ["REPO_ROOT"])
from jax_js_b200 import DType
from jax_js_b200.alu import AluExp, AluVar, Kernel
from jax_js_b200.backend import CudaBackend, CudaError
be = CudaBackend(0)
be.comm_init(1, 2, CudaBackend.comm_unique_id())
n = 4096
inc = be.prepare_kernel(Kernel(1, n, AluExp.add(AluExp.global_index(DType.Float32, 0, n, AluVar.gidx), AluExp.f32(1))))
a, b = be.put(np.zeros(n, np.float32)), be.malloc(n * 4)
be.dispatch(inc, [a], [b])
be.allreduce_sum_f32_async([b])
be.comm_wait(5000)
print("healthy")
open(os.environ["FAKE_NCCL_FLAG"], "w").write("6")
try:
    be.comm_wait(5000)
    print("no error seen")
except CudaError as e:
    print("error:", e)
try:
    be.allreduce_sum_f32([b])
    print("sum accepted")
except ValueError as e:
    print("refused:", e)
be.dispatch(inc, [b], [a])
print("value", float(be.get(a, DType.Float32)[0]))
be.close()
"""
    env = dict(os.environ, JAXCUDA_NCCL_LIB=str(lib), FAKE_NCCL_FLAG=str(tmp_path / "flag"), FAKE_NCCL_ABORTED=str(tmp_path / "aborted"),
               REPO_ROOT=os.path.dirname(here))
    out = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.strip().splitlines()
    assert lines[0] == "healthy"
    assert lines[1].startswith("error:") and "remote process exited" in lines[1] and "aborted" in lines[1], lines
    assert lines[2].startswith("refused:") and "not initialised" in lines[2], lines
    assert lines[3] == "value 2.0", lines
    assert (tmp_path / "aborted").read_text() == "aborted"
