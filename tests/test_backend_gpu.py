"""The reference's backend contract tests (src/backend/backend.test.ts), run against the cuda
backend through the C ABI.  Expected arrays are the ones that file asserts."""
import numpy as np
import pytest

from jax_js_b200 import (AluExp, AluOp, AluVar, DType, Kernel, Reduction, ShapeTracker, accessor_global,
                         global_view, unravel_alu)
from jax_js_b200.backend import SlotError, UnsupportedRoutineError
from jax_js_b200.routine import Routine, Routines, RoutineType

pytestmark = pytest.mark.gpu
F32, U32 = DType.Float32, DType.Uint32
g, r = AluVar.gidx, AluVar.ridx


def f32(*v):
    return np.array(v, dtype=np.float32)


def test_can_run_simple_operations(backend):
    # backend.test.ts:37-85
    shape = ShapeTracker.from_shape([3])
    a, b, c = backend.put(f32(1, 2, 3)), backend.put(f32(4, 5, 6)), backend.malloc(12)
    try:
        arg1 = accessor_global(F32, 0, shape, [g])
        arg2 = accessor_global(F32, 1, shape.flip([True]), [g])
        backend.dispatch(backend.prepare_kernel(Kernel(2, 3, AluExp.mul(arg1, arg2))), [a, b], [c])
        assert backend.get(c, F32).tolist() == [6, 10, 12]
        backend.dispatch(backend.prepare_kernel(Kernel(2, 3, AluExp.add(arg1, arg2))), [a, b], [c])
        assert backend.get(c, F32).tolist() == [7, 7, 7]
    finally:
        for s in (a, b, c):
            backend.dec_ref(s)


def test_can_create_array_from_index(backend):
    # backend.test.ts:190-203
    a = backend.malloc(200 * 4)
    try:
        backend.dispatch(backend.prepare_kernel(Kernel(0, 200, AluExp.cast(F32, g))), [], [a])
        assert backend.get(a, F32).tolist() == list(range(200))
    finally:
        backend.dec_ref(a)


def test_reads_a_buffer_with_byte_ranges(backend):
    # backend.test.ts:219-246
    arr = f32(1, 1, 2, 3, 5, 7)
    a = backend.put(arr)
    try:
        assert backend.read_sync(a).view(np.float32).tolist() == arr.tolist()
        assert backend.read_sync(a, 3 * 4, 2 * 4).view(np.float32).tolist() == [3, 5]
        assert backend.read_sync(a, 0, 0).size == 0  # the barrier form, src/frontend/array.ts:827
    finally:
        backend.dec_ref(a)


def test_performs_reduction_with_fused_epilogue(backend):
    # backend.test.ts:248-286
    a, out = backend.put(f32(1, 1, 2, 3, 5, 7)), backend.malloc(12)
    try:
        exp = global_view(F32, 0, ShapeTracker.from_shape([3, 2]), [g, r])
        backend.dispatch(backend.prepare_kernel_sync(Kernel(1, 3, exp, Reduction(F32, AluOp.Add, 2))), [a], [out])
        assert backend.get(out, F32).tolist() == [2, 5, 12]
        red = Reduction(F32, AluOp.Add, 2, AluExp.add(AluVar.acc(F32), AluExp.f32(1)))
        backend.dispatch(backend.prepare_kernel_sync(Kernel(1, 3, exp, red)), [a], [out])
        assert backend.get(out, F32).tolist() == [3, 6, 13]
    finally:
        backend.dec_ref(a)
        backend.dec_ref(out)


def test_bitwise_operations(backend):
    # backend.test.ts:288-373
    shape = ShapeTracker.from_shape([4])
    a = backend.put(np.array([0xFF00FF00, 0x0F0F0F0F, 0xAAAAAAAA, 7], np.uint32))
    b = backend.put(np.array([0x00FF00FF, 0xF0F0F0F0, 0x55555555, 3], np.uint32))
    sa, sb = backend.put(np.ones(4, np.uint32)), backend.put(np.array([0, 1, 8, 16], np.uint32))
    ra = backend.put(np.array([256, 65536, 0xFFFF0000, 8], np.uint32))
    c = backend.malloc(16)
    x, y = accessor_global(U32, 0, shape, [g]), accessor_global(U32, 1, shape, [g])
    try:
        def run(e, ins):
            backend.dispatch(backend.prepare_kernel(Kernel(2, 4, e)), ins, [c])
            return backend.get(c, U32).tolist()
        assert run(AluExp.bit_combine(x, y, "and"), [a, b]) == [0, 0, 0, 3]
        assert run(AluExp.bit_combine(x, y, "or"), [a, b]) == [0xFFFFFFFF] * 3 + [7]
        assert run(AluExp.bit_combine(x, y, "xor"), [a, b]) == [0xFFFFFFFF] * 3 + [4]
        assert run(AluExp.bit_shift(x, y, "shl"), [sa, sb]) == [1, 2, 256, 65536]
        assert run(AluExp.bit_shift(x, y, "shr"), [ra, sb]) == [256, 32768, 0x00FFFF00, 0]
    finally:
        for s in (a, b, sa, sb, ra, c):
            backend.dec_ref(s)


def _matmul_kernel(M, N, K, gid_b, swapped=False):
    stA = ShapeTracker.from_shape([M, K]).reshape([M, 1, K]).expand([M, N, K])
    stB = ShapeTracker.from_shape([K, N]).permute([1, 0]).reshape([1, N, K]).expand([M, N, K])
    idx = [*unravel_alu([M, N], g), r]
    la, lb = global_view(F32, 0, stA, idx), global_view(F32, gid_b, stB, idx)
    return Kernel(gid_b + 1, M * N, AluExp.mul(lb, la) if swapped else AluExp.mul(la, lb), Reduction(F32, AluOp.Add, K))


def test_performs_64x64_matmul(backend):
    # backend.test.ts:375-409: the same slot feeds both operands
    n = 64
    a, b = backend.put(np.ones(n * n, np.float32)), backend.malloc(n * n * 4)
    try:
        backend.dispatch(backend.prepare_kernel(_matmul_kernel(n, n, n, 0)), [a], [b])
        np.testing.assert_allclose(backend.get(b, F32), n)
    finally:
        backend.dec_ref(a)
        backend.dec_ref(b)


def test_performs_non_square_matmul_both_operand_orders(backend):
    # backend.test.ts:411-464
    M, N, K = 16, 48, 24
    a, b, c = backend.put(np.ones(M * K, np.float32)), backend.put(np.ones(K * N, np.float32)), backend.malloc(M * N * 4)
    try:
        for swapped in (False, True):
            backend.dispatch(backend.prepare_kernel(_matmul_kernel(M, N, K, 1, swapped)), [a, b], [c])
            np.testing.assert_allclose(backend.get(c, F32), K)
    finally:
        for s in (a, b, c):
            backend.dec_ref(s)


def test_keeps_row_dependent_contiguous_reduction_loads_distinct(backend):
    # backend.test.ts:466-507
    M, N, K = 32, 128, 5
    x = np.fromfunction(lambda m, k, n: m * 1000 + k * 10 + n, (M, K, N)).astype(np.float32)
    a, out = backend.put(x), backend.malloc(M * N * 4)
    try:
        mm, nn = unravel_alu([M, N], g)
        exp = global_view(F32, 0, ShapeTracker.from_shape([M, K, N]), [mm, r, nn])
        backend.dispatch(backend.prepare_kernel(Kernel(1, M * N, exp, Reduction(F32, AluOp.Add, K))), [a], [out])
        want = K * (np.arange(M)[:, None] * 1000 + np.arange(N)[None, :]) + 10 * K * (K - 1) / 2
        np.testing.assert_allclose(backend.get(out, F32, (M, N)), want, rtol=1e-6)
    finally:
        backend.dec_ref(a)
        backend.dec_ref(out)


def test_slot_lifetime_errors(backend):
    # src/backend.ts:176-180: decRef of a freed slot throws SlotError; refcounts keep a slot alive
    s = backend.malloc(16)
    backend.inc_ref(s)
    backend.dec_ref(s)
    assert backend.read_sync(s).size == 16
    backend.dec_ref(s)
    with pytest.raises(SlotError):
        backend.dec_ref(s)
    with pytest.raises(SlotError):
        backend.read_sync(s)


def test_malloc_edge_cases(backend):
    # size 0 is legal (src/backend/webgpu.ts:84-86); initialData must match (src/backend/cpu.ts:21-24)
    z = backend.malloc(0)
    assert backend.read_sync(z).size == 0
    backend.dec_ref(z)
    with pytest.raises(ValueError):
        backend.malloc(8, np.zeros(3, np.uint8))


def test_unsupported_routine_raises(backend):
    # src/backend.ts:236-240
    rt = Routine("Conv", RoutineType([[2, 2]], [F32], [[2, 2]], [F32]))   # not a member of Routines
    with pytest.raises(UnsupportedRoutineError, match="routine 'Conv' is not supported in cuda backend"):
        backend.prepare_routine(rt)


def test_dispatch_order_is_execution_order(backend):
    # src/backend.ts:203-210: a chain of dependent kernels on one slot, read once at the end
    n = 1 << 16
    a, b = backend.put(np.zeros(n, np.float32)), backend.malloc(n * 4)
    inc = backend.prepare_kernel(Kernel(1, n, AluExp.add(AluExp.global_index(F32, 0, n, g), AluExp.f32(1))))
    try:
        for _ in range(25):
            backend.dispatch(inc, [a], [b])
            backend.dispatch(inc, [b], [a])
        assert (backend.get(a, F32) == 50).all()
    finally:
        backend.dec_ref(a)
        backend.dec_ref(b)


def test_async_read_and_write_are_ordered_with_dispatches(backend):
    # Backend.read returns a Promise (src/backend.ts:182-186): read_async enqueues, read_wait resolves.
    # Two steps in flight over two input slots, as a caller awaiting the previous step would run them.
    n = 1 << 20
    inc = backend.prepare_kernel(Kernel(1, n, AluExp.add(AluExp.global_index(F32, 0, n, g), AluExp.f32(1))))
    host_in = [backend.host_alloc(n * 4) for _ in range(2)]
    host_out = [backend.host_alloc(n * 4) for _ in range(2)]
    ins, pending, results = [backend.malloc(n * 4) for _ in range(2)], None, []
    for step in range(6):
        k = step % 2
        if pending is not None and pending[0] == k:      # this pair of buffers is still in flight
            backend.read_wait(pending[2]); results.append(host_out[k].view(np.float32).copy()); backend.dec_ref(pending[1]); pending = None
        host_in[k].view(np.float32)[:] = step * 10
        backend.write_async(ins[k], host_in[k])
        out = backend.malloc(n * 4)
        backend.dispatch(inc, [ins[k]], [out])
        ticket = backend.read_async(out, host_out[k])
        if pending is not None:
            backend.read_wait(pending[2]); results.append(host_out[pending[0]].view(np.float32).copy()); backend.dec_ref(pending[1])
        pending = (k, out, ticket)
        backend.sync()                                    # the upload has been consumed: host_in[k] may change
    backend.read_wait(pending[2]); results.append(host_out[pending[0]].view(np.float32).copy()); backend.dec_ref(pending[1])
    assert [float(r[0]) for r in results] == [1, 11, 21, 31, 41, 51] and all((r == r[0]).all() for r in results)
    with pytest.raises(ValueError):
        backend.read_wait(pending[2])                     # a ticket resolves once
    # partial ranges and a read ordered after a later write into the same slot
    backend.write(ins[0], np.arange(n, dtype=np.float32))
    t = backend.read_async(ins[0], host_out[0][:64], start=128)
    backend.write_async(ins[0], host_in[1])               # must not overtake the read above
    backend.read_wait(t)
    assert host_out[0][:64].view(np.float32).tolist() == list(range(32, 48))
    for s in ins:
        backend.dec_ref(s)
    for h in host_in + host_out:
        backend.host_free(h)


def test_empty_and_largest_kernels(backend):
    # size 0: nothing to do, nothing launched out of bounds
    empty = Kernel(1, 0, AluExp.add(AluExp.global_index(F32, 0, 0, g), AluExp.f32(1)))
    a, b = backend.malloc(0), backend.malloc(0)
    backend.dispatch(backend.prepare_kernel(empty), [a], [b])
    assert backend.read_sync(b).size == 0
    backend.dec_ref(a)
    backend.dec_ref(b)
    # the largest index space the int32 gidx of the reference allows (src/alu.ts:1479): 2^31 - 8 outputs, 8.6 GB.
    # out[g] = g * 3 (wrapping), then a wrapping uint32 row sum over [32768 - 1, 65536] checked in closed form.
    n_cols = 1 << 16
    n_rows = (1 << 15) - 1
    n = n_rows * n_cols
    big = backend.malloc(n * 4)
    fill = Kernel(0, n, AluExp.mul(AluExp.cast(U32, g), AluExp.u32(3)))
    backend.dispatch(backend.prepare_kernel(fill), [], [big])
    r = AluVar.ridx
    rows = Kernel(1, n_rows, AluExp.global_index(U32, 0, n, AluExp.add(AluExp.mul(g, AluExp.i32(n_cols)), r)),
                  Reduction(U32, AluOp.Add, n_cols))
    sums = backend.malloc(n_rows * 4)
    backend.dispatch(backend.prepare_kernel(rows), [big], [sums])
    got = backend.get(sums, U32)
    i = np.arange(n_rows, dtype=np.uint64)
    want = (3 * (i * n_cols * n_cols + n_cols * (n_cols - 1) // 2)) % (1 << 32)
    assert np.array_equal(got.astype(np.uint64), want)
    tail = backend.read_sync(big, (n - 4) * 4, 16).view(np.uint32)
    assert tail.tolist() == [((n - 4 + j) * 3) % (1 << 32) for j in range(4)]
    backend.dec_ref(big)
    backend.dec_ref(sums)


def test_block_reuse_is_ordered_behind_a_pending_async_read(backend):
    """A slot released right after `read_async` hands its block back to the allocator; the next owner
    of the block must not overwrite it before the download has finished."""
    n = 8 << 20                                   # 32 MB: the copy takes a while on PCIe
    src = np.arange(n, dtype=np.float32)
    a = backend.put(src)
    host = backend.host_alloc(n * 4)
    before = backend.order_waits()
    t = backend.read_async(a, host)
    backend.dec_ref(a)                            # released while the copy is in flight
    assert backend.order_waits() == before + 1    # the compute stream now waits for that copy
    b = backend.put(np.full(n, -1.0, np.float32)) # same size class: gets the block that was just released
    backend.read_wait(t)
    assert np.array_equal(host.view(np.float32), src)
    backend.dec_ref(b)
    backend.host_free(host)


def test_async_read_can_be_waited_for_on_another_thread(backend):
    """The Promise pattern of a Node-API addon: a worker thread blocks on the ticket's event alone, the
    driving thread keeps dispatching and retires the ticket afterwards."""
    import threading
    n = 1 << 20
    x = np.arange(n, dtype=np.float32)
    k = Kernel(1, n, AluExp.add(AluExp.global_index(F32, 0, n, g), AluExp.f32(1)))
    exe = backend.prepare_kernel(k)
    a, b = backend.put(x), backend.malloc(n * 4)
    backend.dispatch(exe, [a], [b])
    host = backend.host_alloc(n * 4)
    t = backend.read_async(b, host)
    ev = backend.read_event(t)
    th = threading.Thread(target=backend.event_block, args=(ev,))
    th.start()
    for _ in range(20):                           # the driving thread goes on using the context meanwhile
        backend.dispatch(exe, [a], [b])
        t2 = backend.read_async(b, backend_scratch(backend, n * 4))
        backend.read_wait(t2)
    th.join()
    backend.read_wait(t)
    assert np.array_equal(host.view(np.float32), x + 1)
    for s in (a, b):
        backend.dec_ref(s)
    backend.host_free(host)
    backend.host_free(_SCRATCH.pop("buf"))


_SCRATCH = {}


def backend_scratch(backend, nbytes):
    if "buf" not in _SCRATCH:
        _SCRATCH["buf"] = backend.host_alloc(nbytes)
    return _SCRATCH["buf"]


def test_trace_times_every_eager_dispatch(backend):
    """startTrace / stopTrace (src/tracing.ts:15-33): between them every dispatch leaves a record with
    its plan, its start and its duration on the device; records come in dispatch order, do not
    overlap on the one stream, and a larger Kernel takes longer.  Dispatches inside a capture and
    after stop_trace leave none."""
    from jax_js_b200 import AluExp, AluVar, DType, Kernel
    F32 = DType.Float32

    def inc(n):
        return backend.prepare_kernel(Kernel(1, n, AluExp.add(AluExp.global_index(F32, 0, n, AluVar.gidx), AluExp.f32(1))))

    small, large = inc(1 << 12), inc(1 << 26)
    a, b = backend.put(np.zeros(1 << 26, np.float32)), backend.malloc(4 << 26)
    backend.dispatch(large, [a], [b])             # not traced
    backend.start_trace()
    for exe in (small, large, small, large):
        backend.dispatch(exe, [a], [b])
    backend.capture_begin()
    backend.dispatch(small, [a], [b])
    graph = backend.capture_end()
    backend.graph_launch(graph)
    records = backend.stop_trace()
    backend.dispatch(small, [a], [b])             # not traced
    assert [r["exe"] for r in records] == [small.data, large.data, small.data, large.data]
    assert all(r["name"].startswith("elementwise") for r in records)
    assert all(r["start_ms"] >= 0 and r["duration_ms"] > 0 for r in records)
    for before, after in zip(records, records[1:]):
        assert after["start_ms"] >= before["start_ms"] + before["duration_ms"] - 1e-3
    assert records[1]["duration_ms"] > 4 * records[0]["duration_ms"]
    assert 0.05 < records[1]["duration_ms"] < 5.0           # 512 MB through HBM
    backend.start_trace()
    assert backend.stop_trace() == []
    backend.graph_destroy(graph)
    for s in (a, b):
        backend.dec_ref(s)
