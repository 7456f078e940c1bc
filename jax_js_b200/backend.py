"""`CudaBackend`: the reference's `Backend` interface (src/backend.ts:158-211) over
libjaxcuda.so.

Method names, argument meaning and error behaviour follow the TypeScript interface
(malloc / incRef / decRef / read / readSync / prepareKernel[Sync] / prepareRoutine[Sync] /
dispatch), spelled in snake_case; `Executable`, `SlotError`, `UnsupportedOpError` and
`UnsupportedRoutineError` mirror src/backend.ts:213-240.  There is no CPU fallback: without
the shared library or without a B200 the constructor raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Sequence

import numpy as np

from .alu import DType, Kernel
from .routine import Routine

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libjaxcuda.so"
_lib = None

OK, ESLOT, EUNSUPPORTED, EINVAL, ECOMPILE, ECUDA, ENOMEM, ETIMEOUT = range(8)
SIZE_MAX = ctypes.c_size_t(-1).value


class SlotError(RuntimeError):
    """src/backend.ts:222-226."""


class UnsupportedOpError(RuntimeError):
    """src/backend.ts:228-234."""


class UnsupportedRoutineError(RuntimeError):
    """src/backend.ts:236-240."""


class CompileError(RuntimeError):
    """NVRTC rejected generated source; the message carries the log and the source."""


class CudaError(RuntimeError):
    pass


class _RoutineType(ctypes.Structure):
    _fields_ = [("n_inputs", ctypes.c_int), ("n_outputs", ctypes.c_int),
                ("input_dtypes", ctypes.POINTER(ctypes.c_int32)), ("input_ranks", ctypes.POINTER(ctypes.c_int32)),
                ("input_shapes", ctypes.POINTER(ctypes.c_int64)),
                ("output_dtypes", ctypes.POINTER(ctypes.c_int32)), ("output_ranks", ctypes.POINTER(ctypes.c_int32)),
                ("output_shapes", ctypes.POINTER(ctypes.c_int64))]


#: Every symbol include/jaxcuda.h declares, with its ctypes signature (restype, argtypes).
_P, _U32, _U64, _SZ, _I = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_int
SYMBOLS = {
    "jaxcuda_create": (_I, [_I, ctypes.POINTER(_P)]),
    "jaxcuda_destroy": (_I, [_P]),
    "jaxcuda_last_error": (ctypes.c_char_p, [_P]),
    "jaxcuda_max_args": (_I, []),
    "jaxcuda_check_step_list": (_I, None),
    "jaxcuda_malloc": (_I, [_P, _SZ, _P, _SZ, ctypes.POINTER(_U32)]),
    "jaxcuda_incref": (_I, [_P, _U32]),
    "jaxcuda_decref": (_I, [_P, _U32]),
    "jaxcuda_read": (_I, [_P, _U32, _SZ, _SZ, _P]),
    "jaxcuda_write": (_I, [_P, _U32, _SZ, _SZ, _P]),
    "jaxcuda_read_async": (_I, [_P, _U32, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64)]),
    "jaxcuda_read_wait": (_I, [_P, ctypes.c_uint64]),
    "jaxcuda_write_async": (_I, [_P, _U32, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p]),
    "jaxcuda_slot_size": (_I, [_P, _U32, ctypes.POINTER(_SZ)]),
    "jaxcuda_prepare_kernel": (_I, [_P, ctypes.c_char_p, _SZ, _U64, ctypes.POINTER(_P)]),
    "jaxcuda_check_kernel": (_I, [ctypes.c_char_p, _SZ, _I, _I, _I, ctypes.c_char_p, _SZ, ctypes.c_char_p, _SZ]),
    "jaxcuda_prepare_routine": (_I, [_P, ctypes.c_char_p, ctypes.POINTER(_RoutineType), ctypes.c_char_p, ctypes.POINTER(_P)]),
    "jaxcuda_dispatch": (_I, [_P, _P, ctypes.POINTER(_U32), _I, ctypes.POINTER(_U32), _I]),
    "jaxcuda_exe_release": (_I, [_P]),
    "jaxcuda_exe_describe": (ctypes.c_char_p, [_P]),
    "jaxcuda_exe_source": (ctypes.c_char_p, [_P]),
    "jaxcuda_exe_cost": (_I, [_P, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_I)]),
    "jaxcuda_host_alloc": (_I, [_P, _SZ, ctypes.POINTER(_P)]),
    "jaxcuda_host_free": (_I, [_P, _P]),
    "jaxcuda_sync": (_I, [_P]),
    "jaxcuda_event_record": (_I, [_P, _I]),
    "jaxcuda_event_elapsed_ms": (_I, [_P, _I, _I, ctypes.POINTER(ctypes.c_float)]),
    "jaxcuda_checked_counts": (_I, [_P, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    "jaxcuda_trace_start": (_I, [_P]),
    "jaxcuda_trace_stop": (_I, [_P, ctypes.POINTER(ctypes.c_int)]),
    "jaxcuda_trace_record": (_I, [_P, _I, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_double),
                                  ctypes.POINTER(ctypes.c_double), ctypes.c_char_p, ctypes.c_size_t]),
    "jaxcuda_launch_count": (_U64, [_P]),
    "jaxcuda_slot_ptr": (_I, [_P, _U32, ctypes.POINTER(_U64)]),
    "jaxcuda_stream": (_U64, [_P]),
    "jaxcuda_comm_unique_id": (_I, [_P]),
    "jaxcuda_comm_init": (_I, [_P, _I, _I, _P]),
    "jaxcuda_allreduce_sum_f32": (_I, [_P, ctypes.POINTER(_U32), _I]),
    "jaxcuda_allreduce_sum_f32_async": (_I, [_P, ctypes.POINTER(_U32), _I]),
    "jaxcuda_comm_join": (_I, [_P]),
    "jaxcuda_comm_destroy": (_I, [_P]),
    "jaxcuda_comm_wait": (_I, [_P, _I]),
    "jaxcuda_comm_abort": (_I, [_P]),
    "jaxcuda_capture_begin": (_I, [_P]),
    "jaxcuda_capture_end": (_I, [_P, ctypes.POINTER(_P)]),
    "jaxcuda_graph_launch": (_I, [_P, _P]),
    "jaxcuda_graph_destroy": (_I, [_P, _P]),
    "jaxcuda_read_event": (_I, [_P, ctypes.c_uint64, ctypes.POINTER(_P)]),
    "jaxcuda_event_block": (_I, [_P]),
    "jaxcuda_order_waits": (ctypes.c_uint64, [_P]),
    "jaxcuda_graph_cost": (_I, [_P, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int)]),
    "jaxcuda_copy": (_I, [_P, _U32, _U32]),
    "jaxcuda_sort_no_alloc": (_I, [_P, _I, _P, _P, ctypes.c_int64, ctypes.c_int64, ctypes.c_char_p, _SZ]),
}


def load_library():
    """dlopen libjaxcuda.so (built by `python -m jax_js_b200.build`) and bind its C ABI."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise CudaError(f"{_LIB_PATH} is missing: run `python -m jax_js_b200.build` "
                            "(the cuda backend has no CPU fallback)")
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def check_kernel(kernel: Kernel, *, sm_count: int = 148, force_skeleton: int = -1, compile: bool = True):
    """Plan (and NVRTC-compile) a kernel without a GPU.  Returns (describe, source)."""
    lib = load_library()
    image = kernel.serialize()
    desc = ctypes.create_string_buffer(512)
    msg = ctypes.create_string_buffer(1 << 20)
    rc = lib.jaxcuda_check_kernel(image, len(image), sm_count, force_skeleton, 0, desc, len(desc), msg, len(msg))
    source = msg.value.decode()
    if rc == OK and compile:
        rc = lib.jaxcuda_check_kernel(image, len(image), sm_count, force_skeleton, 1, desc, len(desc), msg, len(msg))
    if rc != OK:
        _raise(rc, msg.value.decode())
    return desc.value.decode(), source


def check_step_list(program, *, compile: bool = True):
    """What a capture of `program` (a `JitProgram`) would launch, without a GPU: returns (report
    lines, CUDA C of the fused kernels).  An output counts as released inside the capture when the
    step list frees it."""
    lib = load_library()
    ids: dict = {}
    freed = {s.name for s in program.steps if s.kind == "free"}
    images, n_in, ins, outs, flags = [], [], [], [], []
    for s in program.steps:
        if s.kind != "execute":
            continue
        images.append(s.kernel.serialize())
        n_in.append(len(s.inputs))
        ins += [ids.setdefault(n, len(ids)) for n in s.inputs]
        outs.append(ids.setdefault(s.name, len(ids)))
        flags.append(1 if s.name in freed else 0)
    n = len(images)
    arr = (ctypes.c_char_p * n)(*images)
    lens = (ctypes.c_size_t * n)(*[len(i) for i in images])
    rep = ctypes.create_string_buffer(1 << 16)
    msg = ctypes.create_string_buffer(1 << 22)
    lib.jaxcuda_check_step_list.restype = ctypes.c_int
    lib.jaxcuda_check_step_list.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_size_t),
                                            ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                            ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
    source = ""
    for comp in ((0, 1) if compile else (0,)):
        rc = lib.jaxcuda_check_step_list(n, arr, lens, (ctypes.c_int * n)(*n_in), (ctypes.c_int * max(1, len(ins)))(*ins),
                                         (ctypes.c_int * n)(*outs), bytes(flags), comp, rep, len(rep), msg, len(msg))
        if rc != OK:
            _raise(rc, msg.value.decode())
        if comp == 0:
            source = msg.value.decode()
    return rep.value.decode().splitlines(), source


def _raise(status: int, message: str):
    if status == ESLOT:
        raise SlotError(message)
    if status == EUNSUPPORTED:
        raise (UnsupportedRoutineError if message.startswith("routine ") else UnsupportedOpError)(message)
    if status == EINVAL:
        raise ValueError(message)
    if status == ECOMPILE:
        raise CompileError(message)
    if status == ENOMEM:
        raise MemoryError(message)
    if status == ETIMEOUT:
        raise TimeoutError(message)
    raise CudaError(message)


class Executable:
    """src/backend.ts:213-220: the prepared Kernel or Routine plus backend data."""

    def __init__(self, source, handle: int, backend: "CudaBackend"):
        self.source = source
        self.data = handle
        self._backend = backend

    @property
    def describe(self) -> str:
        return load_library().jaxcuda_exe_describe(self.data).decode()

    @property
    def cuda_source(self) -> str:
        return load_library().jaxcuda_exe_source(self.data).decode()

    def cost(self):
        """(algorithmic bytes, algorithmic flops, kernel launches per dispatch)."""
        b, f, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_int()
        load_library().jaxcuda_exe_cost(self.data, ctypes.byref(b), ctypes.byref(f), ctypes.byref(n))
        return b.value, f.value, n.value


def _prefer_packaged_nccl() -> None:
    """A process holds one libnccl.so.2.  If the `nvidia.nccl` wheel is installed (the copy torch
    links against), point the library at that file, so that a later `import torch` in the same
    process finds the NCCL it was built for instead of an older system one."""
    if os.environ.get("JAXCUDA_NCCL_LIB"):
        return
    import importlib.util
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    for root in (spec.submodule_search_locations if spec and spec.submodule_search_locations else []):
        cand = os.path.join(root, "lib", "libnccl.so.2")
        if os.path.exists(cand):
            os.environ["JAXCUDA_NCCL_LIB"] = cand
            return


class CudaBackend:
    """`Backend` for device "cuda" (src/backend.ts:158-211)."""

    type = "cuda"

    def __init__(self, device: int = 0):
        self._lib = load_library()
        ctx = ctypes.c_void_p()
        rc = self._lib.jaxcuda_create(device, ctypes.byref(ctx))
        if rc != OK:
            _raise(rc, self._lib.jaxcuda_last_error(None).decode())
        self._ctx = ctx
        self.device = device
        self.max_args = self._lib.jaxcuda_max_args()

    # -- helpers ---------------------------------------------------------------------
    def _check(self, rc: int):
        if rc != OK:
            _raise(rc, self._lib.jaxcuda_last_error(self._ctx).decode())

    def close(self):
        if self._ctx:
            self._lib.jaxcuda_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- memory (src/backend.ts:166-190) ----------------------------------------------
    def malloc(self, size: int, initial_data=None) -> int:
        slot = ctypes.c_uint32()
        if initial_data is None:
            self._check(self._lib.jaxcuda_malloc(self._ctx, size, None, 0, ctypes.byref(slot)))
        else:
            buf = np.ascontiguousarray(np.frombuffer(initial_data, dtype=np.uint8) if not isinstance(initial_data, np.ndarray)
                                       else initial_data)
            self._check(self._lib.jaxcuda_malloc(self._ctx, size, buf.ctypes.data, buf.nbytes, ctypes.byref(slot)))
        return slot.value

    def inc_ref(self, slot: int) -> None:
        self._check(self._lib.jaxcuda_incref(self._ctx, slot))

    def dec_ref(self, slot: int) -> None:
        self._check(self._lib.jaxcuda_decref(self._ctx, slot))

    def read_sync(self, slot: int, start: int | None = None, count: int | None = None) -> np.ndarray:
        """Bytes [start, start+count) of the slot as a uint8 array, after all pending work."""
        size = ctypes.c_size_t()
        self._check(self._lib.jaxcuda_slot_size(self._ctx, slot, ctypes.byref(size)))
        start = 0 if start is None else start
        count = size.value - start if count is None else count
        out = np.empty(max(count, 0), dtype=np.uint8)
        self._check(self._lib.jaxcuda_read(self._ctx, slot, start, count, out.ctypes.data))
        return out

    read = read_sync  # the async variant exists so that JS does not block its event loop

    def read_into(self, slot: int, dst: np.ndarray, start: int = 0) -> None:
        self._check(self._lib.jaxcuda_read(self._ctx, slot, start, dst.nbytes, dst.ctypes.data))

    def write(self, slot: int, src: np.ndarray, start: int = 0) -> None:
        self._check(self._lib.jaxcuda_write(self._ctx, slot, start, src.nbytes, src.ctypes.data))

    def read_async(self, slot: int, dst: np.ndarray, start: int = 0) -> int:
        """`read` as a Promise (src/backend.ts:182-186): enqueue the copy into pinned `dst` on the
        download stream and return a ticket; `read_wait(ticket)` is where the Promise resolves."""
        t = ctypes.c_uint64()
        self._check(self._lib.jaxcuda_read_async(self._ctx, slot, start, dst.nbytes, dst.ctypes.data, ctypes.byref(t)))
        return t.value

    def read_wait(self, ticket: int) -> None:
        self._check(self._lib.jaxcuda_read_wait(self._ctx, ticket))

    def write_async(self, slot: int, src: np.ndarray, start: int = 0) -> None:
        """Upload from pinned `src` on the upload stream, ordered between earlier and later dispatches."""
        self._check(self._lib.jaxcuda_write_async(self._ctx, slot, start, src.nbytes, src.ctypes.data))

    def write_ptr(self, slot: int, ptr: int, nbytes: int, start: int = 0) -> None:
        self._check(self._lib.jaxcuda_write(self._ctx, slot, start, nbytes, ptr))

    def read_ptr(self, slot: int, ptr: int, nbytes: int, start: int = 0) -> None:
        self._check(self._lib.jaxcuda_read(self._ctx, slot, start, nbytes, ptr))

    # -- compile (src/backend.ts:192-202) ----------------------------------------------
    def prepare_kernel_sync(self, kernel: Kernel) -> Executable:
        image = kernel.serialize()
        exe = ctypes.c_void_p()
        self._check(self._lib.jaxcuda_prepare_kernel(self._ctx, image, len(image), 0, ctypes.byref(exe)))
        return Executable(kernel, exe.value, self)

    prepare_kernel = prepare_kernel_sync

    def prepare_routine_sync(self, routine: Routine) -> Executable:
        t = routine.type
        flat = lambda shapes: [d for s in shapes for d in s]
        ins, outs = flat(t.input_shapes), flat(t.output_shapes)
        keep = [(ctypes.c_int32 * max(1, len(t.input_dtypes)))(*[int(d) for d in t.input_dtypes]),
                (ctypes.c_int32 * max(1, len(t.input_shapes)))(*[len(s) for s in t.input_shapes]),
                (ctypes.c_int64 * max(1, len(ins)))(*ins),
                (ctypes.c_int32 * max(1, len(t.output_dtypes)))(*[int(d) for d in t.output_dtypes]),
                (ctypes.c_int32 * max(1, len(t.output_shapes)))(*[len(s) for s in t.output_shapes]),
                (ctypes.c_int64 * max(1, len(outs)))(*outs)]
        rt = _RoutineType(len(t.input_shapes), len(t.output_shapes), *keep)
        exe = ctypes.c_void_p()
        import json
        params = json.dumps(routine.params if routine.params is not None else {}).encode()
        self._check(self._lib.jaxcuda_prepare_routine(self._ctx, routine.name.encode(), ctypes.byref(rt), params,
                                                      ctypes.byref(exe)))
        return Executable(routine, exe.value, self)

    prepare_routine = prepare_routine_sync

    # -- run (src/backend.ts:204-211) --------------------------------------------------
    def dispatch(self, exe: Executable, inputs: Sequence[int], outputs: Sequence[int]) -> None:
        ins = (ctypes.c_uint32 * max(1, len(inputs)))(*inputs)
        outs = (ctypes.c_uint32 * max(1, len(outputs)))(*outputs)
        self._check(self._lib.jaxcuda_dispatch(self._ctx, exe.data, ins, len(inputs), outs, len(outputs)))

    # -- extras outside the Backend interface -------------------------------------------
    def sync(self) -> None:
        self._check(self._lib.jaxcuda_sync(self._ctx))

    def event_record(self, index: int) -> None:
        self._check(self._lib.jaxcuda_event_record(self._ctx, index))

    def event_elapsed_ms(self, a: int, b: int) -> float:
        ms = ctypes.c_float()
        self._check(self._lib.jaxcuda_event_elapsed_ms(self._ctx, a, b, ctypes.byref(ms)))
        return ms.value

    def launch_count(self) -> int:
        return int(self._lib.jaxcuda_launch_count(self._ctx))

    def checked_counts(self) -> tuple:
        """Checked build only (JAXCUDA_CHECKED=1 in the environment): (loads the Kernels let fall outside
        their buffers, loads proven in range that were not) since the last call; the second must be 0."""
        a, b = ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self._lib.jaxcuda_checked_counts(self._ctx, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    # -- tracing (src/tracing.ts:15-33, :89-106) ---------------------------------------------
    def start_trace(self) -> None:
        """From here on every eager dispatch is timed on the device (a pair of CUDA events)."""
        self._check(self._lib.jaxcuda_trace_start(self._ctx))

    def stop_trace(self) -> list:
        """Ends the trace and returns one record per dispatch, in dispatch order: the executable's
        handle, its plan, its start relative to `start_trace` and its duration, in milliseconds (what
        the reference passes to `emitTrace`)."""
        n = ctypes.c_int()
        self._check(self._lib.jaxcuda_trace_stop(self._ctx, ctypes.byref(n)))
        out = []
        name = ctypes.create_string_buffer(512)
        for i in range(n.value):
            exe, t0, dt = ctypes.c_void_p(), ctypes.c_double(), ctypes.c_double()
            self._check(self._lib.jaxcuda_trace_record(self._ctx, i, ctypes.byref(exe), ctypes.byref(t0), ctypes.byref(dt), name, 512))
            out.append({"exe": exe.value, "name": name.value.decode(), "start_ms": t0.value, "duration_ms": dt.value})
        return out

    def host_alloc(self, nbytes: int) -> np.ndarray:
        """Pinned host memory as a uint8 array (freed with host_free)."""
        p = ctypes.c_void_p()
        self._check(self._lib.jaxcuda_host_alloc(self._ctx, nbytes, ctypes.byref(p)))
        arr = np.ctypeslib.as_array((ctypes.c_uint8 * max(1, nbytes)).from_address(p.value))[:nbytes]
        arr.flags.writeable = True
        self._pinned = getattr(self, "_pinned", {})
        self._pinned[arr.ctypes.data] = p.value
        return arr

    def host_free(self, arr: np.ndarray) -> None:
        p = self._pinned.pop(arr.ctypes.data, None)
        if p:
            self._check(self._lib.jaxcuda_host_free(self._ctx, p))

    def slot_ptr(self, slot: int) -> int:
        p = ctypes.c_uint64()
        self._check(self._lib.jaxcuda_slot_ptr(self._ctx, slot, ctypes.byref(p)))
        return p.value

    def stream(self) -> int:
        return int(self._lib.jaxcuda_stream(self._ctx))

    def comm_init(self, rank: int, nranks: int, unique_id: bytes) -> None:
        _prefer_packaged_nccl()
        buf = ctypes.create_string_buffer(unique_id, 128)
        self._check(self._lib.jaxcuda_comm_init(self._ctx, rank, nranks, buf))

    @staticmethod
    def comm_unique_id() -> bytes:
        _prefer_packaged_nccl()
        buf = ctypes.create_string_buffer(128)
        if load_library().jaxcuda_comm_unique_id(buf) != OK:
            raise CudaError("ncclGetUniqueId failed (is libnccl.so.2 loadable?)")
        return buf.raw

    def allreduce_sum_f32(self, slots: Sequence[int]) -> None:
        arr = (ctypes.c_uint32 * max(1, len(slots)))(*slots)
        self._check(self._lib.jaxcuda_allreduce_sum_f32(self._ctx, arr, len(slots)))

    def allreduce_sum_f32_async(self, slots: Sequence[int]) -> None:
        """The sum on a second stream, under the kernels dispatched next; `comm_join` before the
        first use of the summed slots."""
        arr = (ctypes.c_uint32 * max(1, len(slots)))(*slots)
        self._check(self._lib.jaxcuda_allreduce_sum_f32_async(self._ctx, arr, len(slots)))

    def comm_join(self) -> None:
        self._check(self._lib.jaxcuda_comm_join(self._ctx))

    def comm_wait(self, timeout_ms: int) -> None:
        """Block until everything issued so far (sums included) has finished.  Raises TimeoutError
        after `timeout_ms` (a peer is late or gone; nothing was cancelled) and CudaError when NCCL
        reports an error, in which case the communicator has been aborted."""
        self._check(self._lib.jaxcuda_comm_wait(self._ctx, int(timeout_ms)))

    def comm_abort(self) -> None:
        """Leave the communicator without waiting for the peers (ncclCommAbort)."""
        self._check(self._lib.jaxcuda_comm_abort(self._ctx))

    # -- captured step lists ---------------------------------------------------------------
    def capture_begin(self) -> None:
        self._check(self._lib.jaxcuda_capture_begin(self._ctx))

    def capture_end(self) -> int:
        g = ctypes.c_void_p()
        self._check(self._lib.jaxcuda_capture_end(self._ctx, ctypes.byref(g)))
        return g.value

    def graph_launch(self, graph: int) -> None:
        self._check(self._lib.jaxcuda_graph_launch(self._ctx, graph))

    def order_waits(self) -> int:
        return int(self._lib.jaxcuda_order_waits(self._ctx))

    def read_event(self, ticket: int) -> int:
        ev = ctypes.c_void_p()
        self._check(self._lib.jaxcuda_read_event(self._ctx, ticket, ctypes.byref(ev)))
        return ev.value

    def event_block(self, event: int) -> None:
        """Waits for a ticket's event; safe on a thread other than the one driving the backend."""
        if self._lib.jaxcuda_event_block(event) != OK:
            raise CudaError("cudaEventSynchronize failed")

    def graph_cost(self, graph: int) -> tuple:
        """(kernel launches, algorithmic bytes, fused runs) of one launch of the graph."""
        n, b, f = ctypes.c_uint64(), ctypes.c_double(), ctypes.c_int()
        self._check(self._lib.jaxcuda_graph_cost(graph, ctypes.byref(n), ctypes.byref(b), ctypes.byref(f)))
        return n.value, b.value, f.value

    def graph_destroy(self, graph: int) -> None:
        self._check(self._lib.jaxcuda_graph_destroy(self._ctx, graph))

    def copy(self, dst: int, src: int) -> None:
        self._check(self._lib.jaxcuda_copy(self._ctx, dst, src))

    def sort_no_alloc(self, dtype: DType, x_slot: int, y_slot: int, batch: int, n: int) -> None:
        """Sort rows of x_slot into y_slot through the entry point that allocates nothing (its
        work buffer is a fixed array inside the library; see include/jaxcuda.h for the limit)."""
        err = ctypes.create_string_buffer(256)
        rc = self._lib.jaxcuda_sort_no_alloc(self.stream(), int(dtype), self.slot_ptr(x_slot), self.slot_ptr(y_slot),
                                             batch, n, err, len(err))
        if rc != OK:
            _raise(rc, err.value.decode())

    # -- conveniences for tests and programs -------------------------------------------
    def put(self, array: np.ndarray) -> int:
        a = np.ascontiguousarray(array)
        return self.malloc(a.nbytes, a.view(np.uint8).reshape(-1))

    def get(self, slot: int, dtype: DType | str, shape=None) -> np.ndarray:
        from .alu import np_dtype
        name = np_dtype(dtype) if isinstance(dtype, DType) else dtype
        out = self.read_sync(slot).view(name)
        return out.reshape(shape) if shape is not None else out
