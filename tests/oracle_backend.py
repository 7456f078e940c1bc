"""Test-only stand-in for a backend: the same slot / prepare / dispatch / read surface as
`CudaBackend`, executing every Kernel with the CPU oracle.  It exists so that multi-kernel
programs (the MLP steps) can be replayed on the oracle side of a parity check, and so that the
data-parallel host logic can run as gloo ranks on CPU.  Nothing in the product imports it."""
import numpy as np

import oracle
from jax_js_b200 import DType, np_dtype


class OracleExecutable:
    def __init__(self, kernel):
        self.source = kernel

    def cost(self):
        return float(self.source.algorithmic_bytes()), 0.0, 1


class OracleBackend:
    type = "oracle"

    def __init__(self, dist=None, threads=None, fma=False):
        self.slots, self.next, self.dist, self.threads, self.fma = {}, 1, dist, threads, fma
        self.async_calls, self.joined = [], True

    def malloc(self, size, initial_data=None):
        buf = np.zeros(size, np.uint8) if initial_data is None else np.frombuffer(bytes(initial_data), np.uint8).copy()
        assert buf.nbytes == size
        self.slots[self.next] = [buf, 1]
        self.next += 1
        return self.next - 1

    def put(self, array):
        a = np.ascontiguousarray(array)
        return self.malloc(a.nbytes, a.view(np.uint8).reshape(-1))

    def inc_ref(self, slot):
        self.slots[slot][1] += 1

    def dec_ref(self, slot):
        self.slots[slot][1] -= 1
        if self.slots[slot][1] == 0:
            del self.slots[slot]

    def read_sync(self, slot, start=None, count=None):
        buf = self.slots[slot][0]
        start = 0 if start is None else start
        return buf[start:len(buf) if count is None else start + count].copy()

    def get(self, slot, dtype, shape=None):
        out = self.read_sync(slot).view(np_dtype(dtype) if isinstance(dtype, DType) else dtype)
        return out.reshape(shape) if shape is not None else out

    def prepare_kernel_sync(self, kernel):
        return OracleExecutable(kernel)

    prepare_kernel = prepare_kernel_sync

    def dispatch(self, exe, inputs, outputs):
        k = exe.source
        args = []
        dtypes = {}
        roots = [k.exp] + ([k.reduction.epilogue] if k.reduction else [])
        for root in roots:
            for e in root.toposort():
                if e.op.name == "GlobalIndex":
                    dtypes[e.arg[0]] = e.dtype
        for i, s in enumerate(inputs):
            args.append(self.slots[s][0].view(np_dtype(dtypes.get(i, DType.Float32))))
        out = self.slots[outputs[0]][0].view(np_dtype(k.dtype))
        oracle.run_kernel(k, args, out=out, threads=self.threads, fma=self.fma)

    def allreduce_sum_f32(self, slots):
        if self.dist is None:
            return
        import torch
        for s in slots:
            t = torch.from_numpy(self.slots[s][0].view(np.float32))
            self.dist.all_reduce(t)

    def allreduce_sum_f32_async(self, slots):
        """The trainer issues one such call per layer as soon as the layer's gradients exist; here the
        sum simply happens at once.  The calls are logged so that a test can check their grouping."""
        self.async_calls.append(len(slots))
        self.joined = False
        self.allreduce_sum_f32(slots)

    def comm_join(self):
        self.joined = True

    def sync(self):
        pass
