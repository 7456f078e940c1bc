"""The checked build (JAXCUDA_CHECKED=1): every scalar load of the generated kernels tests its index.
Run in a child process, because the switch is read once per process.  Loads that the planner has
proven in range must never miss; loads that a Kernel lets fall outside are counted one by one."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import os, sys
import numpy as np
root = os.environ["REPO_ROOT"]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
from jax_js_b200 import AluExp, AluOp, AluVar, DType, Kernel, Reduction
from jax_js_b200 import programs as P
from jax_js_b200.backend import CudaBackend
from util import run_cuda
import test_fuzz_kernels as fuzz
F32, I32 = DType.Float32, DType.Int32
g = AluVar.gidx
be = CudaBackend(0)
rng = np.random.default_rng(5)

# 1. a gather with indices outside the table: they read element 0 and are counted
V, D, B = 1000, 96, 777
table = rng.standard_normal((V, D)).astype(np.float32)
idx = rng.integers(0, V, B).astype(np.int32)
idx[:4] = [0, V - 1, V + 5, -3]
row = AluExp.global_index(I32, 1, B, AluExp.idiv(g, AluExp.i32(D)))
k = Kernel(2, B * D, AluExp.global_index(F32, 0, V * D, AluExp.add(AluExp.mul(row, AluExp.i32(D)), AluExp.mod(g, AluExp.i32(D)))))
got = run_cuda(be, k, [table, idx]).reshape(B, D)
assert np.array_equal(got[4:], table[idx[4:]])
allowed, proven = be.checked_counts()
# row V+5 is outside for every column; row -3 is outside while -3*D + d < 0, i.e. for all d < D (3*D > D)
print("gather", allowed, proven)
assert allowed == 2 * D and proven == 0, (allowed, proven)

# 2. the headline program, dots with epilogues, convolutions on both routes, transposing copies
prog = P.softmax_lse_argmax_program(256, 512)
x = rng.standard_normal((256, 512)).astype(np.float32)
prog.prepare(be)
outs = prog.execute(be, [be.put(x), be.put(P.argmax_iota(512))])
be.sync()
for k, arrays in [
    (P.dot_kernel(300, 200, 136, bias=True, relu=True), [rng.standard_normal((300, 136)), rng.standard_normal((136, 200)), rng.standard_normal(200)]),
    (P.dot_kernel(64, 10, 784), [rng.standard_normal((64, 784)), rng.standard_normal((784, 10))]),
    (P.dot_kernel(1001, 130, 33, a_layout="km", b_layout="nk"), [rng.standard_normal((33, 1001)), rng.standard_normal((130, 33))]),
    (P.conv2d_kernel(2, 3, 17, 19, 5, 3, 3, 1, 1), [rng.standard_normal((2, 3, 17, 19)), rng.standard_normal((5, 3, 3, 3))]),
    (P.conv2d_kernel(8, 64, 28, 28, 128, 3, 3, 1, 1), [rng.standard_normal((8, 64, 28, 28)), rng.standard_normal((128, 64, 3, 3))]),
    (P.conv2d_kernel(6, 48, 31, 29, 80, 3, 3, 2, 1), [rng.standard_normal((6, 48, 31, 29)), rng.standard_normal((80, 48, 3, 3))]),
    (P.matvec_kernel(512, 1000, DType.Float32, orientation="xW"), None),
]:
    if arrays is None:
        arrays = [rng.standard_normal(512), rng.standard_normal((512, 1000))]
    run_cuda(be, k, [np.asarray(a, np.float32) for a in arrays])
allowed, proven = be.checked_counts()
print("programs", allowed, proven)
assert proven == 0, proven

# 3. the seeded random Kernels of the fuzz suite
ran = 0
for seed in range(48):
    kernel, args = fuzz.random_kernel(seed)
    try:
        run_cuda(be, kernel, fuzz._inputs_for(args, seed))
        ran += 1
    except Exception as e:        # a Kernel the planner refuses is refused in the normal build too
        print("refused", seed, type(e).__name__)
allowed, proven = be.checked_counts()
print("random", ran, allowed, proven)
assert ran >= 40 and proven == 0, (ran, proven)
be.close()
print("done")
"""


def test_checked_build_counts_loads_outside_their_buffers(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, JAXCUDA_CHECKED="1", REPO_ROOT=os.path.dirname(here))
    out = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-2500:]
    assert out.stdout.strip().endswith("done"), out.stdout[-1500:]


@pytest.mark.skipif(os.environ.get("JAXCUDA_CHECKED", "0") not in ("", "0"), reason="this session is a checked build")
def test_normal_build_has_no_counters(backend):
    with pytest.raises(ValueError):
        backend.checked_counts()
