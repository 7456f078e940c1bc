"""CPU-side checks of the host logic: the wire format, the planner's skeleton choice, NVRTC
compilation of every skeleton for sm_100a (no GPU needed), and the C ABI's exported symbols."""
import ctypes
import re
import struct
from pathlib import Path

import numpy as np
import pytest

from jax_js_b200 import AluExp, AluOp, AluVar, DType, Kernel, Reduction, ShapeTracker, accessor_global, unravel_alu
from jax_js_b200 import mlp
from jax_js_b200 import programs as P
from jax_js_b200.alu import NODE_WORDS, WIRE_MAGIC
from jax_js_b200.backend import (SYMBOLS, CudaBackend, CudaError, UnsupportedOpError, check_kernel)

ROOT = Path(__file__).resolve().parent.parent
F32, I32, F16 = DType.Float32, DType.Int32, DType.Float16
g, r = AluVar.gidx, AluVar.ridx


def test_every_declared_symbol_is_exported(lib):
    header = (ROOT / "include" / "jaxcuda.h").read_text()
    declared = set(re.findall(r"\b(jaxcuda_[a-z0-9_]+)\s*\(", header))
    declared -= {"jaxcuda_status"}
    assert declared == set(SYMBOLS), declared ^ set(SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None


def test_create_fails_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(CudaError, match="no CPU fallback"):
        CudaBackend(0)


def test_wire_image_layout():
    k = P.row_reduce_kernel(3, 2, AluOp.Add)
    img = k.serialize()
    head = struct.unpack("<10I", img[:40])
    assert head[0] == WIRE_MAGIC and head[1] == 1 and head[2] == 3 and head[4] == 1
    assert head[5] == int(F32) and head[6] == int(AluOp.Add) and head[7] == 2
    assert len(img) == 40 + (head[8] + head[9]) * NODE_WORDS * 4
    assert k.fingerprint() == P.row_reduce_kernel(3, 2, AluOp.Add).fingerprint()
    assert k.fingerprint() != P.row_reduce_kernel(3, 2, AluOp.Max).fingerprint()


def test_f16_add_reduction_accumulates_in_f32():
    # src/alu.ts:1560-1568
    red = Reduction(F16, AluOp.Add, 8)
    assert red.dtype == F32 and red.epilogue.op == AluOp.Cast and red.epilogue.dtype == F16
    assert Reduction(F16, AluOp.Max, 8).dtype == F16


def test_bad_images_are_rejected(lib):
    def check(img):
        msg = ctypes.create_string_buffer(4096)
        return lib.jaxcuda_check_kernel(img, len(img), 148, -1, 0, None, 0, msg, len(msg)), msg.value.decode()
    good = P.lse_finish_kernel(16).serialize()
    assert check(good)[0] == 0
    assert check(good[:-4])[0] == 3
    assert check(b"\0\0\0\0" + good[4:])[0] == 3
    words = list(struct.unpack(f"<{len(good) // 4}I", good))
    words[10 + 3] = 99  # first node: operand index beyond itself
    words[10 + 2] = 1
    assert check(struct.pack(f"<{len(words)}I", *words))[0] == 3


CASES = {
    "k1 row max": (P.row_reduce_kernel(8192, 4096, AluOp.Max), "reduce-row TPR=256 V=4"),
    "k2 exp": (P.softmax_exp_kernel(8192, 4096), "elementwise V=4"),
    "k4 scale": (P.softmax_scale_kernel(8192, 4096), "elementwise V=4"),
    "k2' fused sum": (P.lse_sum_kernel(8192, 4096), "reduce-row TPR=128 V=4"),
    "k3' tiny": (P.lse_finish_kernel(8192), "elementwise"),
    "k5 argmax": (P.argmax_index_kernel(8192, 4096), "reduce-row TPR=256 V=4"),
    "matvec xW": (P.matvec_kernel(4096, 11008, F16, orientation="xW"), "reduce-col V=8"),
    "matvec Wx": (P.matvec_kernel(11008, 4096, F16, orientation="Wx"), "reduce-row TPR=128 V=8"),
    "dot f32": (P.dot_kernel(1024, 1024, 1024), "gemm"),
    "dot f16": (P.dot_kernel(4096, 4096, 4096, F16), "gemm"),
    "dot TN": (P.dot_kernel(784, 2048, 8192, a_layout="km"), "gemm"),
    "dot NT": (P.dot_kernel(8192, 784, 2048, b_layout="nk"), "gemm"),
    "dot bias relu": (P.dot_kernel(256, 1024, 784, bias=True, relu=True), "gemm"),
    "dot batched": (P.dot_kernel(64, 48, 32, batch=5), "gemm-ffma 5x64x48x32"),
    "dot tiny": (P.dot_kernel(16, 48, 24), "reduce-"),
    "short rows": (P.row_reduce_kernel(65536, 10, AluOp.Max), "reduce-col V=1"),
    "mid rows": (P.row_reduce_kernel(4096, 200, AluOp.Add), "reduce-row TPR=32"),
    "scalar sum": (P.row_reduce_kernel(1, 1 << 24, AluOp.Add), "splits="),
    # the 10-class layer of the MLP: forward, weight gradient, back-propagated dot, bias gradient
    "skinny forward": (P.dot_kernel(8192, 10, 2048), "dot-skinny 8192x10x2048"),
    "skinny weight grad": (P.dot_kernel(2048, 10, 8192, a_layout="km"), "dot-skinny-t 2048x10x8192"),
    "small-k backward": (P.dot_kernel(8192, 2048, 10), "dot-small-k 8192x2048x10"),
    "bias grad": (Kernel(1, 2048, AluExp.global_index(F32, 0, 8192 * 2048, AluExp.add(g, AluExp.mul(AluVar.ridx, AluExp.i32(2048)))),
                         Reduction(F32, AluOp.Add, 8192)), "reduce-col V=4"),
    "skinny f16": (P.dot_kernel(4096, 16, 512, F16, a_layout="km"), "dot-skinny-t"),
    "small-k ragged": (P.dot_kernel(65, 1028, 16, a_layout="km", b_layout="nk"), "dot-small-k"),
}


@pytest.mark.parametrize("name", list(CASES))
def test_planner_choice_and_nvrtc_compile(lib, name):
    kernel, expect = CASES[name]
    describe, source = check_kernel(kernel, compile=True)
    assert expect in describe, describe
    assert 'extern "C" __global__' in source


def test_vector_loads_only_where_provably_aligned(lib):
    n = 4096
    aligned = Kernel(1, n, AluExp.global_index(F32, 0, n, g))
    shifted = Kernel(1, n, AluExp.global_index(F32, 0, n + 1, AluExp.add(g, AluExp.i32(1))))
    flipped = Kernel(1, n, accessor_global(F32, 0, ShapeTracker.from_shape([n]).flip([True]), [g]))
    assert "jx_load(pk" in check_kernel(aligned, compile=False)[1]
    assert "jx_load(pk" not in check_kernel(shifted, compile=False)[1]
    assert "jx_load(pk" not in check_kernel(flipped, compile=False)[1]
    bcast = check_kernel(P.softmax_scale_kernel(64, 256), compile=False)[1]
    assert "bc" in bcast  # the per-row scalar is fetched once per 128-bit run


def test_unsupported_combination_uses_reference_wording(lib):
    bad = Kernel(1, 4, AluExp(AluOp.Sub, DType.Bool, [AluExp.global_index(DType.Bool, 0, 4, g), AluExp.bool(False)]))
    with pytest.raises(UnsupportedOpError, match=r"Sub<bool> not supported in cuda backend"):
        check_kernel(bad)


def test_shape_tracker_views_lower_to_expected_indices():
    st = ShapeTracker.from_shape([4, 6]).permute([1, 0])
    ix, valid = st.to_alu_exp([AluExp.i32(5), AluExp.i32(3)])
    assert ix.arg == 3 * 6 + 5 and valid.arg == 1
    padded = ShapeTracker.from_shape([3]).pad([(1, 2)])
    assert padded.shape == (6,) and padded.data_range() == (0, 3)
    e = accessor_global(F32, 0, padded, [g])
    assert e.op == AluOp.Where


def test_shape_tracker_movement_sequences_match_numpy():
    """Random chains of permute / expand / flip / pad / shrink / reshape, including the ones that
    need a second view (reshape after permute, after pad, after flip), lowered to an index and a
    validity expression and evaluated by the oracle, against the same chain applied with numpy."""
    import oracle
    rng = np.random.default_rng(7)
    multi = 0
    for trial in range(300):
        shape = [int(d) for d in rng.integers(1, 5, rng.integers(1, 4))]
        base = rng.standard_normal(shape).astype(np.float32)
        base[base == 0] = 1.0                                   # zeros mark padding below
        arr, st = base, ShapeTracker.from_shape(shape)
        for _ in range(int(rng.integers(1, 6))):
            op = rng.choice(["permute", "expand", "flip", "pad", "shrink", "reshape", "reshape"])
            nd = arr.ndim
            if op == "permute":
                axes = [int(a) for a in rng.permutation(nd)]
                arr, st = arr.transpose(axes), st.permute(axes)
            elif op == "expand":
                arr = arr.reshape((1,) + arr.shape)
                st = st.reshape((1,) + st.shape)
                k = int(rng.integers(1, 4))
                arr, st = np.broadcast_to(arr, (k,) + arr.shape[1:]), st.expand((k,) + st.shape[1:])
            elif op == "flip":
                f = [bool(b) for b in rng.integers(0, 2, nd)]
                arr = arr[tuple(slice(None, None, -1) if b else slice(None) for b in f)]
                st = st.flip(f)
            elif op == "pad":
                w = [(int(a), int(b)) for a, b in rng.integers(0, 3, (nd, 2))]
                arr, st = np.pad(arr, w), st.pad(w)
            elif op == "shrink":
                r = []
                for d in arr.shape:
                    lo = int(rng.integers(0, d))
                    r.append((lo, int(rng.integers(lo + 1, d + 1))))
                arr, st = arr[tuple(slice(a, b) for a, b in r)], st.shrink(r)
            else:
                size = arr.size
                divs = [d for d in range(1, size + 1) if size % d == 0]
                a = int(rng.choice(divs))
                b = int(rng.choice([d for d in divs if (size // a) % d == 0]))
                new = [a, b, size // (a * b)]
                arr, st = np.ascontiguousarray(arr).reshape(new), st.reshape(new)
            assert tuple(st.shape) == arr.shape
            if arr.size > 4096:
                break
        multi += len(st.views) > 1
        k = Kernel(1, arr.size, accessor_global(DType.Float32, 0, st, unravel_alu(st.shape, AluVar.gidx)))
        got = oracle.run_kernel(k, [base.reshape(-1)])
        assert np.array_equal(got, np.ascontiguousarray(arr).reshape(-1)), (trial, [v.shape for v in st.views])
    assert multi >= 30, multi     # the multi-view path was exercised


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (100, 1000), (16, 12), (4, 16384)])
def test_softmax_step_list_becomes_one_row_program(lib, rows, cols):
    """What a capture would launch for the softmax / logsumexp / argmax program: one row-resident kernel
    (NVRTC-compiled here) that moves only the program's own inputs and outputs."""
    from jax_js_b200.backend import check_step_list
    report, source = check_step_list(P.softmax_lse_argmax_program(rows, cols))
    assert len(report) == 1 and report[0].startswith("0-9: row-fused 8 kernels"), report     # 10 Kernels, two repeated row maxima folded
    assert report[0].endswith(f"bytes={2 * rows * cols * 4 + 2 * rows * 4 + cols * 4}")
    assert source.count("__global__") == 1 and "jx_rowfuse" in source
    body = source[source.index("jx_rowfuse"):]
    assert body.count("jx_store(") == 1              # of the rows x cols arrays only the softmax is written


def test_step_lists_that_are_no_row_programs_stay_as_they_are(lib):
    from jax_js_b200 import mlp
    from jax_js_b200.backend import check_step_list
    # rows of 10 classes are not 128-bit runs, GEMMs and transposes are no row stages
    report, _ = check_step_list(mlp.mlp_grad_program(256, [64, 128, 10], global_batch=256), compile=False)
    assert not any("row-fused" in r for r in report), report
    # a row too long for one CTA's registers is left to the row-reduce skeleton
    report, _ = check_step_list(P.softmax_lse_argmax_program(4, 65536), compile=False)
    assert not any("row-fused" in r for r in report), report


def test_step_list_check_substitutes_an_elementwise_producer_into_its_only_consumer(lib):
    """The vmapped gradient program ends in per-example outer products written batch-last and the
    Kernels that move the batch axis first; the step-list check reports each pair as one Kernel
    whose loads are contiguous or broadcast again (the flattened index splits back into its digits)."""
    from jax_js_b200 import mlp
    from jax_js_b200.backend import check_step_list
    prog = mlp.mlp_grad_program(64, [784, 1024, 10], per_example=True)
    report, source = check_step_list(prog, compile=True)
    fused = [l for l in report if "producer substituted" in l]
    big = [l for l in fused if "bytes=205983744" in l]   # x, dz1 in; f32[64, 784, 1024] out, once
    assert len(big) == 1 and len(fused) >= 2, report
    assert big[0].split(":")[1].strip().startswith("elementwise V=4"), big[0]
    body = source[source.index("jx_elementwise("):]
    assert "jx_load(pk" in body.split("jx_store")[0]     # the row of dz1 comes as 128-bit vectors


def test_step_list_check_reports_epilogue_fusion_and_small_batches(lib):
    """Without a GPU: the back-propagated cotangents of the training step go into the epilogues of the
    Dot Kernels that produce them, and the log-softmax chain of the vmapped program, a dozen Kernels
    over a few hundred elements, is one launch."""
    from jax_js_b200 import mlp
    from jax_js_b200.backend import check_step_list
    report, _ = check_step_list(mlp.mlp_grad_program(8192, [784, 2048, 2048, 10], global_batch=65536), compile=True)
    fused = [l for l in report if "consumer in the epilogue" in l]
    assert len(fused) == 2 and any("gemm-tcgen05" in l and "cta-pairs" in l for l in fused) and any("dot-small-k" in l for l in fused), report
    report, source = check_step_list(mlp.mlp_grad_program(64, [784, 1024, 10], per_example=True), compile=True)
    batches = [l for l in report if "batch of" in l]
    assert len(batches) == 1 and "batch of 12 small kernels" in batches[0], report
    assert len(report) == 12                     # 27 Kernels in 12 launches
    body = source[source.index("jx_batch("):]
    assert body.count("__syncthreads();") == 11 and "__restrict__" not in body.split("{")[0]


def test_checked_build_sources_compile_without_a_gpu():
    """JAXCUDA_CHECKED=1 (read once per process, hence the child): every scalar load of the generated
    source goes through jx_ix, and NVRTC accepts the result for each skeleton."""
    import os
    import subprocess
    import sys
    script = r"""
import os, sys
sys.path.insert(0, os.environ["REPO_ROOT"])
from jax_js_b200 import AluOp, programs as P
from jax_js_b200.backend import check_kernel
kernels = [P.softmax_exp_kernel(64, 512), P.row_reduce_kernel(64, 512, AluOp.Max), P.dot_kernel(256, 256, 128, bias=True, relu=True),
           P.dot_kernel(64, 10, 784), P.conv2d_kernel(2, 3, 17, 19, 5, 3, 3, 1, 1), P.conv2d_kernel(8, 64, 28, 28, 128, 3, 3, 1, 1),
           P.matvec_kernel(512, 1024)]
for k in kernels:
    describe, source = check_kernel(k, compile=True)[:2]
    assert "jx_ix(" in source, describe
print("ok", len(kernels))
"""
    env = dict(os.environ, JAXCUDA_CHECKED="1", REPO_ROOT=str(ROOT))
    out = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == "ok 7", out.stdout[-500:] + out.stderr[-1500:]
