"""Writes tests/golden/reference_vectors.json: known-answer vectors copied, as data, from the
reference's own test-suite (each entry cites the file and lines it was read from).

The reference cannot be executed where this repository is built (no JavaScript or WebAssembly
runtime), so these are the expected values its tests assert, not outputs generated here.  The
file is consumed by tests/test_golden_fixture.py on CPU (the oracle) and on the GPU (the cuda
backend).  Run `python tests/golden/make_reference_vectors.py` to rewrite the JSON.
"""
import json
from pathlib import Path

NAN, INF = "nan", "inf"   # JSON has no literals for these; the loader maps the strings back

VECTORS = [
    # ---- Sort (Routines.Sort) ----------------------------------------------------------------
    {"kind": "sort", "cite": "test/numpy.test.ts:4632-4640", "dtype": "float32",
     "x": [3, 1, 4, 1, 5, 9, 2, 6], "want": [1, 1, 2, 3, 4, 5, 6, 9]},
    {"kind": "sort", "cite": "test/numpy.test.ts:4642-4653", "dtype": "float32",
     "x": [[3, 1, 2], [6, 4, 5]], "want": [[1, 2, 3], [4, 5, 6]]},
    {"kind": "sort", "cite": "test/numpy.test.ts:4655-4659 (NaN sorts last)", "dtype": "float32",
     "x": [3, NAN, 1, NAN, 2], "want": [1, 2, 3, NAN, NAN]},
    {"kind": "sort", "cite": "test/numpy.test.ts:4719-4722", "dtype": "int32", "x": [3, 1, 4, 1, 5], "want": [1, 1, 3, 4, 5]},
    {"kind": "sort", "cite": "test/numpy.test.ts:4723-4726", "dtype": "uint32", "x": [3, 1, 4, 1, 5], "want": [1, 1, 3, 4, 5]},
    # ---- Argsort (Routines.Argsort): indices ----------------------------------------------------
    {"kind": "argsort", "cite": "test/numpy.test.ts:4750-4757", "dtype": "float32", "x": [3, 1, 4, 2, 5], "want": [1, 3, 0, 2, 4]},
    {"kind": "argsort", "cite": "test/numpy.test.ts:4759-4767", "dtype": "float32",
     "x": [[3, 1, 2], [6, 4, 5]], "want": [[1, 2, 0], [1, 2, 0]]},
    {"kind": "argsort", "cite": "test/numpy.test.ts:4769-4785 (stable; NaN last; -0 == +0)", "dtype": "float32",
     "x": [3, 1, 1, NAN, INF, 2, NAN, 1, 0, -0.0, INF], "want": [8, 9, 1, 2, 7, 5, 0, 4, 10, 3, 6]},
    # ---- Threefry (AluOp.Threefry2x32) ----------------------------------------------------------
    {"kind": "threefry", "cite": "src/alu.test.ts:202-209", "key": [0, 0], "counter": [0, 0], "want": [1797259609, 2579123966]},
    {"kind": "random_bits", "cite": "test/random.test.ts:21-25 (bits(key(0)) = x0 ^ x1)", "key": [0, 0], "counter": [0, 0], "want": 4070199207},
    # ---- softmax / logsumexp / argmax program ----------------------------------------------------
    {"kind": "softmax", "cite": "test/nn.test.ts:107-117", "x": [[1, 2, 3], [4, 5, 6]],
     "want": [[0.09003057, 0.24472848, 0.66524094], [0.09003057, 0.24472848, 0.66524094]], "rtol": 1e-5},
    {"kind": "logsumexp", "cite": "test/nn.test.ts:164-168", "x": [[-10, -1, 1, 2]], "want": [2.3490167], "atol": 1e-5},
    {"kind": "logsumexp", "cite": "test/nn.test.ts:170-178 (all eight values)", "x": [[1, 2, 3, 4, 5, 6, 7, 8]], "want": [8.45834], "atol": 1e-4},
    {"kind": "argmax", "cite": "test/argreduce.test.ts:15-19 (first index on ties)", "x": [[3, 5, 5, 2, 5, 1]], "want": [1]},
    {"kind": "argmax", "cite": "test/argreduce.test.ts:21-25", "x": [[-10, -5, -20, -5, -15]], "want": [1]},
    {"kind": "argmax", "cite": "test/argreduce.test.ts:27-31", "x": [[1, 1, 1, 1, 1]], "want": [0]},
    {"kind": "argmax", "cite": "test/argreduce.test.ts:33-44 (row-wise)", "x": [[1, 2, 3], [6, 5, 4], [7, 8, 9]], "want": [2, 0, 2]},
    # ---- matmul ---------------------------------------------------------------------------------------
    {"kind": "matmul", "cite": "test/numpy.test.ts:1518-1532", "a": [[1, 2], [3, 4]], "b": [[5, 6], [7, 8]], "want": [[19, 22], [43, 50]]},
    {"kind": "matmul", "cite": "test/numpy.test.ts:1534-1550", "a": [[1, 2, 3], [4, 5, 6]], "b": [[7, 8], [9, 10], [11, 12]],
     "want": [[58, 64], [139, 154]]},
    # ---- a jitted two-layer MLP with logSoftmax, end to end (exact) -------------------------------------
    {"kind": "mlp_predict", "cite": "test/platform-test/node.test.ts:29-58", "dims": [2, 2, 2],
     "x": [[1, 2], [3, 4]], "params": [[[1, 2], [3, 4]], [1, 2], [[1, 2], [3, 4]], [1, 2]], "want": [[-21, 0], [-41, 0]]},
    # ---- linear algebra routines --------------------------------------------------------------------
    {"kind": "lu", "cite": "test/lax-linalg.test.ts:277-290", "a": [[4, 3], [6, 3]],
     "lu": [[6, 3], [0.6666667, 1.0]], "pivots": [1, 1], "permutation": [1, 0], "rtol": 1e-6},
    {"kind": "cholesky_reconstructs", "cite": "test/lax-linalg.test.ts:24-38", "x": [[2.0, 1.0], [1.0, 2.0]], "rtol": 1e-5},
    {"kind": "cholesky_reconstructs", "cite": "test/lax-linalg.test.ts:40-52", "x": [[4.0, 2.0, 1.0], [2.0, 5.0, 3.0], [1.0, 3.0, 6.0]], "rtol": 1e-5},
    {"kind": "jacobi_eigh", "cite": "test/lax-linalg.test.ts:153-165 (unsorted: values 3, 1, 2; vectors = identity)",
     "x": [[3.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 2.0]], "values": [3, 1, 2], "vectors": [[1, 0, 0], [0, 1, 0], [0, 0, 1]]},
    {"kind": "fft", "cite": "test/numpy-fft.test.ts:91-96 (inverse)", "inverse": True, "real": [6, -2, -2, -2], "imag": [0, 2, 0, -2],
     "want_real": [0, 1, 2, 3], "want_imag": [0, 0, 0, 0], "atol": 1e-6},
    {"kind": "fft", "cite": "test/numpy-fft.test.ts:170-174 (rfft of [0,1,2,3] keeps the first three)", "inverse": False,
     "real": [0, 1, 2, 3], "imag": [0, 0, 0, 0], "want_real": [6, -2, -2, -2], "want_imag": [0, 2, 0, -2], "atol": 1e-5},
    # ---- Scatter routine ------------------------------------------------------------------------------
    {"kind": "scatter", "cite": "src/backend/backend.test.ts:118-187", "op": "update", "shape": [4], "updates": [7], "indices": [1], "want": [0, 7, 0, 0]},
    {"kind": "scatter", "cite": "src/backend/backend.test.ts:118-187 (an empty update clears the output)", "op": "update", "shape": [4],
     "updates": [], "indices": [], "want": [0, 0, 0, 0]},
]

if __name__ == "__main__":
    out = Path(__file__).with_name("reference_vectors.json")
    out.write_text(json.dumps(VECTORS, indent=1) + "\n")
    print(f"wrote {len(VECTORS)} vectors to {out}")
