"""ctypes binding of the CPU oracle (oracle/oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Imported by tests/, by the smoke check and by the bench's CPU-baseline legs; never
by the product package.  `build()` compiles oracle.cpp with g++ into
oracle/liboracle.so (kept out of git, shipped with the tree).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "oracle.cpp"
_LIB = _HERE / "liboracle.so"
_lib = None

MODE_AUTO, MODE_WASM, MODE_CPU = 0, 1, 2


def build(force: bool = False) -> Path:
    """g++ -O3 -ffp-contract=off: each f32 operation rounds on its own, as Wasm's do."""
    deps = [_SRC, _HERE.parent / "include" / "jaxcuda_ir.h"]
    if not force and _LIB.exists() and all(_LIB.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists()):
        return _LIB
    cmd = ["g++", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
           "-std=c++17", "-shared", "-fPIC", "-o", str(_LIB), str(_SRC)]
    subprocess.run(cmd, check=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB))
        L.oracle_last_error.restype = ctypes.c_char_p
        L.oracle_kernel.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                    ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64,
                                    ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oracle_sort.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64]
        L.oracle_argsort.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_uint64, ctypes.c_uint64]
        L.oracle_wasm_unary.argtypes = [ctypes.c_int, ctypes.c_float]
        L.oracle_wasm_unary.restype = ctypes.c_float
        L.oracle_threefry2x32.argtypes = [ctypes.c_uint32] * 4 + [ctypes.POINTER(ctypes.c_uint32)]
        L.oracle_double_to_half.argtypes = [ctypes.c_double]
        L.oracle_double_to_half.restype = ctypes.c_uint16
        L.oracle_half_to_double.argtypes = [ctypes.c_uint16]
        L.oracle_half_to_double.restype = ctypes.c_double
        _lib = L
    return _lib


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def run_kernel(kernel, args, *, begin: int = 0, end: int | None = None, mode: int = MODE_AUTO,
               fma: bool = False, threads: int | None = None, out: np.ndarray | None = None) -> np.ndarray:
    """Evaluate `kernel` (a jax_js_b200.alu.Kernel) over outputs [begin, end).

    `args` are numpy arrays, one per kernel argument.  Returns the whole output
    array (elements outside [begin, end) are zero unless `out` is passed in).
    """
    from jax_js_b200.alu import np_dtype  # the IR definition is shared; no device code is touched

    L = lib()
    image = kernel.serialize()
    arrays = [np.ascontiguousarray(a) for a in args]
    if len(arrays) != kernel.nargs:
        raise ValueError(f"kernel takes {kernel.nargs} arguments, got {len(arrays)}")
    ptrs = (ctypes.c_void_p * max(1, len(arrays)))(*[a.ctypes.data for a in arrays])
    if out is None:
        out = np.zeros(kernel.size, dtype=np_dtype(kernel.dtype))
    end = kernel.size if end is None else end
    rc = L.oracle_kernel(image, len(image), ptrs, out.ctypes.data, begin, end, mode, int(fma),
                         threads if threads is not None else default_threads())
    if rc:
        raise RuntimeError(L.oracle_last_error().decode())
    return out


def sort(x: np.ndarray, dtype_code: int) -> np.ndarray:
    x = np.ascontiguousarray(x)
    n = x.shape[-1] if x.ndim else 0
    y = np.empty_like(x)
    if x.size:
        if lib().oracle_sort(dtype_code, x.ctypes.data, y.ctypes.data, x.size // n, n):
            raise RuntimeError(lib().oracle_last_error().decode())
    return y


def argsort(x: np.ndarray, dtype_code: int):
    x = np.ascontiguousarray(x)
    n = x.shape[-1] if x.ndim else 0
    y = np.empty_like(x)
    yi = np.empty(x.shape, dtype=np.int32)
    if x.size:
        if lib().oracle_argsort(dtype_code, x.ctypes.data, y.ctypes.data, yi.ctypes.data, x.size // n, n):
            raise RuntimeError(lib().oracle_last_error().decode())
    return y, yi


def scatter(updates: np.ndarray, indices, params: dict, dtype_code: int) -> np.ndarray:
    """`runScatter` (src/routine.ts:226-296): updates and one int32 index array per indexed axis."""
    L = lib()
    updates = np.ascontiguousarray(updates)
    indices = [np.ascontiguousarray(i, dtype=np.int32) for i in indices]
    out = np.zeros(params["shape"], dtype=updates.dtype)
    i64 = lambda v: (ctypes.c_int64 * max(1, len(v)))(*v)
    i32 = lambda v: (ctypes.c_int32 * max(1, len(v)))(*v)
    ptrs = (ctypes.c_void_p * max(1, len(indices)))(*[i.ctypes.data for i in indices])
    flat = [d for i in indices for d in i.shape]
    L.oracle_scatter.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6
    L.oracle_scatter(dtype_code, int(params["op"] == "add"), int(bool(params["uniqueIndices"])), params["outDim"],
                     len(params["shape"]), i64(params["shape"]), updates.ndim, i64(updates.shape), len(indices),
                     i32(params["axis"]), i32([i.ndim for i in indices]), i64(flat), updates.ctypes.data, ptrs,
                     out.ctypes.data)
    return out


def _float_code(x: np.ndarray) -> int:
    from jax_js_b200.alu import DType
    return int({np.dtype(np.float32): DType.Float32, np.dtype(np.float64): DType.Float64}[x.dtype])


def triangular_solve(a: np.ndarray, b: np.ndarray, unit_diagonal: bool = False) -> np.ndarray:
    """`runTriangularSolve` (src/routine.ts:298-338): a [..., n, n] upper triangular, b [..., rows, n]."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    n, rows = a.shape[-1], b.shape[-2]
    x = np.empty_like(b)
    L = lib()
    L.oracle_triangular_solve.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3 + [ctypes.c_int]
    if a.size and L.oracle_triangular_solve(_float_code(a), a.ctypes.data, b.ctypes.data, x.ctypes.data,
                                            a.size // (n * n), rows, n, int(unit_diagonal)):
        raise RuntimeError("oracle_triangular_solve: unsupported dtype")
    return x


def cholesky(x: np.ndarray) -> np.ndarray:
    """`runCholesky` (src/routine.ts:340-366)."""
    x = np.ascontiguousarray(x)
    n = x.shape[-1]
    y = np.empty_like(x)
    L = lib()
    L.oracle_cholesky.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
    if x.size and L.oracle_cholesky(_float_code(x), x.ctypes.data, y.ctypes.data, x.size // (n * n), n):
        raise RuntimeError("oracle_cholesky: unsupported dtype")
    return y


def lu(a: np.ndarray):
    """`runLU` (src/routine.ts:368-432): returns (lu, pivots int32 [..., min(m, n)], permutation int32 [..., m])."""
    a = np.ascontiguousarray(a)
    m, n = a.shape[-2:]
    batch = a.size // (m * n) if m * n else 0
    out = np.empty_like(a)
    piv = np.zeros(a.shape[:-2] + (min(m, n),), np.int32)
    perm = np.zeros(a.shape[:-2] + (m,), np.int32)
    L = lib()
    L.oracle_lu.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 3
    if a.size and L.oracle_lu(_float_code(a), a.ctypes.data, out.ctypes.data, piv.ctypes.data, perm.ctypes.data, batch, m, n):
        raise RuntimeError("oracle_lu: unsupported dtype")
    return out, piv, perm


def jacobi_eigh(x: np.ndarray, max_sweeps: int, tolerance: float):
    """`runJacobiEigh` (src/routine.ts:434-541): returns (diagonalized, vectors), both [..., n, n]."""
    x = np.ascontiguousarray(x)
    n = x.shape[-1]
    a, v = np.empty_like(x), np.empty_like(x)
    L = lib()
    L.oracle_jacobi_eigh.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 2 + [ctypes.c_int, ctypes.c_double]
    if x.size and L.oracle_jacobi_eigh(_float_code(x), x.ctypes.data, a.ctypes.data, v.ctypes.data, x.size // (n * n), n,
                                       int(max_sweeps), float(tolerance)):
        raise RuntimeError("oracle_jacobi_eigh: unsupported dtype")
    return a, v


def fft(real: np.ndarray, imag: np.ndarray, factors, inverse: bool = False):
    """`runFft` (src/routine.ts:543-624) along the last axis; `factors` multiply to its length."""
    real, imag = np.ascontiguousarray(real), np.ascontiguousarray(imag)
    n = real.shape[-1]
    out_r, out_i = np.empty_like(real), np.empty_like(imag)
    f = (ctypes.c_int * max(1, len(factors)))(*factors)
    L = lib()
    L.oracle_fft.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 2 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    if real.size and L.oracle_fft(_float_code(real), real.ctypes.data, imag.ctypes.data, out_r.ctypes.data, out_i.ctypes.data,
                                  real.size // n, n, f, len(factors), int(inverse)):
        raise RuntimeError("oracle_fft: unsupported dtype")
    return out_r, out_i


def wasm_unary(op: int, x: float) -> float:
    return float(lib().oracle_wasm_unary(int(op), float(x)))


def threefry2x32(k0, k1, c0, c1):
    out = (ctypes.c_uint32 * 2)()
    lib().oracle_threefry2x32(k0, k1, c0, c1, out)
    return int(out[0]), int(out[1])
