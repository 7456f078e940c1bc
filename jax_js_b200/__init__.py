"""B200-native `cuda` device backend for jax-js (host-side mirror of the reference's
backend boundary, src/backend.ts:158-211, over the C ABI of include/jaxcuda.h)."""
from .alu import AluExp, AluOp, AluVar, DType, Kernel, Reduction, byte_width, np_dtype  # noqa: F401
from .shape import ShapeTracker, accessor_global, global_view, unravel_alu  # noqa: F401
