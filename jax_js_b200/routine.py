"""`Routine`: a named, non-fusable backend operation (src/routine.ts:20-123)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

from .alu import DType


class Routines:
    """src/routine.ts:32-102.  The cuda backend implements every member."""
    Sort = "Sort"
    Argsort = "Argsort"
    Scatter = "Scatter"
    TriangularSolve = "TriangularSolve"
    Cholesky = "Cholesky"
    LU = "LU"
    JacobiEigh = "JacobiEigh"
    Fft = "Fft"


@dataclass
class RoutineType:
    """src/routine.ts:112-123."""
    input_shapes: Sequence[Sequence[int]]
    input_dtypes: Sequence[DType]
    output_shapes: Sequence[Sequence[int]]
    output_dtypes: Sequence[DType]


@dataclass
class Routine:
    name: str
    type: RoutineType
    params: Any = field(default=None)
