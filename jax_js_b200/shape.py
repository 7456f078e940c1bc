"""Lazy views lowered to flat index expressions.

Host-side mirror of the part of src/shape.ts the backend boundary depends on:
a strided/masked `View` (shape.ts:168), its lowering to an index and a validity
expression (shape.ts:277-300 `toAluExp`), a `ShapeTracker` as a stack of views
(shape.ts:312: a movement that one view cannot express, such as reshaping a
permuted or padded array, starts a new view over the flattened previous one),
`unravelAlu` (shape.ts:631) and `accessorGlobal` (src/alu.ts:1664-1679).
"""
from __future__ import annotations

from typing import Sequence

from .alu import AluExp, DType


def _contiguous_strides(shape: Sequence[int]) -> tuple:
    strides, acc = [], 1
    for d in reversed(shape):
        strides.append(acc if d != 1 else 0)
        acc *= d
    return tuple(reversed(strides))


class View:
    """Shape, strides, offset and an optional per-axis valid mask."""

    def __init__(self, shape, strides, offset=0, mask=None):
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)
        self.mask = tuple(mask) if mask is not None else None

    @staticmethod
    def from_shape(shape: Sequence[int]) -> "View":
        return View(shape, _contiguous_strides(shape))

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def data_range(self) -> tuple:
        """Half-open range of flat offsets the view can touch (shape.ts:252-274)."""
        lo = hi = self.offset
        for i, (d, s) in enumerate(zip(self.shape, self.strides)):
            a, b = (self.mask[i] if self.mask else (0, d))
            if b <= a:
                return (0, 0)
            ends = (s * a, s * (b - 1))
            lo += min(ends)
            hi += max(ends)
        return (lo, hi + 1)

    def permute(self, axes: Sequence[int]) -> "View":
        return View([self.shape[a] for a in axes], [self.strides[a] for a in axes],
                            self.offset, [self.mask[a] for a in axes] if self.mask else None)

    def expand(self, shape: Sequence[int]) -> "View":
        strides, mask = [], []
        for i, (old, new) in enumerate(zip(self.shape, shape)):
            if old != new and old != 1:
                raise ValueError(f"cannot expand {self.shape} to {tuple(shape)}")
            strides.append(self.strides[i] if old == new else 0)
            if self.mask:
                mask.append(self.mask[i] if old == new else (0, new))
        return View(shape, strides, self.offset, mask if self.mask else None)

    def flip(self, axes: Sequence[bool]) -> "View":
        strides, offset, mask = list(self.strides), self.offset, list(self.mask) if self.mask else None
        for i, f in enumerate(axes):
            if f:
                offset += (self.shape[i] - 1) * strides[i]
                strides[i] = -strides[i]
                if mask:
                    a, b = mask[i]
                    mask[i] = (self.shape[i] - b, self.shape[i] - a)
        return View(self.shape, strides, offset, mask)

    def pad(self, widths: Sequence[tuple]) -> "View":
        shape, offset, mask = [], self.offset, []
        for i, (lo, hi) in enumerate(widths):
            a, b = (self.mask[i] if self.mask else (0, self.shape[i]))
            shape.append(self.shape[i] + lo + hi)
            offset -= lo * self.strides[i]
            mask.append((a + lo, b + lo))
        return View(shape, self.strides, offset, mask)

    def shrink(self, ranges: Sequence[tuple]) -> "View":
        shape, offset, mask = [], self.offset, []
        for i, (lo, hi) in enumerate(ranges):
            shape.append(hi - lo)
            offset += lo * self.strides[i]
            if self.mask:
                a, b = self.mask[i]
                mask.append((max(a - lo, 0), min(b - lo, hi - lo)))
        return View(shape, self.strides, offset, mask if self.mask else None)

    def reshape(self, shape: Sequence[int]) -> "View":
        """Reshape without copying; only the cases one view can express
        (merge/split of axes whose strides nest, and unit axes)."""
        shape = tuple(int(s) for s in shape)
        if self.mask:
            raise ValueError("reshape of a masked view needs a second view")
        old = [(d, s) for d, s in zip(self.shape, self.strides) if d != 1]
        strides = []
        i = 0
        for d in shape:
            if d == 1:
                strides.append(0)
                continue
            if i >= len(old):
                raise ValueError(f"cannot reshape {self.shape} to {shape}")
            od, os_ = old[i]
            if od == d:
                strides.append(os_)
                i += 1
            elif od % d == 0:                      # split an axis
                strides.append(os_ * (od // d))
                old[i] = (od // d, os_)
            else:                                  # merge following axes
                acc, j = od, i
                while acc < d and j + 1 < len(old):
                    nd, ns = old[j + 1]
                    if old[j][1] != ns * nd:
                        raise ValueError(f"cannot reshape {self.shape} to {shape} in one view")
                    acc *= nd
                    j += 1
                if acc != d:
                    raise ValueError(f"cannot reshape {self.shape} to {shape}")
                strides.append(old[j][1])
                i = j + 1
        if i != len(old):
            raise ValueError(f"cannot reshape {self.shape} to {shape}")
        return View(shape, strides, self.offset)

    def to_alu_exp(self, idxs: Sequence[AluExp]) -> tuple:
        """(flat index, valid) for the given per-axis indices (shape.ts:277-300)."""
        iexpr = AluExp.i32(self.offset)
        vexpr = AluExp.bool(True)
        for i in range(self.ndim - 1, -1, -1):
            idx = idxs[i]
            if self.shape[i] != 1 and self.strides[i] != 0:
                iexpr = AluExp.add(AluExp.mul(idx, AluExp.i32(self.strides[i])), iexpr)
            if self.mask:
                a, b = self.mask[i]
                if a != 0:
                    vexpr = AluExp.mul(AluExp.cmplt(idx, AluExp.i32(a)).not_(), vexpr)
                if b != self.shape[i]:
                    vexpr = AluExp.mul(AluExp.cmplt(idx, AluExp.i32(b)), vexpr)
        return iexpr, vexpr


class ShapeTracker:
    """A stack of views (shape.ts:312-420).  The first view addresses the buffer; every later one
    indexes the flattened shape of the view before it.  Movement operations act on the last view;
    a reshape that the last view cannot express pushes a contiguous view of the new shape."""

    def __init__(self, shape=None, strides=None, offset=0, mask=None, views=None):
        self.views = list(views) if views is not None else [View(shape, strides, offset, mask)]

    @staticmethod
    def from_shape(shape: Sequence[int]) -> "ShapeTracker":
        return ShapeTracker(views=[View.from_shape(shape)])

    # the last view is what the tracker looks like from outside
    @property
    def shape(self) -> tuple:
        return self.views[-1].shape

    @property
    def strides(self) -> tuple:
        return self.views[-1].strides

    @property
    def offset(self) -> int:
        return self.views[-1].offset

    @property
    def mask(self):
        return self.views[-1].mask

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def data_range(self) -> tuple:
        """Flat offsets of the buffer that can be touched: only the first view addresses it."""
        if len(self.views) == 1:
            return self.views[0].data_range()
        lo, hi = self.views[0].data_range()
        return (min(lo, 0), hi)

    def _with_last(self, view: View) -> "ShapeTracker":
        return ShapeTracker(views=self.views[:-1] + [view])

    def permute(self, axes: Sequence[int]) -> "ShapeTracker":
        return self._with_last(self.views[-1].permute(axes))

    def expand(self, shape: Sequence[int]) -> "ShapeTracker":
        return self._with_last(self.views[-1].expand(shape))

    def flip(self, axes: Sequence[bool]) -> "ShapeTracker":
        return self._with_last(self.views[-1].flip(axes))

    def pad(self, widths: Sequence[tuple]) -> "ShapeTracker":
        return self._with_last(self.views[-1].pad(widths))

    def shrink(self, ranges: Sequence[tuple]) -> "ShapeTracker":
        return self._with_last(self.views[-1].shrink(ranges))

    def reshape(self, shape: Sequence[int]) -> "ShapeTracker":
        shape = tuple(int(d) for d in shape)
        size = 1
        for d in self.shape:
            size *= d
        new = 1
        for d in shape:
            new *= d
        if new != size:
            raise ValueError(f"cannot reshape {self.shape} to {shape}")
        try:
            return self._with_last(self.views[-1].reshape(shape))
        except ValueError:
            return ShapeTracker(views=self.views + [View.from_shape(shape)])

    def to_alu_exp(self, idxs: Sequence[AluExp]) -> tuple:
        """(flat index into the buffer, valid) for per-axis indices of the last view (shape.ts:404-420)."""
        iexpr, vexpr = self.views[-1].to_alu_exp(idxs)
        for view in reversed(self.views[:-1]):
            iexpr, valid = view.to_alu_exp(unravel_alu(view.shape, iexpr))
            vexpr = AluExp.mul(vexpr, valid)
        return iexpr, vexpr


def unravel_alu(shape: Sequence[int], offset: AluExp) -> list:
    """Per-axis indices of a flat offset (shape.ts:631-640)."""
    acc, idxs = 1, []
    for d in reversed(shape):
        idxs.append(AluExp.mod(AluExp.idiv(offset, AluExp.i32(acc)), AluExp.i32(d)))
        acc *= d
    return list(reversed(idxs))


def accessor_global(dtype: DType, gid: int, st: ShapeTracker, indices: Sequence[AluExp]) -> AluExp:
    """Guarded load of argument `gid` through a view (alu.ts:1664-1679)."""
    index, valid = st.to_alu_exp(indices)
    _, length = st.data_range()
    load = AluExp.global_index(dtype, gid, length, index)
    if valid.op.name == "Const" and valid.arg == 1:
        return load
    return AluExp.where(valid, load, AluExp.const(dtype, 0))


#: `AluExp.globalView` is lowered on construction here, since GlobalView nodes
#: never cross the backend boundary (alu.ts:1355-1362 `rewriteGlobalViews`).
global_view = accessor_global
