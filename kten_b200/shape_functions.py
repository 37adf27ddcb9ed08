"""Host-side shape algebra of the RawTensor SPI (pure Python, no device work).

Restates the parts of kten-api's ShapeFunctions the hot path uses
(kten-api/src/main/kotlin/eu/redbean/kten/api/autograd/utils/ShapeFunctions.kt);
IllegalArgumentException maps to ValueError with the reference's wording.
"""
from __future__ import annotations

from typing import List, Sequence


def to_store_size(shape: Sequence[int]) -> int:
    """List<Int>.toStoreSize() (ShapeFunctions.kt:344): product of extents, 1 for []."""
    n = 1
    for d in shape:
        n *= int(d)
    return n


def reshape(shape: Sequence[int], new_shape: Sequence[int]) -> List[int]:
    """List<Int>.reshape (ShapeFunctions.kt:11-39): one -1 may be inferred."""
    new_shape = [int(d) for d in new_shape]
    if any(d < -1 for d in new_shape):
        raise ValueError(f"Invalid shape: {new_shape}")
    inferred = [i for i, d in enumerate(new_shape) if d == -1]
    if len(inferred) > 1:
        raise ValueError(f"Cannot reshape to {new_shape}. Only one dimension can be inferred")
    res = list(new_shape)
    if inferred:
        res[inferred[0]] = 1
    elements = to_store_size(shape)
    res_elements = to_store_size(res)
    if inferred:
        res[inferred[0]] = elements // res_elements if res_elements else 0
        res_elements = to_store_size(res)
    if elements != res_elements:
        raise ValueError(f"Cannot reshape tensor with shape: {list(shape)} to shape: {new_shape}")
    return res


def normalize_axis(shape: Sequence[int], axis: int) -> int:
    """List<Int>.normalizeAxis (ShapeFunctions.kt:41-48)."""
    res = len(shape) + axis if axis < 0 else axis
    if res < 0 or res >= len(shape):
        raise ValueError(f"Cannot address axis: {axis} in tensor with dimensions: {len(shape)}")
    return res


def squeeze(shape: Sequence[int], axis: int) -> List[int]:
    """List<Int>.squeeze (ShapeFunctions.kt:50-59)."""
    a = normalize_axis(shape, axis)
    if shape[a] != 1:
        raise ValueError(f"Cannot squeeze tensor with shape: {list(shape)} at axis: {axis}")
    res = list(shape)
    del res[a]
    return res


def unsqueeze(shape: Sequence[int], axis: int) -> List[int]:
    """List<Int>.unsqueeze (ShapeFunctions.kt:61-71): axis == size appends; negative
    axes count from the end of the result."""
    n = len(shape)
    if axis != n:
        if axis < 0:
            a = 0 if axis == -(n + 1) else normalize_axis(shape, axis) + 1
        else:
            a = normalize_axis(shape, axis)
    else:
        a = axis
    res = list(shape)
    res.insert(a, 1)
    return res


def aggregate_over(shape: Sequence[int], axis: int, keep_dimensions: bool) -> List[int]:
    """List<Int>.aggregateOver (ShapeFunctions.kt:73-83): a 1-D tensor keeps shape [1]."""
    a = normalize_axis(shape, axis)
    res = list(shape)
    res[a] = 1
    if not keep_dimensions and len(res) > 1:
        del res[a]
    return res


def infer_implicit_broadcast_shape(shape1: Sequence[int], shape2: Sequence[int]) -> List[int]:
    """inferImplicitBroadcastShape (ShapeFunctions.kt:168-185)."""
    n = max(len(shape1), len(shape2))
    e1 = [1] * (n - len(shape1)) + list(shape1)
    e2 = [1] * (n - len(shape2)) + list(shape2)
    out = []
    for a, b in zip(e1, e2):
        if a == b or a == 1 or b == 1:
            out.append(max(a, b))
        else:
            raise ValueError(
                f"Shape {e1} must match {e2} for every non-singleton dimensions (missing dimensions count as "
                "singleton dimension at the beginning of the shapes)")
    return out


def infer_explicit_broadcast_shape(shape: Sequence[int], target: Sequence[int]) -> List[int]:
    """List<Int>.inferExplicitBroadcastShape (ShapeFunctions.kt:187-201)."""
    if len(shape) > len(target):
        raise ValueError(f"Tensor with shape: {list(shape)} cannot be broadcasted to shape: {list(target)}")
    e = [1] * (len(target) - len(shape)) + list(shape)
    out = []
    for a, b in zip(e, target):
        if a == b or a == 1:
            out.append(max(a, b))
        else:
            raise ValueError(
                f"Shape {list(shape)} must match {list(target)} for every non-singleton dimensions (missing "
                "dimensions count as singleton dimension at the beginning of the shapes)")
    return out


def collapse_axis(shape: Sequence[int], axis: int):
    """[outer, axis_len, inner] view of a contiguous row-major tensor around `axis`
    (the strides of StoreIndexing, AbstractIndexing.kt:107-109)."""
    outer = to_store_size(shape[:axis])
    inner = to_store_size(shape[axis + 1:])
    return outer, int(shape[axis]), inner


def strides_of(shape: Sequence[int]) -> List[int]:
    """Row-major element strides (StoreIndexing.strides, AbstractIndexing.kt:107-109)."""
    res, st = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        res[i] = st
        st *= int(shape[i])
    return res


def concat_shapes(shapes: Sequence[Sequence[int]], axis: int) -> List[int]:
    """concatShapes (ShapeFunctions.kt:85-104)."""
    shapes = [list(s) for s in shapes]
    if len({len(s) for s in shapes}) == 1:
        a = normalize_axis(shapes[0], axis)
        if len({tuple(s[:a] + s[a + 1:]) for s in shapes}) == 1:
            res = list(shapes[0])
            res[a] = sum(s[a] for s in shapes)
            return res
    raise ValueError(f"Cannot concatenate tensors with shapes: {shapes} at axis: {axis} (All tensors must have the same number of "
                     "dimenisons, and have the same size at all dimenions except at the dimension indexed by the axis)")


def permute(shape: Sequence[int], axes: Sequence[int]) -> List[int]:
    """List<Int>.permute (ShapeFunctions.kt:106-113): result dimension i is input dimension axes[i]."""
    axes = [int(a) for a in axes]
    if len(shape) != len(axes) or not all(i in axes for i in range(len(shape))):
        raise ValueError(f"Tensor with shape: {list(shape)} cannot be permuted by axes: {axes}. All dimensions must be indexed.")
    return [int(shape[a]) for a in axes]


def transpose_normalize_axes(shape: Sequence[int], axis1: int, axis2: int):
    """List<Int>.transposeNormalizeAxes (ShapeFunctions.kt:115-129)."""
    a1, a2 = normalize_axis(shape, axis1), normalize_axis(shape, axis2)
    if a1 == a2:
        raise ValueError(f"Transpose requires different axes as parameters, but got {axis1} (normalized: {a1}) and {axis2} "
                         f"(normalized: {a2})")
    res = list(shape)
    res[a1], res[a2] = shape[a2], shape[a1]
    return res, a1, a2


def normalize_index(shape: Sequence[int], index: Sequence[int]) -> List[int]:
    """List<Int>.normalizeIndex(IntArray) (ShapeFunctions.kt:217-230)."""
    index = [int(i) for i in index]
    if len(index) > len(shape):
        raise ValueError(f"Cannot index tensor with shape: {list(shape)} with index: {index}")
    res = []
    for d, item in enumerate(index):
        n = shape[d] + item if item < 0 else item
        if n < 0 or n >= shape[d]:
            raise ValueError(f"Cannot index tensor with shape: {list(shape)} with index: {index}")
        res.append(n)
    return res


def normalized_indexed_shape(shape: Sequence[int], index: Sequence[int]):
    """List<Int>.normalizedIndexedShape(IntArray) (ShapeFunctions.kt:232-238): a full index selects a [1] tensor."""
    n = normalize_index(shape, index)
    return n, ([1] if len(n) == len(shape) else list(shape[len(n):]))


def as_range(r, extent: int):
    """One Kotlin IntRange as (first, last), both inclusive.  Accepted: None / slice(None) / ... (the
    reference's `all`), a slice with unit step (stop exclusive, as in Python), a range, or a
    (first, last) pair with the reference's inclusive meaning."""
    if r is None or r is Ellipsis or (isinstance(r, slice) and r.start is None and r.stop is None):
        return None
    if isinstance(r, slice):
        if r.step not in (None, 1):
            raise ValueError("only unit-step ranges index a tensor")
        first = 0 if r.start is None else int(r.start)
        if r.stop is None:
            last = extent - 1
        else:
            last = extent + int(r.stop) - 1 if r.stop < 0 else int(r.stop) - 1
        return first, last
    if isinstance(r, range):
        if r.step != 1 or len(r) == 0:
            raise ValueError("only non-empty unit-step ranges index a tensor")
        return int(r[0]), int(r[-1])
    first, last = r
    return int(first), int(last)


def normalize_index_ranges(shape: Sequence[int], index: Sequence) -> List[tuple]:
    """List<Int>.normalizeIndex(Array<IntRange>) (ShapeFunctions.kt:240-259): negative bounds count from
    the end; every range must lie inside its dimension."""
    if len(index) > len(shape):
        raise ValueError(f"Cannot index tensor with shape: {list(shape)} with index: {list(index)}")
    res = []
    for ext, r in zip(shape, index):
        fl = as_range(r, ext)
        if fl is None:
            first, last = 0, ext - 1
        else:
            first, last = fl
            if first < 0 or last < 0:
                first = ext + first if first < 0 else first
                last = ext + last if last < 0 else last
        if first < 0 or last < 0 or first >= ext or last >= ext or first > last:
            raise ValueError(f"Cannot index tensor with shape: {list(shape)} with index: {list(index)}")
        res.append((first, last))
    return res


def normalized_indexed_shape_ranges(shape: Sequence[int], index: Sequence):
    """List<Int>.normalizedIndexedShape(Array<IntRange>) (ShapeFunctions.kt:261-268)."""
    n = normalize_index_ranges(shape, index)
    return n, [l - f + 1 for f, l in n] + list(shape[len(n):])


def index_select_norm_axis_shape(shape: Sequence[int], axis: int, index_shape: Sequence[int]):
    """List<Int>.indexSelectNormAxisShape (ShapeFunctions.kt:270-278)."""
    a = normalize_axis(shape, axis)
    if len(index_shape) != 1:
        raise ValueError(f"Index select requires singleton tensor as index, but got index tensor with shape: {list(index_shape)}")
    res = list(shape)
    res[a] = int(index_shape[0])
    return a, res


def index_add_check_shapes_norm_axis(shape: Sequence[int], axis: int, index_shape: Sequence[int], src_shape: Sequence[int]) -> int:
    """List<Int>.indexAddCheckShapesNormAxis (ShapeFunctions.kt:280-293)."""
    if len(index_shape) != 1:
        raise ValueError(f"Index add requires index tensor to have 1 dimension, but got tensor with shape: {list(index_shape)}")
    a = normalize_axis(shape, axis)
    expected = list(shape)
    expected[a] = int(index_shape[0])
    if list(src_shape) != expected:
        raise ValueError("Index add expects source tensor to have same size as index size at the specified axis, and same size as "
                         f"this tensor for every other axis, but got source tensor with shape: {list(src_shape)} axis: {axis} and "
                         f"this tensor have shape: {list(shape)}")
    return a


def normalized_axis_scatter(shape: Sequence[int], axis: int, index_shape: Sequence[int], src_shape: Sequence[int]) -> int:
    """List<Int>.normalizedAxisScatter (ShapeFunctions.kt:346-371)."""
    if len(shape) != len(index_shape) or len(shape) != len(src_shape):
        raise ValueError("Scatter expects tensors (target, index, source) to have the same dimensions, but got tensors with shapes: "
                         f"target: {list(shape)}, index: {list(index_shape)}, source: {list(src_shape)}")
    a = normalize_axis(shape, axis)
    for d in range(len(shape)):
        if index_shape[d] > src_shape[d]:
            raise ValueError("Scatter requires that index.shape[a] <= src.shape[a] for all axis 'a', but got tensors with shapes: "
                             f"index: {list(index_shape)}, src: {list(src_shape)}")
        if d != a and index_shape[d] > shape[d]:
            raise ValueError("Scatter requires that index.shape[a] <= target.shape[a] for all axis 'a', except the specified 'axis' "
                             f"of the operation, but got tensors with shapes: index: {list(index_shape)}, target: {list(shape)}")
    return a
