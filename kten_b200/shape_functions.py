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
