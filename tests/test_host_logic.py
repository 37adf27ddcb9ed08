"""Host-side logic that needs no device: shape algebra and the data generator."""
import numpy as np
import pytest

from kten_b200 import datagen as D
from kten_b200 import shape_functions as SF


def test_reshape_infers_one_dimension():
    assert SF.reshape([2, 3, 4], [4, -1]) == [4, 6]
    assert SF.reshape([6], [2, 3]) == [2, 3]
    with pytest.raises(ValueError):
        SF.reshape([2, 3], [-1, -1])
    with pytest.raises(ValueError):
        SF.reshape([2, 3], [4, 2])
    with pytest.raises(ValueError):
        SF.reshape([2, 3], [-2, 3])


def test_normalize_axis_and_aggregate_over():
    assert SF.normalize_axis([2, 3, 4], -1) == 2
    with pytest.raises(ValueError):
        SF.normalize_axis([2, 3], 2)
    assert SF.aggregate_over([3, 4], 0, False) == [4]
    assert SF.aggregate_over([3, 4], 1, True) == [3, 1]
    assert SF.aggregate_over([5], 0, False) == [1]          # a 1-D tensor keeps shape [1]


def test_unsqueeze_axes():
    assert SF.unsqueeze([2, 3], 0) == [1, 2, 3]
    assert SF.unsqueeze([2, 3], 2) == [2, 3, 1]
    assert SF.unsqueeze([2, 3], -1) == [2, 3, 1]
    assert SF.unsqueeze([2, 3], -3) == [1, 2, 3]
    assert SF.unsqueeze([2, 3], 1) == [2, 1, 3]
    assert SF.squeeze([2, 1, 3], 1) == [2, 3]
    with pytest.raises(ValueError):
        SF.squeeze([2, 3], 0)


def test_broadcast_shapes():
    assert SF.infer_implicit_broadcast_shape([32, 64, 128], [64, 1]) == [32, 64, 128]
    assert SF.infer_implicit_broadcast_shape([1024, 1024, 256], [1, 1024, 1]) == [1024, 1024, 256]
    assert SF.infer_implicit_broadcast_shape([3, 1], [1, 4]) == [3, 4]
    with pytest.raises(ValueError):
        SF.infer_implicit_broadcast_shape([2, 3], [4, 3])
    assert SF.infer_explicit_broadcast_shape([1], [3, 3]) == [3, 3]
    with pytest.raises(ValueError):
        SF.infer_explicit_broadcast_shape([3, 3], [3])
    with pytest.raises(ValueError):
        SF.infer_explicit_broadcast_shape([2, 3], [3, 3])


def test_collapse_axis():
    assert SF.collapse_axis([65536, 4096], 1) == (65536, 4096, 1)
    assert SF.collapse_axis([512, 4096, 128], 1) == (512, 4096, 128)
    assert SF.collapse_axis([32, 64, 128], 0) == (1, 32, 64 * 128)
    assert SF.to_store_size([]) == 1


def test_generator_matches_its_numpy_restatement():
    for seed, stream, first in ((0, 0, 0), (1, 0, 12345), (2, 3, 1 << 33)):
        a = D.uniform(4096, seed, 0.1, 2.0, stream=stream, first=first)
        b = D.uniform_numpy(4096, seed, 0.1, 2.0, stream=stream, first=first)
        assert np.array_equal(a, b)
        assert a.min() >= np.float32(0.1) and a.max() <= np.float32(2.0)


def test_generator_is_counter_based():
    whole = D.normal(10000, 7, 0.0, 1.0, stream=2)
    part = D.normal(3000, 7, 0.0, 1.0, stream=2, first=2500)
    assert np.array_equal(whole[2500:5500], part)
    assert not np.array_equal(D.normal(100, 7, stream=0), D.normal(100, 7, stream=1))


def test_generator_distributions():
    x = D.normal(1 << 20, 3, 0.0, 1.0, quantum=16.0)
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 1.0) < 5e-3
    assert np.array_equal(x * 16, np.rint(x * 16))               # multiples of 1/16: ties will occur
    u = D.uniform(1 << 20, 4, -1.0, 1.0)
    assert abs(float(u.mean())) < 5e-3 and abs(float(u.var()) - 1.0 / 3.0) < 5e-3


# ---- shape algebra of indexing and data movement (ShapeFunctions.kt:85-129, 203-293, 346-371) ----------------
def test_index_normalisation_and_indexed_shapes():
    s = [4, 5, 6]
    assert SF.normalized_indexed_shape(s, [1]) == ([1], [5, 6])
    assert SF.normalized_indexed_shape(s, [-1, -5, 2]) == ([3, 0, 2], [1])          # a full index selects a [1] tensor
    for bad in ([4], [0, 5], [0, -6], [0, 0, 0, 0]):
        with pytest.raises(ValueError):
            SF.normalize_index(s, bad)
    assert SF.normalized_indexed_shape_ranges(s, [(1, 2), None]) == ([(1, 2), (0, 4)], [2, 5, 6])
    assert SF.normalized_indexed_shape_ranges(s, [(0, -1), (-2, -1), (3, 3)]) == ([(0, 3), (3, 4), (3, 3)], [4, 2, 1])
    assert SF.normalize_index_ranges(s, [slice(1, 3), slice(None), slice(2, None)]) == [(1, 2), (0, 4), (2, 5)]
    assert SF.normalize_index_ranges(s, [range(0, 4), slice(0, -1)]) == [(0, 3), (0, 3)]
    for bad in ([(2, 1)], [(0, 4)], [(-5, 0)], [None, None, None, None], [slice(0, 4, 2)]):
        with pytest.raises(ValueError):
            SF.normalize_index_ranges(s, bad)


def test_permute_transpose_concat_shapes():
    assert SF.permute([2, 3, 4], [2, 0, 1]) == [4, 2, 3]
    for bad in ([0, 1], [0, 1, 1], [0, 1, 3]):
        with pytest.raises(ValueError):
            SF.permute([2, 3, 4], bad)
    assert SF.transpose_normalize_axes([2, 3, 4], 0, -1) == ([4, 3, 2], 0, 2)
    with pytest.raises(ValueError):
        SF.transpose_normalize_axes([2, 3, 4], 1, -2)
    assert SF.concat_shapes([[2, 3], [1, 3], [4, 3]], 0) == [7, 3]
    assert SF.concat_shapes([[2, 3], [2, 5]], -1) == [2, 8]
    for bad in ([[2, 3], [2, 4]], [[2, 3], [2, 3, 1]]):
        with pytest.raises(ValueError):
            SF.concat_shapes(bad, 0)
    assert SF.strides_of([2, 3, 4]) == [12, 4, 1] and SF.strides_of([]) == []


def test_index_op_shape_checks():
    assert SF.index_select_norm_axis_shape([3, 4, 5], -2, [7]) == (1, [3, 7, 5])
    with pytest.raises(ValueError):
        SF.index_select_norm_axis_shape([3, 4, 5], 0, [2, 2])
    assert SF.index_add_check_shapes_norm_axis([3, 4, 5], 1, [2], [3, 2, 5]) == 1
    for idx_shape, src_shape in (([2, 1], [3, 2, 5]), ([2], [3, 3, 5]), ([2], [3, 2])):
        with pytest.raises(ValueError):
            SF.index_add_check_shapes_norm_axis([3, 4, 5], 1, idx_shape, src_shape)
    assert SF.normalized_axis_scatter([3, 5], -1, [2, 9], [2, 9]) == 1              # the axis itself may be longer than the target
    for idx_shape, src_shape in (([2], [2]), ([4, 5], [4, 5]), ([2, 5], [2, 4])):
        with pytest.raises(ValueError):
            SF.normalized_axis_scatter([3, 5], 1, idx_shape, src_shape)
