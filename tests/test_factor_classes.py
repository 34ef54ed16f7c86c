"""Update factors per distance class (host functions, no GPU): lut[class(i, j)] must equal the N x N table of the
reference's TrainerCommon loop, which the golden fixtures pin to the reference's own classes, bit for bit."""
import ctypes as C

import numpy as np
import pytest

from pink_b200 import capi, engine


def _table_from_classes(layout, dim0, dim1, dim2, lut):
    n = dim0 * dim1 * dim2 if layout == capi.LAYOUT_CARTESIAN else engine.som_size(layout, dim0, dim1)
    xyz = np.empty((n, 4), np.int16)
    assert capi.lib.pink_b200_som_coordinates(layout, dim0, dim1, dim2, xyz.ctypes.data_as(C.c_void_p)) == capi.OK
    p = xyz.astype(np.int64)
    d = p[:, None, :] - p[None, :, :]
    if layout == capi.LAYOUT_HEXAGONAL:
        dx, dy = d[..., 0], d[..., 1]
        cls = np.where((dx >= 0) == (dy >= 0), np.abs(dx + dy), np.maximum(np.abs(dx), np.abs(dy)))
    else:
        cls = (np.abs(d[..., 2]) * dim0 + np.abs(d[..., 1])) * dim1 + np.abs(d[..., 0])
    return lut[cls]


@pytest.mark.parametrize("case", [(0, 10, 10, 1), (0, 3, 7, 1), (0, 7, 3, 1), (1, 9, 9, 1), (1, 61, 61, 1),
                                  (0, 3, 4, 5), (0, 4, 3, 2)])
@pytest.mark.parametrize("func", [capi.FUNC_GAUSSIAN, capi.FUNC_MEXICAN_HAT, capi.FUNC_STEP])
def test_class_table_equals_full_table(case, func):
    layout, dim0, dim1, dim2 = case
    p0, p1, cut = (1.5, 0.3, -1.0) if func != capi.FUNC_STEP else (2.0, 0.0, 3.5)
    n_cls = capi.lib.pink_b200_distance_classes(layout, dim0, dim1, dim2, None, 0)
    assert n_cls > 0
    lut = np.empty(n_cls, np.float32)
    assert capi.lib.pink_b200_update_lut(layout, dim0, dim1, dim2, func, p0, p1, cut, lut.ctypes.data_as(C.c_void_p), n_cls) == capi.OK
    got = _table_from_classes(layout, dim0, dim1, dim2, lut)
    N = got.shape[0]
    want = np.empty((N, N), np.float32)
    if dim2 > 1:
        assert capi.lib.pink_b200_update_factors_3d(dim0, dim1, dim2, func, p0, p1, cut, want.ctypes.data_as(C.c_void_p)) == capi.OK
    else:
        assert capi.lib.pink_b200_update_factors(layout, dim0, dim1, func, p0, p1, cut, want.ctypes.data_as(C.c_void_p)) == capi.OK
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_class_distances_and_errors():
    d = engine.distance_classes(capi.LAYOUT_HEXAGONAL, 7, 7)
    assert d.tolist() == [0, 1, 2, 3, 4, 5, 6]
    d = engine.distance_classes(capi.LAYOUT_CARTESIAN, 2, 3)
    assert np.allclose(d, [0, 1, 2, 1, np.sqrt(2), np.sqrt(5)])
    assert capi.lib.pink_b200_distance_classes(capi.LAYOUT_HEXAGONAL, 6, 6, 1, None, 0) == 0      # even side
    assert capi.lib.pink_b200_distance_classes(capi.LAYOUT_HEXAGONAL, 7, 7, 2, None, 0) == 0      # no third dimension
