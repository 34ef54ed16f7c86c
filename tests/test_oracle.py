"""Pins the CPU oracle (oracle/pink_oracle.c) before anything trusts it:

1. every literal known-answer vector the reference's own unit tests hold for this path (cited per test);
2. bit-exact agreement with outputs of the reference's own CPU implementation on seeded inputs
   (tests/golden/reference_cpu.npz, produced by tests/golden/make_golden.py);
3. internal consistency of the integer-mode restatement (the reference has no CPU integer mode).
"""
import os

import numpy as np
import pytest

import oracle as O

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---- 1. literal vectors of the reference's tests --------------------------------------------

def test_rotated_images_2d_literal():
    """test/SelfOrganizingMapTest/generate_rotated_images.cpp:15-28"""
    rot = O.rotation_set(np.array([[1, 2], [3, 4]], np.float32), 2, 4, False)
    assert rot.ravel().tolist() == [1, 2, 3, 4, 3, 1, 4, 2, 4, 3, 2, 1, 2, 4, 1, 3]


def test_rotated_images_3d_literal():
    """test/SelfOrganizingMapTest/generate_rotated_images.cpp:30-43"""
    rot = O.rotation_set(np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2), 2, 4, False)
    assert rot.ravel().tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 3, 1, 4, 2, 7, 5, 8, 6, 4, 3, 2, 1, 8, 7, 6, 5,
                                    2, 4, 1, 3, 6, 8, 5, 7]


def test_quarter_turn_list_literal():
    """test/CudaTest/rotate_90_degrees_list.cu:16-29: quadrant q+1 is the exact quarter turn of quadrant q."""
    rot = O.rotation_set(np.array([[1, 2], [3, 4]], np.float32), 2, 4, False)
    assert rot[1].ravel().tolist() == [3, 1, 4, 2]


def test_resize_literals():
    """test/ImageProcessingTest/resize.cpp:15-35 and test/CudaTest/resize.cu:16-39 (slot 0 of the rotation set)."""
    big = O.rotation_set(np.array([[1, 2], [3, 4]], np.float32), 4, 1, False)
    assert big.ravel().tolist() == [0, 0, 0, 0, 0, 1, 2, 0, 0, 3, 4, 0, 0, 0, 0, 0]
    small = O.rotation_set(np.arange(1, 17, dtype=np.float32).reshape(4, 4), 2, 1, False)
    assert small.ravel().tolist() == [6, 7, 10, 11]


@pytest.mark.parametrize("src_dim", [1, 2])
def test_rotate_45_degrees_of_constant_image(src_dim):
    """test/ImageProcessingTest/rotate.cpp:24-62: only the centre pixel of the 3x3 output is covered.
    R = 8 makes slot 1 the 45 degree rotation."""
    rot = O.rotation_set(np.ones((src_dim, src_dim), np.float32), 3, 8, False)
    want = np.zeros(9, np.float32)
    want[4] = 1.0
    np.testing.assert_allclose(rot[1].ravel(), want, atol=1e-4)


@pytest.mark.parametrize("layout,a,b,ed,want", [
    ((2, 2), [0, 0, 0, 0], [1, 0, 0, 0], 2, 1),
    ((3, 3), [0] * 9, [0, 0, 1, 0, 0, 1, 1, 1, 1], 2, 0),
    ((4, 4), [0] * 16, [1, 1, 1, 1, 1, 0, 0, 1, 1, 0, 0, 1, 1, 1, 1, 1], 2, 0),
    ((2, 2, 2), [0] * 8, [1, 1, 1, 1, 1, 0, 0, 1], 2, 6),
    ((2, 4, 4), [0] * 32, [0, 0, 0, 0, 0, 1, 1, 0, 0, 1, 1, 0, 0, 0, 0, 0] * 2, 2, 8),
])
def test_euclidean_distance_literals(layout, a, b, ed, want):
    """test/SelfOrganizingMapTest/euclidean_distance.cpp:16-69, incl. the centred-region semantics."""
    shape = (1, 1) + layout if len(layout) == 2 else (1,) + layout
    dist, best = O.distance_f32(np.array(a, np.float32).reshape(shape), np.array(b, np.float32).reshape(shape), ed)
    assert dist[0] == want and best[0] == 0


MAPPER_TABLE = [  # test/SelfOrganizingMapTest/Mapper.cpp:80-98
    (1, 2, 2, 2, 1, False, 0.0, 1.0, 2.0), (1, 3, 3, 2, 1, False, 0.0, 1.0, 2.0), (1, 3, 5, 2, 360, False, 0.0, 1.0, 2.0),
    (2, 3, 5, 2, 360, False, 0.0, 1.0, 2.0), (2, 3, 5, 2, 360, True, 0.0, 1.0, 2.0), (1, 2, 2, 2, 1, False, 1.0, 0.0, 2.0),
    (1, 3, 3, 2, 1, False, 1.0, 0.0, 2.0), (1, 3, 5, 2, 360, False, 1.0, 0.0, 2.0), (2, 3, 5, 2, 360, False, 1.0, 0.0, 2.0),
    (2, 3, 5, 2, 360, True, 1.0, 0.0, 2.0), (1, 2, 2, 2, 1, False, 0.0, 0.5, 1.0), (1, 2, 2, 2, 1, False, 0.5, 0.0, 1.0),
    (1, 2, 2, 2, 1, False, 0.5, 0.5, 0.0), (2, 2, 2, 2, 1, False, 0.0, 0.5, 1.0), (2, 2, 2, 2, 1, False, 0.5, 0.0, 1.0),
]


@pytest.mark.parametrize("row", MAPPER_TABLE)
def test_mapper_table_float(row):
    """test/SelfOrganizingMapTest/Mapper.cpp:62-100: exact float results of the CPU Mapper."""
    som_dim, nd, idim, ed, R, flip, nv, iv, want = row
    som = np.full((som_dim * som_dim, 1, nd, nd), nv, np.float32)
    dist, _ = O.map_image(som, np.full((idim, idim), iv, np.float32), ed, R, flip, O.MODE_F32)
    assert dist.tolist() == [want] * (som_dim * som_dim)


@pytest.mark.parametrize("row", [(1, 2, 2, 2, 1, False), (1, 3, 3, 2, 1, False), (1, 3, 3, 2, 360, False),
                                 (2, 3, 3, 2, 360, False), (2, 3, 3, 2, 360, True)])
@pytest.mark.parametrize("mode", [O.MODE_F32, O.MODE_U8, O.MODE_U16])
def test_mapper_table_all_modes(row, mode):
    """test/CudaTest/mapper.cu:55-120: image = 0, SOM = 1 maps to exactly 2.0 in float, uint8 and uint16."""
    som_dim, nd, idim, ed, R, flip = row
    som = np.ones((som_dim * som_dim, 1, nd, nd), np.float32)
    dist, _ = O.map_image(som, np.zeros((idim, idim), np.float32), ed, R, flip, mode)
    assert dist.tolist() == [2.0] * (som_dim * som_dim)


def test_trainer_step_function_literal():
    """test/SelfOrganizingMapTest/Trainer.cpp:66-88: step neighbourhood copies the centre crop."""
    som = np.zeros((1, 1, 2, 2), np.float32)
    F = O.update_factors(O.LAYOUT_CARTESIAN, 1, 1, O.FUNC_STEP, 10.0)
    O.train_step(som, np.arange(1, 17, dtype=np.float32).reshape(4, 4), F, 2, 1, False, O.MODE_F32)
    assert som.ravel().tolist() == [6, 7, 10, 11]


def test_trainer_gaussian_literal():
    """test/SelfOrganizingMapTest/Trainer.cpp:44-64 (the reference's int instantiation truncates to 290)."""
    som = np.zeros((4, 1, 2, 2), np.float32)
    F = O.update_factors(O.LAYOUT_CARTESIAN, 2, 2, O.FUNC_GAUSSIAN, 1.1, 0.2, 0.0)
    O.train_step(som, np.array([[1000, 2000], [3000, 4000]], np.float32), F, 2, 1, False, O.MODE_F32)
    assert int(som[0, 0, 1, 1]) == 290


def test_trainer_3d_literals():
    """test/SelfOrganizingMapTest/Trainer.cpp:90-151"""
    som = np.zeros((4, 2, 2, 2), np.float32)
    som[1] = np.array([4, 3, 2, 1, 8, 7, 6, 5], np.float32).reshape(2, 2, 2)
    F = O.update_factors(O.LAYOUT_CARTESIAN, 2, 2, O.FUNC_STEP, 0.0)
    O.train_step(som, np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2), F, 2, 4, False, O.MODE_F32)
    assert som[1].ravel().tolist() == [4, 3, 2, 1, 8, 7, 6, 5]
    som = np.zeros((4, 2, 4, 4), np.float32)
    O.train_step(som, np.arange(1, 33, dtype=np.float32).reshape(2, 4, 4), F, 4, 4, False, O.MODE_F32)
    assert not som[1].any()


def test_update_neurons_literal():
    """test/CudaTest/update_neurons.cu:16-41"""
    som = np.zeros((4, 4), np.float32)
    rot = np.arange(1, 9, dtype=np.float32).reshape(2, 4)
    dist = np.array([2, 1, 3, 4], np.float32)
    bmu = int(O.lib.pko_bmu_f32(dist.ctypes.data_as(O.C.c_void_p), 4))
    assert bmu == 1
    O.update(som, rot, np.array([0, 1, 0, 0], np.uint32), bmu, np.eye(4, dtype=np.float32))
    assert som.ravel().tolist() == [0, 0, 0, 0, 5, 6, 7, 8, 0, 0, 0, 0, 0, 0, 0, 0]


def test_hexagonal_layout_literals():
    """test/SelfOrganizingMapTest/Hexagonal.cpp:15-53"""
    assert [int(O.lib.pko_hexagonal_size(d)) for d in (3, 5, 7)] == [7, 19, 37]
    d = lambda i, j: O.lib.pko_hexagonal_distance(i, j, 3)
    assert d(3, 3) == 0.0 and d(3, 4) == 1.0 and d(3, 1) == 1.0 and d(4, 3) == 1.0
    assert d(2, 5) == 1.0 and d(5, 2) == 1.0 and d(0, 5) == 2.0


def test_cartesian_layout_literals():
    """test/SelfOrganizingMapTest/Cartesian.cpp:15-26"""
    d = lambda i, j: O.lib.pko_cartesian_distance(i, j, 10, 10)
    assert d(0, 0) == 0.0 and d(0, 10) == 1.0 and d(0, 20) == 2.0
    assert abs(d(0, 11) - np.float32(np.sqrt(2.0))) < 1e-7 and abs(d(0, 22) - np.float32(np.sqrt(8.0))) < 1e-7


def test_distribution_functor_values():
    """test/UtilitiesTest/DistributionFunctorTest.cpp:28-71"""
    assert abs(O.lib.pko_gaussian(9.0, 1.2, 1.0) - 2.028607587901271e-13) < 1e-6
    for sigma in (1.0, 2.0, 0.5):
        assert abs(O.lib.pko_gaussian(0.0, sigma, 1.0) - 1.0 / (sigma * np.sqrt(2 * np.pi))) < 1e-6
        assert abs(O.lib.pko_gaussian(sigma, sigma, 1.0) - 1.0 / (sigma * np.sqrt(2 * np.pi * np.e))) < 1e-6
        want = 2.0 / np.sqrt(3.0 * sigma * np.sqrt(np.pi))
        assert abs(O.lib.pko_mexican_hat(0.0, sigma, 1.0) - want) < 1e-6
        assert abs(O.lib.pko_mexican_hat(1.0, sigma, 1.0)
                   - want * (1 - 1 / sigma ** 2) * np.exp(-1 / (2 * sigma ** 2))) < 1e-6


def test_uint8_scale_constant():
    """test/UtilitiesTest/ipowTest.cpp:18-22: 255^2 = 65025; S = 65025 reports distance 1."""
    assert O.lib.pko_scaled_distance(65025, O.MODE_U8) == 1.0
    assert O.lib.pko_scaled_distance(65535 * 65535, O.MODE_U16) == 1.0


# ---- 2. the reference's own CPU implementation on seeded inputs --------------------------------

@pytest.mark.parametrize("i", range(8))
def test_rotation_set_matches_reference(i):
    C, idim, nd, R, flip = GOLD["rot%d_cfg" % i]
    got = O.rotation_set(GOLD["rot%d_img" % i], int(nd), int(R), bool(flip))
    assert np.array_equal(bits(got), bits(GOLD["rot%d_out" % i]))


@pytest.mark.parametrize("i", range(6))
def test_train_and_map_match_reference(i):
    lay, s0, s1, C, idim, nd, ed, R, flip, n, func = (int(v) for v in GOLD["step%d_cfg" % i])
    p0, p1, md = (float(v) for v in GOLD["step%d_par" % i])
    som0, imgs = GOLD["step%d_som" % i], GOLD["step%d_imgs" % i]
    F = O.update_factors(lay, s0, s1, func, p0, p1, md)
    som = som0.copy()
    counts = np.zeros(som.shape[0], np.uint32)
    for im in imgs:
        _, _, bmu = O.train_step(som, im, F, ed, R, bool(flip), O.MODE_F32)
        counts[bmu] += 1
    assert np.array_equal(bits(som), bits(GOLD["step%d_trained" % i]))
    assert np.array_equal(counts, GOLD["step%d_counts" % i])
    for k, im in enumerate(imgs):
        dist, rot = O.map_image(som0, im, ed, R, bool(flip), O.MODE_F32)
        assert np.array_equal(bits(dist), bits(GOLD["step%d_map_dist" % i][k]))
        assert np.array_equal(rot, GOLD["step%d_map_rot" % i][k])


@pytest.mark.parametrize("i", range(4))
def test_circular_region_matches_reference(i):
    """Circular distance region (2-D data layout): trained map and mapping results of the reference's CPU
    Trainer / Mapper with EuclideanDistanceShape::CIRCULAR, bit for bit."""
    lay, s0, s1, idim, nd, ed, R, flip, n = (int(v) for v in GOLD["circ%d_cfg" % i])
    som0, imgs = GOLD["circ%d_som" % i], GOLD["circ%d_imgs" % i]
    F = O.update_factors(lay, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    som = som0.copy()
    for im in imgs:
        O.train_step(som, im, F, ed, R, bool(flip), O.MODE_F32, shape=O.SHAPE_CIRCULAR)
    assert np.array_equal(bits(som), bits(GOLD["circ%d_trained" % i].reshape(som.shape)))
    for k, im in enumerate(imgs):
        dist, rot = O.map_image(som0, im, ed, R, bool(flip), O.MODE_F32, shape=O.SHAPE_CIRCULAR)
        assert np.array_equal(bits(dist), bits(GOLD["circ%d_map_dist" % i][k]))
        assert np.array_equal(rot, GOLD["circ%d_map_rot" % i][k])


def test_circular_region_literals():
    """test/SelfOrganizingMapTest/euclidean_distance.cpp:71-89: the circle inscribed in a 200 x 200 region of a
    300 x 300 neuron holds 31428 elements; test/SelfOrganizingMapTest/circular_ed.cpp:23-53: mapper known answers."""
    jb, je = O.circle_rows(300, 200)
    assert int((je - jb).sum()) == 31428
    assert jb.min() >= 50 and je.max() <= 250          # the circle stays inside the centred region
    img = np.zeros((4, 4), np.float32)
    img.flat[4] = 1.0
    som = np.zeros((4, 1, 4, 4), np.float32)
    som.flat[4], som.flat[18], som.flat[43], som.flat[61] = 1.0, 0.5, 0.8, 0.3
    dist, rot = O.map_image(som, img, 4, 4, False, O.MODE_F32, shape=O.SHAPE_CIRCULAR)
    np.testing.assert_allclose(dist, [0.0, 0.5, 0.2, 0.7], atol=0.01)
    assert list(rot) == [0, 1, 2, 3]
    # integer modes on the masked operands: the same elements are kept
    a = O.crop_quantize(np.ones((1, 1, 300, 300), np.float32), 200, O.MODE_U8, shape=O.SHAPE_CIRCULAR)
    assert int((a != 0).sum()) == 31428


@pytest.mark.parametrize("i", range(7))
def test_update_factors_match_reference(i):
    lay, d0, d1, func = (int(v) for v in GOLD["fac%d_cfg" % i])
    p0, p1, md = (float(v) for v in GOLD["fac%d_par" % i])
    assert np.array_equal(bits(O.update_factors(lay, d0, d1, func, p0, p1, md)), bits(GOLD["fac%d_out" % i]))


@pytest.mark.parametrize("i", range(4))
def test_update_factors_of_3d_soms_match_reference(i):
    *dims, func = (int(v) for v in GOLD["fac3d%d_cfg" % i])
    p0, p1, md = (float(v) for v in GOLD["fac3d%d_par" % i])
    assert np.array_equal(bits(O.update_factors_3d(dims, func, p0, p1, md)), bits(GOLD["fac3d%d_out" % i]))


@pytest.mark.skipif(not O.have_ref(), reason="reference-linked checker not built here")
def test_live_reference_agrees_on_fresh_seed():
    """Where the reference-linked library exists, also compare on inputs that are not in the fixture."""
    rng = np.random.default_rng(99)
    img = rng.random((18, 18), dtype=np.float32)
    assert np.array_equal(bits(O.rotation_set(img, 13, 20, True)), bits(O.ref_rotation_set(img, 13, 20, True)))
    som = rng.random((6, 1, 13, 13), dtype=np.float32)
    ref = O.RefSession(som, 0, 3, 2, 0, 18, 13, 9, 20, True)
    ref.train(img)
    mine = som.copy()
    O.train_step(mine, img, O.update_factors(0, 3, 2, 0, 1.1, 0.2), 9, 20, True, O.MODE_F32)
    assert np.array_equal(bits(mine), bits(ref.som()))


# ---- 3. integer-mode restatement ---------------------------------------------------------------

@pytest.mark.parametrize("mode,hi", [(O.MODE_U8, 256), (O.MODE_U16, 65536)])
def test_integer_distance_is_the_sum_of_squared_differences(mode, hi):
    rng = np.random.default_rng(hi)
    dt = np.uint8 if mode == O.MODE_U8 else np.uint16
    a = rng.integers(0, hi, (7, 123)).astype(dt)
    b = rng.integers(0, hi, (9, 123)).astype(dt)
    b[3] = b[1]
    S = O.distance_int(a, b, mode)
    want = ((a[:, None, :].astype(np.int64) - b[None, :, :].astype(np.int64)) ** 2).sum(-1).astype(np.uint64)
    assert np.array_equal(S, want)
    smin, best = O.min_over_transforms_int(S)
    assert np.array_equal(smin, want.min(1)) and np.array_equal(best, want.argmin(1))   # first minimum


def test_quantiser_truncates_and_saturates():
    """src/CudaLib/copy_and_transform_kernel.h:27-28: conversion truncates (0.999 * 255 -> 254)."""
    v = np.array([[[[0.0, 0.999], [1.0, 0.5]]]], np.float32)
    assert O.crop_quantize(v, 2, O.MODE_U8).ravel().tolist() == [0, 254, 255, 127]
    assert O.crop_quantize(v, 2, O.MODE_U16).ravel().tolist() == [0, 65469, 65535, 32767]
    out = np.array([[[[-0.5, 1.5], [2.0, 1e9]]]], np.float32)
    assert O.crop_quantize(out, 2, O.MODE_U8).ravel().tolist() == [0, 255, 255, 255]


def test_crop_offset_for_odd_margin():
    """offset = uint32((nd - ed) * 0.5): 44 -> 31 starts at 6 (not 7)."""
    plane = np.arange(44 * 44, dtype=np.float32).reshape(1, 1, 44, 44) / 4096.0
    got = O.crop_quantize(plane, 31, O.MODE_F32).reshape(31, 31)
    assert np.array_equal(got, plane[0, 0, 6:37, 6:37])


def test_reference_cuda_float_emulation_is_close_to_exact():
    """The reference's CUDA float (256-way partial sums, each divided by 255^2, then tree-summed) differs from
    S / 65025 by a few ulp at most: that is the width of the near-tie set documented for BMU comparisons."""
    rng = np.random.default_rng(4)
    worst = 0.0
    for _ in range(200):
        a = rng.integers(0, 256, 961).astype(np.uint8)
        b = rng.integers(0, 256, 961).astype(np.uint8)
        S = int(((a.astype(np.int64) - b) ** 2).sum())
        emu = O.lib.pko_ref_cuda_float(a.ctypes.data_as(O.C.c_void_p), b.ctypes.data_as(O.C.c_void_p),
                                       O.C.c_uint32(961), O.C.c_int(O.MODE_U8), O.C.c_uint32(256))
        worst = max(worst, abs(emu - S / 65025.0) / (S / 65025.0))
    assert worst < 4e-7


def test_mt19937_fill_matches_reference_fixture():
    """src/UtilitiesLib/Filler.h:16-25 random SOM initialisation, seeds 1234 (CLI default) and 5489."""
    from pink_b200.synthetic import mt19937_uniform
    assert np.array_equal(mt19937_uniform(4096, 1234), GOLD["fill_seed1234"])
    assert np.array_equal(mt19937_uniform(256, 5489), GOLD["fill_default"])
