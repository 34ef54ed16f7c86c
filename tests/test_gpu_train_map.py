"""Whole-step parity through the context entry points of the C ABI (host
buffers in, host buffers out) against the CPU oracle."""
import numpy as np
import pytest

import oracle as O
from pink_b200.synthetic import blob_images
from util import Context, make_config

pytestmark = pytest.mark.gpu

TRAIN_CASES = [
    # layout, s0, s1, C, id, nd, ed, R, flip, n_images
    (0, 3, 3, 1, 16, 12, 7, 16, True, 4),
    (0, 2, 2, 1, 64, 45, 45, 360, True, 2),
    (1, 5, 5, 1, 20, 14, 9, 8, True, 5),
    (0, 3, 2, 2, 15, 10, 7, 12, True, 3),
    (0, 10, 10, 1, 64, 44, 31, 360, True, 6),
    (0, 2, 2, 1, 4, 2, 2, 1, False, 2),
    (0, 2, 2, 1, 2, 4, 4, 4, True, 2),
]


def _som_size(layout, s0, s1):
    return s0 * s1 if layout == 0 else int(O.lib.pko_hexagonal_size(s0))


@pytest.mark.parametrize("case", TRAIN_CASES)
@pytest.mark.parametrize("mode", [2, 1])
def test_train_integer_modes_bit_exact(cuda, case, mode):
    """uint8/uint16: BMU sequence, best rotations and the trained SOM equal the oracle's bit for bit."""
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(abs(hash(case)) % 2**32)
    som0 = rng.random((N, C_, nd, nd), dtype=np.float32)
    imgs = blob_images(n, idim, C_, seed=N + R) if idim >= 15 else rng.random((n, C_, idim, idim), dtype=np.float32)
    imgs = imgs.reshape(n, C_, idim, idim)
    F = O.update_factors(layout, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    want = som0.copy()
    want_bmu = []
    for i in range(n):
        _, _, bmu = O.train_step(want, imgs[i], F, ed, R, flip, mode)
        want_bmu.append(bmu)
    with Context(capi, make_config(capi, N, C_, idim, nd, ed, R, flip, mode)) as ctx:
        ctx.set_som(som0)
        ctx.set_factors(F)
        log = ctx.train(imgs)
        got = ctx.get_som(som0)
        counts = ctx.counts()
    assert list(log) == want_bmu
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert counts.sum() == n and all(counts[b] > 0 for b in want_bmu)


@pytest.mark.parametrize("case", [TRAIN_CASES[0], TRAIN_CASES[4], TRAIN_CASES[3]])
@pytest.mark.parametrize("mode", [2, 1, 0])
def test_step_kernels_agree(cuda, case, mode):
    """The three launch sequences of a training step -- whole batches in the persistent kernel, two kernels per
    image (distance + an update kernel that finds the best matching unit and its work list itself), and four
    kernels per image (distance, reduction, compaction, update) -- give the same SOM, BMU sequence and counters
    bit for bit."""
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(77)
    som0 = rng.random((N, C_, nd, nd), dtype=np.float32)
    n = 19                                              # more than one batch of the persistent kernel
    imgs = blob_images(n, idim, C_, seed=5).reshape(n, C_, idim, idim)
    F = O.update_factors(layout, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    out = []
    for step_kernel in (0, 1, 2):
        with Context(capi, make_config(capi, N, C_, idim, nd, ed, R, flip, mode), {"step_kernel": step_kernel}) as ctx:
            ctx.set_som(som0)
            ctx.set_factors(F)
            log = ctx.train(imgs)
            log2 = ctx.train(imgs[::-1].copy())
            out.append((list(log) + list(log2), ctx.get_som(som0).copy(), ctx.counts().copy(),
                        ctx.e.launch_count(), ctx.e.update_stats()))
    for other in out[1:]:
        assert out[0][0] == other[0]
        assert np.array_equal(out[0][1].view(np.uint32), other[1].view(np.uint32))
        assert np.array_equal(out[0][2], other[2])
    # the intended sequences really ran: one launch per batch, two or four per image
    if mode != 0 and (nd * nd) % 4 == 0:
        assert out[0][3] < out[1][3]
    assert out[1][3] <= out[2][3]
    # the split path rewrites every neuron with a non-zero factor; the others do not even read neurons that
    # provably cannot change and leave neurons whose values did not change unwritten (far from the best
    # matching unit of a 10 x 10 map the products vanish) -- with bit-identical maps, asserted above
    want_read = sum(int((F[bmu] != 0).sum()) for bmu in out[0][0])
    read_s, written_s = out[2][4]
    assert read_s == written_s == want_read
    for k in (0, 1):
        read_f, written_f = out[k][4]
        assert written_f <= read_f <= read_s
    if N == 100 and mode != 0:
        assert out[0][4][1] < read_s and out[0][4][0] < read_s


@pytest.mark.parametrize("case", TRAIN_CASES[:5])
def test_train_float_mode(cuda, case):
    """float32: one teacher-forced step at a time; the SOM must match the oracle bit for bit whenever
    BMU and rotations agree, which they must except at float near-ties (none in these seeds)."""
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(abs(hash(case)) % 2**32 + 1)
    som0 = rng.random((N, C_, nd, nd), dtype=np.float32)
    imgs = blob_images(n, idim, C_, seed=N + R + 1) if idim >= 15 else rng.random((n, C_, idim, idim), dtype=np.float32)
    imgs = imgs.reshape(n, C_, idim, idim)
    F = O.update_factors(layout, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    want = som0.copy()
    with Context(capi, make_config(capi, N, C_, idim, nd, ed, R, flip, 0)) as ctx:
        ctx.set_factors(F)
        for i in range(n):
            ctx.set_som(want)                       # teacher forcing: start every step from the oracle's state
            _, _, bmu = O.train_step(want, imgs[i], F, ed, R, flip, 0)
            log = ctx.train(imgs[i:i + 1])
            got = ctx.get_som(som0)
            assert log[0] == bmu
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-7)


CIRCLE_CASES = [
    # layout, s0, s1, C, id, nd, ed, R, flip, n_images
    (0, 3, 3, 1, 32, 22, 16, 8, True, 4),
    (0, 10, 10, 1, 64, 44, 32, 40, True, 4),       # pipelined update kernel
    (0, 2, 3, 2, 20, 15, 11, 12, True, 3),         # two channels, odd sizes: fallback update kernel
]


@pytest.mark.parametrize("case", CIRCLE_CASES)
@pytest.mark.parametrize("mode", [2, 1, 0])
def test_circular_distance_region(cuda, case, mode):
    """EuclideanDistanceShape::CIRCULAR: training (integer modes bit-exact, float within tolerance with teacher
    forcing) and mapping against the oracle, which is pinned to the reference's CPU code for this shape."""
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(1000 + nd + mode)
    som0 = rng.random((N, C_, nd, nd), dtype=np.float32)
    imgs = blob_images(n, idim, C_, seed=N + ed).reshape(n, C_, idim, idim)
    F = O.update_factors(layout, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    cfg = make_config(capi, N, C_, idim, nd, ed, R, flip, mode)
    cfg.ed_shape = capi.CIRCULAR
    with Context(capi, cfg) as ctx:
        ctx.set_factors(F)
        want = som0.copy()
        if mode != 0:
            ctx.set_som(som0)
            want_bmu = [O.train_step(want, im, F, ed, R, flip, mode, shape=O.SHAPE_CIRCULAR)[2] for im in imgs]
            log = ctx.train(imgs)
            assert list(log) == want_bmu
            assert np.array_equal(ctx.get_som(som0).view(np.uint32), want.view(np.uint32))
        else:
            for i in range(n):
                ctx.set_som(want)
                bmu = O.train_step(want, imgs[i], F, ed, R, flip, 0, shape=O.SHAPE_CIRCULAR)[2]
                assert ctx.train(imgs[i:i + 1])[0] == bmu
                np.testing.assert_allclose(ctx.get_som(som0), want, rtol=1e-5, atol=1e-7)
        ctx.set_som(som0)
        dist, rot = ctx.map(imgs)
    for i in range(n):
        wd, wr = O.map_image(som0, imgs[i], ed, R, flip, mode, shape=O.SHAPE_CIRCULAR)
        if mode != 0:
            assert np.array_equal(rot[i], wr)
            assert np.array_equal(dist[i].view(np.uint32), wd.view(np.uint32))
        else:
            np.testing.assert_allclose(dist[i], wd, rtol=1e-5, atol=1e-7)


MAP_CASES = [
    (0, 3, 3, 1, 16, 12, 7, 16, True, 5),
    (0, 4, 4, 1, 64, 44, 31, 360, True, 3),
    (0, 3, 2, 2, 15, 10, 7, 12, False, 70),      # more images than one internal batch
    (1, 3, 3, 1, 20, 14, 9, 8, True, 4),
]


@pytest.mark.parametrize("case", MAP_CASES)
@pytest.mark.parametrize("mode", [2, 1, 0])
def test_map(cuda, case, mode):
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(abs(hash(case)) % 2**32 + 2)
    som = rng.random((N, C_, nd, nd), dtype=np.float32)
    imgs = rng.random((n, C_, idim, idim), dtype=np.float32)
    with Context(capi, make_config(capi, N, C_, idim, nd, ed, R, flip, mode)) as ctx:
        ctx.set_som(som)
        dist, rot = ctx.map(imgs)
    for i in range(min(n, 6)):
        d, r = O.map_image(som, imgs[i], ed, R, flip, mode)
        if mode == 0:
            np.testing.assert_allclose(dist[i], d, rtol=1e-5)
            # the transform is the oracle's, or a float near-tie: its oracle distance within 1e-5 of the oracle minimum
            rs = O.rotation_set(imgs[i], nd, R, flip)
            _, _, D = O.distance_f32(som, rs, ed, full=True)
            chosen = D[np.arange(N), rot[i]]
            assert (chosen <= D.min(axis=1) * (1 + 1e-5)).all()
            assert (rot[i] == r).mean() > 0.5
        else:
            assert np.array_equal(dist[i].view(np.uint32), d.view(np.uint32))
            assert np.array_equal(rot[i], r)


@pytest.mark.parametrize("mode", [0, 2, 1])
@pytest.mark.parametrize("case", [(1, 2, 2, 2, 1, False), (1, 3, 3, 2, 1, False), (1, 3, 3, 2, 360, False),
                                  (2, 3, 3, 2, 360, False), (2, 3, 3, 2, 360, True)])
def test_map_reference_known_answers(cuda, mode, case):
    """test/CudaTest/mapper.cu:55-120: image = 0, SOM = 1 must map to exactly 2.0 in all three modes."""
    import pink_b200.capi as capi
    som_dim, nd, idim, ed, R, flip = case
    N = som_dim * som_dim
    som = np.ones((N, 1, nd, nd), np.float32)
    img = np.zeros((1, 1, idim, idim), np.float32)
    with Context(capi, make_config(capi, N, 1, idim, nd, ed, R, flip, mode)) as ctx:
        ctx.set_som(som)
        dist, _ = ctx.map(img)
    assert np.array_equal(dist[0], np.full(N, 2.0, np.float32))


def test_config_errors_match_reference_messages():
    import ctypes as C
    import pink_b200.capi as capi
    h = C.c_void_p()
    for R in (0, 3, 90):                        # test/SelfOrganizingMapTest/Trainer.cpp:33-38
        cfg = make_config(capi, 4, 1, 2, 2, 2, R, False, 2)
        assert capi.lib.pink_b200_create(C.byref(cfg), C.byref(h)) == capi.EINVAL
        assert b"Number of rotations must be 1 or larger then 1 and divisible by 4" in capi.lib.pink_b200_last_error()
    cfg = make_config(capi, 4, 1, 8, 4, 5, 4, False, 2)
    assert capi.lib.pink_b200_create(C.byref(cfg), C.byref(h)) == capi.EINVAL
    assert b"Euclidean distance dimension larger than neuron dimension" in capi.lib.pink_b200_last_error()


@pytest.mark.parametrize("case", [TRAIN_CASES[2], TRAIN_CASES[4], TRAIN_CASES[3]])
@pytest.mark.parametrize("step_kernel", [0, 1, 2])
def test_factors_per_distance_class_equal_the_table(cuda, case, step_kernel):
    """pink_b200_set_update_function (one factor per distinct map distance, looked up on the device from the neurons'
    grid positions) trains the same map, bit for bit, as the N x N factor table -- in every launch sequence."""
    import pink_b200.capi as capi
    layout, s0, s1, C_, idim, nd, ed, R, flip, n = case
    N = _som_size(layout, s0, s1)
    rng = np.random.default_rng(5)
    som0 = rng.random((N, C_, nd, nd), dtype=np.float32)
    imgs = blob_images(9, idim, C_, seed=8).reshape(9, C_, idim, idim)
    F = O.update_factors(layout, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2, 2.5)          # with a max_update_distance cut-off
    out = []
    for classes in (False, True):
        with Context(capi, make_config(capi, N, C_, idim, nd, ed, R, flip, 2), {"step_kernel": step_kernel}) as ctx:
            ctx.set_som(som0)
            if classes:
                ctx.e.set_update_function(layout, s0, s1, capi.FUNC_GAUSSIAN, 1.1, 0.2, 2.5)
            else:
                ctx.set_factors(F)
            log = ctx.train(imgs)
            out.append((list(log), ctx.get_som(som0).copy()))
    assert out[0][0] == out[1][0]
    assert np.array_equal(out[0][1].view(np.uint32), out[1][1].view(np.uint32))
