"""Parity at the sizes of the benchmark configurations, where whole CPU-oracle steps would take minutes.

What is independent per neuron (mapped distance, best transform, update) is compared with the oracle on samples or,
where the oracle's arithmetic is cheap (the update), on every neuron; the distance kernels are swept over the
shapes of the precision / shape sweep (neurons {400, 1600, 2791} x distance length {44^2, 64^2, 90^2} x
rotations {90, 360, 720} with flip x {uint8, uint16, float32}) with every neuron's (minimum, first transform)
checked against an exact integer computation and full matrix rows against the oracle."""
import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine
from pink_b200.synthetic import blob_images, mt19937_uniform
from test_gpu_stages import _distance
from util import split_key

pytestmark = pytest.mark.gpu


def _exact_min(a, b):
    """Exact S = |a|^2 + |b|^2 - 2 a.b for integer operands through float64 BLAS (every term is an integer below
    2^53), reduced to (minimum, first transform attaining it) per neuron."""
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    S = (a64 * a64).sum(1)[:, None] + (b64 * b64).sum(1)[None, :] - 2.0 * (a64 @ b64.T)
    return S.min(1).astype(np.uint64), S.argmin(1).astype(np.uint32), S


SWEEP = [(n, k, r) for n in (400, 1600, 2791) for k in (44 * 44, 64 * 64, 90 * 90) for r in (90, 360, 720)]


@pytest.mark.parametrize("mode", [2, 1, 0])
def test_distance_sweep(cuda, mode):
    """All 27 shapes of one mode.  Integer modes: every neuron's key bit-exact, eight full matrix rows bit-exact
    against the oracle.  float32: every distance within 1e-5 relative of a float64 ground truth, the reported
    transform either the ground truth's or one whose true distance is within 1e-5 of the minimum."""
    som_u = mt19937_uniform(2791 * 8100, 1234).reshape(2791, 8100)
    rot_u = mt19937_uniform(1440 * 8100, 4321).reshape(1440, 8100)
    rng = np.random.default_rng(5)
    for N, K, R in SWEEP:
        T = 2 * R
        a_f, b_f = som_u[:N, :K], rot_u[:T, :K]
        if mode == 0:
            a, b = np.ascontiguousarray(a_f), np.ascontiguousarray(b_f)
        else:
            scale, dt = (255.0, np.uint8) if mode == 2 else (65535.0, np.uint16)
            a = np.trunc(a_f * np.float32(scale)).astype(dt)          # truncation, as the reference quantises
            b = np.trunc(b_f * np.float32(scale)).astype(dt)
        keys, mat = _distance(cuda, capi, a, b, mode)
        code, t = split_key(keys[0], mode)
        rows = rng.choice(N, 8, replace=False)
        if mode != 0:
            smin, best, _ = _exact_min(a, b)
            assert np.array_equal(code, smin), (N, K, R)
            assert np.array_equal(t, best), (N, K, R)
            want = O.distance_int(a[rows], b, mode)
            assert np.array_equal(mat[0][rows].astype(np.uint64), want), (N, K, R)
        else:
            # float64 ground truth in the Gram form: its rounding error (~1e-16 |a|^2) is far below the 1e-5 asked of d^2
            _, _, D = _exact_min(a, b)
            got = mat[0].astype(np.float64)
            assert (np.abs(got - D) <= 1e-5 * D).all(), (N, K, R)
            gmin = code.astype(np.uint32).view(np.float32)
            assert np.array_equal(gmin, mat[0].min(1))
            dmin = D.min(1)
            assert (D[np.arange(N), t] <= dmin * (1 + 1e-5)).all(), (N, K, R)     # equal or a float near-tie
            # and the reference's CPU accumulation order on the sampled rows
            side = int(round(K ** 0.5))
            step = max(1, T // 16)
            for n in rows[:2]:
                ref_row = np.array([O.lib.pko_distance_f32_pair(a[n].ctypes.data_as(O.C.c_void_p),
                                                                b[j].ctypes.data_as(O.C.c_void_p), O.C.c_uint32(1),
                                                                O.C.c_uint32(side), O.C.c_uint32(side))
                                    for j in range(0, T, step)], np.float32)
                np.testing.assert_allclose(mat[0][n, ::step], ref_row, rtol=1e-5)


@pytest.mark.parametrize("filtered", [1, 0])
def test_c2_float_map_at_size(cuda, filtered):
    """20 x 20 cartesian SOM of 90 x 90 neurons, 128 x 128 images, 64 x 64 region, 360 rotations + flip, float32:
    through the tensor-core estimate + exact pass (default) and through the all-pairs exact kernel."""
    N, IDIM, ND, ED, R = 400, 128, 90, 64, 360
    som = mt19937_uniform(N * ND * ND, 1234).reshape(N, 1, ND, ND)
    imgs = blob_images(3, IDIM, 1, seed=1002).reshape(3, 1, IDIM, IDIM)
    with engine.Engine(N, 1, IDIM, ND, ED, R, True, capi.FLOAT, options={"f32_filter": filtered}) as eng:
        eng.set_som(som)
        dist, rot = eng.map(imgs)
        stats = eng.map_filter_stats()
    if filtered:
        assert stats["pairs_estimated"] == 3 * N * 2 * R and 3 * N <= stats["pairs_exact"] < stats["pairs_estimated"] / 20
        assert stats["worst_estimate_error"] < stats["error_bound"] / 2       # the assumed bound has room to spare
    else:
        assert stats["pairs_estimated"] == 0
    rng = np.random.default_rng(2)
    for i, img in enumerate(imgs):
        sample = np.unique(np.concatenate([rng.integers(0, N, 24), [0, N - 1, int(np.argmin(dist[i]))]]))
        rotset = O.rotation_set(img[0], ND, R, True)
        wd, wr, D = O.distance_f32(np.ascontiguousarray(som[sample]), rotset, ED, full=True)
        np.testing.assert_allclose(dist[i][sample], np.sqrt(wd), rtol=1e-5)
        # the transform: the oracle's, or one whose oracle distance is within 1e-5 of the oracle's minimum
        at_gpu = D[np.arange(len(sample)), rot[i][sample]]
        assert (at_gpu <= wd * (1 + 1e-5)).all()
        assert (rot[i][sample] == wr).mean() >= 0.9


def test_float_map_of_a_converged_map_through_the_filter(cuda):
    """The estimate |a|^2 + |b|^2 - 2 a.b is weakest where the distances are small against the norms: neurons that
    are rotated copies of the mapped images plus a little noise (what a trained map looks like).  Both float paths
    must agree with the oracle; exact copies give distance 0 at the right transform."""
    N, IDIM, ND, ED, R = 64, 64, 44, 31, 64
    rng = np.random.default_rng(11)
    imgs = blob_images(4, IDIM, 1, seed=77).reshape(4, 1, IDIM, IDIM)
    som = np.empty((N, 1, ND, ND), np.float32)
    for n in range(N):
        rs = O.rotation_set(imgs[n % 4][0], ND, R, True)
        som[n, 0] = rs[(7 * n) % (2 * R)].reshape(ND, ND)
        if n >= 8:
            som[n] += rng.normal(0, 0.003 * (1 + n % 5), som[n].shape).astype(np.float32)
    som = np.clip(som, 0, 1)
    out = {}
    for filtered in (1, 0):
        with engine.Engine(N, 1, IDIM, ND, ED, R, True, capi.FLOAT, options={"f32_filter": filtered}) as eng:
            eng.set_som(som)
            out[filtered] = eng.map(imgs)
            if filtered:
                st = eng.map_filter_stats()
                assert st["worst_estimate_error"] < st["error_bound"] / 2
    for i, img in enumerate(imgs):
        rotset = O.rotation_set(img[0], ND, R, True)
        wd, wr, D = O.distance_f32(som, rotset, ED, full=True)
        for filtered in (1, 0):
            dist, rot = out[filtered][0][i], out[filtered][1][i]
            np.testing.assert_allclose(dist, np.sqrt(wd), rtol=1e-5, atol=1e-7)
            assert (D[np.arange(N), rot] <= wd * (1 + 1e-5) + 1e-12).all()
        for n in range(i, 8, 4):                                   # exact copies of this image
            assert out[1][0][i][n] == 0.0 and out[1][1][i][n] == (7 * n) % (2 * R)


def test_c3_uint16_two_channel_training_at_size(cuda):
    """40 x 40 cartesian SOM of 2 x 106 x 106 neurons, 2 x 150 x 150 images, 75 x 75 region, 360 rotations + flip,
    uint16, three consecutive steps: mapping against the oracle on a sample, the best matching unit = first
    minimum of the mapped distances, and the update of EVERY neuron against the oracle's update arithmetic."""
    S, IDIM, ND, ED, R, C_ = 40, 150, 106, 75, 360, 2
    N, T = S * S, 2 * R
    som0 = mt19937_uniform(N * C_ * ND * ND, 1234).reshape(N, C_, ND, ND)
    imgs = blob_images(3, IDIM, C_, seed=1003).reshape(3, C_, IDIM, IDIM)
    F = engine.update_factors(capi.LAYOUT_CARTESIAN, S, S, capi.FUNC_GAUSSIAN, 2.0, 0.1)
    rng = np.random.default_rng(7)
    with engine.Engine(N, C_, IDIM, ND, ED, R, True, capi.UINT16) as eng:
        eng.set_som(som0)
        eng.set_update_factors(F)
        current = som0.copy()
        for img in imgs:
            dist, rot = eng.map(img[None])
            dist, rot = dist[0], rot[0]
            sample = np.unique(np.concatenate([rng.integers(0, N, 5), [0, N - 1, int(np.argmin(dist))]]))
            wd, wr = O.map_image(np.ascontiguousarray(current[sample]), img, ED, R, True, O.MODE_U16)
            assert np.array_equal(dist[sample].view(np.uint32), wd.view(np.uint32))
            assert np.array_equal(rot[sample], wr)
            eng.train(img[None])
            bmu = int(eng.bmu_log(1)[0])
            assert bmu == int(np.argmin(dist))
            new = eng.get_som(np.empty_like(current))
            rotset = O.rotation_set(img, ND, R, True).reshape(T, -1)
            want = np.ascontiguousarray(current).reshape(N, -1)
            O.update(want, rotset, np.ascontiguousarray(rot), 0, np.ascontiguousarray(F[bmu])[None])
            assert np.array_equal(new.reshape(N, -1).view(np.uint32), want.view(np.uint32))
            current = new
        assert eng.update_counts().sum() == len(imgs)
        assert eng.profile_detail() is not None
