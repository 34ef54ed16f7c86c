"""Checks at the size of the headline configuration (hexagonal map of 2791 neurons, 128 x 128 images, 90 x 90
neurons, 64 x 64 distance region, 720 rotations + flip, uint8), where the CPU oracle is too slow for whole steps:
mapping is compared with the oracle on a sample of neurons (each neuron's result is independent of the others),
the best matching unit must be the first minimum of the mapped distances, and the trained map is compared, for a
sample of neurons and for the whole best-matching neighbourhood, with the oracle's update arithmetic applied to the
old values, the oracle's rotation set, the mapped best transform and the factor table."""
import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine
from pink_b200.synthetic import blob_images, mt19937_uniform

pytestmark = pytest.mark.gpu

SIDE, IDIM, ND, ED, R = 61, 128, 90, 64, 720


def test_headline_size_step(cuda):
    N = engine.som_size(capi.LAYOUT_HEXAGONAL, SIDE, SIDE)
    assert N == 2791
    T = 2 * R
    som0 = mt19937_uniform(N * ND * ND, 1234).reshape(N, 1, ND, ND)
    imgs = blob_images(3, IDIM, 1, seed=9).reshape(3, 1, IDIM, IDIM)
    F = engine.update_factors(capi.LAYOUT_HEXAGONAL, SIDE, SIDE, capi.FUNC_GAUSSIAN, 3.0, 0.05)
    eng = engine.Engine(N, 1, IDIM, ND, ED, R, True, capi.UINT8)
    try:
        eng.set_som(som0)
        eng.set_update_factors(F)
        rng = np.random.default_rng(3)
        current = som0.copy()
        bmus = []
        for img in imgs:
            dist, rot = eng.map(img[None])
            dist, rot = dist[0], rot[0]
            # (1) mapping against the oracle on a sample of neurons
            sample = np.unique(np.concatenate([rng.integers(0, N, 6), [0, N - 1, int(np.argmin(dist))]]))
            wd, wr = O.map_image(np.ascontiguousarray(current[sample]), img, ED, R, True, O.MODE_U8)
            assert np.array_equal(dist[sample].view(np.uint32), wd.view(np.uint32))
            assert np.array_equal(rot[sample], wr)
            # (2) one training step: the best matching unit is the first minimum of the mapped distances
            eng.train(img[None])
            bmu = int(eng.bmu_log(1)[0])
            bmus.append(bmu)
            assert bmu == int(np.argmin(dist))
            # (3) the new map, neuron by neuron: w - (w - r) * f with r the mapped best transform of the image
            new = eng.get_som(np.empty_like(current))
            rotset = O.rotation_set(img[0], ND, R, True).reshape(T, -1)
            near = np.argsort(F[bmu])[-12:]                       # the strongest factors: the neighbourhood of the unit
            check = np.unique(np.concatenate([sample, near, [bmu]]))
            want = np.ascontiguousarray(current[check]).reshape(len(check), -1)
            O.update(want, rotset, np.ascontiguousarray(rot[check]), 0, np.ascontiguousarray(F[bmu, check])[None])
            assert np.array_equal(new[check].reshape(len(check), -1).view(np.uint32), want.view(np.uint32))
            # (4) neurons with a zero factor are untouched, and so is every neuron the step did not rewrite
            zero = np.flatnonzero(F[bmu] == 0)
            assert np.array_equal(new[zero], current[zero])
            current = new
        counts = eng.update_counts()
        assert counts.sum() == len(imgs)
        read, written = eng.update_stats()
        assert 0 < written <= read <= sum(int((F[b] != 0).sum()) for b in bmus)
    finally:
        eng.close()
