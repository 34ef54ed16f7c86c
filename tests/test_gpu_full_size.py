"""Checks at the size of the headline configuration (hexagonal map of 2791 neurons, 128 x 128 images, 90 x 90
neurons, 64 x 64 distance region, 720 rotations + flip, uint8), where the CPU oracle is too slow for whole steps:
mapping is compared with the oracle on a sample of neurons (each neuron's result is independent of the others),
the best matching unit must be the first minimum of the mapped distances, and the trained map is compared, for a
sample of neurons and for the whole best-matching neighbourhood, with the oracle's update arithmetic applied to the
old values, the oracle's rotation set, the mapped best transform and the factor table.  The checksums that
bench.py prints for its untimed training prefix (identical for every number of GPUs) are pinned here too."""
import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine
from pink_b200.synthetic import blob_images, mt19937_uniform

pytestmark = pytest.mark.gpu

SIDE, IDIM, ND, ED, R = 61, 128, 90, 64, 720


def test_bench_check_block(cuda):
    """The `check` block of bench.py at one GPU: its best matching units are the first minima of the distances the
    oracle-checked mapping reports (teacher-forced image by image), and its checksums are reproducible."""
    import bench
    w = bench.WORKLOAD
    N, som, pool = bench.make_inputs(w, bench.CHECK_IMAGES)
    F = engine.update_factors(w["som_layout"], w["som_dim"], w["som_dim"], capi.FUNC_GAUSSIAN, w["sigma"], w["damping"])
    with bench.make_engine(w, N, 0) as eng:
        eng.set_update_factors(F)
        first = bench.training_check(eng, som, pool, bench.CHECK_IMAGES)
        again = bench.training_check(eng, som, pool, bench.CHECK_IMAGES)
        assert first == again
        # the same sequence image by image, each best matching unit against the mapping of the current map
        eng.set_som(som)
        bmus = []
        for i in range(8):
            dist, _ = eng.map(pool[i:i + 1])
            eng.train(pool[i:i + 1])
            bmus.append(int(eng.bmu_log(1)[0]))
            assert bmus[-1] == int(np.argmin(dist[0]))
        assert bmus == first["bmu_first8"]
    with bench.make_engine(w, N, 0, options={"step_kernel": 1}) as eng:      # the older launch sequence agrees
        eng.set_update_factors(F)
        assert bench.training_check(eng, som, pool, bench.CHECK_IMAGES) == first


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
            # (3) the new map, EVERY neuron: w - (w - r) * f with r the mapped best transform of the image (this
            #     covers the neurons the kernel leaves out because it can prove that they cannot change)
            new = eng.get_som(np.empty_like(current))
            rotset = O.rotation_set(img[0], ND, R, True).reshape(T, -1)
            want = np.ascontiguousarray(current).reshape(N, -1)
            O.update(want, rotset, np.ascontiguousarray(rot), 0, np.ascontiguousarray(F[bmu])[None])
            assert np.array_equal(new.reshape(N, -1).view(np.uint32), want.view(np.uint32))
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
