"""One process driving several GPUs (pink_b200_group_*): image-sharded mapping must reproduce a single context's
results byte for byte, and neuron-sharded training the oracle's map bit for bit.  Mapping shards need no
communication, so the mapping test also runs with two shards on ONE GPU; the training test needs two GPUs."""
import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [2, 1, 0])
def test_group_mapping_equals_single_context(cuda, mode):
    N, idim, nd, ed, R = 20, 32, 22, 15, 40
    rng = np.random.default_rng(11 + mode)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    imgs = rng.random((75, 1, idim, idim), dtype=np.float32)          # ragged shares, more than one internal batch
    with engine.Engine(N, 1, idim, nd, ed, R, True, mode) as eng:
        eng.set_som(som)
        want_d, want_r = eng.map(imgs)
    devices = [0, 1, 0] if cuda.cuda.device_count() >= 2 else [0, 0, 0]
    with engine.Group(N, 1, idim, nd, ed, R, True, mode, devices=devices) as grp:
        assert grp.size == 3
        grp.set_som(som)
        got_d, got_r = grp.map(imgs)
        got_d2, got_r2 = grp.map(imgs[:2])                                # fewer images than shards
    assert np.array_equal(got_d.view(np.uint32), want_d.view(np.uint32)) and np.array_equal(got_r, want_r)
    assert np.array_equal(got_d2.view(np.uint32), want_d[:2].view(np.uint32)) and np.array_equal(got_r2, want_r[:2])
    # and against the oracle, one image
    d, r = O.map_image(som, imgs[0], ed, R, True, mode)
    if mode == 0:
        np.testing.assert_allclose(got_d[0], d, rtol=1e-5)
    else:
        assert np.array_equal(got_d[0].view(np.uint32), d.view(np.uint32)) and np.array_equal(got_r[0], r)


def test_single_device_group_trains_and_maps(cuda):
    lay, s0, s1, idim, nd, ed, R, n_img = 0, 4, 3, 32, 22, 15, 40, 21
    N = s0 * s1
    rng = np.random.default_rng(5)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    imgs = rng.random((n_img, 1, idim, idim), dtype=np.float32)
    F = engine.update_factors(lay, s0, s1, capi.FUNC_GAUSSIAN, 1.1, 0.2)
    want = som.copy()
    bmus = [O.train_step(want, im, F, ed, R, True, O.MODE_U8)[2] for im in imgs]
    with engine.Group(N, 1, idim, nd, ed, R, True, capi.UINT8, devices=[0]) as grp:
        grp.set_som(som)
        grp.set_update_factors(F)
        grp.train(imgs)
        got = grp.get_som(np.zeros_like(som))
        counts = grp.update_counts()
        dist, rot = grp.map(imgs[:3])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert counts.sum() == n_img and all(counts[b] > 0 for b in bmus)
    d, r = O.map_image(want, imgs[0], ed, R, True, O.MODE_U8)
    assert np.array_equal(dist[0].view(np.uint32), d.view(np.uint32)) and np.array_equal(rot[0], r)


@pytest.mark.parametrize("mode", [2, 1, 0])
def test_two_gpu_group_training_bit_exact(cuda, mode):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lay, s0, s1, idim, nd, ed, R, n_img = 0, 5, 4, 32, 22, 15, 40, 37
    N = s0 * s1
    rng = np.random.default_rng(77)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    som[13] = som[4]                                   # identical neurons in different shards: BMU ties
    imgs = rng.random((n_img, 1, idim, idim), dtype=np.float32)
    F = engine.update_factors(lay, s0, s1, capi.FUNC_GAUSSIAN, 1.1, 0.2)
    want = som.copy()
    bmus = [O.train_step(want, im, F, ed, R, True, mode)[2] for im in imgs]
    with engine.Group(N, 1, idim, nd, ed, R, True, mode, devices=[0, 1]) as grp:
        grp.set_som(som)
        grp.set_update_factors(F)
        grp.train(imgs[:20])
        grp.train(imgs[20:])
        got = grp.get_som(np.zeros_like(som))
        counts = grp.update_counts()
        dist, rot = grp.map(imgs[:5])                  # image-sharded, on the trained map
    if mode == 0:
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-7)
    else:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        d, r = O.map_image(want, imgs[4], ed, R, True, mode)
        assert np.array_equal(dist[4].view(np.uint32), d.view(np.uint32)) and np.array_equal(rot[4], r)
    assert counts.sum() == n_img and all(counts[b] > 0 for b in bmus)
