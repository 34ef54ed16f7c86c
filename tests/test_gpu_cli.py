"""End-to-end runs of the command line program on a GPU: training and mapping from files, with the options of the
reference's `Pink`, against the CPU oracle fed with the same initial map and the same image order."""
import os
import subprocess

import numpy as np
import pytest

import oracle as O
from pink_b200 import build as B
from pink_b200 import files
from pink_b200.synthetic import blob_images, mt19937_uniform

pytestmark = pytest.mark.gpu


def _run(*args):
    r = subprocess.run([B.CLI] + [str(a) for a in args], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


@pytest.mark.parametrize("shuffle", [False, True])
def test_train_and_map_from_files(cuda, tmp_path, shuffle):
    n, idim, nd, ed, R, w, h, seed = 20, 16, 12, 7, 8, 3, 3, 77
    imgs = blob_images(n, idim, 1, seed=3).reshape(n, idim, idim)
    data, som_path, map_path, rot_path = (str(tmp_path / f) for f in ("data.bin", "som.bin", "map.bin", "rot.bin"))
    files.write_data_file(data, imgs, "# synthetic blobs\n# END OF HEADER\n")
    common = ["--som-width", w, "--som-height", h, "--numrot", R, "--neuron-dimension", nd,
              "--euclidean-distance-dimension", ed, "--seed", seed, "--euclidean-distance-type", "uint8"]
    extra = [] if shuffle else ["--input-shuffle-off"]
    _run(*common, *extra, "--init", "random", "--num-iter", 2, "--dist-func", "gaussian", 1.5, 0.3,
         "--inter-store", "keep", "--progress", 4, "--train", data, som_path)

    # the oracle on the same initial map (libstdc++ uniform_real over mt19937(seed)) and the same order
    N = w * h
    want = mt19937_uniform(N * nd * nd, seed).reshape(N, 1, nd, nd).copy()
    F = O.update_factors(0, w, h, O.FUNC_GAUSSIAN, 1.5, 0.3)
    snapshots, done = [], 0
    points = [10, 20, 30]                      # 40 images, 4 reports: after images 10, 20, 30 (0-based) the map is stored
    for it in range(2):
        order = list(range(n))
        if shuffle:
            order = [int(v) for v in _run("--dump-order", n, seed + it, 1).split()]
        for k in order:
            O.train_step(want, imgs[k].reshape(1, idim, idim), F, ed, R, True, O.MODE_U8)
            if done in points:
                snapshots.append(want.copy())
            done += 1
    got, som_dims, header = files.read_som_file(som_path)
    assert som_dims == [w, h] and got.shape == (N, nd, nd) and header == ""
    assert np.array_equal(got.reshape(want.shape).view(np.uint32), want.view(np.uint32))
    for i, snap in enumerate(snapshots):       # --inter-store keep: som_0.bin, som_1.bin, ...
        inter, _, _ = files.read_som_file(str(tmp_path / ("som_%d.bin" % i)))
        assert np.array_equal(inter.reshape(snap.shape).view(np.uint32), snap.view(np.uint32))

    _run(*common, "--store-rot-flip", rot_path, "--map", data, map_path, som_path)
    dist, dims = files.read_mapping_file(map_path)
    flip, angle, _ = files.read_rot_flip_file(rot_path)
    assert dims == [w, h] and dist.shape == (n, N) and flip.shape == (n, N)
    step = np.float32(2.0 * np.pi) / np.float32(R)
    for k in range(n):
        wd, wr = O.map_image(want, imgs[k].reshape(1, idim, idim), ed, R, True, O.MODE_U8)
        assert np.array_equal(dist[k].view(np.uint32), wd.view(np.uint32))
        assert np.array_equal(flip[k], wr // R == 1)
        assert np.array_equal(angle[k].view(np.uint32), ((wr % R).astype(np.float32) * step).view(np.uint32))


def test_hexagonal_map_from_file_init(cuda, tmp_path):
    """--layout hexagonal with --init <SOM file>, circular region, float distances, two channels."""
    n, idim, nd, ed, R = 6, 20, 14, 10, 12
    rng = np.random.default_rng(5)
    imgs = rng.random((n, 2, idim, idim), dtype=np.float32)
    N = int(O.lib.pko_hexagonal_size(3))
    som0 = rng.random((N, 2, nd, nd), dtype=np.float32)
    data, init, out = (str(tmp_path / f) for f in ("data.bin", "init.bin", "out.bin"))
    files.write_data_file(data, imgs)
    files.write_som_file(init, som0, (3, 3), "# header kept\n# END OF HEADER\n")
    _run("--layout", "hexagonal", "--som-width", 3, "--som-height", 3, "--numrot", R, "-d", nd, "-e", ed,
         "--euclidean-distance-type", "uint16", "--euclidean-distance-shape", "circular", "--input-shuffle-off",
         "--init", init, "--train", data, out)
    want = som0.copy()
    F = O.update_factors(1, 3, 3, O.FUNC_GAUSSIAN, 1.1, 0.2)
    for im in imgs:
        O.train_step(want, im, F, ed, R, True, O.MODE_U16, shape=O.SHAPE_CIRCULAR)
    got, dims, header = files.read_som_file(out)
    assert dims == [3, 3] and header == "# header kept\n# END OF HEADER\n"
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_three_dimensional_map(cuda, tmp_path):
    """--som-depth > 1: a cartesian map of 3 x 2 x 2 neurons; the files carry three SOM dimensions."""
    n, idim, nd, ed, R, dims, seed = 7, 16, 12, 7, 8, (3, 2, 2), 5
    imgs = blob_images(n, idim, 1, seed=8).reshape(n, idim, idim)
    data, som_path, map_path = (str(tmp_path / f) for f in ("data.bin", "som.bin", "map.bin"))
    files.write_data_file(data, imgs)
    common = ["--som-width", dims[0], "--som-height", dims[1], "--som-depth", dims[2], "--numrot", R, "-d", nd, "-e", ed,
              "--seed", seed, "--euclidean-distance-type", "uint8"]
    _run(*common, "--input-shuffle-off", "--init", "random", "--train", data, som_path)
    N = int(np.prod(dims))
    want = mt19937_uniform(N * nd * nd, seed).reshape(N, 1, nd, nd).copy()
    F = O.update_factors_3d(dims, O.FUNC_GAUSSIAN, 1.1, 0.2)
    for im in imgs:
        O.train_step(want, im.reshape(1, idim, idim), F, ed, R, True, O.MODE_U8)
    got, som_dims, _ = files.read_som_file(som_path)
    assert som_dims == list(dims) and got.shape == (N, nd, nd)
    assert np.array_equal(got.reshape(want.shape).view(np.uint32), want.view(np.uint32))
    _run(*common, "--map", data, map_path, som_path)
    dist, mdims = files.read_mapping_file(map_path)
    assert mdims == list(dims) and dist.shape == (n, N)
    wd, _ = O.map_image(want, imgs[0].reshape(1, idim, idim), ed, R, True, O.MODE_U8)
    assert np.array_equal(dist[0].view(np.uint32), wd.view(np.uint32))
