"""Generates tests/golden/reference_cpu.npz from the reference's own CPU code.

Run in a container that has the reference source tree (it is compiled into
oracle/_ref/libpink_ref.so by oracle/Makefile):

    python tests/golden/make_golden.py

Every entry holds seeded inputs and the outputs of the UNMODIFIED reference
templates (SpatialTransformer, Trainer<...,false>, Mapper<...,false>, the
layout distances and distribution functors) run single-threaded so that the
first-minimum winner is the deterministic one.  tests/test_oracle.py checks
the CPU restatement (oracle/pink_oracle.c) against these bit for bit; the GPU
box needs only this file, not the reference tree.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ["OMP_NUM_THREADS"] = "1"

import oracle as O  # noqa: E402

ROT_CASES = [  # channels (0 = 2-D layout), image side, neuron side, rotations, flip
    (0, 10, 8, 8, True), (0, 12, 7, 16, True), (0, 6, 9, 4, False), (0, 16, 12, 360, True), (2, 14, 9, 8, True),
    (3, 9, 12, 12, False), (0, 5, 5, 1, True), (0, 32, 22, 40, True),
]
STEP_CASES = [  # som layout, s0, s1, channels, image, neuron, ed, rotations, flip, n images, func, p0, p1, max_dist
    (0, 3, 3, 0, 16, 12, 7, 16, True, 3, 0, 1.1, 0.2, -1.0),
    (0, 2, 2, 0, 64, 45, 45, 360, True, 2, 0, 1.1, 0.2, -1.0),
    (1, 5, 5, 0, 20, 14, 9, 8, True, 3, 0, 2.0, 0.1, -1.0),
    (0, 3, 2, 2, 15, 10, 7, 12, True, 3, 0, 1.1, 0.2, -1.0),
    (0, 4, 4, 0, 24, 17, 8, 40, True, 3, 2, 1.5, 0.3, 2.5),
    (0, 3, 3, 0, 12, 12, 12, 4, False, 2, 3, 1.0, 0.0, -1.0),
]
CIRCLE_CASES = [  # circular distance region, 2-D data layout: som layout, s0, s1, image, neuron, ed, rotations, flip, n images
    (0, 3, 3, 32, 22, 16, 8, True, 3), (1, 3, 3, 40, 28, 20, 12, True, 3), (0, 2, 2, 64, 45, 32, 40, True, 2),
    (0, 2, 3, 16, 12, 12, 4, False, 2),
]
FACTOR_3D_CASES = [((2, 2, 2), 0, 1.1, 0.2, -1.0), ((3, 4, 2), 0, 1.1, 0.2, -1.0), ((4, 3, 5), 1, 1.5, 0.3, 2.5),
                   ((5, 2, 3), 2, 1.3, 0.4, -1.0)]
FACTOR_CASES = [(0, 3, 4, 0, 1.1, 0.2, -1.0), (0, 10, 10, 0, 1.1, 0.2, 2.5), (1, 7, 7, 0, 2.0, 0.1, -1.0),
                (1, 11, 11, 0, 3.0, 0.05, -1.0), (0, 5, 5, 2, 1.5, 0.3, -1.0), (0, 4, 4, 3, 1.0, 0.0, -1.0),
                (0, 6, 3, 1, 1.3, 0.4, -1.0)]


def main():
    if not O.have_ref():
        sys.exit("oracle/_ref/libpink_ref.so is missing: build it where the reference tree exists (make -C oracle)")
    out = {}
    rng = np.random.default_rng(20240)
    for i, (C, idim, nd, R, flip) in enumerate(ROT_CASES):
        img = rng.random((idim, idim) if C == 0 else (C, idim, idim), dtype=np.float32)
        out["rot%d_cfg" % i] = np.array([C, idim, nd, R, int(flip)])
        out["rot%d_img" % i] = img
        out["rot%d_out" % i] = O.ref_rotation_set(img, nd, R, flip)
    for i, (lay, s0, s1, C, idim, nd, ed, R, flip, n, func, p0, p1, md) in enumerate(STEP_CASES):
        N = s0 * s1 if lay == 0 else int(O.lib.pko_hexagonal_size(s0))
        Cn = max(C, 1)
        som = rng.random((N, Cn, nd, nd), dtype=np.float32)
        imgs = rng.random((n, Cn, idim, idim), dtype=np.float32)
        tr = O.RefSession(som, lay, s0, s1, C, idim, nd, ed, R, flip, func, p0, p1, md)
        tr.train(imgs)
        mp = O.RefSession(som, lay, s0, s1, C, idim, nd, ed, R, flip, for_map=True)
        dist, rot = mp.map(imgs)
        out["step%d_cfg" % i] = np.array([lay, s0, s1, C, idim, nd, ed, R, int(flip), n, func])
        out["step%d_par" % i] = np.array([p0, p1, md], np.float32)
        out["step%d_som" % i] = som
        out["step%d_imgs" % i] = imgs
        out["step%d_trained" % i] = tr.som()
        out["step%d_counts" % i] = tr.counts()
        out["step%d_map_dist" % i] = dist
        out["step%d_map_rot" % i] = rot
    for i, (lay, d0, d1, func, p0, p1, md) in enumerate(FACTOR_CASES):
        out["fac%d_cfg" % i] = np.array([lay, d0, d1, func])
        out["fac%d_par" % i] = np.array([p0, p1, md], np.float32)
        out["fac%d_out" % i] = O.ref_update_factors(lay, d0, d1, func, p0, p1, md)
    out["fill_seed1234"] = O.ref_fill_random_uniform(4096, 1234)
    out["fill_default"] = O.ref_fill_random_uniform(256, 5489)
    # (appended after all other entries so that the random stream of the earlier ones does not change)
    for i, (lay, s0, s1, idim, nd, ed, R, flip, n) in enumerate(CIRCLE_CASES):
        N = s0 * s1 if lay == 0 else int(O.lib.pko_hexagonal_size(s0))
        som = rng.random((N, 1, nd, nd), dtype=np.float32)
        imgs = rng.random((n, 1, idim, idim), dtype=np.float32)
        tr = O.RefSession(som, lay, s0, s1, 0, idim, nd, ed, R, flip, shape=O.SHAPE_CIRCULAR)
        tr.train(imgs)
        mp = O.RefSession(som, lay, s0, s1, 0, idim, nd, ed, R, flip, for_map=True, shape=O.SHAPE_CIRCULAR)
        dist, rot = mp.map(imgs)
        out["circ%d_cfg" % i] = np.array([lay, s0, s1, idim, nd, ed, R, int(flip), n])
        out["circ%d_som" % i] = som
        out["circ%d_imgs" % i] = imgs
        out["circ%d_trained" % i] = tr.som()
        out["circ%d_map_dist" % i] = dist
        out["circ%d_map_rot" % i] = rot
    # order of the reference's shuffled data iterator (SelfOrganizingMapLib/DataIteratorShuffled.h:41-74)
    import ctypes as C
    r = O.ref()
    r.ref_shuffled_order.argtypes = [C.c_uint32, C.c_uint64, C.c_int, C.c_void_p]
    for n, seed in [(8, 1234), (100, 1234), (100, 1235), (1000, 7)]:
        order = np.zeros(n, np.uint32)
        r.ref_shuffled_order(n, seed, 1, order.ctypes.data)
        out["order_%d_%d" % (n, seed)] = order
    # factor tables of three-dimensional cartesian SOMs (CartesianLayout<3>)
    for i, (dims, func, p0, p1, md) in enumerate(FACTOR_3D_CASES):
        out["fac3d%d_cfg" % i] = np.array(list(dims) + [func])
        out["fac3d%d_par" % i] = np.array([p0, p1, md], np.float32)
        out["fac3d%d_out" % i] = O.ref_update_factors_3d(dims, func, p0, p1, md)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
