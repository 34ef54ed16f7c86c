"""A C++ program written against the reference's class API (include/pink_b200.hpp: pink::SOM, pink::Data,
pink::Trainer<..., float, true>, pink::Mapper<..., float, true>) is compiled with g++, run on the GPU and
compared with the CPU oracle bit for bit."""
import os
import subprocess

import numpy as np
import pytest

import oracle as O
from pink_b200 import build as B
from pink_b200 import files

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_program_against_the_class_api(cuda, tmp_path):
    B.build()
    exe = str(tmp_path / "use_pink_hpp")
    libdir = os.path.dirname(B.LIB)
    subprocess.run(["g++", "-O2", "-std=c++17", "-I" + os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "use_pink_hpp.cpp"), "-o", exe, "-L" + libdir, "-lpink_b200",
                    "-Wl,-rpath," + libdir], check=True)
    n, idim, nd, ed, R = 5, 16, 12, 7, 8
    rng = np.random.default_rng(11)
    imgs = rng.random((n, idim, idim), dtype=np.float32)
    som0 = rng.random((9, 1, nd, nd), dtype=np.float32)
    data, init = str(tmp_path / "data.bin"), str(tmp_path / "init.raw")
    files.write_data_file(data, imgs)
    som0.tofile(init)
    r = subprocess.run([exe, data, init], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    out = {line.split()[0]: line.split()[1:] for line in r.stdout.splitlines() if line and not line.startswith("error")}
    error = [line for line in r.stdout.splitlines() if line.startswith("error")][0]

    want = som0.copy()
    F = O.update_factors(0, 3, 3, O.FUNC_GAUSSIAN, 1.1, 0.2)
    counts = np.zeros(9, np.uint32)
    for im in imgs:
        counts[O.train_step(want, im.reshape(1, idim, idim), F, ed, R, True, O.MODE_U8)[2]] += 1
    got = np.array([int(v, 16) for v in out["som"]], np.uint32)
    assert np.array_equal(got, want.view(np.uint32).ravel())
    assert [int(v) for v in out["counts"]] == list(counts)
    wd, wr = O.map_image(want, imgs[0].reshape(1, idim, idim), ed, R, True, O.MODE_U8)
    assert np.array_equal(np.array([int(v, 16) for v in out["dist"]], np.uint32), wd.view(np.uint32))
    assert [int(v) for v in out["rot"]] == list(wr)
    assert error == "error Number of rotations must be 1 or larger then 1 and divisible by 4"
    want3 = som0[:8].copy()
    F3 = O.update_factors_3d((2, 2, 2), O.FUNC_GAUSSIAN, 1.1, 0.2)
    for im in imgs[:2]:
        O.train_step(want3, im.reshape(1, idim, idim), F3, ed, R, True, O.MODE_U8)
    assert np.array_equal(np.array([int(v, 16) for v in out["som3"]], np.uint32), want3.view(np.uint32).ravel())
