"""The command line program's file formats and data order (no GPU): headers written by the Python module are read
back by the C++ program, and the shuffled order equals the reference iterator's (golden vectors from
tests/golden/make_golden.py; compared live where the reference-linked checker library exists)."""
import ctypes as C
import json
import os
import subprocess

import numpy as np
import pytest

import oracle as O
from pink_b200 import build as B
from pink_b200 import files

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu.npz"))


@pytest.fixture(scope="module")
def pink():
    B.build()
    assert os.path.exists(B.CLI)
    return B.CLI


def _inspect(pink, path):
    return json.loads(subprocess.run([pink, "--inspect", path], capture_output=True, text=True, check=True).stdout)


def test_headers_round_trip(pink, tmp_path):
    rng = np.random.default_rng(1)
    p = str(tmp_path / "data.bin")
    files.write_data_file(p, rng.random((5, 6, 6), dtype=np.float32), "# a comment\n# END OF HEADER\n")
    info = _inspect(pink, p)
    assert (info["version"], info["file_type"], info["entries"], info["dims"]) == (2, 0, 5, [6, 6])
    assert info["text_header_bytes"] == len("# a comment\n# END OF HEADER\n")
    back, header = files.read_data_file(p)
    assert back.shape == (5, 6, 6) and header.endswith("# END OF HEADER\n")
    p3 = str(tmp_path / "data3.bin")
    files.write_data_file(p3, rng.random((4, 2, 8, 8), dtype=np.float32))
    assert _inspect(pink, p3)["dims"] == [2, 8, 8]
    ps = str(tmp_path / "som.bin")
    som = rng.random((9, 4, 4), dtype=np.float32)
    files.write_som_file(ps, som, (3, 3))
    info = _inspect(pink, ps)
    assert (info["file_type"], info["som_dims"], info["neuron_dims"]) == (1, [3, 3], [4, 4])
    assert info["data_offset"] == 4 * (9 + 2)            # the position the reference's reader assumes (SOM.h:94)
    got, dims, _ = files.read_som_file(ps)
    assert np.array_equal(got, som) and dims == [3, 3]


@pytest.mark.parametrize("n,seed", [(8, 1234), (100, 1234), (100, 1235), (1000, 7)])
def test_training_order_matches_reference(pink, n, seed):
    out = subprocess.run([pink, "--dump-order", str(n), str(seed), "1"], capture_output=True, text=True, check=True).stdout
    got = np.array(out.split(), np.uint32)
    assert np.array_equal(got, GOLD["order_%d_%d" % (n, seed)])
    assert sorted(got) == list(range(n))
    if O.have_ref():
        r = O.ref()
        r.ref_shuffled_order.argtypes = [C.c_uint32, C.c_uint64, C.c_int, C.c_void_p]
        live = np.zeros(n, np.uint32)
        r.ref_shuffled_order(n, seed, 1, live.ctypes.data)
        assert np.array_equal(got, live)


def test_passes_use_consecutive_seeds(pink):
    two = subprocess.run([pink, "--dump-order", "50", "9", "2"], capture_output=True, text=True, check=True).stdout.splitlines()
    second = subprocess.run([pink, "--dump-order", "50", "10", "1"], capture_output=True, text=True, check=True).stdout.splitlines()
    assert two[1] == second[0] and two[0] != two[1]


def test_option_errors(pink, tmp_path):
    r = subprocess.run([pink, "--numrot", "6", "--train", "a", "b"], capture_output=True, text=True)
    assert r.returncode != 0 and "Number of rotations must be 1 or a multiple of 4" in r.stderr
    r = subprocess.run([pink, "--som-width", "5"], capture_output=True, text=True)
    assert r.returncode != 0 and "Unknown execution path" in r.stderr
    r = subprocess.run([pink, "--train", str(tmp_path / "missing.bin"), "x"], capture_output=True, text=True)
    assert r.returncode != 0 and "Error opening" in r.stderr
    r = subprocess.run([pink, "--layout", "hexagonal", "--som-width", "3", "--som-height", "3", "--som-depth", "2",
                        "--train", "a", "b"], capture_output=True, text=True)
    assert r.returncode != 0 and "For hexagonal layout som-depth must be equal to 1." in r.stderr
    r = subprocess.run([pink, "--som-width", "3", "--som-height", "1", "--som-depth", "2", "--train", "a", "b"],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "som-depth > 1 needs som-height > 1." in r.stderr
