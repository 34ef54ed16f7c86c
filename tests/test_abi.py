"""The C-ABI boundary without a GPU: the library loads, exports exactly what include/pink_b200.h declares,
its host-side helpers agree with the oracle, and compute entries fail loudly (no fallback) where no device is."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pink_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pink_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 25
    lib = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), "header declares %s but the library does not export it" % n
    assert sorted(capi.SYMBOLS) == names, "pink_b200/capi.py must bind exactly the declared entry points"


def test_config_struct_layout():
    assert C.sizeof(capi.Config) == 14 * 4


def test_version_and_error_strings():
    assert b"sm_100a" in capi.lib.pink_b200_version()
    assert isinstance(capi.lib.pink_b200_last_error(), bytes)


def test_configuration_errors_follow_the_reference():
    h = C.c_void_p()
    mk = lambda **kw: capi.Config(**{**dict(n_neurons=4, channels=1, image_dim=2, neuron_dim=2, ed_dim=2, ed_shape=0,
                                            n_rotations=4, use_flip=0, dist_type=2, interpolation=1, device=0, rank=0,
                                            world_size=1, max_batch=0), **kw})
    for R in (0, 3, 90):                                   # test/SelfOrganizingMapTest/Trainer.cpp:33-38
        assert capi.lib.pink_b200_create(C.byref(mk(n_rotations=R)), C.byref(h)) == capi.EINVAL
        assert b"Number of rotations must be 1 or larger then 1 and divisible by 4" in capi.lib.pink_b200_last_error()
    assert capi.lib.pink_b200_create(C.byref(mk(ed_dim=3)), C.byref(h)) == capi.EINVAL      # Mapper.h:63-66
    assert b"Euclidean distance dimension larger than neuron dimension" in capi.lib.pink_b200_last_error()
    assert capi.lib.pink_b200_create(C.byref(mk(ed_dim=0)), C.byref(h)) == capi.EINVAL      # DynamicTrainer.cpp:25
    assert b"euclidean_distance_dim not defined" in capi.lib.pink_b200_last_error()
    assert capi.lib.pink_b200_create(C.byref(mk(interpolation=0)), C.byref(h)) == capi.EINVAL
    assert b"unknown interpolation" in capi.lib.pink_b200_last_error()
    assert capi.lib.pink_b200_create(C.byref(mk(dist_type=7)), C.byref(h)) == capi.EINVAL
    assert capi.lib.pink_b200_create(C.byref(mk(rank=2, world_size=2)), C.byref(h)) == capi.EINVAL
    assert capi.lib.pink_b200_create(None, C.byref(h)) == capi.EINVAL


def test_no_cpu_fallback():
    """Without an sm_100 device a valid configuration must fail with a CUDA error, never compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(capi.PinkError) as e:
        engine.Engine(4, 1, 4, 2, 2, 4, False, capi.UINT8)
    assert e.value.code == capi.ECUDA


@pytest.mark.parametrize("case", [(0, 3, 4, 0, 1.1, 0.2, -1.0), (0, 10, 10, 0, 1.1, 0.2, 2.5), (1, 7, 7, 0, 2.0, 0.1, -1.0),
                                  (1, 61, 61, 0, 3.0, 0.05, -1.0), (0, 5, 5, 2, 1.5, 0.3, -1.0), (0, 4, 4, 3, 1.0, 0.0, -1.0),
                                  (0, 6, 3, 1, 1.3, 0.4, -1.0)])
def test_host_update_factor_table_bit_exact(case):
    lay, d0, d1, func, p0, p1, md = case
    got = engine.update_factors(lay, d0, d1, func, p0, p1, md)
    want = O.update_factors(lay, d0, d1, func, p0, p1, md)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("case", [((2, 2, 2), 0, 1.1, 0.2, -1.0), ((3, 4, 2), 0, 1.1, 0.2, 1.8), ((4, 3, 5), 2, 1.5, 0.3, -1.0),
                                  ((6, 5, 4), 1, 2.0, 0.1, -1.0)])
def test_host_update_factor_table_of_3d_soms_bit_exact(case):
    dims, func, p0, p1, md = case
    N = int(np.prod(dims))
    got = np.empty((N, N), np.float32)
    capi.check(capi.lib.pink_b200_update_factors_3d(*dims, func, p0, p1, md, got.ctypes.data))
    want = O.update_factors_3d(dims, func, p0, p1, md)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    dist = np.empty((N, N), np.float32)
    capi.check(capi.lib.pink_b200_som_distances_3d(*dims, dist.ctypes.data))
    i, j = N - 1, 0
    assert dist[i, j] == np.float32(O.lib.pko_cartesian3_distance(i, j, *dims))
    assert capi.lib.pink_b200_update_factors_3d(0, 1, 1, 0, 1.0, 1.0, -1.0, got.ctypes.data) == capi.EINVAL


def test_som_size_and_operand_stride():
    assert engine.som_size(capi.LAYOUT_HEXAGONAL, 61, 61) == 2791          # radius 30
    assert engine.som_size(capi.LAYOUT_CARTESIAN, 20, 20) == 400
    assert capi.lib.pink_b200_operand_stride(961, capi.UINT8) == 1024
    assert capi.lib.pink_b200_operand_stride(4096, capi.UINT16) == 4096
    assert capi.lib.pink_b200_operand_stride(961, capi.FLOAT) == 992          # whole 128-byte slices of float words


@pytest.mark.parametrize("N,W", [(2791, 8), (2791, 1), (100, 3), (7, 7), (10, 4)])
def test_shard_ranges_partition_the_som(N, W):
    """N / W (+1 for the first N % W ranks), contiguous:
    src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:65-77."""
    nxt = 0
    for r in range(W):
        first, count = engine.shard_range(N, W, r)
        assert first == nxt and count == N // W + (1 if r < N % W else 0)
        nxt += count
    assert nxt == N
    with pytest.raises(capi.PinkError):
        engine.shard_range(3, 4, 0)


def test_bench_reads_tracked_profile_figures():
    """bench.py quotes DRAM traffic from the tracked ncu summary (lines `key = value`); the keys it asks for exist."""
    import bench
    assert bench.tracked_figure("train_steps_kernel_u8_c4.txt", "dram_bytes_per_image") > 1e6
    assert bench.tracked_figure("train_steps_kernel_u8_c4.txt", "moved_bytes_per_image") > 1e6
    assert bench.tracked_figure("train_steps_kernel_u8_c4.txt", "no_such_key") is None
    assert bench.tracked_figure("no_such_file.txt", "x") is None
