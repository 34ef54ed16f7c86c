"""The reference's Python-level tests and usage, run against both front-ends of the library -- the compiled
pybind11 module pink_b200._pink and its ctypes/numpy mirror pink_b200.pink (same names, keywords and results).
Sources: test/SelfOrganizingMapTest/Trainer.cpp, Mapper.cpp; test/CudaTest/mapper.cu, compare_trainer_cpu.cu,
compare_trainer_mixed.cu; test/PythonBindingTest/DynamicTrainer.cpp; python/pink/train.py."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["pink_b200._pink", "pink_b200.pink"])
def pink(request):
    import importlib
    return importlib.import_module(request.param)


class StepFunctor:                      # src/UtilitiesLib/DistributionFunctor.cpp:14-22
    def __init__(self, value):
        self.value = value

    def __call__(self, d):
        return 1.0 if d <= self.value else 0.0


def test_trainer_num_rot(cuda, pink):
    """test/SelfOrganizingMapTest/Trainer.cpp:22-42"""
    som = pink.SOM(np.zeros((2, 2, 2, 2), np.float32))
    for R in (0, 3, 90):
        with pytest.raises(RuntimeError, match="Number of rotations"):
            pink.Trainer(som, number_of_rotations=R, use_flip=False, max_update_distance=1.0, euclidean_distance_dim=2)
    for R in (1, 4, 720):
        pink.Trainer(som, number_of_rotations=R, use_flip=False, max_update_distance=1.0, euclidean_distance_dim=2)


def test_trainer_cartesian_2d_float_step_function(cuda, pink):
    """test/SelfOrganizingMapTest/Trainer.cpp:66-88: expected neuron {6, 7, 10, 11}."""
    som = pink.SOM(np.zeros((1, 1, 2, 2), np.float32))
    trainer = pink.Trainer(som, StepFunctor(10.0), 0, 1, False, 0.0, pink.Interpolation.BILINEAR,
                           euclidean_distance_dim=2, euclidean_distance_type=pink.DataType.FLOAT)
    trainer(pink.Data(np.arange(1, 17, dtype=np.float32).reshape(4, 4)))
    trainer.update_som()
    assert np.array(som, copy=False).ravel().tolist() == [6.0, 7.0, 10.0, 11.0]


def test_trainer_cartesian_3d(cuda, pink):
    """test/SelfOrganizingMapTest/Trainer.cpp:90-151"""
    raw = np.zeros((2, 2, 2, 2, 2), np.float32)
    raw[0, 1] = np.array([4, 3, 2, 1, 8, 7, 6, 5], np.float32).reshape(2, 2, 2)
    som = pink.SOM(raw, neuron_layout="cartesian-3d")
    trainer = pink.Trainer(som, StepFunctor(0.0), 0, 4, False, 0.0, euclidean_distance_dim=2,
                           euclidean_distance_type=pink.DataType.FLOAT)
    trainer(pink.Data(np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2), layout="cartesian-3d"))
    trainer.update_som()
    assert np.array(som)[0, 1].ravel().tolist() == [4, 3, 2, 1, 8, 7, 6, 5]
    assert trainer.get_update_info().tolist() == [0, 1, 0, 0]


@pytest.mark.parametrize("dtype", ["FLOAT", "UINT8", "UINT16"])
@pytest.mark.parametrize("row", [(1, 2, 2, 2, 1, False), (1, 3, 3, 2, 1, False), (1, 3, 3, 2, 360, False),
                                 (2, 3, 3, 2, 360, False), (2, 3, 3, 2, 360, True)])
def test_mapper_exact_values(cuda, pink, row, dtype):
    """test/CudaTest/mapper.cu:55-120: image 0 against SOM 1 maps to exactly 2.0 in all three modes."""
    som_dim, nd, idim, ed, R, flip = row
    som = pink.SOM(np.ones((som_dim, som_dim, nd, nd), np.float32))
    mapper = pink.Mapper(som, 0, R, flip, pink.Interpolation.BILINEAR, euclidean_distance_dim=ed,
                         euclidean_distance_type=getattr(pink.DataType, dtype))
    dist, rot = mapper(pink.Data(np.zeros((idim, idim), np.float32)))
    assert dist == [2.0] * (som_dim * som_dim) and isinstance(rot[0], int)


@pytest.mark.parametrize("row", [(1, 2, 2, 2, 1, False, 0.0, 0.5, 1.0), (1, 2, 2, 2, 1, False, 0.5, 0.5, 0.0),
                                 (2, 3, 5, 2, 360, True, 0.0, 1.0, 2.0), (1, 3, 5, 2, 360, False, 1.0, 0.0, 2.0)])
def test_mapper_float_table(cuda, pink, row):
    """test/SelfOrganizingMapTest/Mapper.cpp:80-98 (float)."""
    som_dim, nd, idim, ed, R, flip, nv, iv, want = row
    som = pink.SOM(np.full((som_dim, som_dim, nd, nd), nv, np.float32))
    mapper = pink.Mapper(som, number_of_rotations=R, use_flip=flip, euclidean_distance_dim=ed,
                         euclidean_distance_type=pink.DataType.FLOAT)
    dist, _ = mapper(pink.Data(np.full((idim, idim), iv, np.float32)))
    np.testing.assert_allclose(dist, [want] * som_dim ** 2, rtol=1e-6, atol=1e-6)


COMPARE = [(2, 2, 2, 2, 1, False), (2, 2, 2, 2, 4, False), (2, 2, 2, 2, 8, True), (2, 4, 4, 4, 1, False),
           (2, 2, 4, 4, 1, False), (2, 64, 45, 45, 360, True), (2, 64, 100, 100, 360, True), (2, 64, 100, 45, 360, True),
           (2, 124, 91, 64, 360, True), (2, 4, 2, 2, 8, True)]


@pytest.mark.parametrize("p", COMPARE)
def test_compare_trainer_with_reference_cpu(cuda, pink, p):
    """test/CudaTest/compare_trainer_cpu.cu:49-98: one step, random image and SOM, GPU float against the
    reference CPU path within 1e-4 absolute (here: the oracle, which equals the reference CPU bit for bit)."""
    som_dim, idim, nd, ed, R, flip = p
    rng = np.random.default_rng(sum(p))
    img = rng.random((idim, idim), dtype=np.float32)
    som0 = rng.random((som_dim, som_dim, nd, nd), dtype=np.float32)
    som = pink.SOM(som0)
    trainer = pink.Trainer(som, pink.GaussianFunctor(1.1, 0.2), 0, R, flip, -1.0, pink.Interpolation.BILINEAR,
                           euclidean_distance_dim=ed, euclidean_distance_type=pink.DataType.FLOAT)
    trainer(pink.Data(img))
    trainer.update_som()
    want = som0.reshape(som_dim * som_dim, 1, nd, nd).copy()
    O.train_step(want, img, O.update_factors(0, som_dim, som_dim, 0, 1.1, 0.2), ed, R, flip, O.MODE_F32)
    np.testing.assert_allclose(np.array(som).ravel(), want.ravel(), atol=1e-4, rtol=0)


@pytest.mark.parametrize("p", COMPARE[:8])
def test_compare_trainer_mixed_precision(cuda, pink, p):
    """test/CudaTest/compare_trainer_mixed.cu:49-93: float and uint8 training agree within 1e-4 (same BMU and
    best rotations) for one step on random inputs."""
    som_dim, idim, nd, ed, R, flip = p
    rng = np.random.default_rng(sum(p) + 1)
    img = rng.random((idim, idim), dtype=np.float32)
    som0 = rng.random((som_dim, som_dim, nd, nd), dtype=np.float32)
    out = []
    for dt in (pink.DataType.FLOAT, pink.DataType.UINT8):
        som = pink.SOM(som0)
        trainer = pink.Trainer(som, pink.GaussianFunctor(1.1, 0.2), 0, R, flip, 0.0, euclidean_distance_dim=ed,
                               euclidean_distance_type=dt)
        trainer(pink.Data(img))
        trainer.update_som()
        out.append(np.array(som).copy())
    np.testing.assert_allclose(out[0], out[1], atol=1e-4, rtol=0)


@pytest.mark.parametrize("layout,shape", [("cartesian-2d", (3, 3, 12, 12)), ("hexagonal-2d", (19, 12, 12))])
def test_dynamic_trainer_layouts_like_train_py(cuda, pink, layout, shape):
    """test/PythonBindingTest/DynamicTrainer.cpp:29-73 and python/pink/train.py:103-118: cartesian and hexagonal
    SOMs, uint8, several images; here also checked against the oracle."""
    rng = np.random.default_rng(5)
    som0 = rng.random(shape, dtype=np.float32)
    imgs = rng.random((5, 16, 16), dtype=np.float32)
    som = pink.SOM(som0, som_layout=layout)
    assert som.get_som_layout() == layout
    trainer = pink.Trainer(som, euclidean_distance_dim=8, verbosity=0,
                           distribution_function=pink.GaussianFunctor(sigma=1.1, damping=1.0),
                           number_of_rotations=16, interpolation=pink.Interpolation.BILINEAR,
                           euclidean_distance_type=pink.DataType.UINT8)
    for i in range(imgs.shape[0]):
        trainer(pink.Data(imgs[i]))
    trainer.update_som()
    lay, d0, d1 = (0, 3, 3) if layout == "cartesian-2d" else (1, 5, 5)
    want = som0.reshape(-1, 1, 12, 12).copy()
    F = O.update_factors(lay, d0, d1, 0, 1.1, 1.0)
    for im in imgs:
        O.train_step(want, im, F, 8, 16, True, O.MODE_U8)
    assert np.array_equal(np.array(som, copy=False).reshape(want.shape).view(np.uint32), want.view(np.uint32))
    assert trainer.get_update_info().sum() == 5


def test_images_given_one_by_one_equal_one_batch(cuda, pink):
    """Trainer.__call__ collects images and hands them to the device in batches; the map after update_som() is the
    one a single train() call over the same images gives, whatever the number of images (more than one batch,
    not a whole number of them) and with a train() call in between."""
    rng = np.random.default_rng(8)
    som0 = rng.random((4, 4, 12, 12), dtype=np.float32)
    imgs = rng.random((37, 16, 16), dtype=np.float32)
    a, b = pink.SOM(som0), pink.SOM(som0)
    ta = pink.Trainer(a, pink.GaussianFunctor(1.1, 0.3), number_of_rotations=8, euclidean_distance_dim=8)
    tb = pink.Trainer(b, pink.GaussianFunctor(1.1, 0.3), number_of_rotations=8, euclidean_distance_dim=8)
    for i in range(20):
        ta(pink.Data(imgs[i]))
    ta.train(imgs[20:30])
    for i in range(30, 37):
        ta(pink.Data(imgs[i]))
    assert ta.get_update_info().sum() == 37
    ta.update_som()
    tb.train(imgs)
    tb.update_som()
    assert np.array_equal(np.array(a).view(np.uint32), np.array(b).view(np.uint32))


def test_python_callable_distribution_function(cuda, pink):
    """Any Python callable works as distribution_function (pybind11/functional.h in the reference)."""
    som0 = np.random.default_rng(1).random((3, 3, 8, 8), dtype=np.float32)
    img = np.random.default_rng(2).random((10, 10), dtype=np.float32)
    g = pink.GaussianFunctor(1.3, 0.4)
    a, b = pink.SOM(som0), pink.SOM(som0)
    ta = pink.Trainer(a, g, number_of_rotations=8, euclidean_distance_dim=5)
    tb = pink.Trainer(b, lambda d: g(d), number_of_rotations=8, euclidean_distance_dim=5, max_update_distance=-1.0)
    for t in (ta, tb):
        t(pink.Data(img))
        t.update_som()
    assert np.array_equal(np.array(a), np.array(b))


def test_error_texts(cuda, pink):
    som = pink.SOM(np.zeros((2, 2, 4, 4), np.float32))
    with pytest.raises((RuntimeError, TypeError)):      # the reference's binding has no default for it: TypeError there
        pink.Trainer(som)
    with pytest.raises(RuntimeError, match="euclidean_distance_dim not defined"):
        pink.Trainer(som, euclidean_distance_dim=0)
    with pytest.raises(RuntimeError, match="data-type not supported"):
        pink.SOM(np.zeros((2, 2, 4, 4)), data_type="float64")
    with pytest.raises(RuntimeError, match="is not supported"):
        pink.SOM(np.zeros((2, 2, 4, 4), np.float32), som_layout="cartesian-3d")
    with pytest.raises(RuntimeError, match="Euclidean distance dimension larger than neuron dimension"):
        pink.Mapper(som, euclidean_distance_dim=5)
    t = pink.Trainer(som, euclidean_distance_dim=2, number_of_rotations=4)
    with pytest.raises(RuntimeError, match="Images must be quadratic"):
        t(pink.Data(np.zeros((4, 6), np.float32)))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        pink.Trainer(som, euclidean_distance_dim=2, use_gpu=False)
