"""Drop-in mirror of the reference's Python module ``pink`` (src/pink/pink.cpp:25-153) on the B200 library.

    import pink_b200.pink as pink
    som = pink.SOM(np_som)                                   # float32 (w, h, nd, nd) or (N, nd, nd) for hexagonal
    trainer = pink.Trainer(som, euclidean_distance_dim=45, number_of_rotations=360,
                           distribution_function=pink.GaussianFunctor(sigma=1.1, damping=1.0),
                           euclidean_distance_type=pink.DataType.UINT8)
    trainer(pink.Data(image)); trainer.update_som(); np.array(som, copy=False)
    mapper = pink.Mapper(som, euclidean_distance_dim=45); distances, rotations = mapper(pink.Data(image))

Same class names, constructor keywords, defaults, return types and error texts as the reference.  All numerical work
runs in the CUDA library through ``pink_b200.engine``; ``use_gpu=False`` is refused because this package has no CPU
implementation.  ``Trainer.train`` / ``Mapper.map`` are additions that take many images per call.
"""
import enum
import math

import numpy as np

from . import capi, engine

__version__ = "2.5 (pink_b200 %s)" % capi.lib.pink_b200_version().decode()


class Interpolation(enum.IntEnum):
    NEAREST_NEIGHBOR = 0
    BILINEAR = 1


class DataType(enum.IntEnum):
    FLOAT = 0
    UINT16 = 1
    UINT8 = 2


class Layout(enum.IntEnum):
    CARTESIAN = 0
    HEXAGONAL = 1


class EuclideanDistanceShape(enum.IntEnum):
    QUADRATIC = 0
    CIRCULAR = 1


# pybind11's export_values(): the enumerators are also module attributes
NEAREST_NEIGHBOR, BILINEAR = Interpolation.NEAREST_NEIGHBOR, Interpolation.BILINEAR
FLOAT, UINT16, UINT8 = DataType.FLOAT, DataType.UINT16, DataType.UINT8
CARTESIAN, HEXAGONAL = Layout.CARTESIAN, Layout.HEXAGONAL
QUADRATIC, CIRCULAR = EuclideanDistanceShape.QUADRATIC, EuclideanDistanceShape.CIRCULAR


class GaussianFunctor:
    """damping / (sigma * sqrt(2 pi)) * exp(-0.5 * (d / sigma)^2) in float32
    (src/UtilitiesLib/DistributionFunctor.cpp:24-33)."""

    def __init__(self, sigma=1.1, damping=0.2):
        self.sigma, self.damping = float(sigma), float(damping)

    def __call__(self, distance):
        f32 = np.float32
        s, d = f32(self.sigma), f32(self.damping)
        q = f32(f32(distance) / s)
        return float(f32(f32(d / f32(s * f32(math.sqrt(f32(2.0) * f32(math.pi))))) * f32(math.exp(f32(-0.5) * f32(q * q)))))


def _as_float32(buf, data_type):
    if data_type != "float32":
        raise RuntimeError("data-type not supported")
    return np.array(buf, dtype=np.float32, order="C", copy=True)      # the reference copies the buffer as well


class Data:
    """pink.Data(buffer, data_type="float32", layout="cartesian-2d") (src/pink/pink.cpp:60-81, DynamicData.cpp:15-43)."""

    def __init__(self, buf, data_type="float32", layout="cartesian-2d"):
        self._a = _as_float32(buf, data_type)
        want = {"cartesian-1d": 1, "cartesian-2d": 2, "cartesian-3d": 3}
        if layout not in want:
            raise RuntimeError("layout " + layout + " is not supported")
        if self._a.ndim != want[layout]:
            raise RuntimeError("layout " + layout + " does not match a buffer of %d dimensions" % self._a.ndim)
        self.layout = layout

    def __array__(self, dtype=None, copy=None):
        return self._a if dtype in (None, np.float32) else self._a.astype(dtype)


class SOM:
    """pink.SOM(buffer, data_type="float32", som_layout="cartesian-2d", neuron_layout="cartesian-2d")
    (src/pink/pink.cpp:83-111, DynamicSOM.cpp:15-48).  ``np.array(som, copy=False)`` exposes the SOM's own storage,
    which holds the trained weights after ``Trainer.update_som()``."""

    def __init__(self, buf, data_type="float32", som_layout="cartesian-2d", neuron_layout="cartesian-2d"):
        self._a = _as_float32(buf, data_type)
        ndim_neuron = {"cartesian-1d": 1, "cartesian-2d": 2, "cartesian-3d": 3}.get(neuron_layout)
        if ndim_neuron is None:
            raise RuntimeError("neuron layout " + neuron_layout + " is not supported")
        shape = self._a.shape
        if som_layout == "cartesian-2d":
            if len(shape) != 2 + ndim_neuron:
                raise RuntimeError("SOM buffer must have shape (som_w, som_h, neuron...)")
            self._layout, self._dim0, self._dim1 = capi.LAYOUT_CARTESIAN, shape[0], shape[1]
            self.neuron_shape = shape[2:]
        elif som_layout == "hexagonal-2d":
            if len(shape) != 1 + ndim_neuron:
                raise RuntimeError("hexagonal SOM buffer must have shape (number_of_neurons, neuron...)")
            dim = int(math.sqrt((4 * shape[0] - 1) // 3))            # HexagonalLayout::get_dim_from_size
            if engine.som_size(capi.LAYOUT_HEXAGONAL, dim, dim) != shape[0]:
                raise RuntimeError("%d is not the size of a hexagonal SOM" % shape[0])
            self._layout, self._dim0, self._dim1 = capi.LAYOUT_HEXAGONAL, dim, dim
            self.neuron_shape = shape[1:]
        else:
            raise RuntimeError("SOM layout " + som_layout + " is not supported")
        self._som_layout, self._neuron_layout = som_layout, neuron_layout
        self.number_of_neurons = engine.som_size(self._layout, self._dim0, self._dim1)

    def get_som_layout(self):
        return self._som_layout

    def __array__(self, dtype=None, copy=None):
        return self._a if dtype in (None, np.float32) else self._a.astype(dtype)

    # geometry of a neuron as the library wants it: channels, side
    def _neuron_geometry(self):
        ns = self.neuron_shape
        if self._neuron_layout == "cartesian-1d":
            raise RuntimeError("Not implemented yet.")                   # generate_rotated_images.h:37-47
        if self._neuron_layout == "cartesian-2d":
            channels, h, w = 1, ns[0], ns[1]
        else:
            channels, h, w = ns
        if h != w:
            raise RuntimeError("neurons must be quadratic")
        return channels, h


def _image_geometry(data, channels):
    a = np.asarray(data)
    if a.ndim == 2:
        c, h, w = 1, a.shape[0], a.shape[1]
    elif a.ndim == 3:
        c, h, w = a.shape
    else:
        raise RuntimeError("Not implemented yet.")
    if h != w:
        raise RuntimeError("Images must be quadratic.")                  # generate_rotated_images.h:69-71
    if c != channels:
        raise RuntimeError("image has %d channels, the SOM neurons have %d" % (c, channels))
    return h


class _Common:
    def __init__(self, som, number_of_rotations, use_flip, interpolation, use_gpu, euclidean_distance_dim,
                 euclidean_distance_shape, euclidean_distance_type):
        if not isinstance(som, SOM):
            raise TypeError("som must be a pink.SOM")
        if not use_gpu:
            raise RuntimeError("CPU execution is not supported by pink_b200 (there is no CPU fallback)")
        if euclidean_distance_dim == 0:
            raise RuntimeError("euclidean_distance_dim not defined")     # DynamicTrainer.cpp:25
        if number_of_rotations == 0 or (number_of_rotations != 1 and number_of_rotations % 4 != 0):
            raise RuntimeError("Number of rotations must be 1 or larger then 1 and divisible by 4")
        self._som = som
        self._channels, self._neuron_dim = som._neuron_geometry()
        if euclidean_distance_dim > self._neuron_dim:
            raise RuntimeError("Euclidean distance dimension larger than neuron dimension")
        self._args = dict(n_rotations=int(number_of_rotations), use_flip=bool(use_flip),
                          dist_type=int(euclidean_distance_type), ed_shape=int(euclidean_distance_shape),
                          interpolation=int(interpolation))
        self._ed = int(euclidean_distance_dim)
        self._eng = None

    def _engine(self, data):
        idim = _image_geometry(data, self._channels)
        if self._eng is None:
            try:
                self._eng = engine.Engine(self._som.number_of_neurons, self._channels, idim, self._neuron_dim,
                                          self._ed, **self._args)
            except capi.PinkError as e:
                raise RuntimeError(str(e)) from None
            self._image_dim = idim
            self._eng.set_som(np.asarray(self._som))
            self._configure()
        elif idim != self._image_dim:
            raise RuntimeError("all images must have the size of the first one")
        return self._eng

    def _configure(self):
        pass


class Trainer(_Common):
    """pink.Trainer (src/pink/pink.cpp:113-135, DynamicTrainer.h:20-90); one call trains on one image."""

    def __init__(self, som, distribution_function=GaussianFunctor(1.1, 0.2), verbosity=0, number_of_rotations=360,
                 use_flip=True, max_update_distance=-1.0, interpolation=Interpolation.BILINEAR, use_gpu=True,
                 euclidean_distance_dim=0, euclidean_distance_shape=EuclideanDistanceShape.QUADRATIC,
                 euclidean_distance_type=DataType.UINT8):
        super().__init__(som, number_of_rotations, use_flip, interpolation, use_gpu, euclidean_distance_dim,
                         euclidean_distance_shape, euclidean_distance_type)
        self._lut = self._update_lut(distribution_function, float(max_update_distance))

    def _update_lut(self, func, max_update_distance):
        """factor(i, j) = func(distance(i, j)) if max_update_distance <= 0 or distance < max_update_distance, else 0
        (TrainerCommon, src/SelfOrganizingMapLib/Trainer.h:69-76) -- held as one value per DISTINCT map distance (a
        SOM grid has few), which gives the factors N^2 evaluations would give without an N x N table.  The built-in
        Gaussian is evaluated by the library in float32 exactly as the reference does; any other callable is
        called once per distinct distance."""
        s = self._som
        if type(func) is GaussianFunctor:
            n = capi.lib.pink_b200_distance_classes(s._layout, s._dim0, s._dim1, 1, None, 0)
            lut = np.empty(n, np.float32)
            capi.check(capi.lib.pink_b200_update_lut(s._layout, s._dim0, s._dim1, 1, capi.FUNC_GAUSSIAN, func.sigma,
                                                     func.damping, max_update_distance, lut.ctypes.data, n))
            return lut
        dist = engine.distance_classes(s._layout, s._dim0, s._dim1)
        lut = np.array([func(float(v)) for v in dist], np.float32)
        if max_update_distance > 0:
            lut[dist >= np.float32(max_update_distance)] = 0.0
        return lut

    def _configure(self):
        s = self._som
        self._eng.set_update_lut(s._layout, s._dim0, s._dim1, self._lut)

    _DEFER = 16          # images collected before they go to the device

    def __call__(self, data):
        """One image.  Nothing of a training step can be observed before update_som() / get_update_info(), so the
        images are collected and handed to the device _DEFER at a time: whole batches of steps run in one launch."""
        self._engine(data)
        pending = self.__dict__.setdefault("_pending", [])
        pending.append(np.array(data, dtype=np.float32, copy=True))
        if len(pending) == self._DEFER:
            self._flush()

    def _flush(self):
        pending = self.__dict__.get("_pending")
        if pending:
            images = np.stack(pending)
            pending.clear()
            self._eng.train(images)

    def train(self, images):
        """Sequential training steps over an array of images (n, id, id) or (n, C, id, id) in one call."""
        images = np.ascontiguousarray(images, dtype=np.float32)
        self._engine(images[0])
        self._flush()
        self._eng.train(images)

    def update_som(self):
        """Copies the trained weights into the SOM's storage (Trainer.h:306-309)."""
        if self._eng is not None:
            self._flush()
            self._eng.synchronize()
            flat = np.asarray(self._som).reshape(self._som.number_of_neurons, -1)
            self._eng.get_som(flat)

    def get_update_info(self):
        """Number of times each neuron was the best matching unit (TrainerCommon::get_update_info)."""
        if self._eng is None:
            return np.zeros(self._som.number_of_neurons, np.uint32)
        self._flush()
        return self._eng.update_counts()


class Mapper(_Common):
    """pink.Mapper (src/pink/pink.cpp:137-152, DynamicMapper.h:20-68): returns (distances, best transforms)."""

    def __init__(self, som, verbosity=0, number_of_rotations=360, use_flip=True, interpolation=Interpolation.BILINEAR,
                 use_gpu=True, euclidean_distance_dim=0, euclidean_distance_shape=EuclideanDistanceShape.QUADRATIC,
                 euclidean_distance_type=DataType.UINT8):
        super().__init__(som, number_of_rotations, use_flip, interpolation, use_gpu, euclidean_distance_dim,
                         euclidean_distance_shape, euclidean_distance_type)

    def __call__(self, data):
        dist, rot = self._engine(data).map(np.asarray(data))
        return dist[0].tolist(), rot[0].tolist()

    def map(self, images):
        """(n, N) float32 distances and (n, N) uint32 transforms for an array of images."""
        images = np.ascontiguousarray(images, dtype=np.float32)
        return self._engine(images[0]).map(images)
