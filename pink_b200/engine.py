"""Python front-end of the C ABI: one `Engine` owns one pink_b200 context.

Everything here is argument marshalling; all computation happens in the CUDA
library (`pink_b200.capi`).  Arrays are numpy float32 / uint32, C-contiguous.
"""
import ctypes as C

import numpy as np

from . import capi


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


def som_size(layout, dim0, dim1):
    return int(capi.lib.pink_b200_som_size(layout, dim0, dim1))


def shard_range(n_neurons, world_size, rank):
    """(first, count) of the contiguous neuron shard of `rank` (host computation)."""
    first, count = C.c_uint32(), C.c_uint32()
    rc = capi.lib.pink_b200_shard_range(n_neurons, world_size, rank, C.byref(first), C.byref(count))
    if rc != capi.OK:
        raise capi.PinkError(rc, "invalid shard request")
    return first.value, count.value


def update_factors(layout, dim0, dim1, func=capi.FUNC_GAUSSIAN, p0=1.1, p1=0.2, max_update_distance=-1.0):
    """N x N table F[bmu, n] of the built-in neighbourhood functions (host computation)."""
    N = som_size(layout, dim0, dim1)
    F = np.empty((N, N), np.float32)
    rc = capi.lib.pink_b200_update_factors(layout, dim0, dim1, func, p0, p1, max_update_distance, _vp(F))
    if rc != capi.OK:
        raise capi.PinkError(rc, "invalid SOM layout or neighbourhood function")
    return F


def distance_classes(layout, dim0, dim1, dim2=1):
    """Distances of the distinct map-distance classes of a SOM grid (float32 array, class order)."""
    n = int(capi.lib.pink_b200_distance_classes(layout, dim0, dim1, dim2, None, 0))
    if n == 0:
        raise capi.PinkError(capi.EINVAL, "unsupported SOM layout")
    d = np.empty(n, np.float32)
    capi.lib.pink_b200_distance_classes(layout, dim0, dim1, dim2, _vp(d), n)
    return d


class Engine:
    """Device state of one trainer/mapper (one neuron shard when world_size > 1)."""

    def __init__(self, n_neurons, channels, image_dim, neuron_dim, ed_dim, n_rotations=360, use_flip=True,
                 dist_type=capi.UINT8, device=0, rank=0, world_size=1, max_batch=0,
                 ed_shape=capi.QUADRATIC, interpolation=capi.BILINEAR, options=None):
        self.cfg = capi.Config(n_neurons, channels, image_dim, neuron_dim, ed_dim, ed_shape, n_rotations,
                               int(bool(use_flip)), dist_type, interpolation, device, rank, world_size, max_batch)
        self._h = C.c_void_p()
        capi.check(capi.lib.pink_b200_create(C.byref(self.cfg), C.byref(self._h)))
        first, count = C.c_uint32(), C.c_uint32()
        capi.check(capi.lib.pink_b200_shard(self._h, C.byref(first), C.byref(count)))
        self.first, self.count = first.value, count.value
        self.image_size = channels * image_dim * image_dim
        self.neuron_size = channels * neuron_dim * neuron_dim
        self._read_shard()
        for name, value in (options or {}).items():
            self.set_option(name, value)

    def set_option(self, name, value):
        """Switches of the context (see pink_b200_set_option); before comm_init / set_som."""
        capi.check(capi.lib.pink_b200_set_option(self._h, name.encode(), int(value)))
        self._read_shard()

    def _read_shard(self):
        first, count = C.c_uint32(), C.c_uint32()
        capi.check(capi.lib.pink_b200_shard(self._h, C.byref(first), C.byref(count)))
        self.first, self.count = first.value, count.value
        self.stride = int(capi.lib.pink_b200_shard_stride(self._h))

    @property
    def neurons(self):
        """Global indices of this context's neurons, in its local order."""
        return self.first + self.stride * np.arange(self.count)

    # -- life cycle ---------------------------------------------------------
    def close(self):
        if self._h:
            capi.lib.pink_b200_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        if capi is not None:          # interpreter shutdown may have cleared the module
            self.close()

    # -- multi-GPU ----------------------------------------------------------
    @staticmethod
    def unique_id():
        buf = (C.c_ubyte * 128)()
        capi.check(capi.lib.pink_b200_comm_unique_id(buf))
        return bytes(buf)

    def comm_init(self, unique_id):
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        capi.check(capi.lib.pink_b200_comm_init(self._h, buf))

    # -- state --------------------------------------------------------------
    def set_som(self, som):
        som = np.ascontiguousarray(som, dtype=np.float32)
        if som.size != self.cfg.n_neurons * self.neuron_size:
            raise ValueError("SOM has %d elements, expected %d" % (som.size, self.cfg.n_neurons * self.neuron_size))
        capi.check(capi.lib.pink_b200_set_som(self._h, _vp(som)))

    def get_som(self, out):
        """Writes this shard's rows into `out` (whole-SOM array) and returns it."""
        assert out.dtype == np.float32 and out.flags.c_contiguous
        capi.check(capi.lib.pink_b200_get_som(self._h, _vp(out)))
        return out

    def set_update_factors(self, F):
        F = np.ascontiguousarray(F, dtype=np.float32)
        if F.size != self.cfg.n_neurons ** 2:
            raise ValueError("update factor table must be N x N")
        capi.check(capi.lib.pink_b200_set_update_factors(self._h, _vp(F)))

    def set_update_function(self, layout, dim0, dim1, func=capi.FUNC_GAUSSIAN, p0=1.1, p1=0.2, max_update_distance=-1.0,
                            dim2=1):
        """Built-in neighbourhood function, one factor per distance class (no N x N table)."""
        capi.check(capi.lib.pink_b200_set_update_function(self._h, layout, dim0, dim1, dim2, func, p0, p1,
                                                          max_update_distance))

    def set_update_lut(self, layout, dim0, dim1, lut, dim2=1):
        """One factor per distance class (order of distance_classes()), e.g. of a Python callable."""
        lut = np.ascontiguousarray(lut, dtype=np.float32)
        capi.check(capi.lib.pink_b200_set_update_lut(self._h, layout, dim0, dim1, dim2, _vp(lut), lut.size))

    # -- training -----------------------------------------------------------
    def _n_images(self, size):
        if size % self.image_size:
            raise ValueError("image buffer is not a whole number of images")
        return size // self.image_size

    def train(self, images):
        """Sequential training steps over host images (any shape holding whole images)."""
        images = np.ascontiguousarray(images, dtype=np.float32)
        capi.check(capi.lib.pink_b200_train(self._h, _vp(images), self._n_images(images.size)))

    def train_device(self, dev_ptr, n):
        capi.check(capi.lib.pink_b200_train_device(self._h, C.c_void_p(dev_ptr), n))

    def exchange_kind(self):
        """0 none, 1 NCCL all-gather per step, 2 peer-memory stores, 3 peer-memory stores and shared rotation work."""
        return int(capi.lib.pink_b200_exchange_kind(self._h))

    def launch_count(self):
        """Kernels launched by this context so far."""
        return int(capi.lib.pink_b200_launch_count(self._h))

    def update_stats(self):
        """(neurons with a non-zero factor, neurons written back), summed over all training steps so far."""
        out = np.zeros(2, np.uint64)
        capi.check(capi.lib.pink_b200_get_update_stats(self._h, _vp(out)))
        return int(out[0]), int(out[1])

    def synchronize(self):
        capi.check(capi.lib.pink_b200_synchronize(self._h))

    def update_counts(self):
        out = np.empty(self.cfg.n_neurons, np.uint32)
        capi.check(capi.lib.pink_b200_get_update_counts(self._h, _vp(out)))
        return out

    def bmu_log(self, n):
        out = np.empty(n, np.uint32)
        capi.check(capi.lib.pink_b200_get_bmu_log(self._h, _vp(out), n))
        return out

    # -- mapping ------------------------------------------------------------
    def map(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        n = self._n_images(images.size)
        dist = np.empty((n, self.count), np.float32)
        rot = np.empty((n, self.count), np.uint32)
        capi.check(capi.lib.pink_b200_map(self._h, _vp(images), n, _vp(dist), _vp(rot)))
        return dist, rot

    def map_device(self, dev_images, n, dev_dist, dev_rot):
        capi.check(capi.lib.pink_b200_map_device(self._h, C.c_void_p(dev_images), n, C.c_void_p(dev_dist),
                                                 C.c_void_p(dev_rot)))

    # -- phase timing ---------------------------------------------------------
    def profile_begin(self, max_steps):
        capi.check(capi.lib.pink_b200_profile_begin(self._h, max_steps))

    def profile_end(self):
        ms = (C.c_double * 4)()
        steps = C.c_uint64()
        capi.check(capi.lib.pink_b200_profile_end(self._h, ms, C.byref(steps)))
        return dict(zip(("rotate", "distance", "bmu", "update"), list(ms))), steps.value

    def profile_detail(self):
        """Persistent-kernel timing of the last profiled pass (see pink_b200_profile_detail)."""
        out = (C.c_double * 8)()
        capi.check(capi.lib.pink_b200_profile_detail(self._h, out))
        keys = ("launch_us", "images_per_launch", "distance_own_us", "barrier1_wait_us", "bmu_list_us",
                "update_own_us", "barrier2_wait_us")
        return dict(zip(keys, list(out)[:7]))

    def map_filter_stats(self):
        """Counters of float32 mapping's estimate + exact pass (see pink_b200_map_filter_stats)."""
        out = (C.c_double * 4)()
        capi.check(capi.lib.pink_b200_map_filter_stats(self._h, out))
        return dict(zip(("pairs_estimated", "pairs_exact", "worst_estimate_error", "error_bound"), list(out)))

    def profile_stamps(self):
        """Raw device-timer stamps of the last profiled pass: uint64 array [steps][blocks][12]."""
        blocks, steps = C.c_uint32(), C.c_uint64()
        capi.check(capi.lib.pink_b200_profile_stamps(self._h, None, 0, C.byref(blocks), C.byref(steps)))
        out = np.zeros((steps.value, blocks.value, 12), np.uint64)
        if out.size:
            capi.check(capi.lib.pink_b200_profile_stamps(self._h, _vp(out), out.size, C.byref(blocks), C.byref(steps)))
        return out

    @property
    def stream(self):
        return capi.lib.pink_b200_stream(self._h)


class Group:
    """All (or the listed) GPUs of this process behind one object: neuron-sharded training, image-sharded mapping
    (pink_b200_group_*).  Arrays are those of the whole map."""

    def __init__(self, n_neurons, channels, image_dim, neuron_dim, ed_dim, n_rotations=360, use_flip=True,
                 dist_type=capi.UINT8, devices=None, max_devices=0, ed_shape=capi.QUADRATIC,
                 interpolation=capi.BILINEAR, options=None):
        self.cfg = capi.Config(n_neurons, channels, image_dim, neuron_dim, ed_dim, ed_shape, n_rotations,
                               int(bool(use_flip)), dist_type, interpolation, 0, 0, 1, 0)
        self._h = C.c_void_p()
        if devices is not None:
            arr = (C.c_int32 * len(devices))(*devices)
            capi.check(capi.lib.pink_b200_group_create(C.byref(self.cfg), arr, len(devices), C.byref(self._h)))
        else:
            capi.check(capi.lib.pink_b200_group_create(C.byref(self.cfg), None, max_devices, C.byref(self._h)))
        self.size = int(capi.lib.pink_b200_group_size(self._h))
        self.image_size = channels * image_dim * image_dim
        self.neuron_size = channels * neuron_dim * neuron_dim
        for name, value in (options or {}).items():
            capi.check(capi.lib.pink_b200_group_set_option(self._h, name.encode(), int(value)))

    def close(self):
        if self._h:
            capi.lib.pink_b200_group_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        if capi is not None:
            self.close()

    def set_som(self, som):
        som = np.ascontiguousarray(som, dtype=np.float32)
        if som.size != self.cfg.n_neurons * self.neuron_size:
            raise ValueError("SOM has %d elements, expected %d" % (som.size, self.cfg.n_neurons * self.neuron_size))
        capi.check(capi.lib.pink_b200_group_set_som(self._h, _vp(som)))

    def get_som(self, out):
        assert out.dtype == np.float32 and out.flags.c_contiguous
        capi.check(capi.lib.pink_b200_group_get_som(self._h, _vp(out)))
        return out

    def set_update_factors(self, F):
        F = np.ascontiguousarray(F, dtype=np.float32)
        if F.size != self.cfg.n_neurons ** 2:
            raise ValueError("update factor table must be N x N")
        capi.check(capi.lib.pink_b200_group_set_update_factors(self._h, _vp(F)))

    def train(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        if images.size % self.image_size:
            raise ValueError("image buffer is not a whole number of images")
        capi.check(capi.lib.pink_b200_group_train(self._h, _vp(images), images.size // self.image_size))

    def synchronize(self):
        capi.check(capi.lib.pink_b200_group_synchronize(self._h))

    def update_counts(self):
        out = np.empty(self.cfg.n_neurons, np.uint32)
        capi.check(capi.lib.pink_b200_group_get_update_counts(self._h, _vp(out)))
        return out

    def map(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        if images.size % self.image_size:
            raise ValueError("image buffer is not a whole number of images")
        n = images.size // self.image_size
        dist = np.empty((n, self.cfg.n_neurons), np.float32)
        rot = np.empty((n, self.cfg.n_neurons), np.uint32)
        capi.check(capi.lib.pink_b200_group_map(self._h, _vp(images), n, _vp(dist), _vp(rot)))
        return dist, rot
