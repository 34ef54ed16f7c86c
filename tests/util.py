"""Helpers shared by the tests: synthetic inputs and thin wrappers that run
single stages of the CUDA library on torch-allocated device buffers."""
import ctypes as C

import numpy as np


def make_config(capi, N, channels, idim, nd, ed, R, flip, mode, rank=0, world=1, max_batch=0, device=0):
    return capi.Config(N, channels, idim, nd, ed, capi.QUADRATIC, R, int(flip), mode, capi.BILINEAR, device,
                       rank, world, max_batch)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def split_key(keys, mode):
    shift = 16 if mode == 1 else 32
    keys = np.asarray(keys, dtype=np.uint64)
    return keys >> np.uint64(shift), (keys & np.uint64((1 << shift) - 1)).astype(np.uint32)


class Context:
    """Test-side wrapper of pink_b200.engine.Engine keyed by a prepared Config."""

    def __init__(self, capi, cfg, options=None):
        from pink_b200.engine import Engine
        self.cfg = cfg
        self.e = Engine(cfg.n_neurons, cfg.channels, cfg.image_dim, cfg.neuron_dim, cfg.ed_dim, cfg.n_rotations,
                        cfg.use_flip, cfg.dist_type, cfg.device, cfg.rank, cfg.world_size, cfg.max_batch,
                        cfg.ed_shape, cfg.interpolation, options=options)
        self.first, self.count = self.e.first, self.e.count

    def set_som(self, som):
        self.e.set_som(som)

    def get_som(self, like):
        return self.e.get_som(np.zeros_like(np.ascontiguousarray(like, dtype=np.float32)))

    def set_factors(self, F):
        self.e.set_update_factors(F)

    def train(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        n = images.size // self.e.image_size
        self.e.train(images)
        self.e.synchronize()
        return self.e.bmu_log(n)

    def counts(self):
        return self.e.update_counts()

    def map(self, images):
        return self.e.map(images)

    def close(self):
        self.e.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
