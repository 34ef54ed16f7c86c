"""Helpers shared by the tests: synthetic inputs and thin wrappers that run
single stages of the CUDA library on torch-allocated device buffers."""
import ctypes as C

import numpy as np


def blob_images(n, dim, channels=1, seed=0):
    """Sum of 1-3 elliptical 2-D Gaussians + noise, clipped at 0, max-normalised
    (the synthetic stand-in for the reference's galaxy images)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    yy, xx = np.mgrid[0:dim, 0:dim].astype(np.float64)
    out = np.empty((n, channels, dim, dim), np.float32)
    for i in range(n):
        k = rng.integers(1, 4)
        blobs = []
        for _ in range(k):
            cx, cy = rng.uniform(0.3 * dim, 0.7 * dim, 2)
            s = rng.uniform(2, 12)
            ratio = rng.uniform(0.3, 1.0)
            pa = rng.uniform(0, np.pi)
            amp = rng.uniform(0.2, 1.0)
            blobs.append((cx, cy, s, ratio, pa, amp))
        for c in range(channels):
            img = np.zeros((dim, dim))
            for (cx, cy, s, ratio, pa, amp) in blobs:
                if c > 0:
                    cx, cy = cx + rng.uniform(-3, 3), cy + rng.uniform(-3, 3)
                    amp = amp * rng.uniform(0.5, 1.5)
                dx, dy = xx - cx, yy - cy
                u = dx * np.cos(pa) + dy * np.sin(pa)
                v = -dx * np.sin(pa) + dy * np.cos(pa)
                img += amp * np.exp(-0.5 * ((u / s) ** 2 + (v / (s * ratio)) ** 2))
            img += rng.normal(0, 0.01, img.shape)
            img = np.clip(img, 0, None)
            out[i, c] = (img / img.max()).astype(np.float32)
    return out[:, 0] if channels == 1 else out


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
    """RAII wrapper of pink_b200_ctx for tests."""

    def __init__(self, capi, cfg):
        self.capi = capi
        self.cfg = cfg
        self.h = C.c_void_p()
        capi.check(capi.lib.pink_b200_create(C.byref(cfg), C.byref(self.h)))
        first, count = C.c_uint32(), C.c_uint32()
        capi.check(capi.lib.pink_b200_shard(self.h, C.byref(first), C.byref(count)))
        self.first, self.count = first.value, count.value

    def set_som(self, som):
        som = np.ascontiguousarray(som, dtype=np.float32)
        self.capi.check(self.capi.lib.pink_b200_set_som(self.h, som.ctypes.data_as(C.c_void_p)))

    def get_som(self, like):
        out = np.zeros_like(np.ascontiguousarray(like, dtype=np.float32))
        self.capi.check(self.capi.lib.pink_b200_get_som(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def set_factors(self, F):
        F = np.ascontiguousarray(F, dtype=np.float32)
        self.capi.check(self.capi.lib.pink_b200_set_update_factors(self.h, F.ctypes.data_as(C.c_void_p)))

    def train(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        isz = max(self.cfg.channels, 1) * self.cfg.image_dim ** 2
        n = images.size // isz
        self.capi.check(self.capi.lib.pink_b200_train(self.h, images.ctypes.data_as(C.c_void_p), n))
        self.capi.check(self.capi.lib.pink_b200_synchronize(self.h))
        log = np.empty(n, np.uint32)
        self.capi.check(self.capi.lib.pink_b200_get_bmu_log(self.h, log.ctypes.data_as(C.c_void_p), n))
        return log

    def counts(self):
        out = np.empty(self.cfg.n_neurons, np.uint32)
        self.capi.check(self.capi.lib.pink_b200_get_update_counts(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def map(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        isz = max(self.cfg.channels, 1) * self.cfg.image_dim ** 2
        n = images.size // isz
        dist = np.empty((n, self.count), np.float32)
        rot = np.empty((n, self.count), np.uint32)
        self.capi.check(self.capi.lib.pink_b200_map(self.h, images.ctypes.data_as(C.c_void_p), n,
                                                    dist.ctypes.data_as(C.c_void_p), rot.ctypes.data_as(C.c_void_p)))
        return dist, rot

    def close(self):
        if self.h:
            self.capi.lib.pink_b200_destroy(self.h)
            self.h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
