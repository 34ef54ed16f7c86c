"""Seeded synthetic inputs with the shapes and value distributions of the
reference's image sets (which are not redistributable with this package):
Gaussian-blob images and a uniform SOM initialisation."""
import numpy as np


def blob_images(n, dim, channels=1, seed=0):
    """Per image: the sum of 1-3 elliptical 2-D Gaussians (centre within the
    central 40 %, major-axis sigma 2-12 px, axis ratio 0.3-1, uniform position
    angle, amplitude U(0.2, 1)) plus N(0, 0.01) noise, clipped at 0 and
    normalised to max = 1.  Further channels repeat the blobs shifted by up to
    3 px and rescaled by U(0.5, 1.5) with independent noise.
    Returns float32 (n, dim, dim) for one channel, else (n, channels, dim, dim)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    yy, xx = np.mgrid[0:dim, 0:dim].astype(np.float64)
    out = np.empty((n, channels, dim, dim), np.float32)
    for i in range(n):
        k = rng.integers(1, 4)
        blobs = []
        for _ in range(k):
            cx, cy = rng.uniform(0.3 * dim, 0.7 * dim, 2)
            blobs.append((cx, cy, rng.uniform(2, 12), rng.uniform(0.3, 1.0), rng.uniform(0, np.pi),
                          rng.uniform(0.2, 1.0)))
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


def mt19937_uniform(n, seed=1234):
    """uniform [0, 1) float32 from a 32-bit Mersenne Twister, one draw per value:
    float32(draw) / 2^32, with values that round up to 1 replaced by the largest
    float below 1 -- the sequence libstdc++ produces for
    std::uniform_real_distribution<float>(0, 1) over std::mt19937(seed), which the
    reference uses to initialise a random SOM (src/UtilitiesLib/Filler.h:16-25)."""
    rs = np.random.RandomState(seed)
    draws = rs.randint(0, 2 ** 32, size=n, dtype=np.uint64).astype(np.uint32)
    vals = draws.astype(np.float32) / np.float32(4294967296.0)
    vals[vals >= 1.0] = np.nextafter(np.float32(1.0), np.float32(0.0))
    return vals
