"""ctypes bindings of the CPU parity checker (TEST INFRASTRUCTURE ONLY).

``oracle.lib`` is the C restatement built from ``oracle/pink_oracle.c``;
``oracle.ref()`` is the reference's own CPU implementation compiled from the
reference source tree into ``oracle/_ref/libpink_ref.so`` (present only where
that tree was available at build time).  Only the test-suite, the smoke check
and the benchmark's CPU-baseline legs may import this package; the shipped
library never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libpink_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libpink_ref.so")
_REF_CUDA = os.path.join(_HERE, "_ref", "libpink_ref_cuda.so")

MODE_F32, MODE_U16, MODE_U8 = 0, 1, 2
FUNC_GAUSSIAN, FUNC_UNITY_GAUSSIAN, FUNC_MEXICAN_HAT, FUNC_STEP = 0, 1, 2, 3
LAYOUT_CARTESIAN, LAYOUT_HEXAGONAL = 0, 1


def build(force=False):
    """Compile the checker (and the reference shim when its sources exist)."""
    src = os.path.join(_HERE, "pink_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libpink_oracle.so"], stdout=subprocess.DEVNULL)
    shim = os.path.join(_HERE, "ref_shim.cpp")
    tree = reference_tree()
    if tree:
        cuda_shim = os.path.join(_HERE, "ref_cuda_shim.cu")
        stale = lambda lib, src: not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(src)
        if force or stale(_REF, shim) or stale(_REF_CUDA, cuda_shim):
            subprocess.check_call(["make", "-C", _HERE, "ref", "PINK_REF=" + tree], stdout=subprocess.DEVNULL,
                                  stderr=subprocess.DEVNULL)


def reference_tree():
    """The reference's source tree: $PINK_REF, else a directory `reference` beside this repository; None if absent."""
    for cand in (os.environ.get("PINK_REF"), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "SelfOrganizingMapLib")):
            return os.path.abspath(cand)
    return None


def _fp(a):
    return a.ctypes.data_as(C.c_void_p)


def _load():
    build()
    lib = C.CDLL(_LIB)
    lib.pko_scaled_distance.restype = C.c_float
    lib.pko_scaled_distance.argtypes = [C.c_uint64, C.c_int]
    lib.pko_ref_cuda_float.restype = C.c_float
    lib.pko_distance_f32_pair.restype = C.c_float
    for n in ("pko_cartesian_distance", "pko_hexagonal_distance", "pko_gaussian", "pko_unity_gaussian",
              "pko_mexican_hat", "pko_step"):
        getattr(lib, n).restype = C.c_float
    lib.pko_cartesian_distance.argtypes = [C.c_uint32] * 4
    lib.pko_cartesian3_distance.restype = C.c_float
    lib.pko_cartesian3_distance.argtypes = [C.c_uint32] * 5
    lib.pko_hexagonal_distance.argtypes = [C.c_uint32] * 3
    lib.pko_gaussian.argtypes = [C.c_float] * 3
    lib.pko_unity_gaussian.argtypes = [C.c_float] * 3
    lib.pko_mexican_hat.argtypes = [C.c_float] * 3
    lib.pko_step.argtypes = [C.c_float] * 2
    lib.pko_hexagonal_size.restype = C.c_uint32
    lib.pko_bmu_f32.restype = C.c_uint32
    lib.pko_bmu_int.restype = C.c_uint32
    return lib


lib = _load()


def have_ref():
    return os.path.exists(_REF)


_ref = None


def ref():
    """The reference-linked library, or None when it was not built."""
    global _ref
    if _ref is None and have_ref():
        r = C.CDLL(_REF)
        r.ref_session_create.restype = C.c_void_p
        r.ref_session_create.argtypes = [C.c_void_p, C.c_int] + [C.c_uint32] * 7 + [C.c_int, C.c_int, C.c_float,
                                                                                   C.c_float, C.c_float, C.c_int]
        r.ref_session_create_shape.restype = C.c_void_p
        r.ref_session_create_shape.argtypes = r.ref_session_create.argtypes + [C.c_int]
        r.ref_session_train.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
        r.ref_session_map.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p,
                                      C.c_void_p]
        r.ref_session_get_som.argtypes = [C.c_void_p, C.c_void_p]
        r.ref_session_get_counts.argtypes = [C.c_void_p, C.c_void_p]
        r.ref_session_destroy.argtypes = [C.c_void_p]
        r.ref_distance_pair.restype = C.c_float
        r.ref_update_factors.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_int, C.c_float, C.c_float, C.c_float,
                                         C.c_void_p]
        r.ref_fill_random_uniform.argtypes = [C.c_void_p, C.c_uint64, C.c_uint32]
        r.ref_set_num_threads.argtypes = [C.c_int]
        _ref = r
    return _ref


# ---------------------------------------------------------------------------
# numpy front-ends of the C restatement
# ---------------------------------------------------------------------------

def n_transforms(R, flip):
    return R * (2 if flip else 1)


def rotation_set(img, nd, R, flip):
    """img: (id, id) or (C, id, id) float32 -> (T, C, nd, nd) float32."""
    img = np.ascontiguousarray(img, dtype=np.float32)
    Cn = 1 if img.ndim == 2 else img.shape[0]
    idim = img.shape[-1]
    out = np.empty((n_transforms(R, flip), Cn, nd, nd), np.float32)
    lib.pko_rotation_set(_fp(img), C.c_uint32(Cn), C.c_uint32(idim), C.c_uint32(nd), C.c_uint32(R),
                         C.c_int(int(flip)), _fp(out))
    return out


_QDT = {MODE_F32: np.float32, MODE_U16: np.uint16, MODE_U8: np.uint8}


SHAPE_QUADRATIC, SHAPE_CIRCULAR = 0, 1


def circle_rows(nd, ed):
    """Neuron-column span [begin, end) of every row of the circular distance region."""
    jb = np.zeros(ed, np.uint32)
    je = np.zeros(ed, np.uint32)
    lib.pko_circle_rows(C.c_uint32(nd), C.c_uint32(ed), _fp(jb), _fp(je))
    return jb, je


def crop_quantize(planes, ed, mode, shape=SHAPE_QUADRATIC):
    """planes: (n, C, nd, nd) float32 -> (n, C*ed*ed) operand of the mode's type (zeros outside a circular region)."""
    planes = np.ascontiguousarray(planes, dtype=np.float32)
    n, Cn, nd, _ = planes.shape
    out = np.empty((n, Cn * ed * ed), _QDT[mode])
    lib.pko_crop_quantize_shape(_fp(planes), C.c_uint32(n), C.c_uint32(Cn), C.c_uint32(nd), C.c_uint32(ed),
                                C.c_int(mode), C.c_int(shape), _fp(out))
    return out


def distance_int(a, b, mode):
    """Exact S[n, t] (uint64) of two integer operands (N, K) and (T, K)."""
    a = np.ascontiguousarray(a, dtype=_QDT[mode])
    b = np.ascontiguousarray(b, dtype=_QDT[mode])
    S = np.empty((a.shape[0], b.shape[0]), np.uint64)
    lib.pko_distance_int(_fp(a), _fp(b), C.c_uint32(a.shape[0]), C.c_uint32(b.shape[0]), C.c_uint32(a.shape[1]),
                         C.c_int(mode), _fp(S))
    return S


def min_over_transforms_int(S):
    S = np.ascontiguousarray(S, dtype=np.uint64)
    smin = np.empty(S.shape[0], np.uint64)
    best = np.empty(S.shape[0], np.uint32)
    lib.pko_min_over_transforms_int(_fp(S), C.c_uint32(S.shape[0]), C.c_uint32(S.shape[1]), _fp(smin), _fp(best))
    return smin, best


def scaled_distance(smin, mode):
    return np.array([lib.pko_scaled_distance(int(s), mode) for s in np.asarray(smin).ravel()], np.float32)


def distance_f32(som, rot, ed, full=False):
    """som (N, C, nd, nd), rot (T, C, nd, nd): reference CPU order float32 distances."""
    som = np.ascontiguousarray(som, dtype=np.float32)
    rot = np.ascontiguousarray(rot, dtype=np.float32)
    N, Cn, nd, _ = som.shape
    T = rot.shape[0]
    dist = np.empty(N, np.float32)
    best = np.empty(N, np.uint32)
    D = np.empty((N, T), np.float32) if full else None
    lib.pko_distance_f32(_fp(som), _fp(rot), C.c_uint32(N), C.c_uint32(T), C.c_uint32(Cn), C.c_uint32(nd),
                         C.c_uint32(ed), _fp(dist), _fp(best), _fp(D) if full else None)
    return (dist, best, D) if full else (dist, best)


def distance_f64(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    D = np.empty((a.shape[0], b.shape[0]), np.float64)
    lib.pko_distance_f64(_fp(a), _fp(b), C.c_uint32(a.shape[0]), C.c_uint32(b.shape[0]), C.c_uint32(a.shape[1]),
                         _fp(D))
    return D


def update(som, rot, best, bmu, factors):
    """In-place neighbourhood update of som (N, P) from rot (T, P)."""
    assert som.dtype == np.float32 and som.flags.c_contiguous
    rot = np.ascontiguousarray(rot, dtype=np.float32)
    best = np.ascontiguousarray(best, dtype=np.uint32)
    factors = np.ascontiguousarray(factors, dtype=np.float32)
    N = som.shape[0]
    P = som.size // N
    lib.pko_update(_fp(som), _fp(rot), _fp(best), C.c_uint32(int(bmu)), _fp(factors), C.c_uint32(N), C.c_uint32(P))
    return som


def update_factors(layout, dim0, dim1, func, p0, p1=0.0, max_update_distance=-1.0):
    N = dim0 * dim1 if layout == LAYOUT_CARTESIAN else int(lib.pko_hexagonal_size(C.c_uint32(dim0)))
    F = np.empty((N, N), np.float32)
    lib.pko_update_factors(C.c_int(layout), C.c_uint32(dim0), C.c_uint32(dim1), C.c_int(func), C.c_float(p0),
                           C.c_float(p1), C.c_float(max_update_distance), _fp(F))
    return F


def update_factors_3d(dims, func, p0, p1=0.0, max_update_distance=-1.0):
    """Factor table of a three-dimensional cartesian SOM with dimensions dims = (dim0, dim1, dim2)."""
    N = int(np.prod(dims))
    F = np.empty((N, N), np.float32)
    lib.pko_update_factors_3d(*[C.c_uint32(int(d)) for d in dims], C.c_int(func), C.c_float(p0), C.c_float(p1),
                              C.c_float(max_update_distance), _fp(F))
    return F


def _shape(som, img):
    N = som.shape[0]
    Cn = 1 if img.ndim == 2 else img.shape[0]
    return N, Cn, img.shape[-1], som.shape[-1]


def train_step(som, img, factors, ed, R, flip, mode, shape=SHAPE_QUADRATIC):
    """One training step in place on som (N, C, nd, nd) or (N, nd, nd).
    Returns (best_rot[N], dist[N], bmu)."""
    assert som.dtype == np.float32 and som.flags.c_contiguous
    img = np.ascontiguousarray(img, dtype=np.float32)
    factors = np.ascontiguousarray(factors, dtype=np.float32)
    N, Cn, idim, nd = _shape(som, img)
    best = np.empty(N, np.uint32)
    dist = np.empty(N, np.float32)
    bmu = C.c_uint32(0)
    rc = lib.pko_train_step_shape(_fp(som), _fp(img), _fp(factors), C.c_uint32(N), C.c_uint32(Cn),
                                  C.c_uint32(idim), C.c_uint32(nd), C.c_uint32(ed), C.c_uint32(R), C.c_int(int(flip)),
                                  C.c_int(mode), C.c_int(shape), _fp(best), _fp(dist), C.byref(bmu))
    assert rc == 0
    return best, dist, bmu.value


def map_image(som, img, ed, R, flip, mode, shape=SHAPE_QUADRATIC):
    som = np.ascontiguousarray(som, dtype=np.float32)
    img = np.ascontiguousarray(img, dtype=np.float32)
    N, Cn, idim, nd = _shape(som, img)
    dist = np.empty(N, np.float32)
    best = np.empty(N, np.uint32)
    rc = lib.pko_map_shape(_fp(som), _fp(img), C.c_uint32(N), C.c_uint32(Cn), C.c_uint32(idim), C.c_uint32(nd),
                           C.c_uint32(ed), C.c_uint32(R), C.c_int(int(flip)), C.c_int(mode), C.c_int(shape),
                           _fp(dist), _fp(best))
    assert rc == 0
    return dist, best


# ---------------------------------------------------------------------------
# front-ends of the reference-linked library (None-safe callers check have_ref)
# ---------------------------------------------------------------------------

class RefSession:
    """One reference Trainer<...,false> or Mapper<...,false> bound to a SOM copy."""

    def __init__(self, som, som_layout, s0, s1, channels, idim, nd, ed, R, flip,
                 func=FUNC_GAUSSIAN, p0=1.1, p1=0.2, max_dist=-1.0, for_map=False, shape=SHAPE_QUADRATIC):
        som = np.ascontiguousarray(som, dtype=np.float32)
        self.N = som.shape[0]
        self.som_shape = som.shape
        self.image_size = max(channels, 1) * idim * idim
        self._h = ref().ref_session_create_shape(_fp(som), som_layout, s0, s1, channels, idim, nd, ed, R, int(flip),
                                                 func, p0, p1, max_dist, int(for_map), int(shape))
        if not self._h:
            raise RuntimeError("reference rejected the configuration")

    def train(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        n = images.size // self.image_size
        ref().ref_session_train(self._h, _fp(images), n, self.image_size)

    def map(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        n = images.size // self.image_size
        dist = np.empty((n, self.N), np.float32)
        rot = np.empty((n, self.N), np.uint32)
        ref().ref_session_map(self._h, _fp(images), n, self.image_size, self.N, _fp(dist), _fp(rot))
        return dist, rot

    def som(self):
        out = np.empty(self.som_shape, np.float32)
        ref().ref_session_get_som(self._h, _fp(out))
        return out

    def counts(self):
        out = np.empty(self.N, np.uint32)
        ref().ref_session_get_counts(self._h, _fp(out))
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            ref().ref_session_destroy(self._h)
            self._h = None


def ref_rotation_set(img, nd, R, flip, as_3d=None):
    img = np.ascontiguousarray(img, dtype=np.float32)
    Cn = 0 if img.ndim == 2 else img.shape[0]
    if as_3d is not None:
        Cn = as_3d
    out = np.empty((n_transforms(R, flip), max(Cn, 1), nd, nd), np.float32)
    ref().ref_rotation_set(_fp(img), C.c_uint32(Cn), C.c_uint32(img.shape[-1]), C.c_uint32(nd), C.c_uint32(R),
                           C.c_int(int(flip)), _fp(out))
    return out


def ref_update_factors(layout, dim0, dim1, func, p0, p1=0.0, max_update_distance=-1.0):
    N = dim0 * dim1 if layout == LAYOUT_CARTESIAN else int(lib.pko_hexagonal_size(C.c_uint32(dim0)))
    F = np.empty((N, N), np.float32)
    ref().ref_update_factors(layout, dim0, dim1, func, p0, p1, max_update_distance, _fp(F))
    return F


def ref_update_factors_3d(dims, func, p0, p1=0.0, max_update_distance=-1.0):
    N = int(np.prod(dims))
    F = np.empty((N, N), np.float32)
    ref().ref_update_factors_3d(*[C.c_uint32(int(d)) for d in dims], C.c_int(func), C.c_float(p0), C.c_float(p1),
                                C.c_float(max_update_distance), _fp(F))
    return F


def ref_fill_random_uniform(n, seed=5489):
    a = np.empty(n, np.float32)
    ref().ref_fill_random_uniform(_fp(a), n, seed)
    return a


# ---------------------------------------------------------------------------
# the reference's own CUDA path, run in a process of its own
# ---------------------------------------------------------------------------

def have_ref_cuda():
    return os.path.exists(_REF_CUDA)


def ref_cuda_run(task, som, images, som_layout, s0, s1, idim, nd, ed, R, flip, mode, sigma=1.1, damping=0.2,
                 timeout=300):
    """Runs the reference's CUDA Trainer (task "train") or Mapper (task "map") on ONE visible GPU in a child process
    (oracle/ref_cuda_worker.py): a failure of that code cannot take the caller's CUDA context with it, and the
    reference's multi-GPU branch is never reached.  som: (N, nd, nd); images: (n, idim, idim).
    Returns a dict: "seconds" (wall time of the n steps after one untimed warm-up step), "som" (train) or
    "dist", "rot" (map).  Raises RuntimeError with the child's output when it fails or runs out of time."""
    import sys
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        inp, out = os.path.join(tmp, "in.npz"), os.path.join(tmp, "out.npz")
        np.savez(inp, som=np.ascontiguousarray(som, dtype=np.float32), images=np.ascontiguousarray(images, dtype=np.float32),
                 cfg=np.array([som_layout, s0, s1, idim, nd, ed, R, int(flip), mode], np.int64),
                 fcfg=np.array([sigma, damping], np.float64), task=np.array(task))
        env = dict(os.environ)
        env["CUDA_VISIBLE_DEVICES"] = env.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
        try:
            proc = subprocess.run([sys.executable, os.path.join(_HERE, "ref_cuda_worker.py"), inp, out], env=env,
                                  capture_output=True, text=True, timeout=timeout)
        except subprocess.TimeoutExpired:
            raise RuntimeError("the reference's CUDA path did not finish within %d s" % timeout)
        if proc.returncode != 0 or not os.path.exists(out):
            raise RuntimeError("the reference's CUDA path failed (exit %d): %s" % (proc.returncode, (proc.stdout + proc.stderr)[-600:]))
        with np.load(out) as z:
            return {k: z[k] for k in z.files}
