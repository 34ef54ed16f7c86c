"""Kernel-level parity: each CUDA stage, called through the C ABI on device
buffers, against the CPU oracle on the same seeded inputs.  Integer and index
results must be bit-exact; float pixels must be bit-exact too (same rounding
order, no FMA); float32 distances are held to 1e-5 relative."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from util import make_config, ptr, split_key

pytestmark = pytest.mark.gpu

QDT = {0: np.float32, 1: np.uint8, 2: np.uint8}


def _rotate(torch, capi, imgs, C_, idim, nd, ed, R, flip, mode):
    n_img = imgs.shape[0]
    T = R * (2 if flip else 1)
    q = max(R // 4, 1)
    K = C_ * ed * ed
    Kp = capi.lib.pink_b200_operand_stride(K, mode)
    cfg = make_config(capi, 1, C_, idim, nd, ed, R, flip, mode)
    d_img = torch.from_numpy(np.ascontiguousarray(imgs)).cuda()
    base = torch.full((n_img, q, C_, nd, nd), -1.0, dtype=torch.float32, device="cuda")
    tdt = torch.float32 if mode == 0 else torch.uint8
    b0 = torch.zeros((n_img * T, Kp), dtype=tdt, device="cuda")
    b1 = torch.zeros((n_img * T, Kp), dtype=tdt, device="cuda") if mode == 1 else None
    bnorm = torch.zeros(n_img * T, dtype=torch.int64 if mode == 1 else torch.int32, device="cuda")
    capi.check(capi.lib.pink_b200_op_rotate(C.byref(cfg), ptr(d_img), n_img, ptr(base), ptr(b0), ptr(b1), ptr(bnorm), None))
    torch.cuda.synchronize()
    return base.cpu().numpy(), b0.cpu().numpy(), None if b1 is None else b1.cpu().numpy(), bnorm.cpu().numpy(), K, Kp


ROT_CASES = [
    # C, id, nd, ed, R, flip
    (1, 10, 8, 5, 8, True), (1, 12, 7, 4, 16, True), (1, 6, 9, 9, 4, False), (1, 16, 12, 7, 360, True),
    (1, 64, 44, 31, 360, True), (2, 30, 21, 15, 24, True), (3, 9, 12, 8, 12, False), (1, 5, 5, 3, 1, True),
    (1, 5, 5, 5, 1, False), (1, 128, 90, 64, 720, True), (2, 150, 106, 75, 8, True),
]


@pytest.mark.parametrize("case", ROT_CASES)
@pytest.mark.parametrize("mode", [2, 1, 0])
def test_rotation_set_and_operand(cuda, case, mode):
    import pink_b200.capi as capi
    C_, idim, nd, ed, R, flip = case
    rng = np.random.default_rng(hash(case) % 2**32)
    n_img = 2
    imgs = rng.random((n_img, C_, idim, idim), dtype=np.float32)
    base, b0, b1, bnorm, K, Kp = _rotate(cuda, capi, imgs, C_, idim, nd, ed, R, flip, mode)
    T = R * (2 if flip else 1)
    q = max(R // 4, 1)
    for i in range(n_img):
        rot = O.rotation_set(imgs[i], nd, R, flip)            # (T, C, nd, nd)
        assert np.array_equal(base[i].view(np.uint32), rot[:q].view(np.uint32)), "base rotations differ"
        want = O.crop_quantize(rot, ed, mode)                  # (T, K)
        rows = slice(i * T, (i + 1) * T)
        if mode == 0:
            assert np.array_equal(b0[rows, :K].view(np.uint32), want.view(np.uint32))
        elif mode == 2:
            assert np.array_equal(b0[rows, :K], want)
            assert np.array_equal(bnorm[rows].astype(np.uint64), (want.astype(np.uint64) ** 2).sum(1))
        else:
            assert np.array_equal(b0[rows, :K], (want >> 8).astype(np.uint8))
            assert np.array_equal(b1[rows, :K], (want & 255).astype(np.uint8))
            assert np.array_equal(bnorm[rows].astype(np.uint64), (want.astype(np.uint64) ** 2).sum(1))
        assert not b0[rows, K:].any(), "operand padding must stay zero"


def _distance(torch, capi, a, b, mode, n_img=1, want_matrix=True):
    """a: (N, K), b: (n_img*T, K) in the mode's natural dtype."""
    N, K = a.shape
    T = b.shape[0] // n_img
    Kp = capi.lib.pink_b200_operand_stride(K, mode)

    def planes(x):
        if mode == 0:
            p = np.zeros((x.shape[0], Kp), np.float32); p[:, :K] = x; return p, None, None
        if mode == 2:
            p = np.zeros((x.shape[0], Kp), np.uint8); p[:, :K] = x
            return p, None, (x.astype(np.uint64) ** 2).sum(1).astype(np.uint32).view(np.int32)
        hi = np.zeros((x.shape[0], Kp), np.uint8); lo = np.zeros_like(hi)
        hi[:, :K] = x >> 8; lo[:, :K] = x & 255
        return hi, lo, (x.astype(np.uint64) ** 2).sum(1).view(np.int64)

    a0, a1, an = planes(a)
    b0, b1, bn = planes(b)
    d = lambda x: None if x is None else torch.from_numpy(x).cuda()
    da0, da1, dan, db0, db1, dbn = d(a0), d(a1), d(an), d(b0), d(b1), d(bn)
    keys = torch.full((n_img, N), -1, dtype=torch.int64, device="cuda")
    mdt = {0: torch.float32, 1: torch.int64, 2: torch.int32}[mode]
    mat = torch.zeros((n_img, N, T), dtype=mdt, device="cuda") if want_matrix else None
    capi.check(capi.lib.pink_b200_op_distance(mode, N, T, K, ptr(da0), ptr(da1), ptr(dan), ptr(db0), ptr(db1),
                                              ptr(dbn), n_img, ptr(keys), ptr(mat), None))
    capi.check(capi.lib.pink_b200_op_status())
    k = keys.cpu().numpy().view(np.uint64)
    m = None
    if want_matrix:
        m = mat.cpu().numpy()
        m = m.view({0: np.float32, 1: np.uint64, 2: np.uint32}[mode])
    return k, m


DIST_CASES = [
    # N, T, K   (ragged in every dimension: not multiples of the 128 / 16 / 128 tile sizes)
    (1, 1, 4), (5, 8, 25), (100, 720, 961), (130, 50, 128), (128, 256, 256), (257, 300, 1000), (400, 180, 1936),
    (77, 1440, 300),
]


@pytest.mark.parametrize("case", DIST_CASES)
@pytest.mark.parametrize("mode", [2, 1])
def test_integer_distance_bit_exact(cuda, case, mode):
    import pink_b200.capi as capi
    N, T, K = case
    rng = np.random.default_rng(N * 7919 + T * 31 + K + mode)
    hi = 256 if mode == 2 else 65536
    dt = np.uint8 if mode == 2 else np.uint16
    a = rng.integers(0, hi, (N, K)).astype(dt)
    b = rng.integers(0, hi, (T, K)).astype(dt)
    if N > 3 and T > 3:                 # plant exact ties and an exact match
        b[3] = b[1]
        a[2] = b[min(5, T - 1)]
    keys, mat = _distance(cuda, capi, a, b, mode)
    S = O.distance_int(a, b, mode)
    assert np.array_equal(mat[0].astype(np.uint64), S), "distance matrix not bit-exact"
    smin, best = O.min_over_transforms_int(S)
    code, t = split_key(keys[0], mode)
    assert np.array_equal(code, smin)
    assert np.array_equal(t, best), "first-minimum transform differs"


@pytest.mark.parametrize("mode", [2, 1])
def test_integer_distance_extremes(cuda, mode):
    """All-zero against all-max operands: the largest S the accumulators must hold."""
    import pink_b200.capi as capi
    K = 8100 if mode == 1 else 8100
    mx = 255 if mode == 2 else 65535
    dt = np.uint8 if mode == 2 else np.uint16
    a = np.zeros((3, K), dt); a[1] = mx
    b = np.full((20, K), mx, dt); b[7] = 0
    keys, mat = _distance(cuda, capi, a, b, mode)
    S = O.distance_int(a, b, mode)
    assert np.array_equal(mat[0].astype(np.uint64), S)
    assert S.max() == K * mx * mx


@pytest.mark.parametrize("case", [(5, 8, 25), (100, 720, 961), (130, 70, 300), (400, 180, 1936)])
def test_float_distance(cuda, case):
    import pink_b200.capi as capi
    N, T, K = case
    rng = np.random.default_rng(K)
    a = rng.random((N, K), dtype=np.float32)
    b = rng.random((T, K), dtype=np.float32)
    b[1] = a[0]                                     # an exact zero distance
    keys, mat = _distance(cuda, capi, a, b, 0)
    D = O.distance_f64(a, b)
    rel = np.abs(mat[0].astype(np.float64) - D) / np.maximum(D, 1e-30)
    assert rel[D > 0].max() < 1e-5                  # float32 tolerance of the path
    assert mat[0][0, 1] == 0.0
    code, t = split_key(keys[0], 0)
    got_min = code.astype(np.uint32).view(np.float32)
    assert np.array_equal(got_min, mat[0].min(1))
    assert np.array_equal(t, mat[0].argmin(1).astype(np.uint32))   # first minimum of its own matrix


def test_distance_batched_images(cuda):
    """Several images in one launch give the same keys as one launch per image."""
    import pink_b200.capi as capi
    rng = np.random.default_rng(5)
    N, T, K, n_img = 150, 48, 200, 3
    a = rng.integers(0, 256, (N, K)).astype(np.uint8)
    b = rng.integers(0, 256, (n_img * T, K)).astype(np.uint8)
    keys, _ = _distance(cuda, capi, a, b, 2, n_img=n_img, want_matrix=False)
    for i in range(n_img):
        S = O.distance_int(a, b[i * T:(i + 1) * T], 2)
        smin, best = O.min_over_transforms_int(S)
        code, t = split_key(keys[i], 2)
        assert np.array_equal(code, smin) and np.array_equal(t, best)
