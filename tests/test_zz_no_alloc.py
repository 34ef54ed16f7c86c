"""pink_b200_op_rotate_static: the rotation-set entry for callers that may not allocate device memory
(allocator callbacks, fully pre-reserved arenas, loops that cannot take cudaMalloc's implicit sync).

Its rotation-angle table sits in a fixed device array inside the library instead of a per-call cudaMalloc,
so every call shares that array and inherits the previous call's contents.  The test therefore makes two
calls in a row with different rotation counts -- the second must not be disturbed by what the first left
behind -- and requires bit-identical outputs to the allocating entry pink_b200_op_rotate.  It is collected
last so that a failure here cannot hide the result of any other test, and it passes alone as well."""
import ctypes as C

import numpy as np
import pytest

from util import make_config, ptr

pytestmark = pytest.mark.gpu


def _run(torch, capi, entry, cfg, d_img, n_img, q, T, Kp, nd, C_, mode):
    base = torch.full((n_img, q, C_, nd, nd), -7.0, dtype=torch.float32, device="cuda")
    tdt = torch.float32 if mode == 0 else torch.uint8
    b0 = torch.zeros((n_img * T, Kp), dtype=tdt, device="cuda")
    b1 = torch.zeros((n_img * T, Kp), dtype=tdt, device="cuda") if mode == 1 else None
    bnorm = torch.zeros(n_img * T, dtype=torch.int64 if mode == 1 else torch.int32, device="cuda")
    capi.check(entry(C.byref(cfg), ptr(d_img), n_img, ptr(base), ptr(b0), ptr(b1), ptr(bnorm), None))
    torch.cuda.synchronize()
    return [x.cpu().numpy() for x in (base, b0, bnorm)] + ([b1.cpu().numpy()] if b1 is not None else [])


def test_static_scratch_entry_matches_allocating_entry_twice(cuda):
    import pink_b200.capi as capi
    torch = cuda
    rng = np.random.default_rng(321)
    # two calls in a row: a long table first, then a short one over the same array; then uint16 for the 2-plane path
    for (C_, idim, nd, ed, R, flip, mode) in [(1, 64, 44, 31, 360, True, 2), (2, 30, 21, 15, 24, True, 2),
                                              (1, 16, 12, 7, 16, False, 1)]:
        n_img = 2
        imgs = rng.random((n_img, C_, idim, idim), dtype=np.float32)
        d_img = torch.from_numpy(imgs).cuda()
        T, q = R * (2 if flip else 1), max(R // 4, 1)
        Kp = capi.lib.pink_b200_operand_stride(C_ * ed * ed, mode)
        cfg = make_config(capi, 1, C_, idim, nd, ed, R, flip, mode)
        want = _run(torch, capi, capi.lib.pink_b200_op_rotate, cfg, d_img, n_img, q, T, Kp, nd, C_, mode)
        got = _run(torch, capi, capi.lib.pink_b200_op_rotate_static, cfg, d_img, n_img, q, T, Kp, nd, C_, mode)
        for w, g in zip(want, got):
            assert np.array_equal(w.view(np.uint8), g.view(np.uint8)), "outputs differ from pink_b200_op_rotate"


def test_static_scratch_entry_rejects_oversized_tables(cuda):
    import pink_b200.capi as capi
    torch = cuda
    cfg = make_config(capi, 1, 1, 8, 6, 4, 16388, False, 2)          # 4097 rotations per quadrant
    img = torch.zeros((1, 1, 8, 8), dtype=torch.float32, device="cuda")
    out = torch.zeros((16388, 128), dtype=torch.uint8, device="cuda")
    rc = capi.lib.pink_b200_op_rotate_static(C.byref(cfg), ptr(img), 1, None, ptr(out), None, ptr(out), None)
    assert rc == capi.EINVAL
    assert b"at most 16384 rotations" in capi.lib.pink_b200_last_error()
