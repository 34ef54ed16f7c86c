"""Child process that drives the reference's own CUDA path (oracle/_ref/libpink_ref_cuda.so): test infrastructure only.

usage: python ref_cuda_worker.py in.npz out.npz      (written and read by oracle.ref_cuda_run)
"""
import ctypes as C
import os
import sys
import time

import numpy as np


def main(inp, out):
    here = os.path.dirname(os.path.abspath(__file__))
    lib = C.CDLL(os.path.join(here, "_ref", "libpink_ref_cuda.so"))
    lib.ref_cuda_session_create.restype = C.c_void_p
    lib.ref_cuda_session_create.argtypes = [C.c_void_p, C.c_int] + [C.c_uint32] * 6 + [C.c_int, C.c_float, C.c_float, C.c_int, C.c_int]
    lib.ref_cuda_session_train.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
    lib.ref_cuda_session_map.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p]
    lib.ref_cuda_session_get_som.argtypes = [C.c_void_p, C.c_void_p]
    lib.ref_cuda_session_destroy.argtypes = [C.c_void_p]
    with np.load(inp) as z:
        som, images, cfg, fcfg, task = z["som"], z["images"], z["cfg"], z["fcfg"], str(z["task"])
    som_layout, s0, s1, idim, nd, ed, R, flip, mode = [int(v) for v in cfg]
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    n, isz, N = images.shape[0], idim * idim, som.shape[0]
    h = lib.ref_cuda_session_create(vp(som), som_layout, s0, s1, idim, nd, ed, R, flip, float(fcfg[0]), float(fcfg[1]),
                                    int(task == "map"), mode)
    if not h:
        sys.exit("the reference rejected the configuration")
    result = {}
    if task == "map":
        dist = np.empty((n, N), np.float32)
        rot = np.empty((n, N), np.uint32)
        lib.ref_cuda_session_map(h, vp(images), 1, isz, N, vp(dist), vp(rot))          # warm-up (module load, allocations)
        t0 = time.perf_counter()
        lib.ref_cuda_session_map(h, vp(images), n, isz, N, vp(dist), vp(rot))
        result.update(seconds=time.perf_counter() - t0, dist=dist, rot=rot)
    else:
        # the warm-up step runs on a session of its own so that the timed session starts from the given map
        w = lib.ref_cuda_session_create(vp(som), som_layout, s0, s1, idim, nd, ed, R, flip, float(fcfg[0]), float(fcfg[1]), 0, mode)
        lib.ref_cuda_session_train(w, vp(images), 1, isz)
        lib.ref_cuda_session_destroy(w)
        t0 = time.perf_counter()
        lib.ref_cuda_session_train(h, vp(images), n, isz)
        seconds = time.perf_counter() - t0
        trained = np.empty_like(som)
        lib.ref_cuda_session_get_som(h, vp(trained))
        result.update(seconds=seconds, som=trained)
    lib.ref_cuda_session_destroy(h)
    np.savez(out, **result)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
