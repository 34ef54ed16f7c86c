"""ctypes binding of the C ABI declared in include/pink_b200.h.

The shared library holds the CUDA kernels; there is no other implementation.
Importing this module fails loudly when the library has not been built
(python -m pink_b200.build), and every compute call fails with a RuntimeError
carrying the library's message when no sm_100 device is present.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpink_b200.so")

OK, EINVAL, ECUDA, ENCCL, ETIMEOUT, ESTATE = 0, -1, -2, -3, -4, -5
FLOAT, UINT16, UINT8 = 0, 1, 2
QUADRATIC, CIRCULAR = 0, 1
NEAREST_NEIGHBOR, BILINEAR = 0, 1
LAYOUT_CARTESIAN, LAYOUT_HEXAGONAL = 0, 1
FUNC_GAUSSIAN, FUNC_UNITY_GAUSSIAN, FUNC_MEXICAN_HAT, FUNC_STEP = 0, 1, 2, 3


class Config(C.Structure):
    """Mirror of struct pink_b200_config."""
    _fields_ = [("n_neurons", C.c_uint32), ("channels", C.c_uint32), ("image_dim", C.c_uint32),
                ("neuron_dim", C.c_uint32), ("ed_dim", C.c_uint32), ("ed_shape", C.c_uint32),
                ("n_rotations", C.c_uint32), ("use_flip", C.c_uint32), ("dist_type", C.c_uint32),
                ("interpolation", C.c_uint32), ("device", C.c_int32), ("rank", C.c_uint32),
                ("world_size", C.c_uint32), ("max_batch", C.c_uint32)]


# name -> (restype, argtypes); the complete list of symbols the header declares
SYMBOLS = {
    "pink_b200_last_error": (C.c_char_p, []),
    "pink_b200_version": (C.c_char_p, []),
    "pink_b200_create": (C.c_int, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "pink_b200_destroy": (C.c_int, [C.c_void_p]),
    "pink_b200_shard": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "pink_b200_shard_stride": (C.c_uint32, [C.c_void_p]),
    "pink_b200_shard_range": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32),
                                        C.POINTER(C.c_uint32)]),
    "pink_b200_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_longlong]),
    "pink_b200_comm_unique_id": (C.c_int, [C.c_void_p]),
    "pink_b200_comm_init": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_set_som": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_get_som": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_set_update_factors": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_train": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "pink_b200_train_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "pink_b200_get_update_counts": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_get_bmu_log": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "pink_b200_map": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "pink_b200_map_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "pink_b200_synchronize": (C.c_int, [C.c_void_p]),
    "pink_b200_stream": (C.c_void_p, [C.c_void_p]),
    "pink_b200_launch_count": (C.c_uint64, [C.c_void_p]),
    "pink_b200_exchange_kind": (C.c_int, [C.c_void_p]),
    "pink_b200_get_update_stats": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_profile_begin": (C.c_int, [C.c_void_p, C.c_uint32]),
    "pink_b200_profile_end": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "pink_b200_profile_detail": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "pink_b200_profile_stamps": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32),
                                           C.POINTER(C.c_uint64)]),
    "pink_b200_map_filter_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "pink_b200_mma_i8_peak": (C.c_int, [C.c_int, C.c_uint32, C.c_int, C.POINTER(C.c_double)]),
    "pink_b200_device_count": (C.c_int, []),
    "pink_b200_group_create": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "pink_b200_group_destroy": (C.c_int, [C.c_void_p]),
    "pink_b200_group_size": (C.c_uint32, [C.c_void_p]),
    "pink_b200_group_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_longlong]),
    "pink_b200_group_set_som": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_group_get_som": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_group_set_update_factors": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_group_train": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "pink_b200_group_get_update_counts": (C.c_int, [C.c_void_p, C.c_void_p]),
    "pink_b200_group_synchronize": (C.c_int, [C.c_void_p]),
    "pink_b200_group_map": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "pink_b200_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_uint64]),
    "pink_b200_host_free": (C.c_int, [C.c_void_p]),
    "pink_b200_som_size": (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32]),
    "pink_b200_som_distances": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]),
    "pink_b200_update_factors": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                           C.c_float, C.c_void_p]),
    "pink_b200_distance_classes": (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32]),
    "pink_b200_som_coordinates": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]),
    "pink_b200_update_lut": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                       C.c_float, C.c_void_p, C.c_uint32]),
    "pink_b200_set_update_lut": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32]),
    "pink_b200_set_update_function": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                                C.c_float, C.c_float, C.c_float]),
    "pink_b200_group_set_update_lut": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                                 C.c_uint32]),
    "pink_b200_som_distances_3d": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]),
    "pink_b200_update_factors_3d": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                               C.c_float, C.c_void_p]),
    "pink_b200_operand_stride": (C.c_uint32, [C.c_uint32, C.c_uint32]),
    "pink_b200_op_rotate": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p]),
    "pink_b200_op_rotate_static": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_void_p]),
    "pink_b200_op_quantize_som": (C.c_int, [C.POINTER(Config), C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_void_p]),
    "pink_b200_op_distance": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
                                        C.c_void_p, C.c_void_p]),
    "pink_b200_op_status": (C.c_int, []),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("pink_b200: %s is missing; build it with `python -m pink_b200.build` "
                          "(there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class PinkError(RuntimeError):
    """A failing C-ABI call; .code is the PINK_B200_E* value."""

    def __init__(self, code, msg):
        super().__init__(msg)
        self.code = code


def check(rc):
    if rc != OK:
        raise PinkError(rc, lib.pink_b200_last_error().decode())
    return rc
