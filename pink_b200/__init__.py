"""pink_b200: B200-native (sm_100a) implementation of PINK's rotation/flip-invariant SOM hot path.

``pink_b200.capi`` binds the C ABI of the CUDA library; ``pink_b200.pink`` mirrors
the reference's Python API (pink.Data / SOM / Trainer / Mapper) on top of it.
"""
__version__ = "0.1"
