"""bullet_b200: a B200-native (sm_100a) implementation of the NNUE training step of jw1912/bullet.

The package is a thin host layer over `libbullet_b200.so` (C ABI in include/bullet_b200.h).
There is no CPU, PyTorch or Triton fallback: without the built library `Net` cannot be used.
"""
from .configs import (ACT_CRELU, ACT_NONE, ACT_SCRELU, KING_BUCKETS_16, AdamWParams, BenchConfig, NetDesc,  # noqa: F401
                      config)


def __getattr__(name):
    # Net and the featurisers need the compiled library; keep plain-data imports usable without it
    if name in ("Net", "featurise", "pack_indices", "unpack_indices", "B200Error"):
        from . import _lib, net

        return getattr(net, name) if hasattr(net, name) else getattr(_lib, name)
    if name == "SavedFormat":
        from .saved_format import SavedFormat

        return SavedFormat
    raise AttributeError(name)
