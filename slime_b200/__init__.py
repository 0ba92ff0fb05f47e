"""B200-native multi-head Flow-Lenia neural-CA step behind the J0pari/Slime pseudopod interface.

The compute lives in libslime_ca.so (hand-written sm_100a CUDA behind the C ABI of include/slime_ca.h);
this package is the host-side mirror of the reference's interfaces plus seeded input generators.
"""
from . import inputs  # noqa: F401

__all__ = ["inputs"]
