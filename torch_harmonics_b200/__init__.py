"""B200-native spherical harmonic transforms with the torch-harmonics module API.

``RealSHT``, ``InverseRealSHT``, ``RealVectorSHT`` and ``InverseRealVectorSHT`` mirror the classes exported
at torch_harmonics/__init__.py:45, ``SpectralConvS2``, ``QuadratureS2`` and ``GaussianRandomFieldS2`` the callers
built on them; ``torch_harmonics_b200.distributed`` mirrors the spatially sharded variants.  All compute runs in ``lib/libshtb200.so`` (hand-written sm_100a CUDA, C ABI in
``include/shtb200.h``); build it with ``python -m torch_harmonics_b200.build``.
"""

from .quadrature import QuadratureS2
from .random_fields import GaussianRandomFieldS2
from .sht import InverseRealSHT, InverseRealVectorSHT, RealSHT, RealVectorSHT
from .spectral_convolution import SpectralConvS2
from .truncation import truncate_sht

__all__ = ["RealSHT", "InverseRealSHT", "RealVectorSHT", "InverseRealVectorSHT", "SpectralConvS2", "QuadratureS2", "GaussianRandomFieldS2", "truncate_sht"]
__version__ = "0.1.0"
