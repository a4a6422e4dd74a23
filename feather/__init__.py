"""Drop-in alias: ``import feather`` resolves to the B200 implementation.

Exposes the README-level names (``feather.pack_fp8_tensor``, ``feather.gemv``,
``feather.dot``) and the reference's module paths ``feather.packers.fp8``,
``feather.routines.gemv`` and ``feather.routines.dot``.
"""
from feather_b200 import *  # noqa: F401,F403
from feather_b200 import __all__, __version__  # noqa: F401
