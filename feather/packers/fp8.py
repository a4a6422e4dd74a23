"""``feather.packers.fp8`` of the reference, served by feather_b200."""
from feather_b200.packers.fp8 import *  # noqa: F401,F403
from feather_b200.packers.fp8 import __all__  # noqa: F401
