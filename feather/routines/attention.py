"""``feather.routines.attention`` of the reference, served by feather_b200."""
from feather_b200.packers.fp8 import pack_fp8_tensor  # the reference module star-imports its packers
from feather_b200.routines.attention import *  # noqa: F401,F403
