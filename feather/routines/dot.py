"""``feather.routines.dot`` (FP8 part) of the reference, served by feather_b200."""
from feather_b200.routines.dot import *  # noqa: F401,F403
