from feather_b200.routines import *  # noqa: F401,F403
