from feather_b200.packers import *  # noqa: F401,F403
