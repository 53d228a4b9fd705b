from .permutation import *  # noqa: F401,F403
