"""Native sm_100a kernels and their Python wrappers."""
from . import functional  # noqa: F401
