"""Direct (ctypes) access to the sm_100a kernel library and functional ops."""
from . import capi  # noqa: F401
