"""Import shim: the package lives in the directory ``nanochat-cpp_b200`` (not an identifier), this makes it
importable as ``nanochat_cpp_b200``."""
import os as _os

__path__.insert(0, _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "nanochat-cpp_b200"))

from .engine import *  # noqa: F401,F403,E402
from . import capi, engine  # noqa: F401,E402
