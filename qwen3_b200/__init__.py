"""Import name of the library.

The sources live in the folder `qwen3-runtime-byyourself_b200/`, whose name is
not a Python identifier; this package makes them importable as `qwen3_b200` by
adding that folder to its own search path.
"""
import os as _os

__path__.insert(0, _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                                 "qwen3-runtime-byyourself_b200"))

from .api import *  # noqa: E402,F401,F403
from .api import __all__  # noqa: E402,F401
