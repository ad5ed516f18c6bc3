"""Short alias of :mod:`tempname_new_b200`: ``import fluxb as flux``; ``fluxb.testing``,
``fluxb.ops`` ... resolve to the same modules."""
import sys as _sys

import tempname_new_b200 as _pkg
from tempname_new_b200 import *  # noqa: F401,F403
from tempname_new_b200 import __version__, _native  # noqa: F401

for _name in ("models", "ops", "parallel", "testing", "tuning", "utils"):
    _mod = getattr(_pkg, _name)
    globals()[_name] = _mod
    _sys.modules[__name__ + "." + _name] = _mod
util = _pkg.util
dist_utils = _pkg.dist_utils
_sys.modules[__name__ + ".util"] = util
_sys.modules[__name__ + ".dist_utils"] = dist_utils
