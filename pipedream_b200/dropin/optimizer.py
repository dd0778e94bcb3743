"""Drop-in module: put this directory ahead of the reference's runtime/ on sys.path and
main_with_runtime.py's `import optimizer` resolves to the B200-native implementation."""
import os as _os
import sys as _sys

_root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _root not in _sys.path:
    _sys.path.insert(0, _root)

from pipedream_b200.optimizer import *  # noqa: F401,F403,E402
from pipedream_b200 import optimizer as _impl  # noqa: E402

globals().update({k: v for k, v in vars(_impl).items() if not k.startswith("__")})
