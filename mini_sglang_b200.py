"""Import name of the package kept in the folder `mini-sglang_b200/`.

The folder's name has a hyphen, which Python's import statement cannot spell; this module
loads that folder's __init__.py under the name `mini_sglang_b200` and hands over to it, so
`import mini_sglang_b200` and `from mini_sglang_b200.engine import Engine` work from a
checkout without installation.
"""

import importlib.util
import os
import sys

_root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mini-sglang_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_root, "__init__.py"), submodule_search_locations=[_root])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
