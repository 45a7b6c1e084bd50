"""Import name of the engine package.

The package lives in the folder ``continuous-batching-inference-server_b200``,
whose name Python cannot import directly; this module loads that folder in its
own place, so ``import cbis_b200`` and ``import cbis_b200.engine`` work.
"""
import importlib.util as _ilu
import os as _os
import sys as _sys

_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)),
                     "continuous-batching-inference-server_b200")
_spec = _ilu.spec_from_file_location(__name__, _os.path.join(_dir, "__init__.py"),
                                     submodule_search_locations=[_dir])
_mod = _ilu.module_from_spec(_spec)
_sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
