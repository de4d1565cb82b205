"""Import name for the package directory `cohere-inference_b200/` (a hyphen cannot appear in a Python module name).

`import cohere_inference_b200` loads `cohere-inference_b200/__init__.py` as this module and makes its sub-modules
importable as `cohere_inference_b200.<name>`.
"""

import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cohere-inference_b200")
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_DIR, "__init__.py"),
                                               submodule_search_locations=[_DIR])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
