"""Import shim: the package directory is named after the project
(``w4a16-dequant-gemm_b200``), which is not a Python identifier. Importing this
module loads that package under the name ``w4a16_dequant_gemm_b200``."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "w4a16-dequant-gemm_b200")
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_dir, "__init__.py"),
                                               submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
