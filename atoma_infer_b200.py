"""Import shim: the package lives in the folder ``atoma-infer_b200`` (the project's
name carries a hyphen, which Python cannot import), and is loaded under the
importable name ``atoma_infer_b200``."""
import importlib.util
import os
import sys

_root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "atoma-infer_b200")
_spec = importlib.util.spec_from_file_location(
    "atoma_infer_b200", os.path.join(_root, "__init__.py"), submodule_search_locations=[_root]
)
_pkg = importlib.util.module_from_spec(_spec)
sys.modules["atoma_infer_b200"] = _pkg
_spec.loader.exec_module(_pkg)
