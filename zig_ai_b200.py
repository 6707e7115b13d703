"""Import shim: the package lives in the folder ``zig-ai_b200`` (a name Python cannot
import directly), so ``import zig_ai_b200`` loads that folder as the package of this name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "zig-ai_b200")
_spec = importlib.util.spec_from_file_location(
    "zig_ai_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["zig_ai_b200"] = _mod
_spec.loader.exec_module(_mod)
