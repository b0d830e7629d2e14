"""Import shim: `import lily_b200` loads the package directory
`lily-qwen3.8-flash-next_b200/` (whose name is not a Python identifier)."""
import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lily-qwen3.8-flash-next_b200")
_spec = importlib.util.spec_from_file_location(
    "lily_b200", os.path.join(_DIR, "__init__.py"), submodule_search_locations=[_DIR])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["lily_b200"] = _mod
_spec.loader.exec_module(_mod)
