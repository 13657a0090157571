"""Import alias for the package folder ``vllm-cpp_b200/``.

The folder's name is not a Python identifier, so ``import vllm_cpp_b200`` lands
here and this module replaces itself in ``sys.modules`` with the real package,
loaded from the folder next to it.  Sub-modules (``vllm_cpp_b200.engine`` …)
then resolve inside that folder as for any package.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vllm-cpp_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_pkg = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _pkg
_spec.loader.exec_module(_pkg)
