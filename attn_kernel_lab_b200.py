"""`import attn_kernel_lab_b200`: the package in the directory `attn-kernel-lab_b200/`.

The directory carries the project's name, which is not a Python identifier; this one-file module,
found on the path next to it, loads that directory as the package `attn_kernel_lab_b200` (its
sub-modules import as `attn_kernel_lab_b200.ops`, `.quant`, `.kernel`, ...).
"""
import importlib.util
import pathlib
import sys

_DIR = pathlib.Path(__file__).resolve().parent / "attn-kernel-lab_b200"
_spec = importlib.util.spec_from_file_location(
    __name__, _DIR / "__init__.py", submodule_search_locations=[str(_DIR)])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
