"""Runs the reference project's own test files against this library.

``turboquant`` and its sub-modules are aliased to ``turboquant_plus_b200`` before the staged files
(tests/reference_suite/_ref/, see stage.py) are imported; every test collected from them gets the ``gpu`` marker,
because the classes compute on the device and there is no CPU fallback.  Nothing in the staged files is edited.
"""
import importlib
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SUBMODULES = ["rotation", "codebook", "polar_quant", "qjl", "turboquant", "kv_cache", "utils", "outlier"]


def _alias():
    if "turboquant" in sys.modules and getattr(sys.modules["turboquant"], "__name__", "") == "turboquant_plus_b200":
        return
    pkg = importlib.import_module("turboquant_plus_b200")
    sys.modules["turboquant"] = pkg
    for name in SUBMODULES:
        sys.modules[f"turboquant.{name}"] = importlib.import_module(f"turboquant_plus_b200.{name}")


def pytest_collectstart(collector):
    # before any staged file is imported
    if os.path.join("reference_suite", "_ref") in str(getattr(collector, "path", "")):
        _alias()


def pytest_collection_modifyitems(config, items):
    for item in items:
        if os.path.join("reference_suite", "_ref") in str(item.path):
            item.add_marker(pytest.mark.gpu)
