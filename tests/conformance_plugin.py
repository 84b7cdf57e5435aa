"""pytest plugin that makes ``import opacus...`` resolve to ``opacus_b200...`` so
that the reference library's own test-suite can be run against this package:

    OPACUS_REFERENCE_TESTS=<reference checkout>/opacus/tests \
        python -m pytest -p tests.conformance_plugin <reference checkout>/opacus/tests/grad_samples

``opacus.tests.*`` is loaded from ``OPACUS_REFERENCE_TESTS``; every other
``opacus.*`` name is served by the module of the same path in this package.
"""
import importlib
import importlib.abc
import importlib.util
import os
import sys
import types

REF_TESTS = os.environ.get("OPACUS_REFERENCE_TESTS", "")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class _Alias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name != "opacus" and not name.startswith("opacus."):
            if name == "opt_einsum":                       # only used by the reference tests, for einsum
                return importlib.util.spec_from_loader(name, self)
            return None
        if name == "opacus.tests" or name.startswith("opacus.tests."):
            base = os.path.join(REF_TESTS, *name.split(".")[2:])
            if os.path.isdir(base):
                return importlib.util.spec_from_file_location(
                    name, os.path.join(base, "__init__.py"), submodule_search_locations=[base])
            if os.path.exists(base + ".py"):
                return importlib.util.spec_from_file_location(name, base + ".py")
            return None
        return importlib.util.spec_from_loader(name, self)

    def create_module(self, spec):
        if spec.name == "opt_einsum":
            import torch

            mod = types.ModuleType("opt_einsum")
            mod.contract = lambda eq, *ops, **kw: torch.einsum(eq, *ops)
            return mod
        return importlib.import_module("opacus_b200" + spec.name[len("opacus"):])

    def exec_module(self, module):
        pass


if not any(isinstance(f, _Alias) for f in sys.meta_path):
    sys.meta_path.insert(0, _Alias())
