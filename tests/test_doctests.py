"""The usage examples in the docstrings run as written."""
import doctest
import importlib
import warnings

import pytest


@pytest.mark.parametrize("name", ["opacus_b200.privacy_engine", "opacus_b200.accountants.analysis.rdp"])
def test_docstring_examples(name):
    mod = importlib.import_module(name)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        result = doctest.testmod(mod, optionflags=doctest.ELLIPSIS | doctest.NORMALIZE_WHITESPACE)
    assert result.attempted > 0 and result.failed == 0
