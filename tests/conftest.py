"""Shared pytest configuration: the `gpu` marker, import paths, and session-wide handles on the oracle."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.build(ref=False)
    return oracle.Oracle()


@pytest.fixture(scope="session")
def ref_strict():
    """The real reference, where it was built (skips elsewhere: the reference tree does not travel)."""
    import oracle
    if not os.path.exists(oracle.REF_STRICT_SO):
        pytest.skip("reference build (oracle/_ref) not present on this machine")
    return oracle.Reference("strict")


@pytest.fixture(scope="session")
def lib():
    """The product: the CUDA library behind its C-ABI, loaded through the package. Fails loudly if it is missing."""
    import __graft_entry__ as entry
    pkg = entry.load_package()
    return pkg
