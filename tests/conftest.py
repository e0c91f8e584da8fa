"""pytest configuration: import paths, the `gpu` marker and the oracle-backed expected values."""

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
for entry in (REPO, REPO / "tirx-kernels_b200", REPO / "tests"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def native():
    """The C-ABI library; a missing build is an error, never a skip."""
    from tirx_kernels import _native

    _native.lib()
    return _native


@pytest.fixture()
def oracle_expected(native):
    """Installs the CPU oracle as the expected-value provider of the kernel modules' run_test."""
    import oracle_provider
    from tirx_kernels import runner

    runner.set_reference_provider(oracle_provider.make_provider(native))
    yield
    runner.set_reference_provider(None)
