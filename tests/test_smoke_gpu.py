"""The smoke entry point the build driver calls must itself stay green."""
import pytest

pytestmark = pytest.mark.gpu


def test_graft_entry_smoke_runs():
    import __graft_entry__ as entry

    entry.smoke()
