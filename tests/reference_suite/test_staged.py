"""Reports whether the reference's test files are staged (see stage.py); the files themselves are collected from
tests/reference_suite/_ref/ by pytest and run against the aliased package."""
import os

import pytest

from tests.reference_suite import stage


@pytest.mark.gpu
def test_reference_files_are_staged():
    have = [f for f in stage.FILES if os.path.exists(os.path.join(stage.DEST, f))]
    if not have:
        pytest.skip("the reference's test files are not staged (python tests/reference_suite/stage.py <checkout>)")
    assert len(have) == len(stage.FILES), f"only {have} staged"
