"""Direct oracle-vs-reference comparison; runs only where a reference checkout exists."""
import os
import subprocess
import sys

import pytest

from tests.util_reference import REF, needs_reference

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@needs_reference
def test_oracle_matches_reference_code():
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "check_against_reference.py"), REF],
                       capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
