"""Direct oracle-vs-reference comparison; runs only where a reference checkout exists."""
import os
import subprocess
import sys

import pytest

REF = os.environ.get("WUSH_REFERENCE_ROOT", "/root/reference")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src", "quantization")), reason="no reference checkout")
def test_oracle_matches_reference_code():
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "check_against_reference.py"), REF],
                       capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
