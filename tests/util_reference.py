"""Where a checkout of the reference lives, for the tests that compare against its code directly.

Set WUSH_REFERENCE_ROOT to the checkout; without it the directory next to this repository named ``reference`` is
tried.  Tests that need it are skipped when it is absent (it never travels with the repository)."""
import os

import pytest

_HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("WUSH_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
HAVE_REFERENCE = os.path.isdir(os.path.join(REF, "src", "quantization"))
needs_reference = pytest.mark.skipif(not HAVE_REFERENCE, reason="no reference checkout (set WUSH_REFERENCE_ROOT)")
