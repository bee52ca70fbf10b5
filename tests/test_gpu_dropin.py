"""The reference's own integration tests and walkthrough, compiled unmodified against the REFERENCE's headers and
linked against this project's library (oracle/Makefile, target `dropin`; built where the reference tree is present,
the binaries travel in oracle/_ref).  They exercise the public interface the way existing callers do: lifecycle,
argument checking, compress -> serialise -> load -> decompress round trips for the quantisation-only and the SVD
configurations, and they return non-zero on any failed check."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


@pytest.mark.parametrize("program", ["dropin_test_quantization", "dropin_test_svd", "dropin_walkthrough"])
def test_reference_program_passes_against_this_library(built, program):
    exe = os.path.join(REF_DIR, program)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/%s was not built (needs the reference tree at build time)" % program)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    tail = (res.stdout + res.stderr)[-2000:]
    assert res.returncode == 0, tail
