"""The bounds-checked / debug-hook build of the library (libmsa_b200_check.so, MSA_BOUNDS_CHECK=1): valid inputs,
an out-of-range page id that is reported instead of followed, and a bounded wait that is made to run out.  The
library is chosen when the package is imported, so the checks run in a child process (checked_build_child.py)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CHECK_SO = os.path.join(ROOT, "msa-for-sail_b200", "python", "msa_for_sail", "libmsa_b200_check.so")


def test_checked_library_exports_the_abi_and_the_hooks():
    """CPU: the checked library has the whole documented ABI plus the debug hooks the shipped one leaves out."""
    if not os.path.exists(CHECK_SO):
        pytest.skip("libmsa_b200_check.so not built (python msa-for-sail_b200/build.py --bounds-check)")
    sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))
    from msa_for_sail import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", CHECK_SO], capture_output=True, text=True).stdout
    names = {ln.split()[-1] for ln in out.splitlines() if ln.strip()}
    assert set(_lib.EXPORTS) <= names
    assert {"msa_debug_tc_stall", "msa_debug_tc_trace", "msa_debug_sparse_trace_cta", "msa_debug_decode_trace"} <= names


@pytest.mark.gpu
def test_checked_build_reports_bad_indices_and_timeouts():
    if not os.path.exists(CHECK_SO):
        pytest.fail("libmsa_b200_check.so is missing: __graft_entry__.build() builds it")
    env = dict(os.environ, MSA_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, os.path.join(HERE, "checked_build_child.py")], capture_output=True, text=True,
                       timeout=900, env=env)
    assert r.returncode == 0 and "CHECKED_BUILD_OK" in r.stdout, r.stdout[-3000:] + "\n--- stderr ---\n" + r.stderr[-3000:]
