"""Acceptance run of the upstream project's own test files against this package.

The files are executed unmodified, where they lie in an upstream checkout whose directory is given
by the environment variable ``MSA_REFERENCE_DIR`` (skipped when it is unset or absent: nothing of
the upstream tree is part of this repository).  Each file runs in its own process through
``tests/upstream_runner.py``; it passes when the process exits 0 and prints no failure marker.
``MINFER_PPU_ARCH=ppu_15`` switches the upstream fp8 cases on (upstream tests/conftest.py:13-32).

Not applicable here: ``integration/test_plan_correctness.py`` and section 4 of
``run_ppu_tests.sh`` decode the upstream planner's internal work-list encoding
(``packed_work_range`` / ``packed_work_info``), which this implementation replaces
(``MsaWorkItem``); ``tests/test_abi_cpu.py`` checks the same coverage property on the new list.
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("MSA_REFERENCE_DIR", "")

CASES = [
    ("smoke/test_sparse_topk_forced.py", ["--dtype", "bf16"]),
    ("smoke/test_sparse_topk_forced.py", ["--dtype", "fp32"]),
    ("smoke/test_proxy_kv_smoke.py", ["--check"]),
    ("smoke/test_onlyscore_smoke.py", ["--check"]),
    ("integration/test_mixed_split.py", []),
    ("integration/test_q_offset_override.py", []),
    ("integration/test_onlyscore_pipeline.py", []),
    ("integration/test_proxy_kv_e2e.py", []),
    ("regression/test_sparse_attn.py", []),
    ("regression/test_onlyscore_correctness.py", ["--check"]),
    ("regression/test_correctness.py", ["--check", "--chaos_only"]),
]
# The fixed sections of regression/test_correctness.py build dense PyTorch references of up to 131 072 x 131 072
# tokens x 48 heads; the file then needs more than 25 minutes of GPU time, nearly all of it in those references.
if os.environ.get("MSA_UPSTREAM_FULL", "") not in ("", "0"):
    CASES.append(("regression/test_correctness.py", ["--check"]))
FAIL_MARK = re.compile(r"\[FAIL\]|\bFAILED\b|SOME FAILED|Traceback \(most recent call last\)")


@pytest.mark.parametrize("rel,args", CASES, ids=[c[0].split("/")[-1] + "".join(c[1]) for c in CASES])
def test_upstream_file_passes_against_this_package(rel, args):
    path = os.path.join(REF, "tests", rel)
    if not REF or not os.path.exists(path):
        pytest.skip("MSA_REFERENCE_DIR does not point to an upstream checkout")
    env = dict(os.environ, MINFER_PPU_ARCH="ppu_15", PYTHONUNBUFFERED="1")
    r = subprocess.run([sys.executable, os.path.join(HERE, "upstream_runner.py"), path] + args,
                       capture_output=True, text=True, timeout=3000, env=env, cwd=os.path.dirname(path))
    tail = (r.stdout[-3000:] + "\n--- stderr ---\n" + r.stderr[-3000:])
    assert r.returncode == 0, tail
    assert not FAIL_MARK.search(r.stdout), tail
