"""Run ONE test file of the upstream project, unmodified and in place, against this package.

    python tests/upstream_runner.py <path/to/upstream/tests/.../test_x.py> [its arguments]

The upstream files put their own checkout's ``python/`` first on ``sys.path`` and then do
``from msa_for_sail import ...``.  Importing this repository's ``msa_for_sail`` beforehand leaves it
in ``sys.modules``, so those imports bind to the sm_100a implementation and the file's own
``__main__`` block exercises it.  Run as a separate process: the upstream files import a module
called ``conftest`` of their own.
"""
import os
import runpy
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))

import msa_for_sail            # noqa: E402,F401
import msa_for_sail.api        # noqa: E402,F401

if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    target = os.path.abspath(sys.argv[1])
    sys.argv = [target] + sys.argv[2:]
    sys.path.insert(0, os.path.dirname(target))
    runpy.run_path(target, run_name="__main__")
