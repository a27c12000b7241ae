"""msa_for_sail for B200: drop-in for the upstream package's attention hot path.

Re-exports the same public names as the upstream ``msa_for_sail/__init__.py:11-18``.
The kernels live in ``libmsa_b200.so`` (hand-written sm_100a CUDA behind a C ABI);
importing the package fails loudly when that library is absent.
"""
from .api import (  # noqa: F401
    fmha_sail_plan,
    fmha_sail,
    sparse_topk_select,
    allocate_graph_workspace,
    _fmha_sail_plan,
    _fmha_sail,
)

__all__ = ["fmha_sail_plan", "fmha_sail", "sparse_topk_select", "allocate_graph_workspace"]
__version__ = "0.1.0"

# TVM-FFI global functions minfer.ops.* (upstream __init__.py:20-78); a no-op without tvm_ffi
from . import ffi as _ffi  # noqa: E402
_ffi.register()
