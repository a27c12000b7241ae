"""TVM-FFI registration (minfer.ops.*): names, argument conversion, fp8 tensors.  No GPU needed:
the registered functions are called with the package's API functions replaced by recorders."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "msa-for-sail_b200", "python"))

tvm_ffi = pytest.importorskip("tvm_ffi")


def test_global_functions_exist_after_import():
    import msa_for_sail  # noqa: F401
    from msa_for_sail import ffi
    for name in ffi.NAMES:
        assert tvm_ffi.get_global_func(name) is not None
    assert ffi.register() is True                            # idempotent


def test_arguments_arrive_as_torch_objects(monkeypatch):
    from msa_for_sail import api, ffi
    seen = {}

    def recorder(*args):
        seen["args"] = args
        return 7
    monkeypatch.setattr(api, "sparse_topk_select", recorder)
    ffi.register()
    t = torch.arange(6, dtype=torch.float32).reshape(1, 2, 3)
    t8 = torch.arange(16, dtype=torch.float32).to(torch.float8_e4m3fn)
    f = tvm_ffi.get_global_func("minfer.ops.sparse_topk_select")
    assert f(tvm_ffi.from_dlpack(t), 2, tvm_ffi.from_dlpack(t8)) == 7
    a0, a1, a2 = seen["args"]
    assert isinstance(a0, torch.Tensor) and a0.dtype == torch.float32 and torch.equal(a0, t)
    assert a0.data_ptr() == t.data_ptr()                     # zero copy
    assert a1 == 2
    assert isinstance(a2, torch.Tensor) and a2.dtype == torch.float8_e4m3fn
    assert torch.equal(a2.view(torch.uint8), t8.view(torch.uint8)) and a2.data_ptr() == t8.data_ptr()


def test_to_torch_passes_other_values_through():
    from msa_for_sail import ffi
    assert ffi.to_torch(3) == 3 and ffi.to_torch(None) is None
    t = torch.zeros(2)
    assert ffi.to_torch(t) is t
