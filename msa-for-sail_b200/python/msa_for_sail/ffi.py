"""TVM-FFI entry points ``minfer.ops.{fmha_sail_plan, fmha_sail, sparse_topk_select}``.

The production caller of the upstream package reaches it through three global functions
registered with ``tvm_ffi`` (upstream ``__init__.py:20-78``).  ``register()`` does the same for
this package: arguments that arrive as ``tvm_ffi`` tensors / maps are turned into torch tensors
/ dicts (zero copy through DLPack), everything else passes through.  ``tvm_ffi`` is optional:
without it ``register()`` returns False and nothing else changes.

fp8 tensors: ``tvm_ffi`` releases up to 0.1.10 export them through DLPack with a type code torch
rejects.  The 8-bit payload is then re-labelled as uint8 in the capsule and viewed back as the
fp8 dtype on the torch side (no copy).
"""
import ctypes

import torch

_FP8 = {"float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2}
NAMES = ("minfer.ops.fmha_sail_plan", "minfer.ops.fmha_sail", "minfer.ops.sparse_topk_select")


def _relabel_capsule_as_uint8(capsule):
    """DLTensor { void* data; DLDevice device (2 x int32); int32 ndim; DLDataType dtype {u8 code,
    u8 bits, u16 lanes}; ... }: the dtype sits 20 bytes into the struct on 64-bit targets."""
    get = ctypes.pythonapi.PyCapsule_GetPointer
    get.restype, get.argtypes = ctypes.c_void_p, [ctypes.py_object, ctypes.c_char_p]
    base = get(capsule, b"dltensor")
    ctypes.c_uint8.from_address(base + 20).value = 1          # kDLUInt
    ctypes.c_uint8.from_address(base + 21).value = 8
    ctypes.c_uint16.from_address(base + 22).value = 1


def to_torch(x):
    """tvm_ffi Tensor -> torch.Tensor, tvm_ffi Map -> dict, anything else unchanged."""
    cls = type(x)
    mod, name = getattr(cls, "__module__", ""), cls.__name__
    if mod.startswith("tvm_ffi") and name == "Tensor":
        fp8 = _FP8.get(str(getattr(x, "dtype", "")))
        if fp8 is None:
            return torch.from_dlpack(x)
        capsule = x._to_dlpack() if hasattr(x, "_to_dlpack") else x.__dlpack__()
        _relabel_capsule_as_uint8(capsule)
        return torch.from_dlpack(capsule).view(fp8)
    if mod.startswith("tvm_ffi") and name == "Map":
        return {str(k): to_torch(x[k]) for k in x}
    if mod.startswith("tvm_ffi") and name == "Array":
        return [to_torch(v) for v in x]
    return x


def register(tvm_ffi=None):
    """Register the three global functions; returns True when ``tvm_ffi`` is available."""
    if tvm_ffi is None:
        try:
            import tvm_ffi                                   # noqa: F811
        except ImportError:
            return False
    from . import api

    def plan(*args):
        return api.fmha_sail_plan(*[to_torch(a) for a in args])

    def run(*args):
        out, max_score = api.fmha_sail(*[to_torch(a) for a in args])
        return out, max_score

    def topk(*args):
        return api.sparse_topk_select(*[to_torch(a) for a in args])

    for name, fn in zip(NAMES, (plan, run, topk)):
        tvm_ffi.register_global_func(name, fn, override=True)   # importing the package twice must not fail
    return True
