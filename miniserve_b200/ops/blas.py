"""The vendor library's bfloat16 matrix product, called directly.

Plain matrix products with more rows than the weight-streaming kernel takes go to cuBLAS, as
the reference's engine sends all of its products there (miniserve/model/qwen3.py:115-117 via
``torch.nn.functional.linear``). Calling ``cublasGemmEx`` through ctypes instead of ``torch.mm``
saves most of the host time per call (a prompt step is otherwise bound by the host), and states
the arithmetic: bfloat16 operands, float32 accumulation (``CUBLAS_COMPUTE_32F``), no reduced-
precision reduction across the split k dimension.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_size_t, c_void_p

import torch

# enum values from cublas_api.h and library_types.h
_OP_N, _OP_T = 0, 1
_R_32F, _R_16BF = 0, 14
_COMPUTE_32F = 68
_GEMM_DEFAULT = -1
_DEFAULT_MATH, _NO_REDUCED_PRECISION_REDUCTION = 0, 16
_WORKSPACE_BYTES = 32 << 20

_lib = None
_handles: dict[int, list] = {}  # device index -> [handle, workspace, stream last set]
_one = ctypes.c_float(1.0)
_zero = ctypes.c_float(0.0)
_p_one, _p_zero = ctypes.addressof(_one), ctypes.addressof(_zero)


class BlasError(RuntimeError):
    pass


def _library():
    global _lib
    if _lib is None:
        try:
            lib = ctypes.CDLL("libcublas.so.12")  # the copy that PyTorch has loaded already
        except OSError as e:
            raise BlasError(f"cuBLAS (libcublas.so.12) cannot be loaded: {e}") from e
        lib.cublasCreate_v2.argtypes, lib.cublasCreate_v2.restype = [ctypes.POINTER(c_void_p)], c_int
        lib.cublasSetStream_v2.argtypes, lib.cublasSetStream_v2.restype = [c_void_p, c_void_p], c_int
        lib.cublasSetWorkspace_v2.argtypes, lib.cublasSetWorkspace_v2.restype = [c_void_p, c_void_p, c_size_t], c_int
        lib.cublasSetMathMode.argtypes, lib.cublasSetMathMode.restype = [c_void_p, c_int], c_int
        lib.cublasGemmEx.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                     c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int]
        lib.cublasGemmEx.restype = c_int
        _lib = lib
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise BlasError(f"{what} failed with cuBLAS status {rc}")


def _handle(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    got = _handles.get(idx)
    if got is None:
        lib = _library()
        handle = c_void_p()
        with torch.cuda.device(idx):
            _check(lib.cublasCreate_v2(ctypes.byref(handle)), "cublasCreate")
            # a workspace of our own: the library then allocates nothing, also under stream capture
            workspace = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
            _check(lib.cublasSetWorkspace_v2(handle, workspace.data_ptr(), _WORKSPACE_BYTES), "cublasSetWorkspace")
            _check(lib.cublasSetMathMode(handle, _DEFAULT_MATH | _NO_REDUCED_PRECISION_REDUCTION), "cublasSetMathMode")
        got = [handle, workspace, None]
        _handles[idx] = got
    return got


def gemm_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, stream: int) -> None:
    """out [M, N] (bfloat16 or float32) = x [M, K] times weight [N, K]^T, row-major, contiguous."""
    m, k = x.shape
    n = weight.shape[0]
    lib = _library()
    entry = _handle(x.device)
    handle = entry[0]
    if entry[2] != stream:
        _check(lib.cublasSetStream_v2(handle, stream), "cublasSetStream")
        # the library drops a workspace of the user's when the stream changes: give it again
        _check(lib.cublasSetWorkspace_v2(handle, entry[1].data_ptr(), _WORKSPACE_BYTES), "cublasSetWorkspace")
        entry[2] = stream
    # column-major view: out^T [N, M] = weight (as [K, N], transposed) times x^T [K, M]
    _check(lib.cublasGemmEx(handle, _OP_T, _OP_N, n, m, k, _p_one, weight.data_ptr(), _R_16BF, k, x.data_ptr(), _R_16BF, k,
                            _p_zero, out.data_ptr(), _R_32F if out.dtype == torch.float32 else _R_16BF, n, _COMPUTE_32F,
                            _GEMM_DEFAULT), "cublasGemmEx")
