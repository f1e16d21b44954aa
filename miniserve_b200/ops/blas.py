"""The vendor library's bfloat16 matrix product, called directly.

Plain matrix products with more rows than the weight-streaming kernel takes go to cuBLAS, as
the reference's engine sends all of its products there (miniserve/model/qwen3.py:115-117 via
``torch.nn.functional.linear``). Calling the library through ctypes instead of ``torch.mm``
saves most of the host time per call (a prompt step is otherwise bound by the host), and states
the arithmetic: bfloat16 operands, float32 accumulation (``CUBLAS_COMPUTE_32F``), no reduction
across a split k dimension in less than float32.

The call is ``cublasLtMatmul`` with the descriptors and the library's first-choice algorithm kept
per shape: asking the library to choose again at every call (as ``cublasGemmEx`` does) costs
about 10 us of host time per product, a cached plan about 4. ``cublasGemmEx`` remains as the path
for when cublasLt cannot be loaded or has no algorithm for a shape.
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


# ---------------------------------------------------------------- cublasLt with a plan per shape
class _Algo(ctypes.Structure):  # cublasLtMatmulAlgo_t
    _fields_ = [("data", ctypes.c_uint64 * 8)]


class _Heuristic(ctypes.Structure):  # cublasLtMatmulHeuristicResult_t
    _fields_ = [("algo", _Algo), ("workspace", c_size_t), ("state", c_int), ("waves", ctypes.c_float), ("reserved", c_int * 4)]


_LT_TRANSA, _LT_TRANSB = 3, 4                     # cublasLtMatmulDescAttributes_t
_LT_PREF_WORKSPACE, _LT_PREF_REDUCTION = 1, 3     # cublasLtMatmulPreferenceAttributes_t
_LT_PREF_ALIGNMENTS = (5, 6, 7, 8)                # minimum alignment of A, B, C, D in bytes
_LT_REDUCE_IN_COMPUTE_TYPE = 0 | 1 | 2            # none, in place, compute type: never the output type
_MAX_PLANS = 8192                                 # shapes beyond this many go through cublasGemmEx
_lt = None
_lt_handles: dict[int, c_void_p] = {}
_plans: dict[tuple, tuple] = {}  # (device, m, n, k, float32 out) -> (desc, layout w, layout x, layout out, algo) or None
_algos: dict[tuple, object] = {}  # (device, rounded m, n, k, float32 out) -> the library's choice for the first m of that kind (None: none)


def _rounded_rows(m: int) -> int:
    """Row counts that share the library's choice of algorithm: asking it costs about 0.8 ms, which a step
    with a number of tokens never seen before would pay for each of its products (measured: 10 ms for such
    a step at Qwen3-0.6B sizes against 3.6 for one seen before). Up to 64 rows every count asks for itself."""
    unit = 1 if m <= 64 else 32 if m <= 256 else 64 if m <= 512 else 128
    return -(-m // unit) * unit


def _lt_library():
    global _lt
    if _lt is None:
        try:
            lt = ctypes.CDLL("libcublasLt.so.12")
        except OSError:
            _lt = False
            return _lt
        lt.cublasLtCreate.argtypes = [ctypes.POINTER(c_void_p)]
        lt.cublasLtMatmulDescCreate.argtypes = [ctypes.POINTER(c_void_p), c_int, c_int]
        lt.cublasLtMatmulDescSetAttribute.argtypes = [c_void_p, c_int, c_void_p, c_size_t]
        lt.cublasLtMatrixLayoutCreate.argtypes = [ctypes.POINTER(c_void_p), c_int, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int64]
        lt.cublasLtMatmulPreferenceCreate.argtypes = [ctypes.POINTER(c_void_p)]
        lt.cublasLtMatmulPreferenceSetAttribute.argtypes = [c_void_p, c_int, c_void_p, c_size_t]
        lt.cublasLtMatmulPreferenceDestroy.argtypes = [c_void_p]
        lt.cublasLtMatmulAlgoGetHeuristic.argtypes = [c_void_p] * 7 + [c_int, ctypes.POINTER(_Heuristic), ctypes.POINTER(c_int)]
        lt.cublasLtMatmul.argtypes = [c_void_p] * 14 + [c_size_t, c_void_p]
        for fn in ("cublasLtCreate", "cublasLtMatmulDescCreate", "cublasLtMatmulDescSetAttribute", "cublasLtMatrixLayoutCreate",
                   "cublasLtMatmulPreferenceCreate", "cublasLtMatmulPreferenceSetAttribute", "cublasLtMatmulPreferenceDestroy",
                   "cublasLtMatmulAlgoGetHeuristic", "cublasLtMatmul"):
            getattr(lt, fn).restype = c_int
        _lt = lt
    return _lt


def _make_plan(lt, idx: int, m: int, n: int, k: int, out_f32: bool):
    """Descriptors of out^T [N, M] = weight (as [K, N], transposed) times x^T [K, M] in the library's
    column-major terms, and the library's first-choice algorithm for them (None: it has none)."""
    handle = _lt_handles.get(idx)
    if handle is None:
        handle = c_void_p()
        _check(lt.cublasLtCreate(ctypes.byref(handle)), "cublasLtCreate")
        _lt_handles[idx] = handle
    desc, lw, lx, lo, pref = c_void_p(), c_void_p(), c_void_p(), c_void_p(), c_void_p()
    _check(lt.cublasLtMatmulDescCreate(ctypes.byref(desc), _COMPUTE_32F, _R_32F), "cublasLtMatmulDescCreate")
    op_t, op_n = ctypes.c_int32(_OP_T), ctypes.c_int32(_OP_N)
    _check(lt.cublasLtMatmulDescSetAttribute(desc, _LT_TRANSA, ctypes.byref(op_t), 4), "cublasLtMatmulDescSetAttribute")
    _check(lt.cublasLtMatmulDescSetAttribute(desc, _LT_TRANSB, ctypes.byref(op_n), 4), "cublasLtMatmulDescSetAttribute")
    _check(lt.cublasLtMatrixLayoutCreate(ctypes.byref(lw), _R_16BF, k, n, k), "cublasLtMatrixLayoutCreate")
    _check(lt.cublasLtMatrixLayoutCreate(ctypes.byref(lx), _R_16BF, k, m, k), "cublasLtMatrixLayoutCreate")
    _check(lt.cublasLtMatrixLayoutCreate(ctypes.byref(lo), _R_32F if out_f32 else _R_16BF, n, m, n), "cublasLtMatrixLayoutCreate")
    _check(lt.cublasLtMatmulPreferenceCreate(ctypes.byref(pref)), "cublasLtMatmulPreferenceCreate")
    size, scheme, align = c_size_t(_WORKSPACE_BYTES), ctypes.c_uint32(_LT_REDUCE_IN_COMPUTE_TYPE), ctypes.c_uint32(16)
    _check(lt.cublasLtMatmulPreferenceSetAttribute(pref, _LT_PREF_WORKSPACE, ctypes.byref(size), 8), "cublasLtMatmulPreferenceSetAttribute")
    _check(lt.cublasLtMatmulPreferenceSetAttribute(pref, _LT_PREF_REDUCTION, ctypes.byref(scheme), 4), "cublasLtMatmulPreferenceSetAttribute")
    for attr in _LT_PREF_ALIGNMENTS:  # what this package's tensors promise; the algorithm must not ask for more
        _check(lt.cublasLtMatmulPreferenceSetAttribute(pref, attr, ctypes.byref(align), 4), "cublasLtMatmulPreferenceSetAttribute")
    kind = (idx, _rounded_rows(m), n, k, out_f32)
    algo = _algos.get(kind, False)
    if algo is False:
        found, count = _Heuristic(), c_int(0)
        rc = lt.cublasLtMatmulAlgoGetHeuristic(handle, desc, lw, lx, lo, lo, pref, 1, ctypes.byref(found), ctypes.byref(count))
        algo = None if rc != 0 or count.value < 1 or found.state != 0 else _Algo.from_buffer_copy(found.algo)
        _algos[kind] = algo
    lt.cublasLtMatmulPreferenceDestroy(pref)
    if algo is None:
        return None
    return (desc, lw, lx, lo, algo)


def gemm_bf16(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, stream: int) -> None:
    """out [M, N] (bfloat16 or float32) = x [M, K] times weight [N, K]^T, row-major, contiguous."""
    m, k = x.shape
    n = weight.shape[0]
    lt = _lt_library()
    if lt:
        idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
        key = (idx, m, n, k, out.dtype == torch.float32)
        plan = _plans.get(key, False)
        if plan is False and len(_plans) < _MAX_PLANS:
            plan = _plans[key] = _make_plan(lt, idx, m, n, k, key[4])
        if plan:
            workspace = _handle(x.device)[1]
            rc = lt.cublasLtMatmul(_lt_handles[idx], plan[0], _p_one, weight.data_ptr(), plan[1], x.data_ptr(), plan[2], _p_zero,
                                   out.data_ptr(), plan[3], out.data_ptr(), plan[3], ctypes.addressof(plan[4]),
                                   workspace.data_ptr(), _WORKSPACE_BYTES, stream)
            if rc == 0:
                return
            kind = (idx, _rounded_rows(m), n, k, key[4])
            if _algos.get(kind) is not None and _algos[kind] is plan[4]:
                # the choice made for another row count of this kind is refused for this one: ask for its own, once
                _algos.pop(kind)
                plan = _plans[key] = _make_plan(lt, idx, m, n, k, key[4])
                if plan and lt.cublasLtMatmul(_lt_handles[idx], plan[0], _p_one, weight.data_ptr(), plan[1], x.data_ptr(), plan[2],
                                              _p_zero, out.data_ptr(), plan[3], out.data_ptr(), plan[3], ctypes.addressof(plan[4]),
                                              workspace.data_ptr(), _WORKSPACE_BYTES, stream) == 0:
                    return
            _plans[key] = None  # the algorithm does not take these operands after all: cublasGemmEx from now on
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
