"""ctypes bindings of the native libraries (built on demand by ``build.py``).

There is no Python or library fallback behind these: if a library cannot be built or
loaded, the import of the function that needs it raises.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_longlong, c_void_p
from functools import lru_cache

from . import build

_p = c_void_p
_i = c_int
_ll = c_longlong
_f = c_float


def pdl_enabled() -> bool:
    """Programmatic dependent launch (a kernel's CTAs become resident while the kernel before it
    drains) is on unless MINISERVE_PDL=0."""
    import os

    return os.environ.get("MINISERVE_PDL", "1") != "0"


class NativeError(RuntimeError):
    pass


class OutOfBlocks(RuntimeError):
    """The pool has fewer free pages than a call needs; nothing was changed."""


def _declare(lib, name, argtypes, restype=c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


@lru_cache(maxsize=None)
def host():
    lib = ctypes.CDLL(str(build.ensure_built(build.HOST)))
    _declare(lib, "ms_host_last_error", [], c_char_p)
    _declare(lib, "ms_alloc_create", [_i, _i], _p)
    _declare(lib, "ms_alloc_destroy", [_p], None)
    _declare(lib, "ms_alloc_num_free", [_p])
    _declare(lib, "ms_alloc_num_blocks", [_p])
    _declare(lib, "ms_alloc_block_size", [_p])
    _declare(lib, "ms_alloc_refcount", [_p, _i, POINTER(c_int)])
    _declare(lib, "ms_alloc_allocate", [_p, _i, POINTER(c_int32)])
    _declare(lib, "ms_alloc_incref", [_p, POINTER(c_int32), _i])
    _declare(lib, "ms_alloc_free", [_p, POINTER(c_int32), _i])
    _declare(lib, "ms_alloc_check", [_p])
    _declare(lib, "ms_table_create", [_p], _p)
    _declare(lib, "ms_table_destroy", [_p], None)
    _declare(lib, "ms_table_num_tokens", [_p], _ll)
    _declare(lib, "ms_table_num_entries", [_p])
    _declare(lib, "ms_table_num_held", [_p])
    _declare(lib, "ms_table_blocks_needed", [_p, _ll, POINTER(c_int)])
    _declare(lib, "ms_table_append_tokens", [_p, _ll])
    _declare(lib, "ms_table_slot", [_p, _ll, POINTER(_ll)])
    _declare(lib, "ms_table_rewind", [_p, _ll])
    _declare(lib, "ms_table_release", [_p])
    _declare(lib, "ms_table_release_below", [_p, _ll, POINTER(c_int)])
    _declare(lib, "ms_table_copy_blocks", [_p, POINTER(c_int32), _i])
    _declare(lib, "ms_pack_step",
             [_p, _ll, POINTER(_ll), _i, _i, _p, _p, _p, _p, _p, _i, _i, POINTER(c_void_p), _p, _ll, _i, _i, _i, _i], _ll)
    return lib


def host_check(rc: int) -> None:
    """Turn a host-core return code into the exception the reference's allocator raises
    (miniserve/cache/block_allocator.py: OutOfBlocks, ValueError, IndexError)."""
    if rc == 0:
        return
    msg = host().ms_host_last_error().decode()
    if rc == 2:
        raise OutOfBlocks(msg)
    if rc == 3:
        raise IndexError(msg)
    raise ValueError(msg)


@lru_cache(maxsize=None)
def kernels():
    lib = ctypes.CDLL(str(build.ensure_built(build.KERNELS)))
    _declare(lib, "ms_kernels_last_error", [], c_char_p)
    _declare(lib, "ms_kernels_set_pdl", [_i], None)
    lib.ms_kernels_set_pdl(int(pdl_enabled()))
    _declare(lib, "ms_device_sm_count", [_i, POINTER(c_int)])
    _declare(lib, "ms_device_arch", [_i, POINTER(c_int), POINTER(c_int)])
    _declare(lib, "ms_wait_selftest", [_p, _ll, _i, _p])
    _declare(lib, "ms_fill_tokens", [_p, _p, _p, _p, _i, _p])
    _declare(lib, "ms_embed_gather", [_p, _p, _p, _i, _i, _i, _i, _p])
    _declare(lib, "ms_add_rmsnorm", [_p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _p])
    _declare(lib, "ms_gemm_skinny_gate_up_bf16", [_p, _p, _p, _i, _i, _i, _p])
    _declare(lib, "ms_gemm_skinny_bf16", [_p, _p, _p, _i, _i, _i, _i, _p])
    _declare(lib, "ms_gemm_skinny_set_stream", [_i], None)
    _declare(lib, "ms_silu_mul", [_p, _p, _i, _i, _i, _p])
    _declare(lib, "ms_to_float", [_p, _p, _ll, _i, _p])
    _declare(lib, "ms_qk_norm_rope_kv",
             [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p, _i, _p])
    _declare(lib, "ms_rope_table", [_p, _p, _p, _i, _i, _p])
    _declare(lib, "ms_rope_table_tile", [_p, _p, _i, _p])
    _declare(lib, "ms_gemm_f32", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p])
    _declare(lib, "ms_attention_rowwise",
             [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _i, _i, _p, _i, _p])
    _declare(lib, "ms_nucleus_bytes", [])
    _declare(lib, "ms_sample_scratch_bytes", [_i, _i], _ll)
    _declare(lib, "ms_sample", [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p])
    return lib


@lru_cache(maxsize=None)
def gemm_tc():
    lib = ctypes.CDLL(str(build.ensure_built(build.GEMM_TC)))
    _declare(lib, "ms_gemm_tc_last_error", [], c_char_p)
    _declare(lib, "ms_gemm_tc_set_pdl", [_i], None)
    _declare(lib, "ms_gemm_tc_bf16", [_p, _p, _p, _i, _i, _i, _i, _p, _p])
    _declare(lib, "ms_gemm_tc_decode_bf16", [_p, _p, _p, _i, _i, _i, _p, _p])
    _declare(lib, "ms_gemm_tc_set_config", [_i], None)
    _declare(lib, "ms_gemm_tc_prefers", [_i, _i, _i, _i])
    _declare(lib, "ms_gemm_tc_qkv_bf16", [_p, _p, _p, _i, _i, _i, _i] + [_p] * 9 + [_i, _f, _p, _p])
    lib.ms_gemm_tc_set_pdl(int(pdl_enabled()))
    return lib


@lru_cache(maxsize=None)
def attn_tc():
    lib = ctypes.CDLL(str(build.ensure_built(build.ATTN_TC)))
    _declare(lib, "ms_attn_tc_last_error", [], c_char_p)
    _declare(lib, "ms_attn_tc_set_pdl", [_i], None)
    _declare(lib, "ms_attn_tc_supports", [_i, _i, _i, _i])
    _declare(lib, "ms_attn_tc_plan", [_p, _p, _i, _i, _i, _i, _i, _p, _p], None)
    _declare(lib, "ms_attn_tc_scratch", [_i, _i, _i, _i, _i, _p, _p], None)
    _declare(lib, "ms_attn_tc_prefill", [_p] * 8 + [_i, _i, _i, _i, _i, _ll, _f, _i, _i, _p, _i, _i, _p, _p, _p, _p])
    _declare(lib, "ms_attn_tc_write_plan", [_p, _p, _p, _i, _i, _i, _i, _i, _i, _ll, _ll, _p])
    lib.ms_attn_tc_set_pdl(int(pdl_enabled()))
    return lib


LAUNCHES = [0]  # launches of this package's own kernels since import (a launcher may launch more than one)


def kernel_check(rc: int, lib=None, errfn: str = "ms_kernels_last_error", launches: int = 1) -> None:
    LAUNCHES[0] += launches
    if rc != 0:
        lib = lib or kernels()
        raise NativeError(getattr(lib, errfn)().decode())
