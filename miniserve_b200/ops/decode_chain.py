"""Python face of ``csrc/decode_chain.cu``: a chain of weight-streaming products for up to 16
tokens, run by one persistent kernel (one CTA per SM, grid-wide barriers between the products,
the weights of every product streamed ahead through a shared-memory ring)."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from . import native

MAX_PHASES = 8
MAX_ROWS = 16
OUT_BF16, OUT_F32, SILU_MUL, RESIDUAL = 0, 1, 2, 3


class _Phase(Structure):
    _fields_ = [("W", c_void_p), ("X", c_void_p), ("sumsq_in", c_void_p), ("out", c_void_p), ("residual", c_void_p),
                ("norm_w", c_void_p), ("xw_out", c_void_p), ("sumsq_out", c_void_p), ("N", c_int), ("K", c_int),
                ("parts_in", c_int), ("epilogue", c_int), ("wrows", c_int), ("eps", c_float)]


class _Program(Structure):
    _fields_ = [("num_phases", c_int), ("M", c_int), ("prefetch", c_void_p), ("prefetch_bytes", c_longlong),
                ("phase", _Phase * MAX_PHASES)]


@dataclass
class Phase:
    """One product ``x [M, K] @ weight^T`` of a chain and what its epilogue does with the result
    (scaled per token by ``rsqrt(sum(sumsq_in) / K + eps)`` when ``sumsq_in`` is given: the row
    scale of the RMSNorm whose weighted input ``x`` is):

    ``OUT_BF16`` / ``OUT_F32``  store to ``out`` [M, N];
    ``SILU_MUL``  ``weight`` is [2N, K], gate rows then up rows; ``out`` [M, N] = silu(gate) * up;
    ``RESIDUAL``  ``residual`` [M, N] float32 += bf16(result), ``xw_out`` = bf16(residual * norm_w),
                  ``sumsq_out`` [M, tiles(N)] = per-tile sums of residual^2 (for the next norm)."""

    weight: torch.Tensor
    x: torch.Tensor
    epilogue: int
    out: torch.Tensor | None = None
    sumsq_in: torch.Tensor | None = None
    eps: float = 0.0
    residual: torch.Tensor | None = None
    norm_w: torch.Tensor | None = None
    xw_out: torch.Tensor | None = None
    sumsq_out: torch.Tensor | None = None


_GRID: dict[int, int] = {}


def grid_size() -> int:
    """CTAs a chain runs on (one per SM of the current device)."""
    dev = torch.cuda.current_device()
    if dev not in _GRID:
        g = c_int()
        native.kernel_check(native.kernels().ms_decode_chain_grid(ctypes.byref(g)), launches=0)
        _GRID[dev] = g.value
    return _GRID[dev]


def _wrows(n: int, epilogue: int) -> int:
    return native.kernels().ms_decode_chain_wrows(n, epilogue, grid_size())


def tiles(n: int, epilogue: int = RESIDUAL) -> int:
    """Output tiles of a product with ``n`` columns: the width of a RESIDUAL phase's ``sumsq_out``."""
    return native.kernels().ms_decode_chain_tiles(n, epilogue, _wrows(n, epilogue))


def fits(rows: int, max_k: int) -> bool:
    """Whether a chain of products with inner sizes up to ``max_k`` fits a CTA's shared memory."""
    return bool(native.kernels().ms_decode_chain_fits(rows, max_k))


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _persistent_default() -> bool:
    import os

    return os.environ.get("MINISERVE_CHAIN_PERSISTENT", "0") == "1"


PERSISTENT = _persistent_default()


def run(phases: list[Phase], rows: int, sync_state: torch.Tensor, status: torch.Tensor, stream: int,
        prefetch: torch.Tensor | None = None, persistent: bool | None = None) -> None:
    """Run ``phases`` (at most ``MAX_PHASES``) over ``rows`` tokens: as ONE persistent kernel with
    grid-wide barriers between the phases (``persistent``), or as one kernel per phase; the same bits
    either way. ``sync_state``: int32 [4], zero before the first launch (and again after a raised
    status word); used by the persistent kernel only."""
    persistent = PERSISTENT if persistent is None else persistent
    assert 1 <= len(phases) <= MAX_PHASES and 1 <= rows <= MAX_ROWS
    assert sync_state.dtype == torch.int32 and sync_state.numel() >= 4 and sync_state.is_cuda
    prog = _Program()
    prog.num_phases, prog.M = len(phases), rows
    prog.prefetch = _ptr(prefetch)
    prog.prefetch_bytes = 0 if prefetch is None else prefetch.numel() * prefetch.element_size()
    for i, ph in enumerate(phases):
        w, x = ph.weight, ph.x
        n = w.shape[0] // 2 if ph.epilogue == SILU_MUL else w.shape[0]
        k = w.shape[1]
        assert w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and w.is_contiguous() and x.is_contiguous()
        assert x.shape[-1] == k and x.numel() >= rows * k, f"phase {i}: x is {tuple(x.shape)}, weight {tuple(w.shape)}"
        c = prog.phase[i]
        c.W, c.X, c.N, c.K, c.epilogue, c.eps = w.data_ptr(), x.data_ptr(), n, k, ph.epilogue, float(ph.eps)
        c.wrows = _wrows(n, ph.epilogue)
        if ph.sumsq_in is not None:
            assert ph.sumsq_in.dtype == torch.float32 and ph.sumsq_in.is_contiguous() and ph.sumsq_in.shape[0] >= rows
            c.sumsq_in, c.parts_in = ph.sumsq_in.data_ptr(), ph.sumsq_in.shape[1]
        if ph.epilogue == RESIDUAL:
            assert ph.residual.dtype == torch.float32 and ph.residual.shape[-1] == n and ph.norm_w.numel() == n
            assert ph.xw_out.dtype == torch.bfloat16 and ph.xw_out.shape[-1] == n
            assert ph.sumsq_out.dtype == torch.float32 and ph.sumsq_out.shape[1] == tiles(n, RESIDUAL)
            c.residual, c.norm_w, c.xw_out, c.sumsq_out = (ph.residual.data_ptr(), ph.norm_w.data_ptr(), ph.xw_out.data_ptr(),
                                                           ph.sumsq_out.data_ptr())
        else:
            want = torch.float32 if ph.epilogue == OUT_F32 else torch.bfloat16
            assert ph.out.dtype == want and ph.out.shape[-1] == n and ph.out.is_contiguous()
            c.out = ph.out.data_ptr()
    native.kernel_check(native.kernels().ms_decode_chain(ctypes.byref(prog), sync_state.data_ptr(), status.data_ptr(),
                                                         int(persistent), stream),
                        launches=1 if persistent else len(phases))


def embed(residual: torch.Tensor, xw: torch.Tensor, sumsq: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
          norm_w: torch.Tensor, stream: int) -> None:
    """The start of a chain: residual[t] = float32(table[ids[t]]), xw[t] = bf16(residual[t] * norm_w),
    sumsq[t, 0] = sum of residual[t]^2."""
    t, h = residual.shape
    assert table.dtype == torch.bfloat16 and xw.dtype == torch.bfloat16 and sumsq.shape == (t, 1) and ids.dtype == torch.int32
    native.kernel_check(native.kernels().ms_chain_embed(residual.data_ptr(), xw.data_ptr(), sumsq.data_ptr(), table.data_ptr(),
                                                        ids.data_ptr(), norm_w.data_ptr(), t, h, table.shape[0], stream))
