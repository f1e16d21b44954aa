"""Python faces of the CUDA kernels: each function takes torch tensors, checks what the
kernel cannot check itself, and launches on the given stream. Tensors are only containers
here; every operation below runs this package's own kernels, except the bfloat16 matrix
product, which may go to the vendor library where the reference's engine does the same
(miniserve/model/qwen3.py:115-131 uses F.linear, i.e. cuBLAS).
"""

from __future__ import annotations

import ctypes

import torch

from . import blas, native
from .native import NativeError, OutOfBlocks

__all__ = [
    "NativeError", "OutOfBlocks", "dtype_code", "embed_gather", "add_rmsnorm", "silu_mul", "linear", "linear_silu_mul",
    "silu_mul_is_fused", "qkv_fused_ok", "qkv_norm_rope_kv", "linear_tc", "device_status", "qk_norm_rope_kv", "rope_table", "rope_table_tiled",
    "attention", "attention_rowwise", "sample", "to_float", "require_cuda_kernels",
]

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"the kernels take float32 or bfloat16, not {dtype}") from None


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream(stream) -> int:
    return torch.cuda.current_stream().cuda_stream if stream is None else stream


def _check_dev(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("kernel operands must be contiguous CUDA tensors")


def require_cuda_kernels():
    """Load (building first if needed) the kernel library; raises if that is impossible."""
    return native.kernels()


def embed_gather(residual: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, stream=None) -> None:
    """residual[t] = float32(table[ids[t]]); residual [T, H] float32, ids int32."""
    _check_dev(residual, table, ids)
    assert residual.dtype == torch.float32 and ids.dtype == torch.int32
    t, h = residual.shape
    assert table.shape[1] == h and ids.numel() >= t
    k = native.kernels()
    native.kernel_check(k.ms_embed_gather(_ptr(residual), _ptr(table), _ptr(ids), t, h, table.shape[0],
                                          dtype_code(table.dtype), _stream(stream)))


def _flag(name: str, default: str) -> bool:
    import os

    return os.environ.get(name, default) == "1"


def _setting(name: str, default: str) -> str:
    import os

    return os.environ.get(name, default)


TC_GEMM = _setting("MINISERVE_TC_GEMM", "auto")   # products with more than 16 rows on the tcgen05 kernels: auto, 1 or 0
QKV_EPILOGUE = _flag("MINISERVE_QKV_EPILOGUE", "1")  # q/k norm, rotation and cache write in the q|k|v product's epilogue
TC_ATTENTION = _flag("MINISERVE_TC_ATTENTION", "1")  # prompts on the tcgen05 attention kernel (head size 128)


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: torch.Tensor | None,
                weight: torch.Tensor, eps: float, rows: torch.Tensor | None = None, num_rows: int | None = None,
                write_residual: bool = True, stream=None) -> None:
    """out[i] = rmsnorm(residual[r] + delta[r]) * weight with r = rows[i] (or i); the sum is
    written back to ``residual`` when there is no gather. Statistics in float32."""
    _check_dev(out, residual, delta, weight, rows)
    assert residual.dtype == torch.float32 and out.dtype == weight.dtype
    assert delta is None or delta.dtype == out.dtype
    hidden = residual.shape[-1]
    n = out.shape[0] if num_rows is None else num_rows
    assert weight.numel() == hidden and out.shape[-1] == hidden and out.shape[0] >= n
    if rows is None:
        assert residual.shape[0] >= n
    k = native.kernels()
    native.kernel_check(k.ms_add_rmsnorm(_ptr(out), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(rows),
                                         float(eps), n, hidden, int(write_residual and rows is None),
                                         dtype_code(out.dtype), _stream(stream)))


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, stream=None) -> None:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, I + c], computed in float32."""
    _check_dev(out, gate_up)
    t, inter = out.shape
    assert gate_up.shape == (t, 2 * inter) and gate_up.dtype == out.dtype
    k = native.kernels()
    native.kernel_check(k.ms_silu_mul(_ptr(out), _ptr(gate_up), t, inter, dtype_code(out.dtype), _stream(stream)))


def to_float(out: torch.Tensor, x: torch.Tensor, stream=None) -> None:
    _check_dev(out, x)
    assert out.dtype == torch.float32 and out.numel() == x.numel()
    k = native.kernels()
    native.kernel_check(k.ms_to_float(_ptr(out), _ptr(x), x.numel(), dtype_code(x.dtype), _stream(stream)))


_STATUS: dict[int, torch.Tensor] = {}


def device_status(device: torch.device | str = "cuda") -> torch.Tensor:
    """The per-device status word (int32 [1]) that kernels raise instead of faulting or hanging:
    inconsistent cache metadata, or a bounded wait in a TMA / tensor-core pipeline that ran out."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _STATUS[idx]


def tc_gemm_enabled() -> bool:
    """Whether plain bfloat16 products with more than 16 rows may run on this package's tcgen05
    kernels (``MINISERVE_TC_GEMM``: ``auto``, the default, where they are the faster choice;
    ``1`` always; ``0`` never)."""
    return TC_GEMM != "0"


TC_EPILOGUE = {"bf16": 0, "f32": 1, "silu_mul": 2}


def linear_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16", stream=None) -> torch.Tensor:
    """x [M, K] times weight^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    ``epilogue``: ``bf16`` / ``f32`` write x W^T [M, N]; ``silu_mul`` takes weight [2I, K] (gate rows
    then up rows) and writes silu(x Wg^T) * (x Wu^T) [M, I] without materialising the 2I-wide tensor."""
    _check_dev(x, weight, out)
    m, kdim = x.shape
    n = out.shape[1]
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] == kdim
    assert weight.shape[0] == (2 * n if epilogue == "silu_mul" else n) and out.shape[0] == m
    assert out.dtype == (torch.float32 if epilogue == "f32" else torch.bfloat16)
    lib = native.gemm_tc()
    native.kernel_check(lib.ms_gemm_tc_bf16(_ptr(out), _ptr(x), _ptr(weight), m, n, kdim, TC_EPILOGUE[epilogue],
                                            _ptr(device_status(x.device)), _stream(stream)),
                        lib=lib, errfn="ms_gemm_tc_last_error")
    return out


def linear_tc_decode(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
    """x [M, K] (M <= 64) times weight [N, K]^T on the tcgen05 tensor cores with the operands swapped (the
    weight's rows are the instruction's M, the tokens its N), the weights streamed by TMA and k cut
    into the CTAs of a thread-block cluster: the decode product for a long k."""
    _check_dev(x, weight, out)
    m, kdim = x.shape
    n = weight.shape[0]
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert weight.shape[1] == kdim and out.shape == (m, n) and m <= 64
    lib = native.gemm_tc()
    native.kernel_check(lib.ms_gemm_tc_decode_bf16(_ptr(out), _ptr(x), _ptr(weight), m, n, kdim, _ptr(device_status(x.device)),
                                                   _stream(stream)), lib=lib, errfn="ms_gemm_tc_last_error")
    return out


_TC_PREFERS: dict[tuple, bool] = {}


def tc_gemm_ok(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None, epilogue: str = "bf16") -> bool:
    """Whether ``linear`` (or ``linear_silu_mul``) sends this product to the tcgen05 kernels rather
    than to the vendor library: always where they are forced, else where they were measured faster
    (wide bfloat16 outputs, see ``ms_gemm_tc_prefers``)."""
    if TC_GEMM == "0" or x.shape[1] % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    if TC_GEMM == "1":
        return True
    if out is not None and (out.dtype != torch.bfloat16 or out.data_ptr() % 16):
        return False
    n = weight.shape[0] // 2 if epilogue == "silu_mul" else weight.shape[0]
    key = (x.shape[0], n, x.shape[1], epilogue)
    known = _TC_PREFERS.get(key)
    if known is None:
        if len(_TC_PREFERS) > 65536:
            _TC_PREFERS.clear()
        known = _TC_PREFERS[key] = bool(native.gemm_tc().ms_gemm_tc_prefers(key[0], key[1], key[2], TC_EPILOGUE[epilogue]))
    return known


SKINNY_MAX_M = 16
_SM_COUNT: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product and is the faster choice. Every CTA
    stages the whole of x, so with a long k the staging costs as much as the weights: measured on
    B200 against cuBLAS the kernel wins for k up to 3,072 at any n (3.0 against 5.4 us for 4096 x
    1024 at 8 rows, 4.5 against 9.1 us for 1024 x 3072) and for 4096 x 4096 up to 8 rows (7.8
    against 12.4 us), and loses beyond (43 against 36 us for 24576 x 4096, twice that at 16 rows).
    Outputs with at least 8 row tiles of 16 per SM (the head over the vocabulary) run on CTAs that
    stage x once and walk the tiles: up to 8 rows that wins for k up to 4,096 too (151,936 x 4,096:
    187 against 208 us; x 2,048: 95 against 106; x 5,120: 292 against 255, so not beyond)."""
    m, k = x.shape
    n = weight.shape[0]
    if not (0 < m <= SKINNY_MAX_M and k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and 16 * (k + 32) * 2 <= 200 * 1024):
        return False
    if k <= 3072:
        return True
    return k <= 4096 and m <= 8 and (n <= 4096 or n >= 8 * 16 * _sm_count(x.device))


TC_DECODE_MAX_M = 32


def _tc_decode_ok(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None) -> bool:
    """Whether a decode product goes to the tcgen05 kernel with swapped operands (``linear_tc_decode``)
    rather than to the register-fed kernel of ``gemm_skinny.cu`` or the vendor library. Its CTAs ask for
    their weights by TMA before they wait for the kernel before them, up to 180 KB each: inside a step
    a weight of a few MB is on the chip when the activations arrive. Measured on B200:

    * a long k onto a narrow output (k at least 2,048 and twice the output's width: the down
      projections, o of a small model), up to 32 rows. Alone, in us against what ran before: 4096 x 12288
      at 1 / 8 / 16 / 28 rows 18.6 / 19.4 / 20.0 / 20.9 against 30.7 / 29.2 / 22.4 / 22.6; 5120 x 25600:
      41.0 / 42.1 / 42.8 / 44.5 against 47.2 / 45.9 / 46.3 / 49.9; 1024 x 3072 at 16 / 28 rows 4.5 / 5.1
      against 6.6 / 7.0. Inside a decode step of Qwen3-0.6B sizes: 1.282 -> 1.199 ms at batch 8,
      1.198 -> 1.096 at batch 4, 1.010 -> 0.994 at batch 2 (and 0.965 -> 1.009 at batch 1: a single
      row stays on the register-fed kernel where that takes the shape, k up to 3,072);
    * any other product whose weight is at most 16 MB (it is then in flight whole), 9 to 32 rows:
      batch 16 1.640 -> 1.604 ms on top of the first rule (with 4 rows the same change loses: 1.096 -> 1.254).

    Large wide outputs (6144 x 4096, 24576 x 4096) tie or lose against the library and stay there."""
    m, k = x.shape
    n = weight.shape[0]
    if TC_GEMM == "0" or not 1 <= m <= TC_DECODE_MAX_M or k % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    if out is not None and (out.dtype != torch.bfloat16 or out.data_ptr() % 16):
        return False
    if k >= 2048 and k >= 2 * n:
        return m >= 2 or not _skinny_ok(x, weight)  # a single row stays on the register-fed kernel where that takes the shape
    return m >= 9 and n * k * 2 <= (16 << 20)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """x [M, K] times weight[N, K]^T -> [M, N].

    float32: this package's FFMA kernel (true 32-bit, fixed summation order per element).
    bfloat16 with at most 16 rows (decode steps): this package's weight-streaming kernel; with up to 32
    rows and a long k onto a narrow output: the tcgen05 kernel with swapped operands (``_tc_decode_ok``).
    bfloat16 otherwise: this package's tcgen05 kernel where it is the faster choice
    (``tc_gemm_ok``), else the vendor library's matrix product with float32 accumulation.
    ``out`` may be float32 (logits) or bfloat16.
    """
    _check_dev(x, weight, out)
    m, kdim = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == kdim, f"linear: x is [{m}, {kdim}], weight is {tuple(weight.shape)}"
    if x.dtype == torch.float32:
        assert weight.dtype == torch.float32
        if out is None:
            out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        assert out.dtype == torch.float32 and out.shape == (m, n)
        k = native.kernels()
        native.kernel_check(k.ms_gemm_f32(_ptr(out), _ptr(x), _ptr(weight), m, n, kdim, kdim, kdim, n, _stream(stream)))
        return out
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    if _tc_decode_ok(x, weight, out):
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        return linear_tc_decode(x, weight, out, stream=stream)
    if _skinny_ok(x, weight):
        k = native.kernels()
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        assert out.shape == (m, n)
        native.kernel_check(k.ms_gemm_skinny_bf16(_ptr(out), _ptr(x), _ptr(weight), m, n, kdim,
                                                  1 if out.dtype == torch.float32 else 0, _stream(stream)))
        return out
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    if tc_gemm_ok(x, weight, out):
        return linear_tc(x, weight, out, "f32" if out.dtype == torch.float32 else "bf16", stream=stream)
    assert out.shape == (m, n) and out.dtype in (torch.float32, torch.bfloat16)
    blas.gemm_bf16(out, x, weight, _stream(stream))
    return out


def silu_mul_is_fused(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether ``linear_silu_mul`` runs as one kernel for these operands (then it needs no scratch)."""
    if x.dtype != torch.bfloat16:
        return False
    return _skinny_ok(x, weight) or (x.shape[0] > SKINNY_MAX_M and tc_gemm_ok(x, weight, out, "silu_mul"))


def linear_silu_mul(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, scratch=None, stream=None) -> torch.Tensor:
    """out [M, I] = silu(x Wg^T) * (x Wu^T) for the stacked weight [2I, K] (gate rows, then up rows;
    miniserve/model/qwen3.py:128-131). bfloat16 with at most 16 rows: one weight-streaming kernel
    whose CTAs hold a gate row and its up row together. More rows: the 2-CTA tcgen05 kernel with
    the activation in its epilogue where that is the faster choice (``tc_gemm_ok``); otherwise the
    product into ``scratch`` ([M, 2I], allocated if None) and the activation kernel."""
    m, kdim = x.shape
    inter = out.shape[1]
    assert weight.shape == (2 * inter, kdim) and out.shape[0] == m and out.dtype == x.dtype
    if x.dtype == torch.bfloat16 and _skinny_ok(x, weight):
        _check_dev(x, weight, out)
        native.kernel_check(native.kernels().ms_gemm_skinny_gate_up_bf16(_ptr(out), _ptr(x), _ptr(weight), m, inter, kdim,
                                                                        _stream(stream)))
        return out
    if x.dtype == torch.bfloat16 and m > SKINNY_MAX_M and tc_gemm_ok(x, weight, out, "silu_mul"):
        return linear_tc(x, weight, out, "silu_mul", stream=stream)  # the activation in the tcgen05 kernel's epilogue
    gate_up = linear(x, weight, out=scratch, stream=stream)
    silu_mul(out, gate_up, stream=stream)
    return out


def qk_norm_rope_kv(q_out: torch.Tensor, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
                    qkv: torch.Tensor, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None,
                    inv_freq: torch.Tensor | None, rotary_dim: int, eps: float, positions: torch.Tensor,
                    row_of_token: torch.Tensor, page_indptr: torch.Tensor, page_indices: torch.Tensor,
                    page_size: int, status: torch.Tensor, stream=None, cos_sin: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotation by position, q written to ``q_out`` [T, nq, d] and the
    new k, v written into their pages. ``k_pool``/``v_pool``: [pages, nkv, page_size, d], or None
    when this entry only reads another entry's cache (then ``qkv`` holds q alone)."""
    _check_dev(q_out, k_pool, v_pool, qkv, q_norm_w, k_norm_w, inv_freq, positions, row_of_token, page_indptr,
               page_indices, status)
    t, nq, d = q_out.shape
    if k_pool is not None:
        nkv = k_pool.shape[1]
        assert k_pool.shape == v_pool.shape and k_pool.shape[2] == page_size and k_pool.shape[3] == d
        assert k_pool.dtype == qkv.dtype
        assert qkv.shape == (t, (nq + 2 * nkv) * d)
    else:
        nkv = 1
        assert qkv.shape == (t, nq * d)
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2)
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (t, rotary_dim) and cos_sin.is_contiguous())
    k = native.kernels()
    native.kernel_check(k.ms_qk_norm_rope_kv(
        _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
        _ptr(cos_sin if inv_freq is not None else None), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr), _ptr(page_indices), t, nq, nkv, d,
        rotary_dim if inv_freq is not None else 0, float(eps), page_size, 0 if k_pool is None else k_pool.shape[0],
        _ptr(status), dtype_code(qkv.dtype), _stream(stream)))


def qkv_fused_ok(x: torch.Tensor, w_qkv: torch.Tensor, nq: int, nkv: int, d: int, rotary_dim: int, k_pool, q_norm_w, k_norm_w) -> bool:
    """Whether ``qkv_norm_rope_kv`` takes this projection: a step wide enough for the 2-CTA tcgen05
    kernel to be the faster choice for the q|k|v product, bfloat16, head size 128 rotated whole (or
    not at all), even head counts (a tile's 256 columns are then two whole heads of one kind)."""
    if TC_GEMM == "0" or not QKV_EPILOGUE or x.dtype != torch.bfloat16 or k_pool is None:
        return False
    if d != 128 or rotary_dim not in (0, 128) or nq % 2 or nkv % 2 or (q_norm_w is None) != (k_norm_w is None):
        return False
    # the epilogue's work per tile does not depend on k and hides behind the products of the next tile
    # (measured at 2,048 rows: 23.0 against 25.4 us for 1024 -> 4096 columns, 79 against 85 us for
    # 4096 -> 6144, 160 against 170 us for 5120 -> 10240; at 4,096 rows 34 against 46 us for 1024 -> 4096)
    if x.shape[0] <= SKINNY_MAX_M or x.shape[1] < 1024:
        return False
    return TC_GEMM == "1" or tc_gemm_ok(x, w_qkv)


def qkv_norm_rope_kv(q_out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor,
                     q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, cos_sin: torch.Tensor | None, eps: float,
                     positions: torch.Tensor, row_of_token: torch.Tensor, page_indptr: torch.Tensor,
                     page_indices: torch.Tensor, page_size: int, stream=None) -> None:
    """The q|k|v projection of x [T, K] with what follows it in its epilogue: per-head norm of q and
    k, rotation by position (``cos_sin``: the step's float32 table as ``rope_table_tiled`` lays it out, None for no rotation),
    q to ``q_out`` [T, nq, 128] and the new k, v into their pages. The same arithmetic as
    ``linear`` followed by ``qk_norm_rope_kv``, without the [T, (nq + 2 nkv) * 128] tensor in between."""
    _check_dev(q_out, k_pool, v_pool, x, w_qkv, q_norm_w, k_norm_w, cos_sin, positions, row_of_token, page_indptr, page_indices)
    t, nq, d = q_out.shape
    nkv = k_pool.shape[1]
    assert d == 128 and k_pool.shape == v_pool.shape and k_pool.shape[2] == page_size and k_pool.shape[3] == d
    assert x.dtype == torch.bfloat16 and w_qkv.shape == ((nq + 2 * nkv) * d, x.shape[1]) and x.shape[0] == t
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (-(-t // 128), 8, 2, 128, 8))
    lib = native.gemm_tc()
    native.kernel_check(lib.ms_gemm_tc_qkv_bf16(
        _ptr(q_out), _ptr(x), _ptr(w_qkv), t, x.shape[1], nq, nkv, _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w), _ptr(k_norm_w),
        _ptr(cos_sin), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr), _ptr(page_indices), page_size, float(eps),
        _ptr(device_status(x.device)), _stream(stream)), lib=lib, errfn="ms_gemm_tc_last_error")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, num_tokens: int, rotary_dim: int, stream=None) -> torch.Tensor:
    """float32 [T, rotary_dim]: cos then sin of position * inv_freq for every token of a step."""
    table = torch.empty((num_tokens, rotary_dim), dtype=torch.float32, device=inv_freq.device)
    k = native.kernels()
    native.kernel_check(k.ms_rope_table(_ptr(table), _ptr(positions), _ptr(inv_freq), num_tokens, rotary_dim,
                                        _stream(stream)))
    return table


def rope_table_tiled(table: torch.Tensor, stream=None) -> torch.Tensor:
    """The cos/sin table [T, 128] of a step laid out by tiles of 128 tokens and eighths of the 64 rotation
    pairs, float32 [ceil(T / 128), 8, 2, 128, 8]: what ``qkv_norm_rope_kv`` reads (a piece per bulk copy).
    Rows of the last tile beyond T are not written."""
    _check_dev(table)
    assert table.dtype == torch.float32 and table.dim() == 2 and table.shape[1] == 128
    t = table.shape[0]
    tiled = torch.empty((-(-t // 128), 8, 2, 128, 8), dtype=torch.float32, device=table.device)
    k = native.kernels()
    native.kernel_check(k.ms_rope_table_tile(_ptr(tiled), _ptr(table), t, _stream(stream)))
    return tiled


def attention_rowwise(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      positions: torch.Tensor, row_of_token: torch.Tensor, page_indptr: torch.Tensor,
                      page_indices: torch.Tensor, scale: float, window: int | None, status: torch.Tensor,
                      stream=None) -> None:
    """Causal attention of every new token over its request's pages; one warp per (token, head),
    float32 arithmetic in a fixed order (bit-identical however the tokens were batched)."""
    _check_dev(out, q, k_pool, v_pool, positions, row_of_token, page_indptr, page_indices, status)
    t, nq, d = q.shape
    nkv, page_size = k_pool.shape[1], k_pool.shape[2]
    assert out.shape == q.shape and k_pool.shape[3] == d and k_pool.dtype == q.dtype
    k = native.kernels()
    native.kernel_check(k.ms_attention_rowwise(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr),
        _ptr(page_indices), t, nq, nkv, d, float(scale), int(window or 0), page_size, k_pool.shape[0], _ptr(status),
        dtype_code(q.dtype), _stream(stream)))


def nucleus_bytes() -> int:
    return native.kernels().ms_nucleus_bytes()


def sample(tokens: torch.Tensor, logits: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seed: torch.Tensor | None = None,
           counter: torch.Tensor | None = None, scratch: torch.Tensor | None = None, stream=None) -> None:
    """tokens[r] (int32) from float32 logits [rows, vocab]: argmax where temperature is 0 (or
    no temperatures are given), Gumbel-max sampling otherwise, inside the nucleus if ``top_p``."""
    _check_dev(tokens, logits, temperature, top_p, seed, counter, scratch)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and tokens.dtype == torch.int32 and tokens.numel() >= rows
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seed.dtype == torch.int64 and counter.dtype == torch.int64
    if top_p is not None:
        assert top_p.dtype == torch.float32 and scratch is not None and scratch.numel() * scratch.element_size() >= rows * nucleus_bytes()
    k = native.kernels()
    partial = None
    if top_p is None:
        need = k.ms_sample_scratch_bytes(rows, vocab)
        if need:
            partial = torch.empty(need, dtype=torch.uint8, device=logits.device)
    native.kernel_check(k.ms_sample(_ptr(tokens), _ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(seed),
                                    _ptr(counter), _ptr(scratch), _ptr(partial), rows, vocab, _stream(stream)),
                        launches=2)


def attention(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: int,
              scale: float, window: int | None) -> None:
    """Causal attention of the step's new tokens over the paged cache of cache group ``group``.

    float32 runs the row-wise kernel (bit-identical however the step was cut). bfloat16 runs the
    tensor-core kernels when they take this head size, else the row-wise kernel too."""
    from . import attention_bf16

    recorder = getattr(ctx, "recorder", None)
    if recorder is not None and q.dtype == torch.bfloat16 and (attention_tc_ok(q, k_pool) or attention_bf16.supports(q.shape[2], k_pool.shape[2])):
        # The pass is being captured into CUDA graphs. Which tensor-core kernels run here, their grids and
        # their key splits depend on each row's length and start, which a graph cannot hold.
        single = ctx.leading_single_rows
        if attention_tc_ok(q, k_pool) and single == recorder.single_rows and (single == 0 or attention_bf16.supports(q.shape[2], k_pool.shape[2])):
            # Steps of this shape have `single` decoding rows at the front and prompt rows behind them. The
            # decoding rows go to the split-key kernel as inside a decode graph (its launch follows their
            # number alone). The prompt rows go to the tcgen05 kernel, launched with a CTA per SM and
            # taking the plan of its rows from device memory, where it is written before every replay.
            # Both launches stay inside the graph.
            if single:
                inside = ctx.graph_bucket
                ctx.graph_bucket = ctx.graph_bucket or single
                try:
                    attention_bf16.run_decode(out, q, k_pool, v_pool, ctx, group, scale, window, single)
                finally:
                    ctx.graph_bucket = inside
            if single < ctx.num_rows:
                _attention_tc_planned(out, q, k_pool, v_pool, ctx, group, scale, window, recorder, single)
            return
        # Else the call is left out of the graphs and made again for every step that replays them, with
        # that step's context (the operand tensors are the captured pass's own and do not move).
        recorder.defer(lambda step: attention(out, q, k_pool, v_pool, step, group, scale, window))
        return
    if q.dtype == torch.bfloat16:
        # rows at the front that bring one token each (a decode step, or the decoding requests
        # of a mixed step) go to the split-key kernel, the rest to a tiled kernel
        split_ok = attention_bf16.supports(q.shape[2], k_pool.shape[2])
        single = ctx.leading_single_rows if split_ok else 0
        if single:
            attention_bf16.run_decode(out, q, k_pool, v_pool, ctx, group, scale, window, single)
        if single == ctx.num_rows:
            return
        if attention_tc_ok(q, k_pool):
            attention_tc_prefill(out, q, k_pool, v_pool, ctx, group, scale, window, single)
            return
        if split_ok:
            attention_bf16.run_prefill(out, q, k_pool, v_pool, ctx, group, scale, window, single)
            return
    attention_rowwise(out, q, k_pool, v_pool, ctx.positions, ctx.row_of_token, ctx.page_indptr[group],
                      ctx.page_indices[group], scale, window, ctx.status, stream=ctx.stream)


_ATTN_TC_SCRATCH_LIMIT = 1 << 29  # bytes of partial results that a step's attention may ask for
ATTN_TC_SPLITS: tuple[int, int] | None = None  # tests: (key splits, least key tiles per split) instead of the planned ones


def attention_tc_ok(q: torch.Tensor, k_pool: torch.Tensor) -> bool:
    """Whether the tcgen05 prefill attention takes this shape (head size 128, pages of 8..128)."""
    if not TC_ATTENTION or q.shape[2] != 128:
        return False
    return bool(native.attn_tc().ms_attn_tc_supports(q.shape[2], k_pool.shape[2], q.shape[1], k_pool.shape[1]))


_ATTN_TC_PLANNED_SCRATCH = 1 << 25  # floats of partial results that a captured launch may use (128 MB)


def _attention_tc_planned(out, q, k_pool, v_pool, ctx, group: int, scale: float, window: int | None, recorder,
                          first_row: int = 0) -> None:
    """The tcgen05 attention of the rows from ``first_row`` on, launched so that a CUDA graph can hold it:
    one CTA per SM, the plan of those rows (query tiles, rows, key splits) read from device memory.
    Launches with the same heads and window in one pass share the plan, which ``recorder`` has
    written before every replay."""
    _check_dev(out, q, k_pool, v_pool)
    t, nq, d = q.shape
    nkv = k_pool.shape[1]
    lib = native.attn_tc()
    key = ("attn_tc_planned", nq, nkv, int(window or 0), first_row)
    held = recorder.shared.get(key)
    if held is None:
        # (not zeros: made during a capture, the fill would be part of the graph and wipe the plan at every replay)
        plan = torch.empty(8, dtype=torch.int32, device=q.device)
        part = recorder.lasting.get("attn_tc_partials")  # one for all captured shapes: steps run one after the other
        if part is None:
            part = recorder.lasting["attn_tc_partials"] = torch.empty(_ATTN_TC_PLANNED_SCRATCH, dtype=torch.float32, device=q.device)
        queue = ctx.scratch.get("attn_tc_queue")
        if queue is None:
            queue = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)  # zero before the first launch, left zero by every launch
            ctx.scratch["attn_tc_queue"] = queue
        held = recorder.shared[key] = (plan, part, queue)

        def write_plan(step, plan=plan, part=part, queue=queue):
            rows = step.num_rows - first_row
            starts = (ctypes.c_int * rows)(*step.host_q_start[first_row:first_row + rows])
            lens = (ctypes.c_int * rows)(*step.host_q_len[first_row:first_row + rows])
            native.kernel_check(lib.ms_attn_tc_write_plan(_ptr(plan), starts, lens, rows, step.max_q_len, nq, nkv, int(window or 0),
                                                          step.sm_count, part.numel(), queue.numel(), step.stream),
                                lib=lib, errfn="ms_attn_tc_last_error")

        recorder.before(write_plan)
    plan, part, queue = held
    skip = 4 * first_row  # the per-row tables are int32
    native.kernel_check(lib.ms_attn_tc_prefill(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(ctx.cu_q) + skip, _ptr(ctx.q_start) + skip, _ptr(ctx.page_indptr[group]) + skip,
        _ptr(ctx.page_indices[group]), 0, t, 0, nq, nkv, k_pool.shape[0], float(scale), int(window or 0), k_pool.shape[2],
        _ptr(device_status(q.device)), 0, 0, _ptr(part), _ptr(queue), _ptr(plan), ctx.stream),
        lib=lib, errfn="ms_attn_tc_last_error")


def attention_tc_prefill(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: int,
                         scale: float, window: int | None, first_row: int = 0) -> None:
    """Causal attention of rows [first_row, num_rows) of the step, any number of new tokens each,
    on the tcgen05 tensor cores (``csrc/attention_tc.cu``)."""
    _check_dev(out, q, k_pool, v_pool)
    t, nq, d = q.shape
    lib = native.attn_tc()
    skip = 4 * first_row  # the per-row tables are int32
    # a step with few query tiles cuts long key ranges between several CTAs, which leave partial results
    rows = ctx.num_rows - first_row
    key = ("attn_tc_plan", first_row, nq, k_pool.shape[1], int(window or 0))
    plan = ctx.step_cache.get(key)
    if plan is None:  # the same for every layer of the step that has this window
        starts = (ctypes.c_int * rows)(*ctx.host_q_start[first_row:first_row + rows])
        lens = (ctypes.c_int * rows)(*ctx.host_q_len[first_row:first_row + rows])
        splits, min_tiles = ctypes.c_int(), ctypes.c_int()
        lib.ms_attn_tc_plan(starts, lens, rows, nq, k_pool.shape[1], int(window or 0), ctx.sm_count, ctypes.byref(splits),
                            ctypes.byref(min_tiles))
        splits, least = splits.value, min_tiles.value
        if ATTN_TC_SPLITS is not None:
            splits, least = ATTN_TC_SPLITS[0], ATTN_TC_SPLITS[1] or least
        need_f, need_i = ctypes.c_longlong(), ctypes.c_longlong()
        while True:
            lib.ms_attn_tc_scratch(ctx.max_q_len, rows, nq, k_pool.shape[1], splits, ctypes.byref(need_f), ctypes.byref(need_i))
            if splits == 1 or need_f.value * 4 <= _ATTN_TC_SCRATCH_LIMIT:
                break
            splits -= 1
        plan = (splits, least, need_f.value, need_i.value)
        ctx.step_cache[key] = plan
    splits, min_tiles, need_floats, need_ints = plan
    part = None
    if splits > 1:
        part = ctx.scratch.get("attn_tc_partials")
        if part is None or part.numel() < need_floats:
            part = torch.empty(need_floats, dtype=torch.float32, device=q.device)
            ctx.scratch["attn_tc_partials"] = part
    queue = ctx.scratch.get("attn_tc_queue")
    if queue is None or queue.numel() < need_ints:
        # the work queue's counters and the merge tickets: zero before the first launch, left zero by every launch
        queue = torch.zeros(max(need_ints, 1 << 16), dtype=torch.int32, device=q.device)
        ctx.scratch["attn_tc_queue"] = queue
    native.kernel_check(lib.ms_attn_tc_prefill(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(ctx.cu_q) + skip, _ptr(ctx.q_start) + skip, _ptr(ctx.page_indptr[group]) + skip,
        _ptr(ctx.page_indices[group]), rows, t, ctx.max_q_len, nq, k_pool.shape[1], k_pool.shape[0], float(scale),
        int(window or 0), k_pool.shape[2], _ptr(device_status(q.device)), splits, min_tiles, _ptr(part), _ptr(queue), None, ctx.stream),
        lib=lib, errfn="ms_attn_tc_last_error")
