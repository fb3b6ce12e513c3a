"""Python faces of the CUDA entry points.

Every function takes torch tensors that live on the current CUDA device,
launches on torch's current stream and raises ``KernelLibraryError`` when the
entry point refuses its arguments.  There is no other implementation behind
these names: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .lib import KernelLibraryError, library

DT_F32, DT_BF16 = 0, 1

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_void_p = ctypes.c_void_p
_c_size_t = ctypes.c_size_t
_c_int64 = ctypes.c_int64


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return DT_F32
    if dt == torch.bfloat16:
        return DT_BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_cuda:
        raise KernelLibraryError("kernel called with a tensor that is not on a CUDA device; "
                                 "there is no CPU implementation of the product path")
    return _c_void_p(t.data_ptr())


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = library().exl3_last_error().decode("utf-8", "replace")
        raise KernelLibraryError(f"{what} failed (code {rc}): {msg}")


def launch_count() -> int:
    """Kernel launches made through the library so far."""
    lib = library()
    lib.exl3_launch_count.restype = ctypes.c_longlong
    return int(lib.exl3_launch_count())


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------

def embed(ids: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale`` as float32 rows."""
    T = ids.numel()
    V, H = table.shape
    _contig(table, "table")
    if ids.dtype != torch.int32:
        raise KernelLibraryError("embed: ids must be int32")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(library().exl3_embed(_ptr(ids), _ptr(table), _c_int(dtype_code(table.dtype)), _ptr(out),
                                _c_int(T), _c_int(H), _c_int(V), _c_float(scale), _stream()), "embed")
    return out


def add_rmsnorm(h: torch.Tensor, y: Optional[torch.Tensor], y_scale: float, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, out_scale: float = 1.0, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += y * y_scale`` (when y is given), then RMSNorm of the rows of h
    (all, or those listed in ``rows``) times ``weight`` times ``out_scale``."""
    T, H = h.shape
    if h.dtype != torch.float32:
        raise KernelLibraryError("add_rmsnorm: the residual stream must be float32")
    _contig(h, "h")
    if y is not None:
        _contig(y, "y")
        if y.shape != h.shape:
            raise KernelLibraryError(f"add_rmsnorm: y is {tuple(y.shape)}, h is {tuple(h.shape)}")
    if weight.numel() != H:
        raise KernelLibraryError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {H}")
    n = T if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelLibraryError("add_rmsnorm: rows must be int32")
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=h.device)
    _check(library().exl3_add_rmsnorm(
        _ptr(h), _ptr(y), _c_int(dtype_code(y.dtype) if y is not None else 0), _c_float(y_scale),
        _ptr(weight), _c_int(dtype_code(weight.dtype)), _c_float(eps), _ptr(out),
        _c_int(dtype_code(out.dtype)), _c_float(out_scale), _ptr(rows), _c_int(n), _c_int(H), _stream()),
        "add_rmsnorm")
    return out


GATE_ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_tanh": 2}


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleave: int = 0,
             act: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` (``act``: ``silu``, ``gelu`` by erf or ``gelu_tanh``).  ``interleave`` 0: ``gate_up =
    [gate | up]``; 8: eight gate columns, then the eight up columns of the same features, and so on."""
    T, I2 = gate_up.shape
    I = I2 // 2
    _contig(gate_up, "gate_up")
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    _check(library().exl3_act_mul(_ptr(gate_up), _ptr(out), _c_int(dtype_code(gate_up.dtype)), _c_int(T),
                                  _c_int(I), _c_int(interleave), _c_int(GATE_ACTIVATIONS[act]), _stream()), "silu_mul")
    return out


def rotary_table(frequencies: torch.Tensor) -> torch.Tensor:
    """Float64 frequencies as the kernels take them: float32 ``[2, n]``, row 0 the frequencies rounded to
    float32, row 1 what the rounding lost, so that the angle ``position * frequency`` keeps its accuracy at
    large positions.  A plain float32 ``[n]`` table is taken too (no second term)."""
    f = frequencies.to(torch.float64)
    hi = f.to(torch.float32)
    lo = (f - hi.to(torch.float64)).to(torch.float32)
    return torch.stack([hi, lo]).contiguous()


def _rotary_rows(inv_freq: torch.Tensor, rot: int, what: str):
    """The frequency table's pointers: (frequencies, their float32 remainders or null)."""
    if inv_freq.dtype != torch.float32 or inv_freq.numel() not in (rot // 2, rot) or \
            (inv_freq.numel() == rot and inv_freq.dim() != 2):
        raise KernelLibraryError(f"{what}: inv_freq must be float32 with rot / 2 entries, or [2, rot / 2] "
                                 "(see rotary_table)")
    _contig(inv_freq, "inv_freq")
    if inv_freq.dim() == 2 and inv_freq.shape[0] == 2:
        return _ptr(inv_freq[0]), _ptr(inv_freq[1])
    return _ptr(inv_freq), _c_void_p(0)


def rope_kv_write(qkv: torch.Tensor, inv_freq: torch.Tensor, rot: int, pos_scale: float,
                  tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                  k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int, page: int, write_kv: bool) -> None:
    """Rotates q and k inside ``qkv`` and writes rotated k and v to the cache."""
    T = qkv.shape[0]
    _contig(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelLibraryError("rope_kv_write: qkv width does not match the head counts")
    hi, lo = _rotary_rows(inv_freq, rot, "rope_kv_write") if rot else (_c_void_p(0), _c_void_p(0))
    if write_kv and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype):
        raise KernelLibraryError("rope_kv_write: cache and activations differ in element type")
    _check(library().exl3_rope_kv_write(
        _ptr(qkv), _c_int(dtype_code(qkv.dtype)), hi, lo, _c_int(rot), _c_float(pos_scale),
        _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), _c_int(block_table.stride(0)),
        _ptr(k_pool) if write_kv else _c_void_p(0), _ptr(v_pool) if write_kv else _c_void_p(0), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(1 if write_kv else 0),
        _stream()), "rope_kv_write")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` on the CUDA cores, float32 accumulation in K order."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != w.dtype or (bias is not None and bias.dtype != w.dtype):
        raise KernelLibraryError("gemm: x, w and bias must share an element type")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(x.dtype)),
                                    _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
                                    _stream()), "gemm_simt")
    return out


GEMV_MAX_ROWS = 16


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None, gated: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for at most 16 rows of x, weights read once.  With
    ``gated`` the rows of w are eight gate rows then the eight up rows of the
    same features, repeated, and ``silu(gate) * up`` comes out (N / 2 wide)."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemv: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemv_bf16: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)),
                                    _c_int(M), _c_int(N), _c_int(K), _c_int(1 if gated else 0), _stream()),
           "gemv_bf16")
    return out


def gemv_bf16_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                  act_p: float, act_n: float) -> torch.Tensor:
    """``xielu(x @ w.T (+ bias))`` for at most 16 rows of x, the activation in the projection's own epilogue:
    ``act_p z^2 + z / 2`` for ``z > 0``, ``act_n (exp(z) - 1 - z) + z / 2`` otherwise."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError(f"gemv_bf16_act: x {tuple(x.shape)} and w {tuple(w.shape)} must be bfloat16 and fit")
    _contig(x, "x")
    _contig(w, "w")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16_act(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)),
                                        _c_int(M), _c_int(N), _c_int(K), _c_float(act_p), _c_float(act_n),
                                        _stream()), "gemv_bf16_act")
    return out


def gemv_bf16_normed(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                     gated: bool = False, scale=None, resid=None):
    """``gemv_bf16`` as one or both sides of a norm that is no kernel of its own (see gemv_bf16.cuh).

    ``scale = (ss, eps, width)``: ``x`` is the ``x_raw`` of a producing call; results are multiplied per batch row
    by ``rsqrt(ss.sum(1) / width + eps)`` before bias and gating.
    ``resid = (h, rho, norm_w)``: nothing is returned as output; ``h += result * rho`` in place (float32), and
    ``(x_raw, ss)`` is returned: ``h * norm_w`` as bfloat16 and the blocks' sums of squares ``[16, ceil(N/16)]``."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemv_bf16_normed: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemv_bf16_normed: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemv_bf16_normed: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemv_bf16_normed: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemv_bf16_normed: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((16, (N + 15) // 16), dtype=torch.float32, device=x.device)
        _check(library().exl3_gemv_bf16_normed(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(DT_BF16), _c_int(M), _c_int(N), _c_int(K), _c_int(2),
            _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _stream()), "gemv_bf16_normed")
        return x_raw, ss_out
    out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16_normed(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
        _c_int(1 if gated else 0), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None),
        _c_float(0.0), _ptr(None), _c_int(DT_BF16), _ptr(None), _ptr(None), _stream()), "gemv_bf16_normed")
    return out


SKINNY_MAX_ROWS = 128


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                gated: bool = False, scale=None, resid=None, split: int = 0, out: Optional[torch.Tensor] = None,
                tiles: int = 0):
    """``x @ w.T (+ bias)`` for up to 128 rows of x on the tcgen05 tensor cores with the weights read once (the
    weights are the 128-row operand, the batch the narrow one; see gemm_skinny.cu).  ``gated``, ``scale`` and
    ``resid`` as in ``gemv_bf16_normed``; the sums of squares are ``[rows, blocks]`` with any number of rows from
    M up.  ``split``: blocks that share one tile's K range, 0 for the kernel's own choice from N and K;
    ``tiles``: 128-row tiles of w per block (1 or 2; changes no result), 0 for the kernel's choice."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_skinny: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_skinny: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_skinny: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    lib = library()
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemm_skinny: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemm_skinny: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((M, (N + 15) // 16), dtype=torch.float32, device=x.device)
        _check(lib.exl3_gemm_skinny(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(DT_BF16), _c_int(M), _c_int(N), _c_int(K), _c_int(2),
            _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _c_int(split), _c_int(tiles), _stream()), "gemm_skinny")
        return x_raw, ss_out
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    elif tuple(out.shape) != (M, N // 2 if gated else N) or not out.is_contiguous():
        raise KernelLibraryError(f"gemm_skinny: out must be contiguous {(M, N // 2 if gated else N)}")
    _check(lib.exl3_gemm_skinny(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(M), _c_int(N), _c_int(K),
        _c_int(1 if gated else 0), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None),
        _c_float(0.0), _ptr(None), _c_int(DT_BF16), _ptr(None), _ptr(None), _c_int(split), _c_int(tiles), _stream()),
        "gemm_skinny")
    return out


def gemm_skinny_status() -> int:
    """0, or the code a skinny GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_skinny_status())


def gemm_skinny_split(N: int, K: int) -> int:
    """The number of K cuts ``gemm_skinny`` chooses for a weight matrix ``[N, K]``."""
    return int(library().exl3_gemm_skinny_split(_c_int(N), _c_int(K)))


def gemm_pair(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
              out_dtype: torch.dtype = torch.bfloat16, gated: bool = False, scale=None, resid=None,
              out: Optional[torch.Tensor] = None):
    """``x @ w.T (+ bias)`` in bfloat16 for many rows of x, two blocks of a cluster as one tensor core
    (tcgen05.mma.cta_group::2, tiles of 256 x 256; see gemm_pair.cu).  ``gated``, ``scale`` and ``resid`` as in
    ``gemm_skinny``; with ``resid`` the sums of squares come back as ``[M, tiles of 256 columns]`` and the product
    is added to the residual without being rounded to bfloat16 first."""
    if out_dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair: the output is bfloat16")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_pair: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_pair: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    lib = library()
    if resid is not None:
        if gated:
            raise KernelLibraryError("gemm_pair: the gated epilogue does not write into the residual")
        h, rho, norm_w = resid
        if h.dtype != torch.float32 or tuple(h.shape) != (M, N) or tuple(norm_w.shape) != (N,):
            raise KernelLibraryError(f"gemm_pair: h {tuple(h.shape)} / norm weight {tuple(norm_w.shape)} "
                                     f"do not fit an output of {(M, N)}")
        _contig(h, "h")
        _contig(norm_w, "norm_w")
        x_raw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ss_out = torch.empty((M, int(lib.exl3_gemm_pair_ss_blocks(_c_int(N)))), dtype=torch.float32, device=x.device)
        _check(lib.exl3_gemm_pair(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(None), _c_int(M), _c_int(N), _c_int(K), _c_int(2), _ptr(ss_in),
            _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(h), _c_float(rho), _ptr(norm_w),
            _c_int(dtype_code(norm_w.dtype)), _ptr(x_raw), _ptr(ss_out), _stream()), "gemm_pair")
        return x_raw, ss_out
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=x.device)
    elif tuple(out.shape) != (M, N // 2 if gated else N) or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise KernelLibraryError(f"gemm_pair: out must be contiguous bfloat16 {(M, N // 2 if gated else N)}")
    _check(lib.exl3_gemm_pair(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(1 if gated else 0),
        _ptr(ss_in), _c_int(ss_blocks), _c_float(eps), _c_float(width), _ptr(None), _c_float(0.0), _ptr(None),
        _c_int(DT_BF16), _ptr(None), _ptr(None), _stream()), "gemm_pair")
    return out


def gemm_pair_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], scale, tok_pos: torch.Tensor,
                   tok_seq: torch.Tensor, block_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                   rot: int, pos_scale: float, heads: int, kv_heads: int, head_dim: int, page: int,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], write_kv: bool) -> torch.Tensor:
    """The q/k/v projection of many rows (``gemm_pair``; ``scale`` as there) with the rotary encoding and the
    cache write of ``rope_kv_write`` in its epilogue, for heads of 64 rotated as a whole (``rot`` 64) or not at
    all (0) and pages of 64.  Returns ``[M, (heads + 2 kv_heads) * 64]`` of which only the queries' columns are
    written: the rotated keys and the values are in the cache (when ``write_kv``) and nowhere else."""
    M, K = x.shape
    N = (heads + 2 * kv_heads) * head_dim
    if tuple(w.shape) != (N, K):
        raise KernelLibraryError(f"gemm_pair_rope: x is {tuple(x.shape)}, w is {tuple(w.shape)}, heads need {N} rows")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_pair_rope: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    ss_in, ss_blocks, eps, width = None, 0, 0.0, 1.0
    if scale is not None:
        ss_in, eps, width = scale
        if ss_in.dtype != torch.float32 or ss_in.dim() != 2 or ss_in.shape[0] < M:
            raise KernelLibraryError("gemm_pair_rope: ss must be float32 [rows >= M, blocks]")
        _contig(ss_in, "ss")
        ss_blocks = ss_in.shape[1]
    if tok_pos.numel() < M or tok_seq.numel() < M:
        raise KernelLibraryError("gemm_pair_rope: a position and a sequence for every row")
    hi, lo = _rotary_rows(inv_freq, rot, "gemm_pair_rope") if rot else (_c_void_p(0), _c_void_p(0))
    pool_rows = 0
    if write_kv:
        if k_pool.dtype != torch.bfloat16 or v_pool.dtype != torch.bfloat16:
            raise KernelLibraryError("gemm_pair_rope: the cache must be bfloat16")
        _contig(k_pool, "k_pool")
        _contig(v_pool, "v_pool")
        pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _check(library().exl3_gemm_pair_rope(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(K), _ptr(ss_in), _c_int(ss_blocks), _c_float(eps),
        _c_float(width), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table) if write_kv else _c_void_p(0),
        _c_int(block_table.stride(0)) if write_kv else _c_int(0), hi, lo, _c_int(rot), _c_float(pos_scale),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _ptr(k_pool) if write_kv else _c_void_p(0),
        _ptr(v_pool) if write_kv else _c_void_p(0), _c_int64(pool_rows), _c_int(1 if write_kv else 0), _stream()),
        "gemm_pair_rope")
    return out


def gemm_pair_efficiency(M: int, N: int, device) -> float:
    """The share of the GPU's pairs of SMs that ``gemm_pair``'s tiles of 256 x 256 keep busy, averaged over its
    rounds of tiles: 72 tiles on 74 pairs 0.97, 32 tiles 0.43, 80 tiles (two rounds, the second nearly empty) 0.54."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    pairs = max(1, sm_count(device) // 2)
    return tiles / float(((tiles + pairs - 1) // pairs) * pairs)


def gemm_pair_status() -> int:
    """0, or the code a paired tensor-core GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_pair_status())


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
            gated: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` in bfloat16 on the tcgen05 tensor cores; with ``gated``
    the rows of w are interleaved in eights and ``silu(gate) * up`` comes out."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelLibraryError(f"gemm_tc: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError("gemm_tc: x and w must be bfloat16")
    _contig(x, "x")
    _contig(w, "w")
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=torch.bfloat16, device=x.device)
    _check(library().exl3_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(M), _c_int(N), _c_int(K),
                                  _c_int(1 if gated else 0), _stream()), "gemm_tc")
    return out


def gemm_tc_status() -> int:
    """0, or the code a tensor-core GEMM left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_gemm_tc_status())


def gemm_tc_wait_selftest() -> None:
    """Runs a kernel whose mbarrier wait is never satisfied; it must give up and set status 9."""
    _check(library().exl3_gemm_tc_wait_selftest(_stream()), "gemm_tc_wait_selftest")


def attn_tokens_scratch_bytes(T: int, heads: int, head_dim: int, max_splits: int) -> int:
    lib = library()
    lib.exl3_attn_tokens_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_attn_tokens_scratch_bytes(_c_int(T), _c_int(heads), _c_int(head_dim), _c_int(max_splits)))


def attn_tokens(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                v_pool: torch.Tensor, block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                T: int, heads: int, kv_heads: int, head_dim: int, page: int, window: int, scale: float,
                split_keys: int, max_splits: int, scratch: Optional[torch.Tensor]) -> torch.Tensor:
    """Attention of T query tokens over the paged cache (see attention_simt.cu)."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_tokens: q, cache and out differ in element type")
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_tokens(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _c_int(dtype_code(q.dtype)), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_float(scale),
        _c_int(split_keys), _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes), _stream()), "attn_tokens")
    return out


def attn_tokens_kv(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                   v_pool: torch.Tensor, block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                   T: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, kv_row: int, page: int,
                   window: int, scale: float, split_keys: int, max_splits: int,
                   scratch: Optional[torch.Tensor]) -> torch.Tensor:
    """``attn_tokens`` with values of ``value_dim <= head_dim`` features and rows of both pools ``kv_row`` elements
    apart; ``out`` is ``[T, heads, value_dim]`` and the scratch is sized with ``value_dim``.  With ``v_pool`` the
    key pool itself, the values are the keys' first ``value_dim`` features."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_tokens_kv: q, cache and out differ in element type")
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_tokens_kv(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _c_int(dtype_code(q.dtype)), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim), _c_int(kv_row), _c_int(page),
        _c_int(window), _c_float(scale), _c_int(split_keys), _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes),
        _stream()), "attn_tokens_kv")
    return out


def attn_tokens_ex(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor,
                   v_pool: torch.Tensor, block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                   T: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, page: int, window: int,
                   chunk: int, sink: bool, scale: float, split_keys: int, max_splits: int,
                   scratch: Optional[torch.Tensor], keep_first: int = 0, softcap: float = 0.0,
                   sink_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attn_tokens`` in its general form: rows of the key pool hold ``head_dim`` features and rows of the value
    pool ``value_dim`` (each pool's last dimension is its row pitch; multiples of 8; values may be wider than keys);
    ``chunk`` > 0 also hides every key before ``floor(pos / chunk) * chunk``; ``sink`` adds one to the softmax's
    denominator (``sink_vals`` float32 ``[heads]``: ``exp`` of a score per head instead of one).  With a window,
    keys at positions below ``keep_first`` stay visible (``max_splits`` then counts their chunks too); ``softcap``
    > 0 caps the scaled scores, ``c tanh(s / c)``.  ``out`` is ``[T, heads, value_dim]`` in the cache's type or
    float32 (for callers that go on in float32) and the scratch is sized with ``value_dim``."""
    if sink_vals is not None and (sink_vals.dtype != torch.float32 or sink_vals.numel() != heads or not sink):
        raise KernelLibraryError("attn_tokens_ex: sink scores must be float32 [heads], with the sink on")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype not in (q.dtype, torch.float32):
        raise KernelLibraryError("attn_tokens_ex: q, cache and out differ in element type")
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_tokens_opt(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _c_int(1 if out.dtype == torch.float32 else 0),
        _c_int(dtype_code(q.dtype)), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T),
        _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim), _c_int(k_pool.shape[-1]),
        _c_int(v_pool.shape[-1]), _c_int(page), _c_int(window), _c_int(chunk), _c_int(1 if sink else 0),
        _c_float(scale), _c_int(split_keys), _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes), _c_int(keep_first),
        _c_float(softcap), _ptr(sink_vals), _stream()), "attn_tokens_ex")
    return out


def embed_hashed(ids: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor, row_start: torch.Tensor,
                 slot_ids: torch.Tensor, table: torch.Tensor, extra: torch.Tensor, buckets: int, mul_prev: int,
                 mul_cur: int, last_token: torch.Tensor) -> torch.Tensor:
    """``table[id] + extra[(prev * mul_prev + id * mul_cur) mod buckets]`` as float32 rows (``extra[buckets]`` at
    position 0); ``last_token`` (int32 per slot) gives the token before a row's first one and is left holding the
    row's last one (see hashed_embed.cu)."""
    T = ids.numel()
    V, H = table.shape
    _contig(table, "table")
    _contig(extra, "extra")
    if ids.dtype != torch.int32 or last_token.dtype != torch.int32:
        raise KernelLibraryError("embed_hashed: ids and last_token must be int32")
    if extra.dtype != table.dtype or tuple(extra.shape) != (buckets + 1, H):
        raise KernelLibraryError(f"embed_hashed: the second table must be {(buckets + 1, H)} in the first one's type")
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(library().exl3_embed_hashed(
        _ptr(ids), _ptr(tok_pos), _ptr(tok_seq), _ptr(row_start), _ptr(slot_ids), _ptr(table), _ptr(extra),
        _c_int(dtype_code(table.dtype)), _c_int(buckets), ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur),
        _ptr(last_token), _ptr(out), _c_int(T), _c_int(H), _c_int(V), _stream()), "embed_hashed")
    return out


def qk_prep(x: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, head_dim: int,
            value_dim: int, head_pad: int, value_pad: int, norm: int, q_w: Optional[torch.Tensor],
            k_w: Optional[torch.Tensor], eps: float, rot: int, layout: int, inv_freq: Optional[torch.Tensor],
            mscale: float, k_mul: float, mix: Optional[tuple], tok_pos: torch.Tensor, tok_seq: torch.Tensor,
            block_table: Optional[torch.Tensor], page: int, q_dtype: torch.dtype,
            k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
            k_dtype: Optional[torch.dtype] = None):
    """Norm, rotation, value mixing and the cache write between an attention's joint projection ``x [T, ld]`` and
    the attention (see qk_prep.cu).  ``mix``: ``(lambda tensor, v_src [T, *] view)`` or None.  Returns ``(q, k)``:
    the queries ``[T, heads * head_pad]`` and, when there is no ``k_pool``, the keys ``[T, kv_heads * head_pad]``
    (else None)."""
    T = x.shape[0]
    if x.stride(1) != 1:
        raise KernelLibraryError("qk_prep: rows of x must be dense")
    hi, lo = (_rotary_rows(inv_freq, rot, "qk_prep") if rot else (_c_void_p(0), _c_void_p(0)))
    q = torch.empty((T, heads * head_pad), dtype=q_dtype, device=x.device)
    k = None
    if k_pool is None:
        k = torch.empty((T, kv_heads * head_pad), dtype=k_dtype or q_dtype, device=x.device)
    lam, v_src = mix if mix is not None else (None, None)
    if v_src is not None and v_src.stride(1) != 1:
        raise KernelLibraryError("qk_prep: rows of the mixed-in values must be dense")
    _check(library().exl3_qk_prep(
        _ptr(x), _c_int(dtype_code(x.dtype)), _c_int64(x.stride(0)), _c_int(q_off), _c_int(k_off), _c_int(v_off),
        _c_int(T), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim), _c_int(head_pad),
        _c_int(value_pad), _c_int(norm), _ptr(q_w), _ptr(k_w), _c_int(dtype_code(q_w.dtype) if q_w is not None else 0),
        _c_float(eps), _c_int(rot), _c_int(layout), hi, lo, _c_float(mscale), _c_float(k_mul), _ptr(lam),
        _c_int(dtype_code(lam.dtype) if lam is not None else 0), _ptr(v_src),
        _c_int(dtype_code(v_src.dtype) if v_src is not None else 0),
        _c_int64(v_src.stride(0) if v_src is not None else 0), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table),
        _c_int(block_table.stride(0) if block_table is not None else 0), _c_int(page), _ptr(q),
        _c_int(dtype_code(q.dtype)), _ptr(k), _c_int(dtype_code(k.dtype) if k is not None else 0), _ptr(k_pool),
        _ptr(v_pool), _c_int(dtype_code(k_pool.dtype) if k_pool is not None else 0), _stream()), "qk_prep")
    return q, k


def token_shift(h: torch.Tensor, mu: torch.Tensor, prev: torch.Tensor, tok_seq: torch.Tensor, row_start: torch.Tensor,
                slot_ids: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]`` for the ``n`` rows of ``mu [n, H]``; the row before a
    sequence's first token of the step comes from ``prev`` (float32 ``[slots, H]``) and the step's last row is
    left there (see linear_scan.cu)."""
    T, H = h.shape
    _contig(h, "h")
    _contig(mu, "mu")
    if prev.dtype != torch.float32 or prev.shape[1] != H or mu.shape[1] != H:
        raise KernelLibraryError("token_shift: prev must be float32 [slots, H] and mu [n, H]")
    out = torch.empty((mu.shape[0], T, H), dtype=out_dtype, device=h.device)
    _check(library().exl3_token_shift(
        _ptr(h), _c_int(dtype_code(h.dtype)), _ptr(mu), _c_int(dtype_code(mu.dtype)), _c_int(mu.shape[0]), _ptr(prev),
        _ptr(tok_seq), _ptr(row_start), _ptr(slot_ids), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(T), _c_int(H),
        _stream()), "token_shift")
    return out


def linear_scan_scratch_bytes(rows: int, T: int, heads: int, dk: int, dv: int, max_new: int) -> int:
    lib = library()
    lib.exl3_linear_scan_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_linear_scan_scratch_bytes(_c_int(rows), _c_int(T), _c_int(heads), _c_int(dk), _c_int(dv),
                                                  _c_int(max_new)))


def linear_scan(mode: int, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor,
                slot_ids: torch.Tensor, row_start: torch.Tensor, rows: int, heads: int, dk: int, dv: int, max_new: int,
                wraw: Optional[torch.Tensor] = None, w0: Optional[torch.Tensor] = None,
                u: Optional[torch.Tensor] = None, decay: Optional[torch.Tensor] = None,
                scratch: Optional[torch.Tensor] = None, in_act: str = "none") -> torch.Tensor:
    """The recurrence with a matrix state per head over a step's packed tokens (see linear_scan.cu).  ``r``, ``k``
    ``[T, heads * dk]`` and ``v [T, heads * dv]`` may be views with their own row pitch; ``state`` float32 ``[slots,
    heads, dk, dv]`` is read and written at ``slot_ids``.  Mode 0: decays ``exp(-exp(wraw + w0))`` per token and key
    channel and the bonus ``u``; mode 1: ``decay`` float32 ``[heads]``.  ``in_act`` ``"silu"``: ``r``, ``k`` and ``v`` go
    through SiLU (float32) as they are read.  Returns float32 ``[T, heads * dv]``."""
    T = r.shape[0]
    for t, name in ((r, "r"), (k, "k"), (v, "v"), (wraw, "wraw")):
        if t is not None and t.stride(1) != 1:
            raise KernelLibraryError(f"linear_scan: rows of {name} must be dense")
    if r.dtype != k.dtype:
        raise KernelLibraryError("linear_scan: r and k differ in element type")
    _contig(state, "state")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dk, dv):
        raise KernelLibraryError(f"linear_scan: state {tuple(state.shape)} must be float32 [slots, {heads}, {dk}, {dv}]")
    if mode == 0 and (w0.dtype != u.dtype or w0.numel() != heads * dk or u.numel() != heads * dk):
        raise KernelLibraryError("linear_scan: w0 and u must hold heads * dk values of one type")
    if mode == 1 and (decay.dtype != torch.float32 or decay.numel() != heads):
        raise KernelLibraryError("linear_scan: decay must be float32 [heads]")
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=r.device)
    _check(library().exl3_linear_scan(
        _c_int(mode), _ptr(r), _c_int64(r.stride(0)), _ptr(k), _c_int64(k.stride(0)), _c_int(dtype_code(r.dtype)),
        _ptr(v), _c_int64(v.stride(0)), _c_int(dtype_code(v.dtype)), _ptr(wraw),
        _c_int64(wraw.stride(0) if wraw is not None else 0), _c_int(dtype_code(wraw.dtype) if wraw is not None else 0),
        _ptr(w0), _ptr(u), _c_int(dtype_code(w0.dtype) if w0 is not None else 0), _ptr(decay), _ptr(state),
        _ptr(slot_ids), _ptr(row_start), _ptr(out), _c_int(rows), _c_int(T), _c_int(heads), _c_int(dk), _c_int(dv),
        _c_int(max_new), _c_int({"none": 0, "silu": 1}[in_act]), _ptr(scratch),
        _c_size_t(0 if scratch is None else scratch.numel() * scratch.element_size()), _stream()), "linear_scan")
    return out


def head_norm_gate(o: torch.Tensor, w: Optional[torch.Tensor], gate: Optional[torch.Tensor], eps: float, heads: int,
                   dv: int, out_dtype: torch.dtype, gate_kind: str = "silu") -> torch.Tensor:
    """``o [T, heads * dv]`` (float32) head by head divided by its root mean square, times ``w [heads * dv]`` and
    ``silu(gate [T, heads * dv])`` (``gate_kind`` ``"sigmoid"``: the sigmoid alone) where given."""
    T = o.shape[0]
    _contig(o, "o")
    if o.dtype != torch.float32 or o.shape[1] != heads * dv:
        raise KernelLibraryError("head_norm_gate: o must be float32 [T, heads * dv]")
    if gate is not None and gate.stride(1) != 1:
        raise KernelLibraryError("head_norm_gate: rows of the gate must be dense")
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o.device)
    _check(library().exl3_head_norm_gate(
        _ptr(o), _ptr(w), _c_int(dtype_code(w.dtype) if w is not None else 0), _ptr(gate),
        _c_int(dtype_code(gate.dtype) if gate is not None else 0), _c_int64(gate.stride(0) if gate is not None else 0),
        _c_int({"silu": 0, "sigmoid": 1}[gate_kind]), _c_float(eps), _ptr(out), _c_int(dtype_code(out.dtype)), _c_int(T),
        _c_int(heads), _c_int(dv), _stream()), "head_norm_gate")
    return out


def normed_sum2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float,
                coef: float) -> torch.Tensor:
    """``coef * (rmsnorm(a) * wa + rmsnorm(b) * wb)`` row by row, float32."""
    T, H = a.shape
    _contig(a, "a")
    _contig(b, "b")
    if a.dtype != b.dtype or a.shape != b.shape or wa.dtype != wb.dtype or wa.numel() != H or wb.numel() != H:
        raise KernelLibraryError("normed_sum2: a and b, and their weights, must agree in shape and type")
    out = torch.empty((T, H), dtype=torch.float32, device=a.device)
    _check(library().exl3_normed_sum2(_ptr(a), _ptr(b), _c_int(dtype_code(a.dtype)), _ptr(wa), _ptr(wb),
                                      _c_int(dtype_code(wa.dtype)), _c_float(eps), _c_float(coef), _ptr(out),
                                      _c_int(T), _c_int(H), _stream()), "normed_sum2")
    return out


ACTIVATION_KINDS = {"gelu": 0, "gelu_tanh": 1, "tanh": 2, "relu2": 3}


def activation(z: torch.Tensor, out_dtype: torch.dtype, kind: str) -> torch.Tensor:
    """An activation of every element, float32 inside: ``gelu`` (exact, by erf), ``gelu_tanh`` (the tanh formula)
    ``tanh`` or ``relu2`` (the square of relu)."""
    _contig(z, "z")
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _check(library().exl3_activation(_ptr(z), _c_int(dtype_code(z.dtype)), _ptr(out), _c_int(dtype_code(out.dtype)),
                                     _c_int64(z.numel()), _c_int(ACTIVATION_KINDS[kind]), _stream()), "activation")
    return out


def attn_latent_supported(dtype: torch.dtype, dk: int, dv: int, page: int) -> bool:
    """Whether the tensor-core kernel for latent rows takes these sizes."""
    return (dtype == torch.bfloat16 and page == 64 and dk % 16 == 0 and dv % 16 == 0 and dv <= min(dk, 512)
            and int(library().exl3_attn_latent_row_tile(_c_int(dk), _c_int(16))) >= 1)


def attn_latent_status() -> int:
    """1 when a block of the latent attention kernel gave up on a bounded wait since the last call; clears it."""
    return int(library().exl3_attn_latent_status())


def attn_latent_row_tile(dk: int, max_rows: int) -> int:
    """Rows of one sequence that a block of the kernel takes for these sizes."""
    return 16 * int(library().exl3_attn_latent_row_tile(_c_int(dk), _c_int(max_rows)))


def attn_latent_scratch_bytes(T: int, heads: int, dv: int, n_splits: int) -> int:
    lib = library()
    lib.exl3_attn_latent_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_attn_latent_scratch_bytes(_c_int(T), _c_int(heads), _c_int(dv), _c_int(n_splits)))


def attn_latent(q: torch.Tensor, out: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                row_start: torch.Tensor, row_pos0: torch.Tensor, rows: int, T: int, max_new: int, heads: int, dk: int,
                dv: int, page: int, scale: float, pages_per_chunk: int, n_splits: int,
                scratch: Optional[torch.Tensor], gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a step's tokens over latent rows on the tensor cores (see attention_latent.cu): ``q [T, heads *
    dk]``, ``out [T, heads * dv]``, one cached row of ``dk`` features per key whose first ``dv`` are the values."""
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelLibraryError("attn_latent: q, out and the cache must be bfloat16")
    _contig(q, "q")
    _contig(out, "out")
    _contig(pool, "pool")
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_latent(
        _ptr(q), _ptr(out), _ptr(pool), _c_int64(pool.numel() // (64 * dk)), _ptr(block_table),
        _c_int(block_table.stride(0)), _ptr(row_start),
        _ptr(row_pos0), _c_int(rows), _c_int(T), _c_int(max_new), _c_int(heads), _c_int(dk), _c_int(dv), _c_int(page),
        _c_float(scale), _c_int(pages_per_chunk), _c_int(n_splits), _ptr(scratch), _c_size_t(nbytes), _ptr(gate),
        _stream()), "attn_latent")
    return out


def norm_add(h: torch.Tensor, y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
             x_dtype: Optional[torch.dtype]) -> Optional[torch.Tensor]:
    """``h += y * rsqrt(mean(y^2) + eps) * weight`` per row, in place and in float32 (nothing when ``y`` is None);
    returns ``h`` in ``x_dtype`` as a new tensor (None when ``x_dtype`` is None)."""
    T, H = h.shape
    if h.dtype != torch.float32:
        raise KernelLibraryError("norm_add: the residual stream must be float32")
    _contig(h, "h")
    if y is not None:
        _contig(y, "y")
        if tuple(y.shape) != (T, H) or weight is None or weight.numel() != H:
            raise KernelLibraryError(f"norm_add: y {tuple(y.shape)} / weight do not fit h {tuple(h.shape)}")
    x = torch.empty((T, H), dtype=x_dtype, device=h.device) if x_dtype is not None else None
    if y is None and x is None:
        return None
    _check(library().exl3_norm_add(
        _ptr(h), _ptr(y), _c_int(dtype_code(y.dtype) if y is not None else 0), _ptr(weight),
        _c_int(dtype_code(weight.dtype) if weight is not None else 0), _c_float(eps), _ptr(x),
        _c_int(dtype_code(x.dtype) if x is not None else 0), _c_int(T), _c_int(H), _stream()), "norm_add")
    return x


def norm_add_norm(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, weight2: torch.Tensor,
                  eps2: float, x_dtype: torch.dtype) -> torch.Tensor:
    """``h += y * rsqrt(mean(y^2) + eps) * weight`` in place (float32) and, in the same kernel, the norm of the new
    residual: returns ``h * rsqrt(mean(h^2) + eps2) * weight2`` in ``x_dtype``."""
    T, H = h.shape
    if h.dtype != torch.float32:
        raise KernelLibraryError("norm_add_norm: the residual stream must be float32")
    _contig(h, "h")
    _contig(y, "y")
    if tuple(y.shape) != (T, H) or weight.numel() != H or weight2.numel() != H:
        raise KernelLibraryError(f"norm_add_norm: y {tuple(y.shape)} / weights do not fit h {tuple(h.shape)}")
    x = torch.empty((T, H), dtype=x_dtype, device=h.device)
    _check(library().exl3_norm_add_norm(
        _ptr(h), _ptr(y), _c_int(dtype_code(y.dtype)), _ptr(weight), _c_int(dtype_code(weight.dtype)), _c_float(eps),
        _ptr(weight2), _c_int(dtype_code(weight2.dtype)), _c_float(eps2), _ptr(x), _c_int(dtype_code(x.dtype)),
        _c_int(T), _c_int(H), _stream()), "norm_add_norm")
    return x


def gemv_bf16_gelu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                   tanh: bool = False, relu2: bool = False) -> torch.Tensor:
    """``gelu(x @ w.T (+ bias))`` for at most 16 rows of x, the activation (exact, or by the tanh formula; with
    ``relu2`` the square of relu instead) in the projection's own epilogue."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelLibraryError(f"gemv_bf16_gelu: x {tuple(x.shape)} and w {tuple(w.shape)} must be bfloat16 and fit")
    _contig(x, "x")
    _contig(w, "w")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(library().exl3_gemv_bf16_gelu(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _c_int(dtype_code(out.dtype)),
                                         _c_int(M), _c_int(N), _c_int(K), _c_int(2 if relu2 else (1 if tanh else 0)), _stream()),
           "gemv_bf16_gelu")
    return out


def xielu(z: torch.Tensor, pq: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """xIELU of every element with the raw parameter pair ``pq`` (see outnorm.cu)."""
    _contig(z, "z")
    if pq.numel() != 2:
        raise KernelLibraryError("xielu: the activation takes two parameters")
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _check(library().exl3_xielu(_ptr(z), _c_int(dtype_code(z.dtype)), _ptr(pq), _c_int(dtype_code(pq.dtype)),
                                _ptr(out), _c_int(dtype_code(out.dtype)), _c_int64(z.numel()), _stream()), "xielu")
    return out


def mingru_scratch_bytes(rows: int, T: int, width: int, max_new: int) -> int:
    lib = library()
    lib.exl3_mingru_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_mingru_scratch_bytes(_c_int(rows), _c_int(T), _c_int(width), _c_int(max_new)))


def mingru_scan(zug: torch.Tensor, state: torch.Tensor, slot_ids: torch.Tensor, row_start: torch.Tensor,
                rows: int, width: int, max_new: int, out_dtype: torch.dtype,
                scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The minGRU recurrence over a step's packed tokens (see recurrent.cu): ``zug [T, 3 * width]``, ``state
    [slots, width]`` float32 read and written at ``slot_ids``; returns ``S_t * silu(g_t)`` as ``[T, width]``."""
    T = zug.shape[0]
    _contig(zug, "zug")
    _contig(state, "state")
    if zug.shape[1] != 3 * width or state.dtype != torch.float32 or state.shape[1] != width:
        raise KernelLibraryError(f"mingru_scan: zug {tuple(zug.shape)} / state {tuple(state.shape)} do not fit width {width}")
    if slot_ids.dtype != torch.int32 or row_start.dtype != torch.int32:
        raise KernelLibraryError("mingru_scan: slot_ids and row_start must be int32")
    y = torch.empty((T, width), dtype=out_dtype, device=zug.device)
    _check(library().exl3_mingru_scan(_ptr(zug), _c_int(dtype_code(zug.dtype)), _ptr(y), _c_int(dtype_code(y.dtype)),
                                      _ptr(state), _ptr(slot_ids), _ptr(row_start), _c_int(rows), _c_int(T),
                                      _c_int(width), _c_int(max_new), _ptr(scratch),
                                      _c_size_t(0 if scratch is None else scratch.numel() * scratch.element_size()),
                                      _stream()), "mingru_scan")
    return y


def latent_prep(a: torch.Tensor, q_off: int, q_rank: int, wq: torch.Tensor, kv_off: int, kv_rank: int, rot_dim: int,
                wkv: Optional[torch.Tensor], g_off: int, heads: int, eps: float, inv_freq: Optional[torch.Tensor],
                rot: int, tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, page: int,
                pool: Optional[torch.Tensor], kv_row: int, rank_pad: int, cq_dtype: torch.dtype):
    """Latent attention's step between the joint input projection ``a`` and the rest (see latent.cu): returns the
    normed query latent ``[T, q_rank]`` and the float32 gates ``[T, heads]``; writes each token's row of the cache
    (``pool``; None for a layer that reads another layer's rows)."""
    T = a.shape[0]
    _contig(a, "a")
    f_hi, f_lo = (_rotary_rows(inv_freq, rot, "latent_prep") if rot > 0 and inv_freq is not None
                  else (_c_void_p(0), _c_void_p(0)))
    cq = torch.empty((T, q_rank), dtype=cq_dtype, device=a.device)
    gate = torch.empty((T, heads), dtype=torch.float32, device=a.device)
    _check(library().exl3_latent_prep(
        _ptr(a), _c_int(dtype_code(a.dtype)), _c_int(a.shape[1]), _c_int(T), _c_int(q_off), _c_int(q_rank), _ptr(wq),
        _c_int(dtype_code(wq.dtype)), _c_int(kv_off), _c_int(kv_rank), _c_int(rot_dim), _ptr(wkv),
        _c_int(dtype_code(wkv.dtype) if wkv is not None else 0), _c_int(g_off), _c_int(heads), _c_float(eps), f_hi, f_lo,
        _c_int(rot), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), _c_int(block_table.stride(0)), _c_int(page),
        _ptr(pool), _c_int(dtype_code(pool.dtype) if pool is not None else 0), _c_int(kv_row), _c_int(rank_pad),
        _ptr(cq), _c_int(dtype_code(cq.dtype)), _ptr(gate), _stream()), "latent_prep")
    return cq, gate


def head_gemm(x: torch.Tensor, x_row: int, x_head: int, w: Optional[torch.Tensor], out: torch.Tensor, out_row: int,
              out_head: int, T: int, heads: int, K: int, N: int, mul: Optional[torch.Tensor] = None, rot_dim: int = 0,
              rot: int = 0, inv_freq: Optional[torch.Tensor] = None, tok_pos: Optional[torch.Tensor] = None,
              tail_off: int = 0) -> torch.Tensor:
    """``out[t, h, n] = mul[t, h] * sum_k x[t, h, k] w[h, k, n]`` with the given row and head pitches (elements);
    with ``rot_dim`` the features behind a head's ``K`` are rotated and written at ``tail_off`` (see latent.cu).  With
    ``w`` None only those tails (and the zeros around them) are written."""
    if w is not None:
        if w.dtype != x.dtype or tuple(w.shape) != (heads, K, N):
            raise KernelLibraryError(f"head_gemm: w {tuple(w.shape)} must be {(heads, K, N)} in the type of x and out")
        _contig(w, "w")
    if out.dtype != x.dtype:
        raise KernelLibraryError("head_gemm: x and out differ in element type")
    f_hi, f_lo = (_rotary_rows(inv_freq, rot, "head_gemm") if rot > 0 and inv_freq is not None
                  else (_c_void_p(0), _c_void_p(0)))
    _check(library().exl3_head_gemm(
        _ptr(x), _c_int64(x_row), _c_int(x_head), _ptr(w), _ptr(out), _c_int64(out_row), _c_int(out_head),
        _c_int(dtype_code(x.dtype)), _c_int(T), _c_int(heads), _c_int(K), _c_int(N), _ptr(mul), _c_int(rot_dim),
        _c_int(rot), f_hi, f_lo, _ptr(tok_pos), _c_int(tail_off), _stream()), "head_gemm")
    return out


def attn_prefill_tc_supported(dtype: torch.dtype, head_dim: int, page: int) -> bool:
    return bool(library().exl3_attn_prefill_tc_supported(_c_int(dtype_code(dtype)), _c_int(head_dim), _c_int(page)))


def attn_prefill_tc_status() -> int:
    """0, or the code a tcgen05 attention kernel left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_attn_prefill_tc_status())


def attn_prefill_tc(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    block_table: torch.Tensor, row_start: torch.Tensor, row_pos0: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, heads: int, kv_heads: int,
                    head_dim: int, page: int, window: int, scale: float, variant: int = 0, chunk: int = 0,
                    sink: bool = False, keep_first: int = 0, softcap: float = 0.0,
                    sink_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of whole prompts on tcgen05 tensor cores (tiles of 128 queries; see
    attention_prefill_tc.cu).  ``k_pool`` / ``v_pool``: one layer's ``[pages, kv_heads, 64, head_dim]``.
    ``variant``: 0 lets the kernel choose by the number of blocks between a tile a block, four blocks per SM (heads
    of 64) and two tiles a block (the list's first with its last, and so on: list the tiles with the most keys
    to visit first); 1, 2 and 3 force one of them (the same numbers every way).  ``chunk``, ``sink``, ``keep_first``,
    ``softcap`` and ``sink_vals`` as in ``attn_tokens_ex``."""
    if sink_vals is not None and (sink_vals.dtype != torch.float32 or sink_vals.numel() != heads or not sink):
        raise KernelLibraryError("attn_prefill_tc: sink scores must be float32 [heads], with the sink on")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_prefill_tc: q, cache and out differ in element type")
    _contig(k_pool, "k_pool")
    _contig(v_pool, "v_pool")
    pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    _check(library().exl3_attn_prefill_tc_opt(
        _ptr(q), _c_int64(q_row_stride), _c_int(q.shape[0]), _ptr(out), _ptr(k_pool), _ptr(v_pool),
        _c_int64(pool_rows), _ptr(block_table), _c_int(block_table.stride(0)), _ptr(row_start), _ptr(row_pos0),
        _ptr(tile_seq), _ptr(tile_q0), _c_int(n_tiles), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
        _c_int(page), _c_int(window), _c_int(chunk), _c_int(1 if sink else 0), _c_float(scale), _c_int(variant),
        _c_int(keep_first), _c_float(softcap), _ptr(sink_vals), _stream()), "attn_prefill_tc")
    return out


_SM_COUNT: dict = {}


def sm_count(device: torch.device) -> int:
    """Streaming multiprocessors of ``device`` (looked up once)."""
    key = torch.device(device).index or 0
    n = _SM_COUNT.get(key)
    if n is None:
        n = _SM_COUNT[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return n


ATTN_DECODE_MAX_CHUNKS = 256      # chunks of one (token, kv head) that attn_decode takes


def attn_decode_supported(dtype: torch.dtype, T: int, heads: int, kv_heads: int, head_dim: int, page: int,
                          split_keys: int, max_splits: int) -> bool:
    return bool(library().exl3_attn_decode_supported(
        _c_int(dtype_code(dtype)), _c_int(T), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page),
        _c_int(split_keys), _c_int(max_splits)))


def attn_decode_status() -> int:
    """0, or the code the decode attention kernel left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_attn_decode_status())


def attn_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                block_table: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor, T: int, heads: int,
                kv_heads: int, head_dim: int, page: int, window: int, scale: float, split_keys: int,
                max_splits: int, scratch: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor] = None,
                rot: int = 0, pos_scale: float = 1.0, write_new: bool = False, head_split: int = 1,
                in_block: int = 0, twins: int = 1, chunk: int = 0, sink: bool = False) -> torch.Tensor:
    """Attention of T query tokens over the paged cache on the tensor cores (see attention_decode.cu);
    arguments and scratch as ``attn_tokens``.  With ``write_new``, ``q`` is the fused q|k|v output of the
    projection, every token is its sequence's only new one and the cache holds the positions before it: the
    kernel adds the token's own key and value to its softmax and writes them to the cache.  With ``rot`` equal to
    ``head_dim`` it applies the half-split rotary encoding (``inv_freq``: head_dim / 2 float32 frequencies, or a ``rotary_table``) to
    the queries and the new key.  ``head_split`` n (a divisor of the query heads per kv head) makes n groups of work
    of a kv head's query heads: n times the work items, each merge an n-th of the size; changes no result.
    ``in_block`` 1 (or True): one block per (token, group of heads), whose four warps take the item's chunks
    (``max_splits`` at most 4) and merge them in shared memory; 2: a cluster of two blocks per item (at most 8
    chunks; the first block merges and reads the second one's records out of its shared memory): no scratch, no
    tickets; results differ from the other way's by rounding (another order of the same sums).  ``twins`` 2 (with
    ``in_block`` 1 or 2, an even ``head_split`` and groups of up to 8 heads): a block takes two groups of query heads
    of a kv head, whose warps walk the same pages out of the same rings; changes no result.  ``chunk`` and ``sink`` as
    in ``attn_tokens_ex``."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelLibraryError("attn_decode: q, cache and out differ in element type")
    _contig(k_pool, "k_pool")
    _contig(v_pool, "v_pool")
    hi = lo = _c_void_p(0)
    if rot:
        if inv_freq is None:
            raise KernelLibraryError("attn_decode: rot needs inv_freq")
        hi, lo = _rotary_rows(inv_freq, rot, "attn_decode")
    pool_rows = k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2]
    nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _check(library().exl3_attn_decode(
        _ptr(q), _c_int64(q_row_stride), _ptr(out), _ptr(k_pool), _ptr(v_pool), _c_int64(pool_rows),
        _ptr(block_table), _c_int(block_table.stride(0)), _ptr(tok_pos), _ptr(tok_seq), _c_int(T), _c_int(heads),
        _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_int(chunk), _c_int(1 if sink else 0),
        _c_float(scale), _c_int(split_keys), _c_int(max_splits), _ptr(scratch), _c_size_t(nbytes), hi, lo, _c_int(rot),
        _c_float(pos_scale), _c_int(1 if write_new else 0), _c_int(head_split), _c_int(int(in_block)),
        _c_int(int(twins)), _stream()), "attn_decode")
    return out


def check_status() -> None:
    """Raises if a kernel with bounded waits (the tcgen05 GEMMs and attention, the TMA decode attention) gave up
    on one since the last call: its results are then not to be trusted.  Reads their flags from the device, so
    it waits for the work launched so far; call it where the host waits anyway."""
    gave_up = [name for name, fn in (("gemm_tc", gemm_tc_status), ("gemm_skinny", gemm_skinny_status),
                                     ("gemm_pair", gemm_pair_status),
                                     ("attn_prefill_tc", attn_prefill_tc_status),
                                     ("attn_decode", attn_decode_status),
                                     ("attn_latent", attn_latent_status), ("moe_gemm_tc", moe_tc_status)) if fn()]
    if gave_up:
        raise KernelLibraryError("a bounded wait ran out in " + ", ".join(gave_up) +
                                 ": a copy or a tensor-core product did not complete in time")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    if logits.dtype != torch.float32:
        raise KernelLibraryError("argmax: logits must be float32")
    _contig(logits, "logits")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    lib = library()
    lib.exl3_argmax_scratch_bytes.restype = _c_size_t
    need = int(lib.exl3_argmax_scratch_bytes(_c_int(R), _c_int(V)))
    scratch = torch.empty(need // 4, dtype=torch.float32, device=logits.device) if need else None
    _check(lib.exl3_argmax(_ptr(logits), _ptr(out), _c_int(R), _c_int(V), _ptr(scratch), _c_size_t(need),
                           _stream()), "argmax")
    return out


def sample_filtered_cap() -> int:
    """The most candidates the device sampler ranks (``top_k`` above it is the host sampler's)."""
    return int(library().exl3_sample_filtered_cap())


def sample_filtered(logits: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The reference's sampler on the device.  ``rows``: float64 ``[R, 5]`` on the device: temperature (<= 0:
    greedy), top_k (0: off), top_p, min_p and the row's uniform number in [0, 1)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or rows.dtype != torch.float64 or tuple(rows.shape) != (R, 5):
        raise KernelLibraryError("sample_filtered: logits [R, V] must be float32 and rows [R, 5] float64")
    _contig(logits, "logits")
    _contig(rows, "rows")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _check(library().exl3_sample_filtered(_ptr(logits), _ptr(rows), _ptr(out), _c_int(R), _c_int(V), _stream()),
           "sample_filtered")
    return out


def sample_penalties(logits: torch.Tensor, counts: torch.Tensor, params: torch.Tensor) -> None:
    """Repetition, presence and frequency penalties, in place.  ``counts``: int64 ``[R]`` on the device, the
    addresses of the rows' int32 ``[V]`` token counts (0: the row has none); ``params``: float32 ``[R, 3]``."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or counts.dtype != torch.int64 or params.dtype != torch.float32 or \
            counts.numel() != R or tuple(params.shape) != (R, 3):
        raise KernelLibraryError("sample_penalties: logits float32 [R, V], counts int64 [R], params float32 [R, 3]")
    _contig(logits, "logits")
    _contig(params, "params")
    _check(library().exl3_sample_penalties(_ptr(logits), _c_int(R), _c_int(V), _ptr(counts), _ptr(params),
                                           _stream()), "sample_penalties")


def sample_count(counts: torch.Tensor, ids: torch.Tensor, vocab: int) -> None:
    """Adds each row's chosen token (``ids`` int32 ``[R]``) to its counts (``counts`` as in ``sample_penalties``)."""
    if counts.dtype != torch.int64 or ids.dtype != torch.int32 or counts.numel() != ids.numel():
        raise KernelLibraryError("sample_count: counts int64 [R] and ids int32 [R]")
    _check(library().exl3_sample_count(_ptr(counts), _ptr(ids), _c_int(ids.numel()), _c_int(vocab), _stream()),
           "sample_count")


# -- a norm without statistics, side-by-side sublayers, routed feed-forwards, heads of several maps -------------------

def tanh_norm_add(h: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], sa: Optional[torch.Tensor],
                  sb: Optional[torch.Tensor], m: float, norms, out_dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None):
    """The residual step of layers whose sublayers read the same residual, and up to two norms of the kind
    ``tanh(alpha x) w + b`` over the result (see tanh_norm.cu).  With ``a`` given: ``h += m * (sa * a + sb * b)`` in
    place (``b`` may be None).  ``norms``: up to two ``(w, b, alpha)`` triples of float32 tensors; returns the list
    of their outputs ``[T, H]`` in ``out_dtype``.  With ``rows`` (and no ``a``) only those rows are normed."""
    T, H = h.shape
    if h.dtype != torch.float32:
        raise KernelLibraryError("tanh_norm_add: the residual stream must be float32")
    _contig(h, "h")
    for t, name in ((a, "a"), (b, "b")):
        if t is not None:
            _contig(t, name)
            if t.shape != h.shape:
                raise KernelLibraryError(f"tanh_norm_add: {name} is {tuple(t.shape)}, h is {tuple(h.shape)}")
    if len(norms) > 2:
        raise KernelLibraryError("tanh_norm_add: at most two norms")
    for w, bias, alpha in norms:
        if any(x.dtype != torch.float32 for x in (w, bias, alpha)) or w.numel() != H or bias.numel() != H:
            raise KernelLibraryError("tanh_norm_add: a norm's weight, bias and alpha must be float32 of the row's width")
    for s_, name in ((sa, "sa"), (sb, "sb")):
        if s_ is not None and (s_.dtype != torch.float32 or s_.numel() != H):
            raise KernelLibraryError(f"tanh_norm_add: {name} must be float32 of the row's width")
    n = T if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelLibraryError("tanh_norm_add: rows must be int32")
    outs = [torch.empty((n, H), dtype=out_dtype, device=h.device) for _ in norms]
    args = []
    for i in range(2):
        if i < len(norms):
            w, bias, alpha = norms[i]
            args += [_ptr(w), _ptr(bias), _ptr(alpha), _ptr(outs[i])]
        else:
            args += [_c_void_p(0)] * 4
    _check(library().exl3_tanh_norm_add(
        _ptr(h), _ptr(a), _c_int(dtype_code(a.dtype) if a is not None else 0), _ptr(b),
        _c_int(dtype_code(b.dtype) if b is not None else 0), _ptr(sa), _ptr(sb), _c_float(m), _ptr(rows), _c_int(n),
        *args, _c_int(dtype_code(out_dtype)), _c_int(T), _c_int(H), _stream()), "tanh_norm_add")
    return outs


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x <- cap * tanh(x / cap)`` in place (float32)."""
    _contig(x, "x")
    if x.dtype != torch.float32:
        raise KernelLibraryError("softcap: float32 only")
    _check(library().exl3_softcap(_ptr(x), _c_int64(x.numel()), _c_float(cap), _stream()), "softcap")
    return x


MOE_ACTIVATIONS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3}
MOE_SCORES = {"softmax": 0, "sigmoid": 1}
MOE_GROUP_SCORES = {"max": 0, "top2": 2}     # added to the score's code


def moe_tile_rows(kind: str = "tile") -> int:
    """Rows of a plan's tiles for the CUDA-core product (``"tile"``), the few-row product (``"few"``) and the
    tensor-core product (``"tc"``)."""
    lib = library()
    return int({"tile": lib.exl3_moe_tile_rows, "few": lib.exl3_moe_gemv_rows, "tc": lib.exl3_moe_tc_rows}[kind]())


def moe_max_tiles(pairs: int, n_experts: int, tile_rows: int) -> int:
    return int(library().exl3_moe_max_tiles(_c_int(pairs), _c_int(n_experts), _c_int(tile_rows)))


def moe_tc_supported(dtype: torch.dtype, n: int, k: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().exl3_moe_tc_supported(_c_int(n), _c_int(k)))


def moe_tc_status() -> int:
    """0, or the code the tensor-core experts' product left when a bounded wait ran out (cleared by this call)."""
    return int(library().exl3_moe_tc_status())


def moe_route(x: torch.Tensor, wr: torch.Tensor, corr: torch.Tensor, outputs: int, extra: int, groups: int, keep: int,
              top: int, scale: float, score: str = "softmax", group_score: str = "max"):
    """The router of a routed feed-forward (see moe.cu): ``wr`` float32 ``[outputs + extra, W]``, ``corr`` float32
    ``[outputs]`` added to the scores for the choice only.  Returns ``(idx int32 [T, top], weight float32 [T, top],
    gate float32 [T] or None)``: the gate is the sigmoid of the extra row's product.  ``group_score``: a group's
    score is its largest choice score (``max``) or the sum of its two largest (``top2``)."""
    T, W = x.shape
    if x.stride(1) != 1:
        raise KernelLibraryError("moe_route: rows of x must be dense")
    _contig(wr, "wr")
    if wr.dtype != torch.float32 or corr.dtype != torch.float32 or tuple(wr.shape) != (outputs + extra, W) or \
            corr.numel() != outputs:
        raise KernelLibraryError("moe_route: the router's matrix and correction must be float32 [outputs (+ 1), W] and [outputs]")
    idx = torch.empty((T, top), dtype=torch.int32, device=x.device)
    wt = torch.empty((T, top), dtype=torch.float32, device=x.device)
    gate = torch.empty((T,), dtype=torch.float32, device=x.device) if extra else None
    _check(library().exl3_moe_route(
        _ptr(x), _c_int(dtype_code(x.dtype)), _c_int64(x.stride(0)), _ptr(wr), _ptr(corr), _c_int(T), _c_int(W),
        _c_int(outputs), _c_int(extra), _c_int(groups), _c_int(keep), _c_int(top), _c_float(scale),
        _c_int(MOE_SCORES[score] + MOE_GROUP_SCORES[group_score]), _ptr(idx), _ptr(wt), _ptr(gate), _stream()),
        "moe_route")
    return idx, wt, gate


def moe_plan(idx: torch.Tensor, n_experts: int, tile_rows: int = 0):
    """Orders a step's (token, pick) pairs by expert and cuts them into tiles of at most ``tile_rows`` rows (0: the
    CUDA-core product's), on the device.  Returns ``(order int32 [pairs], plan int32)`` for the experts' products;
    picks outside ``0 .. n_experts - 1`` (identity outputs) are left out."""
    _contig(idx, "idx")
    P = idx.numel()
    tile_rows = tile_rows or moe_tile_rows()
    order = torch.empty((P,), dtype=torch.int32, device=idx.device)
    plan = torch.empty((4 + 3 * max(1, moe_max_tiles(P, n_experts, tile_rows)),), dtype=torch.int32, device=idx.device)
    _check(library().exl3_moe_plan(_ptr(idx), _c_int(P), _c_int(n_experts), _c_int(tile_rows), _ptr(order), _ptr(plan),
                                   _stream()), "moe_plan")
    return order, plan


def moe_gemv(a: torch.Tensor, a_div: int, w: torch.Tensor, order: torch.Tensor, plan: torch.Tensor,
             out_dtype: torch.dtype, act: str = "none") -> torch.Tensor:
    """``moe_gemm`` for a plan of tiles of at most ``moe_tile_rows("few")`` rows (decode): bfloat16 ``a`` and ``w``, inputs
    a multiple of 8 wide; every expert's matrix is read once, a warp per output feature."""
    E, N, Kd = w.shape
    _contig(w, "w")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or a.shape[1] != Kd:
        raise KernelLibraryError("moe_gemv: a and w must be bfloat16, rows of a dense and as wide as the experts' inputs")
    P = order.numel()
    out = torch.empty((P, N), dtype=out_dtype, device=a.device)
    _check(library().exl3_moe_gemv(
        _ptr(a), _c_int64(a.stride(0)), _c_int(a_div), _ptr(w), _ptr(order), _ptr(plan), _ptr(out),
        _c_int(dtype_code(out_dtype)), _c_int(P), _c_int(E), _c_int(N), _c_int(Kd), _c_int(MOE_ACTIVATIONS[act]),
        _stream()), "moe_gemv")
    return out


def moe_gather(x: torch.Tensor, top: int, order: torch.Tensor, plan: torch.Tensor) -> torch.Tensor:
    """Rows of ``x [T, K]`` (bfloat16) in the plan's order: row i is ``x[order[i] // top]`` for the planned pairs (the
    rest of the ``[pairs, K]`` result is not written)."""
    if x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise KernelLibraryError("moe_gather: x must be bfloat16 with dense rows")
    P = order.numel()
    xs = torch.empty((P, x.shape[1]), dtype=x.dtype, device=x.device)
    _check(library().exl3_moe_gather(_ptr(x), _c_int64(x.stride(0)), _c_int(top), _ptr(order), _ptr(plan), _ptr(xs),
                                     _c_int(P), _c_int(x.shape[1]), _stream()), "moe_gather")
    return xs


def moe_gemm_tc(a: torch.Tensor, w: torch.Tensor, order: torch.Tensor, plan: torch.Tensor, out_dtype: torch.dtype,
                act: str = "none") -> torch.Tensor:
    """The experts' product on tcgen05 tensor cores (see moe_tc.cu) for a plan of tiles of at most
    ``moe_tile_rows("tc")`` rows: ``a [pairs, K]`` bfloat16 in the plan's order, ``w [experts, N, K]`` bfloat16.  A bfloat16
    result is in the plan's order too; a float32 one has every pair at its own place (``order[i]``)."""
    E, N, Kd = w.shape
    _contig(w, "w")
    _contig(a, "a")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[1] != Kd:
        raise KernelLibraryError("moe_gemm_tc: a and w must be bfloat16 and a as wide as the experts' inputs")
    P = order.numel()
    if a.shape[0] != P:
        raise KernelLibraryError("moe_gemm_tc: a must have a row per pair")
    out = torch.empty((P, N), dtype=out_dtype, device=a.device)
    _check(library().exl3_moe_gemm_tc(
        _ptr(a), _ptr(w), _ptr(order), _ptr(plan), _ptr(out), _c_int(dtype_code(out_dtype)), _c_int(P), _c_int(E),
        _c_int(N), _c_int(Kd), _c_int(MOE_ACTIVATIONS[act]), _stream()), "moe_gemm_tc")
    return out


def moe_gemm(a: torch.Tensor, a_div: int, w: torch.Tensor, order: torch.Tensor, plan: torch.Tensor,
             out_dtype: torch.dtype, act: str = "none") -> torch.Tensor:
    """``out[p] = act(w[expert(p)] a[p // a_div])`` for the planned pairs: ``w [experts, N, K]``; ``a [rows, K]`` has
    one row per pair (``a_div`` 1) or per token (``a_div`` = picks per token).  Rows of pairs that are not planned
    are left unwritten."""
    E, N, Kd = w.shape
    _contig(w, "w")
    if a.stride(1) != 1 or a.shape[1] != Kd:
        raise KernelLibraryError("moe_gemm: rows of a must be dense and as wide as the experts' inputs")
    P = order.numel()
    out = torch.empty((P, N), dtype=out_dtype, device=a.device)
    _check(library().exl3_moe_gemm(
        _ptr(a), _c_int(dtype_code(a.dtype)), _c_int64(a.stride(0)), _c_int(a_div), _ptr(w), _c_int(dtype_code(w.dtype)),
        _ptr(order), _ptr(plan), _ptr(out), _c_int(dtype_code(out_dtype)), _c_int(P), _c_int(E), _c_int(N), _c_int(Kd),
        _c_int(MOE_ACTIVATIONS[act]), _stream()), "moe_gemm")
    return out


def moe_combine(y: Optional[torch.Tensor], idx: torch.Tensor, wt: torch.Tensor, x: torch.Tensor,
                shared: Optional[torch.Tensor], gate: Optional[torch.Tensor], n_experts: int) -> torch.Tensor:
    """``out[t] = sum_k wt[t, k] * (y[t, k] or, for picks from ``n_experts`` on, x[t]) + gate[t] * shared[t]``,
    float32 ``[T, H]``; ``y`` float32 ``[T * top, H]``."""
    T, top = idx.shape
    H = x.shape[1]
    if x.stride(1) != 1:
        raise KernelLibraryError("moe_combine: rows of x must be dense")
    if y is not None and (y.dtype != torch.float32 or not y.is_contiguous()):
        raise KernelLibraryError("moe_combine: the experts' outputs must be contiguous float32")
    if shared is not None:
        _contig(shared, "shared")
    out = torch.empty((T, H), dtype=torch.float32, device=x.device)
    _check(library().exl3_moe_combine(
        _ptr(y), _ptr(idx), _ptr(wt), _ptr(x), _c_int(dtype_code(x.dtype)), _c_int64(x.stride(0)), _ptr(shared),
        _c_int(dtype_code(shared.dtype) if shared is not None else 0), _ptr(gate), _ptr(out), _c_int(T), _c_int(H),
        _c_int(top), _c_int(n_experts), _stream()), "moe_combine")
    return out


def maps_prep(x: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, maps: int, d: int,
              dv: int, rot: int, inv_freq: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_seq: torch.Tensor,
              block_table: torch.Tensor, page: int, q_dtype: torch.dtype, k_pool: torch.Tensor,
              v_pool: torch.Tensor) -> torch.Tensor:
    """What stands between the joint projection ``x [T, ld]`` of an attention whose heads hold ``maps`` maps and
    the attention kernels (see diff_attn.cu): half-split rotation of the first ``rot`` features of every map, the
    cache write (a key row holds the kv head's maps side by side, the pools' last dimensions are the row pitches)
    and the queries widened to one head per map: returns ``[T, heads * maps, key row]``."""
    T = x.shape[0]
    if x.stride(1) != 1:
        raise KernelLibraryError("maps_prep: rows of x must be dense")
    row, v_row = k_pool.shape[-1], v_pool.shape[-1]
    hi, lo = (_rotary_rows(inv_freq, rot, "maps_prep") if rot else (_c_void_p(0), _c_void_p(0)))
    q = torch.empty((T, heads * maps * row), dtype=q_dtype, device=x.device)
    _check(library().exl3_maps_prep(
        _ptr(x), _c_int(dtype_code(x.dtype)), _c_int64(x.stride(0)), _c_int(q_off), _c_int(k_off), _c_int(v_off),
        _c_int(T), _c_int(heads), _c_int(kv_heads), _c_int(maps), _c_int(d), _c_int(dv), _c_int(row), _c_int(v_row),
        _c_int(rot), hi, lo, _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), _c_int(block_table.stride(0)),
        _c_int(page), _ptr(q), _c_int(dtype_code(q_dtype)), _ptr(k_pool), _ptr(v_pool),
        _c_int(dtype_code(k_pool.dtype)), _stream()), "maps_prep")
    return q


def diff_combine(a: torch.Tensor, a_row: int, gate: Optional[torch.Tensor], lam: float, eps: float, mult: float,
                 heads: int, dv: int, out_row: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``o = a_0 - lam * a_1`` of every head's two maps (``a [T, heads * 2 * a_row]``), divided by its root mean
    square over the head's ``dv`` values, times ``mult`` and ``sigmoid(gate[t, head])``; rows of ``out_row``
    elements (zeros beyond ``dv``)."""
    T = a.shape[0]
    _contig(a, "a")
    if gate is not None and gate.stride(1) != 1:
        raise KernelLibraryError("diff_combine: rows of the gate must be dense")
    out = torch.empty((T, heads * out_row), dtype=out_dtype, device=a.device)
    _check(library().exl3_diff_combine(
        _ptr(a), _c_int(dtype_code(a.dtype)), _c_int(a_row), _ptr(gate),
        _c_int(dtype_code(gate.dtype) if gate is not None else 0), _c_int64(gate.stride(0) if gate is not None else 0),
        _c_float(lam), _c_float(eps), _c_float(mult), _ptr(out), _c_int(dtype_code(out_dtype)), _c_int(out_row),
        _c_int(T), _c_int(heads), _c_int(dv), _stream()), "diff_combine")
    return out


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``g * sigmoid(alpha g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` for rows
    ``[gate (I) | up (I)]`` of ``gu`` (float32 inside)."""
    T, two = gu.shape
    if gu.stride(1) != 1 or two % 2:
        raise KernelLibraryError("clamped_glu: rows of gu must be dense and hold a gate half and an up half")
    out = torch.empty((T, two // 2), dtype=out_dtype, device=gu.device)
    _check(library().exl3_clamped_glu(_ptr(gu), _c_int(dtype_code(gu.dtype)), _c_int64(gu.stride(0)), _ptr(out),
                                      _c_int(dtype_code(out_dtype)), _c_int(T), _c_int(two // 2), _c_float(limit),
                                      _c_float(alpha), _stream()), "clamped_glu")
    return out


def hyper_max_streams() -> int:
    return int(library().exl3_hyper_max_streams())


def hyper_step(x: torch.Tensor, streams: int, y: Optional[torch.Tensor], mix: Optional[torch.Tensor],
               w_out: Optional[torch.Tensor], w_in: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float,
               out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """One step of a residual of several streams (see hyper.cu).  ``x`` float32 ``[T, streams * W]``; or, with ``out``
    float32 ``[T, streams * W]`` given, ``[T, W]`` standing for ``streams`` equal ones (``out`` then gets the streams).  With ``y [T, W]``: every stream
    becomes ``sum_s mix[s, to] x_s + w_out[to] y`` in place.  With ``w_in``: returns ``rmsnorm(sum_s w_in[s] x_s) *
    norm_w`` in ``out_dtype``, of all tokens or of ``rows`` (only without ``y``).  Returns ``(streams tensor, r or
    None)``."""
    T = x.shape[0]
    if x.dtype != torch.float32:
        raise KernelLibraryError("hyper_step: the streams must be float32")
    _contig(x, "x")
    # with ``out`` given, x is one row per token that stands for ``streams`` equal ones and ``out`` gets the streams
    s_in = 1 if out is not None else streams
    W = x.shape[1] // s_in
    if x.shape[1] != s_in * W or (out is not None and (tuple(out.shape) != (T, streams * W) or out.dtype != torch.float32
                                                       or not out.is_contiguous())):
        raise KernelLibraryError(f"hyper_step: x {tuple(x.shape)} does not hold {streams} streams")
    xout = out if out is not None else x
    for t, n in ((mix, streams * streams), (w_out, streams), (w_in, streams)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelLibraryError("hyper_step: mix, w_out and w_in must be contiguous float32 of [S, S], [S], [S]")
    if y is not None:
        _contig(y, "y")
        if tuple(y.shape) != (T, W) or mix is None or w_out is None:
            raise KernelLibraryError("hyper_step: y must be [T, W] and come with mix and w_out")
    if norm_w is not None and norm_w.numel() != W:
        raise KernelLibraryError("hyper_step: the norm's weight must be [W]")
    n = T if rows is None else rows.numel()
    r = torch.empty((n, W), dtype=out_dtype, device=x.device) if w_in is not None else None
    _check(library().exl3_hyper_step(
        _ptr(x), _c_int(s_in), _ptr(xout), _c_int(streams), _ptr(y), _c_int(dtype_code(y.dtype) if y is not None else 0),
        _ptr(mix), _ptr(w_out), _ptr(w_in), _ptr(norm_w), _c_int(dtype_code(norm_w.dtype) if norm_w is not None else 0),
        _c_float(eps), _ptr(r), _c_int(dtype_code(out_dtype)), _ptr(rows), _c_int(n), _c_int(T), _c_int(W), _stream()),
        "hyper_step")
    return xout, r


def mlstm_scan_scratch_bytes(rows: int, T: int, heads: int, dk: int, dv: int, max_new: int) -> int:
    """Bytes of float32 scratch that ``mlstm_scan`` needs for a step (0 for steps of short rows, which run in order)."""
    lib = library()
    lib.exl3_mlstm_scan_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_mlstm_scan_scratch_bytes(_c_int(rows), _c_int(T), _c_int(heads), _c_int(dk), _c_int(dv),
                                                 _c_int(max_new)))


def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, zi: torch.Tensor, zf: torch.Tensor, cap: float,
               q_scale: float, s_state: torch.Tensor, n_state: torch.Tensor, m_state: torch.Tensor,
               slot_ids: torch.Tensor, row_start: torch.Tensor, rows: int, heads: int, dk: int, dv: int,
               max_new: int, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The matrix memory with exponential gates over a step's packed tokens (see matrix_memory.cu).  ``q``, ``k``
    ``[T, heads * dk]``, ``v [T, heads * dv]`` and the gates' pre-activations ``zi``, ``zf [T, heads]`` may be views
    with their own row pitch; states float32 ``[slots, heads, dv, dk]`` (the matrix column by column), ``[slots, heads, dk]``, ``[slots, heads]``
    are read and written at ``slot_ids``; ``max_new`` is the most tokens a row brings; ``scratch``: float32 memory of
    ``mlstm_scan_scratch_bytes`` bytes when that is not 0 (rows of many tokens run as pieces side by side).  Returns float32
    ``[T, heads * dv]``."""
    T = q.shape[0]
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (zi, "zi"), (zf, "zf")):
        if t.stride(1) != 1:
            raise KernelLibraryError(f"mlstm_scan: rows of {name} must be dense")
    if q.dtype != k.dtype or q.dtype != v.dtype or zi.dtype != zf.dtype or zi.stride(0) != zf.stride(0):
        raise KernelLibraryError("mlstm_scan: q, k, v (and zi, zf) must agree in element type and pitch")
    for t, shape in ((s_state, (heads, dv, dk)), (n_state, (heads, dk)), (m_state, (heads,))):
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != shape or not t.is_contiguous():
            raise KernelLibraryError(f"mlstm_scan: a state of shape {tuple(t.shape)} must be contiguous float32 [slots, {shape}]")
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    _check(library().exl3_mlstm_scan(
        _ptr(q), _c_int64(q.stride(0)), _ptr(k), _c_int64(k.stride(0)), _ptr(v), _c_int64(v.stride(0)),
        _c_int(dtype_code(q.dtype)), _ptr(zi), _ptr(zf), _c_int(dtype_code(zi.dtype)), _c_int64(zi.stride(0)),
        _c_float(cap), _c_float(q_scale), _ptr(s_state), _ptr(n_state), _ptr(m_state), _ptr(slot_ids), _ptr(row_start),
        _ptr(out), _c_int(rows), _c_int(T), _c_int(heads), _c_int(dk), _c_int(dv), _c_int(max_new), _ptr(scratch),
        _c_size_t(0 if scratch is None else scratch.numel() * scratch.element_size()), _stream()), "mlstm_scan")
    return out


def delta_scan_scratch_bytes(rows: int, T: int, heads: int, dk: int, dv: int, max_new: int) -> int:
    """Bytes of float32 scratch that ``delta_scan`` needs for a step (0 for steps of short rows, which run in order)."""
    lib = library()
    lib.exl3_delta_scan_scratch_bytes.restype = _c_size_t
    return int(lib.exl3_delta_scan_scratch_bytes(_c_int(rows), _c_int(T), _c_int(heads), _c_int(dk), _c_int(dv),
                                                 _c_int(max_new)))


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, zb: torch.Tensor, za: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, s_state: torch.Tensor, slot_ids: torch.Tensor,
               row_start: torch.Tensor, rows: int, heads: int, qk_heads: int, dk: int, dv: int, max_new: int,
               scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The gated delta rule over a step's packed tokens (see matrix_memory.cu): ``q``, ``k [T, qk_heads * dk]``,
    ``v [T, heads * dv]`` (one element type), ``zb [T, heads]`` (beta before its sigmoid), ``za [T, heads * dk]``
    (the decay's pre-activation, before ``dt_bias``), ``a_log [heads]``, ``dt_bias [heads * dk]`` float32; state
    float32 ``[slots, heads, dv, dk]`` (the matrix column by column); ``max_new`` is the most tokens a row brings; ``scratch``: float32 memory of
    ``delta_scan_scratch_bytes`` bytes when that is not 0.  Returns float32 ``[T, heads * dv]``."""
    T = q.shape[0]
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (zb, "zb"), (za, "za")):
        if t.stride(1) != 1:
            raise KernelLibraryError(f"delta_scan: rows of {name} must be dense")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise KernelLibraryError("delta_scan: q, k and v must agree in element type")
    if a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or a_log.numel() != heads or \
            dt_bias.numel() != heads * dk:
        raise KernelLibraryError("delta_scan: a_log and dt_bias must be float32 [heads] and [heads * dk]")
    if s_state.dtype != torch.float32 or tuple(s_state.shape[1:]) != (heads, dv, dk) or not s_state.is_contiguous():
        raise KernelLibraryError(f"delta_scan: state {tuple(s_state.shape)} must be float32 [slots, {heads}, {dv}, {dk}]")
    out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
    _check(library().exl3_delta_scan(
        _ptr(q), _c_int64(q.stride(0)), _ptr(k), _c_int64(k.stride(0)), _ptr(v), _c_int64(v.stride(0)),
        _c_int(dtype_code(q.dtype)), _ptr(zb), _c_int(dtype_code(zb.dtype)), _c_int64(zb.stride(0)), _ptr(za),
        _c_int(dtype_code(za.dtype)), _c_int64(za.stride(0)), _ptr(a_log), _ptr(dt_bias), _ptr(s_state), _ptr(slot_ids),
        _ptr(row_start), _ptr(out), _c_int(rows), _c_int(T), _c_int(heads), _c_int(qk_heads), _c_int(dk), _c_int(dv),
        _c_int(max_new), _ptr(scratch), _c_size_t(0 if scratch is None else scratch.numel() * scratch.element_size()),
        _stream()), "delta_scan")
    return out


def conv_prep_max_taps() -> int:
    return int(library().exl3_conv_prep_max_taps())


def conv_prep(x: torch.Tensor, q_off: int, k_off: int, v_off: int, q_taps: torch.Tensor, k_taps: torch.Tensor,
              v_taps: torch.Tensor, qk_heads: int, dk: int, v_heads: int, dv: int, eps: float, q_scale: float,
              state: torch.Tensor, slot_ids: torch.Tensor, row_start: torch.Tensor, rows: int,
              max_new: int) -> torch.Tensor:
    """Short causal convolutions per channel over a step's packed tokens, SiLU, and unit query and key heads (see
    matrix_memory.cu).  ``x [T, *]`` holds the q, k and v channels from the given columns on; taps float32
    ``[channels, taps]`` (the last tap is the current token's); ``state`` float32 ``[slots, channels, taps - 1]`` holds
    every channel's last inputs and is kept up.  Returns float32 ``[T, 2 qk_heads dk + v_heads dv]``: q | k | v."""
    T = x.shape[0]
    if x.stride(1) != 1:
        raise KernelLibraryError("conv_prep: rows of x must be dense")
    n_taps = q_taps.shape[1]
    C = 2 * qk_heads * dk + v_heads * dv
    for t, n in ((q_taps, qk_heads * dk), (k_taps, qk_heads * dk), (v_taps, v_heads * dv)):
        if t.dtype != torch.float32 or tuple(t.shape) != (n, n_taps) or not t.is_contiguous():
            raise KernelLibraryError("conv_prep: taps must be contiguous float32 [channels, taps]")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (C, n_taps - 1) or not state.is_contiguous():
        raise KernelLibraryError(f"conv_prep: state {tuple(state.shape)} must be float32 [slots, {C}, {n_taps - 1}]")
    out = torch.empty((T, C), dtype=torch.float32, device=x.device)
    _check(library().exl3_conv_prep(
        _ptr(x), _c_int(dtype_code(x.dtype)), _c_int64(x.stride(0)), _c_int(q_off), _c_int(k_off), _c_int(v_off),
        _ptr(q_taps), _ptr(k_taps), _ptr(v_taps), _c_int(qk_heads), _c_int(dk), _c_int(v_heads), _c_int(dv),
        _c_int(n_taps), _c_float(eps), _c_float(q_scale), _ptr(state), _ptr(slot_ids), _ptr(row_start), _ptr(out),
        _c_int(rows), _c_int(T), _c_int(max_new), _stream()), "conv_prep")
    return out


def scaled_sum2(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float) -> torch.Tensor:
    """``sa * a + sb * b`` element by element, float32."""
    _contig(a, "a")
    _contig(b, "b")
    if a.dtype != b.dtype or a.shape != b.shape:
        raise KernelLibraryError("scaled_sum2: a and b must agree in shape and type")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    _check(library().exl3_scaled_sum2(_ptr(a), _ptr(b), _c_int(dtype_code(a.dtype)), _c_float(sa), _c_float(sb), _ptr(out),
                                      _c_int64(a.numel()), _stream()), "scaled_sum2")
    return out


def gemm_few_out(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``x @ w.T (+ bias)`` as float32 for a handful of output features and many rows (a warp a row; see gemm_simt.cu)."""
    M, Kd = x.shape
    N = w.shape[0]
    if x.stride(1) != 1 or w.shape[1] != Kd or x.dtype != w.dtype or (bias is not None and bias.dtype != w.dtype):
        raise KernelLibraryError("gemm_few_out: x, w and bias must share an element type and fit")
    _contig(w, "w")
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _check(library().exl3_gemm_few_out(_ptr(x), _c_int64(x.stride(0)), _ptr(w), _ptr(bias), _ptr(out),
                                       _c_int(dtype_code(x.dtype)), _c_int(M), _c_int(N), _c_int(Kd), _stream()),
           "gemm_few_out")
    return out
