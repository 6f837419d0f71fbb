"""Tensor-level wrappers of the kernel entry points.

Each function checks what the kernel cannot (device, dtype, contiguity,
shapes) and launches on the current CUDA stream. Matrix products of the
bfloat16 path go to the library (`torch.mm`, i.e. cuBLAS) here unless a
hand-written kernel takes the shape; everything else is this package's own
CUDA.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.pages import PAGE_TOKENS
from . import lib
from .lib import KernelError, call, code, ptr, stream_ptr

MAX_HEAD_DIM = 256

ST_PAGE_RANGE, ST_POS_RANGE, ST_TOKEN_RANGE, ST_SPLIT_RANGE = 1, 2, 4, 8


def _chk(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {dim}")


@dataclass
class PageTableView:
    """A cache group's page lists for the sequences of one step (device)."""
    indptr: torch.Tensor      # int32 [B+1]
    ids: torch.Tensor         # int32 [>= indptr[B]]
    base: torch.Tensor        # int32 [B]
    n_pages: int


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None,
                 scale: float = 1.0) -> torch.Tensor:
    """x[t] = table[token_t] * scale, fp32 [T, D]."""
    _chk(table, "embedding table", dim=2)
    _chk(tokens, "tokens", torch.int32, 1)
    T, (V, D) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    call("mynah_embed_gather", ptr(table), code(table.dtype), ptr(tokens), ptr(out), T, D, V, float(scale), stream_ptr())
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, act_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, delta_scale: float = 1.0) -> torch.Tensor:
    """h = RMSNorm(x (+ delta_scale * delta)) * gain. Without `rows`, x is updated in place when delta is given; with `rows`
    (which may name a row more than once) x is only read."""
    _chk(x, "residual", torch.float32, 2)
    _chk(gain, "norm gain", dim=1)
    T, D = x.shape
    if gain.numel() != D:
        raise KernelError(f"norm gain has {gain.numel()} elements, the rows have {D}")
    if delta is not None:
        _chk(delta, "delta", act_dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(x.shape)}")
    n = T
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
        n = rows.numel()
    if out is None:
        out = torch.empty((n, D), dtype=act_dtype, device=x.device)
    call("mynah_rmsnorm", ptr(x), ptr(delta), ptr(gain), code(gain.dtype), ptr(rows), ptr(out), code(act_dtype),
         n, D, float(eps), float(delta_scale), stream_ptr())
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor, scale: float = 1.0) -> None:
    _chk(x, "residual", torch.float32)
    _chk(delta, "delta")
    if delta.shape != x.shape:
        raise KernelError("residual_add: shapes differ")
    call("mynah_residual_add", ptr(x), ptr(delta), code(delta.dtype), x.numel(), float(scale), stream_ptr())


def residual_add_row(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[t] += v for every row of the fp32 stream (one learned vector for the whole step)."""
    _chk(x, "residual", torch.float32, 2)
    _chk(v, "row", torch.float32, 1)
    if v.numel() != x.shape[1]:
        raise KernelError("residual_add_row: the row does not have the stream's width")
    call("mynah_residual_add_row", ptr(x), ptr(v), x.shape[0], x.shape[1], stream_ptr())


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(gate_up, "gate_up", dim=2)
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("swiglu: the input must hold gate and up side by side")
    if out is None:
        out = torch.empty((T, F2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("mynah_swiglu", ptr(gate_up), ptr(out), code(gate_up.dtype), T, F2 // 2, stream_ptr())
    return out


class NormedInput:
    """A norm that has not been run yet: the residual rows, the pending add and
    the gain. A matrix product that can compute the norm on its way takes it as
    it is (`linear`, `linear_swiglu`); anything else calls `materialize`."""

    def __init__(self, stream, delta, gain: torch.Tensor, eps: float, act_dtype: torch.dtype, delta_scale: float = 1.0):
        self.stream, self.delta, self.gain, self.eps, self.act_dtype = stream, delta, gain, float(eps), act_dtype
        self.delta_scale = float(delta_scale)
        self.shape = stream.x.shape
        self.dtype = act_dtype
        self._h: Optional[torch.Tensor] = None

    def materialize(self) -> torch.Tensor:
        if self._h is None:
            self._h = rmsnorm(self.stream.x, self.gain, self.eps, self.act_dtype, delta=self.delta,
                              delta_scale=self.delta_scale)
            self.delta = None
        return self._h


_SM_COUNT: dict = {}


def _sm_count(device) -> int:
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[device]


def gemv_decode_mode(mode: int) -> int:
    """How the decode products read their weights: 0 straight into registers, 1 through a ring of asynchronous copies
    in shared memory, 2 (the default) whichever the shape does better with. Returns the mode set before; a row's
    sums are the same bits either way."""
    return int(lib.load().mynah_gemv_decode_mode(int(mode)))


def gemv_decode_supported(M: int, N: int, K: int) -> bool:
    return bool(lib.load().mynah_gemv_decode_supported(M, N, K))


def _gemv_decode(x, w: torch.Tensor, N: int, epilogue: int, out: torch.Tensor) -> torch.Tensor:
    """x: bf16 rows [M, K] or a NormedInput. epilogue 0: bf16, 1: SwiGLU (w holds N gate rows then N up rows), 2: fp32."""
    K = w.shape[1]
    if isinstance(x, NormedInput) and x._h is None and (x.shape[0] > FUSED_NORM_MAX_ROWS or not _norm_prologue_fits(x.shape[0], K)
                                                        or (x.delta is not None and x.delta_scale != 1.0)):
        x.materialize()
    if isinstance(x, NormedInput) and x._h is None:
        st = x.stream
        M = st.x.shape[0]
        new_x = torch.empty_like(st.x) if x.delta is not None else None
        call("mynah_gemv_decode", ptr(w), N, K, M, None, ptr(st.x), ptr(x.delta), ptr(new_x),
             ptr(x.gain), code(x.gain.dtype), x.eps, ptr(out), out.shape[1], epilogue, _sm_count(w.device), stream_ptr())
        if new_x is not None:
            st.x = new_x                       # the residual with the add done, written by the kernel
            x.delta = None
        return out
    if isinstance(x, NormedInput):
        x = x._h
    call("mynah_gemv_decode", ptr(w), N, K, x.shape[0], ptr(x), None, None, None, None, 0, 0.0,
         ptr(out), out.shape[1], epilogue, _sm_count(w.device), stream_ptr())
    return out


# Many outputs of long rows (the q/k/v and gate/up products of the 4B and 8B shapes): the library's kernels stream such
# matrices at 5.4 to 5.6 TB/s where gemv_decode reaches 2.8 to 4.4 (`python bench.py --only products --shape 8b`), so
# they are left to it, as the reference leaves its products to a library. 0 rows: never.
GEMV_LIBRARY_FROM_ROWS = int(os.environ.get("MYNAH_GEMV_LIBRARY_FROM_ROWS", "6144"))
GEMV_LIBRARY_FROM_K = 2048
# From nine rows on (the second half of the tensor cores' sixteen rows is then in use) the library also does better
# on every large matrix of long rows: 8B down 4,096 x 12,288 at 16 rows takes 21.8 us there against 32.2, 8B o 9.8
# against 13.6, 4B down 15.3 against 17.3; at 8 rows the own kernels are level or ahead. 0 elements: never.
GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS = int(os.environ.get("MYNAH_GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS", str(1 << 23)))


def _fusable(x, w: torch.Tensor, N: int) -> bool:
    if w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if GEMV_LIBRARY_FROM_ROWS and w.shape[0] >= GEMV_LIBRARY_FROM_ROWS and w.shape[1] >= GEMV_LIBRARY_FROM_K:
        return False
    if isinstance(x, NormedInput):
        if x.act_dtype != torch.bfloat16:
            return False
        M, K = x.shape
        if x._h is None and (x.gain.numel() != K or not x.stream.x.is_contiguous()):
            return False
    else:
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            return False
        M, K = x.shape
    if (GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS and M > 8 and K >= GEMV_LIBRARY_FROM_K
            and w.shape[0] * w.shape[1] >= GEMV_LIBRARY_FROM_ELEMENTS_9_ROWS):
        return False
    return K == w.shape[1] and N <= GEMV_MAX_OUT_ROWS and gemv_decode_supported(M, N, K)


# Rows up to which the norm runs as the product's prologue. 0: never. Since the products spread over up to four
# CTAs an SM, every CTA recomputing the norm costs as much as the separate norm kernel at one row (0.985 vs
# 0.980 ms a step at batch 1) and more from two rows on (1.155 vs 1.045 ms at batch 2), so it is off; the
# prologue stays in the kernel and in the tests.
FUSED_NORM_MAX_ROWS = int(os.environ.get("MYNAH_FUSED_NORM_MAX_ROWS", "0"))
def _norm_prologue_fits(M: int, K: int) -> bool:
    """The norm prologue keeps its rows (8 or 16 of them, padded) in shared memory beside the 80 KB ring of weights."""
    return (16 if M > 8 else 8) * (K + 32) * 2 + 80 * 1024 <= 200 * 1024
GEMV_MAX_OUT_ROWS = 32768   # wider products (the output head) stream better through the library for now


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x . w^T with w [out, in] row-major (no bias). float32 runs the
    package's FFMA kernel (true 32-bit); bfloat16 accumulates in fp32. `x` may
    be a NormedInput: a few bf16 rows then take the fused norm+product kernel."""
    _chk(w, "linear weight", dim=2)
    out_dtype = out_dtype or (x.dtype if not isinstance(x, NormedInput) else x.act_dtype)
    N = w.shape[0]
    if out_dtype in (torch.bfloat16, torch.float32) and _fusable(x, w, N):
        if out is None:
            out = torch.empty((x.shape[0], N), dtype=out_dtype, device=w.device)
        from . import gemm_bf16
        gemm_bf16.counters["own"] += 1
        return _gemv_decode(x, w, N, 0 if out_dtype == torch.bfloat16 else 2, out)
    if isinstance(x, NormedInput):
        x = x.materialize()
    if x.dim() != 2 or not x.is_cuda or x.stride(1) != 1:
        raise KernelError("linear input must be rows on the device (a column slice of a row-major tensor is fine)")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or x.dtype != w.dtype:
        raise KernelError(f"linear: input [{M},{K}] {x.dtype} does not fit weight [{N},{K2}] {w.dtype}")
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the 32-bit path writes float32")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        call("mynah_gemm_f32", ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0) if M > 1 else K, K, N, stream_ptr())
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")
    from . import gemm_bf16
    return gemm_bf16.linear_bf16(x, w, out_dtype, out)


def linear_swiglu(x, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) with w_gate_up = [Wg; Wu] ([2F, K]); one kernel for a few bf16 rows."""
    F = w_gate_up.shape[0] // 2
    if _fusable(x, w_gate_up, F):
        out = torch.empty((x.shape[0], F), dtype=torch.bfloat16, device=w_gate_up.device)
        from . import gemm_bf16
        gemm_bf16.counters["own"] += 1
        return _gemv_decode(x, w_gate_up, F, 1, out)
    from . import gemm_bf16
    if isinstance(x, NormedInput):
        x = x.materialize()
    if (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and gemm_bf16.USE_TCGEN05 and gemm_bf16.USE_TCGEN05_SWIGLU
            and x.shape[0] >= gemm_bf16.TCGEN05_MIN_ROWS and F % 8 == 0 and x.is_contiguous()
            and w_gate_up.is_contiguous() and gemm_bf16.tcgen05_supported(x.shape[0], F, x.shape[1])):
        out = torch.empty((x.shape[0], F), dtype=torch.bfloat16, device=x.device)
        gemm_bf16.counters["own"] += 1
        return gemm_bf16.gemm_tcgen05(x, w_gate_up, F, 2, out)      # the activation runs on the accumulator
    return swiglu(linear(x, w_gate_up))


def rope_table(n_pos: int, rotary_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    half = rotary_dim // 2
    cos = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    sin = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    # theta is a float in the reference's table builder (mynah-slm src/kernels.c:141)
    theta32 = float(torch.tensor(theta, dtype=torch.float32))
    call("mynah_rope_table", ptr(cos), ptr(sin), n_pos, rotary_dim, theta32, stream_ptr())
    return cos, sin


def qk_norm_rope_store(qkv: torch.Tensor, H: int, KV: int, HD: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                       tok_seq: torch.Tensor, tok_pos: torch.Tensor, pages: PageTableView,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       status: torch.Tensor) -> None:
    _chk(qkv, "qkv", dim=2)
    T, ld = qkv.shape
    if (q_gain is None) != (k_gain is None):
        raise KernelError("qk_norm_rope_store: q and k gains go together")
    gd = 0
    if q_gain is not None:
        if q_gain.dtype != k_gain.dtype or q_gain.numel() != HD or k_gain.numel() != HD:
            raise KernelError("qk_norm_rope_store: the head gains must both have head_dim elements of one dtype")
        gd = code(q_gain.dtype)
    n_pos = 0
    if cos is not None:
        _chk(cos, "cos table", torch.float32, 2)
        n_pos = cos.shape[0]
        if cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_store: the rotation table does not match rotary_dim")
    if k_cache is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_store: the cache and the activations differ in dtype")
        if tuple(k_cache.shape[1:]) != (KV, PAGE_TOKENS, HD):
            raise KernelError(f"qk_norm_rope_store: cache pages are {tuple(k_cache.shape[1:])}, expected {(KV, PAGE_TOKENS, HD)}")
    call("mynah_qk_norm_rope_store", ptr(qkv), code(qkv.dtype), T, H, KV, HD, ld,
         ptr(q_gain), ptr(k_gain), gd, float(eps),
         ptr(cos), ptr(sin), rotary_dim, n_pos,
         ptr(tok_seq), ptr(tok_pos),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         ptr(k_cache), ptr(v_cache), ptr(status), stream_ptr())


def attn_prefill_generic(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """q is read from the first H*HD columns of `qkv` (row stride qkv.shape[1])."""
    _chk(qkv, "q", dim=2)
    _chk(out, "attention output", qkv.dtype, 2)
    call("mynah_attn_prefill_generic", ptr(qkv), ptr(out), code(qkv.dtype), qkv.shape[0], B, max_q_len, H, KV, HD,
         qkv.shape[1], out.shape[1], ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tc_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_prefill_tc_supported(H, KV, HD))


def attn_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                    pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """The tensor-core prompt attention (bfloat16, head_dim 64 or 128); same contract as attn_prefill_generic."""
    _chk(qkv, "q", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    call("mynah_attn_prefill_tc", ptr(qkv), ptr(out), qkv.shape[0], B, max_q_len, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tcgen05_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_prefill_tcgen05_supported(H, KV, HD))


def attn_prefill_tcgen05(qkv: torch.Tensor, out: torch.Tensor, B: int, max_q_len: int, H: int, KV: int, HD: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         pages: PageTableView, window: int, status: torch.Tensor) -> None:
    """The prompt attention on tcgen05 (bfloat16, head_dim 64 or 128); same contract as attn_prefill_generic."""
    _chk(qkv, "q", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(k_cache, "K cache", torch.bfloat16)
    _chk(v_cache, "V cache", torch.bfloat16)
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("attn_prefill_tcgen05: the cache tensors must be contiguous")
    call("mynah_attn_prefill_tcgen05", ptr(qkv), ptr(out), qkv.shape[0], B, max_q_len, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(cu_q), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, ptr(status), stream_ptr())


def attn_prefill_tcgen05_stages(mode: int) -> None:
    """0: the prompt attention chooses its form by the number of CTAs; 1: one stage of K, V and scores, two CTAs an
    SM; 2: two stages, one CTA an SM. Both give the same bits."""
    call("mynah_attn_prefill_tcgen05_stages", int(mode))


def attn_decode_scratch_floats(B: int, H: int, HD: int, n_splits: int) -> int:
    return int(lib.load().mynah_attn_decode_scratch_floats(B, H, HD, n_splits))


def attn_decode(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor, pages: PageTableView,
                window: int, n_splits: int, scratch: torch.Tensor, status: torch.Tensor) -> None:
    _chk(qkv, "q", dim=2)
    _chk(out, "attention output", qkv.dtype, 2)
    _chk(scratch, "scratch", torch.float32)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode", ptr(qkv), ptr(out), code(qkv.dtype), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(status), stream_ptr())


def attn_decode_tc_supported(dtype: torch.dtype, H: int, KV: int, HD: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_attn_decode_tc_supported(H, KV, HD))


def attn_decode_stream_mode(mode: int) -> int:
    """How the tensor-core decode attention walks a step's pages: 0 one page a CTA, 2 persistent CTAs fed by TMA
    wherever that can run, 1 (the default) whichever pays. Returns the mode set before; the results are the same
    bits either way."""
    return int(lib.load().mynah_attn_decode_stream_mode(int(mode)))


def attn_decode_tc(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor, pages: PageTableView,
                   window: int, n_splits: int, scratch: torch.Tensor, status: torch.Tensor,
                   counters: Optional[torch.Tensor] = None) -> None:
    """The tensor-core decode attention (bfloat16, head_dim 64 or 128); same contract as attn_decode. With
    `counters` (B * KV zeroed int32 words, left zero) the pages' kernel also merges and no second launch is made;
    the result is the same."""
    _chk(qkv, "q", torch.bfloat16, 2)
    if counters is not None:
        _chk(counters, "counters", torch.int32, 1)
        if counters.numel() < B * KV:
            raise KernelError(f"attn_decode_tc: {counters.numel()} counters, {B * KV} are needed")
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(scratch, "scratch", torch.float32)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_tc: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_tc", ptr(qkv), ptr(out), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(counters), ptr(status), stream_ptr())


def attn_decode_fused(qkv: torch.Tensor, out: torch.Tensor, B: int, H: int, KV: int, HD: int,
                      q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], qk_eps: float,
                      cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], tok_pos: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, write_kv: bool, kv_len: torch.Tensor,
                      pages: PageTableView, window: int, n_splits: int, scratch: torch.Tensor,
                      counters: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Per-head norm, rotation, cache write and attention of a decode step in one launch (bfloat16, head_dim 64
    or 128, whole-head rotation or none). `qkv` holds the projection's rows; with write_kv False only q is read."""
    _chk(qkv, "qkv", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(scratch, "scratch", torch.float32)
    # counters None: the pages' CTAs do not merge, the merge follows as a launch of its own (the same bits)
    need = B * H * n_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_fused: scratch holds {scratch.numel()} floats, {need} are needed")
    if counters is not None:
        _chk(counters, "counters", torch.int32)
        if counters.numel() < B * KV:
            raise KernelError(f"attn_decode_fused: {counters.numel()} counters, {B * KV} are needed")
    if cos is not None and cos.shape[1] * 2 != HD:
        raise KernelError("attn_decode_fused: the rotation must cover the whole head")
    call("mynah_attn_decode_fused", ptr(qkv), ptr(out), B, H, KV, HD, qkv.shape[1], out.shape[1],
         ptr(q_gain), ptr(k_gain), code(q_gain.dtype) if q_gain is not None else 0, float(qk_eps),
         ptr(cos), ptr(sin), cos.shape[0] if cos is not None else 0, ptr(tok_pos),
         ptr(k_cache), ptr(v_cache), 1 if write_kv else 0, ptr(kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, n_splits, ptr(scratch), ptr(counters), ptr(status), stream_ptr())


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(logits, "logits", torch.float32, 2)
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    call("mynah_argmax", ptr(logits), B, V, V, ptr(out), stream_ptr())
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, rng: torch.Tensor, slots: Optional[torch.Tensor],
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Overwrites `logits`. params: float32 [7] on the device (temp, top_p,
    min_p, top_k, repeat, freq, presence); rng: int64 generator state per slot."""
    _chk(logits, "logits", torch.float32, 2)
    _chk(rng, "rng states", torch.int64, 1)
    _chk(params, "sampling parameters", torch.float32, 1)
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    pv = pi = None
    if V >= SAMPLE_TWO_STEP_MIN_VOCAB:
        pv, pi = _sample_scratch(logits.device, B)
    call("mynah_sample", ptr(logits), B, V, V, ptr(params), ptr(rng), ptr(slots), ptr(out), ptr(pv), ptr(pi), stream_ptr())
    return out


# From this vocabulary size on a row's maximum is found by several CTAs first (one CTA reads a long row slowly).
SAMPLE_TWO_STEP_MIN_VOCAB = 16384
_SAMPLE_SCRATCH: dict = {}


def _sample_scratch(device, B: int):
    """Scratch of the two-step maximum, kept for the life of the process (a captured step holds its address)."""
    key = (str(device), B)
    if key not in _SAMPLE_SCRATCH:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("sample: scratch memory must exist before graph capture")
        n = B * int(lib.load().mynah_argmax_parts())
        _SAMPLE_SCRATCH[key] = (torch.empty((n,), dtype=torch.float32, device=device),
                                torch.empty((n,), dtype=torch.int32, device=device))
    return _SAMPLE_SCRATCH[key]


def apply_penalties(logits: torch.Tensor, ring: torch.Tensor, ring_n: torch.Tensor, slots: Optional[torch.Tensor],
                    params: torch.Tensor) -> None:
    _chk(logits, "logits", torch.float32, 2)
    _chk(ring, "ring", torch.int32, 2)
    B, V = logits.shape
    call("mynah_apply_penalties", ptr(logits), B, V, V, ptr(ring), ptr(ring_n), ring.shape[1], ptr(slots),
         ptr(params), stream_ptr())


def sampler_accept(tokens: torch.Tensor, ring: torch.Tensor, ring_n: torch.Tensor, ring_head: torch.Tensor,
                   slots: Optional[torch.Tensor], params: torch.Tensor) -> None:
    _chk(tokens, "tokens", torch.int32, 1)
    call("mynah_sampler_accept", ptr(tokens), tokens.numel(), ptr(ring), ptr(ring_n), ptr(ring_head),
         ring.shape[1], ptr(slots), ptr(params), stream_ptr())


def decode_advance(tokens: torch.Tensor, sampled: torch.Tensor, tok_pos: torch.Tensor, kv_len: torch.Tensor,
                   slots: torch.Tensor) -> None:
    call("mynah_decode_advance", ptr(tokens), ptr(sampled), ptr(tok_pos), ptr(kv_len), ptr(slots),
         tokens.numel(), stream_ptr())


def l2_prefetch(tensors) -> None:
    """Ask the memory system to bring these tensors (contiguous, at most 8) into L2; returns at once and computes
    nothing. Meant for a second stream beside a chain of kernels that will read the tensors shortly."""
    import ctypes
    ts = [t for t in tensors if t is not None and t.is_cuda and t.is_contiguous() and t.numel()]
    for i in range(0, len(ts), 8):
        part = ts[i:i + 8]
        ptrs = (ctypes.c_void_p * len(part))(*[t.data_ptr() for t in part])
        sizes = (ctypes.c_ulonglong * len(part))(*[t.numel() * t.element_size() for t in part])
        call("mynah_l2_prefetch", ptrs, sizes, len(part), stream_ptr())


# ------------------------------------------------------------------ parts of mixers with recurrent state
ACTIVATIONS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "relu2": 4}


def embed_positions(table: torch.Tensor, pos_table: torch.Tensor, tokens: torch.Tensor, tok_pos: torch.Tensor,
                    status: torch.Tensor) -> torch.Tensor:
    """x[t] = table[token_t] + pos_table[position_t], fp32 [T, D]."""
    _chk(table, "embedding table", dim=2)
    _chk(pos_table, "position table", table.dtype, 2)
    _chk(tokens, "tokens", torch.int32, 1)
    _chk(tok_pos, "positions", torch.int32, 1)
    T, (V, D) = tokens.numel(), table.shape
    if pos_table.shape[1] != D:
        raise KernelError("embed_positions: the two tables differ in width")
    out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    call("mynah_embed_positions", ptr(table), ptr(pos_table), code(table.dtype), ptr(tokens), ptr(tok_pos), ptr(out),
         T, D, V, pos_table.shape[0], ptr(status), stream_ptr())
    return out


def activation(x: torch.Tensor, act: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(x) elementwise (fp32 arithmetic); `out` may be x itself."""
    _chk(x, "activation input")
    if act not in ACTIVATIONS:
        raise KernelError(f"unknown activation {act!r}; known: {', '.join(sorted(ACTIVATIONS))}")
    if out is None:
        out = torch.empty_like(x)
    call("mynah_activation", ptr(x), ptr(out), code(x.dtype), x.numel(), ACTIVATIONS[act], stream_ptr())
    return out


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The fp32 residual rows rounded to the activation type."""
    _chk(x, "residual", torch.float32)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    call("mynah_cast_f32", ptr(x), ptr(out), code(dtype), x.numel(), stream_ptr())
    return out


def layernorm_rows(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, act_dtype: torch.dtype,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LN(x[rows]) * w + b of the fp32 residual stream, in the activation type."""
    _chk(x, "residual", torch.float32, 2)
    _chk(w, "norm weight", dim=1)
    if b is not None:
        _chk(b, "norm bias", w.dtype, 1)
    D = x.shape[1]
    if w.numel() != D or (b is not None and b.numel() != D):
        raise KernelError("layernorm: weight or bias does not match the row")
    n = x.shape[0]
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
        n = rows.numel()
    out = torch.empty((n, D), dtype=act_dtype, device=x.device)
    call("mynah_layernorm_rows", ptr(x), ptr(rows), ptr(w), ptr(b), code(w.dtype), ptr(out), code(act_dtype), n, D,
         float(eps), stream_ptr())
    return out


def layernorm_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float,
                  copy: bool = False, copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += LN(y) * w + b, row by row (x fp32, in place). With `copy` the new x is also returned, in `copy_dtype`
    (y's type unless given; an fp32 y may come with a bfloat16 copy)."""
    _chk(x, "residual", torch.float32, 2)
    if y.dim() != 2 or y.stride(1) != 1 or not y.is_cuda:
        raise KernelError("layernorm_add: the sublayer's output must be rows on the device")
    if y.shape != x.shape:
        raise KernelError(f"layernorm_add: output {tuple(y.shape)} does not match the residual {tuple(x.shape)}")
    _chk(w, "norm weight", dim=1)
    if b is not None:
        _chk(b, "norm bias", w.dtype, 1)
    n, D = x.shape
    copy_dtype = copy_dtype or y.dtype
    xc = torch.empty((n, D), dtype=copy_dtype, device=x.device) if copy else None
    call("mynah_layernorm_add", ptr(y), code(y.dtype), y.stride(0), ptr(w), ptr(b), code(w.dtype), ptr(x), ptr(xc),
         code(copy_dtype), n, D, float(eps), stream_ptr())
    return xc


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor],
                ctx, out_dtype: torch.dtype, act: Optional[str] = None, add_input: bool = False,
                channels: Optional[int] = None) -> torch.Tensor:
    """Per-channel causal convolution along each sequence of the step (see csrc/seq_conv.cu). x [T, >= C] rows
    (a column slice is fine), w [C, taps], state fp32 [max_seqs + 1, taps - 1, C]: read, then shifted."""
    if x.dim() != 2 or x.stride(1) != 1 or not x.is_cuda:
        raise KernelError("causal_conv: the input must be rows on the device")
    _chk(w, "filter", dim=2)
    C, taps = w.shape
    if channels is not None and channels != C:
        raise KernelError("causal_conv: the filter does not match the channels")
    if x.shape[1] != C:
        raise KernelError(f"causal_conv: the input has {x.shape[1]} channels, the filter {C}")
    if bias is not None:
        _chk(bias, "filter bias", w.dtype, 1)
    if taps > 1:
        _chk(state, "convolution state", torch.float32, 3)
        if tuple(state.shape[1:]) != (taps - 1, C):
            raise KernelError(f"causal_conv: state rows are {tuple(state.shape[1:])}, expected {(taps - 1, C)}")
    if act not in (None, "silu"):
        raise KernelError(f"causal_conv: activation {act!r} is not built in (none or 'silu')")
    T = x.shape[0]
    out = torch.empty((T, C), dtype=out_dtype, device=x.device)
    call("mynah_causal_conv", ptr(x), code(x.dtype), x.stride(0), ptr(w), ptr(bias), code(w.dtype),
         ptr(state), (state.shape[0] - 1) if state is not None else 0, ptr(out), code(out_dtype), C,
         ptr(ctx.tok_seq), ptr(ctx.cu_q), ptr(ctx.slots), T, ctx.B, C, taps, 1 if act == "silu" else 0,
         1 if add_input else 0, 1 if ctx.is_decode else 0, stream_ptr())
    return out


def attn_prep(qkv: torch.Tensor, q_out: torch.Tensor, H: int, G: int, dim: int, vd: int, dimp: int, vdp: int,
              q_gain: torch.Tensor, k_gain: torch.Tensor, eps: float, cos, sin, rot: int, ctx, pages: PageTableView,
              k_cache, v_cache, v_first: Optional[torch.Tensor], lam: Optional[torch.Tensor], vmix: int) -> None:
    """Whole-projection q/k norm, partial rotation, per-head value norm, value mixing, cache write (csrc/attn_prep.cu)."""
    _chk(qkv, "qkv", dim=2)
    _chk(q_out, "q", qkv.dtype, 2)
    if q_gain.dtype != k_gain.dtype or q_gain.numel() != H * dim or k_gain.numel() != G * dim:
        raise KernelError("attn_prep: the gains must cover the whole q and k projections, in one dtype")
    if k_cache is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("attn_prep: the cache and the activations differ in dtype")
        if tuple(k_cache.shape[1:]) != (G, PAGE_TOKENS, dimp) or tuple(v_cache.shape[1:]) != (G, PAGE_TOKENS, vdp):
            raise KernelError("attn_prep: the cache pages do not have the stored head sizes")
    if qkv.shape[1] < H * dim + (G * (dim + vd) if k_cache is not None else 0):
        raise KernelError("attn_prep: the projection's rows are too short")
    if v_first is not None:
        _chk(v_first, "v_first", torch.float32, 2)
        if v_first.shape[0] < qkv.shape[0] or v_first.shape[1] != G * vd:
            raise KernelError("attn_prep: v_first does not match the step")
    if lam is not None:
        _chk(lam, "mixing weight", torch.float32)
    n_pos = cos.shape[0] if cos is not None else 0
    call("mynah_attn_prep", ptr(qkv), code(qkv.dtype), qkv.shape[0], qkv.shape[1], ptr(q_out), q_out.shape[1],
         H, G, dim, vd, dimp, vdp, ptr(q_gain), ptr(k_gain), code(q_gain.dtype), float(eps),
         ptr(cos), ptr(sin), rot, n_pos, ptr(ctx.tok_seq), ptr(ctx.tok_pos),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         ptr(k_cache), ptr(v_cache), ptr(v_first), ptr(lam), vmix, ptr(ctx.status), stream_ptr())


def attn_prefill_general(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, VD: int,
                         k_cache: torch.Tensor, v_cache: torch.Tensor, pages: PageTableView,
                         window: int, chunk: int, scale: float) -> None:
    """The general prompt attention with value heads of their own width, a given score scale and a chunk mask."""
    _chk(q, "q", dim=2)
    _chk(out, "attention output", q.dtype, 2)
    call("mynah_attn_prefill_generic_ex", ptr(q), ptr(out), code(q.dtype), q.shape[0], ctx.B, ctx.max_q_len, H, KV, HD, VD,
         q.shape[1], out.shape[1], ptr(k_cache), ptr(v_cache), ptr(ctx.cu_q), ptr(ctx.kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, chunk or 0, float(scale),
         ptr(ctx.status), stream_ptr())


def attn_decode_general(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, VD: int,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, pages: PageTableView,
                        window: int, chunk: int, scale: float, scratch: torch.Tensor) -> None:
    _chk(q, "q", dim=2)
    _chk(out, "attention output", q.dtype, 2)
    _chk(scratch, "scratch", torch.float32)
    need = ctx.B * H * ctx.decode_splits * (VD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_ex", ptr(q), ptr(out), code(q.dtype), ctx.B, H, KV, HD, VD, q.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, chunk or 0, float(scale), ctx.decode_splits, ptr(scratch), ptr(ctx.status), stream_ptr())


def _rows(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
        raise KernelError(f"{name} must be rows on the device (unit stride along a row)")


# Rows of a piece of the selective scan's two-pass form (0: every sequence is walked whole by one CTA).
SCAN_PIECE_ROWS = int(os.environ.get("MYNAH_SCAN_PIECE_ROWS", "64"))


def selective_scan(x: torch.Tensor, z: torch.Tensor, dt_raw: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                   dt_bias, A_log: torch.Tensor, D, state: torch.Tensor, ctx) -> torch.Tensor:
    """The Mamba-1 recurrence with its gate (csrc/selective_scan.cu). x, z [T, inner] (z may be a column slice);
    dt_raw [T, inner], Bm, Cm [T, N] column slices of one tensor; state fp32 [max_seqs + 1, inner, N]."""
    for t, n in ((x, "x"), (z, "z"), (dt_raw, "dt"), (Bm, "B"), (Cm, "C")):
        _rows(t, "selective_scan: " + n)
    _chk(state, "scan state", torch.float32, 3)
    T, inner = x.shape
    N = A_log.shape[1]
    if tuple(state.shape[1:]) != (inner, N) or Bm.shape[1] != N or Cm.shape[1] != N or Bm.stride(0) != Cm.stride(0):
        raise KernelError("selective_scan: sizes do not fit")
    if z.dtype != x.dtype or Bm.dtype != Cm.dtype or dt_raw.dtype != torch.float32:
        raise KernelError("selective_scan: dtypes do not fit (dt in float32, B and C alike, z like x)")
    if A_log.dtype != dt_bias.dtype or A_log.dtype != D.dtype:
        raise KernelError("selective_scan: A_log, dt bias and D must share a dtype")
    y = torch.empty((T, inner), dtype=x.dtype, device=x.device)
    # Prompts of at least two pieces run piece by piece, side by side, in two passes (see the kernel); the pieces'
    # end states and the sums of their step sizes go through scratch memory.
    piece = SCAN_PIECE_ROWS if (not ctx.is_decode and SCAN_PIECE_ROWS and ctx.max_q_len >= 2 * SCAN_PIECE_ROWS) else 0
    n_pieces = T // piece + ctx.B + 1 if piece else 0
    scratch = (torch.empty((n_pieces * inner * (N + 1) + ctx.B * inner * N,), dtype=torch.float32, device=x.device)
               if piece else None)
    call("mynah_selective_scan", ptr(x), x.stride(0), ptr(z), z.stride(0), ptr(y), inner, code(x.dtype),
         ptr(dt_raw), dt_raw.stride(0), ptr(Bm), ptr(Cm), Bm.stride(0), code(Bm.dtype),
         ptr(dt_bias), ptr(A_log), ptr(D), code(A_log.dtype), ptr(state), state.shape[0] - 1,
         ptr(ctx.cu_q), ptr(ctx.slots), ctx.B, inner, N, piece, n_pieces, ctx.max_q_len, ptr(scratch), stream_ptr())
    return y


def delta_prep(qk: torch.Tensor, a_raw: Optional[torch.Tensor], b_raw: torch.Tensor, A_log: torch.Tensor,
               dt_bias: torch.Tensor, H: int, G: int, dim: int, a_channels: Optional[torch.Tensor] = None):
    """Unit q and k per head, beta and the decay of the gated delta rule (csrc/delta_rule.cu); all fp32. The decay is
    one a head from a_raw [T, H], or, with a_channels (fp32 rows of H * dim values; dt_bias likewise), one a head and
    key channel: g is then [T, H * dim]."""
    _rows(qk, "delta_prep: q|k")
    _rows(b_raw, "delta_prep: b")
    if b_raw.dtype != qk.dtype:
        raise KernelError("delta_prep: b must have the activations' type")
    T = qk.shape[0]
    dev = qk.device
    if a_channels is None:
        _rows(a_raw, "delta_prep: a")
        if a_raw.stride(0) != b_raw.stride(0) or a_raw.dtype != qk.dtype:
            raise KernelError("delta_prep: a and b must be column slices of one tensor of the activations' type")
        g = torch.empty((T, H), dtype=torch.float32, device=dev)
    else:
        _rows(a_channels, "delta_prep: a per channel")
        if a_channels.dtype != torch.float32 or a_channels.shape[1] != H * dim or dt_bias.numel() != H * dim:
            raise KernelError("delta_prep: decays per channel need fp32 rows and a bias of heads x dim values")
        g = torch.empty((T, H * dim), dtype=torch.float32, device=dev)
    qn = torch.empty((T, G * dim), dtype=torch.float32, device=dev)
    kn = torch.empty((T, G * dim), dtype=torch.float32, device=dev)
    beta = torch.empty((T, H), dtype=torch.float32, device=dev)
    call("mynah_delta_prep", ptr(qk), qk.stride(0), ptr(a_raw), ptr(b_raw), b_raw.stride(0), code(qk.dtype),
         ptr(A_log), ptr(dt_bias), code(A_log.dtype), ptr(qn), ptr(kn), ptr(g), ptr(beta), T, H, G, dim,
         ptr(a_channels), a_channels.stride(0) if a_channels is not None else 0, stream_ptr())
    return qn, kn, g, beta


def delta_rule(qn: torch.Tensor, kn: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
               state: torch.Tensor, ctx, H: int, G: int, dim: int, vd: int, channel_decay: bool = False) -> torch.Tensor:
    """The recurrence; state fp32 [max_seqs + 1, H, dim, vd]; returns o fp32 [T, H * vd]. g fp32 [T, H], or
    [T, H * dim] with channel_decay (one decay a head and key channel)."""
    _rows(v, "delta_rule: v")
    _chk(state, "delta state", torch.float32, 4)
    if tuple(state.shape[1:]) != (H, dim, vd):
        raise KernelError("delta_rule: the state does not fit")
    T = v.shape[0]
    _chk(g, "decay", torch.float32, 2)
    if g.shape[1] != (H * dim if channel_decay else H):
        raise KernelError("delta_rule: the decay's rows do not fit")
    channel = 1 if channel_decay else 0
    o = torch.empty((T, H * vd), dtype=torch.float32, device=v.device)
    call("mynah_delta_rule", ptr(qn), ptr(kn), ptr(v), v.stride(0), code(v.dtype), ptr(g), ptr(beta), ptr(state),
         state.shape[0] - 1, ptr(o), ptr(ctx.cu_q), ptr(ctx.slots), ctx.B, H, G, dim, vd, channel, stream_ptr())
    return o


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, H: int, vd: int, eps: float,
                  gate_act: str = "silu") -> torch.Tensor:
    """o / rms(o per head) * w * act(gate), act silu or sigmoid; o fp32 [T, H * vd], gate rows (any of the two types),
    the output in the gate's type."""
    _chk(o, "o", torch.float32, 2)
    _rows(gate, "gated_rmsnorm: gate")
    if gate_act not in ("silu", "sigmoid"):
        raise KernelError(f"gated_rmsnorm: gate activation {gate_act!r} is neither 'silu' nor 'sigmoid'")
    T = o.shape[0]
    out = torch.empty((T, H * vd), dtype=gate.dtype, device=o.device)
    call("mynah_gated_rmsnorm", ptr(o), ptr(gate), gate.stride(0), code(gate.dtype), ptr(w), code(w.dtype), ptr(out),
         T, H, vd, float(eps), 1 if gate_act == "sigmoid" else 0, stream_ptr())
    return out


def attn_prefill_tcgen05_masked(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int,
                                k_cache: torch.Tensor, v_cache: torch.Tensor, pages: PageTableView,
                                window: int, chunk: int, scale: float) -> None:
    """The tcgen05 prompt attention with a chunk mask beside the window and a given score scale (> 0). q and out may be
    column slices (some of the heads) of wider rows whose stride is a multiple of 8."""
    for t, n in ((q, "q"), (out, "attention output")):
        _rows(t, "attn_prefill_tcgen05: " + n)
        if t.dtype != torch.bfloat16 or t.stride(0) % 8 or t.data_ptr() % 16:
            raise KernelError(f"attn_prefill_tcgen05: {n} must be bfloat16 rows, 16-byte aligned")
    _chk(k_cache, "K cache", torch.bfloat16)
    _chk(v_cache, "V cache", torch.bfloat16)
    call("mynah_attn_prefill_tcgen05_ex", ptr(q), ptr(out), q.shape[0], ctx.B, ctx.max_q_len, H, KV, HD, q.stride(0), out.stride(0),
         ptr(k_cache), ptr(v_cache), ptr(ctx.cu_q), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base),
         pages.n_pages, window or 0, chunk or 0, float(scale), ptr(ctx.status), stream_ptr())


def attn_decode_tc_masked(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int,
                          k_cache: torch.Tensor, v_cache: torch.Tensor, pages: PageTableView,
                          window: int, chunk: int, scale: float, scratch: torch.Tensor) -> None:
    """The tensor-core decode attention with a chunk mask instead of the window and a given score scale. q and out may
    be column slices (some of the heads) of wider rows whose stride is a multiple of 8."""
    for t, n in ((q, "q"), (out, "attention output")):
        _rows(t, "attn_decode_tc: " + n)
        if t.dtype != torch.bfloat16 or t.stride(0) % 8 or t.data_ptr() % 16:
            raise KernelError(f"attn_decode_tc: {n} must be bfloat16 rows, 16-byte aligned")
    _chk(scratch, "scratch", torch.float32)
    need = ctx.B * H * ctx.decode_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_tc: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_tc_ex", ptr(q), ptr(out), ctx.B, H, KV, HD, q.stride(0), out.stride(0),
         ptr(k_cache), ptr(v_cache), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, chunk or 0, float(scale), ctx.decode_splits, ptr(scratch), None, ptr(ctx.status), stream_ptr())


# ------------------------------------------------------------------ latent attention, retention, routed experts
def scale_(x: torch.Tensor, s: float) -> torch.Tensor:
    """x *= s in place (fp32)."""
    _chk(x, "rows", torch.float32)
    call("mynah_scale_f32", ptr(x), x.numel(), float(s), stream_ptr())
    return x


def rope_table_freqs(n_pos: int, freqs, mult: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [n_pos, pairs] of the angles position * freqs[i], each times `mult`; angles in double."""
    f = torch.as_tensor(freqs, dtype=torch.float64).to(device).contiguous()
    half = f.numel()
    cos = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    sin = torch.empty((n_pos, half), dtype=torch.float32, device=device)
    call("mynah_rope_table_freqs", ptr(cos), ptr(sin), n_pos, half, ptr(f), float(mult), stream_ptr())
    return cos, sin


def latent_prep(q: torch.Tensor, q_off: int, dkv: Optional[torch.Tensor], dkv_off: int, q_out: torch.Tensor,
                H: int, dim: int, rd: int, r: int, HDp: int, w: Optional[torch.Tensor], eps: float, cos, sin, rot: int,
                interleaved: bool, ctx, pages: PageTableView, k_cache: Optional[torch.Tensor]) -> None:
    """Latent norm, rotation of the shared key part and of every head's rotated query part, cache write
    (csrc/latent_attn.cu). q_out [T, H * HDp]: columns [r, HDp) of every head are written."""
    _rows(q, "latent_prep: q")
    _chk(q_out, "packed queries", q.dtype, 2)
    if q_out.shape[1] != H * HDp:
        raise KernelError("latent_prep: the packed query rows do not have heads x stored width columns")
    if q.shape[1] < q_off + H * (dim + rd):
        raise KernelError("latent_prep: the query projection's rows are too short")
    if (dkv is None) != (k_cache is None):
        raise KernelError("latent_prep: the down-projection and the cache go together")
    if dkv is not None:
        _rows(dkv, "latent_prep: down-projection")
        if dkv.dtype != q.dtype or k_cache.dtype != q.dtype:
            raise KernelError("latent_prep: activations and cache differ in dtype")
        if dkv.shape[1] < dkv_off + r + rd:
            raise KernelError("latent_prep: the down-projection's rows are too short")
        if tuple(k_cache.shape[1:]) != (1, PAGE_TOKENS, HDp) or not k_cache.is_contiguous():
            raise KernelError(f"latent_prep: cache pages are {tuple(k_cache.shape[1:])}, expected {(1, PAGE_TOKENS, HDp)}")
        _chk(w, "latent norm weight", dim=1)
        if w.numel() != r:
            raise KernelError("latent_prep: the norm weight does not match the latent")
    n_pos = cos.shape[0] if cos is not None else 0
    if cos is not None and cos.shape[1] * 2 != rot:
        raise KernelError("latent_prep: the rotation table does not match the rotated dims")
    call("mynah_latent_prep", ptr(q), q.stride(0), q_off, ptr(dkv), dkv.stride(0) if dkv is not None else 0, dkv_off,
         code(q.dtype), ptr(q_out), q.shape[0], H, dim, rd, r, HDp, ptr(w), code(w.dtype) if w is not None else 0,
         float(eps), ptr(cos), ptr(sin), rot if cos is not None else 0, 1 if interleaved else 0, n_pos,
         ptr(ctx.tok_seq), ptr(ctx.tok_pos), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         ptr(k_cache), ptr(ctx.status), stream_ptr())


def head_linear(x: torch.Tensor, head_in: int, in_off: int, W: torch.Tensor, out: torch.Tensor, head_out: int,
                out_off: int, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * head_out + out_off + j] = sum_i W[h, j, i] * x[t, h * head_in + in_off + i]: one small product a head
    (csrc/latent_attn.cu). W [H, n_out, n_in] in the rows' type; fp32 accumulation. With `gate` (rows of H logits in
    the rows' type; a column slice is fine) head h's outputs are multiplied by sigmoid(gate[t, h]) before they are
    rounded."""
    _rows(x, "head_linear: input")
    _rows(out, "head_linear: output")
    _chk(W, "head_linear: weights", x.dtype, 3)
    if out.dtype != x.dtype or out.shape[0] != x.shape[0]:
        raise KernelError("head_linear: input and output rows differ")
    H, n_out, n_in = W.shape
    if (H - 1) * head_in + in_off + n_in > x.shape[1] or (H - 1) * head_out + out_off + n_out > out.shape[1]:
        raise KernelError("head_linear: the heads do not fit the rows")
    if gate is not None:
        _rows(gate, "head_linear: gate")
        if gate.dtype != x.dtype or gate.shape[0] != x.shape[0] or gate.shape[1] < H:
            raise KernelError("head_linear: the gate's rows do not fit the heads")
    call("mynah_head_linear_gated", ptr(x), ptr(W), ptr(out), code(x.dtype), x.shape[0], H, n_in, n_out,
         x.stride(0), head_in, in_off, out.stride(0), head_out, out_off, ptr(gate), gate.stride(0) if gate is not None else 0,
         stream_ptr())
    return out


def retention_prep(p: torch.Tensor, q_off: int, k_off: int, H: int, dim: int, cos, sin, rot: int, interleaved: bool,
                   k_scale: float, ctx):
    """fp32 q and k of every head, rotated; k also scaled (csrc/retention.cu). p: the projection's rows."""
    _rows(p, "retention_prep: projection")
    if max(q_off, k_off) + H * dim > p.shape[1]:
        raise KernelError("retention_prep: the projection's rows are too short")
    T = p.shape[0]
    qn = torch.empty((T, H * dim), dtype=torch.float32, device=p.device)
    kn = torch.empty((T, H * dim), dtype=torch.float32, device=p.device)
    n_pos = cos.shape[0] if cos is not None else 0
    if cos is not None and cos.shape[1] * 2 != rot:
        raise KernelError("retention_prep: the rotation table does not match the rotated dims")
    call("mynah_retention_prep", ptr(p), p.stride(0), q_off, k_off, code(p.dtype), ptr(qn), ptr(kn), T, H, dim,
         ptr(cos), ptr(sin), rot if cos is not None else 0, 1 if interleaved else 0, n_pos, float(k_scale),
         ptr(ctx.tok_seq), ptr(ctx.tok_pos), ptr(ctx.status), stream_ptr())
    return qn, kn


def retention_scan(qn: torch.Tensor, kn: torch.Tensor, v: torch.Tensor, v_off: int, decay: torch.Tensor,
                   state: torch.Tensor, ctx, H: int, dim: int, vd: int) -> torch.Tensor:
    """The decayed recurrence; state fp32 [max_seqs + 1, H, dim, vd]; returns o fp32 [T, H * vd]."""
    _rows(v, "retention_scan: v")
    _chk(state, "retention state", torch.float32, 4)
    _chk(decay, "decays", torch.float32, 1)
    if tuple(state.shape[1:]) != (H, dim, vd) or decay.numel() != H:
        raise KernelError("retention_scan: the state or the decays do not fit")
    if v_off + H * vd > v.shape[1]:
        raise KernelError("retention_scan: the value rows are too short")
    T = v.shape[0]
    o = torch.empty((T, H * vd), dtype=torch.float32, device=v.device)
    need = int(lib.load().mynah_retention_scratch_floats(T, H, dim, int(ctx.max_q_len)))      # the chunked form's scores
    scratch = torch.empty((need,), dtype=torch.float32, device=v.device) if need else None
    call("mynah_retention_scan", ptr(qn), ptr(kn), ptr(v), v.stride(0), v_off, code(v.dtype), ptr(decay), ptr(state),
         state.shape[0] - 1, ptr(o), ptr(ctx.cu_q), ptr(ctx.slots), ctx.B, H, dim, vd, int(ctx.max_q_len), T, ptr(scratch),
         stream_ptr())
    if need:
        lib.add_launches(1)
    return o


def retention_chunk_min(n: int) -> int:
    """From how many tokens in a step's longest piece the retention recurrence runs chunk by chunk (keys that are a
    multiple of 32 values up to 256); 0: always token by token. Returns the setting before. The two forms agree to
    rounding."""
    return int(lib.load().mynah_retention_chunk_min(int(n)))


def head_linear_plain(on: bool) -> bool:
    """Run the bfloat16 per-head products on the plain tiled kernel instead of the tensor-core one (the tests compare the
    two). Returns the setting before."""
    return bool(lib.load().mynah_head_linear_plain(1 if on else 0))


def moe_grouped_min(n: int) -> int:
    """From how many (token, choice) pairs a bfloat16 step's expert products run as grouped tcgen05 products; 0: never
    (they then run tile by tile on `mma.sync`). Returns the setting before; the two agree to rounding."""
    return int(lib.load().mynah_moe_grouped_min(int(n)))


def moe_plain(on: bool) -> bool:
    """Run the experts' bfloat16 products on the plain tiled kernels instead of the tensor-core ones (the tests compare
    the two). Returns the setting before."""
    return bool(lib.load().mynah_moe_plain(1 if on else 0))


def moe_table_ffn(h: torch.Tensor, table: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ctx, top: int,
                  limit: float, alpha: float) -> torch.Tensor:
    """Experts picked per token id from `table` [vocab, top], equal weights (csrc/moe.cu). w_gu [E, 2, F, D],
    w_down [E, D, F]; returns [T, D] in the rows' type."""
    _chk(h, "rows", dim=2)
    _chk(table, "expert table", torch.int32, 2)
    _chk(w_gu, "gate/up weights", h.dtype, 4)
    _chk(w_down, "down weights", h.dtype, 3)
    T, D = h.shape
    E, _, F, _ = w_gu.shape
    if tuple(w_gu.shape) != (E, 2, F, D) or tuple(w_down.shape) != (E, D, F) or table.shape[1] != top:
        raise KernelError("moe_table_ffn: sizes do not fit")
    P_ = T * top
    dev = h.device
    # rows of the sorted, padded layout when the step's products run as grouped tensor-core products (prompts), else 0
    grouped = int(lib.load().mynah_moe_grouped_rows(T, top, E, D, F, code(h.dtype)))
    R = max(P_, grouped)
    out = torch.empty((T, D), dtype=h.dtype, device=dev)
    y = torch.empty((R, F), dtype=h.dtype, device=dev)
    o = torch.empty((R, D), dtype=torch.float32, device=dev)
    a = torch.empty((R, D), dtype=h.dtype, device=dev) if grouped else None
    ints = torch.empty((2 * P_ + 1 + 3 * int(lib.load().mynah_moe_max_tiles(T, top, E)) + R + R // 128 + 1,),
                       dtype=torch.int32, device=dev)
    call("mynah_moe_table_ffn", ptr(h), code(h.dtype), ptr(ctx.tokens), ptr(ctx.tok_seq), ptr(table), ptr(w_gu),
         ptr(w_down), ptr(out), ptr(y), ptr(o), ptr(ints), ptr(a), T, table.shape[0], top, E, D, F, float(limit), float(alpha),
         1.0 / top, ptr(ctx.status), stream_ptr())
    lib.add_launches(4 if grouped else 3)     # route, (gather,) two products, combine
    return out


def moe_router_ffn(h: torch.Tensor, w_router: torch.Tensor, b_router: torch.Tensor, w_up: torch.Tensor,
                   w_down: torch.Tensor, ctx, top: int) -> torch.Tensor:
    """Experts picked by a learned router (fp32 logits W_r h + b_r, the `top` largest, softmax over the chosen alone);
    an expert is W_down gelu_erf(W_up h) (csrc/moe.cu). w_router [E, D], b_router [E], w_up [E, F, D], w_down
    [E, D, F]; returns fp32 [T, D]: the weighted sum is not rounded to the rows' type."""
    _chk(h, "rows", dim=2)
    _chk(w_router, "router weights", h.dtype, 2)
    _chk(b_router, "router bias", dim=1)
    _chk(w_up, "up weights", h.dtype, 3)
    _chk(w_down, "down weights", h.dtype, 3)
    T, D = h.shape
    E, F, _ = w_up.shape
    if (tuple(w_up.shape) != (E, F, D) or tuple(w_down.shape) != (E, D, F) or tuple(w_router.shape) != (E, D)
            or b_router.numel() != E or not 1 <= top <= E):
        raise KernelError("moe_router_ffn: sizes do not fit")
    P_ = T * top
    dev = h.device
    grouped = int(lib.load().mynah_moe_grouped_rows(T, top, E, D, F, code(h.dtype)))
    R = max(P_, grouped)
    out = torch.empty((T, D), dtype=torch.float32, device=dev)
    y = torch.empty((R, F), dtype=h.dtype, device=dev)
    o = torch.empty((R, D), dtype=torch.float32, device=dev)
    a = torch.empty((R, D), dtype=h.dtype, device=dev) if grouped else None
    ints = torch.empty((3 * P_ + 1 + 3 * int(lib.load().mynah_moe_max_tiles(T, top, E)) + R + R // 128 + 1,),
                       dtype=torch.int32, device=dev)
    weights = torch.empty((P_,), dtype=torch.float32, device=dev)
    choice = ints[ints.numel() - P_:]
    call("mynah_moe_router_ffn", ptr(h), code(h.dtype), ptr(ctx.tok_seq), ptr(w_router), ptr(b_router), code(b_router.dtype),
         ptr(w_up), ptr(w_down), ptr(out), ptr(y), ptr(o), ptr(ints), ptr(a), ptr(choice), ptr(weights), T, top, E, D, F,
         ptr(ctx.status), stream_ptr())
    lib.add_launches(5 if grouped else 4)     # router, route, (gather,) two products, combine
    return out


def rmsnorm_add(x: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float, extra: Optional[torch.Tensor] = None,
                gain2: Optional[torch.Tensor] = None, eps2: float = 0.0) -> Optional[torch.Tensor]:
    """x <- x (+ extra) + y / rms(y) * gain, all fp32 (csrc/norm_post.cu); with gain2 also returns the RMS norm of the
    new x under gain2 and eps2 as fp32 rows."""
    _chk(x, "residual", torch.float32, 2)
    _chk(y, "sublayer output", torch.float32, 2)
    _chk(gain, "norm gain", dim=1)
    T, D = x.shape
    if y.shape != x.shape or gain.numel() != D or (extra is not None and (extra.shape != x.shape or extra.dtype != torch.float32)):
        raise KernelError("rmsnorm_add: shapes differ")
    h = None
    if gain2 is not None:
        _chk(gain2, "second norm gain", dim=1)
        if gain2.numel() != D:
            raise KernelError("rmsnorm_add: the second gain does not fit the rows")
        h = torch.empty((T, D), dtype=torch.float32, device=x.device)
    call("mynah_rmsnorm_add", ptr(x), ptr(y), ptr(extra), ptr(gain), code(gain.dtype), float(eps), ptr(gain2),
         code(gain2.dtype) if gain2 is not None else 0, float(eps2), ptr(h), T, D, stream_ptr())
    return h


def rms_pair_mean(a: torch.Tensor, b: torch.Tensor, ga: torch.Tensor, gb: torch.Tensor, eps: float,
                  weight: float) -> torch.Tensor:
    """weight * (a / rms(a) * ga + b / rms(b) * gb), fp32 rows in and out (csrc/norm_post.cu)."""
    _chk(a, "first branch", torch.float32, 2)
    _chk(b, "second branch", torch.float32, 2)
    _chk(ga, "first gain", dim=1)
    _chk(gb, "second gain", ga.dtype, 1)
    T, D = a.shape
    if b.shape != a.shape or ga.numel() != D or gb.numel() != D:
        raise KernelError("rms_pair_mean: shapes differ")
    out = torch.empty((T, D), dtype=torch.float32, device=a.device)
    call("mynah_rms_pair_mean", ptr(a), ptr(b), ptr(ga), ptr(gb), code(ga.dtype), float(eps), float(weight), ptr(out), T, D,
         stream_ptr())
    return out


def rglru_in(p: torch.Tensor, y_off: int, x_off: int, width: int, by: torch.Tensor, bx: torch.Tensor):
    """The recurrent unit's two branches from their stacked projection p [T, >= 2 * width]: y = gelu_tanh(p_y + b_y) in p's
    type, x = p_x + b_x in fp32 (csrc/rglru.cu)."""
    _rows(p, "rglru_in: projection")
    _chk(by, "gate bias", dim=1)
    _chk(bx, "input bias", by.dtype, 1)
    T = p.shape[0]
    if by.numel() != width or bx.numel() != width or max(y_off, x_off) + width > p.shape[1]:
        raise KernelError("rglru_in: sizes do not fit")
    y = torch.empty((T, width), dtype=p.dtype, device=p.device)
    x = torch.empty((T, width), dtype=torch.float32, device=p.device)
    call("mynah_rglru_in", ptr(p), p.stride(0), y_off, x_off, code(p.dtype), ptr(by), ptr(bx), code(by.dtype), ptr(y), ptr(x),
         T, width, stream_ptr())
    return y, x


def rglru_gates(u: torch.Tensor, ra: torch.Tensor, ri: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor, lam: torch.Tensor,
                decay_scale: float):
    """a = exp(-decay_scale * sigmoid(Ra u + ba) * softplus(lam)) and b = sqrt(1 - a^2) * sigmoid(Ri u + bi) * u with
    block-diagonal Ra, Ri [blocks, bw, bw]; u fp32 [T, width]; both results fp32 (csrc/rglru.cu)."""
    _chk(u, "recurrent input", torch.float32, 2)
    _chk(ra, "recurrence gate weights", dim=3)
    _chk(ri, "input gate weights", ra.dtype, 3)
    T, width = u.shape
    blocks, bw, _ = ra.shape
    if tuple(ra.shape) != (blocks, bw, bw) or ri.shape != ra.shape or blocks * bw != width:
        raise KernelError("rglru_gates: the gates' matrices do not fit the channels")
    for t, n in ((ba, "recurrence gate bias"), (bi, "input gate bias"), (lam, "decay parameter")):
        _chk(t, n, ba.dtype)
        if t.numel() != width:
            raise KernelError(f"rglru_gates: {n} does not fit the channels")
    a = torch.empty((T, width), dtype=torch.float32, device=u.device)
    b = torch.empty((T, width), dtype=torch.float32, device=u.device)
    call("mynah_rglru_gates", ptr(u), ptr(ra), ptr(ri), code(ra.dtype), ptr(ba), ptr(bi), ptr(lam), code(ba.dtype),
         float(decay_scale), ptr(a), ptr(b), T, width, blocks, stream_ptr())
    return a, b


def rglru_scan(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, state: torch.Tensor, ctx) -> torch.Tensor:
    """S <- a S + b along each sequence of the step, S fp32 per slot ([max_seqs + 1, width]); returns S * y in y's type."""
    _chk(a, "decay", torch.float32, 2)
    _chk(b, "input", torch.float32, 2)
    _chk(y, "gate branch", dim=2)
    _chk(state, "recurrent state", torch.float32, 2)
    T, width = a.shape
    if b.shape != a.shape or y.shape != a.shape or state.shape[1] != width:
        raise KernelError("rglru_scan: shapes differ")
    out = torch.empty((T, width), dtype=y.dtype, device=y.device)
    call("mynah_rglru_scan", ptr(a), ptr(b), ptr(y), code(y.dtype), ptr(state), state.shape[0] - 1, ptr(out), ptr(ctx.cu_q),
         ptr(ctx.slots), ctx.B, width, int(ctx.max_q_len), stream_ptr())
    return out


def sink_attn_prep(qkv: torch.Tensor, q_out: torch.Tensor, k_cache, v_cache, cos_k, sin_k, cos_v: torch.Tensor,
                   sin_v: torch.Tensor, ctx, pages: PageTableView, H: int, G: int, dim: int, vd: int, rot: int,
                   interleaved: bool) -> None:
    """Rotates q and k over their first `rot` dimensions and v over all of its own, writes k and v to the cache pages
    and q to q_out (csrc/sink_attn.cu). k_cache None: only the queries."""
    _rows(qkv, "sink_attn_prep: projection")
    _chk(q_out, "q", qkv.dtype, 2)
    if qkv.shape[1] < H * dim + (G * (dim + vd) if k_cache is not None else 0) or q_out.shape[1] != H * dim:
        raise KernelError("sink_attn_prep: the projection's rows are too short")
    if k_cache is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("sink_attn_prep: the cache and the activations differ in dtype")
        if tuple(k_cache.shape[1:]) != (G, PAGE_TOKENS, dim) or tuple(v_cache.shape[1:]) != (G, PAGE_TOKENS, vd):
            raise KernelError("sink_attn_prep: the cache pages do not have the head sizes")
    _chk(cos_v, "value rotation table", torch.float32, 2)
    if cos_v.shape[1] != vd // 2 or (rot and (cos_k is None or cos_k.shape[1] != rot // 2)):
        raise KernelError("sink_attn_prep: the rotation tables do not fit")
    call("mynah_sink_attn_prep", ptr(qkv), qkv.stride(0), code(qkv.dtype), ptr(q_out), ptr(k_cache), ptr(v_cache),
         ptr(cos_k), ptr(sin_k), cos_k.shape[0] if cos_k is not None else 0, ptr(cos_v), ptr(sin_v), cos_v.shape[0],
         ptr(ctx.tok_seq), ptr(ctx.tok_pos), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         qkv.shape[0], H, G, dim, vd, rot, 1 if interleaved else 0, ptr(ctx.status), stream_ptr())


def sink_attn(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, talk: torch.Tensor,
              sink: torch.Tensor, cos_v: torch.Tensor, sin_v: torch.Tensor, ctx, pages: PageTableView, H: int, G: int,
              dim: int, vd: int, window: int, scale: float, interleaved: bool) -> None:
    """Windowed softmax attention whose denominator holds exp(sink_h), whose heads' weights are mixed by talk [H, H]
    after the softmax, and whose values are rotated in the cache and turned back at the query (csrc/sink_attn.cu)."""
    _chk(q, "q", dim=2)
    _chk(out, "attention output", q.dtype, 2)
    _chk(talk, "head mixing matrix", dim=2)
    _chk(sink, "sinks", talk.dtype, 1)
    if tuple(talk.shape) != (H, H) or sink.numel() != H or q.shape[1] != H * dim or out.shape[1] != H * vd:
        raise KernelError("sink_attn: sizes do not fit")
    call("mynah_sink_attn", ptr(q), ptr(out), code(q.dtype), ptr(k_cache), ptr(v_cache), ptr(talk), ptr(sink),
         code(talk.dtype), ptr(cos_v), ptr(sin_v), cos_v.shape[0], ptr(ctx.tok_seq), ptr(ctx.tok_pos), ptr(pages.indptr),
         ptr(pages.ids), ptr(pages.base), pages.n_pages, q.shape[0], H, G, dim, vd, int(window or 0), float(scale),
         1 if interleaved else 0, ptr(ctx.status), stream_ptr())


def sink_attn_tc_supported(dtype: torch.dtype, H: int, G: int, dim: int, vd: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib.load().mynah_sink_attn_tc_supported(H, G, dim, vd))


def sink_attn_tc_scratch(T: int, H: int, vd: int, splits: int) -> int:
    """fp32 words of scratch: every share's (maximum, sum) of the denominators [splits, T, H, 2], and the shares' partial
    sums when there are several."""
    return 2 * splits * T * H + (splits * T * H * vd if splits > 1 else 0)


def sink_attn_tc(q: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 talk: torch.Tensor, sink: torch.Tensor, cos_v: torch.Tensor, sin_v: torch.Tensor, ctx, pages: PageTableView,
                 H: int, G: int, dim: int, vd: int, window: int, scale: float, interleaved: bool, splits: int) -> None:
    """sink_attn on tensor cores (bfloat16, heads of 64 or 128; csrc/sink_attn_tc.cu): the denominators first, then one
    pass over the keys that mixes the heads' weights and multiplies with V, the keys in `splits` shares."""
    _chk(q, "q", torch.bfloat16, 2)
    _chk(out, "attention output", torch.bfloat16, 2)
    _chk(talk, "head mixing matrix", dim=2)
    _chk(sink, "sinks", talk.dtype, 1)
    _chk(scratch, "scratch", torch.float32, 1)
    T = q.shape[0]
    if tuple(talk.shape) != (H, H) or sink.numel() != H or q.shape[1] != H * dim or tuple(out.shape) != (T, H * vd):
        raise KernelError("sink_attn_tc: sizes do not fit")
    if k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise KernelError("sink_attn_tc: the cache is not bfloat16")
    if tuple(k_cache.shape[1:]) != (G, PAGE_TOKENS, dim) or tuple(v_cache.shape[1:]) != (G, PAGE_TOKENS, vd):
        raise KernelError("sink_attn_tc: the cache pages do not have the head sizes")
    if scratch.numel() < sink_attn_tc_scratch(T, H, vd, splits):
        raise KernelError("sink_attn_tc: scratch too small")
    part = scratch[2 * splits * T * H:] if splits > 1 else None
    call("mynah_sink_attn_tc", ptr(q), ptr(out), ptr(scratch), ptr(part), ptr(k_cache), ptr(v_cache), ptr(talk), ptr(sink),
         code(talk.dtype), ptr(cos_v), ptr(sin_v), cos_v.shape[0], ptr(ctx.cu_q), ptr(ctx.kv_len), ptr(ctx.tok_seq),
         ptr(ctx.tok_pos), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, T, ctx.B, H, G, dim, vd,
         int(window or 0), float(scale), 1 if interleaved else 0, int(splits), ptr(ctx.status), stream_ptr())


# ------------------------------------------------------------------ capped / differential attention, gated heads
def capped_attn_prep(qkv: torch.Tensor, q_out: torch.Tensor, Hq: int, Gk: int, Gv: int, dim: int, vd: int, dimp: int, vdp: int,
                     maps: int, R: int, bias: Optional[torch.Tensor], q_gain: Optional[torch.Tensor],
                     k_gain: Optional[torch.Tensor], eps: float, cos, sin, rot: int, interleaved: bool, ctx,
                     pages: PageTableView, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor]) -> None:
    """Bias, per-unit RMS norm, rotation, packed queries and cache write of grouped-query attention with `maps`
    score maps a head (csrc/capped_attn.cu). qkv: the projection's rows; q_out [T, Hq * dimp]."""
    _rows(qkv, "capped_attn_prep: projection")
    _chk(q_out, "packed queries", qkv.dtype, 2)
    writes = k_cache is not None
    need = Hq * dim + ((Gk * dim + Gv * vd) if writes else 0)
    if qkv.shape[1] < need or q_out.shape[1] != Hq * dimp:
        raise KernelError("capped_attn_prep: the rows do not fit the heads")
    if bias is not None:
        _chk(bias, "projection bias", torch.float32, 1)
        if bias.numel() < need:
            raise KernelError("capped_attn_prep: the bias is shorter than the projection")
    gd = 0
    if q_gain is not None:
        if k_gain is None or q_gain.dtype != k_gain.dtype or q_gain.numel() != dim or k_gain.numel() != dim:
            raise KernelError("capped_attn_prep: the two gains must have `dim` values of one dtype")
        gd = code(q_gain.dtype)
    if writes:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
            raise KernelError("capped_attn_prep: the cache and the activations differ in dtype")
        if tuple(k_cache.shape[1:]) != (Gk, PAGE_TOKENS, dimp) or tuple(v_cache.shape[1:]) != (Gv, PAGE_TOKENS, vdp):
            raise KernelError("capped_attn_prep: the cache pages do not have the stored head sizes")
    n_pos = cos.shape[0] if cos is not None else 0
    if cos is not None and cos.shape[1] * 2 != rot:
        raise KernelError("capped_attn_prep: the rotation table does not match the rotated dims")
    call("mynah_capped_attn_prep", ptr(qkv), code(qkv.dtype), qkv.shape[0], qkv.stride(0), ptr(q_out), q_out.shape[1], Hq, Gk, Gv,
         dim, vd, dimp, vdp, maps, R, ptr(bias), ptr(q_gain), ptr(k_gain), gd, float(eps), ptr(cos), ptr(sin),
         rot if cos is not None else 0, 1 if interleaved else 0, n_pos, ptr(ctx.tok_seq), ptr(ctx.tok_pos),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, ptr(k_cache), ptr(v_cache), ptr(ctx.status),
         stream_ptr())


def attn_prefill_capped(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, VD: int, k_cache, v_cache,
                        pages: PageTableView, window: int, scale: float, softcap: float, keep_first: int, vdiv: int) -> None:
    """The general prompt attention with capped scores, first tokens that the window keeps, and `vdiv` key heads on
    one value head."""
    _chk(q, "q", dim=2)
    _chk(out, "attention output", q.dtype, 2)
    call("mynah_attn_prefill_generic_capped", ptr(q), ptr(out), code(q.dtype), q.shape[0], ctx.B, ctx.max_q_len, H, KV, HD, VD,
         q.shape[1], out.shape[1], ptr(k_cache), ptr(v_cache), ptr(ctx.cu_q), ptr(ctx.kv_len),
         ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages, window or 0, 0, float(scale), float(softcap or 0.0),
         int(keep_first or 0), int(vdiv), ptr(ctx.status), stream_ptr())


def attn_prefill_tcgen05_capped(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, k_cache: torch.Tensor,
                                v_cache: torch.Tensor, pages: PageTableView, window: int, scale: float, softcap: float,
                                keep_first: int, vdiv: int) -> None:
    """The tcgen05 prompt attention with capped scores, first tokens that the window keeps (the page lists must hold
    every page: a cache that gives pages back does not go with kept tokens) and `vdiv` key heads on one value head."""
    for t, n in ((q, "q"), (out, "attention output")):
        _rows(t, "attn_prefill_tcgen05: " + n)
        if t.dtype != torch.bfloat16 or t.stride(0) % 8 or t.data_ptr() % 16:
            raise KernelError(f"attn_prefill_tcgen05: {n} must be bfloat16 rows, 16-byte aligned")
    _chk(k_cache, "K cache", torch.bfloat16)
    _chk(v_cache, "V cache", torch.bfloat16)
    call("mynah_attn_prefill_tcgen05_capped", ptr(q), ptr(out), q.shape[0], ctx.B, ctx.max_q_len, H, KV, HD, q.stride(0),
         out.stride(0), ptr(k_cache), ptr(v_cache), ptr(ctx.cu_q), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids),
         ptr(pages.base), pages.n_pages, window or 0, 0, float(scale), float(softcap or 0.0), int(keep_first or 0), int(vdiv),
         ptr(ctx.status), stream_ptr())


def attn_decode_tc_capped(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, k_cache: torch.Tensor,
                          v_cache: torch.Tensor, pages: PageTableView, window: int, scale: float, softcap: float,
                          keep_first: int, vdiv: int, scratch: torch.Tensor) -> None:
    """The tensor-core decode attention with capped scores, first tokens that the window keeps (the page lists must hold
    every page) and `vdiv` key heads on one value head."""
    for t, n in ((q, "q"), (out, "attention output")):
        _rows(t, "attn_decode_tc: " + n)
        if t.dtype != torch.bfloat16 or t.stride(0) % 8 or t.data_ptr() % 16:
            raise KernelError(f"attn_decode_tc: {n} must be bfloat16 rows, 16-byte aligned")
    _chk(scratch, "scratch", torch.float32)
    need = ctx.B * H * ctx.decode_splits * (HD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode_tc: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_tc_capped", ptr(q), ptr(out), ctx.B, H, KV, HD, q.stride(0), out.stride(0),
         ptr(k_cache), ptr(v_cache), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, 0, float(scale), float(softcap or 0.0), int(keep_first or 0), int(vdiv), ctx.decode_splits,
         ptr(scratch), None, ptr(ctx.status), stream_ptr())
    lib.add_launches(1)        # pages and their merge


def attn_decode_capped(q: torch.Tensor, out: torch.Tensor, ctx, H: int, KV: int, HD: int, VD: int, k_cache, v_cache,
                       pages: PageTableView, window: int, scale: float, softcap: float, keep_first: int, vdiv: int,
                       scratch: torch.Tensor) -> None:
    _chk(q, "q", dim=2)
    _chk(out, "attention output", q.dtype, 2)
    _chk(scratch, "scratch", torch.float32)
    need = ctx.B * H * ctx.decode_splits * (VD + 2)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    call("mynah_attn_decode_capped", ptr(q), ptr(out), code(q.dtype), ctx.B, H, KV, HD, VD, q.shape[1], out.shape[1],
         ptr(k_cache), ptr(v_cache), ptr(ctx.kv_len), ptr(pages.indptr), ptr(pages.ids), ptr(pages.base), pages.n_pages,
         window or 0, 0, float(scale), float(softcap or 0.0), int(keep_first or 0), int(vdiv), ctx.decode_splits,
         ptr(scratch), ptr(ctx.status), stream_ptr())
    lib.add_launches(1)        # pages and their combination


def diff_combine(a: torch.Tensor, H: int, R: int, vd: int, vdp: int, lam: float, mult: float, eps: float, ctx) -> torch.Tensor:
    """o_h = unit_rms(a_h,0 - lam * a_h,1) * mult, from the attention's slots (kv head, map, query head of the group) back
    to head order; returns [T, H * vd] in the rows' type."""
    _chk(a, "attention maps", dim=2)
    if a.shape[1] != 2 * H * vdp:
        raise KernelError("diff_combine: the rows do not hold two maps a head")
    out = torch.empty((a.shape[0], H * vd), dtype=a.dtype, device=a.device)
    call("mynah_diff_combine", ptr(a), code(a.dtype), a.shape[0], a.shape[1], ptr(out), out.shape[1], H, R, vd, vdp,
         float(lam), float(mult), float(eps), ptr(ctx.tok_seq), stream_ptr())
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor, H: int, vd: int) -> torch.Tensor:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; gate may be a column slice of wider rows."""
    _chk(x, "heads", dim=2)
    _rows(gate, "head_gate: gate")
    if x.shape[1] != H * vd or gate.shape[1] < H or gate.dtype != x.dtype or gate.shape[0] != x.shape[0]:
        raise KernelError("head_gate: the rows do not fit the heads")
    call("mynah_head_gate", ptr(x), code(x.dtype), x.shape[0], x.shape[1], ptr(gate), gate.stride(0), H, vd, stream_ptr())
    return x


def moe_group_router_ffn(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, w_gu: torch.Tensor,
                         w_down: torch.Tensor, ctx, top: int, groups: int, keep: int, weight_scale: float, limit: float,
                         alpha: float) -> torch.Tensor:
    """Experts picked by sigmoid scores (fp32) with a correction for the choice, inside the `keep` best of `groups` groups of
    neighbouring experts; clamped-gate experts; weights score * weight_scale (csrc/moe.cu). w_router [E, D], correction
    [E], w_gu [E, 2, F, D], w_down [E, D, F]; returns [T, D] in the rows' type."""
    _chk(h, "rows", dim=2)
    _chk(w_router, "router weights", h.dtype, 2)
    _chk(correction, "router correction", dim=1)
    _chk(w_gu, "gate/up weights", h.dtype, 4)
    _chk(w_down, "down weights", h.dtype, 3)
    T, D = h.shape
    E, _, F, _ = w_gu.shape
    if (tuple(w_gu.shape) != (E, 2, F, D) or tuple(w_down.shape) != (E, D, F) or tuple(w_router.shape) != (E, D)
            or correction.numel() != E or not 1 <= top <= E):
        raise KernelError("moe_group_router_ffn: sizes do not fit")
    P_ = T * top
    dev = h.device
    grouped = int(lib.load().mynah_moe_grouped_rows(T, top, E, D, F, code(h.dtype)))
    R = max(P_, grouped)
    out = torch.empty((T, D), dtype=h.dtype, device=dev)
    y = torch.empty((R, F), dtype=h.dtype, device=dev)
    o = torch.empty((R, D), dtype=torch.float32, device=dev)
    a = torch.empty((R, D), dtype=h.dtype, device=dev) if grouped else None
    ints = torch.empty((3 * P_ + 1 + 3 * int(lib.load().mynah_moe_max_tiles(T, top, E)) + R + R // 128 + 1,),
                       dtype=torch.int32, device=dev)
    weights = torch.empty((P_,), dtype=torch.float32, device=dev)
    choice = ints[ints.numel() - P_:]
    call("mynah_moe_group_router_ffn", ptr(h), code(h.dtype), ptr(ctx.tok_seq), ptr(w_router), ptr(correction),
         code(correction.dtype), ptr(w_gu), ptr(w_down), ptr(out), 0, ptr(y), ptr(o), ptr(ints), ptr(a), ptr(choice),
         ptr(weights), T, top, E, D, F, int(groups), int(keep), float(weight_scale), float(limit), float(alpha),
         ptr(ctx.status), stream_ptr())
    lib.add_launches(5 if grouped else 4)     # router, route, (gather,) two products, combine
    return out
