"""Python face of the CUDA kernels, one function per kernel: argument checks, then one ctypes call
per launch.  The kernel tests and the micro-benchmarks call kernels by name through it; the engine
itself launches the same kernels from the host library (core/ops.cpp), which also holds the choice
among kernels that serve one operation.

Every function works on torch CUDA tensors, launches on torch's current stream and returns nothing;
outputs are written into tensors the caller passes.  Sizes a kernel does not take are refused with
UnsupportedShape before anything runs.  There is no other implementation behind these functions:
if the library cannot be built or loaded, the call raises.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Optional

import torch

from ..errors import KernelError, UnsupportedShape  # noqa: F401  (re-exported)
from .build import load_library

F32, BF16 = 0, 1
# Up to this many rows a bfloat16 product goes to the weight-streaming kernel, above it to tcgen05.
SKINNY_MAX_ROWS = 64
ACT_CODES = {None: 0, "none": 0, "gelu_new": 1, "gelu_tanh": 1, "gelu": 2, "gelu_erf": 2}


@dataclasses.dataclass
class FusedNorm:
    """A LayerNorm that gemm_skinny runs itself on the float32 rows `x`."""
    x: torch.Tensor
    gamma: torch.Tensor
    beta: Optional[torch.Tensor]
    eps: float


@dataclasses.dataclass
class KVTarget:
    """Where the key/value columns of a fused q/k/v product belong: a layer's cache views
    [num_pages, Hkv, page_size, D] and the step's index arrays."""
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    block_table: torch.Tensor
    token_seq: torch.Tensor
    positions: torch.Tensor
    q_cols: int
    kv_cols: int
    head_dim: int


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise UnsupportedShape(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# Number of kernel launches issued through this module (benchmarks report it).
LAUNCHES = 0

def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code == 0:
        return
    if code == -1:
        raise UnsupportedShape(f"{what}: sizes or dtypes not supported by this kernel")
    if code == -2:
        raise KernelError(f"{what}: bad argument (null pointer or impossible size)")
    raise KernelError(f"{what}: CUDA error {code}")


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors (there is no CPU path)")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------------------
def embed_positions(ids, positions, wte, wpe, out, status=None) -> None:
    """out[t] = wte[ids[t]] + wpe[positions[t]] (wpe may be None)."""
    _cuda(ids, positions, wte, wpe, out)
    _i32(ids, "ids")
    n, width = out.shape
    if wpe is not None:
        _i32(positions, "positions")
        if wpe.dtype != wte.dtype or wpe.shape[1] != width:
            raise KernelError("position table must match the token table in dtype and width")
    if wte.shape[1] != width or not (wte.is_contiguous() and out.is_contiguous()):
        raise KernelError("embed_positions: tables and output must be contiguous and of one width")
    lib = load_library("embed")
    code = lib.sandy_embed_pos(_p(ids), _p(positions), _p(wte), _p(wpe), _p(out),
                               ctypes.c_int(n), ctypes.c_int(width), ctypes.c_int(wte.shape[0]),
                               ctypes.c_int(0 if wpe is None else wpe.shape[0]),
                               ctypes.c_int(_dt(wte)), ctypes.c_int(_dt(out)), _p(status), _stream())
    _check(code, "embed_positions")


def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[r] = LayerNorm(x[rows[r]] if rows is given else x[r])."""
    _cuda(x, gamma, beta, out, rows)
    width = x.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() != n_rows:
            raise KernelError("layernorm: rows and out disagree")
    elif x.shape[0] != n_rows:
        raise KernelError("layernorm: x and out disagree")
    if not (x.is_contiguous() and out.is_contiguous()) or out.shape[-1] != width or gamma.numel() != width:
        raise KernelError("layernorm: contiguous [rows, width] tensors expected")
    lib = load_library("norm")
    code = lib.sandy_layernorm(_p(x), _p(gamma), _p(beta), _p(out), _p(rows), ctypes.c_int(n_rows),
                               ctypes.c_int(width), ctypes.c_float(eps), ctypes.c_int(_dt(x)),
                               ctypes.c_int(_dt(gamma)), ctypes.c_int(_dt(out)), _stream())
    _check(code, f"layernorm(width={width})")


def gemm_simt(a, w, bias, out, *, w_out_in: bool, act=None, residual=None) -> None:
    """out = act(a @ W + bias) + residual on the 32-bit pipes.  W is [K,N], or [N,K] with w_out_in."""
    _cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = out.shape[1]
    wk, wn = (w.shape[1], w.shape[0]) if w_out_in else (w.shape[0], w.shape[1])
    if wk != K or wn != N or out.shape[0] != M:
        raise KernelError(f"gemm: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)} "
                          f"({'out_in' if w_out_in else 'in_out'}), out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: innermost stride must be 1")
    if residual is not None and (residual.dtype != torch.float32 or residual.stride(1) != 1
                                 or tuple(residual.shape) != (M, N)):
        raise KernelError("gemm: residual must be float32 [M, N]")
    if bias is not None and (bias.dtype != w.dtype or bias.numel() != N):
        raise KernelError("gemm: bias must have the weight's dtype and N elements")
    lib = load_library("gemm_simt")
    code = lib.sandy_gemm_simt(_p(a), _p(w), _p(bias), _p(residual), _p(out),
                               ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                               ctypes.c_int(a.stride(0)), ctypes.c_int(w.stride(0)),
                               ctypes.c_int(0 if residual is None else residual.stride(0)),
                               ctypes.c_int(out.stride(0)), ctypes.c_int(1 if w_out_in else 0),
                               ctypes.c_int(ACT_CODES[act]), ctypes.c_int(_dt(a)), ctypes.c_int(_dt(w)),
                               ctypes.c_int(_dt(out)), _stream())
    _check(code, f"gemm_simt(M={M},N={N},K={K},{a.dtype}->{out.dtype})")


def _cache_args(k_cache, v_cache):
    """k_cache, v_cache: [num_pages, Hkv, page_size, D] views with one page stride."""
    if k_cache.shape != v_cache.shape or k_cache.dtype != v_cache.dtype or k_cache.dim() != 4:
        raise KernelError("cache views must be [num_pages, Hkv, page_size, D], K and V alike")
    _, hkv, ps, d = k_cache.shape
    want = (k_cache.stride(0), ps * d, d, 1)
    if tuple(k_cache.stride()) != want or tuple(v_cache.stride()) != want:
        raise KernelError("cache views must be dense inside a page")
    return hkv, ps, d, k_cache.stride(0), k_cache.shape[0]


def kv_append(k_src, v_src, k_cache, v_cache, block_table, token_seq, positions) -> None:
    """Write the step's keys/values ([T, Hkv*D] views, one row stride) into their pages."""
    _cuda(k_src, v_src, k_cache, v_cache, block_table, token_seq, positions)
    hkv, ps, d, page_stride, num_pages = _cache_args(k_cache, v_cache)
    T = k_src.shape[0]
    if k_src.shape != v_src.shape or k_src.shape[1] != hkv * d or k_src.stride() != v_src.stride() \
            or k_src.stride(1) != 1 or k_src.dtype != k_cache.dtype:
        raise KernelError("kv_append: sources must be [T, Hkv*D] of the cache's dtype with one stride")
    _i32(block_table, "block_table"); _i32(token_seq, "token_seq"); _i32(positions, "positions")
    lib = load_library("attention")
    code = lib.sandy_kv_append(_p(k_src), _p(v_src), ctypes.c_int(k_src.stride(0)), _p(k_cache), _p(v_cache),
                               ctypes.c_longlong(page_stride), _p(block_table), ctypes.c_int(block_table.shape[1]),
                               _p(token_seq), _p(positions), ctypes.c_int(T), ctypes.c_int(hkv), ctypes.c_int(d),
                               ctypes.c_int(ps), ctypes.c_int(num_pages), ctypes.c_int(_dt(k_cache)),
                               _p(kernel_status(k_cache.device)), _stream())
    _check(code, "kv_append")


def paged_attention(q, k_cache, v_cache, block_table, token_seq, positions, out, *, sink=None, out_gate=None,
                    n_heads: int, scale: float, window: int = 0, softcap: float = 0.0, chunk: int = 0, dist_bias=None) -> None:
    """Causal attention of every token of the step over its request's pages (general kernel).  softcap > 0 presses
    every score into softcap * tanh(score / softcap); chunk > 0 lets a query see the keys of its own chunk of
    positions only; dist_bias (float32 [H, n_dist]) adds entry min(i - j, n_dist - 1) of the head's row to the score of
    query i and key j."""
    _cuda(q, k_cache, v_cache, block_table, token_seq, positions, out)
    hkv, ps, d, page_stride, num_pages = _cache_args(k_cache, v_cache)
    T = q.shape[0]
    if d % 16 != 0 or d > 640:
        raise UnsupportedShape(f"attention: head size {d} must be a multiple of 16, at most 640")
    if n_heads % hkv != 0:
        raise UnsupportedShape(f"attention: {n_heads} heads do not divide into {hkv} key/value heads")
    if q.shape[1] != n_heads * d or out.shape != q.shape or q.stride(1) != 1 or out.stride(1) != 1 \
            or q.dtype != k_cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, H*D] of the cache's dtype")
    _i32(block_table, "block_table"); _i32(token_seq, "token_seq"); _i32(positions, "positions")
    lib = load_library("attention")
    code = lib.sandy_paged_attention_bias(_p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache),
                                     ctypes.c_longlong(page_stride), _p(block_table),
                                     ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out),
                                     ctypes.c_int(out.stride(0)), ctypes.c_int(T), ctypes.c_int(n_heads),
                                     ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(ps), ctypes.c_float(scale),
                                     ctypes.c_int(window), ctypes.c_float(softcap), ctypes.c_int(chunk),
                                     ctypes.c_int(num_pages), ctypes.c_int(_dt(q)),
                                     _p(sink), _p(out_gate), *_bias_args(dist_bias, n_heads), _p(kernel_status(q.device)), _stream())
    _check(code, f"paged_attention(H={n_heads},Hkv={hkv},D={d})")


def _bias_args(dist_bias, n_heads: int):
    if dist_bias is None:
        return None, ctypes.c_int(0)
    if dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[0] != n_heads or not dist_bias.is_contiguous():
        raise KernelError("attention: a bias by distance is a dense float32 [H, n_dist]")
    return _p(dist_bias), ctypes.c_int(dist_bias.shape[1])


_DECODE_HEAD_DIMS = {torch.bfloat16: (16, 32, 64, 128, 256), torch.float32: (16, 32, 64, 128)}


def decode_splits(n_tokens: int, n_heads: int, max_kv: int, sms: Optional[int] = None) -> int:
    """How many blocks share the keys of one (token, head) pair in a decode step (the host library's
    rule, core/ops.cpp): about four blocks an SM in all, more where a block would walk more than some 256
    keys alone (up to eight an SM), no block with fewer than 64 keys, and never a cluster of 6 or 7 blocks."""
    from .. import core

    return core.call("global", None, "decode_splits", n_tokens=n_tokens, n_heads=n_heads, max_kv=max_kv, sms=sms or 0)


CLUSTER_MAX_SPLITS = 8


def decode_attention(q, k_cache, v_cache, block_table, token_seq, positions, out, *, n_heads: int,
                     scale: float, window: int = 0, num_splits: int = 1, scratch=None, cluster: bool = False,
                     bulk: bool = False, mma: bool = False, sink=None, out_gate=None) -> None:
    """Split-KV attention of single tokens (head sizes 16/32/64/128, 256 in bfloat16).  With
    `cluster` (2..8 splits) the splits merge through distributed shared memory inside one
    kernel; otherwise they go through `scratch` and a merge kernel.  `bulk` (at most 8 splits)
    runs the variant that streams whole pages into shared memory with bulk copies, which is
    the faster one when there are hundreds of (token, head) pairs.  `mma` (bfloat16, heads of 64, at
    most 8 splits) runs the variant whose products are mma.sync instructions."""
    _cuda(q, k_cache, v_cache, block_table, token_seq, positions, out, scratch)
    hkv, ps, d, page_stride, num_pages = _cache_args(k_cache, v_cache)
    T = q.shape[0]
    if d not in _DECODE_HEAD_DIMS.get(q.dtype, ()):
        raise UnsupportedShape(f"decode_attention: head size {d} in {q.dtype} is not supported by this kernel")
    if n_heads % hkv != 0:
        raise UnsupportedShape(f"attention: {n_heads} heads do not divide into {hkv} key/value heads")
    if q.shape[1] != n_heads * d or out.shape != q.shape or q.stride(1) != 1 or out.stride(1) != 1 \
            or q.dtype != k_cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, H*D] of the cache's dtype")
    _i32(block_table, "block_table"); _i32(token_seq, "token_seq"); _i32(positions, "positions")
    if mma:
        if q.dtype != torch.bfloat16 or d != 64:
            raise UnsupportedShape("decode_attention: the mma.sync kernel takes bfloat16 heads of 64")
        if num_splits > CLUSTER_MAX_SPLITS:
            raise UnsupportedShape(f"decode_attention: a cluster holds at most {CLUSTER_MAX_SPLITS} splits")
        lib = load_library("attention_decode_mma")
        code = lib.sandy_decode_attention_mma_ext(
            _p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache), ctypes.c_longlong(page_stride),
            _p(block_table), ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out),
            ctypes.c_int(out.stride(0)), ctypes.c_int(T), ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d),
            ctypes.c_int(ps), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(num_splits),
            ctypes.c_int(num_pages), ctypes.c_int(block_table.shape[1] * ps), _p(sink), _p(out_gate), _p(kernel_status(q.device)), _stream())
        _check(code, f"decode_attention_mma(H={n_heads},Hkv={hkv},page={ps},splits={num_splits})")
        return
    if bulk:
        if num_splits > CLUSTER_MAX_SPLITS:
            raise UnsupportedShape(f"decode_attention: a cluster holds at most {CLUSTER_MAX_SPLITS} splits")
        lib = load_library("attention_decode_bulk")
        code = lib.sandy_decode_attention_bulk_ext(
            _p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache), ctypes.c_longlong(page_stride),
            _p(block_table), ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out),
            ctypes.c_int(out.stride(0)), ctypes.c_int(T), ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d),
            ctypes.c_int(ps), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(num_splits),
            ctypes.c_int(num_pages), ctypes.c_int(_dt(q)), _p(sink), _p(out_gate), _p(kernel_status(q.device)), _stream())
        _check(code, f"decode_attention_bulk(H={n_heads},Hkv={hkv},D={d},page={ps},splits={num_splits})")
        return
    if cluster and num_splits > 1:
        if num_splits > CLUSTER_MAX_SPLITS:
            raise UnsupportedShape(f"decode_attention: a cluster holds at most {CLUSTER_MAX_SPLITS} splits")
        lib = load_library("attention_decode")
        code = lib.sandy_decode_attention_cluster_ext(
            _p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache), ctypes.c_longlong(page_stride),
            _p(block_table), ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out),
            ctypes.c_int(out.stride(0)), ctypes.c_int(T), ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d),
            ctypes.c_int(ps), ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_int(num_splits),
            ctypes.c_int(num_pages), ctypes.c_int(_dt(q)), _p(sink), _p(out_gate), _p(kernel_status(q.device)), _stream())
        _check(code, f"decode_attention_cluster(H={n_heads},Hkv={hkv},D={d},splits={num_splits})")
        return
    need = T * n_heads * num_splits * (d + 2) if num_splits > 1 else 0
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need
                 or not scratch.is_contiguous()):
        raise KernelError(f"decode_attention: {num_splits} splits need a float32 scratch of {need} elements")
    lib = load_library("attention_decode")
    code = lib.sandy_decode_attention_ext(_p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache),
                                      ctypes.c_longlong(page_stride), _p(block_table),
                                      ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out),
                                      ctypes.c_int(out.stride(0)), _p(scratch), ctypes.c_int(T), ctypes.c_int(n_heads),
                                      ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(ps), ctypes.c_float(scale),
                                      ctypes.c_int(window), ctypes.c_int(num_splits), ctypes.c_int(num_pages),
                                      ctypes.c_int(_dt(q)), _p(sink), _p(out_gate), _p(kernel_status(q.device)), _stream())
    _check(code, f"decode_attention(H={n_heads},Hkv={hkv},D={d},splits={num_splits})")
    if num_splits > 1:
        global LAUNCHES
        LAUNCHES += 1


def decode_attention_shared(q, k_cache, v_cache, block_table, token_seq, positions, out, *, n_heads: int, scale: float, splits: int = 1,
                            window: int = 0, sink=None, out_gate=None, softcap: float = 0.0, chunk: int = 0, dist_bias=None) -> None:
    """Single-token attention with the query heads of a group as the rows of one tensor-core product (bfloat16, head sizes
    up to 128); v_cache may be k_cache itself (one plane).  softcap, chunk and dist_bias as in paged_attention."""
    _cuda(q, k_cache, v_cache, block_table, token_seq, positions, out)
    hkv, ps, d, page_stride, num_pages = _cache_args(k_cache, v_cache)
    T = q.shape[0]
    lib = load_library("attention_decode_shared")
    lib.sandy_decode_attention_shared_scratch.restype = ctypes.c_longlong
    floats = lib.sandy_decode_attention_shared_scratch(ctypes.c_int(T), ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(splits))
    scratch = torch.empty(max(int(floats), 1), dtype=torch.float32, device=q.device)
    code = lib.sandy_decode_attention_shared_bias(
        _p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache), ctypes.c_longlong(page_stride), _p(block_table),
        ctypes.c_int(block_table.shape[1]), _p(token_seq), _p(positions), _p(out), ctypes.c_int(out.stride(0)), ctypes.c_int(T),
        ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(ps), ctypes.c_float(scale), ctypes.c_int(window),
        ctypes.c_float(softcap), ctypes.c_int(chunk), ctypes.c_int(splits), ctypes.c_int(num_pages), _p(sink), _p(out_gate),
        *_bias_args(dist_bias, n_heads), _p(scratch), _p(kernel_status(q.device)), _stream())
    _check(code, f"decode_attention_shared(H={n_heads},Hkv={hkv},D={d})")


def prefill_attention(q, k_cache, v_cache, block_table, q_start, kv_before, out, *, sink=None, out_gate=None, n_heads: int,
                      max_q_len: int, scale: float, window: int = 0, tc=None, softcap: float = 0.0, chunk: int = 0,
                      dist_bias=None) -> None:
    """Tensor-core attention of prompt portions (bfloat16, head sizes 16..128 in steps of 16).
    q_start: int32 [S+1] first new token of each request; kv_before: int32 [S].
    tc: True asks for the tcgen05 kernel (heads of 64), False for the mma.sync kernel, None
    picks the tcgen05 kernel where it takes the shape.  softcap and chunk as in paged_attention; both kernels
    have the form for them.  dist_bias as in paged_attention: the mma.sync kernel alone has the form for it."""
    _cuda(q, k_cache, v_cache, block_table, q_start, kv_before, out, sink, out_gate)
    hkv, ps, d, page_stride, num_pages = _cache_args(k_cache, v_cache)
    if q.dtype != torch.bfloat16 or d % 16 != 0 or d > 128:
        raise UnsupportedShape(f"prefill_attention: bfloat16 and head sizes 16..128 only, got {q.dtype}, {d}")
    if n_heads % hkv != 0:
        raise UnsupportedShape(f"attention: {n_heads} heads do not divide into {hkv} key/value heads")
    if q.shape[1] != n_heads * d or out.shape != q.shape or q.stride(1) != 1 or out.stride(1) != 1 \
            or q.dtype != k_cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, H*D] of the cache's dtype")
    _i32(block_table, "block_table"); _i32(q_start, "q_start"); _i32(kv_before, "kv_before")
    S = kv_before.numel()
    if q_start.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("prefill_attention: q_start, kv_before and block_table disagree on the requests")
    args = (_p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache), ctypes.c_longlong(page_stride),
            _p(block_table), ctypes.c_int(block_table.shape[1]), _p(q_start), _p(kv_before), _p(out),
            ctypes.c_int(out.stride(0)), ctypes.c_int(S), ctypes.c_int(max_q_len), ctypes.c_int(n_heads),
            ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(ps), ctypes.c_float(scale), ctypes.c_int(window),
            ctypes.c_float(softcap), ctypes.c_int(chunk),
            ctypes.c_int(num_pages), _p(sink), _p(out_gate), _p(kernel_status(q.device)), _stream())
    if dist_bias is not None and tc:
        raise UnsupportedShape("prefill_attention: the tcgen05 kernel takes no bias by distance")
    if tc or (tc is None and d == 64 and dist_bias is None):
        code = load_library("attention_prefill_tc").sandy_prefill_attention_tc_cap(*args)
        if code != -1 or tc:
            _check(code, f"prefill_attention_tc(H={n_heads},Hkv={hkv},D={d})")
            return
    lib = load_library("attention_prefill")
    code = lib.sandy_prefill_attention_bias(_p(q), ctypes.c_int(q.stride(0)), _p(k_cache), _p(v_cache),
                                       ctypes.c_longlong(page_stride), _p(block_table),
                                       ctypes.c_int(block_table.shape[1]), _p(q_start), _p(kv_before), _p(out),
                                       ctypes.c_int(out.stride(0)), ctypes.c_int(S), ctypes.c_int(max_q_len),
                                       ctypes.c_int(n_heads), ctypes.c_int(hkv), ctypes.c_int(d), ctypes.c_int(ps),
                                       ctypes.c_float(scale), ctypes.c_int(window), ctypes.c_float(softcap),
                                       ctypes.c_int(chunk), ctypes.c_int(num_pages),
                                       _p(sink), _p(out_gate), *_bias_args(dist_bias, n_heads), _p(kernel_status(q.device)), _stream())
    _check(code, f"prefill_attention(H={n_heads},Hkv={hkv},D={d})")


def _f32(t, name: str) -> None:
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous float32 tensor")


def rmsnorm(x, gain, eps: float, out, rows=None) -> None:
    """out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * gain; x float32 [*, width], gain float32 [width] or None."""
    _cuda(x, gain, out, rows)
    _f32(x, "x"); _f32(gain, "gain")
    n_rows = out.shape[0]
    code = load_library("rmsnorm").sandy_rmsnorm(_p(x), ctypes.c_int(x.stride(0)), _p(gain), _p(out), ctypes.c_int(out.stride(0)),
                                                 _p(rows), ctypes.c_int(n_rows), ctypes.c_int(x.shape[1]), ctypes.c_float(eps),
                                                 ctypes.c_int(_dt(out)), _stream())
    _check(code, f"rmsnorm(width={x.shape[1]})")


def rmsnorm_add(y, gain, eps: float, mult: float, x) -> None:
    """x += mult * y / sqrt(mean(y^2) + eps) * gain, both float32."""
    _cuda(x, gain, y)
    _f32(x, "x"); _f32(y, "y"); _f32(gain, "gain")
    code = load_library("rmsnorm").sandy_rmsnorm_add(_p(y), ctypes.c_int(y.stride(0)), _p(gain), _p(x), ctypes.c_int(x.stride(0)),
                                                     ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]), ctypes.c_float(eps),
                                                     ctypes.c_float(mult), _stream())
    _check(code, f"rmsnorm_add(width={x.shape[1]})")


def head_norm_gate(o, gain, gate, out, *, n_heads: int, eps: float, act: str = "sigmoid", scale: float = 1.0) -> None:
    """Per (token, head): out = o / rms(o over the head) * gain * act(gate) * scale.  o float32 [T, H * dim]; gain
    float32 [dim] (shared) or [H * dim]; gate [T, H * dim] or None; act "sigmoid" | "silu"."""
    _cuda(o, gain, gate, out)
    _f32(o, "o"); _f32(gain, "gain")
    dim = o.shape[1] // n_heads
    stride = dim if (gain is not None and gain.numel() == o.shape[1] and n_heads > 1) else 0
    code = load_library("rmsnorm").sandy_head_norm_gate(
        _p(o), ctypes.c_int(o.stride(0)), _p(gain), ctypes.c_int(stride), _p(gate), ctypes.c_int(0 if gate is None else gate.stride(0)),
        ctypes.c_int(_dt(out) if gate is None else _dt(gate)), _p(out), ctypes.c_int(out.stride(0)), ctypes.c_int(_dt(out)),
        ctypes.c_int(o.shape[0]), ctypes.c_int(n_heads), ctypes.c_int(dim), ctypes.c_float(eps),
        ctypes.c_int({"sigmoid": 0, "silu": 1}[act]), ctypes.c_float(scale), _stream())
    _check(code, f"head_norm_gate(H={n_heads},dim={dim})")


def glu(a, b, out, act: str = "silu") -> None:
    """out = act(a) * b; act "silu" | "gelu_tanh"."""
    _cuda(a, b, out)
    code = load_library("elementwise").sandy_glu(_p(a), _p(b), ctypes.c_int(a.stride(0)), _p(out), ctypes.c_int(out.stride(0)),
                                                 ctypes.c_int(a.shape[0]), ctypes.c_int(a.shape[1]),
                                                 ctypes.c_int({"silu": 0, "gelu_tanh": 1}[act]), ctypes.c_int(_dt(a)), _stream())
    _check(code, "glu")


def glu_clamped(a, b, out, *, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(a, limit) and u = clamp(b, -limit, limit)."""
    _cuda(a, b, out)
    if a.shape != b.shape or a.stride(0) != b.stride(0) or a.dtype != b.dtype or out.dtype != a.dtype:
        raise KernelError("glu_clamped: a and b of one shape, pitch and type expected")
    code = load_library("elementwise").sandy_glu_clamped(_p(a), _p(b), ctypes.c_int(a.stride(0)), _p(out), ctypes.c_int(out.stride(0)),
                                                         ctypes.c_int(a.shape[0]), ctypes.c_int(a.shape[1]), ctypes.c_float(limit),
                                                         ctypes.c_float(alpha), ctypes.c_int(_dt(a)), _stream())
    _check(code, "glu_clamped")


def stream_add(x, x0=None, row=None) -> None:
    """x += x0 (float32 [rows, cols], optional) + row (float32 [cols], optional)."""
    _cuda(x, x0, row)
    for t, n in ((x, "x"), (x0, "x0"), (row, "row")):
        _f32(t, n)
    code = load_library("elementwise").sandy_stream_add(_p(x), ctypes.c_int(x.stride(0)), _p(x0), ctypes.c_int(0 if x0 is None else x0.stride(0)),
                                                        _p(row), ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]), _stream())
    _check(code, "stream_add")


def softcap(x, cap: float) -> None:
    """x <- cap * tanh(x / cap), float32, in place."""
    _cuda(x)
    _f32(x, "x")
    _check(load_library("elementwise").sandy_softcap_f32(_p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()), "softcap")


def rmsnorm_shift(x, gain, mix, state, token_seq, q_start, seq_slots, out, *, eps: float) -> None:
    """Token shift behind an RMS norm: h[t] = x[t] / rms(x[t]) * gain; out[t] = h[t] + (h[t-1] - h[t]) * mix, where the h
    before a request's first token of the step is its row of `state` (float32 [slots, >= width]); afterwards every
    request's row holds the h of its last token."""
    _cuda(x, gain, mix, state, token_seq, q_start, seq_slots, out)
    for t, n in ((x, "x"), (gain, "gain"), (mix, "mix")):
        _f32(t, n)
    _i32(token_seq, "token_seq"); _i32(q_start, "q_start"); _i32(seq_slots, "seq_slots")
    if state.dtype != torch.float32 or state.stride(1) != 1:
        raise KernelError("rmsnorm_shift: state must be float32 rows")
    T, W = x.shape
    S = seq_slots.numel()
    lib = load_library("rmsnorm")
    _check(lib.sandy_rmsnorm_shift(_p(x), ctypes.c_int(x.stride(0)), _p(gain), _p(mix), _p(state), ctypes.c_longlong(state.stride(0)),
                                   _p(token_seq), _p(q_start), _p(seq_slots), _p(out), ctypes.c_int(out.stride(0)), ctypes.c_int(T),
                                   ctypes.c_int(W), ctypes.c_float(eps), ctypes.c_int(_dt(out)), _stream()), "rmsnorm_shift")
    _check(lib.sandy_rmsnorm_keep(_p(x), ctypes.c_int(x.stride(0)), _p(gain), _p(state), ctypes.c_longlong(state.stride(0)), _p(q_start),
                                  _p(seq_slots), ctypes.c_int(S), ctypes.c_int(W), ctypes.c_float(eps), _stream()), "rmsnorm_keep")


def scale_add(y, gain, x, y2=None, gain2=None) -> None:
    """x += gain * y (+ gain2 * y2), all float32; gains are [width]."""
    _cuda(y, gain, x, y2, gain2)
    for t, n in ((y, "y"), (gain, "gain"), (x, "x"), (y2, "y2"), (gain2, "gain2")):
        _f32(t, n)
    code = load_library("elementwise").sandy_scale_add(_p(y), ctypes.c_int(y.stride(0)), _p(gain), _p(y2),
                                                       ctypes.c_int(0 if y2 is None else y2.stride(0)), _p(gain2), _p(x),
                                                       ctypes.c_int(x.stride(0)), ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]),
                                                       _stream())
    _check(code, "scale_add")


def head_product(a, w, out, *, n_groups: int, a_gcols: int, o_gcols: int) -> None:
    """out[t, g * o_gcols + n] = sum_k w[g * N + n, k] * a[t, g * a_gcols + k]: one matrix [N, K] per head, stacked in w."""
    _cuda(a, w, out)
    N, K = w.shape[0] // n_groups, w.shape[1]
    if a.dtype != w.dtype or w.shape[0] % n_groups or not w.is_contiguous() or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_product: a and w of one type, w [G * N, K] contiguous expected")
    code = load_library("grouped_gemm").sandy_head_product(
        _p(a), ctypes.c_int(a.stride(0)), ctypes.c_int(a_gcols), _p(w), ctypes.c_longlong(N * K), ctypes.c_int(K), _p(out),
        ctypes.c_int(out.stride(0)), ctypes.c_int(o_gcols), ctypes.c_int(a.shape[0]), ctypes.c_int(n_groups), ctypes.c_int(N),
        ctypes.c_int(K), ctypes.c_int(_dt(a)), ctypes.c_int(_dt(out)), _stream())
    _check(code, f"head_product(G={n_groups},N={N},K={K})")


@dataclasses.dataclass
class Routing:
    """The routing of a step's tokens to experts, as device arrays (int32 / float32); entry t * top + j is the j-th
    choice of token t."""
    n_tokens: int
    n_experts: int
    top: int
    expert_of: torch.Tensor
    weight_of: torch.Tensor
    group_start: torch.Tensor
    entry_of_slot: torch.Tensor
    slot_of_entry: torch.Tensor


def moe_route(logits, bias, top: int) -> Routing:
    """Top-`top` experts of every token by float32 logits (+ bias), weights the softmax over the chosen; then the
    entries grouped by expert."""
    _cuda(logits, bias)
    _f32(logits, "logits"); _f32(bias, "bias")
    T, E = logits.shape
    dev = logits.device
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
    r = Routing(T, E, top, i32(T * top), torch.empty(T * top, dtype=torch.float32, device=dev), i32(E + 1), i32(T * top), i32(T * top))
    lib = load_library("moe")
    _check(lib.sandy_moe_route(_p(logits), ctypes.c_int(logits.stride(0)), _p(bias), ctypes.c_int(T), ctypes.c_int(E), ctypes.c_int(top),
                               _p(r.expert_of), _p(r.weight_of), _stream()), f"moe_route(E={E},top={top})")
    _check(lib.sandy_moe_group(_p(r.expert_of), ctypes.c_int(T * top), ctypes.c_int(E), _p(r.group_start), _p(r.entry_of_slot),
                               _p(r.slot_of_entry), _stream()), "moe_group")
    return r


def moe_route_scored(logits, correction, top: int, *, n_groups: int = 1, keep_groups: int = 1, group_rank: int = 2,
                     weight_scale: float = 1.0, norm_eps: float = 0.0) -> Routing:
    """Routing by sigmoid scores: choice scores are the scores plus `correction`; experts form `n_groups` groups of
    neighbours, a group's score is the sum of its `group_rank` largest choice scores, only the `keep_groups` best groups
    can be chosen from; the `top` largest choice scores win, weighted by their plain scores over their sum (+ norm_eps)
    times weight_scale.  Then the entries grouped by expert."""
    _cuda(logits, correction)
    _f32(logits, "logits"); _f32(correction, "correction")
    T, E = logits.shape
    dev = logits.device
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
    r = Routing(T, E, top, i32(T * top), torch.empty(T * top, dtype=torch.float32, device=dev), i32(E + 1), i32(T * top), i32(T * top))
    lib = load_library("moe")
    _check(lib.sandy_moe_route_scored(_p(logits), ctypes.c_int(logits.stride(0)), _p(correction), ctypes.c_int(T), ctypes.c_int(E),
                                      ctypes.c_int(top), ctypes.c_int(n_groups), ctypes.c_int(keep_groups), ctypes.c_int(group_rank),
                                      ctypes.c_float(weight_scale), ctypes.c_float(norm_eps), _p(r.expert_of), _p(r.weight_of), _stream()),
           f"moe_route_scored(E={E},top={top},groups={n_groups},keep={keep_groups})")
    _check(lib.sandy_moe_group(_p(r.expert_of), ctypes.c_int(T * top), ctypes.c_int(E), _p(r.group_start), _p(r.entry_of_slot),
                               _p(r.slot_of_entry), _stream()), "moe_group")
    return r


def moe_route_softmax(logits, correction, top: int, *, weight_scale: float = 1.0, norm_eps: float = 0.0, renormalize: bool = False) -> Routing:
    """Routing by softmax scores over all experts: the `top` largest scores plus `correction` win, weighted by their plain
    scores times weight_scale (over their sum + norm_eps only with renormalize).  Then the entries grouped by expert."""
    _cuda(logits, correction)
    _f32(logits, "logits"); _f32(correction, "correction")
    T, E = logits.shape
    dev = logits.device
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
    r = Routing(T, E, top, i32(T * top), torch.empty(T * top, dtype=torch.float32, device=dev), i32(E + 1), i32(T * top), i32(T * top))
    lib = load_library("moe")
    _check(lib.sandy_moe_route_softmax(_p(logits), ctypes.c_int(logits.stride(0)), _p(correction), ctypes.c_int(T), ctypes.c_int(E),
                                       ctypes.c_int(top), ctypes.c_float(weight_scale), ctypes.c_float(norm_eps),
                                       ctypes.c_int(1 if renormalize else 0), _p(r.expert_of), _p(r.weight_of), _stream()),
           f"moe_route_softmax(E={E},top={top})")
    _check(lib.sandy_moe_group(_p(r.expert_of), ctypes.c_int(T * top), ctypes.c_int(E), _p(r.group_start), _p(r.entry_of_slot),
                               _p(r.slot_of_entry), _stream()), "moe_group")
    return r


def expert_product(r: Routing, a, w, out, *, gather: bool, act: str = "none") -> None:
    """out[s] = act(W_e a[row(s)]) for the slots s of every expert e; w [E * N, K]; with `gather` a slot reads its
    token's row of a [T, K], else row s of a [T * top, K].  act "none" | "relu_squared"."""
    _cuda(a, w, out)
    N, K = w.shape[0] // r.n_experts, w.shape[1]
    if a.dtype != w.dtype or not w.is_contiguous() or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("expert_product: a and w of one type, w [E * N, K] contiguous expected")
    code = load_library("grouped_gemm").sandy_expert_product(
        _p(a), ctypes.c_int(a.stride(0)), _p(w), ctypes.c_longlong(N * K), ctypes.c_int(K), _p(out), ctypes.c_int(out.stride(0)),
        ctypes.c_int(r.n_tokens * r.top), ctypes.c_int(r.n_experts), ctypes.c_int(N), ctypes.c_int(K), _p(r.group_start),
        _p(r.entry_of_slot if gather else None), ctypes.c_int(r.top if gather else 1),
        ctypes.c_int({"none": 0, "relu_squared": 1}[act]), ctypes.c_int(_dt(a)), ctypes.c_int(_dt(out)), _stream())
    _check(code, f"expert_product(E={r.n_experts},N={N},K={K})")


def moe_gather(r: Routing, x, out) -> None:
    """out[s] = x[token of slot s]: the tokens' rows in the order of the slots."""
    _cuda(x, out)
    if x.dtype != out.dtype or x.stride(1) != 1 or out.stride(1) != 1 or out.shape != (r.n_tokens * r.top, x.shape[1]):
        raise KernelError("moe_gather: out must be [tokens * top, cols] of x's type")
    es = x.element_size()
    code = load_library("moe").sandy_moe_gather(_p(x), ctypes.c_longlong(x.stride(0) * es), _p(r.entry_of_slot), ctypes.c_int(r.top), _p(out),
                                                ctypes.c_longlong(out.stride(0) * es), ctypes.c_int(out.shape[0]),
                                                ctypes.c_int(x.shape[1] * es), _stream())
    _check(code, "moe_gather")


def expert_product_tc(r: Routing, a_sorted, w, out, *, act: str = "none") -> None:
    """The per-expert product on tcgen05: a_sorted bfloat16 [T * top, K] with every expert's rows one after another
    (moe_gather), w bfloat16 [E * N, K], out [T * top, N] bfloat16 or float32."""
    _cuda(a_sorted, w, out)
    N, K = w.shape[0] // r.n_experts, w.shape[1]
    if a_sorted.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or a_sorted.stride(1) != 1 or out.stride(1) != 1:
        raise UnsupportedShape("expert_product_tc takes bfloat16 operands, w [E * N, K] contiguous")
    code = load_library("grouped_gemm_tc").sandy_expert_product_tc(
        _p(a_sorted), ctypes.c_int(a_sorted.stride(0)), _p(w), ctypes.c_int(K), _p(out), ctypes.c_int(out.stride(0)),
        ctypes.c_int(r.n_tokens * r.top), ctypes.c_int(r.n_experts), ctypes.c_int(N), ctypes.c_int(K), _p(r.group_start),
        ctypes.c_int({"none": 0, "relu_squared": 1}[act]), ctypes.c_int(_dt(out)), _p(kernel_status(out.device)), _stream())
    _check(code, f"expert_product_tc(E={r.n_experts},N={N},K={K})")


def moe_combine(r: Routing, rows, y, *, add: bool) -> None:
    """y[t] (+)= sum_j weight[t, j] * rows[slot of (t, j)]; float32."""
    _cuda(rows, y)
    _f32(rows, "rows"); _f32(y, "y")
    code = load_library("moe").sandy_moe_combine(_p(rows), ctypes.c_int(rows.stride(0)), _p(r.weight_of), _p(r.slot_of_entry),
                                                 ctypes.c_int(r.n_tokens), ctypes.c_int(r.top), _p(y), ctypes.c_int(y.stride(0)),
                                                 ctypes.c_int(y.shape[1]), ctypes.c_int(1 if add else 0), _stream())
    _check(code, "moe_combine")


def moe_combine_identity(r: Routing, n_real: int, h, rows, y, *, add: bool) -> None:
    """moe_combine where the experts from n_real on hand their input on: such an entry contributes weight * h[t]."""
    _cuda(rows, y, h)
    _f32(rows, "rows"); _f32(y, "y")
    code = load_library("moe").sandy_moe_combine_identity(
        _p(rows), ctypes.c_int(rows.stride(0)), _p(r.weight_of), _p(r.slot_of_entry), _p(r.expert_of), ctypes.c_int(n_real), _p(h),
        ctypes.c_int(h.stride(0)), ctypes.c_int(_dt(h)), ctypes.c_int(r.n_tokens), ctypes.c_int(r.top), _p(y), ctypes.c_int(y.stride(0)),
        ctypes.c_int(y.shape[1]), ctypes.c_int(1 if add else 0), _stream())
    _check(code, "moe_combine_identity")


# ---- a residual stream in several copies; a state-space mixer (streams.cu, ssm_state.cu) ---------------------------
def streams_step(X, n_streams: int, *, y=None, gate=None, gate_bias=None, mix=None, out_w=None, in_w=None, gain=None, eps: float = 0.0,
                 h=None, sum_out=None, taps=None, state=None, tail_off: int = 0, token_seq=None, seq_slots=None, conv_out=None) -> None:
    """One pass over the streams X (float32 [T, S * width], in place), each part optional and in this order: the write
    X_t <- sum_s mix[s, t] X_s + out_w[t] * y * sigmoid(gate + gate_bias); sum_out = sum_s X_s; the read
    h = LayerNorm(sum_s in_w[s] X_s) * gain without an offset.  With `taps` (only in a step in which every request brings
    one token): conv_out = h + conv(h) as canon_conv gives it, and the request's tail in `state` moved on by the token."""
    _cuda(X, y, gate, gate_bias, mix, out_w, in_w, gain, h, sum_out, taps, state, token_seq, seq_slots, conv_out)
    T, W = X.shape[0], X.shape[1] // n_streams
    code = load_library("streams").sandy_streams_step_conv(
        _p(X), ctypes.c_int(X.stride(0)), ctypes.c_int(T), ctypes.c_int(n_streams), ctypes.c_int(W), _p(y),
        ctypes.c_int(0 if y is None else y.stride(0)), _p(gate), ctypes.c_int(0 if gate is None else gate.stride(0)), _p(gate_bias),
        _p(mix), _p(out_w), _p(in_w), _p(gain), ctypes.c_float(eps), _p(h), ctypes.c_int(0 if h is None else h.stride(0)),
        ctypes.c_int(0 if h is None else _dt(h)), _p(sum_out), ctypes.c_int(0 if sum_out is None else sum_out.stride(0)),
        _p(taps), ctypes.c_int(0 if taps is None else taps.shape[1]), _p(state), ctypes.c_longlong(0 if state is None else state.stride(0)),
        ctypes.c_longlong(tail_off), _p(token_seq), _p(seq_slots), _p(conv_out), ctypes.c_int(0 if conv_out is None else conv_out.stride(0)),
        _stream())
    _check(code, f"streams_step(S={n_streams},width={W})")


def canon_conv(h, taps, state, tail_off: int, token_seq, q_start, seq_slots, out) -> None:
    """out = h + conv(h): taps float32 [width, n_taps] (the last column the token's own); rows before the step come from
    the request's tail, float32 [n_taps - 1, width] at tail_off of its row of `state` (float32 [slots, row])."""
    _cuda(h, taps, state, token_seq, q_start, seq_slots, out)
    code = load_library("streams").sandy_canon_conv(
        _p(h), ctypes.c_int(h.stride(0)), _p(taps), ctypes.c_int(taps.shape[1]), _p(state), ctypes.c_longlong(state.stride(0)),
        ctypes.c_longlong(tail_off), _p(token_seq), _p(q_start), _p(seq_slots), _p(out), ctypes.c_int(out.stride(0)),
        ctypes.c_int(h.shape[0]), ctypes.c_int(h.shape[1]), ctypes.c_int(_dt(h)), _stream())
    _check(code, "canon_conv")


def conv_tail(rows, n_taps: int, state, tail_off: int, q_start, seq_slots) -> None:
    """The last n_taps - 1 rows of every request (older ones from the old tail) into its tail in `state`."""
    _cuda(rows, state, q_start, seq_slots)
    code = load_library("matrix_state").sandy_conv_tail(
        _p(rows), ctypes.c_int(rows.stride(0)), ctypes.c_int(_dt(rows)), ctypes.c_int(rows.shape[1]), ctypes.c_int(n_taps), _p(state),
        ctypes.c_longlong(state.stride(0)), ctypes.c_longlong(tail_off), _p(q_start), _p(seq_slots), ctypes.c_int(seq_slots.numel()), _stream())
    _check(code, "conv_tail")


def embed_bigram(ids, positions, token_seq, q_start, seq_slots, wte, bigram, wpe, state, out, *, mul_prev: int, mul_cur: int, keep: bool) -> None:
    """out[t] = wte[id] + bigram[(id_before * mul_prev + id * mul_cur) mod buckets] + wpe[pos]; position 0 reads the last row
    of bigram; `state` int32 [slots, >= 1] holds the token before a step's first one; with keep it takes each token (right
    for steps of single tokens), otherwise bigram_keep follows."""
    _cuda(ids, positions, token_seq, q_start, seq_slots, wte, bigram, wpe, state, out)
    lib = load_library("streams")
    code = lib.sandy_embed_bigram(
        _p(ids), _p(positions), _p(token_seq), _p(q_start), _p(seq_slots), _p(wte), _p(bigram), _p(wpe), ctypes.c_int(bigram.shape[0] - 1),
        ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), _p(state), ctypes.c_longlong(state.stride(0)), _p(out),
        ctypes.c_int(out.stride(0)), ctypes.c_int(ids.numel()), ctypes.c_int(wte.shape[0]), ctypes.c_int(0 if wpe is None else wpe.shape[0]),
        ctypes.c_int(out.shape[1]), ctypes.c_int(_dt(wte)), ctypes.c_int(1 if keep else 0), None, _stream())
    _check(code, "embed_bigram")
    if not keep:
        _check(lib.sandy_bigram_keep(_p(ids), _p(q_start), _p(seq_slots), _p(state), ctypes.c_longlong(state.stride(0)),
                                     ctypes.c_int(seq_slots.numel()), _stream()), "bigram_keep")


def ssm_prepare(proj, taps, conv_bias, dt_raw, dt_bias, a_log, state, tail_off: int, token_seq, q_start, seq_slots, xbc, dta, *,
                keep: bool = False) -> None:
    """xbc = silu(causal conv(proj) + conv_bias), float32; dta = (softplus(dt_raw + dt_bias), -exp(a_log) * that), float32 [T, 2H].
    With keep (steps of single tokens) the convolution's tails move on in the same launch; otherwise conv_tail follows."""
    _cuda(proj, taps, conv_bias, dt_raw, dt_bias, a_log, state, token_seq, q_start, seq_slots, xbc, dta)
    code = load_library("ssm_state").sandy_ssm_prepare(
        _p(proj), ctypes.c_int(proj.stride(0)), ctypes.c_int(_dt(proj)), ctypes.c_int(proj.shape[1]), _p(taps), ctypes.c_int(taps.shape[1]),
        _p(conv_bias), _p(dt_raw), ctypes.c_int(dt_raw.stride(0)), _p(dt_bias), _p(a_log), ctypes.c_int(dt_raw.shape[1]), _p(state),
        ctypes.c_longlong(state.stride(0)), ctypes.c_longlong(tail_off), _p(token_seq), _p(q_start), _p(seq_slots), _p(xbc),
        ctypes.c_int(xbc.stride(0)), _p(dta), ctypes.c_int(proj.shape[0]), ctypes.c_int(1 if keep else 0), _stream())
    _check(code, "ssm_prepare")


def ssm_scan(xbc, dta, d_skip, state, q_start, seq_slots, out, *, n_heads: int, n_groups: int, state_dim: int, v_dim: int) -> None:
    """The state-space recurrence token by token: S <- exp(dta[1]) S + dt B x^T per head, out = S^T C + d_skip x.  xbc float32
    [T, H * P + 2 G * N] (x, B, C); `state` float32 [slots, >= H * P * N], a slot's S as [H][P][N]."""
    _cuda(xbc, dta, d_skip, state, q_start, seq_slots, out)
    code = load_library("ssm_state").sandy_ssm_scan(
        _p(xbc), ctypes.c_int(xbc.stride(0)), _p(dta), _p(d_skip), _p(state), ctypes.c_longlong(state.stride(0)), _p(q_start), _p(seq_slots),
        _p(out), ctypes.c_int(out.stride(0)), ctypes.c_int(seq_slots.numel()), ctypes.c_int(n_heads), ctypes.c_int(n_groups),
        ctypes.c_int(state_dim), ctypes.c_int(v_dim), _stream())
    _check(code, f"ssm_scan(H={n_heads},N={state_dim},P={v_dim})")


def gated_group_norm(y, z, gain, out, *, groups: int, eps: float) -> None:
    """out = (y * silu(z)) over its root mean square in `groups` equal parts of a row, times gain; y float32."""
    _cuda(y, z, gain, out)
    code = load_library("ssm_state").sandy_gated_group_norm(
        _p(y), ctypes.c_int(y.stride(0)), _p(z), ctypes.c_int(z.stride(0)), _p(gain), ctypes.c_float(eps), ctypes.c_int(groups), _p(out),
        ctypes.c_int(out.stride(0)), ctypes.c_int(y.shape[0]), ctypes.c_int(y.shape[1]), ctypes.c_int(_dt(out)), _stream())
    _check(code, "gated_group_norm")


def sample(logits, out_tokens, *, temperature=None, top_k=None, top_p=None, uniform=None, status=None,
           feedback=None) -> None:
    """Choose one token per row of float32 `logits`; per-row option tensors may be None.
    feedback: (token_ids, logit_rows, positions, burst_tokens, row_step) int32 device tensors: the
    drawn token also replaces the row's input token, its position moves on, and the token is
    recorded in burst_tokens[row_step[r], r]; `uniform` then holds [steps, rows] numbers."""
    _cuda(logits, out_tokens, temperature, top_k, top_p, uniform, status)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    n, vocab = logits.shape
    _i32(out_tokens, "out_tokens")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32)):
        if name == "uniform" and feedback is not None:
            continue
        if t is not None and (t.dtype != dt or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be a contiguous {dt} tensor of one value per row")
    if temperature is not None and uniform is None:
        raise KernelError("sample: temperature sampling needs a uniform number per row")
    fb = [None] * 5
    if feedback is not None:
        fb = list(feedback)
        _cuda(*fb)
        for t in fb:
            _i32(t, "feedback array")
        if uniform is None or uniform.dtype != torch.float32 or not uniform.is_contiguous() \
                or uniform.numel() % n or fb[3].numel() < uniform.numel():
            raise KernelError("sample: with feedback, uniform must be float32 [steps, rows] and burst_tokens as large")
    lib = load_library("sampling")
    code = lib.sandy_sample(_p(logits), ctypes.c_int(logits.stride(0)), ctypes.c_int(n), ctypes.c_int(vocab),
                            _p(temperature), _p(top_k), _p(top_p), _p(uniform), _p(out_tokens), _p(status),
                            _p(fb[0]), _p(fb[1]), _p(fb[2]), _p(fb[3]), _p(fb[4]), _stream())
    _check(code, "sample")


# --------------------------------------------------------------------------------------
_kernel_status = {}


def kernel_status(device) -> torch.Tensor:
    """A device int the kernels with bounded waits raise bits in (0 = all waits were met)."""
    key = torch.device(device).index or 0
    t = _kernel_status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _kernel_status[key] = t
    return t


def check_kernel_status(device) -> None:
    t = kernel_status(device)
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(f"a kernel reported a fault (status {code}: bits 0-2 a barrier wait ran out in the "
                          "tensor-core product, bit 3 a key/value write and bit 4 a key read had no page behind "
                          "it, bits 5-6 a wait ran out in the bulk decode attention, "
                          "bit 8 in the tcgen05 prefill attention); the step's output is not valid")


def tensor_core_gemm_supported(K: int, N: int) -> bool:
    """Whether the tcgen05 kernel takes a [*, K] x [N, K] product: its operand rows must start
    on 16-byte boundaries for TMA, so K must be a multiple of 8."""
    return K % 8 == 0 and K >= 8


def gemm_tc(a, w, bias, out, *, act=None, residual=None, tile_n: int = 0, kv=None) -> None:
    """out = act(a @ w.T + bias) + residual on the tcgen05 tensor cores.
    a: bfloat16 [M, K]; w: bfloat16 [N, K]; out: bfloat16 or float32 [M, N].  With `kv` (a
    KVTarget) the key and value columns of the product also go into the cache pages."""
    _cuda(a, w, bias, out, residual)
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise UnsupportedShape("gemm_tc takes bfloat16 operands")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_tc: innermost stride must be 1")
    if K % 8 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        raise UnsupportedShape(f"gemm_tc: K={K} and the row pitches must be multiples of 8 elements, "
                               "operands 16-byte aligned")
    if residual is not None and (residual.dtype != torch.float32 or residual.stride(1) != 1
                                 or tuple(residual.shape) != (M, N)):
        raise KernelError("gemm_tc: residual must be float32 [M, N]")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N):
        raise KernelError("gemm_tc: bias must be bfloat16 [N]")
    kc = vc = table = tseq = tpos = None
    page_stride = max_blocks = q_cols = kv_cols = head_dim = page_size = num_pages = 0
    if kv is not None:
        hkv, page_size, head_dim, page_stride, num_pages = _cache_args(kv.k_cache, kv.v_cache)
        kc, vc, table, tseq, tpos = kv.k_cache, kv.v_cache, kv.block_table, kv.token_seq, kv.positions
        _cuda(kc, vc, table, tseq, tpos)
        _i32(table, "block_table"); _i32(tseq, "token_seq"); _i32(tpos, "positions")
        q_cols, kv_cols, max_blocks = kv.q_cols, kv.kv_cols, table.shape[1]
        if kc.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kv_cols != hkv * head_dim \
                or q_cols + 2 * kv_cols != N or kv.head_dim != head_dim:
            raise KernelError("gemm_tc: the key/value target does not match the product")
    lib = load_library("gemm_tc")

    def launch(tile, dst, res, with_kv=True):
        fn = lib.sandy_gemm_tc
        if tile >= PAIR_TILE:        # two CTAs on one 256-row tile
            fn, tile = load_library("gemm_tc2").sandy_gemm_tc2, tile - PAIR_TILE
        code = fn(_p(a), _p(w), _p(bias), _p(res), _p(dst), ctypes.c_int(M), ctypes.c_int(N),
                  ctypes.c_int(K), ctypes.c_int(a.stride(0)), ctypes.c_int(w.stride(0)),
                  ctypes.c_int(0 if res is None else res.stride(0)),
                  ctypes.c_int(dst.stride(0)), ctypes.c_int(ACT_CODES[act]), ctypes.c_int(_dt(dst)),
                  ctypes.c_int(tile), _p(kc if with_kv else None), _p(vc), ctypes.c_longlong(page_stride), _p(table),
                  ctypes.c_int(max_blocks), _p(tseq), _p(tpos), ctypes.c_int(q_cols), ctypes.c_int(kv_cols),
                  ctypes.c_int(head_dim), ctypes.c_int(page_size), ctypes.c_int(num_pages),
                  _p(kernel_status(a.device)), _stream())
        _check(code, f"gemm_tc(M={M},N={N},K={K},tile={tile},kv={kv is not None})")

    launch(tile_n, out, residual)         # tile_n 0: the kernel's own choice


# The tcgen05 variants (three tile widths, one tile per CTA or persistent; two CTAs on a 256-row
# tile, two widths), as `tile_n` codes: n > 0 one tile of 128 x n per CTA, n < 0 the persistent
# kernel, PAIR_TILE + n the two-CTA kernel (gemm_tc2.cu).  The engine times them on the first
# product of a shape and keeps the winner (core/ops.cpp).
PAIR_TILE = 2000
GEMM_VARIANTS = (-64, -128, -256, 64, 128, 256, PAIR_TILE + 128, PAIR_TILE + 256)


SKINNY_NORM_MAX_ROWS = 16
SKINNY_NORM_MAX_K = 2048

def skinny_norm_fusable(norm: FusedNorm, K: int) -> bool:
    """Whether gemm_skinny can run this LayerNorm inside itself: bfloat16 gain/offset, at most 16
    rows, K at most 2048 (the row is held in registers)."""
    return (norm.gamma.dtype == torch.bfloat16 and norm.x.dtype == torch.float32
            and norm.x.shape[0] <= SKINNY_NORM_MAX_ROWS and K <= SKINNY_NORM_MAX_K and norm.x.stride(1) == 1
            and norm.x.stride(0) % 4 == 0 and norm.x.data_ptr() % 16 == 0 and norm.gamma.data_ptr() % 16 == 0
            and (norm.beta is None or norm.beta.data_ptr() % 16 == 0))


def gemm_skinny(a, w, bias, out, *, act=None, residual=None, norm=None, kv=None) -> None:
    """out = act(a @ w.T + bias) + residual for up to 64 rows (a decode step), weight-streaming.
    Same operand rules as gemm_tc.  With `norm` (a FusedNorm that skinny_norm_fusable accepted)
    `a` is None and the LayerNorm of norm.x runs inside the kernel.  With `kv` (a KVTarget) the
    key and value columns of the product are also written into the cache pages."""
    M, K = (norm.x.shape if norm is not None else a.shape)
    N = w.shape[0]
    x = gamma = beta = None
    eps = 0.0
    if norm is not None:
        x, gamma, beta, eps = norm.x, norm.gamma, norm.beta, float(norm.eps)
        if not skinny_norm_fusable(norm, K):
            raise UnsupportedShape("gemm_skinny: this norm cannot be fused")
    elif a.dtype != torch.bfloat16:
        raise UnsupportedShape("gemm_skinny takes bfloat16 operands")
    _cuda(a, x, gamma, beta, w, bias, out, residual)
    if w.dtype != torch.bfloat16:
        raise UnsupportedShape("gemm_skinny takes bfloat16 operands")
    if M > 64:
        raise UnsupportedShape(f"gemm_skinny takes at most 64 rows, got {M}")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_skinny: shapes disagree: a {(M, K)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if (a is not None and a.stride(1) != 1) or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_skinny: innermost stride must be 1")
    if K % 8 or w.stride(0) % 8 or w.data_ptr() % 16 or \
            (a is not None and (a.stride(0) % 8 or a.data_ptr() % 16)):
        raise UnsupportedShape(f"gemm_skinny: K={K} and the row pitches must be multiples of 8 elements, "
                               "operands 16-byte aligned")
    if residual is not None and (residual.dtype != torch.float32 or residual.stride(1) != 1
                                 or tuple(residual.shape) != (M, N)):
        raise KernelError("gemm_skinny: residual must be float32 [M, N]")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N):
        raise KernelError("gemm_skinny: bias must be bfloat16 [N]")
    kc = vc = table = tseq = tpos = None
    page_stride = max_blocks = q_cols = kv_cols = head_dim = page_size = num_pages = 0
    if kv is not None:
        hkv, page_size, head_dim, page_stride, num_pages = _cache_args(kv.k_cache, kv.v_cache)
        kc, vc, table, tseq, tpos = kv.k_cache, kv.v_cache, kv.block_table, kv.token_seq, kv.positions
        _cuda(kc, vc, table, tseq, tpos)
        _i32(table, "block_table"); _i32(tseq, "token_seq"); _i32(tpos, "positions")
        q_cols, kv_cols, max_blocks = kv.q_cols, kv.kv_cols, table.shape[1]
        if kc.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kv_cols != hkv * head_dim \
                or q_cols + 2 * kv_cols != N or kv.head_dim != head_dim:
            raise KernelError("gemm_skinny: the key/value target does not match the product")
    lib = load_library("gemm_skinny")
    code = lib.sandy_gemm_skinny(
        _p(a), _p(x), ctypes.c_int(0 if x is None else x.stride(0)), _p(gamma), _p(beta), ctypes.c_float(eps),
        _p(w), _p(bias), _p(residual), _p(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(0 if a is None else a.stride(0)), ctypes.c_int(w.stride(0)),
        ctypes.c_int(0 if residual is None else residual.stride(0)), ctypes.c_int(out.stride(0)),
        ctypes.c_int(ACT_CODES[act]), ctypes.c_int(_dt(out)), _p(kc), _p(vc), ctypes.c_longlong(page_stride),
        _p(table), ctypes.c_int(max_blocks), _p(tseq), _p(tpos), ctypes.c_int(q_cols), ctypes.c_int(kv_cols),
        ctypes.c_int(head_dim), ctypes.c_int(page_size), ctypes.c_int(num_pages), _p(kernel_status(w.device)),
        _stream())
    _check(code, f"gemm_skinny(M={M},N={N},K={K},norm={norm is not None},kv={kv is not None})")


def gemm_small(a, w, bias, out, *, act=None, residual=None, kv=None) -> None:
    """out = act(a @ w.T + bias) + residual for up to 256 rows on the tcgen05 tensor cores with the
    weight as the instruction's wide operand and K split over a cluster's blocks (gemm_small.cu).
    Same operand rules as gemm_tc; `kv` as in gemm_skinny."""
    M, K = a.shape
    N = w.shape[0]
    _cuda(a, w, bias, out, residual)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise UnsupportedShape("gemm_small takes bfloat16 operands")
    if M > 256:
        raise UnsupportedShape(f"gemm_small takes at most 256 rows, got {M}")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_small: shapes disagree: a {(M, K)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_small: innermost stride must be 1")
    if K % 8 or w.stride(0) % 8 or w.data_ptr() % 16 or a.stride(0) % 8 or a.data_ptr() % 16:
        raise UnsupportedShape(f"gemm_small: K={K} and the row pitches must be multiples of 8 elements, "
                               "operands 16-byte aligned")
    if residual is not None and (residual.dtype != torch.float32 or residual.stride(1) != 1
                                 or tuple(residual.shape) != (M, N)):
        raise KernelError("gemm_small: residual must be float32 [M, N]")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N):
        raise KernelError("gemm_small: bias must be bfloat16 [N]")
    kc = vc = table = tseq = tpos = None
    page_stride = max_blocks = q_cols = kv_cols = head_dim = page_size = num_pages = 0
    if kv is not None:
        hkv, page_size, head_dim, page_stride, num_pages = _cache_args(kv.k_cache, kv.v_cache)
        kc, vc, table, tseq, tpos = kv.k_cache, kv.v_cache, kv.block_table, kv.token_seq, kv.positions
        _cuda(kc, vc, table, tseq, tpos)
        _i32(table, "block_table"); _i32(tseq, "token_seq"); _i32(tpos, "positions")
        q_cols, kv_cols, max_blocks = kv.q_cols, kv.kv_cols, table.shape[1]
        if kc.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kv_cols != hkv * head_dim \
                or q_cols + 2 * kv_cols != N or kv.head_dim != head_dim:
            raise KernelError("gemm_small: the key/value target does not match the product")
    lib = load_library("gemm_small")
    code = lib.sandy_gemm_small(
        _p(a), _p(w), _p(bias), _p(residual), _p(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(a.stride(0)), ctypes.c_int(w.stride(0)),
        ctypes.c_int(0 if residual is None else residual.stride(0)), ctypes.c_int(out.stride(0)),
        ctypes.c_int(ACT_CODES[act]), ctypes.c_int(_dt(out)), _p(kc), _p(vc), ctypes.c_longlong(page_stride),
        _p(table), ctypes.c_int(max_blocks), _p(tseq), _p(tpos), ctypes.c_int(q_cols), ctypes.c_int(kv_cols),
        ctypes.c_int(head_dim), ctypes.c_int(page_size), ctypes.c_int(num_pages), _p(kernel_status(w.device)),
        _stream())
    _check(code, f"gemm_small(M={M},N={N},K={K},kv={kv is not None})")


def small_gemm_kernel(M: int, N: int, K: int) -> str:
    """Which kernel the engine gives a bfloat16 product of up to 64 rows: "streaming" (gemm_skinny) or
    "split_k" (gemm_small).  A rule of the shape alone (host library, no GPU needed)."""
    from .. import core

    return core.call("global", None, "small_gemm_kernel", M=M, N=N, K=K)


def gemm_small_splits(N: int, K: int) -> int:
    """How many blocks share an output tile of gemm_small for this shape on this device."""
    return int(load_library("gemm_small").sandy_gemm_small_splits(ctypes.c_int(N), ctypes.c_int(K)))
