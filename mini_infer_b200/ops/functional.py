"""Python faces of the CUDA kernels: check the tensors, pass the pointers.

Every function runs on the current CUDA stream of the tensors' device and
returns its output tensor.  Shapes a kernel cannot take are refused with an
error; nothing falls back to PyTorch.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from .library import KernelError, check, library

F32 = torch.float32
BF16 = torch.bfloat16
I32 = torch.int32

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise TypeError(f"{what}: dtype {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _chk(t: Optional[torch.Tensor], what: str, dtype=None, shape=None) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise RuntimeError(f"{what}: tensor is on {t.device}; the kernels run on CUDA only and have no fallback")
    if not t.is_contiguous():
        raise ValueError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{what}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        actual = t.shape
        bad = len(shape) != len(actual)
        if not bad:
            for s, a in zip(shape, actual):
                if s is not None and s != a:
                    bad = True
                    break
        if bad:
            raise ValueError(f"{what}: expected shape {list(shape)}, got {list(actual)}")


# --------------------------------------------------------------------------- #
# Debug mode: with MINI_INFER_DEBUG_BOUNDS=1 in the environment every index that a kernel will follow
# (token ids, row lists, cache slots, block tables, lengths, expert choices and offsets, permutations) is
# checked on the host before the launch, and a bad one raises a KernelError that names the tensor, the
# first bad place and its value, instead of becoming an access outside a buffer.  It synchronises the
# device at every op, so it is for chasing a fault, not for serving.  (The reference checks none of these;
# its kernels return silently on a size they do not take, src/kernels/paged_attn_kernel.cu:313-315.)
# --------------------------------------------------------------------------- #
import os as _os

DEBUG_BOUNDS = _os.environ.get("MINI_INFER_DEBUG_BOUNDS", "0") not in ("", "0")
debug_checks_run = 0


def _bad(what: str, msg: str):
    from .library import KernelError
    raise KernelError(f"{what}: {msg} (found by MINI_INFER_DEBUG_BOUNDS before the launch)")


def _dbg_range(t: Optional[torch.Tensor], lo: int, hi: int, what: str) -> None:
    """Every element of ``t`` lies in ``[lo, hi)``."""
    global debug_checks_run
    if t is None or t.numel() == 0:
        return
    debug_checks_run += 1
    flat = t.reshape(-1)
    bad = ((flat < lo) | (flat >= hi)).nonzero()
    if bad.numel():
        i = int(bad[0, 0])
        _bad(what, f"element {i} is {int(flat[i])}, outside [{lo}, {hi})")


def _dbg_offsets(offsets: torch.Tensor, n_rows: int, what: str) -> None:
    """Expert offsets rise from 0 to the number of rows."""
    global debug_checks_run
    debug_checks_run += 1
    o = offsets.cpu().tolist()
    if o[0] != 0 or o[-1] != n_rows or any(b < a for a, b in zip(o, o[1:])):
        _bad(what, f"offsets {o[:8]}... do not rise from 0 to {n_rows}")


def _dbg_batch(what: str, q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, T: int,
               num_pages: int, page_size: int, window: int, max_q_len: Optional[int] = None) -> None:
    """The layout of a ragged batch over a paged cache: ``q_start`` rises within 0 .. T (a call may cover
    only the first or the last requests of a step's rows), every request's length covers its new tokens and
    fits its table, and every page that a query of this step reads (all of them, or those its window reaches)
    is a real page."""
    global debug_checks_run
    debug_checks_run += 1
    qs, kv, bt = q_start.cpu().tolist(), kv_len.cpu().tolist(), block_table.cpu()
    B, max_pages = bt.shape
    if qs[0] < 0 or qs[-1] > T or any(b <= a for a, b in zip(qs, qs[1:])):
        _bad(what, f"q_start {qs} does not rise within 0 .. {T}")
    for b in range(B):
        n_q, n = qs[b + 1] - qs[b], kv[b]
        if max_q_len is not None and n_q > max_q_len:
            _bad(what, f"request {b} brings {n_q} tokens, max_q_len says {max_q_len}")
        if n < n_q or n > max_pages * page_size:
            _bad(what, f"request {b}: kv_len {n} with {n_q} new tokens and a table of {max_pages} pages of {page_size}")
        first = 0 if window <= 0 else max(0, n - n_q - window + 1)
        row = bt[b]
        for i in range(first // page_size, -(-n // page_size)):
            p = int(row[i])
            if not 0 <= p < num_pages:
                _bad(what, f"request {b} reads page entry {i} = {p}, the cache has {num_pages} pages")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device, as the integer the launchers take."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------------- #

def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` as float32 ``[T, H]``."""
    _chk(ids, "embed_gather ids", I32)
    _chk(table, "embed_gather table")
    T = ids.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty(T, H, dtype=F32, device=table.device)
    _chk(out, "embed_gather out", F32, (T, H))
    if DEBUG_BOUNDS:
        _dbg_range(ids, 0, V, "embed_gather ids")
    check(library().mi_embed_gather(_ptr(ids), _ptr(table), _code(table, "embed_gather table"), _ptr(out),
                                    T, H, V, _stream()), "embed_gather")
    return out


def add_rmsnorm(hidden: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hidden += delta`` (if given; written back unless ``rows``), then RMSNorm.

    ``rows`` (int32) selects and orders the rows to normalise; ``hidden`` is then
    left untouched.
    """
    _chk(hidden, "add_rmsnorm hidden", F32)
    T, H = hidden.shape
    _chk(delta, "add_rmsnorm delta", F32, (T, H))
    _chk(weight, "add_rmsnorm weight", None, (H,))
    _chk(rows, "add_rmsnorm rows", I32)
    n = T if rows is None else rows.numel()
    if out is None:
        out = torch.empty(n, H, dtype=out_dtype, device=hidden.device)
    _chk(out, "add_rmsnorm out", out_dtype, (n, H))
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, T, "add_rmsnorm rows")
    check(library().mi_add_rmsnorm(_ptr(hidden), _ptr(delta), _ptr(rows), _ptr(weight),
                                   _code(weight, "add_rmsnorm weight"), _ptr(out), _code(out, "add_rmsnorm out"),
                                   n, H, float(eps), _stream()), "add_rmsnorm")
    return out


def qkv_post(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
             inv_freq: Optional[torch.Tensor], rot_dim: int, slot_mapping: Optional[torch.Tensor],
             k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int,
             page_size: int, out_dtype: torch.dtype, q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bias, rotary position encoding of q and k, cache write of k and v.

    ``qkv`` is float32 ``[T, (nh + 2*nkv) * d]`` (``nkv = 0``: queries only, nothing
    is written).  ``k_cache``/``v_cache`` are one layer's ``[pages, nkv, page_size, d]``.
    Returns ``q [T, nh, d]`` in ``out_dtype``.
    """
    _chk(qkv, "qkv_post qkv", F32)
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * d
    _chk(qkv, "qkv_post qkv", F32, (T, width))
    _chk(bias, "qkv_post bias", None, (width,))
    _chk(positions, "qkv_post positions", I32, (T,))
    _chk(inv_freq, "qkv_post inv_freq", F32)
    if inv_freq is not None and inv_freq.numel() != rot_dim // 2:
        raise ValueError(f"qkv_post: {inv_freq.numel()} frequencies for {rot_dim} rotary dims")
    if nkv > 0:
        _chk(slot_mapping, "qkv_post slot_mapping", I32, (T,))
        _chk(k_cache, "qkv_post k_cache", out_dtype, (None, nkv, page_size, d))
        _chk(v_cache, "qkv_post v_cache", out_dtype, (None, nkv, page_size, d))
        if slot_mapping is None or k_cache is None or v_cache is None:
            raise ValueError("qkv_post: key/value heads need a cache and a slot mapping")
    if q_out is None:
        q_out = torch.empty(T, nh, d, dtype=out_dtype, device=qkv.device)
    _chk(q_out, "qkv_post q_out", out_dtype, (T, nh, d))
    wcode = _code(bias, "qkv_post bias") if bias is not None else 0
    if DEBUG_BOUNDS and nkv > 0:
        _dbg_range(slot_mapping, -1, k_cache.shape[0] * page_size, "qkv_post slot_mapping")     # -1: not cached
    check(library().mi_qkv_post(_ptr(qkv), _ptr(bias), wcode, _ptr(positions), _ptr(inv_freq),
                                _ptr(slot_mapping), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                _code(q_out, "qkv_post q_out"), T, nh, nkv, d, rot_dim, page_size, _stream()),
          "qkv_post")
    return q_out


def swiglu(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gu[:, :I]) * gu[:, I:]`` for ``gu [T, 2I]``."""
    _chk(gu, "swiglu input")
    T, two_i = gu.shape
    if two_i % 2:
        raise ValueError("swiglu: the input width must be even (gate | up)")
    inter = two_i // 2
    if out is None:
        out = torch.empty(T, inter, dtype=gu.dtype, device=gu.device)
    _chk(out, "swiglu out", gu.dtype, (T, inter))
    check(library().mi_swiglu(_ptr(gu), _ptr(out), _code(gu, "swiglu input"), T, inter, _stream()), "swiglu")
    return out


def moe_combine(y: torch.Tensor, inv_perm: Optional[torch.Tensor], weights: torch.Tensor,
                shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_k weights[t,k] * y[inv_perm[t,k]] + gate[t] * shared[t]`` (float32);
    without ``inv_perm`` the rows of ``y`` are indexed by pair, ``y[t*K + k]``."""
    T, K = weights.shape
    _chk(y, "moe_combine y", F32, (T * K, None))
    H = y.shape[1]
    _chk(inv_perm, "moe_combine inv_perm", I32)
    _chk(weights, "moe_combine weights", F32)
    _chk(shared, "moe_combine shared", F32, (T, H))
    _chk(gate, "moe_combine gate", F32, (T,))
    if (shared is None) != (gate is None):
        raise ValueError("moe_combine: shared output and gate come together")
    if out is None:
        out = torch.empty(T, H, dtype=F32, device=y.device)
    _chk(out, "moe_combine out", F32, (T, H))
    if DEBUG_BOUNDS:
        _dbg_range(inv_perm, 0, T * K, "moe_combine inv_perm")
    check(library().mi_moe_combine(_ptr(y), _ptr(inv_perm), _ptr(weights), _ptr(shared), _ptr(gate), _ptr(out),
                                   T, H, K, _stream()), "moe_combine")
    return out


def combine_add_rmsnorm(hidden: torch.Tensor, y: torch.Tensor, inv_perm: Optional[torch.Tensor],
                        weights: torch.Tensor, shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                        norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                        rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`moe_combine` and the :func:`add_rmsnorm` that takes its result as ``delta``, in one kernel:
    the combined rows are added to ``hidden`` (written back unless ``rows``) and normalised without
    ever being stored.  Bit for bit the result of the two separate calls."""
    _chk(hidden, "combine_add_rmsnorm hidden", F32)
    T, H = hidden.shape
    if weights.shape[0] != T:
        raise ValueError("combine_add_rmsnorm: one row of expert weights per row of hidden")
    K = weights.shape[1]
    _chk(y, "combine_add_rmsnorm y", F32, (T * K, H))
    _chk(inv_perm, "combine_add_rmsnorm inv_perm", I32)
    _chk(weights, "combine_add_rmsnorm weights", F32)
    _chk(shared, "combine_add_rmsnorm shared", F32, (T, H))
    _chk(gate, "combine_add_rmsnorm gate", F32, (T,))
    if (shared is None) != (gate is None):
        raise ValueError("combine_add_rmsnorm: shared output and gate come together")
    _chk(norm_weight, "combine_add_rmsnorm weight", None, (H,))
    _chk(rows, "combine_add_rmsnorm rows", I32)
    n = T if rows is None else rows.numel()
    out = torch.empty(n, H, dtype=out_dtype, device=hidden.device)
    if DEBUG_BOUNDS:
        _dbg_range(inv_perm, 0, T * K, "combine_add_rmsnorm inv_perm")
        _dbg_range(rows, 0, T, "combine_add_rmsnorm rows")
    check(library().mi_combine_add_rmsnorm(_ptr(hidden), _ptr(y), _ptr(inv_perm), _ptr(weights), _ptr(shared),
                                           _ptr(gate), K, _ptr(rows), _ptr(norm_weight),
                                           _code(norm_weight, "combine_add_rmsnorm weight"), _ptr(out),
                                           _code(out, "combine_add_rmsnorm out"), n, H, float(eps), _stream()),
          "combine_add_rmsnorm")
    return out


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
              q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
              scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a ragged batch over the paged cache (tiled kernel, any head size <= 256)."""
    _chk(q, "attention q")
    T, nh, d = q.shape
    _chk(k_cache, "attention k_cache", q.dtype)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "attention v_cache", q.dtype, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "attention block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "attention q_start", I32, (B + 1,))
    _chk(kv_len, "attention kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "attention out", q.dtype, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if DEBUG_BOUNDS:
        _dbg_batch("attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window), int(max_q_len))
    check(library().mi_attn_tiled(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "attention q"),
                                  _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), B, int(max_q_len),
                                  nh, nkv, d, page_size, max_pages, int(window), float(scale), _stream()),
          "attention")
    return out


def prefill_attention_supported(d: int) -> bool:
    return bool(library().mi_attn_prefill_supported(int(d)))


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
                      scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as :func:`attention`, on tensor cores: bfloat16, head sizes 64 and 128."""
    _chk(q, "prefill_attention q", BF16)
    T, nh, d = q.shape
    _chk(k_cache, "prefill_attention k_cache", BF16)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "prefill_attention v_cache", BF16, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"prefill_attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "prefill_attention block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "prefill_attention out", BF16, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(q_start),
                                    _ptr(kv_len), _ptr(out), B, int(max_q_len), nh, nkv, d, page_size, max_pages,
                                    int(window), float(scale), _stream()), "prefill_attention")
    return out


def prefill_attention_tc_supported(d: int, page_size: int) -> bool:
    return bool(library().mi_attn_prefill_tc_supported(int(d), int(page_size)))


def prefill_attention_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                         q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
                         scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                         keep_first: int = 0, softcap: float = 0.0, sink: bool = False) -> torch.Tensor:
    """Same contract as :func:`attention`, on the tcgen05 tensor cores (TMA-fed, accumulators in
    tensor memory): bfloat16, head sizes 64 and 128, pages of 8 to 128 tokens.  ``softcap`` (0: none): every
    scaled score becomes ``softcap * tanh(score / softcap)``; ``sink``: the softmax counts one key more, of
    score 0 and without a value.  Call
    :func:`check_tc_status` after the step: a wait inside the kernel that ran out is reported there."""
    global _tc_pending
    _chk(q, "prefill_attention_tc q", BF16)
    T, nh, d = q.shape
    _chk(k_cache, "prefill_attention_tc k_cache", BF16)
    num_pages, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "prefill_attention_tc v_cache", BF16, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"prefill_attention_tc: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "prefill_attention_tc block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention_tc q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention_tc kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "prefill_attention_tc out", BF16, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    dev = q.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention_tc", q_start, kv_len, block_table, T, num_pages, page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(q_start),
                                       _ptr(kv_len), _ptr(out), _ptr(_tc_status[dev]), T, B, int(max_q_len), nh, nkv,
                                       d, page_size, num_pages, max_pages, int(window), float(scale),
                                       int(keep_first), float(softcap), int(bool(sink)), _stream()),
          "prefill_attention_tc")
    _tc_pending = True
    return out


def prefill_attention_tc_logistic_supported(dk: int, dv: int, page_size: int) -> bool:
    return bool(library().mi_attn_prefill_tc_logistic_supported(int(dk), int(dv), int(page_size)))


def prefill_attention_tc_logistic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                  block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor,
                                  max_q_len: int, window: int, scale: float, head_bias: torch.Tensor) -> torch.Tensor:
    """The tcgen05 attention without a softmax: a visible key's weight is ``logistic(score * scale +
    head_bias[h])`` by itself, not normalised over the keys (what :func:`attention_mix` computes with
    ``head_bias``).  bfloat16; key and value heads of 64 or 128 numbers each, not necessarily alike.  Returns
    ``[T, nh, dv]``.  Call :func:`check_tc_status` after the step."""
    global _tc_pending
    _chk(q, "prefill_attention_tc_logistic q", BF16)
    T, nh, dk = q.shape
    _chk(k_cache, "prefill_attention_tc_logistic k_cache", BF16, (None, None, None, dk))
    num_pages, nkv, page_size, _ = k_cache.shape
    _chk(v_cache, "prefill_attention_tc_logistic v_cache", BF16, (num_pages, nkv, page_size, None))
    dv = v_cache.shape[3]
    _chk(head_bias, "prefill_attention_tc_logistic head_bias", F32, (nh,))
    _chk(block_table, "prefill_attention_tc_logistic block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention_tc_logistic q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention_tc_logistic kv_len", I32, (B,))
    out = torch.empty(T, nh, dv, dtype=BF16, device=q.device)
    dev = q.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention_tc_logistic", q_start, kv_len, block_table, T, num_pages, page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill_tc_logistic(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(q_start),
                                                _ptr(kv_len), _ptr(out), _ptr(_tc_status[dev]), T, B, int(max_q_len),
                                                nh, nkv, dk, dv, page_size, num_pages, max_pages, int(window),
                                                float(scale), _ptr(head_bias), _stream()),
          "prefill_attention_tc_logistic")
    _tc_pending = True
    return out


def prefill_attention_tc_shared_supported(heads: int, dk: int, dv: int, page_size: int) -> bool:
    return bool(library().mi_attn_prefill_tc_shared_supported(int(heads), int(dk), int(dv), int(page_size)))


def prefill_attention_tc_shared(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                                kv_len: torch.Tensor, max_q_len: int, window: int, scale: float, value_dim: int,
                                keep_first: int = 0) -> torch.Tensor:
    """:func:`prefill_attention_tc` for heads that all read ONE key/value head whose values are the first
    ``value_dim`` numbers of its key rows: ``q [T, H, dk]``, ``cache [pages, 1, page_size, dk]``, result
    ``[T, H, value_dim]``.  The rows of a query tile are (query, head) pairs, so a tile of keys is fetched once
    for all heads.  Sizes: :func:`prefill_attention_tc_shared_supported`."""
    global _tc_pending
    _chk(q, "prefill_attention_tc_shared q", BF16)
    T, H, dk = q.shape
    _chk(cache, "prefill_attention_tc_shared cache", BF16, (None, 1, None, dk))
    num_pages, _, page_size, _ = cache.shape
    _chk(block_table, "prefill_attention_tc_shared block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention_tc_shared q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention_tc_shared kv_len", I32, (B,))
    out = torch.empty(T, H, int(value_dim), dtype=BF16, device=q.device)
    dev = q.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention_tc_shared", q_start, kv_len, block_table, T, num_pages, page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill_tc_shared(_ptr(q), _ptr(cache), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
                                              _ptr(out), _ptr(_tc_status[dev]), T, B, int(max_q_len), H, dk,
                                              int(value_dim), page_size, num_pages, max_pages, int(window),
                                              float(scale), int(keep_first), _stream()),
          "prefill_attention_tc_shared")
    _tc_pending = True
    return out


def decode_attention_supported(d: int) -> bool:
    return bool(library().mi_attn_decode_supported(int(d)))


def decode_split_size() -> int:
    """Keys per split of the decode attention by default."""
    return int(library().mi_attn_decode_split_size())


DECODE_SPLIT_SIZES = (128, 256, 512)      # the split sizes the decode attention is built for


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     q_start: torch.Tensor, kv_len: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                     max_splits: int, window: int = 0, scale: Optional[float] = None,
                     out: Optional[torch.Tensor] = None, split: Optional[int] = None, softcap: float = 0.0,
                     sink: bool = False) -> torch.Tensor:
    """Split-KV attention when every request brings exactly one token.  ``softcap`` (0: none): every scaled
    score becomes ``softcap * tanh(score / softcap)``; ``sink``: the softmax counts one key more, of score 0
    and without a value.

    ``part_o`` (``>= B*nh*max_splits*d`` floats) and ``part_ml`` (``>= B*nh*max_splits*2``)
    are scratch; ``max_splits >= ceil(longest kv_len / split)`` with ``split`` keys per split
    (one of ``DECODE_SPLIT_SIZES``, default ``decode_split_size()``): smaller splits spread one or
    two requests over more blocks.
    """
    _chk(q, "decode_attention q")
    T, nh, d = q.shape
    _chk(k_cache, "decode_attention k_cache", q.dtype)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "decode_attention v_cache", q.dtype, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"decode_attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "decode_attention block_table", I32)
    B, max_pages = block_table.shape
    if T != B:
        raise ValueError(f"decode_attention: {T} tokens for {B} requests; each request brings exactly one")
    _chk(q_start, "decode_attention q_start", I32, (B + 1,))
    _chk(kv_len, "decode_attention kv_len", I32, (B,))
    _chk(part_o, "decode_attention part_o", F32)
    _chk(part_ml, "decode_attention part_ml", F32)
    if part_o.numel() < B * nh * max_splits * d or part_ml.numel() < B * nh * max_splits * 2:
        raise ValueError("decode_attention: scratch too small for this batch and split count")
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "decode_attention out", q.dtype, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if split is None:
        split = decode_split_size()
    if DEBUG_BOUNDS:
        _dbg_batch("decode_attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window), 1)
        longest = int(kv_len.max())
        if max_splits * int(split) < longest - int(split) // 4:
            _bad("decode_attention", f"{max_splits} splits of {split} keys cannot hold the longest request ({longest})")
    check(library().mi_attn_decode_split_form(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "decode_attention q"),
                                              _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), _ptr(part_o),
                                              _ptr(part_ml), B, nh, nkv, d, page_size, max_pages, int(max_splits),
                                              int(split), int(window), float(scale), float(softcap), int(bool(sink)),
                                              _stream()), "decode_attention")
    return out


def _selection_mode(norm_topk: bool, scoring: str, groups: Optional[Tuple[int, int]] = None) -> int:
    """The switches of the experts' selection as one word: renormalised weights, logistic scores, and
    ``groups = (count, keep)``: the experts form ``count`` equal groups of neighbours, and only those of the
    ``keep`` groups with the largest best score can be chosen."""
    if scoring not in ("softmax", "sigmoid"):
        raise ValueError(f"router scoring '{scoring}' is not 'softmax' or 'sigmoid'")
    mode = int(bool(norm_topk)) | (2 if scoring == "sigmoid" else 0)
    if groups is not None and groups[0] > 1 and groups[1] < groups[0]:
        count, keep = int(groups[0]), int(groups[1])
        if scoring != "softmax" or not 1 <= keep or count > 0xfff:
            raise ValueError(f"router: {keep} of {count} expert groups with '{scoring}' scores is not built")
        mode |= (count << 8) | (keep << 20)
    return mode


def moe_router(x: torch.Tensor, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor], top_k: int,
               norm_topk: bool, want_probs: bool = False, bias: Optional[torch.Tensor] = None,
               scoring: str = "softmax", groups: Optional[Tuple[int, int]] = None
               ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Router of one layer.  Returns ``(idx [T,K] int32, w [T,K] f32, gate [T] f32 | None, probs | None)``.
    ``bias`` (float32 ``[E]``) is added to the logits before the softmax and the choice.  ``scoring``
    ``sigmoid``: every expert's score is ``1 / (1 + exp(-logit))`` by itself instead of the softmax."""
    _chk(x, "moe_router x")
    T, H = x.shape
    _chk(router_w, "moe_router weight", None, (None, H))
    E = router_w.shape[0]
    _chk(bias, "moe_router bias", F32, (E,))
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_router shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_router: the shared-expert gate must have hidden_size entries")
    dev = x.device
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    z = torch.empty(T, E + 1, dtype=F32, device=dev)
    check(library().mi_moe_router(_ptr(x), _code(x, "moe_router x"), _ptr(router_w), _ptr(shared_gate_w),
                                  _code(router_w, "moe_router weight"), _ptr(z), _ptr(idx), _ptr(w), _ptr(gate),
                                  _ptr(probs), T, H, E, int(top_k), _selection_mode(norm_topk, scoring, groups),
                                  _ptr(bias), _stream()),
          "moe_router")
    return idx, w, gate, probs


def moe_permute(topk_idx: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable sort of the (token, slot) pairs by expert.

    Returns ``(offsets [E+1], sorted_token [T*K], inv_perm [T*K])``, all int32.
    """
    _chk(topk_idx, "moe_permute idx", I32)
    T, K = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty(num_experts + 1, dtype=I32, device=dev)
    sorted_token = torch.empty(T * K, dtype=I32, device=dev)
    inv_perm = torch.empty(T * K, dtype=I32, device=dev)
    counts = torch.empty(num_experts, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_range(topk_idx, 0, int(num_experts), "moe_permute expert indices")
    check(library().mi_moe_permute(_ptr(topk_idx), _ptr(offsets), _ptr(sorted_token), _ptr(inv_perm), _ptr(counts), T,
                                   int(num_experts), K, _stream()), "moe_permute")
    return offsets, sorted_token, inv_perm


def route_small_max_tokens() -> int:
    return int(library().mi_moe_route_small_max_tokens())


def moe_route_small(x: torch.Tensor, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor], top_k: int,
                    norm_topk: bool, ticket: torch.Tensor, want_probs: bool = False, permute: bool = True,
                    bias: Optional[torch.Tensor] = None, scoring: str = "softmax",
                    groups: Optional[Tuple[int, int]] = None):
    """:func:`moe_router` and (with ``permute``) :func:`moe_permute` of a step of a few tokens in
    one launch.

    ``ticket`` holds ``1 + T`` (or more) int32 counters that are zero before the first call and
    belong to the caller (the kernel leaves them zero); calls that share them must not overlap.  Returns
    ``(idx, w, gate, probs, offsets, sorted_token, inv_perm)``, the last three None without
    ``permute``.
    """
    _chk(x, "moe_route_small x")
    T, H = x.shape
    _chk(router_w, "moe_route_small weight", None, (None, H))
    E = router_w.shape[0]
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_route_small shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_route_small: the shared-expert gate must have hidden_size entries")
    _chk(ticket, "moe_route_small ticket", I32)
    _chk(bias, "moe_route_small bias", F32, (E,))
    if ticket.numel() < 1 + T:
        raise ValueError(f"moe_route_small: {ticket.numel()} ticket counters for {T} tokens (1 + T wanted)")
    dev = x.device
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    z = torch.empty(T, E + 1, dtype=F32, device=dev)
    offsets = sorted_token = inv_perm = None
    if permute:
        offsets = torch.empty(E + 1, dtype=I32, device=dev)
        sorted_token = torch.empty(T * top_k, dtype=I32, device=dev)
        inv_perm = torch.empty(T * top_k, dtype=I32, device=dev)
    check(library().mi_moe_route_small(
        _ptr(x), _code(x, "moe_route_small x"), _ptr(router_w), _ptr(shared_gate_w),
        _code(router_w, "moe_route_small weight"), _ptr(z), _ptr(ticket), _ptr(idx), _ptr(w), _ptr(gate), _ptr(probs),
        _ptr(offsets), _ptr(sorted_token), _ptr(inv_perm), T, H, E, int(top_k),
        _selection_mode(norm_topk, scoring, groups), _ptr(bias), _stream()), "moe_route_small")
    return idx, w, gate, probs, offsets, sorted_token, inv_perm


def norm_route_small_takes(hidden_size: int, num_experts: int = 1, gated: bool = False,
                           weight_dtype: torch.dtype = torch.bfloat16) -> bool:
    """Whether :func:`moe_norm_route_small` takes a router of these sizes (its blocks keep their share of the
    router's rows in shared memory)."""
    return bool(library().mi_moe_norm_route_small_takes(int(hidden_size), int(num_experts), int(bool(gated)),
                                                        2 if weight_dtype == torch.bfloat16 else 4))


def moe_norm_route_small(hidden: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                         out_dtype: torch.dtype, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor],
                         top_k: int, norm_topk: bool, want_probs: bool = False):
    """:func:`add_rmsnorm` and the routing of a step of a few tokens in one launch (a cluster of blocks per token):
    ``hidden += delta``, the normalised rows ``x`` (of ``out_dtype``) and the routing computed from
    them.  Returns ``(x, idx, w, gate, probs)``."""
    _chk(hidden, "moe_norm_route_small hidden", F32)
    T, H = hidden.shape
    _chk(delta, "moe_norm_route_small delta", F32, (T, H))
    _chk(norm_weight, "moe_norm_route_small norm weight", None, (H,))
    _chk(router_w, "moe_norm_route_small weight", None, (None, H))
    E = router_w.shape[0]
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_norm_route_small shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_norm_route_small: the shared-expert gate must have hidden_size entries")
    dev = hidden.device
    x = torch.empty(T, H, dtype=out_dtype, device=dev)
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    check(library().mi_moe_norm_route_small(
        _ptr(hidden), _ptr(delta), _ptr(norm_weight), _code(norm_weight, "moe_norm_route_small norm weight"),
        float(eps), _ptr(x), _code(x, "moe_norm_route_small x"), _ptr(router_w), _ptr(shared_gate_w),
        _code(router_w, "moe_norm_route_small weight"), _ptr(idx), _ptr(w), _ptr(gate),
        _ptr(probs), T, H, E, int(top_k), int(bool(norm_topk)), _stream()), "moe_norm_route_small")
    return x, idx, w, gate, probs


def _glu_args(glu) -> Tuple[int, float, float]:
    """``glu`` None: the gated units of a paired product are ``silu(gate) * up``; ``(limit, slope)``: the
    bounded form ``g * logistic(slope * g) * (u + 1)``, ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``."""
    if glu is None:
        return 0, 0.0, 0.0
    limit, slope = glu
    return 1, float(limit), float(slope)


def grouped_gemm_plain(a: torch.Tensor, gather: Optional[torch.Tensor], w: torch.Tensor, offsets: torch.Tensor,
                       n_rows: int, swiglu_pair: bool, out_dtype: torch.dtype, glu=None,
                       row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-expert product of sorted rows (float arithmetic).

    ``w`` is ``[E, Nout, K]`` or, with ``swiglu_pair``, ``[E, 2*Nout, K]`` (gate rows,
    then up rows) and the result is ``silu(gate) * up`` (or the bounded form that ``glu`` names,
    :func:`_glu_args`).  Row ``r`` of the result
    uses ``a[gather[r]]`` (or ``a[r]``) and the expert whose offset range holds ``r``.  ``row_scale``
    (float32, one number per result row, paired products only): both halves are multiplied by the row's number
    before they meet, which is the gated unit of the scaled input row.
    """
    _chk(a, "grouped_gemm a")
    Kd = a.shape[1]
    _chk(w, "grouped_gemm w", None, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(gather, "grouped_gemm gather", I32)
    _chk(offsets, "grouped_gemm offsets", I32, (E + 1,))
    out = torch.empty(n_rows, nout, dtype=out_dtype, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_plain")
        _dbg_range(gather, 0, a.shape[0], "grouped_gemm_plain gather")
        if gather is None and a.shape[0] < n_rows:
            _bad("grouped_gemm_plain", f"{n_rows} rows wanted, the input has {a.shape[0]}")
    check(library().mi_grouped_gemm_plain(_ptr(a), _code(a, "grouped_gemm a"), _ptr(gather), _ptr(w),
                                          _code(w, "grouped_gemm w"), _ptr(offsets), _ptr(out),
                                          _code(out, "grouped_gemm out"), int(n_rows), E, nout, Kd,
                                          1 if swiglu_pair else 0, *_glu_args(glu),
                                          _row_scale(row_scale, int(n_rows), swiglu_pair, "grouped_gemm_plain"),
                                          _stream()), "grouped_gemm_plain")
    return out


def l2_prefetch(t: torch.Tensor, max_bytes: Optional[int] = None) -> None:
    """Ask L2 for the first ``max_bytes`` bytes (all, if None) of a contiguous tensor; a hint, on the
    current stream, that returns at once."""
    _chk(t, "l2_prefetch tensor")
    n = t.numel() * t.element_size()
    if max_bytes is not None:
        n = min(n, int(max_bytes))
    check(library().mi_l2_prefetch(_ptr(t), n, _stream()), "l2_prefetch")


class dependent_launch:
    """``with dependent_launch(True):`` the kernels of decode-sized steps that are written for it (they wait
    for the kernels before them at their first line) are launched so that the device may place their blocks
    while the kernel before them in the stream is still running; a pass captured under it replays so."""

    def __init__(self, on: bool):
        self.on = bool(on)

    def __enter__(self):
        self.before = library().mi_set_dependent_launch(int(self.on))
        return self

    def __exit__(self, *exc):
        library().mi_set_dependent_launch(self.before)
        return False


def dense_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` in true float32 (``x [T, K]``, ``w [N, K]``): every output element is one chain of
    fused multiply-adds over ``k`` in ascending order, so a row's result does not depend on how many rows
    there are.  The dense product of the float32 path."""
    _chk(x, "dense_f32 x", F32)
    T, K = x.shape
    _chk(w, "dense_f32 w", F32, (None, K))
    N = w.shape[0]
    out = torch.empty(T, N, dtype=F32, device=x.device)
    check(library().mi_dense_f32(_ptr(x), _ptr(w), _ptr(out), T, N, K, _stream()), "dense_f32")
    return out


def grouped_gemm_skinny_supported(kd: int) -> bool:
    return bool(library().mi_grouped_gemm_skinny_supported(int(kd)))


def grouped_gemm_skinny(a: torch.Tensor, gather: Optional[torch.Tensor], w: torch.Tensor, offsets: torch.Tensor,
                        n_rows: int, swiglu_pair: bool, glu=None,
                        row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The grouped product for a few rows per expert (decode), bfloat16 on tensor cores.

    Same contract as :func:`grouped_gemm_plain`; the result is bfloat16 with ``swiglu_pair``
    (the activation that feeds the down projection) and float32 without.
    """
    _chk(a, "grouped_gemm_skinny a", BF16)
    Kd = a.shape[1]
    _chk(w, "grouped_gemm_skinny w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(gather, "grouped_gemm_skinny gather", I32)
    _chk(offsets, "grouped_gemm_skinny offsets", I32, (E + 1,))
    out = torch.empty(n_rows, nout, dtype=BF16 if swiglu_pair else F32, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_skinny")
        _dbg_range(gather, 0, a.shape[0], "grouped_gemm_skinny gather")
        if gather is None and a.shape[0] < n_rows:
            _bad("grouped_gemm_skinny", f"{n_rows} rows wanted, the input has {a.shape[0]}")
    check(library().mi_grouped_gemm_skinny(_ptr(a), _ptr(gather), _ptr(w), _ptr(offsets), _ptr(out), E, nout, Kd,
                                           1 if swiglu_pair else 0, *_glu_args(glu),
                                           _row_scale(row_scale, int(n_rows), swiglu_pair, "grouped_gemm_skinny"),
                                           _stream()), "grouped_gemm_skinny")
    return out


def dense_skinny_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether :func:`dense_skinny` takes this product: bfloat16, a few rows, inner size a multiple of 32."""
    return (x.dtype == BF16 and w.dtype == BF16 and x.dim() == 2 and x.is_contiguous() and w.is_contiguous()
            and 1 <= x.shape[0] <= library().mi_dense_skinny_max_rows() and x.shape[1] % 32 == 0)


def dense_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 swiglu_pair: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for a step of a few tokens (decode), every weight read once.

    ``x`` [T, K] and ``w`` [N, K] bfloat16, ``bias`` float32 [N] or None.  Returns float32
    [T, N]; with ``swiglu_pair`` the rows of ``w`` are N/2 gate rows then N/2 up rows and the
    result is ``silu(gate) * up`` as bfloat16 [T, N/2].
    """
    _chk(x, "dense_skinny x", BF16)
    T, Kd = x.shape
    _chk(w, "dense_skinny w", BF16, (None, Kd))
    wrows = w.shape[0]
    if swiglu_pair and wrows % 2:
        raise KernelError(f"dense_skinny: {wrows} weight rows cannot hold gate and up halves")
    nout = wrows // 2 if swiglu_pair else wrows
    if bias is not None:
        _chk(bias, "dense_skinny bias", F32, (wrows,))
    out = torch.empty(T, nout, dtype=BF16 if swiglu_pair else F32, device=x.device)
    check(library().mi_dense_skinny(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), T, nout, Kd,
                                    1 if swiglu_pair else 0, _stream()), "dense_skinny")
    return out


def qkv_skinny_supported(kd: int, d: int, rot_dim: int) -> bool:
    """Whether :func:`qkv_skinny` takes this geometry (``rot_dim`` 0: no rotation)."""
    return bool(library().mi_qkv_skinny_supported(int(kd), int(d), int(rot_dim)))


def qkv_skinny_max_rows() -> int:
    return int(library().mi_dense_skinny_max_rows())


def qkv_skinny(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
               inv_freq: Optional[torch.Tensor], slot_mapping: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, nh: int, nkv: int, d: int, page_size: int) -> torch.Tensor:
    """The q/k/v projection of a step of a few tokens with bias, rotary encoding and cache write
    in the same kernel (what a library product followed by :func:`qkv_post` does).

    ``x`` [T, K] and ``w_qkv`` [(nh + 2*nkv) * d, K] bfloat16, ``bias`` float32 or None.  Returns
    ``q [T, nh, d]`` bfloat16; k and v of row ``t`` go to ``slot_mapping[t]`` of the caches.
    """
    _chk(x, "qkv_skinny x", BF16)
    T, Kd = x.shape
    width = (nh + 2 * nkv) * d
    _chk(w_qkv, "qkv_skinny weight", BF16, (width, Kd))
    _chk(bias, "qkv_skinny bias", F32, (width,))
    _chk(positions, "qkv_skinny positions", I32, (T,))
    _chk(inv_freq, "qkv_skinny inv_freq", F32, (d // 2,))
    _chk(slot_mapping, "qkv_skinny slot_mapping", I32, (T,))
    _chk(k_cache, "qkv_skinny k_cache", BF16, (None, nkv, page_size, d))
    _chk(v_cache, "qkv_skinny v_cache", BF16, tuple(k_cache.shape))
    q = torch.empty(T, nh, d, dtype=BF16, device=x.device)
    if DEBUG_BOUNDS:
        _dbg_range(slot_mapping, -1, k_cache.shape[0] * page_size, "qkv_skinny slot_mapping")   # -1: not cached
    check(library().mi_qkv_skinny(_ptr(x), _ptr(w_qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq),
                                  _ptr(slot_mapping), _ptr(q), _ptr(k_cache), _ptr(v_cache), T, Kd, nh, nkv, d,
                                  page_size, _stream()), "qkv_skinny")
    return q


def skinny_pairs_max_tokens() -> int:
    return int(library().mi_grouped_gemm_skinny_pairs_max_tokens())


def skinny_pairs_split_inner_max_tokens() -> int:
    """Steps of up to this many tokens take the form of :func:`grouped_gemm_skinny_pairs` whose blocks own
    16 features and split the inner dimension over their warps."""
    return int(library().mi_grouped_gemm_skinny_pairs_split_inner_max_tokens())


def grouped_gemm_skinny_pairs(a: torch.Tensor, topk_idx: torch.Tensor, w: torch.Tensor,
                              swiglu_pair: bool, glu=None, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decode-sized grouped product without a permutation: row ``t*K + k`` of the result
    belongs to the pair (token t, slot k) and is computed under expert ``topk_idx[t, k]``.

    With ``swiglu_pair`` ``a`` is ``[T, Kd]`` (a token's row serves its K pairs) and the result is
    the bfloat16 activation ``[T*K, Nout]``; without, ``a`` is ``[T*K, Kd]`` indexed by pair and
    the result float32.
    """
    _chk(topk_idx, "grouped_gemm_skinny_pairs idx", I32)
    T, K = topk_idx.shape
    _chk(a, "grouped_gemm_skinny_pairs a", BF16, (T if swiglu_pair else T * K, None))
    Kd = a.shape[1]
    _chk(w, "grouped_gemm_skinny_pairs w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    out = torch.empty(T * K, nout, dtype=BF16 if swiglu_pair else F32, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_range(topk_idx, 0, E, "grouped_gemm_skinny_pairs expert indices")
    check(library().mi_grouped_gemm_skinny_pairs(_ptr(a), _ptr(topk_idx), _ptr(w), _ptr(out), T, K, E, nout, Kd,
                                                 1 if swiglu_pair else 0, *_glu_args(glu),
                                                 _row_scale(row_scale, T * K, swiglu_pair, "grouped_gemm_skinny_pairs"),
                                                 _stream()),
          "grouped_gemm_skinny_pairs")
    return out


def grouped_gemm_tc_supported(kd: int) -> bool:
    """The tcgen05 grouped product takes any number of output features; its inner size must be a multiple
    of 64 (one 128-byte swizzle row of bfloat16)."""
    return bool(library().mi_grouped_gemm_tc_supported(int(kd)))


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """``x[rows]`` for a bfloat16 matrix (the sorted copy the tensor-core grouped product reads)."""
    _chk(x, "gather_rows x", BF16)
    _chk(rows, "gather_rows rows", I32)
    out = torch.empty(rows.numel(), x.shape[1], dtype=BF16, device=x.device)
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, x.shape[0], "gather_rows rows")
    check(library().mi_gather_rows_bf16(_ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1], _stream()),
          "gather_rows")
    return out


def scatter_values(values: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
    """``out[dest[i]] = values[i]`` over the flattened operands (float32 values, int32 places that are a
    permutation): one number per (token, slot) pair brought into expert order."""
    _chk(values, "scatter_values values", F32)
    _chk(dest, "scatter_values dest", I32)
    n = values.numel()
    if dest.numel() != n:
        raise ValueError(f"scatter_values: {dest.numel()} places for {n} values")
    out = torch.empty(n, dtype=F32, device=values.device)
    if DEBUG_BOUNDS:
        _dbg_range(dest, 0, n, "scatter_values dest")
    check(library().mi_scatter_values(_ptr(values), _ptr(dest), _ptr(out), n, _stream()), "scatter_values")
    return out


def _row_scale(row_scale: Optional[torch.Tensor], rows: int, swiglu_pair: bool, what: str):
    """Pointer of the optional float32 number per result row that scales both halves of a gated unit."""
    if row_scale is None:
        return None
    if not swiglu_pair:
        raise ValueError(f"{what}: a scale per row belongs to a paired product's gated units")
    _chk(row_scale, what + " row_scale", F32)
    if row_scale.numel() != rows:
        raise ValueError(f"{what}: {row_scale.numel()} row scales for {rows} rows")
    return _ptr(row_scale)


_tc_status = {}
_tc_pending = False


TC_FORMS = (0, 1, 2, 3)


def grouped_gemm_tc(a_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, swiglu_pair: bool,
                    form: Optional[int] = None, glu=None, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The grouped product for many rows per expert (prefill): tcgen05 tensor cores fed by TMA.

    ``a_sorted [N, K]`` holds the rows already in expert order.  Result as for
    :func:`grouped_gemm_skinny`.  Call :func:`check_tc_status` after the step: a wait inside the
    kernel that ran out is reported there rather than hanging the device.  ``form`` picks one of the
    kernel's forms (``TC_FORMS``: one block per tile with row tiles of 128 or 256, persistent with
    row tiles of 160 or 256); the library chooses by the rows per expert when it is None.
    """
    global _tc_pending
    _chk(a_sorted, "grouped_gemm_tc a", BF16)
    n_rows, Kd = a_sorted.shape
    _chk(w, "grouped_gemm_tc w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(offsets, "grouped_gemm_tc offsets", I32, (E + 1,))
    dev = a_sorted.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    out = torch.empty(n_rows, nout, dtype=BF16 if swiglu_pair else F32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_tc")
    check(library().mi_grouped_gemm_tc_form(_ptr(a_sorted), _ptr(w), _ptr(offsets), _ptr(out), _ptr(_tc_status[dev]),
                                            n_rows, E, nout, Kd, 1 if swiglu_pair else 0,
                                            -1 if form is None else int(form), *_glu_args(glu),
                                            _row_scale(row_scale, n_rows, swiglu_pair, "grouped_gemm_tc"), _stream()),
          "grouped_gemm_tc")
    _tc_pending = True
    return out


def grouped_gemm_tc_inject_wait_fault(skip_k_block: int, wait_limit: int) -> None:
    """For the test of the bounded waits: the next :func:`grouped_gemm_tc` with ``form`` 0 or 1 leaves out
    the loads of one k block and waits at most ``wait_limit`` rounds, so a wait runs out, the kernel
    returns by itself, and :func:`check_tc_status` raises.  The launch after it is a normal one."""
    lib = library()
    lib.mi_grouped_gemm_tc_test_fault.argtypes = [ctypes.c_int, ctypes.c_uint]
    lib.mi_grouped_gemm_tc_test_fault.restype = None
    lib.mi_grouped_gemm_tc_test_fault(int(skip_k_block), int(wait_limit))


def check_tc_status() -> None:
    """Raise if a bounded wait inside a tensor-core kernel gave up since the last check (synchronises
    only when such a kernel was launched)."""
    global _tc_pending
    if not _tc_pending:
        return
    _tc_pending = False
    for dev, st in _tc_status.items():
        code = int(st.item())
        if code:
            st.zero_()
            from .library import KernelError
            raise KernelError(f"tcgen05 kernel on {dev}: a wait ran out (code {code}; grouped product: "
                              f"1 = producer waiting for a free stage, 2 = MMA waiting for data, "
                              f"3 = epilogue waiting for the accumulators; prefill attention: 11-19); "
                              f"results of that step are invalid")


def random_fill(out: torch.Tensor, key: Tuple[int, int], scale: float, offset: float) -> torch.Tensor:
    """Fill ``out`` (float32, bfloat16 or float16, contiguous) with the counter-based values of
    ``weights.random_init``: element ``i`` depends on ``(key, i)`` only."""
    _chk(out, "random_fill out")
    codes = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
    if out.dtype not in codes:
        raise TypeError(f"random_fill: dtype {out.dtype} is not float32, bfloat16 or float16")
    with torch.cuda.device(out.device):
        check(library().mi_random_fill(_ptr(out), codes[out.dtype], out.numel(), int(key[0]) & 0xFFFFFFFF,
                                       int(key[1]) & 0xFFFFFFFF, float(scale), float(offset), _stream()),
              "random_fill")
    return out


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                top_p: Optional[torch.Tensor] = None, u: Optional[torch.Tensor] = None,
                probs_scratch: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits [R, V]``; rows with temperature <= 0 are greedy."""
    _chk(logits, "sample_rows logits", F32)
    R, V = logits.shape
    _chk(temperature, "sample_rows temperature", F32, (R,))
    _chk(top_p, "sample_rows top_p", F32, (R,))
    _chk(u, "sample_rows u", F32, (R,))
    if temperature is not None and probs_scratch is None:
        probs_scratch = torch.empty(R, V, dtype=F32, device=logits.device)
    _chk(probs_scratch, "sample_rows scratch", F32, (R, V))
    if out is None:
        out = torch.empty(R, dtype=I32, device=logits.device)
    _chk(out, "sample_rows out", I32, (R,))
    check(library().mi_sample_rows(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(u), _ptr(probs_scratch),
                                   _ptr(out), R, V, _stream()), "sample_rows")
    return out


# --------------------------------------------------------------------------- #
# residual arrangements with two parts side by side, gated feed-forward with gelu
# --------------------------------------------------------------------------- #

def add2_rmsnorm_scalar(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor],
                        gain1: torch.Tensor, gain2: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                        rows: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``hidden += a + b`` (each optional; written back unless ``rows``), one root mean square per row, and the
    rows times ``gain1`` and (if given) times ``gain2``: two norms of the same residual whose weights are
    single numbers (float32 tensors of one element on the device)."""
    _chk(hidden, "add2_rmsnorm_scalar hidden", F32)
    T, H = hidden.shape
    _chk(a, "add2_rmsnorm_scalar a", F32, (T, H))
    _chk(b, "add2_rmsnorm_scalar b", F32, (T, H))
    _chk(rows, "add2_rmsnorm_scalar rows", I32)
    _chk(gain1, "add2_rmsnorm_scalar gain1", F32, (1,))
    _chk(gain2, "add2_rmsnorm_scalar gain2", F32, (1,))
    n = T if rows is None else rows.numel()
    out1 = torch.empty(n, H, dtype=out_dtype, device=hidden.device)
    out2 = torch.empty(n, H, dtype=out_dtype, device=hidden.device) if gain2 is not None else None
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, T, "add2_rmsnorm_scalar rows")
    check(library().mi_add2_rmsnorm_scalar(_ptr(hidden), _ptr(a), _ptr(b), _ptr(rows), _ptr(gain1), _ptr(gain2),
                                           _ptr(out1), _ptr(out2), _code(out1, "add2_rmsnorm_scalar out"), n, H,
                                           float(eps), _stream()), "add2_rmsnorm_scalar")
    return out1, out2


def out_norm_add(hidden: torch.Tensor, y, weight: torch.Tensor, eps: float, mult: float,
                 out_dtype: Optional[torch.dtype], groups: int = 1) -> Optional[torch.Tensor]:
    """``hidden += mult * y / rms(y) * weight`` row by row (float32), and the new rows once more in ``out_dtype``
    (None: not wanted).  With ``groups`` the root mean square is taken over each of that many equal consecutive
    parts of a row by itself.  ``y`` is a float32 tensor ``[T, H]`` or the tuple ``(rows, index, weights, extra,
    scale)`` of a sum of rows, ``y[t] = sum_k weights[t, k] rows[index[t, k]] + scale[t] extra[t]`` (``weights``
    None: ones, then ``index`` gives the number of slots; ``index`` None: rows in order), which is formed inside
    the kernel and never written out."""
    _chk(hidden, "out_norm_add hidden", F32)
    T, H = hidden.shape
    _chk(weight, "out_norm_add weight", None, (H,))
    yt = rows = index = wk = extra = scale = None
    K = 0
    if isinstance(y, torch.Tensor):
        yt = y
        _chk(yt, "out_norm_add y", F32, (T, H))
    else:
        rows, index, wk, extra, scale = y
        _chk(rows, "out_norm_add rows", F32, (None, H))
        _chk(index, "out_norm_add index", I32)
        _chk(wk, "out_norm_add weights", F32)
        _chk(extra, "out_norm_add extra", F32, (T, H))
        _chk(scale, "out_norm_add scale", F32, (T,))
        n = wk.numel() if wk is not None else (index.numel() if index is not None else rows.shape[0])
        if T == 0 or n % T:
            raise ValueError(f"out_norm_add: {n} slots for {T} rows")
        K = n // T
        if index is None and rows.shape[0] != T * K:
            raise ValueError(f"out_norm_add: {rows.shape[0]} rows in order for {T} x {K} slots")
        if DEBUG_BOUNDS:
            _dbg_range(index, 0, rows.shape[0], "out_norm_add index")
    out = torch.empty(T, H, dtype=out_dtype, device=hidden.device) if out_dtype is not None else None
    if groups != 1:
        if groups < 1 or H % groups:
            raise ValueError(f"out_norm_add: rows of {H} do not split into {groups} groups")
        check(library().mi_out_norm_add_groups(
            _ptr(hidden), _ptr(yt), _ptr(rows), _ptr(index), _ptr(wk), _ptr(extra), _ptr(scale), K, _ptr(weight),
            _code(weight, "out_norm_add weight"), _ptr(out), _CODES[out_dtype] if out_dtype is not None else 0, T, H,
            float(eps), float(mult), int(groups), _stream()), "out_norm_add")
        return out
    check(library().mi_out_norm_add(_ptr(hidden), _ptr(yt), _ptr(rows), _ptr(index), _ptr(wk), _ptr(extra), _ptr(scale),
                                    K, _ptr(weight), _code(weight, "out_norm_add weight"), _ptr(out),
                                    _CODES[out_dtype] if out_dtype is not None else 0, T, H, float(eps), float(mult),
                                    _stream()), "out_norm_add")
    return out


def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x / rms * weight`` of float32 rows ``[T, H]`` with the root mean square (``eps`` inside the root) taken
    over each of ``groups`` equal consecutive parts of a row by itself; ``rows`` (int32) picks the rows that are
    wanted.  Returns ``[T or len(rows), H]`` in ``out_dtype``."""
    _chk(x, "group_rmsnorm x", F32)
    T, H = x.shape
    _chk(weight, "group_rmsnorm weight", None, (H,))
    _chk(rows, "group_rmsnorm rows", I32)
    if groups < 1 or H % groups:
        raise ValueError(f"group_rmsnorm: rows of {H} do not split into {groups} groups")
    n = rows.numel() if rows is not None else T
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, T, "group_rmsnorm rows")
    out = torch.empty(n, H, dtype=out_dtype, device=x.device)
    check(library().mi_group_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _code(weight, "group_rmsnorm weight"), _ptr(out),
                                     _code(out, "group_rmsnorm out"), n, H, int(groups), float(eps), _stream()),
          "group_rmsnorm")
    return out


def softcap_rows(z: torch.Tensor, cap: float) -> torch.Tensor:
    """``z <- cap * tanh(z / cap)`` in place (float32)."""
    _chk(z, "softcap_rows z", F32)
    check(library().mi_softcap_rows(_ptr(z), z.numel(), float(cap), _stream()), "softcap_rows")
    return z


def cast_rows(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Float32 rows rounded to ``out_dtype``."""
    _chk(x, "cast_rows x", F32)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(library().mi_cast_rows(_ptr(x), _ptr(out), _code(out, "cast_rows out"), x.numel(), _stream()), "cast_rows")
    return out


def geglu_tanh(gu: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(gu[:, :I]) * gu[:, I:]`` in the type of ``gu``."""
    _chk(gu, "geglu_tanh gu")
    T, two_i = gu.shape
    if two_i % 2:
        raise ValueError("geglu_tanh: the row holds gate and up halves of equal size")
    out = torch.empty(T, two_i // 2, dtype=gu.dtype, device=gu.device)
    check(library().mi_geglu_tanh(_ptr(gu), _ptr(out), _code(gu, "geglu_tanh gu"), T, two_i // 2, _stream()),
          "geglu_tanh")
    return out


def concat_cast(hidden: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], other: torch.Tensor,
                out_dtype: torch.dtype) -> torch.Tensor:
    """``[hidden + a + b | other]`` row by row in ``out_dtype`` (``hidden`` is left as it is)."""
    _chk(hidden, "concat_cast hidden", F32)
    T, H = hidden.shape
    _chk(a, "concat_cast a", F32, (T, H))
    _chk(b, "concat_cast b", F32, (T, H))
    _chk(other, "concat_cast other", F32, (T, H))
    out = torch.empty(T, 2 * H, dtype=out_dtype, device=hidden.device)
    check(library().mi_concat_cast(_ptr(hidden), _ptr(a), _ptr(b), _ptr(other), _ptr(out), _code(out, "concat_cast out"),
                                   T, H, _stream()), "concat_cast")
    return out


def rows_plus_vec(hidden: torch.Tensor, y: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """``hidden[t] = y[t] + vec`` (float32 rows; ``vec`` float32 or bfloat16)."""
    _chk(hidden, "rows_plus_vec hidden", F32)
    T, H = hidden.shape
    _chk(y, "rows_plus_vec y", F32, (T, H))
    _chk(vec, "rows_plus_vec vec", None, (H,))
    check(library().mi_rows_plus_vec(_ptr(hidden), _ptr(y), _ptr(vec), _code(vec, "rows_plus_vec vec"), T, H, _stream()),
          "rows_plus_vec")
    return hidden


# --------------------------------------------------------------------------- #
# mixers with a fixed-size state per request
# --------------------------------------------------------------------------- #

CONV_MAX_TAPS = 8


def causal_conv_silu(x: torch.Tensor, col0: int, channels: int, w: torch.Tensor, bias: Optional[torch.Tensor],
                     state: torch.Tensor, state_offset: int, q_start: torch.Tensor, req_of_token: torch.Tensor,
                     state_slot: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time per channel, then silu, on the columns ``col0 .. col0 + channels`` of the
    float32 rows ``x``; returns float32 ``[T, channels]``.  ``w [channels, taps]`` (the last column weighs the
    current token).  The ``taps - 1`` inputs before a request's portion come from ``state[slot,
    state_offset : state_offset + (taps-1)*channels]`` (time-major), which is brought up to date afterwards."""
    _chk(x, "causal_conv_silu x", F32)
    T, ld = x.shape
    C = int(channels)
    _chk(w, "causal_conv_silu w", None, (C, None))
    taps = w.shape[1]
    _chk(bias, "causal_conv_silu bias", w.dtype, (C,))
    _chk(state, "causal_conv_silu state", F32)
    if col0 < 0 or col0 + C > ld or state.dim() != 2 or state_offset + (taps - 1) * C > state.shape[1]:
        raise ValueError("causal_conv_silu: columns or state section out of range")
    B = state_slot.numel()
    _chk(q_start, "causal_conv_silu q_start", I32, (B + 1,))
    _chk(req_of_token, "causal_conv_silu req_of_token", I32, (T,))
    _chk(state_slot, "causal_conv_silu state_slot", I32, (B,))
    if DEBUG_BOUNDS:
        _dbg_range(state_slot, 0, state.shape[0], "causal_conv_silu state_slot")
        _dbg_range(req_of_token, 0, B, "causal_conv_silu req_of_token")
    out = torch.empty(T, C, dtype=F32, device=x.device)
    check(library().mi_causal_conv_silu(x.data_ptr() + 4 * col0, ld, _ptr(w), _ptr(bias), _code(w, "causal_conv_silu w"),
                                        state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start),
                                        _ptr(req_of_token), _ptr(state_slot), _ptr(out), C, C, taps, T, B, _stream()),
          "causal_conv_silu")
    return out


def causal_conv_residual(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, state_offset: int,
                         q_start: torch.Tensor, req_of_token: torch.Tensor, state_slot: torch.Tensor,
                         out_dtype: torch.dtype) -> torch.Tensor:
    """``x + conv(x)`` of float32 rows ``[T, C]``: a causal convolution over time per channel without an
    activation, ``conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j)`` with ``w [C, taps]``.  The ``taps - 1`` rows
    before a request's portion come from ``state[slot, state_offset : state_offset + (taps-1)*C]`` (time-major),
    which is brought up to date afterwards.  Returns ``[T, C]`` in ``out_dtype``."""
    _chk(x, "causal_conv_residual x", F32)
    T, C = x.shape
    _chk(w, "causal_conv_residual w", None, (C, None))
    taps = w.shape[1]
    _chk(state, "causal_conv_residual state", F32)
    if state.dim() != 2 or state_offset + (taps - 1) * C > state.shape[1]:
        raise ValueError("causal_conv_residual: state section out of range")
    B = state_slot.numel()
    _chk(q_start, "causal_conv_residual q_start", I32, (B + 1,))
    _chk(req_of_token, "causal_conv_residual req_of_token", I32, (T,))
    _chk(state_slot, "causal_conv_residual state_slot", I32, (B,))
    if DEBUG_BOUNDS:
        _dbg_range(state_slot, 0, state.shape[0], "causal_conv_residual state_slot")
        _dbg_range(req_of_token, 0, B, "causal_conv_residual req_of_token")
    out = torch.empty(T, C, dtype=out_dtype, device=x.device)
    check(library().mi_causal_conv_residual(_ptr(x), C, _ptr(w), _code(w, "causal_conv_residual w"),
                                            state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start),
                                            _ptr(req_of_token), _ptr(state_slot), _ptr(out),
                                            _code(out, "causal_conv_residual out"), C, C, taps, T, B, _stream()),
          "causal_conv_residual")
    return out


def norm_conv_decode(hidden: torch.Tensor, norm_weight: torch.Tensor, groups: int, eps: float, w: torch.Tensor,
                     state: torch.Tensor, state_offset: int, q_start: torch.Tensor, state_slot: torch.Tensor,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """:func:`group_rmsnorm` and :func:`causal_conv_residual` of a step in which EVERY request brings exactly one
    token, in one launch: ``n = norm(hidden)``, ``n + conv(n)`` over the request's last ``taps - 1`` normalised rows
    and this one, the state moved on by one token.  ``norm_weight`` and ``w [C, taps]`` float32.  Returns ``[T, C]``
    in ``out_dtype``.  (Its sums run in another order than the two kernels': the two agree within rounding.)"""
    _chk(hidden, "norm_conv_decode hidden", F32)
    T, C = hidden.shape
    B = state_slot.numel()
    if T != B:
        raise ValueError(f"norm_conv_decode: {T} rows for {B} requests (this kernel takes one token of each)")
    _chk(norm_weight, "norm_conv_decode norm weight", F32, (C,))
    _chk(w, "norm_conv_decode w", F32, (C, None))
    taps = w.shape[1]
    _chk(state, "norm_conv_decode state", F32)
    if state.dim() != 2 or state_offset + (taps - 1) * C > state.shape[1] or groups < 1 or C % groups:
        raise ValueError("norm_conv_decode: state section or groups out of range")
    _chk(q_start, "norm_conv_decode q_start", I32, (B + 1,))
    _chk(state_slot, "norm_conv_decode state_slot", I32, (B,))
    if DEBUG_BOUNDS:
        _dbg_range(state_slot, 0, state.shape[0], "norm_conv_decode state_slot")
    out = torch.empty(T, C, dtype=out_dtype, device=hidden.device)
    check(library().mi_norm_conv_decode(_ptr(hidden), _ptr(norm_weight), int(groups), float(eps), _ptr(w),
                                        state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start),
                                        _ptr(state_slot), _ptr(out), _code(out, "norm_conv_decode out"), B, C, taps,
                                        _stream()), "norm_conv_decode")
    return out


DELTA_FORMS = {"channel_decay": 0, "head_decay": 1, "sigmoid_decay": 2}


def scan_segments(max_q_len: int, min_tokens: int, segment_tokens: int, max_segments: int) -> Tuple[int, int]:
    """``(segments, tokens per segment)`` for a step whose longest portion has ``max_q_len`` tokens: one segment
    below ``min_tokens``; else runs of about ``segment_tokens`` tokens (whole chunks of 16), at most
    ``max_segments`` of them."""
    if max_q_len < max(min_tokens, 2):
        return 1, 0
    segs = max(2, min(max_segments, -(-max_q_len // segment_tokens)))
    per = -(-max_q_len // segs)
    per = -(-per // 16) * 16
    return -(-max_q_len // per), per


def delta_scan(qkv: torch.Tensor, beta_raw: Optional[torch.Tensor], beta_col: int, a_raw: torch.Tensor, a_col: int,
               a_log: Optional[torch.Tensor], dt_bias: torch.Tensor, state: torch.Tensor, state_offset: int,
               q_start: torch.Tensor, state_slot: torch.Tensor, heads: int, key_heads: int, d: int, dv: int,
               q_scale: float, form: str = "channel_decay", tau: float = 1.0, segments: int = 1,
               segment_tokens: int = 0) -> torch.Tensor:
    """Gated delta rule with a decay per head and key channel, token by token over every request's portion.

    ``form`` ``head_decay``: ONE decay per head (``a_raw`` holds ``heads`` columns and ``dt_bias`` ``heads``
    numbers).  ``form`` ``sigmoid_decay``: gated linear attention, ``S <- diag(g) S + k v^T; o = S^T q`` with
    q (times ``q_scale``) and k as they are and ``g = sigmoid(a + dt_bias)^(1 / tau)`` per head and key channel;
    ``beta_raw`` and ``a_log`` are not read.

    ``segments`` > 1 (``sigmoid_decay`` only, whose transition is diagonal): every request's portion is cut into that
    many runs of ``segment_tokens`` tokens which are walked side by side from zero; the runs' final states are then
    chained into every run's true start state and the read-outs corrected by ``(b_t q_t)^T S_start`` with ``b_t`` the
    product of the decays since the run's start.  The chain of dependent steps is a run's length, not the portion's;
    the sums of a token run in another order than in one piece, so the two agree within rounding, not bit for bit.

    ``qkv`` float32 ``[T, 2*key_heads*d + heads*dv]`` (q | k | v after their convolutions; the rows may go on
    with columns that are not read); ``beta_raw`` holds
    the ``heads`` write strengths before the sigmoid from column ``beta_col``; ``a_raw`` the ``heads*d`` decay
    inputs before ``dt_bias`` and the softplus from column ``a_col``.  Per head, with unit q (times
    ``q_scale``) and unit k: ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` where
    ``g = exp(-exp(a_log) * softplus(a + dt_bias))``.  ``S`` (``heads x d x dv`` floats) lives in
    ``state[slot, state_offset:]``.  Returns ``o`` float32 ``[T, heads*dv]``."""
    _chk(qkv, "delta_scan qkv", F32)
    T = qkv.shape[0]
    if qkv.shape[1] < 2 * key_heads * d + heads * dv:
        raise ValueError("delta_scan: the rows of qkv do not hold q, k and v of the given sizes")
    if form not in DELTA_FORMS:
        raise ValueError(f"delta_scan: form '{form}' is not one of {sorted(DELTA_FORMS)}")
    n_decay = heads if form == "head_decay" else heads * d
    _chk(beta_raw, "delta_scan beta_raw", F32)
    _chk(a_raw, "delta_scan a_raw", F32)
    _chk(a_log, "delta_scan a_log", F32, (heads,))
    _chk(dt_bias, "delta_scan dt_bias", F32, (n_decay,))
    _chk(state, "delta_scan state", F32)
    B = state_slot.numel()
    _chk(q_start, "delta_scan q_start", I32, (B + 1,))
    _chk(state_slot, "delta_scan state_slot", I32, (B,))
    if form != "sigmoid_decay" and (beta_raw is None or a_log is None):
        raise ValueError("delta_scan: the delta rule needs its write strengths and decay rates")
    if ((beta_raw is not None and beta_col + heads > beta_raw.shape[1]) or a_col + n_decay > a_raw.shape[1]
            or state_offset + heads * d * dv > state.shape[1]):
        raise ValueError("delta_scan: columns or state section out of range")
    if DEBUG_BOUNDS:
        _dbg_range(state_slot, 0, state.shape[0], "delta_scan state_slot")
    out = torch.empty(T, heads * dv, dtype=F32, device=qkv.device)
    # unit vectors, decays and write strengths of all tokens, made ready by a kernel before the walk
    prep = torch.empty(T * heads * library().mi_delta_scan_prep_row(d), dtype=F32, device=qkv.device)
    if segments > 1:
        if form != "sigmoid_decay" or segment_tokens < 1 or B * segments > 65535:
            raise ValueError(f"delta_scan: {segments} segments of {segment_tokens} tokens for {B} requests in the form "
                             f"'{form}' (segments are built for 'sigmoid_decay')")
        seg_state = torch.empty(B * segments * heads * d * dv, dtype=F32, device=qkv.device)
        qt = torch.empty(T * heads * d, dtype=F32, device=qkv.device)
        bend = torch.empty(B * segments * heads * d, dtype=F32, device=qkv.device)
        check(library().mi_gla_scan_segments(
            _ptr(qkv), qkv.shape[1], a_raw.data_ptr() + 4 * a_col, a_raw.shape[1], _ptr(dt_bias),
            state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start), _ptr(state_slot), _ptr(out), _ptr(prep), T,
            B, heads, d, dv, float(q_scale), float(tau), int(segments), int(segment_tokens), _ptr(seg_state), _ptr(qt),
            _ptr(bend), _stream()), "delta_scan")
        return out
    if form == "channel_decay":
        check(library().mi_delta_scan(_ptr(qkv), qkv.shape[1], beta_raw.data_ptr() + 4 * beta_col, beta_raw.shape[1],
                                      a_raw.data_ptr() + 4 * a_col, a_raw.shape[1], _ptr(a_log), _ptr(dt_bias),
                                      state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start),
                                      _ptr(state_slot), _ptr(out), _ptr(prep), T, B, heads, key_heads, d, dv,
                                      float(q_scale), _stream()), "delta_scan")
        return out
    check(library().mi_delta_scan_form(
        _ptr(qkv), qkv.shape[1], None if beta_raw is None else beta_raw.data_ptr() + 4 * beta_col,
        0 if beta_raw is None else beta_raw.shape[1], a_raw.data_ptr() + 4 * a_col, a_raw.shape[1], _ptr(a_log),
        _ptr(dt_bias), state.data_ptr() + 4 * state_offset, state.shape[1], _ptr(q_start), _ptr(state_slot), _ptr(out),
        _ptr(prep), T, B, heads, key_heads, d, dv, float(q_scale), DELTA_FORMS[form], float(tau), _stream()),
          "delta_scan")
    return out


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             d_skip: torch.Tensor, state: torch.Tensor, state_offset: int, q_start: torch.Tensor,
             state_slot: torch.Tensor, heads: int, groups: int, n_state: int, head_dim: int) -> torch.Tensor:
    """State-space recurrence with a scalar decay per head: ``dt = softplus(dt_raw + dt_bias)``,
    ``S <- exp(-exp(a_log) dt) S + dt B x^T``, ``y = S^T C + d_skip x``.  ``xbc`` float32
    ``[T, heads*head_dim + 2*groups*n_state]`` (x | B | C after the convolution); ``S``
    (``heads x n_state x head_dim`` floats) lives in ``state[slot, state_offset:]``.  Returns float32
    ``[T, heads*head_dim]``."""
    _chk(xbc, "ssd_scan xbc", F32)
    T = xbc.shape[0]
    if xbc.shape[1] != heads * head_dim + 2 * groups * n_state:
        raise ValueError("ssd_scan: the rows of xbc do not hold x, B and C of the given sizes")
    _chk(dt_raw, "ssd_scan dt_raw", F32)
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _chk(t, "ssd_scan " + name, F32, (heads,))
    _chk(state, "ssd_scan state", F32)
    B = state_slot.numel()
    _chk(q_start, "ssd_scan q_start", I32, (B + 1,))
    _chk(state_slot, "ssd_scan state_slot", I32, (B,))
    if dt_col + heads > dt_raw.shape[1] or state_offset + heads * n_state * head_dim > state.shape[1]:
        raise ValueError("ssd_scan: columns or state section out of range")
    if DEBUG_BOUNDS:
        _dbg_range(state_slot, 0, state.shape[0], "ssd_scan state_slot")
    out = torch.empty(T, heads * head_dim, dtype=F32, device=xbc.device)
    check(library().mi_ssd_scan(_ptr(xbc), xbc.shape[1], dt_raw.data_ptr() + 4 * dt_col, dt_raw.shape[1], _ptr(dt_bias),
                                _ptr(a_log), _ptr(d_skip), state.data_ptr() + 4 * state_offset, state.shape[1],
                                _ptr(q_start), _ptr(state_slot), _ptr(out), B, heads, groups, n_state, head_dim,
                                _stream()), "ssd_scan")
    return out


def gated_group_rmsnorm(y: torch.Tensor, gate: torch.Tensor, gate_col: int, weight: torch.Tensor, groups: int,
                        gate_first: bool, eps: float, out_dtype: torch.dtype, silu_after: bool = False) -> torch.Tensor:
    """RMS norm over ``groups`` equal parts of every float32 row of ``y`` with a gate from the columns
    ``gate_col ..`` of ``gate``: ``gate_first``: ``norm(y * silu(gate)) * w``; else ``norm(y) * w *
    sigmoid(gate)``, or, with ``silu_after``, ``norm(y) * w * silu(gate)``.  Column ``c`` uses
    ``weight[c % len(weight)]``."""
    _chk(y, "gated_group_rmsnorm y", F32)
    T, n = y.shape
    _chk(gate, "gated_group_rmsnorm gate", F32)
    _chk(weight, "gated_group_rmsnorm weight")
    if gate.shape[0] != T or gate_col + n > gate.shape[1] or n % groups or n % weight.numel():
        raise ValueError("gated_group_rmsnorm: gate columns, groups or weight do not fit the rows")
    out = torch.empty(T, n, dtype=out_dtype, device=y.device)
    check(library().mi_gated_group_rmsnorm(_ptr(y), gate.data_ptr() + 4 * gate_col, gate.shape[1], _ptr(weight),
                                           _code(weight, "gated_group_rmsnorm weight"), weight.numel(), _ptr(out),
                                           _code(out, "gated_group_rmsnorm out"), T, n, int(groups),
                                           0 if gate_first else (2 if silu_after else 1), float(eps), _stream()),
          "gated_group_rmsnorm")
    return out


# --------------------------------------------------------------------------- #
# attention with capped scores mixed over the heads
# --------------------------------------------------------------------------- #

def rope_store(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dim: int,
               slot_mapping: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, nh: int, nkv: int,
               dk: int, dv: int, page_size: int, out_dtype: torch.dtype,
               q_gain: Optional[torch.Tensor] = None, k_gain: Optional[torch.Tensor] = None,
               eps: float = 0.0, neighbours: bool = False, v_first: Optional[torch.Tensor] = None,
               blend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotary encoding of the first ``rot_dim`` dimensions of the query and key heads of float32 rows
    ``[nh*dk | nkv*dk | nkv*dv]``, cache write of keys ``[pages, nkv, page_size, dk]`` and values
    ``[pages, nkv, page_size, dv]`` (slot -1: not written).  With ``q_gain`` and ``k_gain`` (float32
    ``[dk]``) every query and key head is first divided by its root mean square (``eps`` inside the root) and
    multiplied by the gain.  The rotation pairs dimension ``i`` with ``i + rot_dim / 2``, or, with
    ``neighbours``, dimension ``2i`` with ``2i + 1``.  With ``v_first`` (float32 ``[T, nkv*dv]``; rows may be a
    column slice of a wider matrix) and ``blend`` (one float32 on the device) the values that are cached are
    ``(1 - blend) v + blend v_first``.  Returns ``q [T, nh, dk]`` in ``out_dtype``."""
    vf_stride = 0
    if v_first is not None:
        if (not v_first.is_cuda or v_first.dtype != F32 or v_first.dim() != 2 or v_first.stride(1) != 1
                or tuple(v_first.shape) != (qkv.shape[0], nkv * dv)):
            raise ValueError(f"rope_store: v_first must be float32 [{qkv.shape[0]}, {nkv * dv}] with unit column stride")
        _chk(blend, "rope_store blend", F32, (1,))
        if blend is None:
            raise ValueError("rope_store: v_first comes with its blending weight")
        vf_stride = v_first.stride(0)
    _chk(q_gain, "rope_store q_gain", F32, (dk,))
    _chk(k_gain, "rope_store k_gain", F32, (dk,))
    _chk(qkv, "rope_store qkv", F32)
    T = qkv.shape[0]
    _chk(qkv, "rope_store qkv", F32, (T, (nh + nkv) * dk + nkv * dv))
    _chk(positions, "rope_store positions", I32, (T,))
    _chk(inv_freq, "rope_store inv_freq", F32)
    if rot_dim and (inv_freq is None or inv_freq.numel() != rot_dim // 2):
        raise ValueError(f"rope_store: {rot_dim} rotary dims need {rot_dim // 2} frequencies")
    _chk(slot_mapping, "rope_store slot_mapping", I32, (T,))
    _chk(k_cache, "rope_store k_cache", out_dtype, (None, nkv, page_size, dk))
    _chk(v_cache, "rope_store v_cache", out_dtype, (None, nkv, page_size, dv))
    q = torch.empty(T, nh, dk, dtype=out_dtype, device=qkv.device)
    if DEBUG_BOUNDS:
        _dbg_range(slot_mapping, -1, k_cache.shape[0] * page_size, "rope_store slot_mapping")
    check(library().mi_rope_store(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(slot_mapping), _ptr(q),
                                  _ptr(k_cache), _ptr(v_cache), _code(q, "rope_store q"), T, nh, nkv, dk, dv,
                                  int(rot_dim), page_size, _ptr(q_gain), _ptr(k_gain), float(eps),
                                  int(bool(neighbours)), _ptr(v_first), int(vf_stride),
                                  _ptr(blend) if v_first is not None else None, _stream()),
          "rope_store")
    return q


def attention_mix_supported(nh: int, nkv: int, dk: int, dv: int, dtype: torch.dtype) -> bool:
    return bool(library().mi_attn_mix_supported(nh, nkv, dk, dv, 4 if dtype == F32 else 2))


def attention_mix(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, mix: Optional[torch.Tensor],
                  block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int,
                  window: int, scale: float, softcap: float, keep_first: int = 0,
                  value_dim: int = 0, sink: bool = False, head_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a ragged batch over the paged cache with ``score <- softcap * tanh(score / softcap)``
    (``softcap`` 0: none) and then ``score_h <- sum_g mix[h, g] score_g`` (``mix`` None: none) before the
    softmax over the visible keys: key ``j`` is visible from position ``p`` iff ``j <= p`` and (``window`` is
    0 or ``j > p - window`` or ``j < keep_first``).  With ``value_dim`` a token's value is the first
    ``value_dim`` numbers of its row of ``v_cache`` (which may be the key cache itself).  With ``sink`` the
    softmax counts one key more, of score 0 and without a value: ``p_j = exp(s_j) / (1 + sum exp(s_j))``.
    With ``head_bias`` (float32 ``[nh]``) there is no softmax: a visible key's weight is
    ``logistic(score + head_bias[h])`` by itself, not normalised over the keys.
    Returns ``[T, nh, dv]``."""
    _chk(q, "attention_mix q")
    _chk(head_bias, "attention_mix head_bias", F32, (q.shape[1],))
    T, nh, dk = q.shape
    _chk(k_cache, "attention_mix k_cache", q.dtype)
    _, nkv, page_size, dk2 = k_cache.shape
    _chk(v_cache, "attention_mix v_cache", q.dtype, (k_cache.shape[0], nkv, page_size, None))
    vrs = v_cache.shape[3]
    dv = int(value_dim) or vrs
    if dv > vrs:
        raise ValueError(f"attention_mix: values of {dv} in rows of {vrs}")
    if dk2 != dk:
        raise ValueError(f"attention_mix: key size of q ({dk}) and of the cache ({dk2}) differ")
    _chk(mix, "attention_mix mix", F32, (nh, nh))
    _chk(block_table, "attention_mix block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "attention_mix q_start", I32, (B + 1,))
    _chk(kv_len, "attention_mix kv_len", I32, (B,))
    out = torch.empty(T, nh, dv, dtype=q.dtype, device=q.device)
    if DEBUG_BOUNDS:
        _dbg_batch("attention_mix", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window),
                   int(max_q_len))
    if head_bias is not None:
        check(library().mi_attn_mix_form(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "attention_mix q"), _ptr(mix),
                                         _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), B, int(max_q_len),
                                         nh, nkv, dk, dv, page_size, max_pages, int(window), float(scale),
                                         float(softcap), int(keep_first), vrs, int(bool(sink)), _ptr(head_bias),
                                         _stream()), "attention_mix")
        return out
    check(library().mi_attn_mix(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "attention_mix q"), _ptr(mix),
                                _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), B, int(max_q_len), nh, nkv,
                                dk, dv, page_size, max_pages, int(window), float(scale), float(softcap),
                                int(keep_first), vrs, int(bool(sink)), _stream()), "attention_mix")
    return out


def attention_mix_tc_supported(nh: int, nkv: int, dk: int, dv: int) -> bool:
    """The tensor-core form (bfloat16) takes these sizes."""
    return bool(library().mi_attn_mix_tc_supported(nh, nkv, dk, dv))


def attention_mix_tc_splits(span: int, keep_first: int = 0) -> int:
    """Blocks over the keys that a step of single tokens is cut into when a query sees up to ``span`` keys
    of its window (one block more for kept first keys)."""
    return int(library().mi_attn_mix_tc_splits(int(span))) + (1 if keep_first > 0 else 0)


def attention_mix_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, mix: Optional[torch.Tensor],
                     block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int,
                     window: int, scale: float, softcap: float, splits: int = 1,
                     part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                     keep_first: int = 0, value_dim: int = 0, sink: bool = False,
                     head_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`attention_mix` on the tensor cores (bfloat16).  ``splits > 1`` (steps of one token per request
    only): the keys of a request are cut into ``splits`` blocks whose partial results go through the float32
    scratch ``part_o`` (``B * splits * nh * dv``) and ``part_ml`` (``B * splits * nh * 2``); with
    ``keep_first`` the last of the blocks takes the kept first keys, so ``splits`` counts one more
    (:func:`attention_mix_tc_splits`)."""
    _chk(q, "attention_mix_tc q", BF16)
    T, nh, dk = q.shape
    _chk(head_bias, "attention_mix_tc head_bias", F32, (nh,))
    _chk(k_cache, "attention_mix_tc k_cache", BF16, (None, None, None, dk))
    _, nkv, page_size, _ = k_cache.shape
    _chk(v_cache, "attention_mix_tc v_cache", BF16, (k_cache.shape[0], nkv, page_size, None))
    vrs = v_cache.shape[3]
    dv = int(value_dim) or vrs
    _chk(mix, "attention_mix_tc mix", F32, (nh, nh))
    _chk(block_table, "attention_mix_tc block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "attention_mix_tc q_start", I32, (B + 1,))
    _chk(kv_len, "attention_mix_tc kv_len", I32, (B,))
    if splits > 1:
        _chk(part_o, "attention_mix_tc part_o", F32)
        _chk(part_ml, "attention_mix_tc part_ml", F32)
        if part_o is None or part_ml is None or part_o.numel() < B * splits * nh * dv or part_ml.numel() < B * splits * nh * 2:
            raise ValueError("attention_mix_tc: scratch for the partial results is missing or too small")
    out = torch.empty(T, nh, dv, dtype=BF16, device=q.device)
    if DEBUG_BOUNDS:
        _dbg_batch("attention_mix_tc", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window),
                   int(max_q_len))
    if head_bias is not None:
        check(library().mi_attn_mix_tc_form(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(mix), _ptr(block_table),
                                            _ptr(q_start), _ptr(kv_len), _ptr(out), _ptr(part_o), _ptr(part_ml), B,
                                            int(max_q_len), nh, nkv, dk, dv, page_size, max_pages, int(window),
                                            float(scale), float(softcap), int(splits), int(keep_first), vrs,
                                            int(bool(sink)), _ptr(head_bias), _stream()), "attention_mix_tc")
        return out
    check(library().mi_attn_mix_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(mix), _ptr(block_table), _ptr(q_start),
                                   _ptr(kv_len), _ptr(out), _ptr(part_o), _ptr(part_ml), B, int(max_q_len), nh, nkv, dk,
                                   dv, page_size, max_pages, int(window), float(scale), float(softcap), int(splits),
                                   int(keep_first), vrs, int(bool(sink)), _stream()), "attention_mix_tc")
    return out


def clamped_glu(gu: torch.Tensor, limit: float, slope: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``g * logistic(slope * g) * (u + 1)`` with ``g = min(gate, limit)`` and ``u = clamp(up, -limit, limit)``
    of float32 rows ``[T, 2 I]`` (gate half, then up half); returns ``[T, I]`` in ``out_dtype``."""
    _chk(gu, "clamped_glu", F32)
    T, I2 = gu.shape
    if I2 % 2:
        raise ValueError("clamped_glu: rows hold a gate half and an up half")
    out = torch.empty(T, I2 // 2, dtype=out_dtype, device=gu.device)
    check(library().mi_clamped_glu(_ptr(gu), _ptr(out), _code(out, "clamped_glu out"), T, I2 // 2, float(limit),
                                   float(slope), _stream()), "clamped_glu")
    return out


def dense_f32_heads(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, x_col: int = 0,
                    x_head_stride: Optional[int] = None, out_col: int = 0,
                    out_head_stride: Optional[int] = None) -> torch.Tensor:
    """A product per head in true float32: ``out[t, h] = w[h] @ x[t, h]`` with ``w [H, N, K]``.  ``x`` is
    ``[T, *]`` float32 rows in which head ``h`` starts at column ``x_col + h * x_head_stride`` (default: heads
    of ``K`` side by side); ``out`` likewise (default ``[T, H * N]``).  The same fixed chain of additions per
    element as :func:`dense_f32`."""
    _chk(x, "dense_f32_heads x", F32)
    _chk(w, "dense_f32_heads w", F32)
    H, N, K = w.shape
    T = x.shape[0]
    xs = K if x_head_stride is None else int(x_head_stride)
    os_ = N if out_head_stride is None else int(out_head_stride)
    lda = x.numel() // max(T, 1)
    if out is None:
        out = torch.empty(T, H * N, dtype=F32, device=x.device)
    _chk(out, "dense_f32_heads out", F32)
    ldc = out.numel() // max(T, 1)
    if x_col + (H - 1) * xs + K > lda or out_col + (H - 1) * os_ + N > ldc:
        raise ValueError("dense_f32_heads: the heads do not fit the rows")
    check(library().mi_dense_f32_batched(x.data_ptr() + 4 * x_col, _ptr(w), out.data_ptr() + 4 * out_col, T, N, K,
                                         lda, ldc, H, xs, N * K, os_, _stream()), "dense_f32_heads")
    return out


def latent_store(src: torch.Tensor, col0: int, positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                 gain: torch.Tensor, eps: float, slot_mapping: torch.Tensor, cache: torch.Tensor, rank: int,
                 rot_dim: int) -> None:
    """The cached row of every token: columns ``col0 .. col0 + rank`` of the float32 rows ``src`` divided by
    their root mean square (``eps`` inside the root) times ``gain``, then ``rot_dim`` columns rotated by
    position in pairs of neighbours.  ``cache [pages, 1, page_size, rank + rot_dim]``; slot -1: not written."""
    _chk(src, "latent_store src", F32)
    T, ld = src.shape
    _chk(positions, "latent_store positions", I32, (T,))
    _chk(inv_freq, "latent_store inv_freq", F32, (rot_dim // 2,))
    _chk(gain, "latent_store gain", F32, (rank,))
    _chk(slot_mapping, "latent_store slot_mapping", I32, (T,))
    _chk(cache, "latent_store cache", None, (None, 1, None, rank + rot_dim))
    if DEBUG_BOUNDS:
        _dbg_range(slot_mapping, -1, cache.shape[0] * cache.shape[2], "latent_store slot_mapping")
    check(library().mi_latent_store(_ptr(src), ld, int(col0), _ptr(positions), _ptr(inv_freq), _ptr(gain), float(eps),
                                    _ptr(slot_mapping), _ptr(cache), _code(cache, "latent_store cache"), T, int(rank),
                                    int(rot_dim), _stream()), "latent_store")


def latent_query(q: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], heads: int, dim: int,
                 rot_dim: int, rank: int, out_dtype: torch.dtype, want_plain: bool):
    """Float32 rows of ``heads`` queries ``[dim unrotated | rot_dim rotated]``: returns ``(q_full, q_plain)``
    where ``q_full [T, heads, rank + rot_dim]`` (``out_dtype``) has its last ``rot_dim`` columns filled with the
    parts rotated by position (pairs of neighbours; the first ``rank`` are left for the folded queries) and
    ``q_plain [T, heads, dim]`` holds the unrotated parts in ``out_dtype`` (None unless wanted)."""
    _chk(q, "latent_query q", F32)
    T = q.shape[0]
    _chk(q, "latent_query q", F32, (T, heads * (dim + rot_dim)))
    _chk(positions, "latent_query positions", I32, (T,))
    _chk(inv_freq, "latent_query inv_freq", F32, (rot_dim // 2,))
    q_full = torch.empty(T, heads, rank + rot_dim, dtype=out_dtype, device=q.device)
    q_plain = torch.empty(T, heads, dim, dtype=out_dtype, device=q.device) if want_plain else None
    check(library().mi_latent_query(_ptr(q), _ptr(positions), _ptr(inv_freq), _ptr(q_plain), _ptr(q_full),
                                    _code(q_full, "latent_query out"), T, heads, dim, rot_dim, rank, _stream()),
          "latent_query")
    return q_full, q_plain


def sigmoid_gate(a: torch.Tensor, head_major: bool, g: torch.Tensor, col0: int, heads: int, size: int) -> torch.Tensor:
    """``out[t, h, :] = a[t, h, :] * logistic(g[t, col0 + h * size : ...])``; ``a`` is ``[T, heads, size]`` or,
    with ``head_major``, ``[heads, T, size]``; ``g`` float32 rows.  Returns ``[T, heads * size]`` in ``a``'s type."""
    _chk(a, "sigmoid_gate a")
    _chk(g, "sigmoid_gate g", F32)
    T = g.shape[0]
    if a.numel() != T * heads * size:
        raise ValueError("sigmoid_gate: sizes of the heads' outputs and of the gate differ")
    out = torch.empty(T, heads * size, dtype=a.dtype, device=a.device)
    a_head, a_tok = (T * size, size) if head_major else (size, heads * size)
    check(library().mi_sigmoid_gate(_ptr(a), a_head, a_tok, _ptr(g), g.shape[1], int(col0), _ptr(out),
                                    _code(a, "sigmoid_gate a"), T, heads, size, _stream()), "sigmoid_gate")
    return out
