"""Python face of the CUDA kernels: loads the library and wraps each entry point.

There is no CPU fallback and no library model code here.  If the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call fails loudly.
Wrappers check dtypes and shapes, pass raw pointers and the current stream, and
raise `KernelError` with the entry point's own message on a non-zero return.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None
_flavor = None


def use_flavor(flavor) -> None:
    """Chooses another build of the kernels (csrc/build.py FLAVORS) for this process; before the library is first used."""
    global _flavor
    if _lib is not None and flavor != _flavor:
        raise KernelError("the kernel library is loaded already; choose the flavor before the first kernel call")
    _flavor = flavor


def lib():
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is None:
        path = _build.library_path(flavor=_flavor)
        try:
            L = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
        L.ms_last_error.restype = ctypes.c_char_p
        for name in dir(_Signatures):
            if name.startswith("ms_"):
                fn = getattr(L, name)
                fn.argtypes = getattr(_Signatures, name)
                fn.restype = c_int
        _lib = L
    return _lib


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it (on by default)."""
    lib().ms_set_pdl(1 if on else 0)


def library_file() -> str:
    return str(_build.library_path(flavor=_flavor))


class _Signatures:
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    ms_embed_gather = [P, I, P, P, I, I, I, P]
    ms_add_rmsnorm = [P, P, I, P, P, I, P, I, I, F, P]
    ms_add_bias = [P, I, P, I, I, I, P]
    ms_silu_mul = [P, P, I, I, I, P]
    ms_rope_kv_store = [P, I, I, P, P, P, P, I, I, P, I, I, P, P, P, I, I, I, I, I, I, P]
    ms_attention_generic = [P, P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    ms_gemm_f32 = [P, I, P, P, P, I, I, I, I, P]
    ms_attention_decode = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    ms_gemm_small_m_plan = [I, I, I, I, I, I, P]
    ms_attention_decode_cluster = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, I, I, P, LL, P, I, P]
    ms_attention_decode_cluster_rope = [P, I, P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, I, I, P, LL, P, I, P]
    ms_attention_prefill_tc = [P, P, P, P, I, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, LL, P, LL, P]
    ms_attention_prefill_tc_plan = [I, I, I, I, I, I, I, P]
    ms_attention_prefill = [P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P]
    ms_gemm_small_m = [P, I, P, P, I, I, I, I, I, I, P]
    ms_gemm_small_m_silu_mul = [P, I, P, P, P, I, I, I, I, I, P]
    ms_gemm_small_m_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_small_m_scaled = [P, I, P, I, F, P, P, P, I, I, I, I, I, P]
    ms_gemm_tc = [P, I, P, P, I, I, I, I, I, P]
    ms_gemm_tc_silu_mul = [P, I, P, P, I, I, I, I, P]
    ms_gemm_rows_tc = [P, I, P, P, I, I, I, I, I, I, P]
    ms_gemm_rows_tc_silu_mul = [P, I, P, P, P, I, I, I, I, I, P]
    ms_gemm_rows_tc_scaled = [P, I, P, I, F, P, P, P, I, I, I, I, I, P]
    ms_gemm_rows_tc_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_pair_tc = [P, I, P, P, I, I, I, I, P, I, F, I, P]
    ms_gemm_pair_tc_silu_mul = [P, I, P, P, I, I, I, I, P, I, F, I, P]
    ms_gemm_pair_tc_resadd = [P, I, P, P, I, P, P, I, I, I, I, I, P]
    ms_gemm_tc_wait_probe = [I, P]
    ms_attention_tc_wait_probe = [I, P]
    ms_take_sampled_tokens = [P, P, P, I, I, P]
    ms_apply_logit_offsets = [P, I, I, P, P, P, P]
    ms_sample = [P, I, I, P, P, P, P, P, P, P]
    ms_top_logprobs = [P, I, I, P, P, P, P, P]


_launches = 0


def launches() -> int:
    """How many of this library's kernels were launched so far in this process."""
    return _launches


def count_launches(n: int) -> None:
    """Adds launches that did not pass through the wrappers: kernels replayed from a captured graph."""
    global _launches
    _launches += n


def _check(code: int, name: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{name}: {lib().ms_last_error().decode()}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle (the capturing stream while a graph is captured).  Asked for with every launch, so
    through torch's raw getter where it exists: `torch.cuda.current_stream()` builds a Python object each time."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("a tensor on the CPU was given to a CUDA kernel; there is no CPU path")
    return c_void_p(t.data_ptr())


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ---------------------------------------------------------------------------


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, :] = table[ids[r], :] widened to float32.  table [V, d]; ids int32 [R]; out float32 [R, d]."""
    rows, d = out.shape
    _need(out.dtype == torch.float32 and ids.dtype == torch.int32 and ids.numel() >= rows, "embed_gather: bad arguments")
    _need(table.is_contiguous() and out.is_contiguous() and table.shape[1] == d, "embed_gather: bad layout")
    _check(
        lib().ms_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), rows, d, table.shape[0], _stream()),
        "embed_gather",
    )
    return out


def take_sampled_tokens(ids: torch.Tensor, from_rows: torch.Tensor, sampled: torch.Tensor) -> None:
    """ids[i] = sampled[from_rows[i]] where from_rows[i] >= 0 (all int32, on the device)."""
    _need(ids.dtype == torch.int32 and from_rows.dtype == torch.int32 and sampled.dtype == torch.int32 and
          from_rows.numel() >= ids.numel(), "take_sampled_tokens: bad arguments")
    _check(lib().ms_take_sampled_tokens(_ptr(ids), _ptr(from_rows), _ptr(sampled), ids.numel(), sampled.numel(), _stream()),
           "take_sampled_tokens")


def add_rmsnorm(
    residual: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    rows: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out = rmsnorm(residual + delta) * weight; without `rows` the sum is written back to `residual`.

    residual float32 [T, d]; delta [T, d] float32 or bfloat16 or None; weight float32 [d];
    out [n_out, d]; rows int32 [n_out] picks input rows (then nothing is written back).
    """
    d = residual.shape[1]
    n_out = out.shape[0]
    _need(residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d, "add_rmsnorm: bad dtypes")
    _need(residual.is_contiguous() and out.is_contiguous() and out.shape[1] == d, "add_rmsnorm: bad layout")
    if delta is not None:
        _need(delta.shape[1] == d and delta.is_contiguous() and delta.shape[0] >= residual.shape[0], "add_rmsnorm: bad delta")
    if rows is None:
        _need(n_out == residual.shape[0], "add_rmsnorm: out must have the residual's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_out, "add_rmsnorm: bad row list")
    _check(
        lib().ms_add_rmsnorm(
            _ptr(residual),
            _ptr(delta),
            _code(delta) if delta is not None else F32,
            _ptr(weight),
            _ptr(out),
            _code(out),
            _ptr(rows),
            n_out,
            d,
            float(eps),
            _stream(),
        ),
        "add_rmsnorm",
    )
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[r, c] += bias[c]: out [rows, n] float32 or bfloat16 (unit column stride), bias float32 [n]."""
    rows, n = out.shape
    _need(out.stride(1) == 1 and bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n, "add_bias: bad arguments")
    _check(lib().ms_add_bias(_ptr(out), _code(out), _ptr(bias), rows, n, out.stride(0), _stream()), "add_bias")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c].  gate_up [R, 2*inter], out [R, inter]."""
    rows, inter = out.shape
    _need(gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype, "silu_mul: bad shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous(), "silu_mul: bad layout")
    _check(lib().ms_silu_mul(_ptr(gate_up), _ptr(out), _code(out), rows, inter, _stream()), "silu_mul")
    return out


def rope_kv_store(
    qkv: torch.Tensor,
    bias: Optional[torch.Tensor],
    positions: torch.Tensor,
    seq_of_token: torch.Tensor,
    block_table: Optional[torch.Tensor],
    cos_sin: Optional[torch.Tensor],
    rotary_dim: int,
    interleaved: bool,
    q_out: torch.Tensor,
    k_pages: Optional[torch.Tensor],
    v_pages: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
) -> torch.Tensor:
    """Bias, rotary encoding of q and k, and the write of k, v into their pages.

    qkv [T, >= (Hq + 2*Hkv)*hd]; q_out [T, Hq*hd]; pages [num_pages, Hkv, page, hd];
    block_table int32 [S, max_pages]; cos_sin float32 [positions, rotary_dim/2, 2].
    With num_kv_heads == 0 only q is encoded.
    """
    tokens = q_out.shape[0]
    _need(qkv.stride(1) == 1 and q_out.is_contiguous() and q_out.dtype == qkv.dtype, "rope_kv_store: bad layout")
    _need(positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32, "rope_kv_store: index arrays must be int32")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() >= (num_heads + 2 * num_kv_heads) * head_dim),
          "rope_kv_store: bias must be float32 over q|k|v")
    if num_kv_heads:
        _need(k_pages is not None and k_pages.is_contiguous() and v_pages.is_contiguous(), "rope_kv_store: bad pages")
        _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "rope_kv_store: bad page shape")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "rope_kv_store: bad block table")
        num_pages, page_size, max_pages = k_pages.shape[0], k_pages.shape[2], block_table.shape[1]
        cache_code = _code(k_pages)
    else:
        num_pages = page_size = max_pages = 0
        cache_code = _code(qkv)
    if rotary_dim:
        _need(cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous(), "rope_kv_store: bad table")
        _need(cos_sin.shape[1] * 2 == rotary_dim, "rope_kv_store: table width does not match the rotary size")
    _check(
        lib().ms_rope_kv_store(
            _ptr(qkv), _code(qkv), qkv.stride(0), _ptr(bias), _ptr(positions), _ptr(seq_of_token), _ptr(block_table),
            max_pages, num_pages, _ptr(cos_sin), rotary_dim, int(interleaved), _ptr(q_out), _ptr(k_pages), _ptr(v_pages),
            cache_code, tokens, num_heads, num_kv_heads, head_dim, page_size, _stream(),
        ),
        "rope_kv_store",
    )
    return q_out


def attention_generic(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    positions: torch.Tensor,
    seq_of_token: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: Optional[int],
    scale: float,
    share_rows: bool = False,
) -> torch.Tensor:
    """The exact paged attention kernel.  q, out [T, Hq*hd]; pages [num_pages, Hkv, page, hd].  `share_rows`: rows that
    follow one another in a sequence (portions of prompts) share the tiles of keys they read, eight rows a block; the
    results are the same bits either way.  (A negative `share_rows`, for measurements: the float32 decoding form with
    that many heads of a group to a block.)"""
    tokens = q.shape[0]
    _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype, "attention: bad layout")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype, "attention: bad pages")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")
    _check(
        lib().ms_attention_generic(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _code(q), _code(k_pages), _ptr(positions),
            _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(share_rows), _stream(),
        ),
        "attention_generic",
    )
    return out


def attention_decode_supports(head_dim: int, groups: int) -> bool:
    return bool(lib().ms_attention_decode_supports(int(head_dim), int(groups)))


def attention_decode_scratch_words(tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, num_splits: int) -> int:
    """4-byte words of scratch for `num_splits` > 1: partial results, and one counter per (row, kv head)
    at the end, which must be zero before the first launch and is left zero by every launch."""
    return tokens * num_heads * num_splits * (head_dim + 2) + tokens * num_kv_heads if num_splits > 1 else 0


def attention_decode(q, k_pages, v_pages, out, scratch, positions, slot_of_token, block_table, num_heads, num_kv_heads,
                     head_dim, window, scale, num_splits, rows=None, num_rows=None):
    """Tensor-core paged attention for rows that are each attended on their own (decoding), bfloat16.
    `scratch` is float32 with at least attention_decode_scratch_words(...) elements whose tail (the
    counters) is zero (None for one split).
    `rows` (int32) lists the rows to attend, `num_rows` of them; by default every row of q."""
    tokens = q.shape[0] if rows is None else int(num_rows)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode: bad row list")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_decode: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode: bad block table")
    need = attention_decode_scratch_words(tokens, num_heads, num_kv_heads, head_dim, num_splits)
    _need(need == 0 or (scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need),
          "attention_decode: scratch is too small")
    _check(
        lib().ms_attention_decode(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(rows), _ptr(positions),
            _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(num_splits), _stream(),
        ),
        "attention_decode",
    )
    return out


def attention_decode_cluster_max_stages(head_dim: int) -> int:
    return int(lib().ms_attention_decode_cluster_max_stages(int(head_dim)))


def attention_decode_cluster_blocks_per_sm(head_dim: int, stages: int, warps: int = 4) -> int:
    """How many blocks of the kernel with `stages` tiles each an SM holds at once."""
    return int(lib().ms_attention_decode_cluster_blocks_per_sm(int(head_dim), int(stages), int(warps)))


def attention_decode_cluster_scratch_words(tokens: int, num_heads: int, num_kv_heads: int, head_dim: int, parts: int) -> int:
    """float32 words of scratch for `parts` > 1 clusters per (row, kv head); beside them, tokens * num_kv_heads int32
    counters that are zero before the first launch."""
    fn = lib().ms_attention_decode_cluster_scratch_words
    fn.restype = c_longlong
    return int(fn(int(tokens), int(num_heads), int(num_kv_heads), int(head_dim), int(parts)))


def _outer_args(name, tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters):
    if parts <= 1:
        return 1, None, 0, None, 0
    need = attention_decode_cluster_scratch_words(tokens, num_heads, num_kv_heads, head_dim, parts)
    _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
          f"{name}: {parts} clusters a row need {need} float32 words of scratch")
    _need(counters is not None and counters.dtype == torch.int32 and counters.is_contiguous() and counters.numel() >= tokens * num_kv_heads,
          f"{name}: {parts} clusters a row need {tokens * num_kv_heads} int32 counters")
    return int(parts), _ptr(scratch), scratch.numel(), _ptr(counters), counters.numel()


def attention_decode_cluster(q, k_pages, v_pages, out, positions, slot_of_token, block_table, num_heads, num_kv_heads,
                             head_dim, window, scale, num_splits, stages, rows=None, num_rows=None, warps=4, keys_per_warp=0,
                             parts=1, scratch=None, counters=None):
    """As attention_decode, with the splits of a row held by one thread-block cluster (1, 2, 4 or 8) and merged in
    shared memory: no scratch.  Keys and values of earlier positions are requested before the kernel waits for its
    predecessor in the stream.  `stages`: tiles of 64 keys a block holds at once.  `parts` > 1 (few rows with long
    contexts): a row's keys go to that many clusters, which leave their sums in `scratch`; the one that ends last
    merges them in order (`counters`: int32 zeros, left zero)."""
    tokens = q.shape[0] if rows is None else int(num_rows)
    outer = _outer_args("attention_decode_cluster", tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode_cluster: bad row list")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_decode_cluster: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode_cluster: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode_cluster: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode_cluster: bad block table")
    _check(
        lib().ms_attention_decode_cluster(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(rows), _ptr(positions), _ptr(slot_of_token),
            _ptr(block_table), block_table.shape[1], k_pages.shape[0], tokens, num_heads, num_kv_heads, head_dim,
            k_pages.shape[2], int(window or 0), float(scale), int(num_splits), int(stages), int(warps), int(keys_per_warp), *outer, _stream(),
        ),
        "attention_decode_cluster",
    )
    return out


def attention_decode_cluster_rope(qkv, bias, cos_sin, store, k_pages, v_pages, out, positions, slot_of_token, block_table,
                                  num_heads, num_kv_heads, head_dim, window, scale, num_splits, stages, rows=None,
                                  num_rows=None, warps=4, keys_per_warp=0, parts=1, scratch=None, counters=None):
    """rope_kv_store and attention_decode_cluster in one kernel, for rows that are alone in their sequences: reads
    rows of q|k|v (k and v only if `store`) as the projection left them, adds the bias, rotates q and k (full rotary,
    pairs j and j + head_dim/2, table [positions, head_dim/2, 2]), writes k and v into the cache, and attends."""
    tokens = qkv.shape[0] if rows is None else int(num_rows)
    outer = _outer_args("attention_decode_cluster_rope", tokens, num_heads, num_kv_heads, head_dim, parts, scratch, counters)
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= tokens), "attention_decode_cluster_rope: bad row list")
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and
          v_pages.dtype == torch.bfloat16, "attention_decode_cluster_rope: bfloat16 only")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_decode_cluster_rope: bad layout")
    width = (num_heads + (2 * num_kv_heads if store else 0)) * head_dim
    _need(qkv.shape[1] >= width, "attention_decode_cluster_rope: rows are narrower than q|k|v")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() >= width),
          "attention_decode_cluster_rope: bad bias")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == head_dim,
          "attention_decode_cluster_rope: the table must be [positions, head_dim/2, 2] float32")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_decode_cluster_rope: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_decode_cluster_rope: bad block table")
    _check(
        lib().ms_attention_decode_cluster_rope(
            _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(cos_sin), 1 if store else 0, _ptr(k_pages), _ptr(v_pages), _ptr(out),
            _ptr(rows), _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0],
            tokens, num_heads, num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(num_splits),
            int(stages), int(warps), int(keys_per_warp), *outer, _stream(),
        ),
        "attention_decode_cluster_rope",
    )
    return out


def attention_prefill_supports(head_dim: int) -> bool:
    return bool(lib().ms_attention_prefill_supports(int(head_dim)))


def attention_prefill(q, k_pages, v_pages, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table,
                      num_heads, num_kv_heads, head_dim, window, scale):
    """Tensor-core paged causal attention for tiles of up to 64 consecutive rows of one sequence, bfloat16."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_prefill: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_prefill: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_prefill: bad block table")
    _need(tile_row0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and min(tile_row0.numel(), tile_rows.numel()) >= num_tiles,
          "attention_prefill: bad tile lists")
    _check(
        lib().ms_attention_prefill(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tile_row0), _ptr(tile_rows), int(num_tiles),
            _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), _stream(),
        ),
        "attention_prefill",
    )
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias), all float32, on the CUDA cores."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: all operands must be float32")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_f32: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_f32: bad output shape")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == n), "gemm_f32: bad bias")
    _check(
        lib().ms_gemm_f32(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), out.stride(0), m, n, k, _stream()),
        "gemm_f32",
    )
    return out


SMALL_M = 16  # up to this many rows the weight-streaming kernel is used instead of the library
SMALL_M_MAX_WEIGHT_BYTES = 64 << 20  # a larger matrix (the vocabulary head) streams faster through the library
_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def gemm_small_m_supports(m: int, n: int, k: int) -> bool:
    """Whether the kernel covers the sizes (M up to 64, K in steps of 8)."""
    return 1 <= m <= 64 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_small_m_preferred(m: int, n: int, k: int) -> bool:
    """Whether the engine uses it: measured on B200 against the library at the decoder's sizes."""
    return gemm_small_m_supports(m, n, k) and m <= SMALL_M and 2 * n * k <= SMALL_M_MAX_WEIGHT_BYTES


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64: bfloat16 operands, bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_small_m: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_small_m: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_small_m: bad output shape")
    _check(
        lib().ms_gemm_small_m(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, sm_count(),
                              _stream()),
        "gemm_small_m",
    )
    return out


def gemm_small_m_silu_mul(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) for M <= 64, all bfloat16, in one kernel."""
    m, k = x.shape
    i = w_gate.shape[0]
    _need(x.dtype == w_gate.dtype == w_up.dtype == out.dtype == torch.bfloat16, "gemm_small_m_silu_mul: bfloat16 only")
    _need(w_gate.is_contiguous() and w_up.is_contiguous() and tuple(w_up.shape) == (i, k) and w_gate.shape[1] == k,
          "gemm_small_m_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_small_m_silu_mul: bad layout")
    _check(
        lib().ms_gemm_small_m_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(out), out.stride(0), m, i, k,
                                       sm_count(), _stream()),
        "gemm_small_m_silu_mul",
    )
    return out


def gemm_small_m_plan(m: int, n: int, k: int, gated: bool = False, residual: bool = False, sms: Optional[int] = None) -> dict:
    """How the few-row product of m rows with n outputs over k is spread over a GPU of `sms` SMs (this one's by default):
    host arithmetic only."""
    plan = (c_int * 7)()
    _check(lib().ms_gemm_small_m_plan(int(m), int(n), int(k), 1 if gated else 0, 1 if residual else 0,
                                      int(sms) if sms else sm_count(), plan), "gemm_small_m_plan")
    names = ("warps", "row_blocks", "cluster", "staged_chunks", "held_chunks", "activation_stride", "shared_bytes")
    return dict(zip(names, (int(v) for v in plan)))


def gemm_small_m_stats_blocks(n: int) -> int:
    """How many blocks of 16 columns `gemm_small_m_resadd` leaves sums of squares for."""
    return (n + 15) // 16


def gemm_small_m_resadd(x, w, residual, stats_out, copy_out=None):
    """residual[M, N] += x[M, K] . w[N, K]^T in place (float32); stats_out[m][b] = sum of squares of the new
    residual's row m over its b-th block of 16 columns; copy_out (optional, bfloat16 [M, N]) = the new residual
    rounded.  M <= 16."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_small_m_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_small_m_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_small_m_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_small_m_stats_blocks(n),
          "gemm_small_m_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_small_m_resadd: the copy must be bfloat16 [rows, N]")
    _check(
        lib().ms_gemm_small_m_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                     _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                     _stream()),
        "gemm_small_m_resadd",
    )
    return residual


def gemm_small_m_scaled(x, stats, stats_blocks, eps, w, w_up, out):
    """out = (x . w^T) / rms(row), or silu(. w^T / rms) * (. w_up^T / rms) when w_up is given: x is the residual
    rounded to bfloat16 [M, K] (the copy gemm_small_m_resadd leaves), `stats` [M, stats_blocks] its sums of squares;
    the RMS norm for matrices that have the norm's weight folded into their columns.  M <= 16."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and stats.dtype == torch.float32 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "gemm_small_m_scaled: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k, "gemm_small_m_scaled: bad weights")
    _need(w_up is None or (w_up.dtype == torch.bfloat16 and w_up.is_contiguous() and tuple(w_up.shape) == (n, k)),
          "gemm_small_m_scaled: bad up weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n), "gemm_small_m_scaled: bad layout")
    _need(stats.is_contiguous() and stats.numel() >= m * stats_blocks, "gemm_small_m_scaled: bad stats buffer")
    _check(
        lib().ms_gemm_small_m_scaled(_ptr(x), x.stride(0), _ptr(stats), int(stats_blocks), float(eps), _ptr(w), _ptr(w_up),
                                     _ptr(out), out.stride(0), m, n, k, sm_count(), _stream()),
        "gemm_small_m_scaled",
    )
    return out


def gemm_tc_supports(m: int, n: int, k: int) -> bool:
    return m >= 1 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T on tcgen05 tensor cores with TMA-fed operands; bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_tc: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_tc: bad output shape")
    _check(lib().ms_gemm_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, _stream()), "gemm_tc")
    return out


def gemm_tc_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w[:I]^T) * (x . w[I:]^T) in one tcgen05 kernel; w_gate_up is [2I, K], gate rows first."""
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    _need(x.dtype == w_gate_up.dtype == out.dtype == torch.bfloat16, "gemm_tc_silu_mul: bfloat16 only")
    _need(w_gate_up.is_contiguous() and w_gate_up.shape[1] == k and w_gate_up.shape[0] == 2 * i, "gemm_tc_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_tc_silu_mul: bad layout")
    _check(lib().ms_gemm_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(out), out.stride(0), m, i, k, _stream()),
           "gemm_tc_silu_mul")
    return out


def gemm_rows_tc_supports(m: int, n: int, k: int) -> bool:
    """Up to 64 rows, K in steps of 8."""
    return 1 <= m <= 64 and n >= 1 and k >= 8 and k % 8 == 0


def gemm_rows_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64 on tcgen05 tensor cores with the weights as the 128-row operand,
    streamed once through TMA stages; bfloat16 operands, bfloat16 or float32 out."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_rows_tc: operands must be bfloat16")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1, "gemm_rows_tc: bad layout")
    _need(tuple(out.shape) == (m, n), "gemm_rows_tc: bad output shape")
    _check(lib().ms_gemm_rows_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), _code(out), out.stride(0), m, n, k, sm_count(), _stream()),
           "gemm_rows_tc")
    return out


def gemm_rows_tc_silu_mul(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) for M <= 64, all bfloat16, in one kernel."""
    m, k = x.shape
    i = w_gate.shape[0]
    _need(x.dtype == w_gate.dtype == w_up.dtype == out.dtype == torch.bfloat16, "gemm_rows_tc_silu_mul: bfloat16 only")
    _need(w_gate.is_contiguous() and w_up.is_contiguous() and tuple(w_up.shape) == (i, k) and w_gate.shape[1] == k,
          "gemm_rows_tc_silu_mul: bad weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_rows_tc_silu_mul: bad layout")
    _check(lib().ms_gemm_rows_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(out), out.stride(0), m, i, k,
                                          sm_count(), _stream()), "gemm_rows_tc_silu_mul")
    return out


def gemm_rows_tc_resadd(x, w, residual, stats_out, copy_out=None):
    """As gemm_small_m_resadd, for up to 64 rows: residual += x . w^T (float32, in place), the sums of squares of the
    new residual per row and block of 16 columns, and optionally its bfloat16 copy."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_rows_tc_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_rows_tc_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_rows_tc_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_small_m_stats_blocks(n),
          "gemm_rows_tc_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_rows_tc_resadd: the copy must be bfloat16 [rows, N]")
    _check(lib().ms_gemm_rows_tc_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                        _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                        _stream()), "gemm_rows_tc_resadd")
    return residual


def gemm_rows_tc_scaled(x, stats, stats_blocks, eps, w, w_up, out):
    """As gemm_small_m_scaled, for up to 64 rows: out = (x . w^T) / rms(row), or the gated form with w_up."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and stats.dtype == torch.float32 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "gemm_rows_tc_scaled: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k, "gemm_rows_tc_scaled: bad weights")
    _need(w_up is None or (w_up.dtype == torch.bfloat16 and w_up.is_contiguous() and tuple(w_up.shape) == (n, k)),
          "gemm_rows_tc_scaled: bad up weights")
    _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n), "gemm_rows_tc_scaled: bad layout")
    _need(stats.is_contiguous() and stats.numel() >= m * stats_blocks, "gemm_rows_tc_scaled: bad stats buffer")
    _check(lib().ms_gemm_rows_tc_scaled(_ptr(x), x.stride(0), _ptr(stats), int(stats_blocks), float(eps), _ptr(w), _ptr(w_up),
                                        _ptr(out), out.stride(0), m, n, k, sm_count(), _stream()), "gemm_rows_tc_scaled")
    return out


def gemm_pair_tc(x, w, out, stats=None, stats_blocks=0, eps=0.0):
    """out[M, N] = x[M, K] . w[N, K]^T for many rows on the tcgen05 tensor cores (a pair of SMs per tile, resident
    blocks that go through their tiles, two accumulators in tensor memory), all bfloat16.  With `stats` ([M, stats_blocks] sums of
    squares of the rows x was rounded from) every output row is divided by that row's rms: the RMS norm for a matrix
    with the norm's weight folded into its columns."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "gemm_pair_tc: bfloat16 only")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == (m, n),
          "gemm_pair_tc: bad layout")
    _need(stats is None or (stats.dtype == torch.float32 and stats.is_contiguous() and stats.numel() >= m * stats_blocks >= m),
          "gemm_pair_tc: bad stats buffer")
    _check(lib().ms_gemm_pair_tc(_ptr(x), x.stride(0), _ptr(w), _ptr(out), out.stride(0), m, n, k, _ptr(stats), int(stats_blocks),
                                   float(eps), sm_count(), _stream()), "gemm_pair_tc")
    return out


# From where the gated product with the gating in its epilogue beats the library's product followed by the gating
# kernel (measured on B200 at K = 896, 1,536, 2,048 and 3,584, 256 to 4,152 rows: from 1,024 rows on by 6 to 17 %,
# at K = 896 only from 2,048 rows on; below 1,024 rows the library wins).
PAIR_TC_SILU_MIN_ROWS = 1024
PAIR_TC_SILU_MIN_ROWS_NARROW = 2048  # for K below 1,024


def gemm_pair_tc_silu_preferred(m: int, i: int, k: int) -> bool:
    return m >= (PAIR_TC_SILU_MIN_ROWS if k >= 1024 else PAIR_TC_SILU_MIN_ROWS_NARROW) and i % 8 == 0 and k % 8 == 0


def gemm_pair_tc_silu_mul(x, w_gate_up, out, stats=None, stats_blocks=0, eps=0.0):
    """out[M, I] = silu(x . w_gate^T) * (x . w_up^T) with w_gate_up = [gate rows; up rows] ([2I, K]); row scaling as in
    gemm_pair_tc."""
    m, k = x.shape
    i = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "gemm_pair_tc_silu_mul: bfloat16 only")
    _need(w_gate_up.is_contiguous() and w_gate_up.shape[1] == k and w_gate_up.shape[0] == 2 * i and x.stride(1) == 1 and
          out.stride(1) == 1 and tuple(out.shape) == (m, i), "gemm_pair_tc_silu_mul: bad layout")
    _need(stats is None or (stats.dtype == torch.float32 and stats.is_contiguous() and stats.numel() >= m * stats_blocks >= m),
          "gemm_pair_tc_silu_mul: bad stats buffer")
    _check(lib().ms_gemm_pair_tc_silu_mul(_ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(out), out.stride(0), m, i, k, _ptr(stats),
                                            int(stats_blocks), float(eps), sm_count(), _stream()), "gemm_pair_tc_silu_mul")
    return out


def gemm_pair_tc_stats_blocks(m: int, n: int) -> int:
    """How many sums of squares per row `gemm_pair_tc_resadd` leaves for a residual of [m, n] (one per tile of columns)."""
    return int(lib().ms_gemm_pair_tc_stats_blocks(int(m), int(n), sm_count()))


def gemm_pair_tc_resadd(x, w, residual, stats_out, copy_out=None):
    """residual[M, N] += x[M, K] . w[N, K]^T in place (float32), the sums of squares of the new residual per row and
    tile of columns (`gemm_pair_tc_stats_blocks` of them a row; a consumer adds up all of a row's), and optionally its
    bfloat16 copy; any number of rows."""
    m, k = x.shape
    n = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32, "gemm_pair_tc_resadd: bad dtypes")
    _need(w.is_contiguous() and w.shape[1] == k and x.stride(1) == 1 and residual.stride(1) == 1, "gemm_pair_tc_resadd: bad layout")
    _need(tuple(residual.shape) == (m, n), "gemm_pair_tc_resadd: the residual must be [rows, N]")
    _need(stats_out.dtype == torch.float32 and stats_out.is_contiguous() and stats_out.numel() >= m * gemm_pair_tc_stats_blocks(m, n),
          "gemm_pair_tc_resadd: bad stats buffer")
    _need(copy_out is None or (copy_out.dtype == torch.bfloat16 and tuple(copy_out.shape) == (m, n) and copy_out.stride(1) == 1),
          "gemm_pair_tc_resadd: the copy must be bfloat16 [rows, N]")
    _check(lib().ms_gemm_pair_tc_resadd(_ptr(x), x.stride(0), _ptr(w), _ptr(residual), residual.stride(0), _ptr(stats_out),
                                          _ptr(copy_out), copy_out.stride(0) if copy_out is not None else 0, m, n, k, sm_count(),
                                          _stream()), "gemm_pair_tc_resadd")
    return residual


def gemm_tc_status(reset: bool = True) -> int:
    """0, or which bounded wait of a tcgen05 kernel gave up (products: 1 producer, 2 issuer, 3 epilogue, 21-23 the same of the
    resident-block product; attention: 11 producer, 12-14 and 16 issuer, 15 softmax threads).  Synchronizes."""
    codes = tc_status_codes(reset)
    return codes[0] or codes[1]


def tc_status_codes(reset: bool = True):
    """(code of the tcgen05 products, code of the tcgen05 attention): both are read, and cleared with `reset`,
    whichever of them is set.  Synchronizes."""
    return int(lib().ms_gemm_tc_status(1 if reset else 0)), int(lib().ms_attention_tc_status(1 if reset else 0))


def tc_wait_probe(kernel: str, polls: int = 1000) -> None:
    """Launches one thread that waits `polls` polls on a barrier nothing arrives on, through the bounded-wait helper
    of the tcgen05 products (`kernel="gemm"`, leaves code 9) or of the tcgen05 attention (`"attention"`, code 19):
    the way to see the give-up path run (error word set, kernel returns, context usable) without a hang."""
    _need(kernel in ("gemm", "attention"), "tc_wait_probe: kernel is 'gemm' or 'attention'")
    fn = lib().ms_gemm_tc_wait_probe if kernel == "gemm" else lib().ms_attention_tc_wait_probe
    _check(fn(int(polls), _stream()), "tc_wait_probe")


def attention_prefill_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().ms_attention_prefill_tc_supports(int(head_dim), int(page_size)))


def attention_prefill_tc_plan(num_tiles: int, num_heads: int, num_kv_heads: int, head_dim: int, max_keys: int,
                              key_tiles: int = 0):
    """(splits, alone, run_tiles): into how many runs the kernel should cut an item's key tiles so that the launch fills
    the GPU (1 to 4), whether, at head size 128, every block should take one head instead of two of a group, and (if
    not 0) the most key tiles of a run, so that only longer items are cut.
    `key_tiles`: the tiles of 128 keys that the launch's tiles of rows see, in all (0: every tile sees `max_keys`)."""
    plan = (ctypes.c_int * 3)()
    lib().ms_attention_prefill_tc_plan(int(num_tiles), int(num_heads), int(num_kv_heads), int(head_dim), int(max_keys),
                                       int(key_tiles), sm_count(), plan)
    return int(plan[0]), bool(plan[1]), int(plan[2])


def attention_prefill_tc_scratch_words(num_tiles: int, num_heads: int, head_dim: int, splits: int) -> int:
    """float32 words of scratch memory for `splits` > 1 (beside num_tiles * num_heads int32 counters, which must be zero
    before the first launch and are left zero by every launch)."""
    fn = lib().ms_attention_prefill_tc_scratch_words
    fn.restype = c_longlong
    return int(fn(int(num_tiles), int(num_heads), int(head_dim), int(splits)))


def attention_prefill_tc(q, k_pages, v_pages, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table,
                         num_heads, num_kv_heads, head_dim, window, scale, splits=1, scratch=None, counters=None, alone=False,
                         run_tiles=0):
    """Paged causal attention for tiles of up to 128 consecutive rows of one sequence on tcgen05 tensor cores
    (TMA-fed, scores in tensor memory and taken into registers a row per thread, probabilities back into tensor
    memory, outputs accumulated there over all key tiles).  Head sizes 64 (one head per block) and 128 (two heads of a
    group per block, which share the keys and values), page sizes 8, 16, 32, ...  With `splits` > 1 the key tiles of
    every (tile, head) go to that many blocks, which meet in `scratch` (float32) and count themselves in `counters`
    (int32, num_tiles * num_heads of them, all zero before and after).  `alone` (head size 128): one head per block.
    `run_tiles` > 0: only items with more key tiles are cut, into runs of at most that many."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16,
          "attention_prefill_tc: bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous(),
          "attention_prefill_tc: bad layout")
    _need(tuple(k_pages.shape[1:]) == (num_kv_heads, k_pages.shape[2], head_dim), "attention_prefill_tc: bad page shape")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention_prefill_tc: bad block table")
    _need(tile_row0.dtype == torch.int32 and tile_rows.dtype == torch.int32 and min(tile_row0.numel(), tile_rows.numel()) >= num_tiles,
          "attention_prefill_tc: bad tile lists")
    _need(scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()), "attention_prefill_tc: scratch must be float32")
    _need(counters is None or (counters.dtype == torch.int32 and counters.is_contiguous()), "attention_prefill_tc: counters must be int32")
    _check(
        lib().ms_attention_prefill_tc(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), q.shape[0], _ptr(tile_row0), _ptr(tile_rows), int(num_tiles),
            _ptr(positions), _ptr(slot_of_token), _ptr(block_table), block_table.shape[1], k_pages.shape[0], num_heads,
            num_kv_heads, head_dim, k_pages.shape[2], int(window or 0), float(scale), int(splits), 1 if alone else 0, int(run_tiles), _ptr(scratch),
            scratch.numel() if scratch is not None else 0, _ptr(counters), counters.numel() if counters is not None else 0,
            _stream(),
        ),
        "attention_prefill_tc",
    )
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out = x . w^T (+ bias, float32 [n]).  float32 goes to the CUDA-core kernel.  bfloat16 with few rows
    (decoding) goes to the weight-streaming tensor-core kernel; with many rows it goes to the
    library matrix product (cuBLAS through torch), where the reference too calls its library
    (hipBLAS GemmEx, crates/mach-model/src/kernels.rs:6416-6455 of gqf2008/machserve); a bias is then
    added by a kernel of its own (the built-in attention adds its bias inside its rotary kernel instead)."""
    if x.dtype == torch.float32:
        return gemm_f32(x, w, bias, out)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16 or float32")
    if gemm_small_m_preferred(x.shape[0], w.shape[0], x.shape[1]) and x.stride(0) % 8 == 0:
        gemm_small_m(x, w, out)
    elif out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return add_bias(out, bias) if bias is not None else out


def apply_logit_offsets(logits, row_ptr, tokens, amounts):
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "apply_logit_offsets: bad logits")
    _need(row_ptr.dtype == torch.int32 and tokens.dtype == torch.int32 and amounts.dtype == torch.float32,
          "apply_logit_offsets: bad dtypes")
    _check(
        lib().ms_apply_logit_offsets(_ptr(logits), rows, vocab, _ptr(row_ptr), _ptr(tokens), _ptr(amounts), _stream()),
        "apply_logit_offsets",
    )
    return logits


def sample(logits, temperature, top_k, top_p, rng_state, out_token, out_logprob):
    """One token per row.  rng_state int64 [R] holds the SplitMix64 states and is advanced in place."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and top_k.dtype == torch.int32, "sample: bad dtypes")
    _need(rng_state.dtype == torch.int64 and out_token.dtype == torch.int32 and out_logprob.dtype == torch.float32,
          "sample: bad dtypes")
    _need(min(temperature.numel(), top_k.numel(), top_p.numel(), rng_state.numel(), out_token.numel(),
              out_logprob.numel()) >= rows, "sample: per-row arrays are shorter than the rows")
    _check(
        lib().ms_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(rng_state),
                        _ptr(out_token), _ptr(out_logprob), _stream()),
        "sample",
    )
    return out_token


TOP_LOGPROBS_MAX = 20


def top_logprobs(logits, temperature, want, out_token, out_logprob):
    """The want[r] (at most 20) most probable tokens of every row and their log-probabilities at the row's
    temperature, ranked; out_token int32 and out_logprob float32 are [rows, 20]."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "top_logprobs: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and want.dtype == torch.int32 and min(temperature.numel(), want.numel()) >= rows,
          "top_logprobs: bad per-row arrays")
    _need(out_token.dtype == torch.int32 and out_logprob.dtype == torch.float32 and out_token.is_contiguous() and
          out_logprob.is_contiguous() and min(out_token.numel(), out_logprob.numel()) >= rows * TOP_LOGPROBS_MAX,
          "top_logprobs: the outputs must be [rows, 20]")
    _check(lib().ms_top_logprobs(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(want), _ptr(out_token), _ptr(out_logprob),
                                 _stream()), "top_logprobs")
