"""Python bindings of the CUDA library: one function per kernel launcher.

Tensors are passed as raw device pointers through ctypes, on torch's current
stream.  There is no fallback of any kind: if the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

_lib = None
_launches = 0      # kernels of this library launched so far (for the bench's count)

_c_int, _c_ll, _c_float, _c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library; built on first use."""
    global _lib
    if _lib is None:
        path = build.ensure_built()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the engine's CUDA library {path}: {e}") from None
    return _lib


def launches() -> int:
    return _launches


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported activation dtype {t.dtype} (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the engine's kernels take CUDA tensors only (no CPU path)")
    return _c_void_p(t.data_ptr())


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")


_profiler = None   # an object with begin(name) / end(name), set by binfer_b200.profiling


def set_profiler(p) -> None:
    global _profiler
    _profiler = p


def _run(name: str, fn, *args) -> None:
    p = _profiler
    if p is not None:
        p.begin(name)
    code = fn(*args)
    if p is not None:
        p.end(name)
    _check(code, name)


def count_library_launch(name: str = "gemm") -> None:
    """A library matrix product was launched (counted apart from the engine's own kernels)."""
    global _library_launches
    _library_launches += 1


_library_launches = 0


def library_launches() -> int:
    return _library_launches


def _want(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float,
                 err: torch.Tensor) -> None:
    """out[t] = table[ids[t]] * scale; out is the float residual stream [T, H]."""
    _want(ids, torch.int32, "ids"); _want(out, torch.float32, "out")
    T, H = out.shape
    _run("embed_gather", lib().bf_embed_gather, _ptr(table), _c_int(_dtype_code(table)), _ptr(ids), _ptr(out),
                                 _c_int(T), _c_int(H), _c_int(table.shape[0]), _c_float(scale),
                                 _ptr(err), _stream())


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                write_back: bool = True) -> None:
    """out[i] = rmsnorm(resid[r] + delta[r]) * weight with r = rows[i] (or i); the
    sum is written back to resid when ``write_back``."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight")
    n, H = out.shape
    if delta is not None and (delta.dtype != out.dtype or not delta.is_contiguous()):
        raise KernelError("delta must be contiguous and of the output's dtype")
    if rows is not None:
        _want(rows, torch.int32, "rows")
    _run("add_rmsnorm", lib().bf_add_rmsnorm, _ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows),
                                _c_int(n), _c_int(H), _c_float(eps), _c_int(_dtype_code(out)),
                                _c_int(1 if write_back else 0), _stream())


def residual_add(resid: torch.Tensor, delta: torch.Tensor) -> None:
    _want(resid, torch.float32, "resid")
    _run("residual_add", lib().bf_residual_add, _ptr(resid), _ptr(delta), _c_ll(resid.numel()),
                                 _c_int(_dtype_code(delta)), _stream())


class RowScale:
    """A factor per row that is still to be applied: ``rsqrt(partials[t].sum() / width + eps)``.

    It is what a product that also prepared the next norm (``gemm_bf16_cluster_add_norm``)
    leaves out, because no CTA of it sees a whole row.  A linear map commutes with the
    factor, so the kernel after the next product applies it (``qk_norm_rope_kv_write``,
    ``silu_mul``).  ``partials`` is float32 ``[rows, count]``, contiguous."""
    __slots__ = ("partials", "width", "eps")

    def __init__(self, partials: torch.Tensor, width: int, eps: float):
        self.partials, self.width, self.eps = partials, int(width), float(eps)

    def factors(self) -> torch.Tensor:
        """The factors themselves, float32 ``[rows]`` (for tests and for parts that cannot
        take a RowScale)."""
        return torch.rsqrt(self.partials.sum(dim=1) / self.width + self.eps)


def _row_scale_args(rs: Optional["RowScale"], rows: int):
    if rs is None:
        return _ptr(None), _c_int(0), _c_int(0), _c_float(0.0)
    p = rs.partials
    if p.dtype != torch.float32 or not p.is_contiguous() or p.dim() != 2 or p.shape[0] < rows:
        raise KernelError("row scale: partials must be contiguous float32 [rows, count]")
    return _ptr(p), _c_int(p.shape[1]), _c_int(rs.width), _c_float(rs.eps)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor,
             row_scale: Optional[RowScale] = None) -> None:
    """out[t, c] = silu(f gate_up[t, c]) * f gate_up[t, I + c]; f = 1 without ``row_scale``
    (which is taken for bfloat16 and I a multiple of 8, at least 256)."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: gate_up must be contiguous [T, 2*I] of the output's dtype")
    if row_scale is not None:
        if out.dtype != torch.bfloat16 or I % 8 or I < 256:
            raise KernelError("silu_mul: a row scale needs bfloat16 and I % 8 == 0, I >= 256")
        _run("silu_mul_scaled", lib().bf_silu_mul_scaled, _ptr(gate_up), _ptr(out), _c_int(T),
             _c_int(I), *_row_scale_args(row_scale, T), _stream())
        return
    _run("silu_mul", lib().bf_silu_mul, _ptr(gate_up), _ptr(out), _c_int(T), _c_int(I),
                             _c_int(_dtype_code(out)), _stream())


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def gated_act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out[t, c] = act(gate_up[t, c]) * gate_up[t, I + c]; ``activation`` one of
    ``GATE_ACTIVATIONS``."""
    T, I = out.shape
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"gated_act_mul: unknown activation {activation!r}")
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or gate_up.dtype != out.dtype:
        raise KernelError("gated_act_mul: gate_up must be contiguous [T, 2*I] of the output's dtype")
    _run("gated_act_mul", lib().bf_gated_act_mul, _ptr(gate_up), _ptr(out), _c_int(T), _c_int(I),
         _c_int(GATE_ACTIVATIONS[activation]), _c_int(_dtype_code(out)), _stream())


def copy_ids(dst: torch.Tensor, src: torch.Tensor, pairs: torch.Tensor, n: int) -> None:
    """dst[pairs[i, 0]] = src[pairs[i, 1]] for i < n (int32 everywhere)."""
    _want(dst, torch.int32, "dst"); _want(src, torch.int32, "src"); _want(pairs, torch.int32, "pairs")
    _run("copy_ids", lib().bf_copy_ids, _ptr(dst), _ptr(src), _ptr(pairs), _c_int(n), _stream())


# ------------------------------------------------------------------- attention
def qk_norm_rope_kv_write(qkv: torch.Tensor, q_w: Optional[torch.Tensor],
                          k_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                          positions: torch.Tensor, slots: Optional[torch.Tensor],
                          q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int,
                          eps: float, err: torch.Tensor,
                          row_scale: Optional[RowScale] = None) -> None:
    """Per-head RMSNorm of q and k, rotation, q to ``q_out [T, nh*d]``, k and v into
    cache pages ``[pages, nkv, page_size, d]`` at ``slots``.  With ``row_scale`` the rows of
    ``qkv`` are first multiplied by their factors."""
    T = qkv.shape[0]
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    page_size = k_cache.shape[2] if k_cache is not None else 1
    num_slots = k_cache.shape[0] * page_size if k_cache is not None else 0
    if k_cache is not None and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    _run("qk_norm_rope_kv_write", lib().bf_qk_norm_rope_kv_write, 
        _ptr(qkv), _c_ll(qkv.stride(0)), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _c_int(rot_half),
        _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(T),
        _c_int(nh), _c_int(nkv if k_cache is not None else 0), _c_int(d), _c_int(page_size),
        _c_ll(num_slots), _c_float(eps), _c_int(_dtype_code(qkv)),
        *_row_scale_args(row_scale, T), _ptr(err), _stream())


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor,
                            block_tables: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                            d: int, window: Optional[int], scale: float,
                            err: torch.Tensor, softcap: float = 0.0,
                            slopes: Optional[torch.Tensor] = None,
                            sinks: Optional[torch.Tensor] = None, value_dim: Optional[int] = None,
                            keep_first: int = 0, out_scale: float = 1.0,
                            v_stride: int = 0, log_slope: Optional[torch.Tensor] = None,
                            log_rate: Optional[torch.Tensor] = None) -> None:
    """Attention of every token row over its request's pages, any sizes.  ``softcap``,
    ``slopes`` (float32 ``[nh]``) and ``sinks`` (float32 ``[nh]``) change the scores as
    ``config.specs.ScoreSpec`` says; by default nothing is changed.  ``value_dim``: size of a
    value head where it differs from ``d``.  ``keep_first``: with a window, the request's
    first that many tokens stay visible behind it.  ``q`` and ``out`` may be column blocks of
    wider buffers (rows ``nh * d`` and ``nh * value_dim`` long); ``out_scale`` multiplies the
    result.  ``v_stride``: elements between the value rows of neighbouring tokens of a page
    (0: ``value_dim``); with ``v_cache = k_cache`` and ``v_stride = d`` a token's value is the
    first ``value_dim`` numbers of its key.  ``log_slope`` and ``log_rate`` (float32 ``[nh]``
    each, together or not at all): ``log_slope_h ln(1 + log_rate_h (p - j))`` is taken off the
    score of the query at p and the key at j."""
    T = q.shape[0]
    dv = d if value_dim is None else int(value_dim)
    if (log_slope is None) != (log_rate is None):
        raise KernelError("attention: log_slope and log_rate go together")
    if d > GENERIC_MAX_HEAD_DIM or dv > GENERIC_MAX_VALUE_DIM:
        raise KernelError(f"attention: head sizes {d}, {dv} are not supported (at most "
                          f"{GENERIC_MAX_HEAD_DIM}, {GENERIC_MAX_VALUE_DIM})")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: rows of q and out must be contiguous")
    for name, t in (("slopes", slopes), ("sinks", sinks), ("log_slope", log_slope),
                    ("log_rate", log_rate)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != nh:
                raise KernelError(f"attention: {name} must have one entry per query head")
    _run("paged_attention_generic", lib().bf_paged_attention_generic, 
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_of_token), _ptr(positions),
        _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _c_int(T), _c_int(nh),
        _c_int(nkv), _c_int(d), _c_int(k_cache.shape[2]), _c_int(k_cache.shape[0]),
        _c_int(window or 0), _c_float(scale), _c_float(softcap), _ptr(slopes), _ptr(sinks),
        _c_int(_dtype_code(q)), _ptr(err), _c_int(dv), _c_int(keep_first), _c_ll(q.stride(0)),
        _c_ll(out.stride(0)), _c_float(out_scale), _c_ll(v_stride), _ptr(log_slope),
        _ptr(log_rate), _stream())


GENERIC_MAX_HEAD_DIM, GENERIC_MAX_VALUE_DIM = 1024, 512
DECODE_HEAD_DIMS = (32, 64, 96, 128, 256)
DECODE_SPLIT_KEYS = 128


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     rows: Optional[torch.Tensor], n_rows: int, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, block_tables: torch.Tensor, out: torch.Tensor,
                     nh: int, nkv: int, d: int, window: Optional[int], scale: float,
                     max_ctx_len: int, err: torch.Tensor, variant: str = "auto",
                     scratch=None, softcap: float = 0.0, out_scale: float = 1.0) -> None:
    """Split-KV attention for rows that bring one token each (bfloat16 only).

    ``softcap`` c > 0: the scaled scores pass ``c tanh(s / c)``; ``out_scale``: a factor on
    the result; ``out`` may then also be a column block of a wider buffer.  These three are
    the persistent variant's alone (``decode_attention_takes_capped`` says whether it
    applies).

    ``rows`` lists the token rows to run (None: rows 0..n_rows-1); ``max_ctx_len``
    bounds the context of every such row (a row beyond it sets the error word's
    "splits" bit and loses its far keys; nothing is read or written past the scratch).
    Scratch for the splits' partial results is taken from torch's allocator, or given as
    ``scratch = (part_o [n_rows, nh, splits, d], part_ml [n_rows, nh, splits, 2])`` float32,
    whose ``splits`` then is the room there is.  ``variant``: ``persistent`` (resident CTAs that walk
    the work with a ring of TMA-fed tiles; head sizes 64/128/256, page sizes 8..128 that
    divide 128, at most 16 query heads per kv head and 512 rows), ``tma`` (one CTA per split,
    bulk tensor copies; the same head and page sizes), ``cp_async`` (every size in
    DECODE_HEAD_DIMS, any page size), or ``auto``: the first of these that applies."""
    if q.dtype != torch.bfloat16 or d not in DECODE_HEAD_DIMS:
        raise KernelError(f"decode_attention: bfloat16 and head_dim in {DECODE_HEAD_DIMS} only")
    if variant not in ("auto", "persistent", "tma", "cp_async"):
        raise KernelError(f"decode_attention: unknown variant {variant!r}")
    page_size = k_cache.shape[2]
    tma_ok = d in (64, 128, 256) and 8 <= page_size <= 128 and 128 % page_size == 0
    persistent_ok = (tma_ok and nh // nkv <= 16 and n_rows <= 512 and q.is_contiguous()
                     and q.data_ptr() % 16 == 0)
    if variant == "tma" and not tma_ok:
        raise KernelError(f"decode_attention: the tma variant does not take head_dim {d} with "
                          f"pages of {page_size}")
    if variant == "persistent" and not persistent_ok:
        raise KernelError(f"decode_attention: the persistent variant does not take head_dim {d}, "
                          f"pages of {page_size}, {nh // nkv} heads per kv head, {n_rows} rows")
    capped = softcap > 0 or out_scale != 1.0 or not out.is_contiguous()
    if capped:
        if not persistent_ok or variant not in ("auto", "persistent"):
            raise KernelError("decode_attention: a soft cap, an output factor or an output in a "
                              "column block are the persistent variant's alone")
        if out.stride(1) != 1 or out.stride(0) % 4 or out.data_ptr() % 8 or out.dtype != q.dtype:
            raise KernelError("decode_attention: out must have contiguous rows a multiple of 4 "
                              "elements apart, 8-byte aligned")
        name, fn = "decode_attention_persistent", lib().bf_decode_attention_persistent_capped
    elif persistent_ok and variant in ("auto", "persistent"):
        name, fn = "decode_attention_persistent", lib().bf_decode_attention_persistent
    elif tma_ok and variant != "cp_async":
        name, fn = "decode_attention_tma", lib().bf_decode_attention_tma
    else:
        name, fn = "decode_attention", lib().bf_decode_attention
    if scratch is None:
        max_splits = max(1, -(-int(max_ctx_len) // DECODE_SPLIT_KEYS))
        part_o = torch.empty((n_rows, nh, max_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_rows, nh, max_splits, 2), dtype=torch.float32, device=q.device)
    else:
        part_o, part_ml = scratch
        max_splits = part_o.shape[2]
        _want(part_o, torch.float32, "part_o"); _want(part_ml, torch.float32, "part_ml")
        if (tuple(part_o.shape) != (n_rows, nh, max_splits, d)
                or tuple(part_ml.shape) != (n_rows, nh, max_splits, 2)):
            raise KernelError("decode_attention: scratch must be [n_rows, nh, splits, d] and "
                              "[n_rows, nh, splits, 2]")
    _run(name, fn,
         _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(rows), _ptr(seq_of_token), _ptr(positions),
         _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _ptr(part_o),
         _ptr(part_ml), _c_int(n_rows), _c_int(nh), _c_int(nkv), _c_int(d),
         _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
         _c_int(max_splits), _c_float(scale), _ptr(err),
         *((_c_float(softcap), _c_ll(out.stride(0)), _c_float(out_scale)) if capped else ()),
         _stream())
    global _launches
    _launches += 1          # two kernels: the splits and their merge


def decode_attention_takes_capped(q: torch.Tensor, k_cache: torch.Tensor, nh: int, nkv: int,
                                  d: int, dv: int, n_rows: int) -> bool:
    """Whether ``decode_attention`` with a soft cap, an output factor or a strided output
    (the persistent variant) takes these sizes."""
    page_size = k_cache.shape[2]
    return (q.dtype == torch.bfloat16 and d == dv and d in (64, 128, 256)
            and 8 <= page_size <= 128 and 128 % page_size == 0 and nh // nkv <= 16
            and n_rows <= 512 and q.is_contiguous() and q.data_ptr() % 16 == 0)


# scratch for the shares of split prefill attention, per device (grown as needed, up to a limit)
_prefill_split_scratch = {}
_PREFILL_SPLIT_BYTES = 256 << 20


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      items: torch.Tensor, n_items: int, max_rows: int,
                      block_tables: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, d: int,
                      window: Optional[int], scale: float, err: torch.Tensor,
                      variant: str = "auto", max_ctx: int = 0, splits: int = 0,
                      softcap: float = 0.0, out_scale: float = 1.0) -> None:
    """Causal flash attention over the pages for prompt portions (bfloat16 only).
    ``items`` int32 [n, 4]: (request index, first token row, rows, first position).
    ``variant``: ``umma2`` (tcgen05 tensor cores, one CTA per SM with two query tiles sharing a
    K/V ring; head size 128, page sizes 8..64 that divide 64), ``umma`` (two CTAs of one
    query tile per SM; head sizes 64/128, the same page sizes), ``mma_sync`` (every size in
    DECODE_HEAD_DIMS, any page size), or ``auto``: umma2 where it applies and there are
    blocks of 256 rows for most SMs, else umma where it applies, else mma_sync.
    ``max_ctx``: the longest context among the portions, if the caller knows it: few query
    rows after many cached keys then have their keys shared out over several CTAs of the umma2
    kernel, whose partial results a second kernel merges (``splits`` forces a number).

    ``softcap`` c > 0: the scaled scores pass ``c tanh(s / c)``; ``out_scale``: a factor on
    the result; ``out`` may then also be a column block of a wider buffer.  These three are
    the umma2 variant's alone (``prefill_attention_takes_capped``)."""
    global _launches
    if q.dtype != torch.bfloat16 or d not in DECODE_HEAD_DIMS:
        raise KernelError(f"prefill_attention: bfloat16 and head_dim in {DECODE_HEAD_DIMS} only")
    if variant not in ("auto", "umma2", "umma", "mma_sync"):
        raise KernelError(f"prefill_attention: unknown variant {variant!r}")
    _want(items, torch.int32, "items")
    page_size = k_cache.shape[2]
    umma_ok = (d in (64, 128) and 8 <= page_size <= 64 and 64 % page_size == 0
               and q.is_contiguous() and q.data_ptr() % 16 == 0)
    umma2_ok = umma_ok and d == 128
    if variant == "umma" and not umma_ok or variant == "umma2" and not umma2_ok:
        raise KernelError(f"prefill_attention: the {variant} variant does not take head_dim {d} "
                          f"with pages of {page_size}")
    # umma2 gives an SM one block of 256 rows.  One portion, 32 heads, umma against umma2:
    # 12.8 / 15.0 us at 256 rows from position 0, 20.8 / 20.0 at 512, 44.4 / 29.7 at 1024;
    # after 8192 cached tokens 258 / 162 at 256 rows (58 with the keys shared out, below).
    blocks2 = -(-max_rows // 256) * nh * n_items
    use2 = umma2_ok and (variant == "umma2" or (variant == "auto" and (
        blocks2 >= 120 or max_rows > 256 or max_ctx >= 2048)))
    capped = softcap > 0 or out_scale != 1.0 or not out.is_contiguous()
    fn2, tail2 = lib().bf_prefill_attention_umma2, ()
    if capped:
        if not umma2_ok or variant not in ("auto", "umma2"):
            raise KernelError("prefill_attention: a soft cap, an output factor or an output in a "
                              "column block are the umma2 variant's alone")
        if out.stride(1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16 or out.dtype != q.dtype:
            raise KernelError("prefill_attention: out must have contiguous rows a multiple of 8 "
                              "elements apart, 16-byte aligned")
        use2 = True
        fn2 = lib().bf_prefill_attention_umma2_capped
        tail2 = (_c_float(softcap), _c_ll(out.stride(0)), _c_float(out_scale))
    # Few blocks and long contexts: share the keys of each block out (at least 16 key tiles a
    # share, at most 8 shares, no more CTAs than SMs).
    if splits <= 0:
        splits = 1
        if umma2_ok and variant in ("auto", "umma2") and not window and blocks2 * 2 <= num_sms(q.device):
            splits = max(1, min(8, num_sms(q.device) // blocks2, max_ctx // 1024))
    if splits > 1 and umma2_ok:
        T = q.shape[0]
        need = T * nh * splits
        if need * d * 4 <= _PREFILL_SPLIT_BYTES:
            key = q.device.index
            buf = _prefill_split_scratch.get(key)
            if buf is None or buf[0].numel() < need * d:
                buf = _prefill_split_scratch[key] = (
                    torch.empty(need * d, dtype=torch.float32, device=q.device),
                    torch.empty(need * 2, dtype=torch.float32, device=q.device))
            _run("prefill_attention_umma2", fn2,
                 _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
                 _c_int(max_rows), _c_int(T), _ptr(block_tables),
                 _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
                 _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
                 _c_float(scale), _c_int(splits), _ptr(buf[0]), _ptr(buf[1]), _ptr(err),
                 *tail2, _stream())
            _launches += 1          # two kernels: the shares and their merge
            return
    if use2:
        _run("prefill_attention_umma2", fn2,
             _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
             _c_int(max_rows), _c_int(q.shape[0]), _ptr(block_tables),
             _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
             _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0), _c_float(scale),
             _c_int(1), None, None, _ptr(err), *tail2, _stream())
        return
    if umma_ok and variant != "mma_sync":
        name = "prefill_attention_umma"
        _run(name, getattr(lib(), "bf_" + name),
             _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
             _c_int(max_rows), _c_int(q.shape[0]), _ptr(block_tables),
             _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
             _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0), _c_float(scale),
             _ptr(err), _stream())
        return
    _run("prefill_attention", lib().bf_prefill_attention,
         _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items), _c_int(max_rows),
         _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv),
         _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
         _c_float(scale), _ptr(err), _stream())


def prefill_attention_takes_capped(q: torch.Tensor, k_cache: torch.Tensor, d: int,
                                   dv: int) -> bool:
    """Whether ``prefill_attention`` with a soft cap, an output factor or a strided output (the
    umma2 variant) takes these sizes."""
    page_size = k_cache.shape[2]
    return (q.dtype == torch.bfloat16 and d == dv == 128 and 8 <= page_size <= 64
            and 64 % page_size == 0 and q.is_contiguous() and q.data_ptr() % 16 == 0)


# ------------------------------------------------------------------ layer norm
def add_layernorm(resid: torch.Tensor, delta: Optional[torch.Tensor],
                  delta2: Optional[torch.Tensor], weight: torch.Tensor,
                  bias: Optional[torch.Tensor], out: torch.Tensor, eps: float,
                  rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """out[i] = layernorm(resid[r] + delta[r] + delta2[r]) * weight + bias with r = rows[i]
    (or i); the sum is written back to resid when ``write_back``."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight")
    if bias is not None:
        _want(bias, torch.float32, "bias")
    n, H = out.shape
    for d in (delta, delta2):
        if d is not None and (d.dtype != out.dtype or not d.is_contiguous()
                              or d.shape != resid.shape):
            raise KernelError("a delta must be contiguous, of the stream's shape and of the "
                              "output's dtype")
    if rows is not None:
        _want(rows, torch.int32, "rows")
    _run("add_layernorm", lib().bf_add_layernorm, _ptr(resid), _ptr(delta), _ptr(delta2),
         _ptr(weight), _ptr(bias), _ptr(out), _ptr(rows), _c_int(n), _c_int(H), _c_float(eps),
         _c_int(_dtype_code(out)), _c_int(1 if write_back else 0), _stream())


# --------------------------------- projections that pass a short convolution over time
CONV_MAX_TAPS = 16


def conv_encode(proj: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int,
                state: Optional[torch.Tensor], state_slots: torch.Tensor,
                seq_of_token: torch.Tensor, q_start: torch.Tensor,
                inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                slots: Optional[torch.Tensor], q_out: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nh: int,
                nkv: int, dk: int, dv: int, unit_norm: bool, eps: float,
                err: torch.Tensor, pre_factor: Optional[torch.Tensor] = None,
                pre_weight: Optional[torch.Tensor] = None, rot_magnitude: float = 1.0,
                head_weight: Optional[torch.Tensor] = None,
                q_head_scale: Optional[torch.Tensor] = None) -> None:
    """``proj`` rows hold ``[q: nh dk | k: nkv dk | v: nkv dv]`` (a column block of a wider
    buffer is fine).  Per channel a causal convolution over the request's tokens with
    ``conv_w`` float32 ``[channels, taps]`` (``taps`` 0: none), whose reach behind the
    step's first row is read from ``state`` float32 ``[slots, (taps-1) * channels]`` (a column
    block of the slots' storage); then q and k turned by the position (``inv_freq``), each
    head of them divided by its root mean square when ``unit_norm``; q to ``q_out``, k and v
    into the pages at ``slots``.  The state is not changed: see :func:`conv_state_shift`.
    ``pre_factor`` float32 ``[T, 2]`` and ``pre_weight`` float32 ``[(nh + nkv) dk]``: q and k are
    multiplied by their token's factor and their channel's weight before the rotation (a norm
    over a whole projection: :func:`section_rms` takes the factors).  ``rot_magnitude``
    multiplies cosines and sines.  ``head_weight`` float32 ``[2, dk]``: behind the heads' norm,
    every q head is multiplied by the first row and every k head by the second.
    ``q_head_scale`` float32 ``[nh]``: q head h is multiplied by its number."""
    T = proj.shape[0]
    if head_weight is not None:
        _want(head_weight, torch.float32, "head_weight")
        if tuple(head_weight.shape) != (2, dk) or not head_weight.is_contiguous():
            raise KernelError("conv_encode: head_weight must be contiguous [2, dk]")
    if q_head_scale is not None:
        _want(q_head_scale, torch.float32, "q_head_scale")
        if q_head_scale.numel() != nh:
            raise KernelError("conv_encode: q_head_scale must have one number per query head")
    if pre_factor is not None:
        _want(pre_factor, torch.float32, "pre_factor"); _want(pre_weight, torch.float32, "pre_weight")
        if tuple(pre_factor.shape) != (T, 2) or pre_weight.numel() != (nh + nkv) * dk:
            raise KernelError("conv_encode: pre_factor must be [T, 2], pre_weight [(nh + nkv) dk]")
    C = nh * dk + nkv * (dk + dv)
    if proj.stride(1) != 1 or proj.shape[1] != C or q_out.stride(1) != 1:
        raise KernelError("conv_encode: proj must be [T, nh dk + nkv (dk + dv)] with contiguous rows")
    if taps > CONV_MAX_TAPS:
        raise KernelError(f"conv_encode: at most {CONV_MAX_TAPS} taps")
    if taps >= 1:
        _want(conv_w, torch.float32, "conv_w")
        if tuple(conv_w.shape) != (C, taps):
            raise KernelError("conv_encode: conv_w must be [channels, taps]")
    if taps > 1:
        if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] != (taps - 1) * C:
            raise KernelError("conv_encode: state must be float32 [slots, (taps-1) * channels]")
    if inv_freq is not None:
        _want(inv_freq, torch.float32, "inv_freq")
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    if 2 * rot_half > dk:
        raise KernelError("conv_encode: more rotated sizes than a head has")
    page_size = k_cache.shape[2] if k_cache is not None else 1
    num_slots = k_cache.shape[0] * page_size if k_cache is not None else 0
    if k_cache is not None and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    # cosines and sines of every token's angles, written by a small kernel in front
    table = (torch.empty((T, rot_half, 2), dtype=torch.float32, device=proj.device)
             if rot_half else None)
    _run("conv_encode", lib().bf_conv_encode, _ptr(proj), _c_ll(proj.stride(0)), _ptr(conv_w),
         _c_int(taps), _ptr(state), _c_ll(state.stride(0) if state is not None else 0),
         _ptr(state_slots), _c_int(state.shape[0] if state is not None else 0),
         _ptr(seq_of_token), _ptr(q_start), _ptr(inv_freq), _c_int(rot_half), _ptr(positions),
         _ptr(slots), _ptr(q_out), _c_ll(q_out.stride(0)), _ptr(k_cache), _ptr(v_cache), _c_int(T),
         _c_int(nh), _c_int(nkv), _c_int(dk), _c_int(dv), _c_int(page_size), _c_ll(num_slots),
         _c_int(1 if unit_norm else 0), _c_float(eps), _c_int(_dtype_code(proj)), _ptr(table),
         _ptr(err), _ptr(pre_factor), _ptr(pre_weight), _c_float(rot_magnitude),
         _ptr(head_weight), _ptr(q_head_scale), _stream())


def conv_state_shift(proj: torch.Tensor, state: torch.Tensor, state_slots: torch.Tensor,
                     q_start: torch.Tensor, B: int, taps: int) -> None:
    """After :func:`conv_encode`: every request's state becomes the projected values of its
    last ``taps - 1`` tokens (old rows stay where the step brought fewer)."""
    C = proj.shape[1]
    if taps <= 1:
        return
    if state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] != (taps - 1) * C:
        raise KernelError("conv_state_shift: state must be float32 [slots, (taps-1) * channels]")
    _run("conv_state_shift", lib().bf_conv_state_shift, _ptr(proj), _c_ll(proj.stride(0)),
         _ptr(state), _c_ll(state.stride(0)), _ptr(state_slots), _c_int(state.shape[0]),
         _ptr(q_start), _c_int(B), _c_int(C), _c_int(taps), _c_int(_dtype_code(proj)), _stream())


# ------------------------------------------------------------------------- retention
RETENTION_MAX_QK_DIM = 1024


def retention_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decays: torch.Tensor,
                   inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                   state: torch.Tensor, q_start: torch.Tensor, state_slots: torch.Tensor,
                   o_raw: torch.Tensor, B: int, heads: int, dk: int, dv: int, k_scale: float,
                   err: torch.Tensor, max_q: int = 0, silu: bool = False) -> None:
    """The recurrence ``S <- decay_h S + k v^T, o = S^T q`` over every request's tokens of the
    step.  ``proj`` rows hold q (``heads dk`` numbers from column ``q_off``), k (from
    ``k_off``) and v (``heads dv`` from ``v_off``); q and k are turned by the position
    (``inv_freq`` float32, None: not) and k multiplied by ``k_scale``.  ``state`` float32
    ``[slots, heads * dv * dk]`` (a column block of the slots' storage); ``o_raw`` float32
    ``[T, heads dv]``.  ``max_q``: the most tokens one request brings to the step, if the
    caller knows it (0: not known).  ``silu``: q, k and v pass silu first."""
    _want(decays, torch.float32, "decays"); _want(o_raw, torch.float32, "o_raw")
    if proj.stride(1) != 1 or dk > RETENTION_MAX_QK_DIM:
        raise KernelError(f"retention_scan: contiguous rows and a key size of at most "
                          f"{RETENTION_MAX_QK_DIM}")
    if (state.dtype != torch.float32 or state.stride(1) != 1
            or state.shape[1] != heads * dk * dv or decays.numel() != heads):
        raise KernelError("retention_scan: state must be float32 [slots, heads * dk * dv] and "
                          "decays [heads]")
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    if 2 * rot_half > dk:
        raise KernelError("retention_scan: more rotated sizes than a head has")
    T = proj.shape[0]
    # the turned q and k and the values of every token in float: written by the first of the
    # two kernels
    qk = torch.empty((T, 2, heads, dk), dtype=torch.float32, device=proj.device)
    vf = torch.empty((T, heads, dv), dtype=torch.float32, device=proj.device)
    _run("retention_scan", lib().bf_retention_scan, _ptr(proj), _c_ll(proj.stride(0)),
         _c_ll(q_off), _c_ll(k_off), _c_ll(v_off), _ptr(decays), _ptr(inv_freq), _c_int(rot_half),
         _ptr(positions), _ptr(state), _c_ll(state.stride(0)), _ptr(q_start), _ptr(state_slots),
         _c_int(state.shape[0]), _ptr(o_raw), _ptr(qk), _ptr(vf), _c_int(T), _c_int(B),
         _c_int(max_q if max_q > 0 else T), _c_int(heads), _c_int(dk), _c_int(dv), _c_float(k_scale), _c_int(_dtype_code(proj)), _ptr(err),
         _c_int(1 if silu else 0), _stream())
    global _launches
    _launches += 1          # two kernels: the rotation and the scan


def linear_scan(qk: torch.Tensor, vf: torch.Tensor, tok_decay: torch.Tensor, state: torch.Tensor,
                q_start: torch.Tensor, state_slots: torch.Tensor, o_raw: torch.Tensor, B: int,
                heads: int, qk_heads: int, dk: int, dv: int, err: torch.Tensor,
                max_q: int = 0) -> None:
    """The recurrence ``S <- decay[t, h] S + k v^T, o = S^T q`` over every request's tokens of
    the step, on inputs that are float already: ``qk [T, 2, qk_heads, dk]`` (q, then k; head h
    reads head ``h // (heads / qk_heads)``), ``vf [T, heads, dv]``, ``tok_decay [T, heads]``.
    ``state`` float32 ``[slots, heads * dv * dk]`` (a column block of the slots' storage);
    ``o_raw`` float32 ``[T, heads dv]``.  ``max_q``: the most tokens one request brings."""
    for name, t in (("qk", qk), ("vf", vf), ("tok_decay", tok_decay), ("o_raw", o_raw)):
        _want(t, torch.float32, name)
        if not t.is_contiguous():
            raise KernelError(f"linear_scan: {name} must be contiguous")
    T = vf.shape[0]
    if (dk > RETENTION_MAX_QK_DIM or qk_heads <= 0 or heads % qk_heads
            or qk.numel() != T * 2 * qk_heads * dk or vf.numel() != T * heads * dv
            or tok_decay.numel() != T * heads or o_raw.numel() != T * heads * dv):
        raise KernelError(f"linear_scan: qk [T, 2, qk_heads, dk], vf [T, heads, dv], tok_decay "
                          f"[T, heads], keys of at most {RETENTION_MAX_QK_DIM}")
    if (state.dtype != torch.float32 or state.stride(1) != 1
            or state.shape[1] != heads * dk * dv):
        raise KernelError("linear_scan: state must be float32 [slots, heads * dk * dv]")
    _run("linear_scan", lib().bf_linear_scan, _ptr(qk), _ptr(vf), _ptr(tok_decay), _ptr(state),
         _c_ll(state.stride(0)), _ptr(q_start), _ptr(state_slots), _c_int(state.shape[0]),
         _ptr(o_raw), _c_int(T), _c_int(B), _c_int(max_q if max_q > 0 else T), _c_int(heads),
         _c_int(qk_heads), _c_int(dk), _c_int(dv), _ptr(err), _stream())


def mamba2_encode(proj: torch.Tensor, xbc_off: int, dt_off: int, conv_w: Optional[torch.Tensor],
                  conv_b: Optional[torch.Tensor], taps: int, state: Optional[torch.Tensor],
                  state_slots: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor,
                  A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor, qk: torch.Tensor,
                  vf: torch.Tensor, skip: torch.Tensor, decay: torch.Tensor, heads: int,
                  groups: int, N: int, P: int, err: torch.Tensor) -> None:
    """What lies between a state space layer's input projection and its recurrence.  ``proj``
    rows hold, from ``xbc_off``, ``[x: heads P | B: groups N | C: groups N]`` (the channels that
    pass the causal convolution ``conv_w`` float32 ``[channels, taps]`` with the bias ``conv_b``
    and ``silu``; the reach behind the step's first row is read from ``state`` float32
    ``[slots, (taps-1) * channels]``, which is not changed: :func:`conv_state_shift`) and, from
    ``dt_off``, one step size per head.  Results, float32: ``qk [T, 2, groups, N]`` (C, then
    B), ``vf [T, heads, P]`` (``dt x``), ``skip [T, heads, P]`` (``D_h x``), ``decay [T, heads]``
    (``exp(-exp(A_log_h) dt)``) with ``dt = softplus(dt + dt_bias_h)``."""
    T = proj.shape[0]
    C = heads * P + 2 * groups * N
    if proj.stride(1) != 1 or xbc_off + C > proj.shape[1] or dt_off + heads > proj.shape[1]:
        raise KernelError("mamba2_encode: proj rows must be contiguous and hold the channels")
    if taps > CONV_MAX_TAPS:
        raise KernelError(f"mamba2_encode: at most {CONV_MAX_TAPS} taps")
    if taps >= 1:
        _want(conv_w, torch.float32, "conv_w")
        if tuple(conv_w.shape) != (C, taps) or not conv_w.is_contiguous():
            raise KernelError("mamba2_encode: conv_w must be [channels, taps]")
    if conv_b is not None:
        _want(conv_b, torch.float32, "conv_b")
        if conv_b.numel() != C:
            raise KernelError("mamba2_encode: conv_b must be [channels]")
    if taps > 1 and (state.dtype != torch.float32 or state.stride(1) != 1
                     or state.shape[1] != (taps - 1) * C):
        raise KernelError("mamba2_encode: state must be float32 [slots, (taps-1) * channels]")
    for name, t, n in (("A_log", A_log, heads), ("dt_bias", dt_bias, heads), ("D", D, heads),
                       ("qk", qk, T * 2 * groups * N), ("vf", vf, T * heads * P),
                       ("skip", skip, T * heads * P), ("decay", decay, T * heads)):
        _want(t, torch.float32, name)
        if t.numel() != n or not t.is_contiguous():
            raise KernelError(f"mamba2_encode: {name} has the wrong size")
    _run("mamba2_encode", lib().bf_mamba2_encode, _ptr(proj), _c_ll(proj.stride(0)),
         _c_ll(xbc_off), _c_ll(dt_off), _ptr(conv_w if taps >= 1 else None), _ptr(conv_b),
         _c_int(taps), _ptr(state), _c_ll(state.stride(0) if state is not None else 0),
         _ptr(state_slots), _c_int(state.shape[0] if state is not None else 0),
         _ptr(seq_of_token), _ptr(q_start), _ptr(A_log), _ptr(dt_bias), _ptr(D), _ptr(qk),
         _ptr(vf), _ptr(skip), _ptr(decay), _c_int(T), _c_int(heads), _c_int(groups), _c_int(N),
         _c_int(P), _c_int(_dtype_code(proj)), _ptr(err), _stream())


def gate_norm_out(o_raw: torch.Tensor, skip: Optional[torch.Tensor], proj: torch.Tensor,
                  z_off: int, weight: Optional[torch.Tensor], out: torch.Tensor, parts: int,
                  eps: float) -> None:
    """``y = (o_raw + skip) * silu(proj[:, z_off:])``, then an RMS norm in ``parts`` equal parts
    of the row (each by its own root mean square), times ``weight`` float32 ``[n]``; the gate
    comes before the norm.  ``o_raw`` and ``skip`` float32 ``[T, n]``; ``out [T, n]`` of the
    projection's type (a column block of a wider buffer is fine)."""
    _want(o_raw, torch.float32, "o_raw")
    T, n = o_raw.shape
    if skip is not None:
        _want(skip, torch.float32, "skip")
        if skip.numel() != T * n or not skip.is_contiguous():
            raise KernelError("gate_norm_out: skip must be contiguous [T, n]")
    if weight is not None:
        _want(weight, torch.float32, "weight")
        if weight.numel() != n:
            raise KernelError("gate_norm_out: weight must have n numbers")
    if (not o_raw.is_contiguous() or out.stride(1) != 1 or out.dtype != proj.dtype
            or proj.stride(1) != 1 or parts <= 0 or n % parts or z_off + n > proj.shape[1]):
        raise KernelError("gate_norm_out: contiguous rows, out of the projection's type, parts "
                          "that divide the row")
    _run("gate_norm_out", lib().bf_gate_norm_out, _ptr(o_raw), _ptr(skip), _ptr(proj),
         _c_ll(proj.stride(0)), _c_ll(z_off), _ptr(weight), _ptr(out), _c_ll(out.stride(0)),
         _c_int(T), _c_int(n), _c_int(parts), _c_float(eps), _c_int(_dtype_code(proj)), _stream())


def retention_out(o_raw: torch.Tensor, proj: torch.Tensor, g_off: int, out: torch.Tensor,
                  heads: int, dv: int, eps: float, out_scale: float = 1.0) -> None:
    """``out = o_raw / rms_per_head(o_raw) * silu(proj[:, g_off:]) * out_scale``; ``out`` may be
    a column block of a wider buffer."""
    _want(o_raw, torch.float32, "o_raw")
    T = o_raw.shape[0]
    if out.stride(1) != 1 or out.dtype != proj.dtype or proj.stride(1) != 1:
        raise KernelError("retention_out: rows must be contiguous, out of the projection's type")
    _run("retention_out", lib().bf_retention_out, _ptr(o_raw), _ptr(proj), _c_ll(proj.stride(0)),
         _c_ll(g_off), _ptr(out), _c_ll(out.stride(0)), _c_int(T), _c_int(heads), _c_int(dv),
         _c_float(eps), _c_float(out_scale), _c_int(_dtype_code(proj)), _stream())


# ------------------------------------------- between a mixer's projection and its core
def section_rms(x: torch.Tensor, off0: int, n0: int, off1: int, n1: int, eps: float,
                out: torch.Tensor) -> None:
    """``out[t, s] = rsqrt(mean(x[t, off_s : off_s + n_s]^2) + eps)`` for two column sections
    of every row: the factors of RMS norms over whole projections."""
    T = x.shape[0]
    _want(out, torch.float32, "out")
    if x.stride(1) != 1 or tuple(out.shape) != (T, 2):
        raise KernelError("section_rms: contiguous rows and out [T, 2]")
    _run("section_rms", lib().bf_section_rms, _ptr(x), _c_ll(x.stride(0)), _c_int(off0),
         _c_int(n0), _c_int(off1), _c_int(n1), _c_float(eps), _ptr(out), _c_int(T),
         _c_int(_dtype_code(x)), _stream())


def section_norm(x: torch.Tensor, off: int, n: int, weight: torch.Tensor, eps: float,
                 out: torch.Tensor) -> None:
    """``out[t] = rmsnorm(x[t, off:off + n]) * weight``: an RMS norm with a weight (float32
    ``[n]``) over a column section of every row, into ``out [T, n]`` of ``x``'s type."""
    _want(weight, torch.float32, "weight")
    T = x.shape[0]
    if (x.stride(1) != 1 or out.stride(1) != 1 or out.dtype != x.dtype or weight.numel() != n
            or tuple(out.shape) != (T, n) or off < 0 or off + n > x.shape[1]):
        raise KernelError("section_norm: contiguous rows, weight [n], out [T, n] of x's type")
    _run("section_norm", lib().bf_section_norm, _ptr(x), _c_ll(x.stride(0)), _c_ll(off), _c_int(n),
         _ptr(weight), _c_float(eps), _ptr(out), _c_ll(out.stride(0)), _c_int(T),
         _c_int(_dtype_code(x)), _stream())


def latent_encode(proj: torch.Tensor, q_off: int, kv_off: int, norm_w: torch.Tensor, eps: float,
                  inv_freq: Optional[torch.Tensor], interleaved: bool, rot_magnitude: float,
                  positions: torch.Tensor, slots: Optional[torch.Tensor], q_abs: torch.Tensor,
                  cache: Optional[torch.Tensor], heads: int, d: int, dr: int, rank: int,
                  err: torch.Tensor, q: Optional[torch.Tensor] = None) -> None:
    """Attention over a cached latent, before the scores: ``proj`` rows hold ``heads`` query
    heads of ``[d plain | dr rotated]`` from ``q_off`` (or ``q [T, heads (d + dr)]`` holds
    them, a buffer of its own of ``proj``'s type) and ``[rank | dr]`` from ``kv_off``.
    The cache row of a token (pages ``[pages, 1, page_size, rank + dr]``, at ``slots``)
    becomes ``[rmsnorm(first rank) * norm_w | rotated dr]``; ``q_abs [T, heads, rank + dr]``
    gets every head's rotated part at ``[rank, rank + dr)`` and is otherwise left alone."""
    T = proj.shape[0]
    _want(norm_w, torch.float32, "norm_w")
    if proj.stride(1) != 1 or not q_abs.is_contiguous() or q_abs.dtype != proj.dtype:
        raise KernelError("latent_encode: contiguous rows, q_abs contiguous and of proj's type")
    if tuple(q_abs.shape) != (T, heads, rank + dr) or norm_w.numel() != rank:
        raise KernelError("latent_encode: q_abs must be [T, heads, rank + dr], norm_w [rank]")
    if q is None:
        q = proj[:, q_off:q_off + heads * (d + dr)]
    if q.dtype != proj.dtype or q.stride(1) != 1 or tuple(q.shape) != (T, heads * (d + dr)):
        raise KernelError("latent_encode: q must be [T, heads (d + dr)] of proj's type")
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    page_size, num_slots = 1, 0
    if cache is not None:
        if not cache.is_contiguous() or cache.shape[1] != 1 or cache.shape[3] != rank + dr:
            raise KernelError("latent_encode: pages must be contiguous [pages, 1, size, rank + dr]")
        page_size, num_slots = cache.shape[2], cache.shape[0] * cache.shape[2]
    _run("latent_encode", lib().bf_latent_encode, _ptr(proj), _c_ll(proj.stride(0)), _ptr(q),
         _c_ll(q.stride(0)), _c_ll(kv_off), _ptr(norm_w), _c_float(eps), _ptr(inv_freq), _c_int(rot_half),
         _c_int(1 if interleaved else 0), _c_float(rot_magnitude), _ptr(positions),
         _ptr(slots if cache is not None else None), _ptr(q_abs), _ptr(cache), _c_int(T),
         _c_int(heads), _c_int(d), _c_int(dr), _c_int(rank), _c_int(page_size), _c_ll(num_slots),
         _c_int(_dtype_code(proj)), _ptr(err), _stream())


def delta_encode(proj: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int,
                 state: Optional[torch.Tensor], state_slots: torch.Tensor,
                 seq_of_token: torch.Tensor, q_start: torch.Tensor, b_off: int, a_off: int,
                 A_log: torch.Tensor, dt_bias: torch.Tensor, qkv: torch.Tensor,
                 gates: torch.Tensor, heads: int, qk_heads: int, dk: int, dv: int,
                 unit_eps: float, q_scale: float, err: torch.Tensor) -> None:
    """The gated delta rule's inputs.  ``proj`` rows hold ``[q: qk_heads dk | k: qk_heads dk |
    v: heads dv]`` from column 0 and one logit per value head at ``b_off`` and at ``a_off``.
    The first block passes a causal convolution per channel (``conv_w`` float32 ``[channels,
    taps]``, reach behind the step's first row from ``state`` float32 ``[slots, (taps-1)
    channels]``) and silu; q and k heads become unit vectors, q times ``q_scale``.  ``qkv``
    float32 ``[T, channels]``; ``gates`` float32 ``[T, 2, heads]``: ``sigmoid(b)`` and
    ``exp(-exp(A_log) softplus(a + dt_bias))``.  The state is not changed: see
    :func:`conv_state_shift`."""
    T = proj.shape[0]
    C = 2 * qk_heads * dk + heads * dv
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (qkv, "qkv"), (gates, "gates")):
        _want(t, torch.float32, n)
    if proj.stride(1) != 1 or tuple(qkv.shape) != (T, C) or tuple(gates.shape) != (T, 2, heads):
        raise KernelError("delta_encode: contiguous rows, qkv [T, channels], gates [T, 2, heads]")
    if taps > CONV_MAX_TAPS:
        raise KernelError(f"delta_encode: at most {CONV_MAX_TAPS} taps")
    if taps >= 1:
        _want(conv_w, torch.float32, "conv_w")
        if tuple(conv_w.shape) != (C, taps):
            raise KernelError("delta_encode: conv_w must be [channels, taps]")
    if taps > 1 and (state.dtype != torch.float32 or state.stride(1) != 1
                     or state.shape[1] != (taps - 1) * C):
        raise KernelError("delta_encode: state must be float32 [slots, (taps-1) * channels]")
    has_state = taps > 1
    _run("delta_encode", lib().bf_delta_encode, _ptr(proj), _c_ll(proj.stride(0)),
         _ptr(conv_w if taps >= 1 else None), _c_int(taps), _ptr(state if has_state else None),
         _c_ll(state.stride(0) if has_state else 0), _ptr(state_slots),
         _c_int(state.shape[0] if has_state else 0), _ptr(seq_of_token), _ptr(q_start),
         _c_ll(b_off), _c_ll(a_off), _ptr(A_log), _ptr(dt_bias), _ptr(qkv), _ptr(gates), _c_int(T),
         _c_int(heads), _c_int(qk_heads), _c_int(dk), _c_int(dv), _c_float(unit_eps),
         _c_float(q_scale), _c_int(_dtype_code(proj)), _ptr(err), _stream())


DELTA_MAX_QK_DIM = 1024


def delta_scan(qkv: torch.Tensor, gates: torch.Tensor, state: torch.Tensor,
               q_start: torch.Tensor, state_slots: torch.Tensor, o_raw: torch.Tensor, B: int,
               heads: int, qk_heads: int, dk: int, dv: int, err: torch.Tensor,
               max_q: int = 0) -> None:
    """The recurrence ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` over every
    request's tokens of the step, from :func:`delta_encode`'s ``qkv`` and ``gates``.  ``state``
    float32 ``[slots, heads * dv * dk]`` (a column block of the slots' storage); ``o_raw``
    float32 ``[T, heads dv]``."""
    T = qkv.shape[0]
    for t, n in ((qkv, "qkv"), (gates, "gates"), (o_raw, "o_raw")):
        _want(t, torch.float32, n)
    if (state.dtype != torch.float32 or state.stride(1) != 1
            or state.shape[1] != heads * dk * dv or dk > DELTA_MAX_QK_DIM):
        raise KernelError("delta_scan: state must be float32 [slots, heads * dk * dv]")
    _run("delta_scan", lib().bf_delta_scan, _ptr(qkv), _ptr(gates), _ptr(state),
         _c_ll(state.stride(0)), _ptr(q_start), _ptr(state_slots), _c_int(state.shape[0]),
         _ptr(o_raw), _c_int(T), _c_int(B), _c_int(max_q if max_q > 0 else T), _c_int(heads),
         _c_int(qk_heads), _c_int(dk), _c_int(dv), _ptr(err), _stream())


def gated_norm_out(o_raw: torch.Tensor, proj: torch.Tensor, g_off: int,
                   weight: Optional[torch.Tensor], out: torch.Tensor, heads: int, dv: int,
                   eps: float, over_all: bool = False, gate: str = "silu",
                   out_scale: float = 1.0) -> None:
    """``out = o_raw / rms(o_raw) * weight * act(proj[:, g_off:]) * out_scale``: the root mean
    square per head, or over all heads of a token (``over_all``); ``weight`` None, float32
    ``[dv]`` (shared by the heads) or ``[heads dv]``; ``gate`` "silu" or "sigmoid".  ``out``
    may be a column block of a wider buffer."""
    _want(o_raw, torch.float32, "o_raw")
    T = o_raw.shape[0]
    if out.stride(1) != 1 or out.dtype != proj.dtype or proj.stride(1) != 1:
        raise KernelError("gated_norm_out: rows must be contiguous, out of the projection's type")
    w_mode = 0
    if weight is not None:
        _want(weight, torch.float32, "weight")
        if weight.numel() == dv and heads > 1:
            w_mode = 1
        elif weight.numel() == heads * dv:
            w_mode = 2
        else:
            raise KernelError("gated_norm_out: weight must have dv or heads * dv numbers")
    if gate not in ("silu", "sigmoid"):
        raise KernelError(f"gated_norm_out: unknown gate {gate!r}")
    _run("gated_norm_out", lib().bf_gated_norm_out, _ptr(o_raw), _ptr(proj),
         _c_ll(proj.stride(0)), _c_ll(g_off), _ptr(weight), _c_int(w_mode),
         _c_int(1 if over_all else 0), _c_int(1 if gate == "sigmoid" else 0), _ptr(out),
         _c_ll(out.stride(0)), _c_int(T), _c_int(heads), _c_int(dv), _c_float(eps),
         _c_float(out_scale), _c_int(_dtype_code(proj)), _stream())


def head_gate_mul(x: torch.Tensor, gate: torch.Tensor, heads: int, dv: int) -> None:
    """``x[t, h, :] *= sigmoid(gate[t, h])``; ``x [T, heads dv]`` contiguous, ``gate`` a view
    ``[T, heads]`` of rows of the same type."""
    if not x.is_contiguous() or gate.stride(1) != 1 or gate.dtype != x.dtype:
        raise KernelError("head_gate_mul: x contiguous, gate rows contiguous and of x's type")
    _run("head_gate_mul", lib().bf_head_gate_mul, _ptr(x), _ptr(gate), _c_ll(gate.stride(0)),
         _c_int(x.shape[0]), _c_int(heads), _c_int(dv), _c_int(_dtype_code(x)), _stream())


def stream_inject(resid: torch.Tensor, delta: Optional[torch.Tensor],
                  table: Optional[torch.Tensor], ids: Optional[torch.Tensor], scale: float,
                  vec: Optional[torch.Tensor], err: torch.Tensor) -> None:
    """``resid[t] += delta[t] + table[ids[t]] * scale + vec``; each of the three may be None."""
    _want(resid, torch.float32, "resid")
    T, width = resid.shape
    if delta is not None and (not delta.is_contiguous() or delta.shape != resid.shape):
        raise KernelError("stream_inject: delta must be contiguous and of the stream's shape")
    if vec is not None:
        _want(vec, torch.float32, "vec")
        if vec.numel() != width:
            raise KernelError("stream_inject: vec must have the stream's width")
    if table is not None:
        _want(ids, torch.int32, "ids")
    _run("stream_inject", lib().bf_stream_inject, _ptr(resid), _ptr(delta),
         _c_int(_dtype_code(delta) if delta is not None else 0), _ptr(table),
         _c_int(_dtype_code(table) if table is not None else 0), _ptr(ids),
         _c_int(table.shape[0] if table is not None else 0), _c_float(scale), _ptr(vec),
         _c_int(T), _c_int(width), _ptr(err), _stream())


# ---------------------------------------------------------------- mixture of experts
def moe_route(h: torch.Tensor, w: torch.Tensor, experts: int, top: int, shared_gate: bool,
              route_w: torch.Tensor, top_ids: torch.Tensor, top_w: torch.Tensor,
              scoring: str = "softmax_top", correction: Optional[torch.Tensor] = None,
              groups: int = 1, groups_keep: int = 1, identity: int = 0,
              route_scale: float = 1.0, weight_eps: float = 0.0) -> None:
    """Router of a mixture of experts: ``w`` float32 ``[experts + identity (+1), width]`` (the
    last row the shared expert's gate when ``shared_gate``), ``h [T, width]``.  ``route_w``
    float32 ``[T, experts (+1) (+1)]`` gets every expert's weight for the token (zero: not
    chosen), then ``sigmoid(w_sg . h)`` when ``shared_gate``, then (``identity`` > 0) the sum of
    the weights of the chosen outputs that stand for experts returning their input;
    ``top_ids`` int32 and ``top_w`` float32 ``[T, top]`` the chosen outputs, best first.

    ``scoring`` "softmax_top": the largest logits are chosen and weighted by the softmax over
    them alone.  "softmax_all": scores are the softmax over all ``experts + identity``
    outputs, ``correction`` (float32, one number per output) is added for the choice only,
    with ``groups`` > 1 only the outputs of the ``groups_keep`` groups with the largest best
    choice score can be chosen, and the weights are the chosen scores over their sum (plus
    ``weight_eps``) times ``route_scale``."""
    T, width = h.shape
    if scoring not in ("softmax_top", "softmax_all"):
        raise KernelError(f"moe_route: unknown scoring {scoring!r}")
    mode = 1 if scoring == "softmax_all" else 0
    if mode == 0 and (identity or groups > 1 or correction is not None):
        raise KernelError("moe_route: corrections, groups and identity outputs go with the "
                          "softmax over all outputs")
    rows = experts + identity + (1 if shared_gate else 0)
    cols = experts + (1 if shared_gate else 0) + (1 if identity else 0)
    _want(w, torch.float32, "w"); _want(route_w, torch.float32, "route_w")
    _want(top_ids, torch.int32, "top_ids"); _want(top_w, torch.float32, "top_w")
    if (tuple(w.shape) != (rows, width) or tuple(route_w.shape) != (T, cols) or h.stride(1) != 1
            or not route_w.is_contiguous()):
        raise KernelError("moe_route: w must be [experts + identity (+1), width], route_w "
                          "[T, experts (+1) (+1)]")
    if correction is not None:
        _want(correction, torch.float32, "correction")
        if correction.numel() != experts + identity:
            raise KernelError("moe_route: correction must have one number per router output")
    n = experts + identity
    if (groups < 1 or n % groups or not 1 <= groups_keep <= groups or not 1 <= top <= n
            or top > groups_keep * (n // groups)):
        raise KernelError("moe_route: groups must divide the outputs and hold the choices")
    _run("moe_route", lib().bf_moe_route, _ptr(h), _c_ll(h.stride(0)), _ptr(w), _c_int(T),
         _c_int(width), _c_int(experts), _c_int(top), _c_int(1 if shared_gate else 0),
         _ptr(route_w), _ptr(top_ids), _ptr(top_w), _c_int(_dtype_code(h)), _c_int(mode),
         _ptr(correction), _c_int(groups), _c_int(groups_keep), _c_int(identity),
         _c_float(route_scale), _c_float(weight_eps), _stream())


def moe_act(gu: torch.Tensor, route_w: torch.Tensor, act: torch.Tensor, experts: int,
            ff: int, shared_gate: Optional[bool] = None) -> None:
    """``act[t, c] = silu(gu[t, c]) * gu[t, F + c] * route_w[t, expert(c)]`` with
    ``expert(c) = c // ff`` for ``c < experts * ff``; the columns behind the experts' (a shared
    expert) take column ``experts`` of ``route_w`` when ``shared_gate``, else the weight one
    (None: when ``route_w`` has exactly one column more than there are experts)."""
    T, F = act.shape
    _want(route_w, torch.float32, "route_w")
    if tuple(gu.shape) != (T, 2 * F) or not gu.is_contiguous() or not act.is_contiguous() \
            or gu.dtype != act.dtype or route_w.shape[0] != T or not route_w.is_contiguous():
        raise KernelError("moe_act: gu must be contiguous [T, 2 F] of act's type")
    if shared_gate is None:
        shared_gate = route_w.shape[1] == experts + 1
    _run("moe_act", lib().bf_moe_act, _ptr(gu), _ptr(route_w), _ptr(act), _c_int(T), _c_int(F),
         _c_int(experts), _c_int(ff), _c_int(route_w.shape[1]), _c_int(1 if shared_gate else 0),
         _c_int(_dtype_code(act)), _stream())


def moe_identity_add(out: torch.Tensor, h: torch.Tensor, route_w: torch.Tensor, col: int) -> None:
    """``out[t] += h[t] * route_w[t, col]``: the experts that return their input."""
    _want(route_w, torch.float32, "route_w")
    T, width = out.shape
    if (not out.is_contiguous() or h.stride(1) != 1 or h.dtype != out.dtype
            or tuple(h.shape) != (T, width) or route_w.shape[0] != T
            or not route_w.is_contiguous() or not 0 <= col < route_w.shape[1]):
        raise KernelError("moe_identity_add: out contiguous [T, width], h of its shape and type")
    _run("moe_identity_add", lib().bf_moe_identity_add, _ptr(out), _ptr(h), _c_ll(h.stride(0)),
         _ptr(route_w), _c_int(route_w.shape[1]), _c_int(col), _c_int(T), _c_int(width),
         _c_int(_dtype_code(out)), _stream())


def moe_sparse_takes(width: int, ff: int, ff_sh: int, top: int) -> bool:
    """Whether :func:`moe_sparse` takes these sizes (a token's input and its chosen experts'
    activations each fit a block's shared memory as float)."""
    return width * 4 <= 48 * 1024 and (top * ff + ff_sh) * 4 <= 48 * 1024


def moe_sparse(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
               top_ids: torch.Tensor, top_w: torch.Tensor, route_w: torch.Tensor,
               out: torch.Tensor, experts: int, ff: int, ff_sh: int, top: int,
               shared_gate: Optional[bool] = None, identity_col: int = -1) -> None:
    """The mixture's output for a step of very few tokens, reading only the experts that
    were chosen (and the shared one): ``w_gate_up [2 F, width]`` and ``w_down [width, F]`` are
    the stacked weights (``F = experts * ff + ff_sh``), ``top_ids``/``top_w``/``route_w`` what
    :func:`moe_route` left; ``out [T, width]``.  ``shared_gate``: column ``experts`` of
    ``route_w`` is the shared expert's weight (None: when ``route_w`` has exactly one column
    more than there are experts).  ``identity_col`` >= 0: chosen ids from ``experts`` on return
    their input, and that column of ``route_w`` holds their weights' sum."""
    T, width = h.shape
    F = experts * ff + ff_sh
    if shared_gate is None:
        shared_gate = route_w.shape[1] == experts + 1
    if (tuple(w_gate_up.shape) != (2 * F, width) or tuple(w_down.shape) != (width, F)
            or not w_gate_up.is_contiguous() or not w_down.is_contiguous()
            or w_gate_up.dtype != h.dtype or w_down.dtype != h.dtype or h.stride(1) != 1
            or not out.is_contiguous() or out.dtype != h.dtype):
        raise KernelError("moe_sparse: stacked weights [2 F, width] and [width, F] of h's type")
    if not moe_sparse_takes(width, ff, ff_sh, top):
        raise KernelError("moe_sparse: sizes too large for a block's shared memory")
    _want(top_ids, torch.int32, "top_ids"); _want(top_w, torch.float32, "top_w")
    _want(route_w, torch.float32, "route_w")
    act = torch.empty((T, top * ff + ff_sh), dtype=h.dtype, device=h.device)
    _run("moe_sparse", lib().bf_moe_sparse, _ptr(h), _c_ll(h.stride(0)), _ptr(w_gate_up),
         _ptr(w_down), _ptr(top_ids), _ptr(top_w), _ptr(route_w), _c_int(route_w.shape[1]),
         _ptr(act), _ptr(out), _c_int(T), _c_int(width), _c_int(experts), _c_int(ff),
         _c_int(ff_sh), _c_int(top), _c_int(_dtype_code(h)), _c_int(1 if shared_gate else 0),
         _c_int(identity_col), _stream())
    global _launches
    _launches += 1          # two kernels


# ----------------------------------------------------- norm on a sublayer's output
def rmsnorm_add(resid: torch.Tensor, y: torch.Tensor, weight: torch.Tensor,
                reading: Optional[torch.Tensor], eps: float) -> None:
    """``resid += y * rsqrt(mean(y^2) + eps) * weight`` row by row (``resid`` float32
    ``[T, H]``), and, if ``reading`` is given, the new rows in its type."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight")
    T, H = resid.shape
    if y.shape != resid.shape or not y.is_contiguous():
        raise KernelError("rmsnorm_add: y must be contiguous and of the stream's shape")
    if reading is not None and (reading.dtype != y.dtype or reading.shape != resid.shape
                                or not reading.is_contiguous()):
        raise KernelError("rmsnorm_add: the reading must be contiguous, of y's type and shape")
    _run("rmsnorm_add", lib().bf_rmsnorm_add, _ptr(resid), _ptr(y), _ptr(weight), _ptr(reading),
         _c_int(T), _c_int(H), _c_float(eps), _c_int(_dtype_code(y)), _stream())


def stream_to_bf16(x: torch.Tensor, out: torch.Tensor) -> None:
    _want(x, torch.float32, "x"); _want(out, torch.bfloat16, "out")
    _run("stream_to_bf16", lib().bf_stream_to_bf16, _ptr(x), _ptr(out), _c_ll(x.numel()),
         _stream())


# ------------------------------------------------------------------ matrix memory (mLSTM)
def mlstm_gates(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                gates: torch.Tensor, heads: int, cap: float) -> None:
    """``gates [T, 2 heads]`` float32 from ``h [T, width]`` and ``w [2 heads, width]`` (input
    gate rows, then forget gate rows): the capped pre-activation for an input gate, its
    log-sigmoid for a forget gate."""
    T, width = h.shape
    if h.stride(1) != 1 or w.shape != (2 * heads, width) or not w.is_contiguous() \
            or w.dtype != h.dtype:
        raise KernelError("mlstm_gates: w must be contiguous [2 heads, width] of h's type")
    _want(gates, torch.float32, "gates")
    if bias is not None:
        _want(bias, torch.float32, "bias")
    _run("mlstm_gates", lib().bf_mlstm_gates, _ptr(h), _c_ll(h.stride(0)), _ptr(w), _ptr(bias),
         _ptr(gates), _c_int(T), _c_int(width), _c_int(heads), _c_float(cap),
         _c_int(_dtype_code(h)), _stream())


MLSTM_MAX_QK_DIM = 256


def mlstm_state_size(dk: int, dv: int) -> int:
    """Floats of one head's state: S, n, m and padding to a multiple of four."""
    return dk * dv + dk + 4


def mlstm_scan(proj: torch.Tensor, gates: torch.Tensor, state: torch.Tensor,
               q_start: torch.Tensor, state_slots: torch.Tensor, o_raw: torch.Tensor, B: int,
               heads: int, dk: int, dv: int, q_scale: float, err: torch.Tensor) -> None:
    """The recurrence over every request's tokens of this step.  ``proj`` rows hold
    ``[q: heads dk | k: heads dk | v: heads dv | ...]``; ``state`` is float32
    ``[slots, heads, mlstm_state_size]``; ``o_raw`` float32 ``[T, heads dv]`` receives the
    memory's output before its norm and gate."""
    _want(gates, torch.float32, "gates"); _want(state, torch.float32, "state")
    _want(o_raw, torch.float32, "o_raw")
    if proj.stride(1) != 1 or dk > MLSTM_MAX_QK_DIM:
        raise KernelError(f"mlstm_scan: contiguous rows and a key size of at most "
                          f"{MLSTM_MAX_QK_DIM}")
    if state.shape[1:] != (heads, mlstm_state_size(dk, dv)):
        raise KernelError("mlstm_scan: state must be [slots, heads, mlstm_state_size(dk, dv)]")
    _run("mlstm_scan", lib().bf_mlstm_scan, _ptr(proj), _c_ll(proj.stride(0)), _ptr(gates),
         _ptr(state), _c_ll(state.stride(0)), _c_int(state.shape[2]), _ptr(q_start),
         _ptr(state_slots), _c_int(state.shape[0]), _ptr(o_raw), _c_int(B), _c_int(heads),
         _c_int(dk), _c_int(dv), _c_float(q_scale), _c_int(_dtype_code(proj)), _ptr(err),
         _stream())


def mlstm_out(o_raw: torch.Tensor, proj: torch.Tensor, g_off: int, norm_w: torch.Tensor,
              out: torch.Tensor, heads: int, dv: int, eps: float) -> None:
    """``out = o_raw / rms_per_head(o_raw) * norm_w * sigmoid(proj[:, g_off:])``."""
    _want(o_raw, torch.float32, "o_raw"); _want(norm_w, torch.float32, "norm_w")
    T = o_raw.shape[0]
    if not out.is_contiguous() or out.dtype != proj.dtype:
        raise KernelError("mlstm_out: out must be contiguous and of the projection's type")
    _run("mlstm_out", lib().bf_mlstm_out, _ptr(o_raw), _ptr(proj), _c_ll(proj.stride(0)),
         _c_ll(g_off), _ptr(norm_w), _ptr(out), _c_int(T), _c_int(heads), _c_int(dv),
         _c_float(eps), _c_int(_dtype_code(proj)), _stream())


# ------------------------------------------- windowed attention with pooled blocks
def apw_encode(proj: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
               inv_freq: Optional[torch.Tensor], v_inv_freq: Optional[torch.Tensor],
               interleaved: bool, positions: torch.Tensor, slots: Optional[torch.Tensor],
               q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], nh: int, nkv: int, dk: int, dv: int,
               eps: float, err: torch.Tensor) -> None:
    """Head norms and rotation of q and k, rotation of v over its whole head; q to
    ``q_out [T, nh dk]``, k and v into their pages at ``slots``.  Without caches only the
    queries are taken (``proj`` rows then need hold nothing else at their start)."""
    T = proj.shape[0]
    if proj.stride(1) != 1:
        raise KernelError("apw_encode: rows must be contiguous")
    writes = k_cache is not None
    if writes and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    page_size = k_cache.shape[2] if writes else 1
    num_slots = k_cache.shape[0] * page_size if writes else 0
    _run("apw_encode", lib().bf_apw_encode, _ptr(proj), _c_ll(proj.stride(0)), _ptr(q_w),
         _ptr(k_w), _ptr(inv_freq), _c_int(0 if inv_freq is None else inv_freq.numel()),
         _ptr(v_inv_freq), _c_int(1 if interleaved else 0), _ptr(positions),
         _ptr(slots if writes else None), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(T),
         _c_int(nh), _c_int(nkv if writes else 0), _c_int(dk), _c_int(dv), _c_int(page_size),
         _c_ll(num_slots), _c_float(eps), _c_int(_dtype_code(proj)), _ptr(err), _stream())


def apw_pool_blocks(k_cache: torch.Tensor, v_cache: torch.Tensor, ks_cache: torch.Tensor,
                    vs_cache: torch.Tensor, q_start: torch.Tensor, ctx_lens: torch.Tensor,
                    tables: torch.Tensor, s_tables: torch.Tensor, B: int, max_new_blocks: int,
                    nkv: int, dk: int, dv: int, pool: int, err: torch.Tensor) -> None:
    """Mean key and value of every block of ``pool`` tokens that this step completed, into
    the summary pages (entry ``block`` of the request's summary table)."""
    _run("apw_pool_blocks", lib().bf_apw_pool_blocks, _ptr(k_cache), _ptr(v_cache),
         _ptr(ks_cache), _ptr(vs_cache), _ptr(q_start), _ptr(ctx_lens), _ptr(tables),
         _c_int(tables.stride(0)), _ptr(s_tables), _c_int(s_tables.stride(0)), _c_int(B),
         _c_int(max_new_blocks), _c_int(nkv), _c_int(dk), _c_int(dv), _c_int(k_cache.shape[2]),
         _c_int(k_cache.shape[0]), _c_int(ks_cache.shape[2]), _c_int(ks_cache.shape[0]),
         _c_int(pool), _c_int(_dtype_code(k_cache)), _ptr(err), _stream())


def apw_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  ks_cache: Optional[torch.Tensor], vs_cache: Optional[torch.Tensor],
                  seq_of_token: torch.Tensor, positions: torch.Tensor, tables: torch.Tensor,
                  s_tables: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                  v_inv_freq: Optional[torch.Tensor], interleaved: bool, out: torch.Tensor,
                  nh: int, nkv: int, dk: int, dv: int, window: Optional[int], pool: int,
                  scale: float, sink: Optional[float], err: torch.Tensor) -> None:
    """Attention of every token row over the window's tokens and the pooled blocks behind
    it (one softmax, ``exp(sink)`` in its denominator if a sink is given), the head's output
    turned back by the row's position (``v_inv_freq``) and multiplied by the sigmoid of
    ``gate[t, h]`` (a strided view ``[T, nh]``).  Any sizes: values up to 256 a head."""
    T = q.shape[0]
    if not q.is_contiguous() or not out.is_contiguous():
        raise KernelError("apw_attention: q and out must be contiguous")
    if gate is not None and (gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("apw_attention: gate rows must be contiguous and of q's type")
    has_s = ks_cache is not None
    _run("apw_attention", lib().bf_apw_attention, _ptr(q), _ptr(k_cache), _ptr(v_cache),
         _ptr(ks_cache), _ptr(vs_cache), _ptr(seq_of_token), _ptr(positions), _ptr(tables),
         _c_int(tables.stride(0)), _ptr(s_tables), _c_int(s_tables.stride(0) if has_s else 0),
         _ptr(gate), _c_ll(gate.stride(0) if gate is not None else 0), _ptr(v_inv_freq),
         _c_int(1 if interleaved else 0), _ptr(out), _c_int(T), _c_int(nh), _c_int(nkv),
         _c_int(dk), _c_int(dv), _c_int(k_cache.shape[2]), _c_int(k_cache.shape[0]),
         _c_int(ks_cache.shape[2] if has_s else 1), _c_int(ks_cache.shape[0] if has_s else 0),
         _c_int(window or 0), _c_int(pool if has_s else 0), _c_float(scale),
         _c_int(0 if sink is None else 1), _c_float(sink or 0.0), _c_int(_dtype_code(q)),
         _ptr(err), _stream())


def pwm_attention_takes(dtype: torch.dtype, nh: int, nkv: int, dk: int, dv: int) -> bool:
    """Whether the tensor-core kernel of the pooled-window attention takes these sizes."""
    return (dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and dk <= 128
            and dv <= 128 and nh // nkv <= 64)      # (and a positive score scale)


def pwm_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  ks_cache: Optional[torch.Tensor], vs_cache: Optional[torch.Tensor],
                  q_start: torch.Tensor, positions: torch.Tensor, tables: torch.Tensor,
                  s_tables: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                  v_inv_freq: Optional[torch.Tensor], interleaved: bool, out: torch.Tensor,
                  B: int, max_tokens: int, nh: int, nkv: int, dk: int, dv: int,
                  window: Optional[int], pool: int, scale: float, sink: Optional[float],
                  err: torch.Tensor, max_ctx: int = 0, sinks: Optional[torch.Tensor] = None,
                  keep_first: int = 0, out_scale: float = 1.0, softcap: float = 0.0,
                  log_slope: Optional[torch.Tensor] = None,
                  log_rate: Optional[torch.Tensor] = None) -> None:
    """``apw_attention`` on the tensor cores (bfloat16; sizes: ``pwm_attention_takes``):
    request ``b`` of the batch owns the token rows ``q_start[b] .. q_start[b+1]-1``, at most
    ``max_tokens`` of them.  ``max_ctx``: the longest context in the batch, if the caller
    knows it: a step of single tokens then shares each row's key tiles out over several CTAs
    (four tiles of 64 keys each) whose partial results a second kernel makes one.
    ``sinks`` (float32 ``[nh]``): a learned logit per query head in the softmax's denominator
    instead of the constant ``sink``.  ``keep_first``: with a window, the request's first
    that many tokens stay visible behind it.  ``out`` may be a column block of a wider
    buffer; ``out_scale`` multiplies the result.  ``softcap`` c > 0: a scaled score z becomes
    ``c tanh(z / c)``.  ``log_slope`` and ``log_rate`` (float32 ``[nh]`` each, together or not
    at all; not with pooled blocks): ``log_slope_h ln(1 + log_rate_h (p - j))`` is taken off
    the scaled score of the query at p and the key at j."""
    if (log_slope is None) != (log_rate is None) or (log_slope is not None
                                                     and ks_cache is not None):
        raise KernelError("pwm_attention: log_slope and log_rate go together, without pooled "
                          "blocks")
    for name, t in (("log_slope", log_slope), ("log_rate", log_rate)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != nh:
                raise KernelError(f"pwm_attention: {name} must have one entry per query head")
    if not pwm_attention_takes(q.dtype, nh, nkv, dk, dv):
        raise KernelError("pwm_attention: bfloat16, head sizes multiples of 16 up to 128")
    if not q.is_contiguous() or out.stride(1) != 1 or q.data_ptr() % 16:
        raise KernelError("pwm_attention: q must be contiguous and 16-byte aligned, rows of out "
                          "contiguous")
    if sinks is not None:
        _want(sinks, torch.float32, "sinks")
        if sinks.numel() != nh:
            raise KernelError("pwm_attention: sinks must have one entry per query head")
    keep_first = int(keep_first) if window else 0
    if gate is not None and (gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("pwm_attention: gate rows must be contiguous and of q's type")
    has_s = ks_cache is not None
    part_o = part_ml = None
    shares = 0
    if max_ctx > 0 and max_tokens * (nh // nkv) <= 16:
        span = (min(window, max_ctx) if window else max_ctx) + 16     # (+ the step's own tokens)
        tiles = (span + 63) // 64 + 1
        if has_s and window and pool:
            tiles += (max(0, max_ctx - window) // pool + 63) // 64
        tiles += (keep_first + 63) // 64
        shares = (tiles + 3) // 4
        if 1 < shares <= 32:
            part_o = torch.empty((B, nkv, shares, 16, dv), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((B, nkv, shares, 16, 2), dtype=torch.float32, device=q.device)
        else:
            shares = 0
    _run("pwm_attention", lib().bf_pwm_attention, _ptr(q), _ptr(k_cache), _ptr(v_cache),
         _ptr(ks_cache), _ptr(vs_cache), _ptr(q_start), _ptr(positions), _ptr(tables),
         _c_int(tables.stride(0)), _ptr(s_tables), _c_int(s_tables.stride(0) if has_s else 0),
         _ptr(gate), _c_ll(gate.stride(0) if gate is not None else 0), _ptr(v_inv_freq),
         _c_int(1 if interleaved else 0), _ptr(out), _c_int(B), _c_int(max_tokens), _c_int(nh),
         _c_int(nkv), _c_int(dk), _c_int(dv), _c_int(k_cache.shape[2]), _c_int(k_cache.shape[0]),
         _c_int(ks_cache.shape[2] if has_s else 1), _c_int(ks_cache.shape[0] if has_s else 0),
         _c_int(window or 0), _c_int(pool if has_s else 0), _c_float(scale),
         _c_int(0 if sink is None and sinks is None else 1), _c_float(sink or 0.0),
         _ptr(part_o), _ptr(part_ml), _c_int(shares), _ptr(err), _ptr(sinks), _c_int(keep_first),
         _c_ll(q.stride(0)), _c_ll(out.stride(0)), _c_float(out_scale), _c_float(softcap),
         _ptr(log_slope), _ptr(log_rate), _stream())


def latent_attention_takes(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """Whether the tensor-core kernel of the attention over a cached latent takes these
    sizes."""
    return (dtype == torch.bfloat16 and rank % 16 == 0 and rot % 16 == 0 and 0 < rank <= 512
            and rank + rot <= 640)


LATENT_ROWS, LATENT_KEYS = 32, 64


def latent_attention(q: torch.Tensor, cache: torch.Tensor, q_start: torch.Tensor,
                     positions: torch.Tensor, tables: torch.Tensor, out: torch.Tensor, B: int,
                     max_tokens: int, H: int, rank: int, scale: float, err: torch.Tensor,
                     max_ctx: int = 0) -> None:
    """Causal softmax attention of query rows ``q [T, H, W]`` (already in the latent's
    coordinates) over a cache of one row ``[latent (rank) | shared key part]`` of ``W`` numbers
    per token, whose first ``rank`` numbers are also the value: ``out [T, H, rank]``, on the
    tensor cores (bfloat16; sizes: ``latent_attention_takes``).  Request ``b`` owns the token
    rows ``q_start[b] .. q_start[b+1]-1``, at most ``max_tokens`` of them.  ``max_ctx``: the
    longest context in the batch, if the caller knows it: a step with few rows then shares
    each request's key tiles out over several CTAs whose partial results a second kernel
    makes one."""
    W = q.shape[-1]
    if not latent_attention_takes(q.dtype, rank, W - rank):
        raise KernelError("latent_attention: bfloat16, a latent of a multiple of 16 up to 512, "
                          "with the shared part at most 640")
    if not q.is_contiguous() or not out.is_contiguous() or cache.shape[1] != 1 or cache.shape[3] != W:
        raise KernelError("latent_attention: q and out must be contiguous, the cache one head "
                          "of q's width per token")
    max_rows = max_tokens * H
    tiles = (max_rows + LATENT_ROWS - 1) // LATENT_ROWS
    part_o = part_ml = None
    splits = 1
    if max_ctx > 0:
        key_tiles = (max_ctx + LATENT_KEYS - 1) // LATENT_KEYS
        room = num_sms(q.device) // max(1, tiles * B)
        splits = max(1, min(room, (key_tiles + 1) // 2, 32))
        if splits > 1:
            part_o = torch.empty((B, tiles, splits, LATENT_ROWS, rank), dtype=torch.float32,
                                 device=q.device)
            part_ml = torch.empty((B, tiles, splits, LATENT_ROWS, 2), dtype=torch.float32,
                                  device=q.device)
    _run("latent_attention", lib().bf_latent_attention, _ptr(q), _ptr(cache), _ptr(q_start),
         _ptr(positions), _ptr(tables), _c_int(tables.stride(0)), _ptr(out), _c_int(B),
         _c_int(max_rows), _c_int(H), _c_int(W), _c_int(rank), _c_int(cache.shape[2]),
         _c_int(cache.shape[0]), _c_float(scale), _ptr(part_o), _ptr(part_ml), _c_int(splits),
         _ptr(err), _stream())


# ------------------------------------------------------------- matrix products
def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic."""
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or t.stride(-1) != 1:
            raise KernelError(f"sgemm_nt: {n} must be float32 with contiguous rows")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"sgemm_nt: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> "
                          f"{tuple(out.shape)} do not agree")
    _run("sgemm_nt", lib().bf_sgemm_nt, _ptr(a), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K),
                             _c_ll(a.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
                             _stream())


def sgemm_nt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, b] = a[:, b] @ w[b]^T for every b, in true 32-bit arithmetic: ``a [M, B, K]`` and
    ``out [M, B, N]`` may be strided views (innermost stride 1), ``w [B, N, K]``."""
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or t.stride(-1) != 1 or t.dim() != 3:
            raise KernelError(f"sgemm_nt_batched: {n} must be a float32 [.., .., ..] with contiguous rows")
    M, Bn, K = a.shape
    N = w.shape[1]
    if w.shape != (Bn, N, K) or out.shape != (M, Bn, N):
        raise KernelError("sgemm_nt_batched: shapes do not agree")
    _run("sgemm_nt_batched", lib().bf_sgemm_nt_batched, _ptr(a), _ptr(w), _ptr(out), _c_int(M),
         _c_int(N), _c_int(K), _c_ll(a.stride(0)), _c_ll(w.stride(1)), _c_ll(out.stride(0)),
         _c_int(Bn), _c_ll(a.stride(1)), _c_ll(w.stride(0)), _c_ll(out.stride(1)), _stream())


_num_sms = {}
_err_words = {}


def error_word(device: torch.device) -> torch.Tensor:
    """The device's int32 error word, which kernels OR bits into instead of faulting."""
    w = _err_words.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _err_words[device.index] = w
    return w


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
              bn: int = 0) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float
    accumulate, bfloat16 or float32 out).  ``bn``: feature rows per tile (0: chosen by the
    library).  Returns False, having done nothing, for shapes the kernel does not take
    (K not a multiple of 8, misaligned rows)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16: operands must be bfloat16")
    M, K = x.shape
    N = w.shape[0]
    if (K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8
            or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1):
        return False
    sms = _num_sms.get(x.device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        _num_sms[x.device.index] = sms
    _run("gemm_bf16_tcgen05", lib().bf_gemm_bf16_tcgen05, _ptr(x), _ptr(w), _ptr(out),
         _c_int(M), _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)),
         _c_ll(out.stride(0)), _c_int(_dtype_code(out)), _c_int(bn), _c_int(sms), _ptr(err),
         _stream())
    return True


def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
                   bn: int = 0, gated: bool = False, accumulate: bool = False) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T on pairs of SMs (``tcgen05.mma.cta_group::2``, tiles of
    256 token rows): the product for many token rows.  ``gated``: ``w`` is the stacked
    ``[2 N, K]`` gate/up weight and ``out[M, N] = silu(x w_gate^T) * (x w_up^T)``, bfloat16
    only.  ``accumulate``: ``out`` (float32) ``+=`` the product.  ``bn``: accumulator columns
    per tile (0: chosen by the library).  Returns False, having done nothing, for shapes the
    kernel does not take."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16_pair: operands must be bfloat16")
    if accumulate and (gated or out.dtype != torch.float32):
        raise KernelError("gemm_bf16_pair: accumulate needs a float32 output and no gate")
    M, K = x.shape
    N = out.shape[1]
    if (K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8
            or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1
            or out.shape[0] != M or w.shape[0] != (2 * N if gated else N) or w.shape[1] != K
            or (gated and out.dtype != torch.bfloat16)
            or out.dtype not in (torch.bfloat16, torch.float32)):
        return False
    _run("gemm_bf16_pair", lib().bf_gemm_bf16_pair, _ptr(x), _ptr(w), _ptr(out), _c_int(M),
         _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
         _c_int(_dtype_code(out)), _c_int(1 if gated else 0), _c_int(1 if accumulate else 0),
         _c_int(bn), _c_int(num_sms(x.device)), _ptr(err), _stream())
    return True


def gemm_cluster_plan(features: int, K: int, device: torch.device):
    """(bn, cluster) for the split-K cluster product, or None when it does not apply."""
    sms = _num_sms.get(device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device.index] = sms
    bn, c = _c_int(0), _c_int(0)
    n = lib().bf_gemm_cluster_plan(_c_int(features), _c_int(K), _c_int(sms), ctypes.byref(bn),
                                   ctypes.byref(c))
    return (bn.value, c.value) if n > 0 else None


CLUSTER_MAX_TOKENS = 64


def gemm_bf16_cluster(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
                      bn: int, cluster: int) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 with the K range split over clusters of
    ``cluster`` CTAs (partials combined through distributed shared memory).  Returns False,
    having done nothing, for shapes the kernel does not take."""
    M, K = x.shape
    N = w.shape[0]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1):
        return False
    _run("gemm_bf16_cluster", lib().bf_gemm_bf16_cluster, _ptr(x), _ptr(w), _ptr(out), _c_int(M),
         _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
         _c_int(_dtype_code(out)), _c_int(bn), _c_int(cluster), _ptr(err), _stream())
    return True


def gemm_bf16_cluster_add_norm(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor,
                               norm_w: torch.Tensor, eps: float, err: torch.Tensor, bn: int,
                               cluster: int):
    """``resid += x @ w^T`` (float32 stream ``[M, N]``), and the next norm's output short of its
    row factor: returns ``(xt, RowScale)`` with ``xt = bfloat16(resid * norm_w)``, or None,
    having done nothing, for shapes the kernel does not take (M <= 64, see
    ``gemm_bf16_cluster``)."""
    M, K = x.shape
    N = w.shape[0]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16
            or resid.dtype != torch.float32 or resid.shape != (M, N) or resid.stride(1) != 1
            or norm_w.dtype != torch.float32 or norm_w.numel() != N or not norm_w.is_contiguous()):
        return None
    count = -(-N // bn) * cluster
    xt = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    partials = torch.empty((M, count), dtype=torch.float32, device=x.device)
    n = _c_int(0)
    _run("gemm_bf16_cluster_add_norm", lib().bf_gemm_bf16_cluster_add_norm, _ptr(x), _ptr(w),
         _c_int(M), _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_int(bn),
         _c_int(cluster), _ptr(resid), _c_ll(resid.stride(0)), _ptr(norm_w), _ptr(xt),
         _c_ll(xt.stride(0)), _ptr(partials), ctypes.byref(n), _ptr(err), _stream())
    if n.value != count:
        raise KernelError("gemm_bf16_cluster_add_norm: the kernel counts its CTAs differently")
    return xt, RowScale(partials, N, eps)


def num_sms(device: torch.device) -> int:
    sms = _num_sms.get(device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device.index] = sms
    return sms


def gemm_cluster_qkv_plan(features: int, K: int, d: int, device: torch.device,
                          min_fill: float = 0.6):
    """(bn, cluster, CTAs) for the q/k/v projection with the head norms, the rotation and the
    store into the pages in its epilogue: the narrowest tile of whole heads whose clusters,
    all resident at once, occupy ``min_fill`` of the SMs (or, if none does, the arrangement
    with the most CTAs), or None where the kernel has no such arrangement."""
    bn, c = _c_int(0), _c_int(0)
    sms = num_sms(device)
    n = lib().bf_gemm_cluster_qkv_plan(_c_int(features), _c_int(K), _c_int(d), _c_int(sms),
                                       _c_int(max(1, int(min_fill * sms))), ctypes.byref(bn),
                                       ctypes.byref(c))
    return (bn.value, c.value, n) if n > 0 else None


def gemm_bf16_cluster_qkv(x: torch.Tensor, w: torch.Tensor, q_w: Optional[torch.Tensor],
                          k_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                          positions: torch.Tensor, slots: Optional[torch.Tensor],
                          q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int, eps: float,
                          err: torch.Tensor, bn: int, cluster: int,
                          row_scale: Optional[RowScale] = None) -> bool:
    """``qk_norm_rope_kv_write(x @ w^T, ...)`` as one kernel for at most 64 token rows:
    ``w`` is ``[(nh + 2 nkv) d, K]``, or ``[nh d, K]`` with no caches given (queries only).
    Returns False, having done nothing, for what the kernel does not take."""
    M, K = x.shape
    writes = k_cache is not None
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or d % 32 or d > 256
            or rot_half % 32 or 2 * rot_half > d or not q_out.is_contiguous()
            or w.shape[0] != (nh + (2 * nkv if writes else 0)) * d):
        return False
    if writes and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    page_size = k_cache.shape[2] if writes else 1
    num_slots = k_cache.shape[0] * page_size if writes else 0
    _run("gemm_bf16_cluster_qkv", lib().bf_gemm_bf16_cluster_qkv, _ptr(x), _ptr(w), _c_int(M),
         _c_int(w.shape[0]), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_int(bn),
         _c_int(cluster), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _c_int(rot_half), _ptr(positions),
         _ptr(slots if writes else None), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(nh),
         _c_int(nkv if writes else 0), _c_int(d), _c_int(page_size), _c_ll(num_slots),
         _c_float(eps), *_row_scale_args(row_scale, M), _ptr(err), _stream())
    return True


def gemm_swiglu_plan(inter: int, K: int, device: torch.device):
    """(bn, CTAs) for ``gemm_bf16_swiglu``, or None where its tiles would not fit one wave."""
    bn = _c_int(0)
    n = lib().bf_gemm_swiglu_plan(_c_int(inter), _c_int(K), _c_int(num_sms(device)),
                                  ctypes.byref(bn))
    return (bn.value, n) if n > 0 else None


def gemm_bf16_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor,
                     err: torch.Tensor, bn: int, row_scale: Optional[RowScale] = None) -> bool:
    """``silu_mul(x @ w_gate_up^T)`` as one kernel for at most 64 token rows: ``w_gate_up`` is
    ``[2 I, K]`` with the gate rows first, ``out`` is ``[M, I]``.  Returns False, having done
    nothing, for what the kernel does not take."""
    M, K = x.shape
    I = out.shape[1]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w_gate_up.stride(1) != 1
            or x.stride(0) % 8 or w_gate_up.stride(0) % 8 or x.data_ptr() % 16
            or w_gate_up.data_ptr() % 16 or out.stride(1) != 1 or out.stride(0) % 8
            or out.data_ptr() % 16 or w_gate_up.shape[0] != 2 * I or out.shape[0] != M
            or out.dtype != torch.bfloat16):
        return False
    _run("gemm_bf16_swiglu", lib().bf_gemm_bf16_swiglu, _ptr(x), _ptr(w_gate_up), _c_int(M),
         _c_int(I), _c_int(K), _c_ll(x.stride(0)), _c_ll(w_gate_up.stride(0)), _c_int(bn),
         _ptr(out), _c_ll(out.stride(0)), *_row_scale_args(row_scale, M), _ptr(err), _stream())
    return True


# -------------------------------------------------------------------- sampling
def repetition_penalty(logits: torch.Tensor, items: torch.Tensor, penalty: torch.Tensor) -> None:
    """items: int32 [n, 3] of (row, token, count)."""
    _want(logits, torch.float32, "logits"); _want(items, torch.int32, "items")
    _run("repetition_penalty", lib().bf_repetition_penalty, _ptr(logits), _c_int(logits.shape[1]), _ptr(items),
                                       _c_int(items.shape[0]), _ptr(penalty), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    _want(logits, torch.float32, "logits"); _want(temperature, torch.float32, "temperature")
    _want(top_k, torch.int32, "top_k"); _want(top_p, torch.float32, "top_p")
    _want(uniform, torch.float32, "uniform"); _want(out, torch.int32, "out")
    R, V = logits.shape
    _run("sample", lib().bf_sample, _ptr(logits), _c_int(R), _c_int(V), _ptr(temperature), _ptr(top_k),
                           _ptr(top_p), _ptr(uniform), _ptr(out), _stream())
