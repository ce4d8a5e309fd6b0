"""Python face of the CUDA kernels: checks on the host, then one C call.

Every function here validates what the kernel cannot (device, dtype, layout,
size limits) and raises a clear error instead of launching; the launchers
return an error code for what they refuse themselves.  There is no CPU path
and no library stand-in: a tensor that is not on a CUDA device is an error.

Matrix products are the exception the engine shares with the reference, which
also leaves them to a library (`F.linear`, python/logssms/layers/linear.py:26):
bfloat16 products go to cuBLAS through torch, float32 products to the engine's
own FFMA kernel so that no reduced-precision matrix mode can take part.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build
from .fusion import NormedRows, ResidualJoin, ScaledRows, SummedRows      # the fusion protocol (re-exported here)
from .profiler import PROFILER

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {-1: "dtype is neither float32 nor bfloat16", -2: "a size the kernel does not take",
           -3: "a size beyond the kernel's limit"}
_fn_cache: dict[tuple[str, str], ctypes._CFuncPtr] = {}
launch_count = 0        # kernels of this package launched so far (a launcher adds what it launches)


class KernelError(RuntimeError):
    pass


def _fn(lib: str, name: str, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(build.load(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    if PROFILER.enabled:                  # opt-in: every launch between two events, summed per kernel class
        return lambda *args: PROFILER.timed(lib, name, lambda: f(*args))
    return f


def _check(code: int, name: str, detail: str = "", launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code < 0:
        raise KernelError(f"{name} refused the call: {_ERRORS.get(code, code)} {detail}")
    raise KernelError(f"{name}: CUDA error {code} at launch {detail}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """Raw handle of torch's current stream on the current device (the C call: the Python `Stream` object
    costs microseconds, and every launch asks)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}: the kernels take float32 and bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("logssms_b200 kernels run on CUDA tensors only; there is no CPU path")


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- embedding
def embed_gather(table: torch.Tensor, ids: torch.Tensor, multiplier: float,
                 bad_ids: torch.Tensor | None = None) -> torch.Tensor:
    _cuda(table, ids)
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous [vocab, hidden] matrix")
    V, H = table.shape
    out = torch.empty((ids.numel(), H), dtype=table.dtype, device=table.device)
    f = _fn("embed", "lb_embed_gather", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                                         c_int, c_void_p])
    _check(f(_ptr(out), _ptr(table), _ptr(ids), ids.numel(), H, V, multiplier, _ptr(bad_ids), _code(table),
             _stream()), "embed_gather")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _cuda(src, rows)
    _i32(rows, "rows")
    _need(src.dim() == 2 and src.is_contiguous(), "gather_rows wants a contiguous matrix")
    out = torch.empty((rows.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
    f = _fn("embed", "lb_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(src), _ptr(rows), rows.numel(), src.shape[1], _code(src), _stream()), "gather_rows")
    return out


# --------------------------------------------------------------------------- norms
def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None, *,
                other: torch.Tensor | None = None, in_scales=(1.0, 1.0), out_scales=(1.0,),
                want_residual: bool = True, residual_out: torch.Tensor | None = None, in_place: bool = True):
    """(outputs, new_residual): residual add + RMSNorm with one or two scaled outputs.
    The new residual is written in place of `residual` when one is given, unless `in_place` is off
    (then into `residual_out`, or a new tensor)."""
    _cuda(x, weight, residual, other)
    _need(x.dim() == 2 and x.is_contiguous(), "add_rmsnorm wants a contiguous [rows, width] input")
    rows, H = x.shape
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(),
          "norm weight must be a contiguous float32 vector of the row width")
    for t, name in ((residual, "residual"), (other, "other")):
        if t is not None:
            _need(t.shape == x.shape and t.dtype == x.dtype and t.is_contiguous(), f"{name} must match the input")
    _need(1 <= len(out_scales) <= 2, "one or two outputs")
    out0 = torch.empty_like(x)
    out1 = torch.empty_like(x) if len(out_scales) == 2 else None
    if in_place:
        res_out = residual if residual is not None else (torch.empty_like(x) if want_residual else None)
    else:
        res_out = (residual_out if residual_out is not None else torch.empty_like(x)) if want_residual else None
    f = _fn("norm", "lb_add_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(other), _ptr(residual), _ptr(res_out), _ptr(weight), _ptr(out0), _ptr(out1), rows, H,
             eps, in_scales[0], in_scales[1], out_scales[0], out_scales[-1], _code(x), _stream()),
           "add_rmsnorm", f"(width {H})")
    return ((out0,) if out1 is None else (out0, out1)), res_out


GATE_ONLY, NORM_BEFORE_GATE, NORM_AFTER_GATE = 0, 1, 2


def gated_rmsnorm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, eps: float, groups: int,
                  gate_scale: float, mode: int) -> torch.Tensor:
    """Grouped RMSNorm with SiLU gate (`mode` NORM_BEFORE_GATE / NORM_AFTER_GATE) or the bare
    y * silu(gate) product (`GATE_ONLY`).  `gate` may be a column view of a wider matrix."""
    _cuda(y, gate, weight)
    _need(y.dim() == 2 and y.is_contiguous(), "gated_rmsnorm wants a contiguous [rows, width] input")
    rows, width = y.shape
    _need(gate.shape == y.shape and gate.dtype == y.dtype and gate.stride(1) == 1, "gate must match y, unit column stride")
    _need(width % groups == 0, "width must be a multiple of groups")
    if mode != GATE_ONLY:
        _need(weight is not None and weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(),
              "gated norm weight must be a contiguous float32 vector of the row width")
    out = torch.empty_like(y)
    f = _fn("norm", "lb_gated_rmsnorm", [c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_float, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), rows, width // groups, groups, eps,
             gate_scale, mode, _code(y), _stream()), "gated_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, act_scale: float) -> torch.Tensor:
    _cuda(gate_up)
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0,
          "swiglu wants a contiguous [rows, 2*I] matrix")
    rows, two_i = gate_up.shape
    out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("norm", "lb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), rows, two_i // 2, act_scale, _code(gate_up), _stream()), "swiglu")
    return out


def scale(x: torch.Tensor, s: float, to_f32: bool = False) -> torch.Tensor:
    """round(x * s) in x's dtype, or float32(x) * s with `to_f32`."""
    _cuda(x)
    _need(x.is_contiguous(), "scale wants a contiguous tensor")
    out = torch.empty(x.shape, dtype=torch.float32 if to_f32 else x.dtype, device=x.device)
    f = _fn("norm", "lb_scale", [c_void_p, c_void_p, c_long, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(out), x.numel(), s, int(to_f32), _code(x), _stream()), "scale")
    return out


# --------------------------------------------------------------------------- rotary + cache store
def rope_table(inv_freq: torch.Tensor, rows: int, magnitude: float = 1.0) -> torch.Tensor:
    """[rows, 2*half] float32: cos | sin of position * inv_freq, both times `magnitude`."""
    _cuda(inv_freq)
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be contiguous float32")
    half = inv_freq.numel()
    table = torch.empty((rows, 2 * half), dtype=torch.float32, device=inv_freq.device)
    f = _fn("rope", "lb_rope_table", [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(table), _ptr(inv_freq), rows, half, magnitude, _stream()), "rope_table")
    return table


def rope_kv_store(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                  slot_mapping: torch.Tensor, cos_sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  key_scale: float, write_kv: bool = True) -> torch.Tensor:
    """qkv: [tokens, (Hq + 2*Hkv) * head_dim], columns q | k | v (row stride free).  Returns the rotated
    queries [tokens, Hq, head_dim]; stores scaled+rotated keys and the values at `slot_mapping` (token
    index in the page pool) unless `write_kv` is off."""
    _cuda(qkv, positions, slot_mapping, cos_sin, k_cache, v_cache)
    Hq, Hkv, hd = num_heads, num_kv_heads, head_dim
    tokens = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.shape[1] == (Hq + 2 * Hkv) * hd and qkv.stride(1) == 1,
          "qkv must be [tokens, (Hq + 2*Hkv) * head_dim] with unit column stride")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    _need(positions.numel() == tokens and slot_mapping.numel() == tokens, "one position and one slot per token")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 2,
          "cos/sin table must be contiguous float32 [positions, rotary_dim]")
    rotary_dim = cos_sin.shape[1]
    _need(rotary_dim % 2 == 0 and rotary_dim <= hd, f"rotary_dim {rotary_dim} must be even and within head_dim {hd}")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == qkv.dtype == v_cache.dtype
          and k_cache.shape[-2:] == (Hkv, hd) and v_cache.shape == k_cache.shape,
          "k/v cache must be contiguous [..., kv_heads, head_dim] of the activation dtype")
    q_out = torch.empty((tokens, Hq, hd), dtype=qkv.dtype, device=qkv.device)
    row_stride = qkv.stride(0) if tokens > 1 else qkv.shape[1]
    base = qkv.data_ptr()
    item = qkv.element_size()
    f = _fn("rope", "lb_rope_kv_store", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                         c_int, c_int, c_void_p])
    _check(f(base, base + Hq * hd * item, base + (Hq + Hkv) * hd * item, row_stride, _ptr(positions),
             _ptr(slot_mapping), _ptr(cos_sin), cos_sin.shape[0], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), tokens,
             Hq, Hkv, hd, rotary_dim, key_scale, int(write_kv), _code(qkv), _stream()), "rope_kv_store")
    return q_out


# --------------------------------------------------------------------------- attention
def attention_splits(num_tokens: int, num_heads: int, num_kv_heads: int, max_context: int) -> int:
    """How many ranges each context is cut into so that the grid covers the SMs a few times over."""
    G = num_heads // num_kv_heads
    tile = 8 if G >= 8 else (4 if G > 2 else G)
    items = max(1, num_tokens * num_kv_heads * (-(-G // tile)))
    return max(1, min(_SPLIT_TARGET_CTAS // items, -(-max_context // 64), 256))


_SPLIT_TARGET_CTAS = 592        # 4 CTAs on each of the 148 SMs


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     token_req: torch.Tensor, positions: torch.Tensor, scale: float, window: int = 0, *,
                     splits: int = 1, token_list: torch.Tensor | None = None, out: torch.Tensor | None = None,
                     scratch: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """Split-KV attention, each token on its own over its request's pages.  q: [tokens, Hq, hd]; caches:
    [pages, page_size, Hkv, hd]; block_table: [requests, max_pages] int32; token_req / positions: per token its
    request row and absolute position.  Returns [tokens, Hq, hd].  `token_list` (int32) restricts the call to those tokens; the other rows of `out`
    are left as they are.  `scratch`: float32 buffers (>= tokens*Hq*splits*hd and >= tokens*Hq*splits*2
    elements) for the ranges' partial results; allocated here when missing."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, token_list)
    tokens, Hq, hd = q.shape
    _need(q.is_contiguous(), "q must be contiguous")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == q.dtype == v_cache.dtype and k_cache.shape[3] == hd,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(token_req, "token_req")
    _i32(positions, "positions")
    sel = tokens
    if token_list is not None:
        _i32(token_list, "token_list")
        sel = token_list.numel()
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    part_o = part_ml = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(sel * Hq * splits * hd, dtype=torch.float32, device=q.device),
                       torch.empty(sel * Hq * splits * 2, dtype=torch.float32, device=q.device))
        part_o, part_ml = scratch
        _need(part_o.dtype == torch.float32 == part_ml.dtype and part_o.numel() >= sel * Hq * splits * hd
              and part_ml.numel() >= sel * Hq * splits * 2, "attention scratch is too small or not float32")
    f = _fn("attention_decode", "lb_attention_decode",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(token_req), _ptr(positions), _ptr(token_list), sel, Hq, Hkv, hd, page_size, scale, int(window or 0),
             int(splits), _ptr(part_o), _ptr(part_ml), _code(q), _stream()), "attention_decode",
           launches=2 if splits > 1 else 1)
    return out


_decode_counters: dict[torch.device, torch.Tensor] = {}


def _counters_for(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed int32 counters kept per device; the fused decode kernel leaves them at zero."""
    t = _decode_counters.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _decode_counters[device] = t
    return t


def decode_step_splits(num_tokens: int, num_heads: int, num_kv_heads: int, max_context: int, listed: bool = False,
                       head_dim: int = 64) -> int:
    """Most key ranges per token for `attention_decode_step` (about one CTA per SM with heads of up to 64, about two
    with larger ones) or, `listed`, for `attention_decode_listed` (about two), never more ranges than 256-key pieces of
    the longest context (the kernel itself uses fewer ranges for a short context)."""
    G = num_heads // num_kv_heads
    tile = 8 if G >= 8 else (4 if G > 2 else G)
    items = max(1, num_tokens * num_kv_heads * (-(-G // tile)))
    target = _WIDE_TARGET_CTAS if (listed or head_dim > 64) else _STEP_TARGET_CTAS
    splits = max(1, min(target // items, -(-max_context // 256), 256))
    # up to 8 ranges are the CTAs of one cluster and merge through distributed shared memory (about 2 us off the
    # kernel); with a dozen (token, head) items that many ranges fill the GPU, so more would only cost that path
    return min(splits, 8) if items >= 12 else splits


# Heads of up to 64: about one CTA per SM.  Up to 9 tokens the 256-key pieces of the context set the number of ranges,
# not this; from 10 tokens on fewer, longer ranges win, the more so beside the state update that shares the SMs:
# 36-layer decode steps over 2,048-key contexts (head 64) with 296 / 160 took 1.66 / 1.62 ms at batch 16, 1.92 / 1.90 ms
# at 32, 2.56 / 2.39 ms at 64 (444: 2.68 ms).
_STEP_TARGET_CTAS = 160
# Heads of 128 (a CTA's chain per key is twice as long), and the listed rows of a step that also holds a prompt portion
# (the last link of the attention branch, with little beside them): shorter ranges win.  16 layers of 1.5B-Deep size
# (head 128) with 296 / 160: 1.38 / 1.42 ms at batch 24, 1.52 / 1.62 ms at 32; the 1.5B-Deep serving run 2,220 / 1,970
# generated tok/s; 64 tokens of 4,096 keys at 7B size (one range either way): no difference.
_WIDE_TARGET_CTAS = 296


def attention_decode_step(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                          slot_mapping: torch.Tensor, cos_sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, token_req: torch.Tensor, scale: float, key_scale: float,
                          window: int = 0, write_kv: bool = True, *, splits: int = 1) -> torch.Tensor:
    """The whole attention of a decode step in one launch: every row of `qkv` ([tokens, (Hq + 2 Hkv) * hd],
    columns q | k | v) is the only new token of its request.  Rotates q and the new key, stores the new
    key/value at `slot_mapping` (unless `write_kv` is off: then the position was stored by another layer
    and is read from the cache), attends over the request's pages and merges the key ranges.
    Returns [tokens, Hq, hd]."""
    _cuda(qkv, positions, slot_mapping, cos_sin, k_cache, v_cache, block_table, token_req)
    Hq, Hkv, hd = num_heads, num_kv_heads, head_dim
    tokens = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.shape[1] == (Hq + 2 * Hkv) * hd and qkv.stride(1) == 1,
          "qkv must be [tokens, (Hq + 2*Hkv) * head_dim] with unit column stride")
    for t_, n_ in ((positions, "positions"), (slot_mapping, "slot_mapping"), (token_req, "token_req")):
        _i32(t_, n_)
        _need(t_.numel() == tokens, f"one entry of {n_} per token")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 2,
          "cos/sin table must be contiguous float32 [positions, rotary_dim]")
    rotary_dim = cos_sin.shape[1]
    _need(rotary_dim % 2 == 0 and rotary_dim <= hd, f"rotary_dim {rotary_dim} must be even and within head_dim {hd}")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == qkv.dtype == v_cache.dtype and k_cache.shape[2:] == (Hkv, hd),
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of the activation dtype")
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    page_size = k_cache.shape[1]
    out = torch.empty((tokens, Hq, hd), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = counters = None
    splits = int(splits)
    if splits > 1:
        part_o = torch.empty(tokens * Hq * splits * hd, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(tokens * Hq * splits * 2, dtype=torch.float32, device=qkv.device)
        counters = _counters_for(qkv.device, tokens * Hq)
    row_stride = qkv.stride(0) if tokens > 1 else qkv.shape[1]
    f = _fn("attention_decode_fused", "lb_attention_decode_fused",
            [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_long, c_void_p, c_int, c_void_p])
    _check(f(_ptr(qkv), row_stride, _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(token_req), _ptr(positions), _ptr(slot_mapping), _ptr(cos_sin), cos_sin.shape[0], rotary_dim, tokens,
             Hq, Hkv, hd, page_size, scale, key_scale, int(window or 0), int(write_kv), splits, _ptr(part_o),
             _ptr(part_ml), _ptr(counters), k_cache.shape[0], _ptr(error_word(qkv.device)), _code(qkv), _stream()),
           "attention_decode_step")
    return out


def attention_decode_listed_ok(q: torch.Tensor, k_cache: torch.Tensor) -> bool:
    """Does `attention_decode_listed` take these operands (bfloat16, head size up to 128, at most 16 query heads per
    key/value head)?  Else `attention_decode`."""
    return (q.dtype == torch.bfloat16 and q.dim() == 3 and k_cache.dim() == 4 and q.shape[2] <= 128 and q.shape[2] % 16 == 0
            and q.shape[1] % k_cache.shape[2] == 0 and q.shape[1] // k_cache.shape[2] <= 16 and q.is_contiguous())


def attention_decode_listed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            token_req: torch.Tensor, positions: torch.Tensor, token_list: torch.Tensor, count: int,
                            scale: float, window: int = 0, *, splits: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """The decode-step attention kernel (tensor-core form: the query heads of a key/value head as one tile, key ranges
    merged through the cluster's shared memory) for `count` listed rows of a step that holds prompt portions as well.
    q [rows, Hq, hd]: rotated queries; every key and value, the rows' own included, is in the cache already.  Rows of
    `out` that are not listed are left as they are."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, token_list, out)
    _need(attention_decode_listed_ok(q, k_cache), "attention_decode_listed takes bfloat16, head sizes up to 128, groups up to 16")
    rows, Hq, hd = q.shape
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape and k_cache.dtype == q.dtype
          == v_cache.dtype and k_cache.shape[3] == hd, "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    for t_, n_ in ((token_req, "token_req"), (positions, "positions"), (token_list, "token_list")):
        _i32(t_, n_)
    _need(token_list.numel() >= count and token_req.numel() == rows == positions.numel(), "one entry per row; a list of `count` rows")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    part_o = part_ml = counters = None
    splits = int(splits)
    if splits > 1:
        part_o = torch.empty(count * Hq * splits * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(count * Hq * splits * 2, dtype=torch.float32, device=q.device)
        counters = _counters_for(q.device, count * Hq)
    f = _fn("attention_decode_fused", "lb_attention_decode_listed",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0), _ptr(token_req),
             _ptr(positions), _ptr(token_list), count, Hq, Hkv, hd, page_size, scale, int(window or 0), splits, _ptr(part_o),
             _ptr(part_ml), _ptr(counters), k_cache.shape[0], _ptr(error_word(q.device)), _stream()), "attention_decode_listed")
    return out


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, start_pos: torch.Tensor, tiles: torch.Tensor, num_tiles: int,
                      scale: float, window: int = 0, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention for prompt portions (bfloat16).  `tiles`: int32 [n, 2] = (request index,
    first token of a 64-token tile within that request's portion).  Rows of `out` that no tile covers
    are left as they are.  Other arguments as for `attention_decode`."""
    _cuda(q, k_cache, v_cache, block_table, cu_seqlens, start_pos, tiles)
    tokens, Hq, hd = q.shape
    _need(q.dtype == torch.bfloat16, "attention_prefill is the bfloat16 kernel; float32 runs the general kernel")
    _need(q.is_contiguous(), "q must be contiguous")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == q.dtype == v_cache.dtype and k_cache.shape[3] == hd,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(start_pos, "start_pos")
    _i32(tiles, "tiles")
    _need(tiles.numel() >= 2 * num_tiles, "tiles holds fewer pairs than num_tiles")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    f = _fn("attention_prefill", "lb_attention_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(tiles), num_tiles, Hq, Hkv, hd, page_size, scale,
             int(window or 0), _code(q), _stream()), "attention_prefill")
    return out


ATTENTION_TILE = 64        # query tokens per CTA of the prefill kernel
ATTENTION_TC_TILE = 128    # and of its tcgen05 form
ATTENTION_TC = os.environ.get("LOGSSMS_B200_ATTN_TC", "1") != "0"


def attention_prefill_tc_ok(q: torch.Tensor, k_cache: torch.Tensor) -> bool:
    """Does the tcgen05 prompt-attention kernel take these operands (bfloat16, head size 64 or 128, pages of a
    multiple of 64 tokens)?  Else `attention_prefill`."""
    return (ATTENTION_TC and q.dtype == torch.bfloat16 and q.dim() == 3 and q.shape[2] in (64, 128) and k_cache.dim() == 4
            and k_cache.shape[1] % 64 == 0 and k_cache.shape[3] == q.shape[2] and q.shape[1] % k_cache.shape[2] == 0
            and q.is_contiguous() and k_cache.is_contiguous())


def prefill_splits(num_tiles: int, num_heads: int, max_context: int) -> int:
    """Key ranges per 128-query tile for `attention_prefill_tc`: a step of few tiles over a long context (a prompt
    portion far into its prompt) would leave most SMs idle with one CTA per (tile, head), so the keys are shared out
    until the grid fills the SMs, each range keeping at least 512 keys."""
    items = max(1, num_tiles * num_heads)
    return max(1, min(_SM_COUNT // items, max_context // 512, 16))


_SM_COUNT = 148


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, start_pos: torch.Tensor, tiles: torch.Tensor, num_tiles: int,
                         scale: float, window: int = 0, *, out: torch.Tensor | None = None, splits: int = 1) -> torch.Tensor:
    """`attention_prefill` on the tcgen05 tensor cores: the same arguments, but `tiles` lists 128-token tiles.
    `splits` > 1 cuts every tile's keys into that many ranges, each a CTA of its own, merged by a second kernel.
    `check_kernel_errors()` reports a kernel whose internal wait gave up."""
    _cuda(q, k_cache, v_cache, block_table, cu_seqlens, start_pos, tiles)
    _need(attention_prefill_tc_ok(q, k_cache), "attention_prefill_tc takes bfloat16, head size 64 or 128 and pages of a multiple of 64 tokens")
    tokens, Hq, hd = q.shape
    _need(v_cache.shape == k_cache.shape and v_cache.is_contiguous() and v_cache.dtype == k_cache.dtype == q.dtype,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    pages, page_size, Hkv = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(start_pos, "start_pos")
    _i32(tiles, "tiles")
    _need(tiles.numel() >= 2 * num_tiles, "tiles holds fewer pairs than num_tiles")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    err = error_word(q.device)
    splits = max(1, int(splits))
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(num_tiles * Hq * splits * ATTENTION_TC_TILE * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(num_tiles * Hq * splits * ATTENTION_TC_TILE * 2, dtype=torch.float32, device=q.device)
    f = _fn("attention_prefill_tc", "lb_attention_prefill_tc",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), tokens, pages, _ptr(block_table), block_table.stride(0),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(tiles), num_tiles, Hq, Hkv, hd, page_size, scale, int(window or 0),
             _ptr(err), splits, _ptr(part_o), _ptr(part_ml), _stream()), "attention_prefill_tc", launches=2 if splits > 1 else 1)
    return out


# --------------------------------------------------------------------------- Mamba2
def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                  cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, num_requests: int,
                  max_len: int, region_ends: tuple[int, int], region_scales: tuple[float, float, float],
                  activation: str = "silu") -> torch.Tensor:
    """x: [tokens, C] (column view allowed); weight: [C, K] float32; state: [slots, C, K-1] of x's dtype,
    read then rewritten in place (None with one tap: nothing is carried).  Returns silu(conv), or with `activation`
    "none" conv itself, as a contiguous [tokens, C]."""
    _cuda(x, weight, bias, state, cu_seqlens, start_pos, slots)
    tokens, C = x.shape
    K = weight.shape[1]
    _need(x.stride(1) == 1, "conv input needs unit column stride")
    _need(weight.dtype == torch.float32 and weight.shape == (C, K) and weight.is_contiguous(), "conv weight must be float32 [C, K]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (C,) and bias.is_contiguous()), "conv bias must be float32 [C]")
    _need(1 <= K <= 8, f"conv kernel sizes 1..8 are built, got {K}")
    _need(activation in ("silu", "none"), "the convolution is followed by silu or by nothing")
    _need((K == 1 and state is None) or (state is not None and state.dtype == x.dtype and state.is_contiguous()
                                         and state.shape[1:] == (C, K - 1)),
          "conv state must be contiguous [slots, C, K-1] of the activation dtype")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, n)
    out = torch.empty((tokens, C), dtype=x.dtype, device=x.device)
    f = _fn("conv", "lb_causal_conv1d", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                         c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(state), _ptr(out), _ptr(cu_seqlens),
             _ptr(start_pos), _ptr(slots), num_requests, max_len, C, K, region_ends[0], region_ends[1],
             region_scales[0], region_scales[1], region_scales[2], int(activation == "none"), _code(x), _stream()), "causal_conv1d",
           launches=1 if max_len <= 8 else 2)
    return out


def _ssm_state_ok(state: torch.Tensor, act: torch.dtype) -> bool:
    return state.is_contiguous() and (state.dtype == torch.float32 or (state.dtype == torch.bfloat16 == act))


def ssm_scan(conv: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
             num_requests: int, num_heads: int, head_dim: int, state_dim: int, num_groups: int,
             dt_scale: float, gate: torch.Tensor | None = None, gate_scale: float = 1.0, *,
             request_list: torch.Tensor | None = None, num_listed: int = 0,
             out: torch.Tensor | None = None, beside: bool = False) -> torch.Tensor:
    """conv: [tokens, nh*P + 2*G*N] (x | B | C; a column view is fine); dt: [tokens, nh] view; state: float32 (or,
    with bfloat16 activations, bfloat16: rounded once per call) [slots, nh, P, N], updated in place.  Returns y [tokens, nh*P]; with `gate` ([tokens, nh*P] view)
    the result is y * silu(gate * gate_scale), the gate of a mixer that has no norm.  `request_list`
    (int32 indices into the batch, `num_listed` of them) restricts the call to those requests; the rows
    of `out` that belong to other requests are left as they are.  `beside`: other kernels of the step run at the same
    time (on another stream): the launch then takes a grid that is resident at once and walks its items, instead of one
    CTA per item that would take every SM slot before them."""
    _cuda(conv, dt, A_log, dt_bias, D, state, cu_seqlens, start_pos, slots, gate, request_list, out)
    if request_list is not None:
        _i32(request_list, "request_list")
        _need(request_list.numel() >= num_listed, "request_list is shorter than num_listed")
        num_requests = num_listed
    if gate is not None:
        _need(gate.shape == (conv.shape[0], num_heads * head_dim) and gate.stride(1) == 1 and gate.dtype == conv.dtype,
              "gate must be a [tokens, heads * head_dim] view of the activation dtype")
    tokens, C = conv.shape
    _need(conv.stride(1) == 1, "conv output needs unit column stride")
    _need(dt.shape == (tokens, num_heads) and dt.stride(1) == 1 and dt.dtype == conv.dtype, "dt must be a [tokens, heads] view")
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (D, "D")):
        _need(t.dtype == torch.float32 and t.shape == (num_heads,) and t.is_contiguous(), f"{n} must be float32 [heads]")
    _need(_ssm_state_ok(state, conv.dtype) and state.shape[1:] == (num_heads, head_dim, state_dim),
          "SSM state must be contiguous float32 (or bfloat16 beside bfloat16 activations) [slots, heads, P, N]")
    _need(state_dim % 4 == 0 and state_dim <= 256, f"state sizes in steps of 4 up to 256 are built, got {state_dim}")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, n)
    y = out if out is not None else torch.empty((tokens, num_heads * head_dim), dtype=conv.dtype, device=conv.device)
    _need(y.shape == (tokens, num_heads * head_dim) and y.dtype == conv.dtype and y.is_contiguous(), "out must be [tokens, heads * head_dim]")
    f = _fn("ssm", "lb_ssm_scan", [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                   c_long, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(conv), C, conv.stride(0) if tokens > 1 else C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D),
             _ptr(state), _ptr(y), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), num_requests, num_heads, head_dim,
             state_dim, num_groups, dt_scale, _ptr(gate), gate.stride(0) if gate is not None else 0, gate_scale,
             _ptr(request_list), int(bool(beside)), int(state.dtype == torch.bfloat16), _code(conv), _stream()), "ssm_scan")
    return y


SSD_TC = os.environ.get("LOGSSMS_B200_SSD_TC", "1") != "0"
SSD_TC_CHUNK = 128


def ssd_chunk_scan_tc_ok(head_dim: int, state_dim: int, chunk_len: int) -> bool:
    """Does the tcgen05 chunk-scan kernel take these sizes (head size 64 or 128: the kernels that make the chunk
    states before it take no larger heads; state size 64..256 in steps of 64, chunks of 128 tokens)?"""
    return (SSD_TC and head_dim in (64, 128) and state_dim % 64 == 0 and 64 <= state_dim <= 256
            and chunk_len == SSD_TC_CHUNK)


def ssd_chunk_len(chunk_size: int, head_dim: int, state_dim: int) -> int:
    """Chunk length the tensor-core SSD kernels will use for these sizes (at most `chunk_size`), or 0
    when they do not take them (then the token-by-token scan runs everything)."""
    if chunk_size >= SSD_TC_CHUNK and ssd_chunk_scan_tc_ok(head_dim, state_dim, SSD_TC_CHUNK):
        return SSD_TC_CHUNK                   # the tcgen05 chunk scan wants its 128 rows
    lib = build.load("ssd")
    f = lib.lb_ssd_chunk_len
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return int(f(int(chunk_size), int(head_dim), int(state_dim)))


def ssd_prefill(conv: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
                state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
                chunks: torch.Tensor, num_chunks: int, req_chunks: torch.Tensor, num_long: int, chunk_len: int,
                num_heads: int, head_dim: int, state_dim: int, num_groups: int, dt_scale: float,
                gate: torch.Tensor | None = None, gate_scale: float = 1.0, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """Chunked scan of the listed prompt portions (bfloat16, tensor cores).  `chunks`: int32 [n, 2] =
    (request index, first token of the chunk within its portion); `req_chunks`: int32 [m, 3] = (request
    index, its first chunk, its number of chunks).  Arguments otherwise as `ssm_scan`; rows of `out`
    outside the listed requests are left as they are."""
    _cuda(conv, dt, A_log, dt_bias, D, state, cu_seqlens, start_pos, slots, chunks, req_chunks, gate, out)
    tokens, C = conv.shape
    _need(conv.dtype == torch.bfloat16 and conv.is_contiguous(), "ssd_prefill takes a contiguous bfloat16 conv output")
    _need(dt.shape == (tokens, num_heads) and dt.stride(1) == 1 and dt.dtype == conv.dtype, "dt must be a [tokens, heads] view")
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (D, "D")):
        _need(t.dtype == torch.float32 and t.shape == (num_heads,) and t.is_contiguous(), f"{n} must be float32 [heads]")
    _need(_ssm_state_ok(state, conv.dtype) and state.shape[1:] == (num_heads, head_dim, state_dim),
          "SSM state must be contiguous float32 or bfloat16 [slots, heads, P, N]")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots"), (chunks, "chunks"), (req_chunks, "req_chunks")):
        _i32(t, n)
    _need(chunks.numel() >= 2 * num_chunks and req_chunks.numel() >= 3 * num_long, "work lists are shorter than their counts")
    if gate is not None:
        _need(gate.shape == (tokens, num_heads * head_dim) and gate.stride(1) == 1 and gate.dtype == conv.dtype,
              "gate must be a [tokens, heads * head_dim] view of the activation dtype")
    y = out if out is not None else torch.empty((tokens, num_heads * head_dim), dtype=conv.dtype, device=conv.device)
    _need(y.shape == (tokens, num_heads * head_dim) and y.dtype == conv.dtype and y.is_contiguous(), "out must be [tokens, heads * head_dim]")
    scratch = torch.empty((max(num_chunks, 1), num_heads, head_dim, state_dim), dtype=torch.float32, device=conv.device)
    chunk_a = torch.empty((max(num_chunks, 1), num_heads), dtype=torch.float32, device=conv.device)
    s_in = torch.empty(scratch.shape, dtype=torch.bfloat16, device=conv.device)
    gate_stride = gate.stride(0) if gate is not None else 0
    # the chunk scan on the tcgen05 kernel where it takes the sizes
    tc = ssd_chunk_scan_tc_ok(head_dim, state_dim, chunk_len) and conv.data_ptr() % 16 == 0 and y.data_ptr() % 16 == 0
    f = _fn("ssd", "lb_ssd_prefill", [c_void_p, c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_float, c_int, c_int, c_int,
                                      c_void_p])
    _check(f(_ptr(conv), C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D), _ptr(state), _ptr(y),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(chunks), num_chunks, _ptr(req_chunks), num_long,
             _ptr(scratch), _ptr(s_in), _ptr(chunk_a), num_heads, head_dim, state_dim, num_groups, chunk_len, dt_scale,
             _ptr(gate), gate_stride, gate_scale, 0 if tc else 1, int(state.dtype == torch.bfloat16), _code(conv), _stream()),
           "ssd_prefill", f"(head_dim {head_dim}, state_dim {state_dim}, chunk {chunk_len})", launches=2 if tc else 3)
    if tc:
        err = error_word(conv.device)
        g = _fn("ssd_tc", "lb_ssd_chunk_scan_tc",
                [c_void_p, c_long, c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_float, c_void_p, c_void_p])
        _check(g(_ptr(conv), tokens, C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D), _ptr(y),
                 _ptr(cu_seqlens), _ptr(chunks), num_chunks, _ptr(s_in), num_heads, head_dim, state_dim, num_groups,
                 chunk_len, dt_scale, _ptr(gate), gate_stride, gate_scale, _ptr(err), _stream()),
               "ssd_chunk_scan_tc", f"(head_dim {head_dim}, state_dim {state_dim}, chunk {chunk_len})")
    return y


# --------------------------------------------------------------------------- matrix products
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    _cuda(a, w, bias)
    _need(a.dtype == w.dtype == torch.float32, "gemm_f32 takes float32 operands")
    _need(a.dim() == 2 and a.stride(1) == 1 and w.dim() == 2 and w.is_contiguous() and a.shape[1] == w.shape[1],
          "gemm_f32 wants a [M, K] (row-strided) and w [N, K]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (w.shape[0],)), "bias must be float32 [N]")
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    f = _fn("gemm_f32", "lb_gemm_f32", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                                        c_float, c_void_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, K, out_scale, _stream()), "gemm_f32")
    return out


def linear_join_ok(x, w: torch.Tensor, bias, join: ResidualJoin | None) -> bool:
    """Can `linear_join` take this product?  Few bfloat16 rows (the consumers norm at most 16), whole blocks of 16
    output columns, a residual of the output's shape."""
    if join is None or isinstance(x, NormedRows) or not _skinny_ok(x, w, bias, 16) or w.shape[0] % 16:
        return False
    r = join.residual
    return r is None or (r.dtype == torch.bfloat16 and r.shape == (x.shape[0], w.shape[0]) and r.is_contiguous())


def linear_join(x: torch.Tensor, w: torch.Tensor, bias, join: ResidualJoin, *, out_scale: float = 1.0) -> SummedRows:
    """x @ w^T (+ bias, * out_scale) whose epilogue joins the residual stream: see `ResidualJoin`, `SummedRows`."""
    _need(linear_join_ok(x, w, bias, join), "linear_join takes at most 16 bfloat16 rows and N a multiple of 16")
    M, Kdim = x.shape
    N = w.shape[0]
    other = join.other_tensor()
    _need(other is None or (other.dtype == torch.bfloat16 and other.shape == (M, N) and other.is_contiguous()),
          "the other branch must be contiguous bfloat16 [M, N]")
    _cuda(x, w, bias, other, join.residual)
    vsum = torch.empty((M, N), dtype=torch.float32, device=x.device)
    partial = torch.empty((N // 16, M), dtype=torch.float32, device=x.device)
    res_out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    f = _fn("linear_skinny", "lb_linear_skinny_join",
            [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_float,
             c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), M, N, Kdim, out_scale, _ptr(other), _ptr(join.residual),
             join.in_scales[0], join.in_scales[1], _ptr(vsum), _ptr(res_out), _ptr(partial), _stream()), "linear_skinny_join")
    return SummedRows(vsum, res_out, partial)


def summed_rmsnorm(rows: SummedRows, weight: torch.Tensor, eps: float, out_scales) -> tuple:
    """The RMSNorm of summed rows as a kernel of its own: for a consumer that cannot norm them itself (the built-in
    products can), same rounding points as `add_rmsnorm`."""
    v = rows.vsum
    _cuda(v, weight)
    M, H = v.shape
    _need(v.dtype == torch.float32 and v.is_contiguous(), "summed rows are contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(),
          "norm weight must be a contiguous float32 vector of the row width")
    _need(1 <= len(out_scales) <= 2, "one or two outputs")
    act = rows.residual.dtype
    out0 = torch.empty((M, H), dtype=act, device=v.device)
    out1 = torch.empty((M, H), dtype=act, device=v.device) if len(out_scales) == 2 else None
    f = _fn("norm", "lb_summed_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float,
                                          c_int, c_void_p])
    _check(f(_ptr(v), _ptr(weight), _ptr(out0), _ptr(out1), M, H, eps, out_scales[0], out_scales[-1],
             _DTYPE_CODE[act], _stream()), "summed_rmsnorm")
    return (out0,) if out1 is None else (out0, out1)


# Rows up to which a norm rides in the products that consume it (and a product's epilogue joins the residual stream
# for it).  The kernels take 16; measured on 36-layer decode steps, 12 rows take 1.57 instead of 1.65 ms and 16 rows
# 1.78 instead of 1.96 ms with the norm as a kernel of its own: every CTA of a consumer norms all rows for itself.
DEFERRED_NORM_MAX_ROWS = 8


def deferred_norm_ok(x) -> bool:
    """Can a norm over these rows ride in the prologue of the products that consume it?"""
    if isinstance(x, SummedRows):
        return 0 < x.shape[0] <= DEFERRED_NORM_MAX_ROWS and x.shape[1] % 8 == 0
    return (x.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= DEFERRED_NORM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.shape[1] <= 2048 and x.is_contiguous())


def _skinny_normed(nr: NormedRows, w: torch.Tensor, bias, out_scale: float, out_f32: bool, swiglu_scale) -> torch.Tensor:
    M, Kdim = nr.x.shape
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=w.device)
    if nr.summed:
        _check(_summed_fn()(_ptr(nr.x.vsum), _ptr(nr.x.partial), nr.x.partial.shape[0], _ptr(nr.weight), nr.eps, nr.scale,
                            _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
                            swiglu_scale if swiglu_scale is not None else 1.0, mode,
                            None, None, None, None, None, 0, 0, 0, 0, 0, 1.0, 1.0, 1.0, _stream()), "linear_skinny_summed")
        return out
    write = nr.shared["residual_out"] is not None and not nr.shared["written"]
    f = _fn("linear_skinny", "lb_linear_skinny_normed",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_void_p, c_void_p,
             c_void_p, c_long, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(nr.x), _ptr(nr.other), _ptr(nr.residual), _ptr(nr.shared["residual_out"]) if write else None,
             _ptr(nr.weight), nr.eps, nr.in_scales[0], nr.in_scales[1], nr.scale, _ptr(w), _ptr(bias), _ptr(out), N, M, N,
             Kdim, out_scale, swiglu_scale if swiglu_scale is not None else 1.0, mode, _stream()), "linear_skinny_normed")
    if write:
        nr.shared["written"] = True
    return out


def _summed_fn():
    return _fn("linear_skinny", "lb_linear_skinny_summed",
               [c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                c_float, c_float, c_float, c_void_p])


# At or below this many rows a bfloat16 product goes to the weight-streaming kernel (which takes up to 64).  Measured
# on 36-layer decode steps: with the library above 32 rows a step of 48 rows takes 2.48 instead of 2.72 ms and one of
# 64 rows 2.77 instead of 3.07 ms; with the library above 16 rows a step of 24 rows 2.62 instead of 2.18 ms.
SKINNY_MAX_ROWS = 32


def _skinny_ok(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, max_rows: int | None = None) -> bool:
    max_rows = SKINNY_MAX_ROWS if max_rows is None else max_rows
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= max_rows
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())))


_PLAIN, _OUT_F32, _SWIGLU = 0, 1, 2


def linear_skinny(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
                  out_f32: bool = False, swiglu_scale: float | None = None) -> torch.Tensor:
    """The weight-streaming product for at most 64 bfloat16 rows: x [M, K] @ w[N, K]^T, with the bias,
    output multiplier, float32 output or SwiGLU (w = [gate rows; up rows]) done on the sums."""
    _cuda(x, w, bias)
    _need(_skinny_ok(x, w, bias, 64), "linear_skinny takes at most 64 bfloat16 rows, K a multiple of 8, 16-byte aligned operands")
    M, Kdim = x.shape
    _need(w.dim() == 2 and w.shape[1] == Kdim, "weight must be [N, K]")
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        _need(N % 2 == 0 and bias is None and not out_f32 and out_scale == 1.0, "the SwiGLU form takes [gate; up] rows and nothing else")
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    _need(bias is None or bias.shape == (N,), "bias must be [N]")
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    f = _fn("linear_skinny", "lb_linear_skinny", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int,
                                                  c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
             swiglu_scale if swiglu_scale is not None else 1.0, mode, _stream()), "linear_skinny")
    return out


_gemm_error: dict[torch.device, torch.Tensor] = {}
# Which kernel takes bfloat16 products of more rows than the weight streamer.  "auto" and "library": cuBLAS through
# torch, the SwiGLU as a kernel of its own behind it.  "tcgen05": the engine's own tcgen05 kernel with its fused
# epilogues.  Measured at 2048 x 4096 x 1024 (gate|up of a 2,048-token prompt): the library product 16.3 us + SwiGLU
# kernel 7.1 us = 23.4 us against 33.4 us for the fused tcgen05 kernel, whose 128 x 128 one-CTA tiles are bound by
# L2 -> SM traffic (64 FLOP per byte; the library runs 256 x 256 two-CTA tiles); at 64 rows its 128-row tile is
# half empty.  It stays selectable and tested, and is not the default until it wins.
GEMM_MODE = os.environ.get("LOGSSMS_B200_GEMM", "auto")


def _tcgen05_ok(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] > 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
                 out_f32: bool = False, swiglu_scale: float | None = None) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), with the
    bias, output multiplier, float32 output or SwiGLU (w = [gate rows; up rows]) done on the sums.
    `check_kernel_errors()` reports a kernel whose internal wait gave up."""
    _cuda(x, w, bias)
    _need(_tcgen05_ok(x, w, bias), "gemm_tcgen05 takes bfloat16 operands, K a multiple of 8, 16-byte aligned")
    M, Kdim = x.shape
    _need(w.dim() == 2 and w.shape[1] == Kdim, "weight must be [N, K]")
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        _need(N % 2 == 0 and bias is None and not out_f32 and out_scale == 1.0, "the SwiGLU form takes [gate; up] rows and nothing else")
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    _need(bias is None or bias.shape == (N,), "bias must be [N]")
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    err = error_word(x.device)
    f = _fn("gemm_tcgen05", "lb_gemm_tcgen05", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                                                c_float, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
             swiglu_scale if swiglu_scale is not None else 1.0, mode, _ptr(err), _stream()), "gemm_tcgen05")
    return out


def error_word(device) -> torch.Tensor:
    """The int32 word on `device` into which a kernel whose bounded wait gave up writes where it stopped (0: none
    did).  One per device, shared by all such kernels; the scheduler reads it with every step's sampled ids, the
    trace replay after every step."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device(device.type, torch.cuda.current_device())
    err = _gemm_error.get(device)
    if err is None:
        with torch.inference_mode(False):      # an ordinary tensor, whoever asks first: the host may set and clear it anywhere
            err = _gemm_error[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return err


def raise_kernel_error(code: int, device=None) -> None:
    """Clear the error word of `device` (all devices when None) and raise what `code` says."""
    for dev, err in _gemm_error.items():
        if device is None or _same_device(dev, device):
            err.zero_()
    raise KernelError(f"a wait inside a kernel gave up, its results are not valid (role {(code >> 24) & 0x3F}, "
                      f"block {(code >> 12) & 0xFFF}, step {code & 0xFFF})")


def _same_device(a, b) -> bool:
    a, b = torch.device(a), torch.device(b)
    return a.type == b.type and (a.index is None or b.index is None or a.index == b.index)


def check_kernel_errors(device=None) -> None:
    """Raise if a kernel gave up on one of its bounded waits since the last check (synchronises)."""
    for dev, err in _gemm_error.items():
        if device is not None and not _same_device(dev, device):
            continue
        code = int(err.item())
        if code:
            raise_kernel_error(code, dev)


def linear_conv_step_ok(x, w: torch.Tensor, bias, conv_state: torch.Tensor, max_rows: int | None = None) -> bool:
    """Should `linear_conv_step` take these operands (else: `linear`, then `causal_conv1d`)?  `max_rows`: the most
    rows (default: as many as go to the weight streamer at all; the kernel itself takes 64)."""
    if conv_state.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.data_ptr() % 16:
        return False
    if bias is not None and not (bias.dtype == torch.bfloat16 and bias.is_contiguous()):
        return False
    if isinstance(x, NormedRows):
        return w.shape[1] == x.shape[1]
    return _skinny_ok(x, w, bias, max_rows)


def linear_conv_step(x, w: torch.Tensor, bias, conv_weight: torch.Tensor, conv_bias, conv_state: torch.Tensor,
                     slots: torch.Tensor, start_pos: torch.Tensor, first: int, last: int,
                     region_ends: tuple[int, int], region_scales: tuple[float, float, float]) -> torch.Tensor:
    """x @ w^T (+ bias) for a decode batch (every row the single new token of its own request), with the
    depthwise conv step done on the output columns [first, last) before they are stored: those columns come
    back as silu(conv(...)) and `conv_state` ([slots, last - first, taps - 1]) is shifted in place.  `x` may be
    `NormedRows`.  `region_ends` are column indices relative to `first`."""
    normed = isinstance(x, NormedRows)
    _need(linear_conv_step_ok(x, w, bias, conv_state, 64), "linear_conv_step takes few bfloat16 rows (see linear_skinny)")
    C = last - first
    taps = conv_weight.shape[1]
    _need(conv_weight.dtype == torch.float32 and conv_weight.shape == (C, taps) and conv_weight.is_contiguous(), "conv weight must be float32 [C, K]")
    _need(conv_bias is None or (conv_bias.dtype == torch.float32 and conv_bias.shape == (C,) and conv_bias.is_contiguous()), "conv bias must be float32 [C]")
    _need(conv_state.is_contiguous() and conv_state.shape[1:] == (C, taps - 1), "conv state must be contiguous [slots, C, K-1]")
    _i32(slots, "slots")
    _i32(start_pos, "start_pos")
    M, Kdim = x.shape
    N = w.shape[0]
    _need(slots.numel() >= M and start_pos.numel() >= M and 0 <= first <= last <= N, "one slot and start per row; columns within the output")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
    if normed and x.summed:
        _check(_summed_fn()(_ptr(x.x.vsum), _ptr(x.x.partial), x.x.partial.shape[0], _ptr(x.weight), x.eps, x.scale,
                            _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, 1.0, 1.0, _PLAIN,
                            _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state), _ptr(slots), _ptr(start_pos), first, last, taps,
                            region_ends[0], region_ends[1], region_scales[0], region_scales[1], region_scales[2], _stream()),
               "linear_conv_step")
        return out
    write = normed and x.shared["residual_out"] is not None and not x.shared["written"]
    f = _fn("linear_skinny", "lb_linear_skinny_conv",
            [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_void_p,
             c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    if normed:
        head = (None, 0, _ptr(x.x), _ptr(x.other), _ptr(x.residual), _ptr(x.shared["residual_out"]) if write else None,
                _ptr(x.weight), x.eps, x.in_scales[0], x.in_scales[1], x.scale)
    else:
        _cuda(x)
        head = (_ptr(x), x.stride(0), None, None, None, None, None, 0.0, 1.0, 1.0, 1.0)
    _check(f(*head, _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state),
             _ptr(slots), _ptr(start_pos), first, last, taps, region_ends[0], region_ends[1], region_scales[0],
             region_scales[1], region_scales[2], _stream()), "linear_conv_step")
    if write:
        x.shared["written"] = True
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
           out_f32: bool = False, lazy_scale: bool = False):
    """round(round(x [M, K] @ w[N, K]^T + bias) * out_scale) in x's dtype, or as float32 with `out_f32`.
    With `lazy_scale` (the caller's consumer takes `ScaledRows`) a product whose kernel has no epilogue for the
    multiplier comes back as `ScaledRows` instead of going through the scale kernel.

    float32 activations: the engine's own 32-bit kernel.  bfloat16: at most 64 rows go to the
    weight-streaming kernel (a decode step is bound by reading the weights once); more rows go to
    cuBLAS through torch (32-bit accumulation).  bfloat16 activations with a weight that is stored in
    32-bit: the 32-bit kernel on widened activations, result rounded once.  `x` may be `NormedRows`."""
    if isinstance(x, NormedRows):
        if (w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == x.shape[1] and w.data_ptr() % 16 == 0
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))):
            return _skinny_normed(x, w, bias, out_scale, out_f32, None)
        x = x.tensor()
    _cuda(x, w, bias)
    if x.dtype == torch.float32:
        return gemm_f32(x, w.float(), None if bias is None else bias.float(), out_scale)
    if w.dtype == torch.float32:
        y = gemm_f32(x.float(), w, None if bias is None else bias.float()).to(x.dtype)
    elif _skinny_ok(x, w, bias):
        return linear_skinny(x, w, bias, out_scale=out_scale, out_f32=out_f32)
    elif GEMM_MODE == "tcgen05" and _tcgen05_ok(x, w, bias):
        return gemm_tcgen05(x, w, bias, out_scale=out_scale, out_f32=out_f32)
    else:
        # the library product, asked for as mm / addmm: the same cuBLAS call as `F.linear` makes, with 4 us less of
        # dispatch on the host per call (a prompt step of a new shape is bound by the host)
        product = (lambda: torch.mm(x, w.t())) if bias is None else (lambda: torch.addmm(bias.to(x.dtype), x, w.t()))
        y = PROFILER.timed("library", "mm", product) if PROFILER.enabled else product()
    if lazy_scale and not out_f32 and out_scale != 1.0:
        return ScaledRows(y, out_scale)
    if out_f32 or out_scale != 1.0:
        y = scale(y, out_scale, to_f32=out_f32)
    return y


def linear_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T as float32 whose sums were never rounded to the activation dtype: what enters a recurrence's
    32-bit arithmetic (a decay's input).  Few bfloat16 rows: the weight-streaming kernel with its float32 output; more: the
    library product with float32 output; float32 activations: the engine's own 32-bit kernel."""
    _cuda(x, w)
    if x.dtype == torch.float32:
        return gemm_f32(x, w.float())
    if w.dtype == torch.bfloat16 and _skinny_ok(x, w, None):
        return linear_skinny(x, w, out_f32=True)
    product = lambda: torch.mm(x, w.to(x.dtype).t(), out_dtype=torch.float32)
    return PROFILER.timed("library", "mm", product) if PROFILER.enabled else product()


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act_scale: float) -> torch.Tensor:
    """silu(round(gate * act_scale)) * up with [gate | up] = x @ w_gate_up^T (w rows: gate, then up).
    `x` may be `NormedRows`."""
    if isinstance(x, NormedRows):
        if (w_gate_up.dtype == torch.bfloat16 and w_gate_up.is_contiguous() and w_gate_up.shape[1] == x.shape[1]
                and w_gate_up.shape[0] % 2 == 0 and w_gate_up.data_ptr() % 16 == 0):
            return _skinny_normed(x, w_gate_up, None, 1.0, False, act_scale)
        x = x.tensor()
    if _skinny_ok(x, w_gate_up, None):
        return linear_skinny(x, w_gate_up, swiglu_scale=act_scale)
    if GEMM_MODE == "tcgen05" and _tcgen05_ok(x, w_gate_up, None):
        return gemm_tcgen05(x, w_gate_up, swiglu_scale=act_scale)
    return swiglu(linear(x, w_gate_up), act_scale)


# --------------------------------------------------------------------------- a 32-bit residual stream (post-norm layers)
from .fusion import StreamRows      # noqa: E402  (re-exported like the other classes of the protocol)


def embed_pair(table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, token_req: torch.Tensor,
               cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, prev_state: torch.Tensor,
               scale: float, buckets: int, mul_prev: int, mul_cur: int, bad_ids: torch.Tensor | None = None) -> StreamRows:
    """table[id] * scale + pairs[(previous id * mul_prev + id * mul_cur) mod buckets] (row `buckets` for a sequence's
    first token), summed in 32-bit.  `prev_state`: int32 [slots, 1], the last id each request has fed so far; read
    for a portion's first token and replaced by the portion's last id."""
    _cuda(table, pairs, ids, token_req, cu_seqlens, start_pos, slots, prev_state)
    for t, name in ((ids, "ids"), (token_req, "token_req"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, name)
    _need(prev_state.dtype == torch.int32 and prev_state.is_contiguous(), "prev_state must be contiguous int32")
    _need(table.dim() == 2 and table.is_contiguous() and pairs.is_contiguous() and pairs.dtype == table.dtype
          and pairs.shape == (buckets + 1, table.shape[1]), "pairs table must be [buckets + 1, hidden] of the embedding's dtype")
    V, H = table.shape
    T = ids.numel()
    f32 = torch.empty((T, H), dtype=torch.float32, device=table.device)
    act = f32 if table.dtype == torch.float32 else torch.empty((T, H), dtype=table.dtype, device=table.device)
    f = _fn("embed", "lb_embed_pair", [c_void_p] * 10 + [c_int, c_int, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong,
                                                          c_float, c_void_p, c_int, c_void_p])
    _check(f(_ptr(f32), None if act is f32 else _ptr(act), _ptr(table), _ptr(pairs), _ptr(ids), _ptr(token_req),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(prev_state), T, H, V, buckets, mul_prev, mul_cur, scale,
             _ptr(bad_ids), _code(table), _stream()), "embed_pair")
    return StreamRows(f32, act)


def skip_rmsnorm(stream: StreamRows, y: torch.Tensor | None, skip: float, weight: torch.Tensor, eps: float, *,
                 extra: torch.Tensor | None = None, row_scale: torch.Tensor | None = None, want_f32: bool = True,
                 act_dtype: torch.dtype | None = None) -> StreamRows:
    """RMSNorm(skip * stream + y [+ row_scale[t] * extra]) * weight in 32-bit: the new stream and its copy rounded to
    the activation dtype (`act_dtype`, default y's).  Without `want_f32` only the rounded copy is made (the norm in
    front of the output head)."""
    x = stream.f32
    _cuda(x, y, weight, extra, row_scale)
    rows, H = x.shape
    act_dtype = act_dtype or (y.dtype if y is not None else stream.act.dtype)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "the stream must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(), "norm weight must be float32 [width]")
    for t, name in ((y, "y"), (extra, "extra")):
        _need(t is None or (t.shape == x.shape and t.dtype == act_dtype and t.is_contiguous()), f"{name} must match the stream's shape")
    _need((extra is None) == (row_scale is None), "extra rows come with a scale per row")
    _need(row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() == rows and row_scale.is_contiguous()),
          "row_scale must be float32 [rows]")
    f32 = torch.empty_like(x) if want_f32 else None
    act = f32 if (act_dtype == torch.float32 and want_f32) else torch.empty((rows, H), dtype=act_dtype, device=x.device)
    f = _fn("stream_norm", "lb_skip_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(y), _ptr(extra), _ptr(row_scale), skip, _ptr(weight), eps, _ptr(f32), None if act is f32 else _ptr(act),
             rows, H, _DTYPE_CODE[act_dtype], _stream()), "skip_rmsnorm", f"(width {H})")
    return StreamRows(f32, act)


# --------------------------------------------------------------------------- gated linear attention
def _gla_decay_checks(z, head_decay, T: int, H: int, dk: int) -> None:
    if head_decay is None:
        _need(z is not None and z.dtype == torch.float32 and z.shape == (T, H * dk) and z.is_contiguous(),
              "z must be contiguous float32 [tokens, H*key_dim]")
    else:
        _need(z is None and head_decay.dtype == torch.float32 and head_decay.shape == (H,) and head_decay.is_contiguous(),
              "a fixed decay per head is float32 [H] and comes without z")


def gla_scan(qkv: torch.Tensor, z: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
             slots: torch.Tensor, num_requests: int, num_heads: int, key_dim: int, value_dim: int, tau: float,
             q_scale: float, request_list: torch.Tensor | None = None, out: torch.Tensor | None = None,
             head_decay: torch.Tensor | None = None) -> torch.Tensor:
    """Token-by-token recurrence S <- diag(sigmoid(z)^(1/tau)) S + k v^T, o = S^T (q * q_scale) per head over every
    request's tokens.  qkv: [tokens, >= 2*H*key_dim + H*value_dim] with columns q | k | v first (unit column stride);
    z: float32 [tokens, H*key_dim]; state: float32 [slots, H, key_dim, value_dim], updated in place.  Returns float32
    [tokens, H*value_dim].  With `head_decay` (float32 [H]) every key channel of head h decays by head_decay[h] at every
    token, and z (then None) is not read."""
    _cuda(qkv, z, state, cu_seqlens, start_pos, slots, request_list, head_decay)
    H, dk, dv = num_heads, key_dim, value_dim
    T = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= H * (2 * dk + dv), "qkv must hold the columns q | k | v")
    _gla_decay_checks(z, head_decay, T, H, dk)
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dk, dv),
          "the state must be contiguous float32 [slots, H, key_dim, value_dim]")
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, name)
    n = num_requests
    if request_list is not None:
        _i32(request_list, "request_list")
        n = request_list.numel()
    o = out if out is not None else torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    item, base = qkv.element_size(), qkv.data_ptr()
    stride = qkv.stride(0) if T > 1 else qkv.shape[1]
    f = _fn("gla", "lb_gla_scan", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p])
    _check(f(base, base + H * dk * item, base + 2 * H * dk * item, stride, _ptr(z), _ptr(o), _ptr(state), _ptr(cu_seqlens),
             _ptr(start_pos), _ptr(slots), _ptr(request_list), n, H, dk, dv, tau, q_scale, _ptr(head_decay), _code(qkv), _stream()),
           "gla_scan", f"(key_dim {dk}, value_dim {dv})")
    return o


GLA_CHUNKED = os.environ.get("LOGSSMS_B200_GLA_CHUNKED", "1") != "0"
GLA_CHUNK = 16


def gla_chunked_ok(qkv: torch.Tensor, key_dim: int) -> bool:
    """Does the chunked form take these operands (else: the token-by-token scan)?  bfloat16, key channels a multiple of 16
    up to 256."""
    return GLA_CHUNKED and qkv.dtype == torch.bfloat16 and key_dim % 16 == 0 and key_dim <= 256


def gla_chunked(qkv: torch.Tensor, z: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
                slots: torch.Tensor, chunks: torch.Tensor, num_chunks: int, per_request: torch.Tensor, num_long: int,
                num_heads: int, key_dim: int, value_dim: int, tau: float, q_scale: float, out: torch.Tensor,
                segments: torch.Tensor | None = None, segment_requests: torch.Tensor | None = None,
                head_decay: torch.Tensor | None = None) -> torch.Tensor:
    """The recurrence of `gla_scan` over the long portions of a step in chunks of `GLA_CHUNK` tokens on the tensor cores
    (see `csrc/gla.cu`); the rows of the other requests in `out` (float32 [tokens, H*value_dim]) are left alone.
    `chunks`, `per_request`: the work lists of `StepContext.long_portion_chunks(GLA_CHUNK)`.  With `segments` and
    `segment_requests` (`StepContext.long_portion_segments`) every request's segments run side by side, twice, with a
    pass over their states between: for steps whose few long portions would leave most of the GPU idle."""
    _cuda(qkv, z, state, cu_seqlens, start_pos, slots, chunks, per_request, out, head_decay)
    H, dk, dv = num_heads, key_dim, value_dim
    T = qkv.shape[0]
    _need(gla_chunked_ok(qkv, dk), "gla_chunked takes bfloat16 operands with key channels a multiple of 16 up to 256")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= H * (2 * dk + dv), "qkv must hold the columns q | k | v")
    _gla_decay_checks(z, head_decay, T, H, dk)
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dk, dv),
          "the state must be contiguous float32 [slots, H, key_dim, value_dim]")
    _need(out.dtype == torch.float32 and out.shape == (T, H * dv) and out.is_contiguous(), "out must be contiguous float32 [tokens, H*value_dim]")
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots"), (chunks, "chunks"), (per_request, "per_request")):
        _i32(t, name)
    q_in = torch.empty((T, H, dk), dtype=torch.bfloat16, device=qkv.device)
    k_end = torch.empty((T, H, dk), dtype=torch.bfloat16, device=qkv.device)
    A = torch.empty((T, H, GLA_CHUNK), dtype=torch.float32, device=qkv.device)
    D = torch.empty((max(num_chunks, 1), H, dk), dtype=torch.float32, device=qkv.device)
    seg_state = seg_decay = None
    n_seg = 0
    if segments is not None:
        _need(segment_requests is not None, "segments come with their per-request list")
        _i32(segments, "segments")
        _i32(segment_requests, "segment_requests")
        n_seg = segments.shape[0]
        seg_state = torch.empty((max(n_seg, 1), H, dk, dv), dtype=torch.float32, device=qkv.device)
        seg_decay = torch.empty((max(n_seg, 1), H, dk), dtype=torch.float32, device=qkv.device)
        per_request, num_long = segment_requests, segment_requests.shape[0]
    item, base = qkv.element_size(), qkv.data_ptr()
    f = _fn("gla", "lb_gla_chunked", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_float, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(base, base + H * dk * item, base + 2 * H * dk * item, qkv.stride(0) if T > 1 else qkv.shape[1], _ptr(z), _ptr(out),
             _ptr(state), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(chunks), num_chunks, _ptr(per_request), num_long,
             _ptr(q_in), _ptr(k_end), _ptr(A), _ptr(D), H, dk, dv, tau, q_scale, _ptr(segments), n_seg, _ptr(seg_state),
             _ptr(seg_decay), _ptr(head_decay), _stream()), "gla_chunked", f"(key_dim {dk}, value_dim {dv})", launches=2 if segments is None else 4)
    return out


GLA_SEGMENT = 16      # chunks per segment of the side-by-side form


def gla_segmented_pays(num_tokens: int, num_long: int, num_heads: int, value_dim: int) -> bool:
    """Should the long portions of a step run as segments side by side?  When one CTA per (request, head, 32 value
    columns) would leave most SMs idle and the portions are long enough to be cut."""
    return num_tokens >= 2 * GLA_SEGMENT * GLA_CHUNK and num_long * num_heads * -(-value_dim // 32) < _SM_COUNT


def gla_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, num_heads: int,
                  sigmoid_gate: bool = False) -> torch.Tensor:
    """RMSNorm of every head's float32 output with one weight [value_dim] for all heads, times silu(gate) (or, with
    `sigmoid_gate`, sigmoid(gate)); the result has the gate's dtype.  `gate` may be a column view of a wider matrix.  With
    `num_heads` 1 it is the gated norm over the whole row."""
    _cuda(o, gate, weight)
    rows, width = o.shape
    dv = width // num_heads
    _need(o.dtype == torch.float32 and o.is_contiguous() and width == num_heads * dv, "o must be contiguous float32 [rows, H*value_dim]")
    _need(gate.shape == o.shape and gate.stride(1) == 1, "gate must match o, unit column stride")
    _need(weight.dtype == torch.float32 and weight.shape == (dv,) and weight.is_contiguous(), "weight must be float32 [value_dim]")
    out = torch.empty((rows, width), dtype=gate.dtype, device=o.device)
    f = _fn("gla", "lb_gla_norm_gate", [c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(o), _ptr(gate), gate.stride(0) if rows > 1 else gate.shape[1], _ptr(weight), _ptr(out), rows, num_heads, dv,
             eps, int(sigmoid_gate), _code(gate), _stream()), "gla_norm_gate")
    return out


# --------------------------------------------------------------------------- attention over a cache of latents
def latent_prepare(proj: torch.Tensor, num_heads: int, nope_dim: int, rot_dim: int, rank: int, positions: torch.Tensor,
                   slot_mapping: torch.Tensor, cos_sin: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                   c_cache: torch.Tensor, kr_cache: torch.Tensor, write_cache: bool = True, neighbours: bool = False) -> None:
    """proj: [tokens, H*(nope+rot) + rank + rot] = queries | down-projection.  Stores the normalised latent and the
    rotated shared key part at `slot_mapping`, and rotates every head's rotated query part in place.  `neighbours`: the
    rotation pairs column 2i with 2i + 1 (else i with i + n/2).  Without `write_cache` proj may hold the queries alone
    (`norm_weight` may then be None): nothing but their rotation happens."""
    _cuda(proj, positions, slot_mapping, cos_sin, norm_weight, c_cache, kr_cache)
    T = proj.shape[0]
    q_cols = num_heads * (nope_dim + rot_dim)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and (proj.shape[1] == q_cols + rank + rot_dim or (not write_cache and proj.shape[1] == q_cols)),
          "proj must hold queries | latent | rotated key")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    _need(cos_sin.dtype == torch.float32 and cos_sin.dim() == 2 and cos_sin.is_contiguous(), "cos/sin table must be contiguous float32")
    _need((norm_weight is None and not write_cache) or (norm_weight.dtype == torch.float32 and norm_weight.shape == (rank,)
                                                        and norm_weight.is_contiguous()), "latent norm weight must be float32 [rank]")
    _need(c_cache.is_contiguous() and kr_cache.is_contiguous() and c_cache.dtype == proj.dtype == kr_cache.dtype
          and c_cache.shape[-1] == rank and kr_cache.shape[-1] == rot_dim, "latent caches must be [..., rank] and [..., rot_dim] of the activation dtype")
    f = _fn("attention_latent", "lb_latent_prepare", [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                      c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0) if T > 1 else proj.shape[1], q_cols, num_heads, nope_dim, rot_dim, rank, _ptr(positions),
             _ptr(slot_mapping), _ptr(cos_sin), cos_sin.shape[0], cos_sin.shape[1], _ptr(norm_weight), eps, _ptr(c_cache),
             _ptr(kr_cache), int(write_cache), int(neighbours), T, _code(proj), _stream()), "latent_prepare")


def heads_matmul(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h, :] = a[t, h, :] @ w[h]  with a [tokens, H, K] (any token and head strides, unit stride in K), w
    contiguous [H, K, N]; 32-bit accumulation, result in a's dtype."""
    _cuda(a, w, out)
    T, H, Kd = a.shape
    _need(a.stride(2) == 1 and w.is_contiguous() and w.shape[:2] == (H, Kd) and w.dtype == a.dtype, "heads_matmul wants a [T, H, K] and w [H, K, N]")
    N = w.shape[2]
    if out is None and a.dtype == torch.bfloat16 and T > SKINNY_MAX_ROWS:
        # many rows: the library's batched product over the heads (as `linear` leaves its products of many rows to it);
        # the result is a [T, H, N] view of its [H, T, N] output
        product = lambda: torch.bmm(a.transpose(0, 1), w).transpose(0, 1)
        return PROFILER.timed("library", "bmm", product) if PROFILER.enabled else product()
    if out is None:
        out = torch.empty((T, H, N), dtype=a.dtype, device=a.device)
    _need(out.shape == (T, H, N) and out.stride(2) == 1 and out.dtype == a.dtype, "out must be [T, H, N]")
    f = _fn("attention_latent", "lb_heads_matmul", [c_void_p, c_long, c_long, c_void_p, c_void_p, c_long, c_long, c_int, c_int,
                                                    c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), a.stride(0), a.stride(1), _ptr(w), _ptr(out), out.stride(0), out.stride(1), T, H, Kd, N, _code(a), _stream()),
           "heads_matmul", f"(K {Kd}, N {N})")
    return out


def latent_attention(qa: torch.Tensor, q_rot: torch.Tensor, c_cache: torch.Tensor, kr_cache: torch.Tensor,
                     block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor, scale: float,
                     window: int = 0, token_list: torch.Tensor | None = None, out: torch.Tensor | None = None,
                     sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Softmax attention in the latent space.  qa: [tokens, H, rank] (queries folded through the key expansion);
    q_rot: [tokens, H, rot] (a strided view); caches [pages, page_size, rank] and [pages, page_size, rot].  Token t at
    position p sees keys j of its request with 0 <= p - j < window (0: all).  Returns the weighted sums of the cached
    latents [tokens, H, rank]; with `token_list` only those rows are written.  `sinks` (float32 [H] or None): exp(sinks[h])
    joins head h's softmax denominator, with no key and no value."""
    _cuda(qa, q_rot, c_cache, kr_cache, block_table, token_req, positions, token_list, sinks)
    T, H, rank = qa.shape
    _latent_sinks(sinks, H)
    rot = kr_cache.shape[-1]
    _need(qa.is_contiguous() and q_rot.shape == (T, H, rot) and (rot == 0 or q_rot.stride(2) == 1) and q_rot.dtype == qa.dtype,
          "q_rot must be [tokens, H, rot] with unit stride in its last axis")
    _need(c_cache.dim() == 3 and c_cache.is_contiguous() and kr_cache.is_contiguous() and c_cache.shape[2] == rank
          and c_cache.dtype == qa.dtype == kr_cache.dtype and kr_cache.shape[:2] == c_cache.shape[:2], "latent caches do not fit the queries")
    _i32(block_table, "block_table")
    _i32(token_req, "token_req")
    _i32(positions, "positions")
    n = T
    if token_list is not None:
        _i32(token_list, "token_list")
        n = token_list.numel()
    if out is None:
        out = torch.empty((T, H, rank), dtype=qa.dtype, device=qa.device)
    f = _fn("attention_latent", "lb_latent_attention", [c_void_p, c_void_p, c_long, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                                        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                        c_float, c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(qa), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1), _ptr(c_cache), _ptr(kr_cache), _ptr(block_table),
             block_table.shape[1], _ptr(token_req), _ptr(positions), _ptr(token_list), n, _ptr(out), H, rank, rot,
             c_cache.shape[1], scale, window, _ptr(sinks), _code(qa), _stream()), "latent_attention", f"(rank {rank}, rot {rot})")
    return out


def _latent_sinks(sinks, num_heads: int) -> None:
    _need(sinks is None or (sinks.is_cuda and sinks.dtype == torch.float32 and sinks.shape == (num_heads,) and sinks.is_contiguous()),
          "sinks must be float32 [heads] on the device")


LATENT_MMA = os.environ.get("LOGSSMS_B200_LATENT_MMA", "1") != "0"


def latent_attention_mma_ok(qa: torch.Tensor, rot: int) -> bool:
    """Does the tensor-core form take these sizes (else: `latent_attention`)?"""
    return LATENT_MMA and qa.dtype == torch.bfloat16 and qa.shape[2] % 32 == 0 and qa.shape[2] <= 512 and rot % 16 == 0


def latent_splits(num_blocks: int, num_heads: int, keys: int) -> int:
    """Key ranges per tile so that the grid covers the SMs about twice; a range has at least two 32-key tiles."""
    ctas = max(1, num_blocks * -(-num_heads // 16))
    return max(1, min(2 * _SM_COUNT // ctas, -(-keys // 32) // 2, 64))


def latent_attention_mma(qa: torch.Tensor, q_rot: torch.Tensor, c_cache: torch.Tensor, kr_cache: torch.Tensor,
                         block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor, blocks: torch.Tensor | None,
                         scale: float, window: int = 0, splits: int = 1, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """`latent_attention` on the tensor cores for all tokens of a step.  `blocks`: int32 [n, 2] (first token row, number
    of tokens) of `StepContext.token_blocks(max(1, 16 // H))`: every token of the step in exactly one block; None: every
    token a block of its own (a step of single tokens needs no list)."""
    _cuda(qa, q_rot, c_cache, kr_cache, block_table, token_req, positions, blocks, sinks)
    T, H, rank = qa.shape
    _latent_sinks(sinks, H)
    rot = kr_cache.shape[-1]
    _need(latent_attention_mma_ok(qa, rot), "latent_attention_mma takes bfloat16, rank a multiple of 32 up to 512, rot a multiple of 16")
    _need(qa.stride(2) == 1 and q_rot.shape == (T, H, rot) and (rot == 0 or q_rot.stride(2) == 1) and q_rot.dtype == qa.dtype,
          "qa [tokens, H, rank] and q_rot [tokens, H, rot] must have unit stride in their last axis")
    _need(c_cache.dim() == 3 and c_cache.is_contiguous() and kr_cache.is_contiguous() and c_cache.shape[2] == rank
          and c_cache.dtype == qa.dtype == kr_cache.dtype and kr_cache.shape[:2] == c_cache.shape[:2], "latent caches do not fit the queries")
    for t, name in ((block_table, "block_table"), (token_req, "token_req"), (positions, "positions")):
        _i32(t, name)
    if blocks is not None:
        _i32(blocks, "blocks")
    out = torch.empty((T, H, rank), dtype=qa.dtype, device=qa.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((T * H, splits, rank), dtype=torch.float32, device=qa.device)
        part_ml = torch.empty((T * H, splits, 2), dtype=torch.float32, device=qa.device)
    f = _fn("attention_latent", "lb_latent_attention_mma", [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                                            c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                            c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(qa), qa.stride(0), qa.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1), _ptr(c_cache), _ptr(kr_cache), _ptr(block_table),
             block_table.shape[1], _ptr(token_req), _ptr(positions), _ptr(blocks), T if blocks is None else blocks.shape[0], _ptr(out), _ptr(part_o),
             _ptr(part_ml), T, H, rank, rot, c_cache.shape[1], scale, window, splits, _ptr(sinks), _stream()), "latent_attention_mma",
           f"(rank {rank}, rot {rot})", launches=2 if splits > 1 else 1)
    return out


def latent_wide_rows(num_tokens: int, num_heads: int, rank: int) -> int:
    """Rows of a CTA of `latent_attention_wide`: 64 (a warp per tile of 16 rows) where the rank fits a warp's registers,
    else 32 (two warps per row tile, each with half of the output columns).  (32 rows for more, lighter CTAs on a short
    prompt was measured too: a 2,048-token prompt of 8 heads at rank 256, 256 CTAs of 64 rows against 512 of 32: 0.288
    against 0.298 ms for the mixer.)"""
    return 64 if rank <= 256 else 32


def latent_wide_tokens(num_heads: int, rows: int) -> int:
    """Most neighbouring tokens of one request in a block of `latent_attention_wide` with `rows` rows per CTA (its work
    list: `StepContext.token_blocks` of this many)."""
    return rows // 16 if num_heads >= 16 else rows // num_heads


def latent_attention_wide(qa: torch.Tensor, q_rot: torch.Tensor, c_cache: torch.Tensor, kr_cache: torch.Tensor,
                          block_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor, blocks: torch.Tensor,
                          scale: float, window: int = 0, rows: int = 32, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """`latent_attention_mma` for steps with prompt portions: a CTA holds `rows` (32 or 64) (token, head) rows of
    neighbouring tokens, so a staged key tile serves more rows, and a warp keeps its rows' weights in registers.
    `blocks`: `StepContext.token_blocks(latent_wide_tokens(H, rows))`."""
    _cuda(qa, q_rot, c_cache, kr_cache, block_table, token_req, positions, blocks, sinks)
    T, H, rank = qa.shape
    _latent_sinks(sinks, H)
    rot = kr_cache.shape[-1]
    _need(latent_attention_mma_ok(qa, rot), "latent_attention_wide takes bfloat16, rank a multiple of 32 up to 512, rot a multiple of 16")
    _need(qa.stride(2) == 1 and q_rot.shape == (T, H, rot) and (rot == 0 or q_rot.stride(2) == 1) and q_rot.dtype == qa.dtype,
          "qa [tokens, H, rank] and q_rot [tokens, H, rot] must have unit stride in their last axis")
    _need(c_cache.dim() == 3 and c_cache.is_contiguous() and kr_cache.is_contiguous() and c_cache.shape[2] == rank
          and c_cache.dtype == qa.dtype == kr_cache.dtype and kr_cache.shape[:2] == c_cache.shape[:2], "latent caches do not fit the queries")
    for t, name in ((block_table, "block_table"), (token_req, "token_req"), (positions, "positions"), (blocks, "blocks")):
        _i32(t, name)
    out = torch.empty((T, H, rank), dtype=qa.dtype, device=qa.device)
    f = _fn("attention_latent", "lb_latent_attention_wide", [c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_void_p,
                                                             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                             c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(qa), qa.stride(0), qa.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1), _ptr(c_cache), _ptr(kr_cache),
             _ptr(block_table), block_table.shape[1], _ptr(token_req), _ptr(positions), _ptr(blocks), blocks.shape[0], _ptr(out),
             H, rank, rot, c_cache.shape[1], scale, window, rows, _ptr(sinks), _stream()), "latent_attention_wide", f"(rank {rank}, rot {rot}, rows {rows})")
    return out


# --------------------------------------------------------------------------- routed feed-forward
def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor | None, num_experts: int, top: int, groups: int,
              keep: int, scale: float, sigmoid_scores: bool = False, bias: torch.Tensor | None = None, chosen_softmax: bool = False):
    """(dense weights float32 [T, n], chosen int32 [T, top], their weights float32 [T, top], identity weight float32 [T]):
    see `csrc/moe.cu`.  `w_router` float32 [n, width]; outputs num_experts .. n-1 are identity experts.  Scores are the
    softmax over all outputs, or with `sigmoid_scores` the sigmoid of each; `correction` (may be None) moves the choice only.
    With `chosen_softmax` the logits themselves are ranked and the weights are the softmax over the chosen logits alone.
    `bias` (float32 [n], may be None) is added to the logits."""
    _cuda(h, w_router, correction, bias)
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (w_router.shape[0],) and bias.is_contiguous()), "router bias float32 [n]")
    _need(not (chosen_softmax and (sigmoid_scores or correction is not None)), "the softmax over the chosen logits takes no other score")
    T, width = h.shape
    n = w_router.shape[0]
    _need(h.is_contiguous() and w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == width
          and (correction is None or (correction.dtype == torch.float32 and correction.shape == (n,))),
          "router weight float32 [n, width], correction float32 [n]")
    dense = torch.empty((T, n), dtype=torch.float32, device=h.device)
    chosen = torch.empty((T, top), dtype=torch.int32, device=h.device)
    chosen_w = torch.empty((T, top), dtype=torch.float32, device=h.device)
    idw = torch.empty((T,), dtype=torch.float32, device=h.device)
    f = _fn("moe", "lb_moe_route", [c_void_p] * 7 + [c_int] * 7 + [c_float, c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(w_router), _ptr(correction), _ptr(dense), _ptr(chosen), _ptr(chosen_w), _ptr(idw), T, width, n,
             num_experts, top, groups, keep, scale, 2 if chosen_softmax else int(sigmoid_scores), _ptr(bias), _code(h), _stream()), "moe_route",
           f"({n} outputs, top {top}, {groups} groups)")
    return dense, chosen, chosen_w, idw


EXPERT_MODES = {"clamped": 0, "silu_input": 1, "silu": 2, "gelu_tanh": 3}


def moe_activation(gate_up: torch.Tensor, dense: torch.Tensor | None, num_experts: int, limit: float, act_alpha: float,
                   mode: str = "clamped", out: torch.Tensor | None = None) -> torch.Tensor:
    """gate_up: [T, experts * 2 * ff] (per expert gate | up); returns [T, experts * ff] with every expert's gated
    activation and the token's weight for that expert (0 where the expert was not chosen).  Mode "clamped": weight *
    g~ sigmoid(act_alpha g~) (u~ + 1) with gate and up clamped at `limit`; "silu_input": silu(w g) * (w u), the expert on
    an input that was multiplied by the weight; "silu", "gelu_tanh": weight * act(g) * u.  `dense` None: every weight is 1 (a
    dense gated layer: one expert).  `gate_up` and `out` ([T, experts * ff]) may be column views of wider matrices."""
    _cuda(gate_up, dense, out)
    T = gate_up.shape[0]
    ff = gate_up.shape[1] // (2 * num_experts)
    _need(gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.shape[1] == 2 * num_experts * ff, "gate_up must be [T, experts*2*ff], unit column stride")
    _need(dense is None or (dense.dtype == torch.float32 and dense.is_contiguous() and dense.shape[0] == T and dense.shape[1] >= num_experts),
          "dense weights float32 [T, n]")
    y = out if out is not None else torch.empty((T, num_experts * ff), dtype=gate_up.dtype, device=gate_up.device)
    _need(y.shape == (T, num_experts * ff) and y.dtype == gate_up.dtype and y.stride(1) == 1, "out must be [T, experts*ff] of gate_up's dtype")
    f = _fn("moe", "lb_moe_activation", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_long, c_long,
                                         c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(dense), _ptr(y), T, num_experts, ff, 0 if dense is None else dense.shape[1], limit, act_alpha,
             EXPERT_MODES[mode], gate_up.stride(0) if T > 1 else max(gate_up.stride(0), gate_up.shape[1]),
             y.stride(0) if T > 1 else max(y.stride(0), y.shape[1]), _code(gate_up), _stream()), "moe_activation")
    return y


def silu_columns(x: torch.Tensor, cols: int, scale: torch.Tensor | None = None) -> torch.Tensor:
    """silu over the first `cols` columns of every row of x, in place; with `scale` (float32 [cols]) of x * scale."""
    _cuda(x, scale)
    _need(x.dim() == 2 and x.stride(1) == 1 and 0 <= cols <= x.shape[1], "silu_columns wants rows with unit column stride")
    _need(scale is None or (scale.dtype == torch.float32 and scale.shape == (cols,) and scale.is_contiguous()), "scale must be float32 [cols]")
    f = _fn("moe", "lb_silu_columns", [c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0) if x.shape[0] > 1 else x.shape[1], x.shape[0], cols, _ptr(scale), _code(x), _stream()), "silu_columns")
    return x


def moe_add_identity(out: torch.Tensor, h: torch.Tensor, id_weight: torch.Tensor) -> torch.Tensor:
    """out += id_weight[t] * h, in place."""
    _cuda(out, h, id_weight)
    _need(out.is_contiguous() and h.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype and id_weight.dtype == torch.float32,
          "moe_add_identity wants matching contiguous rows and float32 weights")
    f = _fn("moe", "lb_moe_add_identity", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(h), _ptr(id_weight), out.shape[0], out.shape[1], _code(out), _stream()), "moe_add_identity")
    return out


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    _cuda(x)
    _need(x.is_contiguous(), "gelu_tanh wants a contiguous tensor")
    out = torch.empty_like(x)
    f = _fn("moe", "lb_gelu_tanh", [c_void_p, c_void_p, c_long, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(out), x.numel(), _code(x), _stream()), "gelu_tanh")
    return out


# --------------------------------------------------------------------------- pre-norm layers on a 32-bit stream
NORM_KINDS = {"layernorm": 0, "rmsnorm": 1, "none": 2}


def embed_norm(table: torch.Tensor, ids: torch.Tensor, weight: torch.Tensor, eps: float, kind: str,
               bad_ids: torch.Tensor | None = None) -> torch.Tensor:
    """float32 [tokens, width]: norm(table[id]) * weight, the first value of a 32-bit stream."""
    _cuda(table, ids, weight)
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous [vocab, hidden] matrix")
    V, H = table.shape
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(), "norm weight must be float32 [width]")
    out = torch.empty((ids.numel(), H), dtype=torch.float32, device=table.device)
    f = _fn("stream_layer", "lb_embed_norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p,
                                              c_int, c_void_p])
    _check(f(_ptr(out), _ptr(table), _ptr(ids), _ptr(weight), eps, ids.numel(), H, V, NORM_KINDS[kind], _ptr(bad_ids), _code(table),
             _stream()), "embed_norm", f"(width {H})")
    return out


def stream_add_norm(x: torch.Tensor, y: torch.Tensor | None, channel_scale: torch.Tensor | None, weight: torch.Tensor | None,
                    eps: float, kind: str, act_dtype: torch.dtype, unit_eps: float | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """x += channel_scale * y in place (x: the float32 stream; y: activations or None; with `unit_eps` y is first divided
    by sqrt(mean(y^2) + unit_eps)), then norm(x) * weight rounded to `act_dtype` (None without a weight; kind "none": x
    rounded).  Returns (x, normed)."""
    _cuda(x, y, channel_scale, weight)
    rows, H = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "the stream must be contiguous float32")
    _need(y is None or (y.shape == x.shape and y.dtype == act_dtype and y.is_contiguous()), "y must match the stream's shape")
    for v, name in ((channel_scale, "channel_scale"), (weight, "weight")):
        _need(v is None or (v.dtype == torch.float32 and v.shape == (H,) and v.is_contiguous()), f"{name} must be float32 [width]")
    _need(y is not None or weight is not None or kind == "none", "nothing to do")
    h = None if (weight is None and kind != "none") else torch.empty((rows, H), dtype=act_dtype, device=x.device)
    f = _fn("stream_layer", "lb_stream_add_norm", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                                   c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(y), _ptr(channel_scale), -1.0 if unit_eps is None else unit_eps, _ptr(weight), eps,
             _ptr(x) if y is not None else None, _ptr(h), rows, H, NORM_KINDS[kind], _DTYPE_CODE[act_dtype], _stream()),
           "stream_add_norm", f"(width {H})")
    return x, h


def side_gate(z: torch.Tensor, ids: torch.Tensor, side_table: torch.Tensor, offset: int) -> torch.Tensor:
    """gelu_tanh(z) * e for z [tokens, dim], e the columns [offset, offset + dim) of side_table[id]."""
    _cuda(z, ids, side_table)
    _i32(ids, "ids")
    _need(z.dim() == 2 and z.is_contiguous() and side_table.dim() == 2 and side_table.is_contiguous() and side_table.dtype == z.dtype,
          "side_gate wants contiguous z [tokens, dim] and a table of its dtype")
    a = torch.empty_like(z)
    f = _fn("stream_layer", "lb_side_gate", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(z), _ptr(ids), _ptr(side_table), side_table.shape[1], offset, side_table.shape[0], _ptr(a), z.shape[0], z.shape[1],
             _code(z), _stream()), "side_gate")
    return a


def stream_side(x: torch.Tensor, y: torch.Tensor | None, channel_scale: torch.Tensor | None, ids: torch.Tensor,
                side_table: torch.Tensor, offset: int, gate_w: torch.Tensor, proj_t: torch.Tensor, side_w: torch.Tensor,
                side_eps: float, next_weight: torch.Tensor | None, next_eps: float, next_kind: str,
                act_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor | None]:
    """x += channel_scale * y, then the token's side input x += RMSNorm(proj (gelu_tanh(gate_w x) * e)) * side_w with e the
    columns [offset, offset + dim) of side_table[id], all in place on the float32 stream; with `next_weight` also the
    norm that reads the stream next, rounded to `act_dtype`.  `proj_t` is the projection transposed, [dim, width].
    Returns (x, normed or None)."""
    _cuda(x, y, channel_scale, ids, side_table, gate_w, proj_t, side_w, next_weight)
    _i32(ids, "ids")
    rows, H = x.shape
    dim = gate_w.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "the stream must be contiguous float32")
    _need(y is None or (y.shape == x.shape and y.dtype == act_dtype and y.is_contiguous()), "y must match the stream's shape")
    _need(gate_w.shape == (dim, H) and proj_t.shape == (dim, H) and gate_w.is_contiguous() and proj_t.is_contiguous()
          and gate_w.dtype == proj_t.dtype == side_table.dtype == act_dtype and side_table.dim() == 2 and side_table.is_contiguous(),
          "side input wants gate [dim, width], the projection transposed [dim, width] and a [vocab, columns] table in the activation dtype")
    for v, name in ((channel_scale, "channel_scale"), (side_w, "side norm weight"), (next_weight, "next norm weight")):
        _need(v is None or (v.dtype == torch.float32 and v.shape == (H,) and v.is_contiguous()), f"{name} must be float32 [width]")
    h = None if next_weight is None else torch.empty((rows, H), dtype=act_dtype, device=x.device)
    f = _fn("stream_layer", "lb_stream_side", [c_void_p] * 5 + [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int,
                                               c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(y), _ptr(channel_scale), _ptr(ids), _ptr(side_table), side_table.shape[1], offset, side_table.shape[0],
             _ptr(gate_w), _ptr(proj_t), _ptr(side_w), side_eps, dim, _ptr(next_weight), next_eps, NORM_KINDS[next_kind], _ptr(x),
             _ptr(h), rows, H, _DTYPE_CODE[act_dtype], _stream()), "stream_side", f"(width {H}, side {dim})")
    return x, h


# --------------------------------------------------------------------------- minGRU
_mingru_chunk = None


def mingru_chunk() -> int:
    """Tokens per chunk of the chunked form (the kernels' constant)."""
    global _mingru_chunk
    if _mingru_chunk is None:
        _mingru_chunk = int(_fn("mingru", "lb_mingru_chunk", [])())
    return _mingru_chunk


def _mingru_checks(proj, bias_z, bias_x, state, W):
    _cuda(proj, bias_z, bias_x, state)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[1] == 3 * W, "proj must be [tokens, 3 * width] with unit column stride")
    for b in (bias_z, bias_x):
        _need(b.dtype == torch.float32 and b.shape == (W,) and b.is_contiguous(), "biases must be float32 [width]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == W and state.is_contiguous(),
          "the state must be contiguous float32 [slots, width]")


def mingru_scan(proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                start_pos: torch.Tensor, slots: torch.Tensor, num_requests: int, width: int,
                request_list: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Token by token S <- (1 - z) S + z c over every (listed) request's tokens; returns S * silu(gate) [tokens, width]
    in proj's dtype.  proj: [tokens, 3 * width] = z | candidate | gate products; state float32 [slots, width]."""
    _mingru_checks(proj, bias_z, bias_x, state, width)
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, name)
    if out is None:
        out = torch.empty((proj.shape[0], width), dtype=proj.dtype, device=proj.device)
    n = num_requests if request_list is None else request_list.numel()
    f = _fn("mingru", "lb_mingru_scan", [c_void_p, c_long] + [c_void_p] * 8 + [c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), _ptr(bias_z), _ptr(bias_x), _ptr(state), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots),
             _ptr(request_list), _ptr(out), n, width, _code(proj), _stream()), "mingru_scan", f"(width {width})")
    return out


def mingru_chunked(proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                   start_pos: torch.Tensor, slots: torch.Tensor, chunks: torch.Tensor, num_chunks: int, per_request: torch.Tensor,
                   num_long: int, num_requests: int, width: int, out: torch.Tensor) -> torch.Tensor:
    """The same recurrence over the long portions' chunks side by side (work lists of `StepContext.long_portion_chunks`
    with chunks of `mingru_chunk()` tokens): three launches.  Writes the rows of the long portions into `out`."""
    _mingru_checks(proj, bias_z, bias_x, state, width)
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots"), (chunks, "chunks"), (per_request, "per_request")):
        _i32(t, name)
    fold = torch.empty((2, num_chunks, width), dtype=torch.float32, device=proj.device)
    new_state = torch.empty((num_requests, width), dtype=torch.float32, device=proj.device)
    f = _fn("mingru", "lb_mingru_chunked", [c_void_p, c_long] + [c_void_p] * 7 + [c_int, c_void_p, c_int] + [c_void_p] * 4 + [c_int, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), _ptr(bias_z), _ptr(bias_x), _ptr(state), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots),
             _ptr(chunks), num_chunks, _ptr(per_request), num_long, _ptr(fold[0]), _ptr(fold[1]), _ptr(new_state), _ptr(out), width,
             _code(proj), _stream()), "mingru_chunked", f"(width {width})", launches=3)
    return out


# --------------------------------------------------------------------------- attention over a window and pooled blocks
def pooled_prepare(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, positions: torch.Tensor,
                   slot_mapping: torch.Tensor, qk_table: torch.Tensor, v_table: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, write_kv: bool = True) -> torch.Tensor:
    """Rotated queries [tokens, heads, head_dim]; rotated keys and values go to the caches at the tokens' slots.  qkv:
    [tokens, heads*head_dim + kv_heads*head_dim + kv_heads*value_dim].  Tables: float32 [positions, n] (cos | sin of n/2
    neighbouring pairs); n = 0: no rotation."""
    _cuda(qkv, positions, slot_mapping, qk_table, v_table, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slot_mapping, "slot_mapping")
    T = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim,
          "qkv must be [tokens, q | k | v] with unit column stride")
    _need(k_cache.dtype == v_cache.dtype == qkv.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
          and k_cache.shape[2:] == (num_kv_heads, head_dim) and v_cache.shape[2:] == (num_kv_heads, value_dim), "caches must be [pages, page, kv_heads, dim]")
    for tb in (qk_table, v_table):
        _need(tb.dtype == torch.float32 and tb.dim() == 2 and tb.is_contiguous(), "rotation tables must be contiguous float32")
    rows = max(qk_table.shape[0] if qk_table.shape[1] else 0, v_table.shape[0] if v_table.shape[1] else 0, 1)
    _need((qk_table.shape[1] == 0 or qk_table.shape[0] == rows) and (v_table.shape[1] == 0 or v_table.shape[0] == rows),
          "both rotation tables must have a row per position")
    q = torch.empty((T, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    f = _fn("attention_pooled", "lb_pooled_prepare", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                      c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(slot_mapping), _ptr(qk_table), qk_table.shape[1], _ptr(v_table),
             v_table.shape[1], rows, _ptr(q), _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim, value_dim,
             int(write_kv), _code(qkv), _stream()), "pooled_prepare")
    return q


def normed_prepare(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, positions: torch.Tensor,
                   slot_mapping: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, temp_coef: float,
                   temp_every: int, k_cache: torch.Tensor, v_cache: torch.Tensor, write_kv: bool = True) -> torch.Tensor:
    """Queries [tokens, heads, head_dim], RMS-normed per head over the head's columns with `q_weight` [head_dim] and times
    1 + temp_coef * ln(floor((position + 1) / temp_every) + 1) (`temp_every` 0: times 1); keys normed the same way with
    `k_weight`, and the values as they are, go to the caches at the tokens' slots.  Norm and temperature are 32-bit."""
    _cuda(qkv, positions, slot_mapping, q_weight, k_weight, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slot_mapping, "slot_mapping")
    T = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim,
          "qkv must be [tokens, q | k | v] with unit column stride")
    _need(k_cache.dtype == v_cache.dtype == qkv.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
          and k_cache.shape[2:] == (num_kv_heads, head_dim) and v_cache.shape[2:] == (num_kv_heads, value_dim), "caches must be [pages, page, kv_heads, dim]")
    for w in (q_weight, k_weight):
        _need(w.dtype == torch.float32 and w.shape == (head_dim,) and w.is_contiguous(), "norm weights must be float32 [head_dim]")
    q = torch.empty((T, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    f = _fn("attention_pooled", "lb_normed_prepare", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_int,
                                                      c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p])
    _check(f(_ptr(qkv), qkv.stride(0) if T > 1 else qkv.shape[1], _ptr(positions), _ptr(slot_mapping), _ptr(q_weight), _ptr(k_weight), eps,
             temp_coef, temp_every, _ptr(q), _ptr(k_cache), _ptr(v_cache), T, num_heads, num_kv_heads, head_dim, value_dim,
             int(write_kv), _code(qkv), _stream()), "normed_prepare")
    return q


def rownorm_prepare(qk: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                    slot_mapping: torch.Tensor, table: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, write_kv: bool = True) -> torch.Tensor:
    """Queries [tokens, heads, head_dim] from qk = [tokens, q | k]: q and k are each RMS-normed over their WHOLE row (all
    heads at once) with a weight per column of the row (`q_weight` [heads*head_dim], `k_weight` [kv_heads*head_dim]), then
    rotated over neighbouring pairs of every head's first `table.shape[1]` columns (table: float32 [positions, n], cos | sin
    of n/2 pairs; n = 0: no rotation).  The normed, rotated keys go to `k_cache` at the tokens' slots, the keys as they
    came in go to `v_cache` (the values of this attention are its un-normed keys).  Norms and rotation are 32-bit."""
    _cuda(qk, positions, slot_mapping, table, q_weight, k_weight, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slot_mapping, "slot_mapping")
    T = qk.shape[0]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    _need(qk.dim() == 2 and qk.stride(1) == 1 and qk.shape[1] == nq + nk, "qk must be [tokens, q | k] with unit column stride")
    _need(k_cache.dtype == v_cache.dtype == qk.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
          and k_cache.shape[2:] == (num_kv_heads, head_dim) and v_cache.shape[2:] == (num_kv_heads, head_dim),
          "caches must be [pages, page, kv_heads, head_dim], keys and values alike")
    _need(q_weight.dtype == torch.float32 and q_weight.shape == (nq,) and q_weight.is_contiguous() and k_weight.dtype == torch.float32
          and k_weight.shape == (nk,) and k_weight.is_contiguous(), "norm weights must be float32 over the whole q and k rows")
    _need(table.dtype == torch.float32 and table.dim() == 2 and table.is_contiguous(), "the rotation table must be contiguous float32")
    q = torch.empty((T, num_heads, head_dim), dtype=qk.dtype, device=qk.device)
    f = _fn("attention_pooled", "lb_rownorm_prepare", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                       c_float, c_void_p, c_void_p, c_void_p] + [c_int] * 6 + [c_void_p])
    _check(f(_ptr(qk), qk.stride(0) if T > 1 else qk.shape[1], _ptr(positions), _ptr(slot_mapping), _ptr(table), table.shape[1],
             max(table.shape[0], 1), _ptr(q_weight), _ptr(k_weight), eps, _ptr(q), _ptr(k_cache), _ptr(v_cache), T, num_heads,
             num_kv_heads, head_dim, int(write_kv), _code(qk), _stream()), "rownorm_prepare")
    return q


def head_gate(o: torch.Tensor, gate: torch.Tensor, num_heads: int) -> torch.Tensor:
    """o [tokens, heads * width] (contiguous) times sigmoid(gate[t, h]) per token and head, in place.  gate: [tokens, heads]
    logits in float32 or o's dtype (a column view is fine)."""
    _cuda(o, gate)
    T = o.shape[0]
    _need(o.dim() == 2 and o.is_contiguous() and o.shape[1] % num_heads == 0, "o must be contiguous [tokens, heads * width]")
    _need(gate.shape == (T, num_heads) and gate.stride(1) == 1 and gate.dtype in (torch.float32, o.dtype),
          "gate must be [tokens, heads] in float32 or the activation dtype")
    f = _fn("attention_pooled", "lb_head_gate", [c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(o), _ptr(gate), gate.stride(0) if T > 1 else max(gate.stride(0), num_heads), int(gate.dtype == torch.float32), T,
             num_heads, o.shape[1] // num_heads, _code(o), _stream()), "head_gate")
    return o


def pooled_blocks(k_cache: torch.Tensor, v_cache: torch.Tensor, kp_cache: torch.Tensor, vp_cache: torch.Tensor,
                  positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, pooled_slots: torch.Tensor,
                  pool: int) -> None:
    """Every token of the step that ends a block of `pool` tokens writes the means of the block's cached keys and values
    to the block's entry (`pooled_slots[t]`) of the pooled caches."""
    _cuda(k_cache, v_cache, kp_cache, vp_cache, positions, token_req, block_table, pooled_slots)
    for t, name in ((positions, "positions"), (token_req, "token_req"), (block_table, "block_table"), (pooled_slots, "pooled_slots")):
        _i32(t, name)
    _need(kp_cache.shape[2:] == k_cache.shape[2:] and vp_cache.shape[2:] == v_cache.shape[2:] and kp_cache.dtype == k_cache.dtype
          and kp_cache.is_contiguous() and vp_cache.is_contiguous(), "pooled caches must have the token caches' entry shapes")
    G, dim, vdim = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    f = _fn("attention_pooled", "lb_pooled_blocks", [c_void_p] * 7 + [c_int, c_void_p] + [c_int] * 7 + [c_void_p])
    _check(f(_ptr(k_cache), _ptr(v_cache), _ptr(kp_cache), _ptr(vp_cache), _ptr(positions), _ptr(token_req), _ptr(block_table),
             block_table.shape[1], _ptr(pooled_slots), positions.numel(), G, dim, vdim, k_cache.shape[1], pool, _code(k_cache), _stream()),
           "pooled_blocks")


def _width(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.shape[1]


def _rows(t: torch.Tensor | None) -> int:
    return 1 if t is None else max(t.shape[0], 1)


def _score_extras(num_heads: int, pool: int, pooled_table, slopes, sinks) -> None:
    """Checks of the options that the pooled-attention kernels share.  `slopes[h] * (i - j)` is taken off the scaled score of
    query i (head h) and token j; `exp(sinks[h])` joins the softmax's denominator with no key and no value."""
    _need(pool >= 0 and (pool == 0 or pooled_table is not None), "pooled blocks need their caches and table (pool 0: none)")
    for t, name in ((slopes, "slopes"), (sinks, "sinks")):
        _need(t is None or (t.is_cuda and t.dtype == torch.float32 and t.shape == (num_heads,) and t.is_contiguous()),
              f"{name} must be float32 [heads] on the device")


def pooled_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kp_cache: torch.Tensor, vp_cache: torch.Tensor,
                     block_table: torch.Tensor, pooled_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                     v_table: torch.Tensor, scale: float, window: int, pool: int, token_list: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """[tokens, heads * value_dim]: attention of every (listed) token over its window's tokens and the pooled blocks
    behind it, a warp per (token, head), everything in float32; the summed values are turned back by the query's position.
    `pool` 0: no blocks (the pooled caches and their table may be None); `v_table` None: values are not rotated; `slopes`,
    `sinks` (float32 per query head, may be None): see `_score_extras`."""
    _cuda(q, k_cache, v_cache, kp_cache, vp_cache, block_table, pooled_table, token_req, positions, v_table, token_list)
    for t, name in ((block_table, "block_table"), (pooled_table, "pooled_table"), (token_req, "token_req"), (positions, "positions")):
        if t is not None:
            _i32(t, name)
    T, H, dim = q.shape
    _score_extras(H, pool, pooled_table, slopes, sinks)
    G, vdim = v_cache.shape[2], v_cache.shape[3]
    _need(q.is_contiguous() and q.dtype == k_cache.dtype, "queries must be contiguous [tokens, heads, dim] in the cache's dtype")
    if out is None:
        out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    n = T if token_list is None else token_list.numel()
    f = _fn("attention_pooled", "lb_pooled_attention", [c_void_p] * 6 + [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                        c_void_p, c_int, c_int, c_void_p] + [c_int] * 5
            + [c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(kp_cache), _ptr(vp_cache), _ptr(block_table), block_table.shape[1],
             _ptr(pooled_table), _width(pooled_table), _ptr(token_req), _ptr(positions), _ptr(token_list), n, _ptr(v_table),
             _width(v_table), _rows(v_table), _ptr(out), H, G, dim, vdim, k_cache.shape[1], scale, window, pool, _ptr(slopes),
             _ptr(sinks), _code(q), _stream()), "pooled_attention", f"(dim {dim}, value dim {vdim})")
    return out


POOLED_TILE = os.environ.get("LOGSSMS_B200_POOLED_TILE", "1") != "0"
_pooled_tile_q = None


def pooled_attention_tile_q() -> int:
    """Query tokens per CTA of the tensor-core form (the kernel's constant)."""
    global _pooled_tile_q
    if _pooled_tile_q is None:
        _pooled_tile_q = int(_fn("attention_pooled", "lb_pooled_attention_tile_q", [])())
    return _pooled_tile_q


def pooled_attention_tile_ok(q: torch.Tensor, v_cache: torch.Tensor) -> bool:
    """Does the tensor-core form take these sizes?  bfloat16, a head size that is a multiple of 16 and a value head size
    that is a multiple of 8, both up to 128."""
    dim, vdim = q.shape[2], v_cache.shape[3]
    return POOLED_TILE and q.dtype == torch.bfloat16 and dim % 16 == 0 and dim <= 128 and vdim % 8 == 0 and vdim <= 128


def pooled_tile_splits(num_tiles: int, num_heads: int) -> int:
    """CTAs that share a run's chunks of keys in the tensor-core form: 1 where the runs fill the GPU twice by themselves,
    up to 4 for a lone prompt."""
    return max(1, min(4, -(-2 * _SM_COUNT // max(num_tiles * num_heads, 1))))


def pooled_attention_tile(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kp_cache: torch.Tensor, vp_cache: torch.Tensor,
                          block_table: torch.Tensor, pooled_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
                          positions: torch.Tensor, tiles: torch.Tensor, v_table: torch.Tensor, scale: float, window: int, pool: int,
                          out: torch.Tensor, splits: int = 1, slopes: torch.Tensor | None = None,
                          sinks: torch.Tensor | None = None) -> torch.Tensor:
    """The same attention for the long portions' runs of `pooled_attention_tile_q()` tokens (work list of
    `StepContext.long_portion_tiles`) on the tensor cores; writes those tokens' rows of `out` [tokens, heads * value_dim].
    With `splits` > 1 that many CTAs share a run's keys and a merge follows, which also writes the rows that no run covers
    (with nothing of meaning: the caller fills them afterwards)."""
    _cuda(q, k_cache, v_cache, kp_cache, vp_cache, block_table, pooled_table, cu_seqlens, start_pos, positions, tiles, v_table, out)
    for t, name in ((block_table, "block_table"), (pooled_table, "pooled_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"),
                    (tiles, "tiles"), (positions, "positions")):
        if t is not None:
            _i32(t, name)
    T, H, dim = q.shape
    _score_extras(H, pool, pooled_table, slopes, sinks)
    G, vdim = v_cache.shape[2], v_cache.shape[3]
    _need(q.is_contiguous() and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
          and out.is_contiguous() and out.shape == (T, H * vdim), "the tensor-core form takes contiguous bfloat16 tensors")
    partial = torch.empty((T, H, splits, vdim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    f = _fn("attention_pooled", "lb_pooled_attention_tile", [c_void_p] * 6 + [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                             c_void_p, c_int, c_void_p, c_int, c_int, c_void_p] + [c_int] * 5
            + [c_float, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(kp_cache), _ptr(vp_cache), _ptr(block_table), block_table.shape[1],
             _ptr(pooled_table), _width(pooled_table), _ptr(cu_seqlens), _ptr(start_pos), _ptr(tiles), tiles.shape[0], _ptr(positions), T,
             _ptr(v_table), _width(v_table), _rows(v_table), _ptr(out), H, G, dim, vdim, k_cache.shape[1], scale, window, pool,
             _ptr(partial), splits, _ptr(slopes), _ptr(sinks), _stream()),
           "pooled_attention_tile", f"(dim {dim}, value dim {vdim})", launches=2 if splits > 1 else 1)
    return out


def pooled_attention_split_ok(q: torch.Tensor, v_cache: torch.Tensor) -> bool:
    """Does the form with key ranges take these sizes?  A value head size up to 128, a head size that is a multiple of 4."""
    return q.shape[2] % 4 == 0 and q.shape[2] <= 1024 and v_cache.shape[3] <= 128


def pooled_splits(num_tokens: int, num_kv_heads: int, keys: int) -> int:
    """Key ranges per token so that the CTAs fill the GPU about twice (each takes at least 128 keys)."""
    return max(1, min(-(-keys // 128), -(-2 * _SM_COUNT // max(num_tokens * num_kv_heads, 1)), 64))


def pooled_attention_split(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kp_cache: torch.Tensor, vp_cache: torch.Tensor,
                           block_table: torch.Tensor, pooled_table: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                           v_table: torch.Tensor, scale: float, window: int, pool: int, splits: int,
                           token_list: torch.Tensor | None = None, out: torch.Tensor | None = None,
                           slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """The attention of `pooled_attention` with every token's keys cut into `splits` ranges that run side by side and all
    query heads of a key/value head in one CTA; a merge kernel joins the ranges (two launches)."""
    _cuda(q, k_cache, v_cache, kp_cache, vp_cache, block_table, pooled_table, token_req, positions, v_table, token_list)
    for t, name in ((block_table, "block_table"), (pooled_table, "pooled_table"), (token_req, "token_req"), (positions, "positions")):
        if t is not None:
            _i32(t, name)
    T, H, dim = q.shape
    _score_extras(H, pool, pooled_table, slopes, sinks)
    G, vdim = v_cache.shape[2], v_cache.shape[3]
    _need(q.is_contiguous() and q.dtype == k_cache.dtype, "queries must be contiguous [tokens, heads, dim] in the cache's dtype")
    if out is None:
        out = torch.empty((T, H * vdim), dtype=q.dtype, device=q.device)
    n = T if token_list is None else token_list.numel()
    partial = torch.empty((n, H, splits, vdim + 2), dtype=torch.float32, device=q.device)
    f = _fn("attention_pooled", "lb_pooled_attention_split", [c_void_p] * 6 + [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                              c_void_p, c_int, c_int, c_void_p, c_void_p] + [c_int] * 5
            + [c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(kp_cache), _ptr(vp_cache), _ptr(block_table), block_table.shape[1],
             _ptr(pooled_table), _width(pooled_table), _ptr(token_req), _ptr(positions), _ptr(token_list), n, _ptr(v_table),
             _width(v_table), _rows(v_table), _ptr(partial), _ptr(out), H, G, dim, vdim, k_cache.shape[1], scale, window, pool,
             splits, _ptr(slopes), _ptr(sinks), _code(q), _stream()), "pooled_attention_split", f"(dim {dim}, value dim {vdim}, {splits} ranges)", launches=2)
    return out


# --------------------------------------------------------------------------- gated delta rule
def delta_scan(qkv: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, num_requests: int, num_heads: int,
               num_key_heads: int, key_dim: int, value_dim: int, q_scale: float, unit_eps: float,
               request_list: torch.Tensor | None = None, out: torch.Tensor | None = None, head_decay: bool = False) -> torch.Tensor:
    """Token-by-token gated delta rule per head over every request's tokens (see `csrc/delta.cu`): queries and keys made unit
    vectors (the query times `q_scale`), a decay exp(-exp(A_log) softplus(z + dt_bias)) per key channel, a write gated by
    sigmoid(beta), read-out after the write.  qkv: [tokens, >= 2*Hk*key_dim + H*value_dim] with columns q | k | v first
    (unit column stride; query/key head of value head h is h // (H / Hk)); z: float32 [tokens, H*key_dim]; dt_bias: float32
    [H*key_dim]; A_log: float32 [H]; beta: [tokens, H] logits (float32 or qkv's dtype, a column view allowed); state: float32
    [slots, H, key_dim, value_dim], updated in place.  Returns float32 [tokens, H*value_dim].  `head_decay`: one decay per
    head instead of one per key channel: z is float32 [tokens, H] and dt_bias float32 [H]."""
    _cuda(qkv, z, dt_bias, A_log, beta, state, cu_seqlens, start_pos, slots, request_list)
    H, Hk, dk, dv = num_heads, num_key_heads, key_dim, value_dim
    T = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= 2 * Hk * dk + H * dv, "qkv must hold the columns q | k | v")
    zdim = 1 if head_decay else dk
    _need(z.dtype == torch.float32 and z.shape == (T, H * zdim) and z.is_contiguous(), "z must be contiguous float32 [tokens, H*key_dim] (head_decay: [tokens, H])")
    _need(dt_bias.dtype == torch.float32 and dt_bias.numel() == H * zdim and dt_bias.is_contiguous() and A_log.dtype == torch.float32
          and A_log.shape == (H,) and A_log.is_contiguous(), "dt_bias float32 [H*key_dim] (head_decay: [H]), A_log float32 [H]")
    _need(beta.dim() == 2 and beta.shape == (T, H) and beta.stride(1) == 1 and beta.dtype in (torch.float32, qkv.dtype),
          "beta must be [tokens, H] in float32 or the activation dtype")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dk, dv),
          "the state must be contiguous float32 [slots, H, key_dim, value_dim]")
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, name)
    n = num_requests
    if request_list is not None:
        _i32(request_list, "request_list")
        n = request_list.numel()
    o = out if out is not None else torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    item, base = qkv.element_size(), qkv.data_ptr()
    stride = qkv.stride(0) if T > 1 else qkv.shape[1]
    f = _fn("delta", "lb_delta_scan", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                       c_float, c_float, c_int, c_int, c_void_p])
    _check(f(base, base + Hk * dk * item, base + 2 * Hk * dk * item, stride, _ptr(z), _ptr(dt_bias), _ptr(A_log), _ptr(beta),
             beta.stride(0) if T > 1 else max(beta.stride(0), H), int(beta.dtype == torch.float32), _ptr(o), _ptr(state),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(request_list), n, H, Hk, dk, dv, q_scale, unit_eps, zdim, _code(qkv),
             _stream()), "delta_scan", f"(key_dim {dk}, value_dim {dv})")
    return o


DELTA_MIN_PADDED = 16   # the long portions' kernel pads key channels to a power of two, this at least (kMinPadded of csrc/delta.cu)


def delta_scan_rows_ok(key_dim: int) -> bool:
    """Does the kernel of long portions take this many key channels?"""
    return 0 < key_dim <= 512


def delta_scan_rows(qkv: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
                    cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, num_requests: int, num_heads: int,
                    num_key_heads: int, key_dim: int, value_dim: int, q_scale: float, unit_eps: float,
                    request_list: torch.Tensor | None = None, out: torch.Tensor | None = None, rows_per_thread: int = 0,
                    head_decay: bool = False) -> torch.Tensor:
    """`delta_scan` for portions of many tokens: one launch turns every token's unit vectors, decays and gates into 32-bit
    rows, a second one runs the recurrence of the requests of `request_list` (all, if None) with nothing but the state's
    update in its loop.  Operands and result as `delta_scan`; rows of `out` that belong to other requests are left alone."""
    _cuda(qkv, z, dt_bias, A_log, beta, state, cu_seqlens, start_pos, slots, request_list)
    H, Hk, dk, dv = num_heads, num_key_heads, key_dim, value_dim
    T = qkv.shape[0]
    _need(delta_scan_rows_ok(dk), "delta_scan_rows takes up to 512 key channels")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= 2 * Hk * dk + H * dv, "qkv must hold the columns q | k | v")
    zdim = 1 if head_decay else dk
    _need(z.dtype == torch.float32 and z.shape == (T, H * zdim) and z.is_contiguous(), "z must be contiguous float32 [tokens, H*key_dim] (head_decay: [tokens, H])")
    _need(dt_bias.dtype == torch.float32 and dt_bias.numel() == H * zdim and dt_bias.is_contiguous() and A_log.dtype == torch.float32
          and A_log.shape == (H,) and A_log.is_contiguous(), "dt_bias float32 [H*key_dim] (head_decay: [H]), A_log float32 [H]")
    _need(beta.dim() == 2 and beta.shape == (T, H) and beta.stride(1) == 1 and beta.dtype in (torch.float32, qkv.dtype),
          "beta must be [tokens, H] in float32 or the activation dtype")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dk, dv),
          "the state must be contiguous float32 [slots, H, key_dim, value_dim]")
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, name)
    n = num_requests
    if request_list is not None:
        _i32(request_list, "request_list")
        n = request_list.numel()
    o = out if out is not None else torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    _need(o.dtype == torch.float32 and o.shape == (T, H * dv) and o.is_contiguous(), "out must be contiguous float32 [tokens, H*value_dim]")
    padded = DELTA_MIN_PADDED
    while padded < dk:                               # key channels padded to a power of two
        padded *= 2
    prepared = torch.empty((T, H, 3 * padded + 4), dtype=torch.float32, device=qkv.device)
    values = torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    item, base = qkv.element_size(), qkv.data_ptr()
    stride = qkv.stride(0) if T > 1 else qkv.shape[1]
    f = _fn("delta", "lb_delta_scan_rows", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_long,
                                            c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p])
    _check(f(base, base + Hk * dk * item, base + 2 * Hk * dk * item, stride, _ptr(z), _ptr(dt_bias), _ptr(A_log), _ptr(beta),
             beta.stride(0) if T > 1 else max(beta.stride(0), H), int(beta.dtype == torch.float32), _ptr(prepared), _ptr(values),
             _ptr(o), _ptr(state), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(request_list), n, T, H, Hk, dk, dv, q_scale,
             unit_eps, rows_per_thread, zdim, _code(qkv), _stream()), "delta_scan_rows", f"(key_dim {dk}, value_dim {dv})", launches=2)
    return o


DELTA_CHUNK = 8         # tokens per chunk of the chunked form (kDeltaChunk of csrc/delta.cu)


def delta_scan_chunks_ok(key_dim: int) -> bool:
    """Does the chunked kernel of long portions take this many key channels?"""
    return 0 < key_dim <= 256


def delta_scan_chunks(qkv: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
                      cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, chunks: torch.Tensor, num_chunks: int,
                      per_request: torch.Tensor, num_long: int, num_heads: int, num_key_heads: int, key_dim: int, value_dim: int,
                      q_scale: float, unit_eps: float, out: torch.Tensor | None = None, rows_per_thread: int = 0,
                      head_decay: bool = False) -> torch.Tensor:
    """`delta_scan` for the long portions of a step in chunks of `DELTA_CHUNK` tokens: one launch turns every chunk into a
    32-bit record (unit vectors times the chunk's running decays, the two small triangular matrices between its tokens), a
    second one walks each listed request's chunks with one reduction round per chunk (the 16 sums of a chunk reduced by
    halving over the lanes that share a value column, the writes' sizes by forward substitution across those lanes).  `chunks` int32 [num_chunks, 2] and
    `per_request` int32 [num_long, 3] are the work lists of `StepContext.long_portion_chunks(DELTA_CHUNK)`.  Operands and
    result as `delta_scan`; rows of `out` that belong to other requests are left alone."""
    _cuda(qkv, z, dt_bias, A_log, beta, state, cu_seqlens, start_pos, slots, chunks, per_request)
    H, Hk, dk, dv = num_heads, num_key_heads, key_dim, value_dim
    T = qkv.shape[0]
    _need(delta_scan_chunks_ok(dk), "delta_scan_chunks takes up to 256 key channels")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= 2 * Hk * dk + H * dv, "qkv must hold the columns q | k | v")
    zdim = 1 if head_decay else dk
    _need(z.dtype == torch.float32 and z.shape == (T, H * zdim) and z.is_contiguous(), "z must be contiguous float32 [tokens, H*key_dim] (head_decay: [tokens, H])")
    _need(dt_bias.dtype == torch.float32 and dt_bias.numel() == H * zdim and dt_bias.is_contiguous() and A_log.dtype == torch.float32
          and A_log.shape == (H,) and A_log.is_contiguous(), "dt_bias float32 [H*key_dim] (head_decay: [H]), A_log float32 [H]")
    _need(beta.dim() == 2 and beta.shape == (T, H) and beta.stride(1) == 1 and beta.dtype in (torch.float32, qkv.dtype),
          "beta must be [tokens, H] in float32 or the activation dtype")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dk, dv),
          "the state must be contiguous float32 [slots, H, key_dim, value_dim]")
    for t, name in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots"), (chunks, "chunks"), (per_request, "per_request")):
        _i32(t, name)
    _need(chunks.numel() >= 2 * num_chunks and per_request.numel() >= 3 * num_long, "work lists shorter than their counts")
    o = out if out is not None else torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    _need(o.dtype == torch.float32 and o.shape == (T, H * dv) and o.is_contiguous(), "out must be contiguous float32 [tokens, H*value_dim]")
    padded = 64                                      # 16 or 32 lanes of a warp share a column, 4 or 8 rows each
    while padded < dk:                               # key channels padded to a power of two
        padded *= 2
    C = DELTA_CHUNK
    records = torch.empty((max(num_chunks, 1), H, 3 * C * padded + padded + 2 * C * C + C), dtype=torch.float32, device=qkv.device)
    values = torch.empty((T, H * dv), dtype=torch.float32, device=qkv.device)
    item, base = qkv.element_size(), qkv.data_ptr()
    stride = qkv.stride(0) if T > 1 else qkv.shape[1]
    f = _fn("delta", "lb_delta_scan_chunks", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                              c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p])
    _check(f(base, base + Hk * dk * item, base + 2 * Hk * dk * item, stride, _ptr(z), _ptr(dt_bias), _ptr(A_log), _ptr(beta),
             beta.stride(0) if T > 1 else max(beta.stride(0), H), int(beta.dtype == torch.float32), _ptr(records), _ptr(values),
             _ptr(o), _ptr(state), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(chunks), num_chunks, _ptr(per_request), num_long,
             H, Hk, dk, dv, q_scale, unit_eps, rows_per_thread, zdim, _code(qkv), _stream()), "delta_scan_chunks", f"(key_dim {dk}, value_dim {dv})", launches=2)
    return o


# --------------------------------------------------------------------------- a 32-bit stream whose sublayers all read one norm
def stream_add_many(x: torch.Tensor, addends, weight: torch.Tensor | None, eps: float, kind: str,
                    act_dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor | None]:
    """x += sum of scale * y over `addends` (up to four pairs (y, scale), y activations of the stream's shape) in place on the
    float32 stream, then norm(x) * weight rounded to `act_dtype` (None without a weight; kind "none": x rounded).
    Returns (x, normed)."""
    rows, H = x.shape
    ys = [y for y, _ in addends]
    _cuda(x, weight, *ys)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "the stream must be contiguous float32")
    _need(len(addends) <= 4, "at most four addends join the stream in one kernel")
    for y in ys:
        _need(y.shape == x.shape and y.dtype == act_dtype and y.is_contiguous(), "an addend must match the stream's shape")
    _need(weight is None or (weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous()), "weight must be float32 [width]")
    h = None if (weight is None and kind != "none") else torch.empty((rows, H), dtype=act_dtype, device=x.device)
    if not addends and h is None:
        return x, None
    ptrs = [_ptr(y) for y in ys] + [None] * (4 - len(ys))
    scales = [float(s) for _, s in addends] + [0.0] * (4 - len(ys))
    f = _fn("stream_layer", "lb_stream_add_many", [c_void_p] * 5 + [c_float] * 4 + [c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_int,
                                                   c_int, c_void_p])
    _check(f(_ptr(x), *ptrs, *scales, len(ys), _ptr(weight), eps, _ptr(h), rows, H, NORM_KINDS[kind], _DTYPE_CODE[act_dtype], _stream()),
           "stream_add_many", f"(width {H})")
    return x, h


def stream_pair_rows(x: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
    """[rows, 2 * width] in x0's dtype: the float32 stream x rounded, beside x0."""
    _cuda(x, x0)
    _need(x.dtype == torch.float32 and x.is_contiguous() and x0.is_contiguous() and x0.shape == x.shape, "stream and first rows must match")
    out = torch.empty((x.shape[0], 2 * x.shape[1]), dtype=x0.dtype, device=x.device)
    f = _fn("stream_layer", "lb_stream_pair_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(x0), _ptr(out), x.shape[0], x.shape[1], _code(x0), _stream()), "stream_pair_rows")
    return out
