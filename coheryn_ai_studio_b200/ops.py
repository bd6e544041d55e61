"""Python face of the CUDA kernels: every function takes torch tensors that live on the
GPU, checks them, and launches a kernel of this package's own library on the current
CUDA stream.  There is no other implementation behind these functions: without a GPU
or without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_long, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


class KernelError(RuntimeError):
    pass


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("this engine runs on a CUDA GPU (sm_100a) only; "
                          "torch.cuda.is_available() is False and there is no CPU path")


_core = None
_attn_libs = {}
_recurrent = None
_routed = None


def core():
    global _core
    if _core is None:
        lib = build.core_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        lib.coheryn_argmax_scratch_slots.restype = ctypes.c_long
        lib.coheryn_gemm_tc_workspace_floats.restype = ctypes.c_long
        _core = lib
    return _core


def launch_count() -> int:
    """Kernel launches made through the core library since it was loaded."""
    return int(core().coheryn_launch_count())


def total_launch_count() -> int:
    """Kernel launches made through every library of this package that is loaded."""
    n = launch_count()
    for lib in list(_attn_libs.values()) + list(_maps_libs.values()) + [l for l in (_recurrent, _variants, _routed) if l is not None]:
        n += int(lib.coheryn_launch_count())
    return n


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


try:
    _raw_stream, _current_device = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:          # another torch: the documented, slower way
    _raw_stream = _current_device = None


def _stream():
    """The current CUDA stream of the current device as a pointer (asked on every launch: a few
    microseconds through ``torch.cuda.current_stream``, a tenth of one through the raw call)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(lib, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.coheryn_last_error().decode("utf-8", "replace"))


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                 scale: Optional[float] = None) -> None:
    """out[t] = table[ids[t]] (* scale) as float32.  An id outside the table sets status to 1."""
    _dev(table, ids, out, status)
    _i32(ids, "ids")
    V, H = table.shape
    T = ids.numel()
    assert out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous()
    assert table.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), c_int(T),
                                         c_int(H), c_int(V), _ptr(status), c_float(1.0 if scale is None else scale),
                                         _stream()))


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """src[rows] for a matrix (or a vector) whose rows are contiguous; ``rows`` int32 on the device."""
    _dev(src, rows)
    _i32(rows, "rows")
    R = rows.numel()
    if src.dim() == 1:
        out = torch.empty((R,), dtype=src.dtype, device=src.device)
        row_bytes, stride = src.element_size(), src.stride(0) * src.element_size()
    else:
        assert src.dim() == 2 and src.stride(1) == 1
        out = torch.empty((R, src.shape[1]), dtype=src.dtype, device=src.device)
        row_bytes, stride = src.shape[1] * src.element_size(), src.stride(0) * src.element_size()
    if R:
        lib = core()
        _check(lib, lib.coheryn_gather_rows(_ptr(src), c_long(stride), _ptr(rows), _ptr(out), c_int(R), c_int(row_bytes),
                                            _stream()))
    return out


def scatter_words(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[rows[r]] = src[r] for vectors of 32-bit elements."""
    _dev(src, rows, out)
    _i32(rows, "rows")
    assert src.element_size() == 4 and out.element_size() == 4 and src.is_contiguous() and out.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_scatter_words(_ptr(src), _ptr(rows), _ptr(out), c_int(rows.numel()), _stream()))


def scale_add_bias(x: torch.Tensor, scale: Optional[float], bias: Optional[torch.Tensor],
                   softcap: Optional[float] = None) -> None:
    """In place on float32 rows: x = x * scale + bias (either may be absent); with ``softcap`` c then
    x = c * tanh(x / c)."""
    _dev(x, bias)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    if bias is not None:
        assert bias.shape == (x.shape[1],) and bias.is_contiguous()
    if softcap is not None and not softcap > 0:
        raise KernelError("a logit cap must be positive")
    lib = core()
    _check(lib, lib.coheryn_scale_bias_cap(_ptr(x), c_long(x.stride(0)), c_int(x.shape[0]), c_int(x.shape[1]),
                                           c_float(1.0 if scale is None else scale), _ptr(bias),
                                           c_int(_code(bias) if bias is not None else F32),
                                           c_float(0.0 if softcap is None else softcap), _stream()))


def stream_inject(x: torch.Tensor, table: Optional[torch.Tensor], ids: Optional[torch.Tensor], scale: Optional[float],
                  vector: Optional[torch.Tensor]) -> None:
    """In place on the float32 stream: x[t] += table[ids[t]] * scale (when a table is given) + vector (when given)."""
    _dev(x, table, ids, vector)
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    V = 0
    if table is not None:
        _i32(ids, "ids")
        assert table.is_contiguous() and table.shape[1] == H and ids.numel() == T
        V = table.shape[0]
    if vector is not None:
        assert vector.shape == (H,) and vector.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_stream_inject(_ptr(x), _ptr(table), c_int(_code(table) if table is not None else F32), _ptr(ids),
                                          c_float(1.0 if scale is None else scale), _ptr(vector),
                                          c_int(_code(vector) if vector is not None else F32), c_int(T), c_int(H), c_int(V),
                                          _stream()))


def stream_join(x: torch.Tensor, delta: Optional[torch.Tensor], table: torch.Tensor, ids: torch.Tensor,
                scale: Optional[float], dtype: torch.dtype) -> torch.Tensor:
    """[x + pending summands | table[ids] * scale] as [T, 2 H] in ``dtype``: the input of a product that mixes the stream
    with the embedding output.  ``delta``: None, a float32 [T, H] or stack [P, T, H], or a bfloat16 [T, H]."""
    _dev(x, delta, table, ids)
    _i32(ids, "ids")
    T, H = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous() and table.shape[1] == H
    parts, P, stride, d16 = None, 0, 0, None
    if delta is not None:
        assert delta.is_contiguous() and tuple(delta.shape[-2:]) == (T, H)
        if delta.dtype == torch.float32:
            parts, P, stride = delta, (delta.shape[0] if delta.dim() == 3 else 1), T * H
        elif delta.dtype == torch.bfloat16 and delta.dim() == 2:
            d16 = delta
        else:
            raise KernelError("stream_join: a pending summand is float32 (one or a stack) or one bfloat16 tensor")
    out = torch.empty((T, 2 * H), dtype=dtype, device=x.device)
    lib = core()
    _check(lib, lib.coheryn_stream_join(_ptr(x), _ptr(parts), c_int(P), c_long(stride), _ptr(d16), _ptr(table),
                                        c_int(_code(table)), _ptr(ids), c_float(1.0 if scale is None else scale), _ptr(out),
                                        c_int(_CODES[dtype]), c_int(T), c_int(H), c_int(table.shape[0]), _stream()))
    return out


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, update: bool = True) -> None:
    """x = resid (+ delta); resid = x if update; out = x / sqrt(mean(x^2) + eps) * weight.
    With ``rows`` only those rows are read (out[r] comes from row rows[r]) and the
    residual is left as it is.  ``delta`` may be a float32 stack [splits, n, H] of partial sums
    (see ``linear(partial_ok=True)``): they are added in order, then to the residual."""
    _dev(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert out.is_contiguous() and out.shape[-1] == H and weight.shape == (H,)
    n = out.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        assert rows.numel() == n
        update = False
    else:
        assert resid.shape[0] >= n
    lib = core()
    if delta is not None and delta.dim() == 3:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[1:] == resid.shape
        _check(lib, lib.coheryn_add_parts_rmsnorm(
            _ptr(resid), _ptr(delta), c_int(delta.shape[0]), c_long(delta.stride(0)), _ptr(rows), _ptr(weight),
            c_int(_code(weight)), c_float(eps), _ptr(out), c_int(_code(out)), c_int(n), c_int(H),
            c_int(1 if update else 0), _stream()))
        return
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == resid.shape
    _check(lib, lib.coheryn_add_rmsnorm(
        _ptr(resid), _ptr(delta), c_int(_code(delta) if delta is not None else F32), _ptr(rows),
        _ptr(weight), c_int(_code(weight)), c_float(eps), _ptr(out), c_int(_code(out)), c_int(n),
        c_int(H), c_int(1 if (update and delta is not None) else 0), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, code: int = 1, param: float = 0.0) -> None:
    """out[m, j] = act(gate_up[m, 2j], gate_up[m, 2j + 1]) (gate and up interleaved); ``code`` names the
    activation as the gated epilogues do (``GATED_ACTIVATIONS``; 1 = SiLU), ``param`` is its constant where
    it has one (in full float32 here).  The rows of ``out`` may be strided."""
    _dev(gate_up, out)
    M, I2 = gate_up.shape
    assert I2 % 2 == 0 and out.shape == (M, I2 // 2) and out.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and out.stride(1) == 1
    lib = core()
    _check(lib, lib.coheryn_act_mul_ex(_ptr(gate_up), _ptr(out), c_int(_code(out)), c_int(M), c_int(I2 // 2),
                                       c_int(code & 0xff), c_float(param), c_long(out.stride(0)), _stream()))


def add_normed_rmsnorm(resid: torch.Tensor, parts: torch.Tensor, inner_weights: Optional[torch.Tensor], coef: float,
                       post_weight: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor],
                       rows: Optional[torch.Tensor] = None) -> None:
    """A residual add whose summand is normalised first, fused with the norm that reads the sum.  ``parts`` float32
    [P, n, H] (or [n, H]): y = sum of the parts, or with ``inner_weights`` [P, H] y = coef * sum_p parts[p] /
    rms(parts[p]) * inner_weights[p]; x = resid + y / rms(y) * post_weight; resid = x (without ``rows``);
    out = x / rms(x) * weight (when a weight and an output are given).  rms(z) = sqrt(mean(z^2) + eps).
    With ``rows`` only those rows are read and the residual stays as it is."""
    _dev(resid, parts, inner_weights, post_weight, weight, out, rows)
    if parts.dim() == 2:
        parts = parts.unsqueeze(0)
    P, n_all, H = parts.shape
    assert parts.dtype == torch.float32 and parts.stride(2) == 1 and resid.dtype == torch.float32 and resid.is_contiguous()
    assert resid.shape[-1] == H and post_weight.shape == (H,) and post_weight.is_contiguous()
    if inner_weights is not None:
        assert inner_weights.shape == (P, H) and inner_weights.is_contiguous()
    n = resid.shape[0]
    if rows is not None:
        _i32(rows, "rows")
        n = rows.numel()
    else:
        assert n_all == n
    if out is not None:
        assert weight is not None and weight.shape == (H,) and out.is_contiguous() and out.shape == (n, H)
    lib = core()
    _check(lib, lib.coheryn_add_normed_rmsnorm(
        _ptr(resid), _ptr(parts), c_int(P), c_long(parts.stride(0)), c_long(parts.stride(1)), _ptr(inner_weights),
        c_int(_code(inner_weights) if inner_weights is not None else F32), c_float(coef), _ptr(post_weight),
        c_int(_code(post_weight)), _ptr(rows), _ptr(weight if out is not None else None),
        c_int(_code(weight) if weight is not None else F32), c_float(eps), _ptr(out),
        c_int(_code(out) if out is not None else F32), c_int(n), c_int(H), c_int(0 if rows is not None else 1), _stream()))


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                  slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int, page_size: int) -> None:
    """Rotate q (in place) and k by position; write rotated k and v into cache pages
    laid out [page, kv head, slot, head_dim] at ``slots`` (page * page_size + offset).
    Without caches (a layer that reads another layer's cache) the buffer holds query
    heads only and they are rotated in place."""
    _dev(qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions")
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    if rotary_dim:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
        assert cos_sin.shape[1:] == (rotary_dim // 2, 2)
    write = k_cache is not None
    if write:
        _i32(slots, "slots")
        assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    else:
        assert num_kv_heads == 0, "without a cache to write, only query heads are rotated"
    lib = core()
    _check(lib, lib.coheryn_rope_kv_write(
        _ptr(qkv), c_int(_code(qkv)), _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache),
        _ptr(v_cache), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(rotary_dim), c_int(page_size), c_int(1 if write else 0), _stream()))


# Up to this many rows the q/k/v product rotates and writes the cache in its own epilogue.
QKV_ROPE_M = int(os.environ.get("COHERYN_QKV_ROPE_M", "16"))


def qkv_rope_ok(x, w_qkv, k_cache, rotary_dim: int, head_dim: int) -> bool:
    return (0 < x.shape[0] <= QKV_ROPE_M and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and k_cache is not None and k_cache.dtype == torch.bfloat16 and rotary_dim == head_dim
            and head_dim % 16 == 0 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w_qkv.is_contiguous() and w_qkv.data_ptr() % 16 == 0)


def qkv_rope_small(x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], positions: torch.Tensor,
                   cos_sin: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> torch.Tensor:
    """q, k, v = x @ w_qkv.T (+ b) for at most 16 rows with the rotation of q and k and the
    cache write of k and v in the product's epilogue (see ``rope_kv_write`` for the layout).
    Returns the rotated q ``[T, num_heads * head_dim]``; the whole head is rotated."""
    _dev(x, w_qkv, b_qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slots, "slots")
    T, K = x.shape
    assert w_qkv.shape == ((num_heads + 2 * num_kv_heads) * head_dim, K)
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    q = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    lib = core()
    _check(lib, lib.coheryn_qkv_rope_bf16_small(
        _ptr(x), _ptr(w_qkv), _ptr(b_qkv), c_int(_code(b_qkv) if b_qkv is not None else F32), _ptr(q),
        c_long(q.stride(0)), _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T),
        c_int(K), c_long(x.stride(0)), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size),
        _stream()))
    return q


def seeded_fill(out: torch.Tensor, key: int, first: int, mean: float, deviation: float) -> None:
    """out.flatten()[i] = the seeded random value of element first + i of the tensor with ``key``
    (see weights/seeded.py), float32 or bfloat16."""
    _dev(out)
    assert out.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_seeded_fill(_ptr(out), c_int(_code(out)), ctypes.c_ulonglong(key), ctypes.c_ulonglong(first),
                                        ctypes.c_ulonglong(out.numel()), ctypes.c_double(mean), ctypes.c_double(deviation),
                                        _stream()))


# Up to this many rows a q/k/v product whose K the many-rows kernel splits leaves the addition of
# its slices to the rotation kernel (one kernel less between the product and the attention).
QKV_PARTS_M = int(os.environ.get("COHERYN_QKV_PARTS_M", "256"))
# ... by the few-rows product above this many rows (up to FEW_DEFER_M), by the many-rows product otherwise
# (at 64 rows the latter is 2 % of a decode step faster).
QKV_PARTS_FEW_FROM = 64


def qkv_parts_count(x, w_qkv, k_cache, rotary_dim: int, head_dim: int) -> int:
    """The K slices that ``qkv_rope_parts`` would leave for this step's q/k/v product (0: not that path)."""
    M, K = x.shape
    if not (QKV_ROPE_M < M <= QKV_PARTS_M and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and k_cache is not None and k_cache.dtype == torch.bfloat16 and rotary_dim == head_dim and head_dim % 16 == 0
            and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_qkv.is_contiguous()
            and w_qkv.data_ptr() % 16 == 0):
        return 0
    few = few_splits(w_qkv.shape[0], K)           # the few-rows product (weights streamed once) where it cuts K
    if few > 1 and QKV_PARTS_FEW_FROM < M <= FEW_DEFER_M:
        return few
    return int(core().coheryn_gemm_tc_parts_count(c_int(M), c_int(w_qkv.shape[0]), c_int(K)))


def qkv_rope_parts(x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], positions: torch.Tensor,
                   cos_sin: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, count: int) -> torch.Tensor:
    """q, k, v = x @ w_qkv.T (+ b) by the few-rows product (or, where that does not cut K, the many-rows
    product) with K cut into ``count`` slices, whose
    addition, the bias, the rotation of q and k and the cache write of k and v happen in ONE following
    kernel (see ``rope_kv_write``).  Returns the rotated q ``[T, num_heads * head_dim]``."""
    _dev(x, w_qkv, b_qkv, positions, cos_sin, slots, k_cache, v_cache)
    _i32(positions, "positions"); _i32(slots, "slots")
    T, K = x.shape
    N = w_qkv.shape[0]
    assert N == (num_heads + 2 * num_kv_heads) * head_dim
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
    lib = core()
    parts = torch.empty((count, T, N), dtype=torch.float32, device=x.device)
    if count == few_splits(N, K):
        gemm_bf16_tc_few(x, w_qkv, None, parts, defer=True)
    else:
        _check(lib, lib.coheryn_gemm_bf16_tc_parts(_ptr(x), _ptr(w_qkv), _ptr(parts), c_int(T), c_int(N), c_int(K),
                                                   c_long(x.stride(0)), _ptr(tc_status(x.device)), _stream()))
    q = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    _check(lib, lib.coheryn_rope_kv_write_parts(
        _ptr(parts), c_int(count), c_long(T * N), _ptr(b_qkv), c_int(_code(b_qkv) if b_qkv is not None else F32), _ptr(q),
        _ptr(positions), _ptr(cos_sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_int(page_size), _stream()))
    return q


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ w.T (+ bias) with float32 FMA accumulation (no tensor cores)."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape == (N, K) and w.is_contiguous() and out.shape == (M, N)
    assert x.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.shape == (N,) and bias.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_gemm_simt(
        _ptr(x), c_int(_code(x)), _ptr(w), c_int(_code(w)), _ptr(bias),
        c_int(_code(bias) if bias is not None else F32), _ptr(out), c_int(_code(out)), c_int(M),
        c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)), _stream()))


def attention_simple(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, token_req: torch.Tensor, positions: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                     window: Optional[int], scale: float, v_head_dim: Optional[int] = None,
                     slopes: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """Causal attention of each token over its request's cache pages (float32 math).
    ``q`` may be a column slice of a wider buffer (its row stride is honoured).  ``v_head_dim``: values
    of another head size than keys; ``slopes`` (float32 [heads]): the score of a key at distance d loses
    slopes[h] * d; ``out_scale`` multiplies the output."""
    _dev(q, out, k_cache, v_cache, block_tables, token_req, positions, slopes)
    _i32(block_tables, "block_tables"); _i32(token_req, "token_req"); _i32(positions, "positions")
    T = q.shape[0]
    vd = head_dim if v_head_dim is None else v_head_dim
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape[1] == num_heads * vd
    assert k_cache.dtype == q.dtype and out.dtype == q.dtype and v_cache.dtype == q.dtype
    if slopes is not None:
        assert slopes.dtype == torch.float32 and slopes.is_contiguous() and slopes.numel() == num_heads
    lib = core()
    _check(lib, lib.coheryn_attention_simple_ex(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(_code(q)), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(token_req),
        _ptr(positions), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(vd),
        c_int(page_size), c_int(window or 0), c_float(scale), _ptr(slopes), c_float(out_scale), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[r] = lowest index of the maximum of logits[r]; non-finite logits set status 2."""
    _dev(logits, out, status)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _i32(out, "out")
    lib = core()
    slots = int(lib.coheryn_argmax_scratch_slots(c_int(R), c_int(V)))
    scratch = torch.empty(2 * slots, dtype=torch.int32, device=logits.device) if slots else None
    _check(lib, lib.coheryn_argmax(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                   _ptr(out), _ptr(status), _ptr(scratch), c_long(slots), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """Temperature / top-k / top-p sampling of one token per row from host-made draws."""
    _dev(logits, temperature, top_k, top_p, uniform, out, status)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert uniform.dtype == torch.float64
    _i32(top_k, "top_k"); _i32(out, "out")
    lib = core()
    _check(lib, lib.coheryn_sample(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                   _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
                                   _ptr(out), _ptr(status), _stream()))


def apply_penalties(logits, rows, ids, counts, rep, freq, pres) -> None:
    """In place: the reference's penalties on logits[rows[i], ids[i]] (each pair once)."""
    _dev(logits, rows, ids, counts, rep, freq, pres)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    for t in (rows, ids, counts):
        _i32(t, "penalty index")
    lib = core()
    _check(lib, lib.coheryn_apply_penalties(_ptr(logits), c_long(logits.stride(0)), c_int(rows.numel()),
                                            _ptr(rows), _ptr(ids), _ptr(counts), _ptr(rep), _ptr(freq),
                                            _ptr(pres), _stream()))


# ------------------------------------------------------------------------------------
def gemm_bf16_small(x, w, bias, out, gated: int = 0) -> None:
    """Tensor-core product for at most 64 rows (decode); see csrc/gemm_bf16_small.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    _check(lib, lib.coheryn_gemm_bf16_small(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _stream()))


# Up to this many rows the weight-streaming mma.sync kernel runs; beyond it the TMA/tcgen05
# kernel (which re-reads nothing of x through L2 and so scales to many rows).
SMALL_M = 16
_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """Device word that the tensor-core GEMM sets when one of its bounded waits runs out."""
    t = _tc_status.get(device)
    if t is None:
        t = _tc_status[device] = _tc_status.setdefault(str(torch.device(device)), torch.zeros(1, dtype=torch.int32, device=device))
    return t


STATUS_MESSAGES = {1: "a token id was outside the embedding table", 2: "non-finite logits"}


def describe_status(code: int) -> str:
    """What a non-zero device status word means."""
    if code in STATUS_MESSAGES:
        return STATUS_MESSAGES[code]
    if 11 <= code <= 39:
        return (f"a kernel gave up a bounded wait and left its output unfinished (code {code}: 11-13 tensor-core product: "
                "producer, MMA issuer, epilogue; 19 self-test; 31-39 prompt attention: 31 producer, 32-36 MMA issuer, "
                "37-39 softmax)")
    return f"device status {code}"


def check_tc_status(device) -> None:
    code = int(tc_status(device).item())
    if code:
        tc_status(device).zero_()
        raise KernelError(describe_status(code))


def selftest_bounded_wait(device, tries: int = 300, code: int = 19) -> None:
    """Launch the self-test kernel: it waits ``tries`` times on a barrier nothing arrives on, gives
    up, and records ``code`` in the status word of the tensor-core kernels (see csrc/selftest.cu)."""
    lib = core()
    _check(lib, lib.coheryn_selftest_bounded_wait(_ptr(tc_status(device)), ctypes.c_uint(tries), c_int(code), _stream()))


def gemm_bf16_tc(x, w, bias, out, gated: int = 0) -> None:
    """TMA + tcgen05 product for many rows (prompt portions); see csrc/gemm_tc.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    floats = _tc_workspace_floats(M, N, K)   # > 0: K is split
    workspace = torch.empty(floats, dtype=torch.float32, device=x.device) if floats else None
    _check(lib, lib.coheryn_gemm_bf16_tc(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _ptr(workspace), c_long(floats), _stream()))


def set_gemm_pairs(on: bool) -> None:
    """Whether ``gemm_bf16_tc`` hands suitable shapes to the kernel of CTA pairs (default: yes)."""
    core().coheryn_gemm_tc_set_pairs(c_int(1 if on else 0))
    _tc_workspace_floats.cache_clear()      # the pairs take shapes that would otherwise split K


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """K splits that ``gemm_bf16_tc`` uses for this shape (1: none; a shape run by CTA pairs: 1)."""
    return max(1, _tc_workspace_floats(M, N, K) // (M * N))


def gemm_bf16_tc_pair(x, w, bias, out, gated: int = 0) -> None:
    """The many-rows product by pairs of CTAs sharing 256 x 256 tiles (tcgen05 cta_group::2);
    see gemm_tc_pair_kernel in csrc/gemm_tc.cu."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape == (M, N // 2 if gated else N)
    lib = core()
    _check(lib, lib.coheryn_gemm_bf16_tc_pair(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(0)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _stream()))


_few_workspaces = {}
_few_retired = []     # outgrown workspaces stay alive: captured graphs may still name them


def _few_workspace(device, floats: int) -> torch.Tensor:
    """Zero-initialised scratch of the few-rows product: counters, then the K splits' tiles.
    One per device: the products that share it must run in stream order on one stream."""
    key = str(device)
    ws = _few_workspaces.get(key)
    if ws is None or ws.numel() < floats:
        if ws is not None:
            _few_retired.append(ws)
        ws = torch.zeros(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _few_workspaces[key] = ws
    return ws


@functools.lru_cache(maxsize=None)
def few_splits(N: int, K: int) -> int:
    """Into how many slices of K the few-rows product cuts this weight shape (1: none)."""
    return int(core().coheryn_gemm_tc_few_splits(c_int(N), c_int(K)))


@functools.lru_cache(maxsize=None)
def _tc_workspace_floats(M: int, N: int, K: int) -> int:
    return int(core().coheryn_gemm_tc_workspace_floats(c_int(M), c_int(N), c_int(K)))


@functools.lru_cache(maxsize=None)
def _few_workspace_floats(M: int, N: int, K: int) -> int:
    return int(core().coheryn_gemm_tc_few_workspace_floats(c_int(M), c_int(N), c_int(K)))


def gemm_bf16_tc_few(x, w, bias, out, gated: int = 0, defer: bool = False) -> None:
    """TMA + tcgen05 product for at most 64 rows with the features on the accumulator's
    lanes (decode, short portions); see csrc/gemm_tc_few.cu.  ``defer``: ``out`` is a float32
    stack [splits, M, N] of the K slices' sums, left for the consumer to add."""
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K
    assert x.stride(1) == 1 and out.stride(-1) == 1
    lib = core()
    if defer:
        assert not gated and out.dtype == torch.float32 and out.is_contiguous()
        assert out.shape == (few_splits(N, K), M, N)
        floats = 0
    else:
        assert out.shape == (M, N // 2 if gated else N)
        floats = _few_workspace_floats(M, N, K)   # > 0: K is split
    workspace = _few_workspace(x.device, floats) if floats else None
    _check(lib, lib.coheryn_gemm_bf16_tc_few(
        _ptr(x), _ptr(w), _ptr(bias), c_int(_code(bias) if bias is not None else F32), _ptr(out),
        c_int(_code(out)), c_int(M), c_int(N), c_int(K), c_long(x.stride(0)), c_long(out.stride(-2)),
        c_int(int(gated)), _ptr(tc_status(x.device)), _ptr(workspace),
        c_long(workspace.numel() if workspace is not None else 0), c_int(1 if defer else 0), _stream()))


# Up to this many rows the few-rows tcgen05 kernel takes the products whose K it need not
# split, or whose consumer adds the splits (0 switches it off).  A product that would have to
# add its own splits goes to the mma.sync kernel instead: measured on a B200, the in-kernel
# addition through memory costs several dependent round trips.
FEW_M = int(os.environ.get("COHERYN_FEW_M", "32"))
# ... and up to this many rows the products whose K slices the consumer adds.  The kernel takes up to
# 256 rows, but every CTA re-reads all rows of x beside its weight tile, and from 129 rows on that costs
# what the many-rows kernel with its extra kernel for the K slices costs (1.5B sizes, down projection:
# 128 rows 15.9 -> 12.7 us, 256 rows 21.1 -> 18.8; a decode step at batch 128 3.64 -> 3.45 ms, at 256 no change).
FEW_DEFER_M = int(os.environ.get("COHERYN_FEW_DEFER_M", "128"))
# The output head (a very large weight) takes the few-rows product up to this many rows only: every CTA
# re-reads all rows of x, which beyond that costs more than the weight stream.
FEW_HEAD_M = 64


# A product hands its K slices to the consumer only from this K on.  Measured on a B200 at 8
# rows: for K = 1536 (12 slices of two steps) the norm that adds twelve parts loses more than
# the product gains over the mma.sync kernel; for K = 8960 the pair is 5 us faster.
DEFER_MIN_K = 4096
# With more than SMALL_M_SHORT rows the alternative is the many-rows kernel plus the kernel that adds
# its K splits: there the slices pay from K = 1024 on (1 % of a decode step at 40 and 64 rows).
DEFER_MIN_K_WIDE = int(os.environ.get("COHERYN_DEFER_MIN_K_WIDE", "1024"))


# A weight matrix of at least this many elements (the output head over a large vocabulary) goes
# through the few-rows product up to FEW_HEAD_M rows: its stream is all that matters there.
FEW_LARGE_WEIGHT = 128 << 20


def _few_ok(x, w, partial_ok: bool = False) -> bool:
    if not _few_shape_ok(x, w, FEW_HEAD_M if w.numel() >= FEW_LARGE_WEIGHT else None):
        return False
    return partial_ok or few_splits(w.shape[0], w.shape[1]) == 1


def _few_shape_ok(x, w, limit: Optional[int] = None) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= (FEW_M if limit is None else limit)
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def _tc_ok(x, w) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > SMALL_M
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


# ... and up to this many rows when the weight matrix is small (a few MB: the q/k/v and output
# products of a decode batch), where one launch of the mma.sync kernel beats the tcgen05 kernel
# plus the kernel that adds its K splits.
SMALL_M_SHORT = int(os.environ.get("COHERYN_SMALL_M_SHORT", "32"))
SMALL_WEIGHT_ELEMENTS = 4 << 20


def _small_ok(x, w) -> bool:
    M = x.shape[0]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and (0 < M <= SMALL_M or (0 < M <= SMALL_M_SHORT and w.numel() <= SMALL_WEIGHT_ELEMENTS))
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
           partial_ok: bool = False) -> torch.Tensor:
    """y = x @ w.T (+ bias), float32 accumulation.  float32 operands use FMA on the CUDA
    cores (no reduced-precision tensor mode); bfloat16 operands use the tensor-core
    kernels where the shape allows and the FMA kernel otherwise.  With ``partial_ok`` the
    result may come as a float32 stack [splits, M, N] of partial sums whose addition is left
    to the consumer (``add_rmsnorm`` takes such a stack as its delta)."""
    M, N = x.shape[0], w.shape[0]
    if (partial_ok and out is None and M and w.shape[1] >= (DEFER_MIN_K_WIDE if M > SMALL_M_SHORT else DEFER_MIN_K)
            and _few_shape_ok(x, w, FEW_DEFER_M)):
        splits = few_splits(N, w.shape[1])
        if splits > 1:
            parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            gemm_bf16_tc_few(x, w, bias, parts, defer=True)
            return parts
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    if _few_ok(x, w):
        gemm_bf16_tc_few(x, w, bias, out)
    elif _small_ok(x, w):
        gemm_bf16_small(x, w, bias, out)
    elif _tc_ok(x, w):
        gemm_bf16_tc(x, w, bias, out)
    else:
        gemm_simt(x, w, bias, out)
    return out


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step,
              group: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
              window: Optional[int], scale: float) -> None:
    """Attention of every token of the step over its request's cache pages of ``group``
    (``step`` is a StepContext).  Chooses the kernel by dtype and shape."""
    attention_rows(q, out, k_cache, v_cache, step.block_tables[group], step.token_req,
                   step.positions, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                   cu_q=step.cu_q, kv_lens=step.kv_lens, q_lens=step.q_lens, max_kv_len=step.max_kv_len,
                   settled=step.prior_positions_settled)


LOG2_E = 1.4426950408889634


def attention_biased(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, page_size: int,
                     window: Optional[int], scale: float, slopes: Optional[torch.Tensor],
                     slopes_log2: Optional[torch.Tensor] = None, out_scale: float = 1.0, force_simple: bool = False) -> None:
    """Attention of every token of the step over its request's cache pages of ``group`` with a score that loses
    slopes[h] times the distance (``slopes_log2``: the same times log2 e, for the tensor-core kernels; made here when
    absent), values of their own head size and a scaled output.  bfloat16 with keys and values of one head size that is
    a multiple of 16 runs the mma.sync kernels (prompt tiles, decode splits); everything else the float32-arithmetic one."""
    fast = (not force_simple and q.dtype == torch.bfloat16 and head_dim == v_head_dim and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and out_scale == 1.0 and q.stride(0) % 8 == 0 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0
            and getattr(step, "max_kv_len", None) is not None and getattr(step, "q_lens", None))
    if not fast:
        attention_simple(q, out, k_cache, v_cache, step.block_tables[group], step.token_req, step.positions, num_heads,
                         num_kv_heads, head_dim, page_size, window, scale, v_head_dim=v_head_dim, slopes=slopes,
                         out_scale=out_scale)
        return
    if slopes is not None and slopes_log2 is None:
        slopes_log2 = slopes * LOG2_E
    attention_rows(q, out, k_cache, v_cache, step.block_tables[group], step.token_req, step.positions, num_heads, num_kv_heads,
                   head_dim, page_size, window, scale, cu_q=step.cu_q, kv_lens=step.kv_lens, q_lens=step.q_lens,
                   max_kv_len=step.max_kv_len, settled=step.prior_positions_settled, slopes_log2=slopes_log2)


def attention_lib(head_dim: int):
    lib = _attn_libs.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_attn_scratch_floats.restype = ctypes.c_long
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        if lib.coheryn_attn_head_dim() != head_dim:
            raise KernelError(f"attention library was built for head size {lib.coheryn_attn_head_dim()}, not {head_dim}")
        _attn_libs[head_dim] = lib
    return lib


def set_attention_split(head_dim: int, keys: int) -> None:
    """Fix the positions per CTA of the decode attention kernel for this head size (a power of two
    from 128 to 2048, capped at 256 pages); 0 restores the choice by batch size and context.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_split(c_int(keys))


def set_attention_tc_two_tiles(head_dim: int, on: Optional[bool]) -> None:
    """Whether the prompt-portion attention kernel gives a CTA two consecutive row tiles that share
    every fetched key tile (head sizes up to 128): always, never, or (None, the default) when the
    pairs still fill the GPU.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_tc_two_tiles(c_int(2 if on is None else (1 if on else 0)))


def set_attention_tc_cluster(head_dim: int, cluster: int) -> None:
    """Fix the number of CTAs (1, 2, 4 or 8) that share a row tile of the prompt-portion attention
    kernel and split its keys; 0 restores the choice by shape.  For tests and experiments."""
    attention_lib(head_dim).coheryn_attn_set_tc_cluster(c_int(cluster))


def attention_rows(q, out, k_cache, v_cache, block_tables, token_req, positions, num_heads, num_kv_heads,
                   head_dim, page_size, window, scale, cu_q=None, kv_lens=None, q_lens=None,
                   max_kv_len=None, force_simple=False, settled=True, slopes_log2=None) -> None:
    """Attention of rows (request token_req[i] at position positions[i]) over cache pages.
    bfloat16 rows that are whole runs of consecutive positions per request, ending at the
    request's last position (``cu_q``, ``kv_lens`` on the device, ``q_lens`` and
    ``max_kv_len`` on the host) go to the tensor-core kernels when the head size is a
    multiple of 16 up to 256; everything else goes to the float32-arithmetic kernel.
    ``settled``: the keys and values at positions before each request's first row were written by
    earlier steps, so the decode kernel may fetch them before it waits for the step's earlier
    kernels; False when this step itself wrote them (the wanted rows of a portion)."""
    fast = (not force_simple and q.dtype == torch.bfloat16 and cu_q is not None and kv_lens is not None
            and q_lens is not None and max_kv_len is not None and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and q.stride(0) % 8 == 0 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0)
    if not fast:
        attention_simple(q, out, k_cache, v_cache, block_tables, token_req, positions, num_heads,
                         num_kv_heads, head_dim, page_size, window, scale,
                         slopes=slopes_log2 / LOG2_E if slopes_log2 is not None else None)
        return
    _dev(q, out, k_cache, v_cache, block_tables, cu_q, kv_lens, slopes_log2)
    _i32(block_tables, "block_tables"); _i32(cu_q, "cu_q"); _i32(kv_lens, "kv_lens")
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == q.dtype and k_cache.dtype == q.dtype
    G = num_heads // num_kv_heads
    B = len(q_lens)
    rows = [n * G for n in q_lens]
    any_small = any(r <= 16 for r in rows)
    any_large = any(r > 16 for r in rows)
    lib = attention_lib(head_dim)
    scratch, floats = None, 0
    if any_small and G <= 16:
        floats = int(lib.coheryn_attn_scratch_floats(c_int(B), c_int(num_kv_heads), c_int(max_kv_len)))
        scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    args = (_ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
            _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(cu_q), _ptr(kv_lens), c_int(B),
            c_int(num_heads), c_int(num_kv_heads), c_int(page_size), c_int(window or 0), c_float(scale),
            c_int(max(rows)), c_int(1 if any_small else 0), c_int(1 if any_large else 0), c_int(max_kv_len),
            _ptr(scratch), c_long(floats), _ptr(tc_status(q.device)), c_int(q.shape[0]), c_int(k_cache.shape[0]),
            c_int(1 if settled else 0))
    if slopes_log2 is not None:     # a score that loses a slope per head times the distance
        assert slopes_log2.dtype == torch.float32 and slopes_log2.is_contiguous() and slopes_log2.numel() == num_heads
        _check(lib, lib.coheryn_attention_bf16_biased(*args, _ptr(slopes_log2), _stream()))
    else:
        _check(lib, lib.coheryn_attention_bf16(*args, _stream()))


# Decode steps of at most this many requests merge the attention splits inside the output
# projection's kernel (0 switches that off: the splits are merged by a kernel of their own and the
# projection is an ordinary product).
ATTN_OPROJ_M = int(os.environ.get("COHERYN_ATTN_OPROJ_M", "16"))


# ... and only while the merging stays cheap: every CTA of the merged kernel (one per head and tile of
# 128 output features) reads the splits of its head for all requests again, so the bytes read grow with
# width / 128 x heads x requests x splits.  Beyond this many bytes the splits are merged once, by the
# kernel of their own.
ATTN_OPROJ_MERGE_BYTES = int(os.environ.get("COHERYN_ATTN_OPROJ_BYTES", str(32 << 20)))


# Whether a pre-norm block made of the built-in parts is enqueued by one call into the library
# (csrc/block_runner.cu) instead of part by part; the kernels and their order are the same.
NATIVE_BLOCK = os.environ.get("COHERYN_NATIVE_BLOCK", "1") != "0"


# Whether a block whose producers can hand over their activations multiplies them by the stacked output matrices in
# ONE product (parts/block.py: ParallelResidual) instead of one product per producer.
JOINED_OUTPUT = os.environ.get("COHERYN_JOINED_OUTPUT", "1") != "0"


def set_joined_output(on: bool) -> None:
    global JOINED_OUTPUT
    JOINED_OUTPUT = bool(on)


def set_native_block(on: bool) -> None:
    global NATIVE_BLOCK
    NATIVE_BLOCK = bool(on)


def attention_oproj_ok(q: torch.Tensor, w_o: torch.Tensor, step, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    if step.max_kv_len is None or step.max_q_len != 1:
        return False
    tiles = -(-w_o.shape[0] // 128)
    merge_bytes = tiles * num_heads * step.num_requests * (-(-step.max_kv_len // 128)) * head_dim * 4
    return (merge_bytes <= ATTN_OPROJ_MERGE_BYTES and q.dtype == torch.bfloat16 and w_o.dtype == torch.bfloat16 and step.max_q_len == 1
            and 0 < step.num_requests <= min(ATTN_OPROJ_M, 16) and q.shape[0] == step.num_requests
            and num_heads // num_kv_heads <= 16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and step.max_kv_len is not None and (step.max_kv_len + 127) // 128 + 1 <= 512
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and w_o.stride(1) == 1 and w_o.stride(0) % 8 == 0
            and w_o.data_ptr() % 16 == 0 and w_o.shape[0] % 4 == 0)


def attention_oproj(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int, num_heads: int,
                    num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int], scale: float,
                    w_o: torch.Tensor, b_o: Optional[torch.Tensor]) -> torch.Tensor:
    """Decode attention of one token per request and the output projection: returns a float32 stack
    [num_heads, B, H] whose sum over the heads is attention(q) @ w_o.T (+ b_o); the consumer (a norm
    that takes partial sums) adds the heads in order.  See attn_merge_oproj in csrc/attention_bf16.cu."""
    block_tables, cu_q, kv_lens = step.block_tables[group], step.cu_q, step.kv_lens
    _dev(q, k_cache, v_cache, block_tables, cu_q, kv_lens, w_o, b_o)
    _i32(block_tables, "block_tables"); _i32(cu_q, "cu_q"); _i32(kv_lens, "kv_lens")
    B, H = step.num_requests, w_o.shape[0]
    assert w_o.shape[1] == num_heads * head_dim and k_cache.dtype == q.dtype
    lib = attention_lib(head_dim)
    floats = int(lib.coheryn_attn_scratch_floats(c_int(B), c_int(num_kv_heads), c_int(step.max_kv_len)))
    scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    parts = torch.empty((num_heads, B, H), dtype=torch.float32, device=q.device)
    _check(lib, lib.coheryn_attention_oproj_bf16(
        _ptr(q), c_long(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(cu_q), _ptr(kv_lens), c_int(B), c_int(num_heads), c_int(num_kv_heads), c_int(page_size), c_int(window or 0),
        c_float(scale), c_int(step.max_kv_len), _ptr(scratch), c_long(floats), _ptr(w_o), c_long(w_o.stride(0)), c_int(H),
        _ptr(b_o), c_int(_code(b_o) if b_o is not None else F32), _ptr(parts), c_int(1 if step.prior_positions_settled else 0),
        _stream()))
    return parts


# Activations of the gated epilogue, by the code that the kernels take as their ``gated`` argument
# (0 means "no gate").  The gate is applied in float32 inside the product's epilogue; an activation
# that is not built is refused here by name, before anything is launched.
# "swish_clamped" has a constant c: g <- min(g, c), u <- clamp(u, -c, c), result g sigmoid(1.702 g) (u + 1).
GATED_ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "swish_clamped": 3}
GATED_WITH_CONSTANT = ("swish_clamped",)


def gated_activation_code(activation: str) -> int:
    try:
        return GATED_ACTIVATIONS[activation]
    except KeyError:
        raise KernelError(f"the gated epilogue of the matrix products is not built for activation {activation!r} "
                          f"(built: {', '.join(sorted(GATED_ACTIVATIONS))})") from None


def gated_epilogue_word(activation: str, param: Optional[float] = None) -> int:
    """What the products take as their ``gated`` argument: the activation's code in the low byte and, for an
    activation with a constant, the constant rounded to the upper 24 bits of its float32 form (15 bits of
    mantissa, far below what a bfloat16 result can show; the unfused kernel takes it whole)."""
    code = gated_activation_code(activation)
    if activation not in GATED_WITH_CONSTANT:
        return code
    if param is None or not param > 0:
        raise KernelError(f"activation {activation!r} needs a positive constant")
    import struct
    bits = struct.unpack("<I", struct.pack("<f", float(param)))[0]
    bits = (bits + 0x80) & 0xffffff00
    if bits >= 0x7f800000:
        raise KernelError(f"the constant {param!r} of activation {activation!r} is out of range")
    return bits | code


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu",
                 out: Optional[torch.Tensor] = None, param: Optional[float] = None) -> torch.Tensor:
    """act(x @ Wg.T) * (x @ Wu.T) for w_gate_up with INTERLEAVED rows (row 2j = gate_j,
    row 2j+1 = up_j), so that a gate/up pair lands in one thread of the epilogue.  ``out`` ([M, I] of x's dtype, rows
    may be strided: a column slice of a wider buffer) receives the result when given.  ``param``: the constant of an
    activation that has one."""
    code = gated_epilogue_word(activation, param)
    M = x.shape[0]
    I = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    else:
        assert out.shape == (M, I) and out.dtype == x.dtype and out.stride(1) == 1
    if M == 0:
        return out
    if _few_ok(x, w_gate_up):
        gemm_bf16_tc_few(x, w_gate_up, None, out, gated=code)
        return out
    if _small_ok(x, w_gate_up):
        gemm_bf16_small(x, w_gate_up, None, out, gated=code)
        return out
    if _tc_ok(x, w_gate_up):
        gemm_bf16_tc(x, w_gate_up, None, out, gated=code)
        return out
    gu = torch.empty((M, 2 * I), dtype=x.dtype, device=x.device)
    gemm_simt(x, w_gate_up, None, gu)
    silu_mul(gu, out, code, float(param or 0.0))
    return out


# ------------------------------------------------------------------------------------
# Mixers with a state of fixed size per request (csrc/recurrent.cu, a library of its own that is
# compiled when a model with such a mixer is first run).
def recurrent():
    global _recurrent
    if _recurrent is None:
        lib = build.recurrent_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        _recurrent = lib
    return _recurrent


def _f32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.float32 or t.stride(-1) != 1:
        raise KernelError(f"{name} must be float32 with contiguous rows")


def _scan_scratch(T: int, B: int, heads: int, dv: int, extra: int, device):
    """Scratch for a scan that may split the columns of its heads over several CTAs (a long prompt of few requests; the
    library decides by the same numbers): the unnormalised outputs, then ``extra`` floats.  None when it will not."""
    if dv <= 64 or B * heads > 74 or T < 64 * B:
        return None
    return torch.empty(T * heads * dv + extra, dtype=torch.float32, device=device)


def short_conv_silu(x: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, step, update_state: bool = True) -> torch.Tensor:
    """y[t, c] = silu(sum_j taps[c, j] * x[t - (n-1) + j, c]) over each request's run of tokens; inputs before the
    step's first token come from ``state`` (a float32 view [slots, (n-1) * C] whose rows may be strided), which then
    receives the last n-1 inputs.  ``x`` float32 [T, C] (a column slice is fine); returns float32 [T, C]."""
    _dev(x, taps, state, step.token_req, step.cu_q, step.state_slots)
    _f32(x, "x"); _f32(state, "state")
    T, C = x.shape
    n = taps.shape[1]
    assert taps.shape == (C, n) and taps.is_contiguous() and state.shape[1] == (n - 1) * C
    y = torch.empty((T, C), dtype=torch.float32, device=x.device)
    lib = recurrent()
    _check(lib, lib.coheryn_short_conv_silu(
        _ptr(x), c_long(x.stride(0)), _ptr(y), c_long(y.stride(0)), _ptr(taps), c_int(_code(taps)), c_int(n), c_int(C),
        _ptr(state), c_long(state.stride(0)), _ptr(step.token_req), _ptr(step.cu_q), _ptr(step.state_slots), c_int(T),
        c_int(step.num_requests), c_int(1 if update_state else 0), _stream()))
    return y


def gated_delta_scan(q, k, v, beta, step_pre, step_bias, rate_log, state, step, heads: int, kv_heads: int, dk: int, dv: int,
                     out: torch.Tensor, norm_weight: torch.Tensor, gate: torch.Tensor, eps: float, out_scale: float = 1.0,
                     decay_per_channel: bool = True, gate_activation: str = "sigmoid") -> None:
    """The gated delta rule over each request's run of tokens, continued from and left in ``state`` (float32 view
    [slots, heads * dk * dv]), followed by the per-head RMS norm, its weight ([dv], shared by the heads) and the sigmoid
    (or, ``gate_activation = "silu"``, the SiLU) of ``gate``.  q, k [T, kv_heads*dk] and v [T, heads*dv]: float32 with ONE
    row stride (slices of one buffer); beta [T, heads], step_pre [T, heads*dk] (``decay_per_channel``: a decay per head and
    key channel) or [T, heads] (one per head), gate [T, heads*dv]: float32 pre-activations; out [T, heads*dv] in the
    compute dtype."""
    _dev(q, k, v, beta, step_pre, step_bias, rate_log, state, out, norm_weight, gate)
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (beta, "beta"), (step_pre, "step"), (state, "state"), (gate, "gate")):
        _f32(t, name)
    assert q.stride(0) == k.stride(0) == v.stride(0)
    assert q.shape[1] == kv_heads * dk and k.shape[1] == kv_heads * dk and v.shape[1] == heads * dv
    dc = dk if decay_per_channel else 1
    assert beta.shape[1] == heads and step_pre.shape[1] == heads * dc and gate.shape[1] == heads * dv
    assert step_bias.numel() == heads * dc and rate_log.numel() == heads and norm_weight.numel() == dv
    gate_code = {"sigmoid": 0, "silu": 1}[gate_activation]
    assert state.shape[1] == heads * dk * dv and out.shape == (q.shape[0], heads * dv) and out.stride(1) == 1
    lib = recurrent()
    scratch = _scan_scratch(q.shape[0], step.num_requests, heads, dv, q.shape[0] * (2 * kv_heads * dk + heads * dk + heads), q.device)
    _check(lib, lib.coheryn_gated_delta_scan(
        _ptr(q), _ptr(k), _ptr(v), c_long(q.stride(0)), _ptr(beta), c_long(beta.stride(0)), _ptr(step_pre),
        c_long(step_pre.stride(0)), _ptr(step_bias), c_int(_code(step_bias)), _ptr(rate_log), c_int(_code(rate_log)),
        _ptr(state), c_long(state.stride(0)), _ptr(step.cu_q), _ptr(step.state_slots), c_int(step.num_requests),
        c_int(heads), c_int(kv_heads), c_int(dk), c_int(dv), _ptr(out), c_int(_code(out)), c_long(out.stride(0)),
        _ptr(norm_weight), c_int(_code(norm_weight)), c_int(0), _ptr(gate), c_long(gate.stride(0)), c_float(eps),
        c_float(out_scale), c_int(q.shape[0]), _ptr(scratch), c_long(scratch.numel() if scratch is not None else 0),
        c_int(dc), c_int(gate_code), _stream()))


def matrix_memory_scan(q, k, v, gate_i, gate_f, bias_i, bias_f, cap: float, state, step, heads: int, dk: int, dv: int,
                       out: torch.Tensor, norm_weight: torch.Tensor, gate: torch.Tensor, eps: float, out_scale: float = 1.0) -> None:
    """The stabilised matrix memory over each request's run of tokens, continued from and left in ``state`` (float32
    view [slots, heads * (dk * dv + dk + 1)]: S, n, m), followed by the per-head RMS norm, its weight [heads*dv] and the
    sigmoid of ``gate``.  q, k [T, heads*dk], v [T, heads*dv]: float32 with one row stride; gate_i, gate_f [T, heads] with
    one row stride; biases [heads]; out [T, heads*dv] in the compute dtype."""
    _dev(q, k, v, gate_i, gate_f, bias_i, bias_f, state, out, norm_weight, gate)
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (gate_i, "gate_i"), (gate_f, "gate_f"), (state, "state"), (gate, "gate")):
        _f32(t, name)
    assert q.stride(0) == k.stride(0) == v.stride(0) and gate_i.stride(0) == gate_f.stride(0)
    assert q.shape[1] == heads * dk and k.shape[1] == heads * dk and v.shape[1] == heads * dv
    assert gate_i.shape[1] == heads and gate_f.shape[1] == heads and gate.shape[1] == heads * dv
    assert bias_i.numel() == heads and bias_f.numel() == heads and bias_i.dtype == bias_f.dtype
    assert norm_weight.numel() == heads * dv
    assert state.shape[1] == heads * (dk * dv + dk + 1) and out.shape == (q.shape[0], heads * dv) and out.stride(1) == 1
    lib = recurrent()
    scratch = _scan_scratch(q.shape[0], step.num_requests, heads, dv, step.num_requests * heads * (dk + 1), q.device)
    _check(lib, lib.coheryn_matrix_memory_scan(
        _ptr(q), _ptr(k), _ptr(v), c_long(q.stride(0)), _ptr(gate_i), _ptr(gate_f), c_long(gate_i.stride(0)), _ptr(bias_i),
        _ptr(bias_f), c_int(_code(bias_i)), c_float(cap), _ptr(state), c_long(state.stride(0)), _ptr(step.cu_q),
        _ptr(step.state_slots), c_int(step.num_requests), c_int(heads), c_int(dk), c_int(dv), _ptr(out), c_int(_code(out)),
        c_long(out.stride(0)), _ptr(norm_weight), c_int(_code(norm_weight)), c_int(dv), _ptr(gate), c_long(gate.stride(0)),
        c_float(eps), c_float(out_scale), c_int(q.shape[0]), _ptr(scratch), c_long(scratch.numel() if scratch is not None else 0),
        _stream()))


def qk_norm_kv_write(q, k, v, q_weight, k_weight, eps: float, slots, k_cache, v_cache, num_heads: int, num_kv_heads: int,
                     dk: int, dv: int, page_size: int, dtype: torch.dtype, v_scale: float = 1.0) -> torch.Tensor:
    """Queries and keys divided by the root mean square of their WHOLE projection (all heads at once) and multiplied by
    a weight (skipped when ``q_weight`` is None); keys and values written into cache pages ``[page, kv head, slot, size]``
    at ``slots`` (None: nothing is written), the values multiplied by ``v_scale``.  q, k, v: float32 with one row stride.
    Returns q [T, heads*dk] in ``dtype``."""
    _dev(q, k, v, q_weight, k_weight, slots, k_cache, v_cache)
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _f32(t, name)
    assert q.stride(0) == k.stride(0) == v.stride(0)
    T = q.shape[0]
    assert q.shape[1] == num_heads * dk and k.shape[1] == num_kv_heads * dk and v.shape[1] == num_kv_heads * dv
    normalise = q_weight is not None
    if normalise:
        assert q_weight.numel() == num_heads * dk and k_weight.numel() == num_kv_heads * dk and q_weight.dtype == k_weight.dtype
    if slots is not None:
        _i32(slots, "slots")
        assert k_cache.dtype == dtype and v_cache.dtype == dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, dk) and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, dv)
    q_out = torch.empty((T, num_heads * dk), dtype=dtype, device=q.device)
    lib = recurrent()
    _check(lib, lib.coheryn_qk_norm_kv_write(
        _ptr(q), _ptr(k), _ptr(v), c_long(q.stride(0)), _ptr(q_weight), _ptr(k_weight),
        c_int(_code(q_weight) if normalise else F32), c_float(eps), c_int(1 if normalise else 0), _ptr(q_out),
        c_int(_CODES[dtype]), c_long(q_out.stride(0)), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(dk), c_int(dv), c_int(page_size), c_float(v_scale), _stream()))
    return q_out


# ------------------------------------------------------------------------------------
# Attention with several score maps per head, a mask by chunks, a sink and a normalised output, and the kernel that
# prepares its queries and keys (csrc/attention_variants.cu, a library of its own that is compiled when a model with
# such a mixer is first run).
_variants = None


def variants():
    global _variants
    if _variants is None:
        lib = build.variants_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        _variants = lib
    return _variants


def unit_norm_rope_kv_write(q, k, v, q_weight, k_weight, eps: float, positions, freq, rot: int, rot_scale: float, slots,
                            k_cache, v_cache, q_units: int, k_units: int, num_kv_heads: int, dk: int, dv: int,
                            page_size: int, dtype: torch.dtype) -> torch.Tensor:
    """Queries and keys in units of ``dk`` channels (a head has one unit per score map): each unit divided by its root
    mean square and multiplied by a weight [dk] shared by the units (skipped when ``q_weight`` is None), then its first
    ``rot`` channels rotated by the token's position (pairs (i, i + rot/2); ``freq`` float32 [rot/2, 2] holds each pair's
    frequency as a high and a low part, angle = position * frequency; cos and sin are multiplied by ``rot_scale``).  Keys
    ([page, kv head, slot, k_units / kv heads * dk]) and values ([page, kv head, slot, dv]) go to the cache at ``slots``
    (None: only the queries are made; k and v are not read).  q, k, v: float32 with one row stride.  Returns q
    [T, q_units * dk] in ``dtype``."""
    _dev(q, k, v, q_weight, k_weight, positions, freq, slots, k_cache, v_cache)
    _f32(q, "q")
    T = q.shape[0]
    assert q.shape[1] == q_units * dk
    if slots is not None:
        _f32(k, "k"); _f32(v, "v"); _i32(slots, "slots")
        assert q.stride(0) == k.stride(0) == v.stride(0)
        assert k.shape[1] == k_units * dk and v.shape[1] == num_kv_heads * dv
        assert k_cache.dtype == dtype and v_cache.dtype == dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, k_units // num_kv_heads * dk)
        assert tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, dv)
    normalise = q_weight is not None
    if normalise:
        assert q_weight.numel() == dk and k_weight.numel() == dk and q_weight.dtype == k_weight.dtype
    if rot:
        _i32(positions, "positions")
        assert freq.dtype == torch.float32 and freq.is_contiguous() and tuple(freq.shape) == (rot // 2, 2)
    q_out = torch.empty((T, q_units * dk), dtype=dtype, device=q.device)
    lib = variants()
    _check(lib, lib.coheryn_unit_norm_rope_kv_write(
        _ptr(q), _ptr(k), _ptr(v), c_long(q.stride(0)), _ptr(q_weight), _ptr(k_weight),
        c_int(_code(q_weight) if normalise else F32), c_float(eps), c_int(1 if normalise else 0), _ptr(positions), _ptr(freq),
        c_int(rot), c_float(rot_scale), _ptr(q_out), c_int(_CODES[dtype]), c_long(q_out.stride(0)), _ptr(slots),
        _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(q_units), c_int(k_units), c_int(num_kv_heads), c_int(dk), c_int(dv),
        c_int(page_size), _stream()))
    return q_out


_maps_libs = {}
# Whether bfloat16 steps take the tensor-core kernels of the attention with score maps (the float32-arithmetic kernel
# otherwise); for tests and measurements.
MAPS_TC = os.environ.get("COHERYN_MAPS_TC", "1") != "0"


def set_maps_tc(on: bool) -> None:
    global MAPS_TC
    MAPS_TC = bool(on)


def maps_attention_lib(dk: int, dv: int, maps: int, values_in_keys: bool = False):
    key = (dk, dv, maps) + ((True,) if values_in_keys else ())
    lib = _maps_libs.get(key)
    if lib is None:
        lib = build.maps_attention_library(dk, dv, maps, values_in_keys)
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        lib.coheryn_maps_scratch_floats.restype = ctypes.c_long
        got = [ctypes.c_int(), ctypes.c_int(), ctypes.c_int()]
        lib.coheryn_maps_shape(*[ctypes.byref(g) for g in got])
        if tuple(g.value for g in got) != key[:3] or bool(lib.coheryn_maps_values_in_keys()) != bool(values_in_keys):
            raise KernelError(f"the attention library was built for {tuple(g.value for g in got)}, not {key}")
        _maps_libs[key] = lib
    return lib


def attention_maps(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int,
                   num_heads: int, num_kv_heads: int, dk: int, dv: int, maps: int, page_size: int, window: Optional[int],
                   chunk: Optional[int], sink: bool, scale: float, lam: float, head_norm: bool, eps: float,
                   out_scale: float, force_simple: bool = False, sink_scores: Optional[torch.Tensor] = None,
                   values_in_keys: bool = False, head_gates: Optional[torch.Tensor] = None) -> None:
    """Attention of every token of the step over its request's cache pages of ``group`` with ``maps`` score maps per
    head (output a_0 - lam * a_1 for two), a mask by chunks (``chunk``: position i sees j <= i with i // chunk ==
    j // chunk), by a window or causal, an optional sink term in the softmax's denominator, the head's output divided
    by its root mean square over dv (``head_norm``) and multiplied by ``out_scale``.  q [T, heads * maps * dk],
    out [T, heads * dv]; float32 arithmetic on either storage type.  ``sink_scores`` (float32 [heads]): the sink's score
    per head instead of 0.  ``values_in_keys``: the values are the first dv channels of the key rows (``v_cache`` is not
    read).  ``head_gates`` (float32 [T, heads]): head h's output of token t is multiplied by sigmoid(head_gates[t, h])."""
    block_tables = step.block_tables[group]
    if head_gates is not None:
        _dev(head_gates)
        _f32(head_gates, "head_gates")
        assert head_gates.shape == (q.shape[0], num_heads)
    if sink_scores is not None:
        _dev(sink_scores)
        assert sink and sink_scores.dtype == torch.float32 and sink_scores.is_contiguous() and sink_scores.numel() == num_heads
    if values_in_keys:
        v_cache = k_cache
    _dev(q, out, k_cache, v_cache, block_tables, step.token_req, step.positions)
    _i32(block_tables, "block_tables")
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * maps * dk and out.shape == (T, num_heads * dv)
    assert k_cache.dtype == q.dtype and out.dtype == q.dtype and v_cache.dtype == q.dtype
    q_lens = getattr(step, "q_lens", None)
    # what the tensor-core kernels keep in shared memory: 64 query rows, two tiles of 32 key rows (and of value rows when
    # those are rows of their own), up to 4,096 block-table entries; values wider than 256 channels go in chunks
    tc_smem = 2 * (128 * (maps * dk + 8) + (0 if values_in_keys else 64 * (dv + 8))) + 16384
    fast = (MAPS_TC and not force_simple and q.dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and 16 <= dk <= 1024
            and 16 <= dv <= 1024 and tc_smem <= 227 * 1024 and not (head_norm and dv > 256)
            and q_lens and getattr(step, "max_kv_len", None) and getattr(step, "cu_q", None) is not None
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)
    if fast:
        # rows that are whole runs of consecutive positions per request, ending at the request's last position
        _i32(step.cu_q, "cu_q"); _i32(step.kv_lens, "kv_lens")
        lib = maps_attention_lib(dk, dv, maps, values_in_keys)
        B = len(q_lens)
        single = any(n == 1 for n in q_lens) and num_heads // num_kv_heads <= 16
        floats = int(lib.coheryn_maps_scratch_floats(c_int(B), c_int(num_heads), c_int(step.max_kv_len), c_int(window or 0),
                                                     c_int(chunk or 0))) if single else 0
        scratch = torch.empty(floats, dtype=torch.float32, device=q.device) if floats else None
        _check(lib, lib.coheryn_attention_maps_bf16(
            _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            c_int(block_tables.shape[1]), _ptr(step.cu_q), _ptr(step.kv_lens), c_int(B), c_int(num_heads), c_int(num_kv_heads),
            c_int(page_size), c_int(window or 0), c_int(chunk or 0), c_int(1 if sink else 0), c_float(scale), c_float(lam),
            c_int(1 if head_norm else 0), c_float(eps), c_float(out_scale), c_int(max(q_lens)), c_int(step.max_kv_len),
            c_int(1 if any(n == 1 for n in q_lens) else 0), c_int(1 if any(n > 1 for n in q_lens) else 0), _ptr(scratch),
            c_long(floats), _ptr(sink_scores), _ptr(head_gates), c_long(head_gates.stride(0) if head_gates is not None else 0),
            _stream()))
        return
    lib = variants()
    _check(lib, lib.coheryn_attention_maps(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(_code(q)),
        _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(step.token_req), _ptr(step.positions), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(dk), c_int(dv), c_int(maps), c_int(page_size), c_int(window or 0),
        c_int(chunk or 0), c_int(1 if sink else 0), c_float(scale), c_float(lam), c_int(1 if head_norm else 0), c_float(eps),
        c_float(out_scale), _ptr(sink_scores), c_int(1 if values_in_keys else 0), _stream()))
    if head_gates is not None:
        head_gate(out, head_gates, num_heads)


# ------------------------------------------------------------------------------------
# Kernels on the residual stream of blocks that normalise after the sum, and an embedding with a hashed pair row
# (csrc/stream_ops.cu, part of the core library).
def embed_pair(table: torch.Tensor, pair: Optional[torch.Tensor], step, last_ids: Optional[torch.Tensor], mul_prev: int,
               mul_cur: int, buckets: int, scale: Optional[float], norm_weight: Optional[torch.Tensor], eps: float,
               out: torch.Tensor, out_cast: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """out[t] = table[id_t] * scale + pair[(prev_t * mul_prev + id_t * mul_cur) mod buckets] (row ``buckets`` at position
    0), then divided by its root mean square and multiplied by ``norm_weight`` when given; float32, with a copy in
    ``out_cast``'s dtype when given.  prev_t is the step's token before t, or for the first token of a request's portion
    ``last_ids[state slot of the request]`` (int32 [slots, 1]): the last token of its previous step."""
    ids = step.token_ids
    _dev(table, pair, ids, last_ids, norm_weight, out, out_cast, status)
    _i32(ids, "ids")
    V, H = table.shape
    T = ids.numel()
    assert out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous() and table.is_contiguous()
    if pair is not None:
        assert pair.shape == (buckets + 1, H) and pair.dtype == table.dtype and pair.is_contiguous()
        assert last_ids is not None and last_ids.dtype == torch.int32 and last_ids.is_contiguous()
    if out_cast is not None:
        assert out_cast.shape == (T, H) and out_cast.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_embed_pair(
        _ptr(table), _ptr(pair), c_int(_code(table)), _ptr(ids), _ptr(step.positions), _ptr(step.token_req), _ptr(step.cu_q),
        _ptr(step.state_slots), _ptr(last_ids), ctypes.c_longlong(mul_prev % buckets if pair is not None else 0),
        ctypes.c_longlong(mul_cur % buckets if pair is not None else 0), ctypes.c_longlong(buckets if pair is not None else 1),
        c_float(1.0 if scale is None else scale), _ptr(norm_weight), c_int(_code(norm_weight) if norm_weight is not None else F32),
        c_float(eps), _ptr(out), _ptr(out_cast), c_int(_code(out_cast) if out_cast is not None else F32), c_int(T), c_int(H),
        c_int(V), _ptr(status), _stream()))


def store_last_ids(step, last_ids: torch.Tensor) -> None:
    """last_ids[state slot of request b] = the last token of b's portion in this step."""
    _dev(step.token_ids, last_ids)
    lib = core()
    _check(lib, lib.coheryn_store_last_ids(_ptr(step.token_ids), _ptr(step.cu_q), _ptr(step.state_slots), _ptr(last_ids),
                                           c_int(step.num_requests), _stream()))


def scaled_add_norm(x: torch.Tensor, parts: torch.Tensor, alpha: float, weight: torch.Tensor, eps: float,
                    out_cast: Optional[torch.Tensor] = None, normed_summand: bool = False) -> None:
    """In place on the float32 stream x [n, H], with d the sum of ``parts`` (float32 [n, H] or a stack [P, n, H]):
    x <- (alpha x + d) / rms(alpha x + d) * weight, or with ``normed_summand`` x <- x + d / rms(d) * weight;
    ``out_cast`` receives a copy of the new x in its dtype."""
    _dev(x, parts, weight, out_cast)
    if parts.dim() == 2:
        parts = parts.unsqueeze(0)
    P, n, H = parts.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (n, H)
    assert parts.dtype == torch.float32 and parts.stride(2) == 1 and weight.shape == (H,) and weight.is_contiguous()
    if out_cast is not None:
        assert out_cast.shape == (n, H) and out_cast.is_contiguous()
    lib = core()
    _check(lib, lib.coheryn_scaled_add_norm(
        _ptr(x), _ptr(parts), c_int(P), c_long(parts.stride(0)), c_long(parts.stride(1)), c_float(alpha),
        c_int(1 if normed_summand else 0), _ptr(weight), c_int(_code(weight)), c_float(eps), _ptr(out_cast),
        c_int(_code(out_cast) if out_cast is not None else F32), c_int(n), c_int(H), _stream()))


def gated_table_mul(z: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j]."""
    _dev(z, table, ids, out)
    _i32(ids, "ids")
    T, n = z.shape
    assert z.stride(1) == 1 and table.is_contiguous() and out.is_contiguous() and out.shape == (T, n) and out.dtype == table.dtype
    assert 0 <= col0 and col0 + n <= table.shape[1]
    lib = core()
    _check(lib, lib.coheryn_gated_table_mul(_ptr(z), c_int(_code(z)), c_long(z.stride(0)), _ptr(table), c_int(_code(table)),
                                            c_long(table.stride(0)), c_int(col0), _ptr(ids), _ptr(out), c_int(T), c_int(n),
                                            c_int(table.shape[0]), _stream()))


def copy_head_columns(src: torch.Tensor, src_head: int, src_off: int, dst: torch.Tensor, dst_head: int, dst_off: int, n: int,
                      heads: int) -> None:
    """dst[t, h * dst_head + dst_off + j] = src[t, h * src_head + src_off + j] for j < n and every head h (``src_head`` 0:
    the same block for every head); matrices of 16-bit elements with contiguous rows."""
    _dev(src, dst)
    T = src.shape[0]
    assert src.dtype == dst.dtype and src.element_size() == 2 and src.stride(1) == 1 and dst.stride(1) == 1 and dst.shape[0] == T
    assert (heads - 1) * src_head + src_off + n <= src.shape[1] and (heads - 1) * dst_head + dst_off + n <= dst.shape[1]
    lib = core()
    _check(lib, lib.coheryn_copy_head_columns(_ptr(src), c_long(src.stride(0)), c_long(src_head), c_long(src_off), _ptr(dst),
                                              c_long(dst.stride(0)), c_long(dst_head), c_long(dst_off), c_int(n), c_int(heads),
                                              c_int(T), _stream()))


def head_gate(x: torch.Tensor, logits: torch.Tensor, heads: int) -> None:
    """In place: the columns of head h of ``x`` [T, heads * n] times sigmoid(logits[t, h]); ``logits`` float32 [T, heads]."""
    _dev(x, logits)
    _f32(logits, "logits")
    T = x.shape[0]
    assert x.stride(1) == 1 and logits.stride(1) == 1 and x.shape[1] % heads == 0 and logits.shape == (T, heads)
    lib = core()
    _check(lib, lib.coheryn_head_gate(_ptr(x), c_int(_code(x)), c_long(x.stride(0)), _ptr(logits), c_long(logits.stride(0)),
                                      c_int(x.shape[1] // heads), c_int(heads), c_int(T), _stream()))


# A latent attention expands the cached rows of whole prompts into keys and values per head when the step brings at
# least this many tokens and attending in the latent space would multiply at least RATIO times the channels per score.
LATENT_EXPAND_MIN_TOKENS = int(os.environ.get("COHERYN_LATENT_EXPAND_MIN_TOKENS", "512"))
LATENT_EXPAND_RATIO = float(os.environ.get("COHERYN_LATENT_EXPAND_RATIO", "1.5"))


# ------------------------------------------------------------------------------------
# Routed experts and products over groups of rows (csrc/routed.cu, a library of its own that is compiled when a model
# with such a part is first run).
def routed():
    global _routed
    if _routed is None:
        lib = build.routed_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        _routed = lib
    return _routed


GROUPED_TC = os.environ.get("COHERYN_GROUPED_TC", "1") != "0"


def set_grouped_tc(on: bool) -> None:
    """Whether bfloat16 grouped products take the tensor cores (the FMA kernel otherwise); for tests and measurements."""
    global GROUPED_TC
    GROUPED_TC = bool(on)


def route_select(logits: torch.Tensor, correction: Optional[torch.Tensor], n_groups: int, keep: int, top: int,
                 scale: float, chosen_softmax: bool = False):
    """From router logits (float32 [T, N]) the chosen outputs per token (int32 [T, top], by choice score = softmax +
    correction, only within the ``keep`` best of ``n_groups`` equal groups of neighbours) and their weights (float32
    [T, top]: the chosen probabilities over their sum, times ``scale``).  ``chosen_softmax``: the choice scores are the
    logits themselves plus ``correction`` (a bias), and the weights the softmax over the chosen scores alone."""
    _dev(logits, correction)
    _f32(logits, "logits")
    T, N = logits.shape
    assert logits.stride(1) == 1
    if correction is not None:
        assert correction.shape == (N,) and correction.is_contiguous()
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    lib = routed()
    _check(lib, lib.coheryn_route_select(_ptr(logits), c_long(logits.stride(0)), _ptr(correction),
                                         c_int(_code(correction) if correction is not None else F32), c_int(T), c_int(N),
                                         c_int(n_groups), c_int(keep), c_int(top), c_float(scale),
                                         c_int(1 if chosen_softmax else 0), _ptr(ids), _ptr(weights), _stream()))
    return ids, weights


class RoutedRows:
    """The (token, choice) pairs of a step ordered by expert, as ``route_sort`` leaves them on the device."""
    __slots__ = ("n", "experts", "offsets", "row_of", "token_of", "tile_group", "tile_row0", "n_tiles", "max_tiles", "tile_rows")


def route_sort(ids: torch.Tensor, experts: int, wide_tiles: bool = False) -> RoutedRows:
    """Order the pairs whose id names one of the first ``experts`` outputs by expert.  ``wide_tiles``: row tiles for
    ``gemm_bf16_tc_grouped`` instead of ``grouped_linear``; every index of the book is then a valid one (rows that no pair
    takes name token 0)."""
    _dev(ids)
    _i32(ids, "ids")
    T, top = ids.shape
    n = T * top
    lib = routed()
    bm = int(core().coheryn_gemm_tc_grouped_tile_rows()) if wide_tiles else int(lib.coheryn_grouped_tile_rows())
    r = RoutedRows()
    r.n, r.experts, r.max_tiles, r.tile_rows = n, experts, n // bm + experts, bm
    book = (torch.zeros if wide_tiles else torch.empty)(experts + 1 + 2 * n + 2 * r.max_tiles + 1, dtype=torch.int32, device=ids.device)
    o = 0
    r.offsets = book[o:o + experts + 1]; o += experts + 1
    r.row_of = book[o:o + n]; o += n
    r.token_of = book[o:o + n]; o += n
    r.tile_group = book[o:o + r.max_tiles]; o += r.max_tiles
    r.tile_row0 = book[o:o + r.max_tiles]; o += r.max_tiles
    r.n_tiles = book[o:o + 1]
    _check(lib, lib.coheryn_route_sort(_ptr(ids), c_int(n), c_int(top), c_int(experts), _ptr(r.offsets), _ptr(r.row_of),
                                       _ptr(r.token_of), _ptr(r.tile_group), _ptr(r.tile_row0), _ptr(r.n_tiles),
                                       c_int(bm if wide_tiles else 0), _stream()))
    return r


# Pairs per expert (on average) from which the routed products take the TMA + tcgen05 kernel: its row tiles are 128 rows.
GROUPED_TC_MIN_ROWS = int(os.environ.get("COHERYN_GROUPED_TC_MIN_ROWS", "48"))


def grouped_tc_suits(x: torch.Tensor, pairs: int, experts: int, *weights: torch.Tensor) -> bool:
    """Whether the routed products of ``pairs`` (token, choice) pairs over ``experts`` matrices run on the TMA + tcgen05
    kernel: bfloat16, inner sizes in multiples of 8, and rows enough to fill its tiles."""
    return (GROUPED_TC and x.dtype == torch.bfloat16 and pairs >= GROUPED_TC_MIN_ROWS * experts
            and all(w.dtype == torch.bfloat16 and w.shape[2] % 8 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0
                    for w in weights))


def gemm_bf16_tc_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: RoutedRows, epilogue: int = 0) -> None:
    """out[r] = a[r] . w[expert of sorted row r]^T for the rows of ``route_sort(..., wide_tiles=True)``, on the TMA +
    tcgen05 kernel of ``csrc/gemm_tc.cu``; ``a`` [pairs, K] bfloat16 in sorted order, ``w`` [G, N, K]; ``epilogue``: a gated
    epilogue word (``out`` then has N / 2 columns).  Rows beyond the last expert's are not written."""
    _dev(a, w, out)
    G, N, K = w.shape
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and a.shape == (rows.n, K)
    assert a.stride(1) == 1 and out.stride(1) == 1 and out.shape == (rows.n, N // 2 if epilogue else N) and G == rows.experts
    lib = core()
    assert rows.tile_rows == int(lib.coheryn_gemm_tc_grouped_tile_rows())
    _check(lib, lib.coheryn_gemm_bf16_tc_grouped(
        _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(rows.n), c_int(N), c_int(K), c_int(G), c_long(a.stride(0)),
        c_long(out.stride(0)), c_int(int(epilogue)), _ptr(rows.tile_group), _ptr(rows.tile_row0), _ptr(rows.offsets),
        _ptr(rows.n_tiles), c_int(rows.max_tiles), _ptr(tc_status(a.device)), _stream()))


def grouped_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: Optional[RoutedRows] = None,
                   gather: bool = False, a_col: int = 0, c_col: int = 0, epilogue: int = 0,
                   factor: Optional[torch.Tensor] = None, factor_sigmoid: bool = False) -> None:
    """Products of groups of rows with a matrix per group; ``w`` [G, N, K].

    With ``rows`` (from ``route_sort``) group g is expert g's rows of the sorted order: row r reads a[token_of[r]] when
    ``gather`` (else a[r]) and writes out[r].  Without, every row of ``a`` belongs to every group: group g reads columns
    g * a_col .. g * a_col + K of ``a`` and writes columns g * c_col .. of ``out``.  ``epilogue``: a gated epilogue word
    (output columns (2j, 2j+1) are gate and up; ``out`` then has N / 2 columns per group).  ``factor`` float32 [rows, G]:
    every output of (row, group) is multiplied by it (through a sigmoid when ``factor_sigmoid``)."""
    _dev(a, w, out, factor)
    G, N, K = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1
    if factor is not None:
        _f32(factor, "factor")
        assert factor.stride(1) == 1 and factor.shape[1] == G
    lib = routed()
    M = a.shape[0] if rows is None else rows.n
    _check(lib, lib.coheryn_grouped_linear(
        _ptr(a), c_int(_code(a)), c_long(a.stride(0)), c_long(a_col), _ptr(w), c_int(_code(w)), c_long(N * K), _ptr(out),
        c_int(_code(out)), c_long(out.stride(0)), c_long(c_col),
        _ptr(rows.token_of) if rows is not None and gather else c_void_p(0),
        _ptr(rows.tile_group) if rows is not None else c_void_p(0), _ptr(rows.tile_row0) if rows is not None else c_void_p(0),
        _ptr(rows.offsets) if rows is not None else c_void_p(0), _ptr(rows.n_tiles) if rows is not None else c_void_p(0),
        c_int(rows.max_tiles if rows is not None else 0), _ptr(factor), c_long(factor.stride(0) if factor is not None else 0),
        c_int(1 if factor_sigmoid else 0), c_int(M), c_int(N), c_int(K), c_int(G), c_int(epilogue),
        c_int(1 if GROUPED_TC else 0), _stream()))


def route_combine(y: torch.Tensor, h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, rows: RoutedRows,
                  out: torch.Tensor, extra: Optional[torch.Tensor] = None, extra_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over the token's choices in order of weight * (y[row of the pair] for an expert, h[t] for an
    identity output); y float32 in sorted order, out float32 [T, H].  ``extra`` (float32 [T, H]) is one more summand,
    added last, multiplied by sigmoid(extra_gate[t]) when ``extra_gate`` (float32 [T], may be a strided column) is given."""
    _dev(y, h, ids, weights, out, extra, extra_gate)
    if extra is not None:
        _f32(extra, "extra")
        assert extra.shape == out.shape and extra.stride(1) == 1
    if extra_gate is not None:
        assert extra is not None and extra_gate.dtype == torch.float32 and extra_gate.shape == (out.shape[0],)
    _f32(y, "y"); _f32(out, "out")
    T, top = ids.shape
    H = out.shape[1]
    assert y.stride(1) == 1 and h.stride(1) == 1 and out.is_contiguous() and h.shape == (T, H)
    lib = routed()
    _check(lib, lib.coheryn_route_combine(_ptr(y), c_long(y.stride(0)), _ptr(h), c_int(_code(h)), c_long(h.stride(0)), _ptr(ids),
                                          _ptr(weights), _ptr(rows.row_of), c_int(top), c_int(rows.experts), _ptr(out), c_int(T),
                                          c_int(H), _ptr(extra), c_long(extra.stride(0) if extra is not None else 0),
                                          _ptr(extra_gate), c_long(extra_gate.stride(0) if extra_gate is not None else 0),
                                          _stream()))


def latent_prepare(proj: torch.Tensor, heads: int, dim: int, rd: int, rank: int, kv_col: Optional[int],
                   norm_weight: Optional[torch.Tensor], eps: float, positions: torch.Tensor, freq: Optional[torch.Tensor],
                   rot: int, rot_scale: float, slots: Optional[torch.Tensor], cache: Optional[torch.Tensor], page_size: int,
                   dtype: torch.dtype):
    """The step of a latent attention in front of its scores.  ``proj`` float32 [T, ...]: queries head by head as
    [dim plain | rd rotated] from column 0 and, from column ``kv_col`` (None: a layer that reads another's cache),
    ``rank`` latent channels and ``rd`` key channels.  Returns (q_plain [T, heads * dim], q_wide [T, heads * (rank + rd)]
    whose last rd columns per head hold the rotated query part; the first ``rank`` are left for the product that
    carries the plain part into the latent space), both in ``dtype``; writes the cache rows [latent normalised |
    rotated key] ([page, 1, page_size, rank + rd]) at ``slots``."""
    _dev(proj, norm_weight, positions, freq, slots, cache)
    _f32(proj, "proj")
    T = proj.shape[0]
    assert proj.stride(1) == 1
    write = kv_col is not None
    if write:
        _i32(slots, "slots")
        assert cache.dtype == dtype and cache.is_contiguous() and tuple(cache.shape[1:]) == (1, page_size, rank + rd)
        assert norm_weight.shape == (rank,) and norm_weight.is_contiguous()
    if rot:
        _i32(positions, "positions")
        assert freq.dtype == torch.float32 and freq.is_contiguous() and tuple(freq.shape) == (rot // 2, 2)
    q_plain = torch.empty((T, heads * dim), dtype=dtype, device=proj.device)
    q_wide = torch.empty((T, heads * (rank + rd)), dtype=dtype, device=proj.device)
    lib = variants()
    _check(lib, lib.coheryn_latent_prepare(
        _ptr(proj), _ptr(proj[:, kv_col:]) if write else c_void_p(0), c_long(proj.stride(0)), _ptr(norm_weight) if write else c_void_p(0),
        c_int(_code(norm_weight) if write else F32), c_float(eps), _ptr(positions), _ptr(freq), c_int(rot), c_float(rot_scale),
        _ptr(q_plain), _ptr(q_wide), c_int(_CODES[dtype]), _ptr(slots) if write else c_void_p(0),
        _ptr(cache) if write else c_void_p(0), c_int(T), c_int(heads), c_int(dim), c_int(rd), c_int(rank), c_int(page_size),
        _stream()))
    return q_plain, q_wide


# ------------------------------------------------------------------------------------
# A gated linear recurrence per channel (csrc/linear_recurrence.cu, a library of its own that is compiled when a model
# with such a mixer is first run).
_linear_recurrence = None


def linear_recurrence():
    global _linear_recurrence
    if _linear_recurrence is None:
        lib = build.linear_recurrence_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        lib.coheryn_gated_scan_scratch.restype = ctypes.c_long
        _linear_recurrence = lib
    return _linear_recurrence


def conv_bias(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, step,
              update_state: bool = True) -> torch.Tensor:
    """y[t, c] = bias[c] + sum_j taps[c, j] * x[t - (n-1) + j, c] over each request's run of tokens, no activation; inputs
    before the step's first token come from ``state`` (a float32 view [slots, (n-1) * C] whose rows may be strided), which
    then receives the last n-1 inputs.  ``x`` float32 [T, C] (a column slice is fine); returns float32 [T, C]."""
    _dev(x, taps, bias, state, step.token_req, step.cu_q, step.state_slots)
    _f32(x, "x"); _f32(state, "state")
    T, C = x.shape
    n = taps.shape[1]
    assert taps.shape == (C, n) and taps.is_contiguous() and state.shape[1] == (n - 1) * C
    if bias is not None:
        assert bias.shape == (C,) and bias.is_contiguous()
    y = torch.empty((T, C), dtype=torch.float32, device=x.device)
    lib = linear_recurrence()
    _check(lib, lib.coheryn_conv_bias(
        _ptr(x), c_long(x.stride(0)), _ptr(y), c_long(y.stride(0)), _ptr(taps), c_int(_code(taps)), _ptr(bias),
        c_int(_code(bias) if bias is not None else F32), c_int(n), c_int(C), _ptr(state), c_long(state.stride(0)),
        _ptr(step.token_req), _ptr(step.cu_q), _ptr(step.state_slots), c_int(T), c_int(step.num_requests),
        c_int(1 if update_state else 0), _stream()))
    return y


def gated_scan(gates: torch.Tensor, bias_r: Optional[torch.Tensor], bias_i: Optional[torch.Tensor], u: torch.Tensor,
               y: torch.Tensor, lam: torch.Tensor, rate: float, block: int, state: torch.Tensor, step,
               out: torch.Tensor) -> None:
    """S_t = a S_(t-1) + sqrt(1 - a^2) * i * u per channel and request, a = exp(-rate * r * softplus(lam)), r and i the
    sigmoids of the gates' pre-activations (+ biases); out_t = S_t * gelu_tanh(y_t).  ``gates`` float32 [T, 2 C]: per block
    of ``block`` channels [r | i]; ``u``, ``y`` float32 [T, C]; ``state`` float32 [slots, C] (rows may be strided), read at a
    request's first token of the step and written at its last; ``out`` [T, C] float32 or bfloat16."""
    _dev(gates, bias_r, bias_i, u, y, lam, state, out, step.token_req, step.cu_q, step.state_slots)
    _f32(gates, "gates"); _f32(u, "u"); _f32(y, "y"); _f32(state, "state")
    T, C = u.shape
    assert gates.shape == (T, 2 * C) and y.shape == (T, C) and out.shape == (T, C) and out.stride(1) == 1
    assert lam.shape == (C,) and lam.is_contiguous() and state.shape[1] == C
    if bias_r is not None:
        assert bias_i is not None and bias_r.dtype == bias_i.dtype and bias_r.numel() == C and bias_i.numel() == C
        assert bias_r.is_contiguous() and bias_i.is_contiguous()
    lib = linear_recurrence()
    B = step.num_requests
    floats = int(lib.coheryn_gated_scan_scratch(c_int(T), c_int(B), c_int(C)))
    scratch = torch.empty(floats, dtype=torch.float32, device=u.device)
    _check(lib, lib.coheryn_gated_scan(
        _ptr(gates), c_long(gates.stride(0)), _ptr(bias_r), _ptr(bias_i), c_int(_code(bias_r) if bias_r is not None else F32),
        _ptr(u), c_long(u.stride(0)), _ptr(y), c_long(y.stride(0)), _ptr(lam), c_int(_code(lam)), c_float(rate), c_int(block),
        _ptr(state), c_long(state.stride(0)), _ptr(step.token_req), _ptr(step.cu_q), _ptr(step.state_slots), _ptr(scratch),
        c_long(floats), _ptr(out), c_int(_code(out)), c_long(out.stride(0)), c_int(T), c_int(B), c_int(C), _stream()))


# ------------------------------------------------------------------------------------
# Window attention over positions and block means (csrc/attention_pooled.cu, a library of its own that is compiled when
# a model with such a mixer is first run).
_pooled = None


def pooled():
    global _pooled
    if _pooled is None:
        lib = build.pooled_attention_library()
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        _pooled = lib
    return _pooled


_pooled_tc_libs = {}
# Whether bfloat16 prompt portions take the tensor-core kernel of the window attention (the float32-arithmetic kernel
# otherwise); for tests and measurements.
POOLED_TC = os.environ.get("COHERYN_POOLED_TC", "1") != "0"
# From how many rows of its longest request a step takes the tensor-core kernel (its row tiles hold 64).
POOLED_TC_MIN_ROWS = int(os.environ.get("COHERYN_POOLED_TC_MIN_ROWS", "5"))


def set_pooled_tc(on: bool) -> None:
    global POOLED_TC
    POOLED_TC = bool(on)


def pooled_tc_lib(dk: int, dv: int):
    lib = _pooled_tc_libs.get((dk, dv))
    if lib is None:
        lib = build.pooled_attention_tc_library(dk, dv)
        lib.coheryn_last_error.restype = ctypes.c_char_p
        lib.coheryn_launch_count.restype = ctypes.c_ulonglong
        got = [ctypes.c_int(), ctypes.c_int()]
        lib.coheryn_pooled_tc_shape(*[ctypes.byref(g) for g in got])
        if tuple(g.value for g in got) != (dk, dv):
            raise KernelError(f"the window attention library was built for {tuple(g.value for g in got)}, not {(dk, dv)}")
        _pooled_tc_libs[(dk, dv)] = lib
    return lib


def pooled_prepare(proj: torch.Tensor, positions: torch.Tensor, freq_k: Optional[torch.Tensor], rot: int,
                   freq_v: Optional[torch.Tensor], slots: Optional[torch.Tensor], k_cache, v_cache, heads: int, kv_heads: int,
                   dk: int, dv: int, page_size: int, dtype: torch.dtype) -> torch.Tensor:
    """``proj`` float32 [T, >= heads * dk + kv_heads * (dk + dv)]: queries, keys, values side by side.  The first ``rot``
    channels of every query and key head are rotated by the row's position (``freq_k`` float32 [rot/2, 2], high and low
    part of each pair's frequency), all ``dv`` channels of every value head by ``freq_v`` ([dv/2, 2]; None: values stay as
    they are); keys and values go to the cache at ``slots`` (None: only queries are made).  Returns q [T, heads * dk]."""
    _dev(proj, positions, freq_k, freq_v, slots, k_cache, v_cache)
    _f32(proj, "proj"); _i32(positions, "positions")
    T = proj.shape[0]
    assert proj.shape[1] >= heads * dk + (kv_heads * (dk + dv) if slots is not None else 0)
    for f, n in ((freq_k, rot), (freq_v, dv)):
        if f is not None:
            assert f.dtype == torch.float32 and f.is_contiguous() and tuple(f.shape) == (n // 2, 2)
    if slots is not None:
        _i32(slots, "slots")
        assert k_cache.dtype == dtype and v_cache.dtype == dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (kv_heads, page_size, dk) and tuple(v_cache.shape[1:]) == (kv_heads, page_size, dv)
    q = torch.empty((T, heads * dk), dtype=dtype, device=proj.device)
    lib = pooled()
    _check(lib, lib.coheryn_pooled_prepare(
        _ptr(proj), c_long(proj.stride(0)), _ptr(positions), _ptr(freq_k), c_int(rot if freq_k is not None else 0), _ptr(freq_v),
        _ptr(q), c_long(q.stride(0)), c_int(_CODES[dtype]), _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(heads),
        c_int(kv_heads), c_int(dk), c_int(dv), c_int(page_size), _stream()))
    return q


def pooled_means(k_cache, v_cache, pk_cache, pv_cache, step, group: int, pool_group: int, kv_heads: int, dk: int, dv: int,
                 page_size: int, pool: int) -> None:
    """For every block of ``pool`` positions whose last position the step wrote: the mean of its keys and of its values
    (read from the cache, added in position order, float32) into the block cache, whose pages ([page, kv head, rows,
    channels], rows = ceil(page_size / pool)) hang on the block table of ``pool_group``."""
    tables, ptables = step.block_tables[group], step.block_tables[pool_group]
    _dev(k_cache, v_cache, pk_cache, pv_cache, tables, ptables, step.cu_q, step.kv_lens)
    rows = pk_cache.shape[2]
    assert pk_cache.dtype == k_cache.dtype and tuple(pk_cache.shape[1:]) == (kv_heads, rows, dk)
    assert tuple(pv_cache.shape[1:]) == (kv_heads, rows, dv) and pk_cache.is_contiguous() and pv_cache.is_contiguous()
    lib = pooled()
    _check(lib, lib.coheryn_pooled_means(
        _ptr(k_cache), _ptr(v_cache), _ptr(pk_cache), _ptr(pv_cache), c_int(_code(k_cache)), _ptr(tables), c_int(tables.shape[1]),
        _ptr(ptables), c_int(ptables.shape[1]), _ptr(step.cu_q), _ptr(step.kv_lens), c_int(step.num_requests),
        c_int(max(int(step.max_q_len), 1)), c_int(kv_heads), c_int(dk), c_int(dv), c_int(page_size), c_int(pool), c_int(rows),
        _stream()))


def pooled_attention(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, pk_cache, pv_cache, step, group: int,
                     pool_group: Optional[int], heads: int, kv_heads: int, dk: int, dv: int, page_size: int,
                     window: Optional[int], pool: Optional[int], scale: float, softcap: Optional[float],
                     temps: Optional[torch.Tensor], sinks: Optional[torch.Tensor], gates: Optional[torch.Tensor],
                     freq_v: Optional[torch.Tensor]) -> None:
    """Attention of every row of the step over the last ``window`` positions of its request and the means of the blocks
    of ``pool`` positions that lie wholly before them (see csrc/attention_pooled.cu).  q [T, heads * dk], out
    [T, heads * dv] in the caches' dtype; ``temps``, ``sinks`` float32 [heads]; ``gates`` float32 [T, heads * dv] (rows may
    be strided): the output passes sigmoid(gates); ``freq_v``: the values were rotated, the output is turned back."""
    tables = step.block_tables[group]
    ptables = step.block_tables[pool_group] if pool else None
    _dev(q, out, k_cache, v_cache, pk_cache, pv_cache, tables, ptables, step.token_req, step.positions, temps, sinks, gates, freq_v)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == heads * dk and out.shape == (T, heads * dv)
    assert k_cache.dtype == q.dtype and v_cache.dtype == q.dtype and out.dtype == q.dtype
    for v in (temps, sinks):
        if v is not None:
            assert v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads
    if gates is not None:
        _f32(gates, "gates")
        assert gates.shape == (T, heads * dv)
    if pool and not window:
        raise KernelError("pooled_attention: block means stand for positions before a window; without a window there are none")
    q_lens = getattr(step, "q_lens", None)
    if (POOLED_TC and q.dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and dk <= 256 and dv <= 128 and q_lens
            and max(q_lens) >= POOLED_TC_MIN_ROWS and getattr(step, "cu_q", None) is not None and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and k_cache.is_contiguous() and v_cache.is_contiguous()):
        # rows that are whole runs of consecutive positions per request, ending at the request's last position
        _dev(step.cu_q, step.kv_lens)
        lib = pooled_tc_lib(dk, dv)
        _check(lib, lib.coheryn_pooled_attention_tc(
            _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pk_cache),
            _ptr(pv_cache), _ptr(tables), c_int(tables.shape[1]), _ptr(ptables), c_int(ptables.shape[1] if ptables is not None else 0),
            _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(temps), _ptr(sinks), _ptr(gates),
            c_long(gates.stride(0) if gates is not None else 0), _ptr(freq_v), c_int(len(q_lens)), c_int(max(q_lens)), c_int(heads),
            c_int(kv_heads), c_int(page_size), c_int(window or 0), c_int(pool or 0), c_int(pk_cache.shape[2] if pool else 0),
            c_float(scale), c_float(softcap or 0.0), _stream()))
        return
    lib = pooled()
    # few rows (decoding): the keys of a row are shared out over several CTAs, whose parts meet in a scratch area
    floats = T * heads * (dv + 2) * 8 if T * kv_heads < 148 else 0
    scratch = torch.empty(floats, dtype=torch.float32, device=q.device) if floats else None
    _check(lib, lib.coheryn_pooled_attention(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pk_cache),
        _ptr(pv_cache), c_int(_code(q)), _ptr(tables), c_int(tables.shape[1]), _ptr(ptables),
        c_int(ptables.shape[1] if ptables is not None else 0), _ptr(step.token_req), _ptr(step.positions), _ptr(temps), _ptr(sinks),
        _ptr(gates), c_long(gates.stride(0) if gates is not None else 0), _ptr(freq_v), c_int(T), c_int(heads), c_int(kv_heads),
        c_int(dk), c_int(dv), c_int(page_size), c_int(window or 0), c_int(pool or 0),
        c_int(pk_cache.shape[2] if pool else 0), c_float(scale), c_float(softcap or 0.0), _ptr(scratch), c_long(floats), _stream()))
