"""Python side of the CUDA kernels: argument checks, pointers, the current stream.

Every function takes CUDA tensors and launches on ``torch.cuda.current_stream()``.
There is no CPU path: a tensor that is not on a CUDA device raises, and so does a
missing or failing extension (``csrc/build.py``).  A kernel that cannot run a size
correctly refuses it (``UNSUPPORTED_SIZE``) instead of giving a wrong result.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_module
from ..errors import ErrorCode, PhotonError

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_launch_count = 0


def launch_count() -> int:
    """Kernels of this package launched so far in this process."""
    return _launch_count


_sm_counts = {}


def sm_count(device) -> int:
    """Streaming multiprocessors of ``device`` (asked once)."""
    key = (device.type, device.index)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[key]


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT,
                              "a tensor on the CPU was passed to a CUDA kernel; there is no CPU path")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(t.data_ptr() if t is not None else 0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global _launch_count
    if status == 0:
        _launch_count += 1
        return
    if status == -2:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, f"{what}: this size is not supported by the kernel")
    if status == -3:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{what}: invalid argument")
    raise PhotonError(ErrorCode.CUDA_ERROR, f"{what}: CUDA error {status}")


_sigs_done = set()


def _fn(module: str, name: str, argtypes, defines=None):
    lib = load_module(module, defines)
    f = getattr(lib, name)
    key = (id(lib), name)
    if key not in _sigs_done:
        f.argtypes = argtypes
        f.restype = c_int
        _sigs_done.add(key)
    return f


def _int32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"{what} must be a contiguous int32 tensor")


# ----------------------------------------------------------------------------- row kernels

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor]) -> None:
    """``out[t, :] = table[ids[t], :]`` as float32; ids outside the table set the error word."""
    _cuda(ids, table, out, err)
    _int32(ids, "ids")
    T, (V, H) = ids.numel(), table.shape
    if out.dtype != torch.float32 or out.shape != (T, H) or not out.is_contiguous() or not table.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "embedding: out must be contiguous float32 [T, H]")
    f = _fn("elementwise", "photon_embedding",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _dtype_code(table), _ptr(out), T, H, V, _ptr(err), _stream()), "embedding")


def add_rmsnorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, delta2: Optional[torch.Tensor] = None,
                delta_scale: Optional[torch.Tensor] = None) -> None:
    """``residual += delta`` in float32 (in place; skipped when ``rows`` is given), then
    ``out = weight * (residual / sqrt(mean(residual^2) + eps))``.  With ``rows`` (int32 list)
    only those rows are read and ``out`` has one row per list entry.  ``delta2`` (the second output of a
    parallel block, same shape and type as ``delta``): ``residual += delta + delta2``.  ``delta_scale`` (float32
    ``[H]``): ``delta`` is multiplied by it channel by channel first (a layer scale)."""
    _cuda(delta, residual, weight, out, rows, delta2, delta_scale)
    _check_delta_scale(delta_scale, delta, delta2, residual.shape[-1])
    if delta2 is not None:
        if delta is None:
            delta, delta2 = delta2, None
        elif delta2.shape != delta.shape or delta2.dtype != delta.dtype or not delta2.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_rmsnorm: delta2 must match delta")
    H = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "add_rmsnorm: the residual stream must be contiguous float32")
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_rmsnorm: delta must match the residual stream")
    if out.shape != (n, H) or not out.is_contiguous() or weight.numel() != H:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_rmsnorm: out must be [rows, H] and weight [H]")
    if rows is not None:
        _int32(rows, "rows")
    f = _fn("elementwise", "photon_add_rmsnorm_scaled",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
             c_void_p])
    _check(f(_ptr(delta), _dtype_code(delta) if delta is not None else F32, _ptr(delta2), _ptr(residual), _ptr(weight),
             _dtype_code(weight), _ptr(out), _dtype_code(out), _ptr(rows), n, H, float(eps), _ptr(delta_scale), _stream()),
           "add_rmsnorm")


def _check_delta_scale(scale: Optional[torch.Tensor], delta, delta2, H: int) -> None:
    if scale is None:
        return
    if delta is None or delta2 is not None:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "a channel scale goes with exactly one pending output")
    if scale.dtype != torch.float32 or scale.numel() != H or not scale.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "the channel scale must be contiguous float32 [H]")


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu": 2, "relu": 3}     # gelu: the exact (erf) form
ACT_NONE = -1


def add_layernorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                  eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                  delta2: Optional[torch.Tensor] = None, delta_scale: Optional[torch.Tensor] = None) -> None:
    """As ``add_rmsnorm`` with a layer norm: ``out = (x - mean(x)) / sqrt(var(x) + eps) * weight + bias`` with
    ``x = residual + delta (+ delta2)``, all in 32-bit; the variance is the mean of the squared deviations."""
    _cuda(delta, residual, weight, bias, out, rows, delta2, delta_scale)
    _check_delta_scale(delta_scale, delta, delta2, residual.shape[-1])
    if delta2 is not None:
        if delta is None:
            delta, delta2 = delta2, None
        elif delta2.shape != delta.shape or delta2.dtype != delta.dtype or not delta2.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_layernorm: delta2 must match delta")
    H = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "add_layernorm: the residual stream must be contiguous float32")
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_layernorm: delta must match the residual stream")
    if out.shape != (n, H) or not out.is_contiguous() or weight.numel() != H or (bias is not None and bias.numel() != H):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "add_layernorm: out must be [rows, H], weight and bias [H]")
    if rows is not None:
        _int32(rows, "rows")
    f = _fn("elementwise", "photon_add_layernorm_scaled",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
             c_float, c_void_p, c_void_p])
    _check(f(_ptr(delta), _dtype_code(delta) if delta is not None else F32, _ptr(delta2), _ptr(residual), _ptr(weight),
             _dtype_code(weight), _ptr(bias), _dtype_code(bias) if bias is not None else F32, _ptr(out), _dtype_code(out),
             _ptr(rows), n, H, float(eps), _ptr(delta_scale), _stream()), "add_layernorm")


def activation(x: torch.Tensor, activation: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(x)`` element by element (in place unless ``out`` is given), 32-bit arithmetic."""
    _cuda(x, out)
    if activation not in ACTIVATIONS:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"unknown activation {activation!r} ({', '.join(ACTIVATIONS)})")
    out = x if out is None else out
    if not x.is_contiguous() or not out.is_contiguous() or out.shape != x.shape or out.dtype != x.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "activation: x and out contiguous, of one shape and dtype")
    f = _fn("elementwise", "photon_activation", [c_void_p, c_void_p, c_int, c_long, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(out), _dtype_code(x), x.numel(), ACTIVATIONS[activation], _stream()), "activation")
    return out


def gate_mul(x: torch.Tensor, gate: torch.Tensor) -> None:
    """``x [T, W] *= sigmoid(gate [T, W])`` in place; both may be views with a row stride, ``gate`` may be 32-bit
    beside a bfloat16 ``x``."""
    _cuda(x, gate)
    if x.dim() != 2 or gate.shape != x.shape or x.stride(1) != 1 or gate.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gate_mul: x and gate [T, W] with contiguous rows")
    f = _fn("elementwise", "photon_gate_mul", [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _dtype_code(x), _ptr(gate), gate.stride(0), _dtype_code(gate), x.shape[0], x.shape[1],
             _stream()), "gate_mul")


def stream_add(residual: torch.Tensor, delta: Optional[torch.Tensor], delta2: Optional[torch.Tensor],
               other: Optional[torch.Tensor], bias: Optional[torch.Tensor]) -> None:
    """``residual += (delta + delta2) + other + bias`` in 32-bit, in place: what is pending on the stream, a second
    32-bit stream of the same shape and one vector ``[H]`` for all rows; each may be None."""
    _cuda(residual, delta, delta2, other, bias)
    T, H = residual.shape
    if delta is None and delta2 is not None:
        delta, delta2 = delta2, None
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "stream_add: the residual stream must be contiguous float32")
    for t in (delta, delta2):
        if t is not None and (t.shape != residual.shape or not t.is_contiguous() or t.dtype != delta.dtype):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_add: pending outputs must match the residual stream")
    if other is not None and (other.shape != residual.shape or other.dtype != torch.float32 or not other.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_add: the second stream must be contiguous float32 [T, H]")
    if bias is not None and (bias.numel() != H or not bias.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_add: bias must be [H]")
    f = _fn("elementwise", "photon_stream_add",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _ptr(delta2), _dtype_code(delta) if delta is not None else F32, _ptr(other),
             _ptr(bias), _dtype_code(bias) if bias is not None else F32, T, H, _stream()), "stream_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """``out = act(gate_up[:, :I]) * gate_up[:, I:]`` with ``act`` silu or the tanh form of gelu."""
    _cuda(gate_up, out)
    if activation not in ACTIVATIONS:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"unknown activation {activation!r} (silu or gelu_tanh)")
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2) or out.dtype != gate_up.dtype \
            or not gate_up.is_contiguous() or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "swiglu: gate_up [T, 2I] and out [T, I] of one dtype")
    f = _fn("elementwise", "photon_glu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _dtype_code(out), T, I2 // 2, ACTIVATIONS[activation], _stream()), "glu")


def stream_concat(residual: torch.Tensor, delta: Optional[torch.Tensor], delta2: Optional[torch.Tensor],
                  other: torch.Tensor, out: torch.Tensor) -> None:
    """``out [T, 2H] = [residual + delta + delta2 ; other]``: the running stream (its pending sums applied in
    32-bit) beside a second stream of the same width, rounded once to ``out``'s type."""
    _cuda(residual, delta, delta2, other, out)
    T, H = residual.shape
    if delta is None and delta2 is not None:
        delta, delta2 = delta2, None
    for t in (residual, other):
        if t.dtype != torch.float32 or t.shape != (T, H) or not t.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_concat: both streams must be contiguous float32 [T, H]")
    for d in (delta, delta2):
        if d is not None and (d.shape != (T, H) or not d.is_contiguous() or d.dtype != (delta.dtype)):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_concat: the pending sums must be contiguous [T, H] of one type")
    if out.shape != (T, 2 * H) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "stream_concat: out must be contiguous [T, 2H]")
    f = _fn("elementwise", "photon_stream_concat",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _ptr(delta2), _dtype_code(delta) if delta is not None else _dtype_code(out),
             _ptr(other), _ptr(out), _dtype_code(out), T, H, _stream()), "stream_concat")


def scale_bias_rows(x: torch.Tensor, scale: float = 1.0, bias: Optional[torch.Tensor] = None) -> None:
    """``x [T, H]`` (float32, in place) ``= x * scale + bias``; ``bias [H]`` float32 or bfloat16, may be None."""
    _cuda(x, bias)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "scale_bias_rows: x must be contiguous float32 [T, H]")
    T, H = x.shape
    if bias is not None and (bias.numel() != H or not bias.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "scale_bias_rows: bias must be contiguous [H]")
    f = _fn("elementwise", "photon_scale_bias_rows", [c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), float(scale), _ptr(bias), _dtype_code(bias) if bias is not None else F32, T, H, _stream()),
           "scale_bias_rows")


# ----------------------------------------------------------------------------- rope and cache write

def rope_kv_write(q: Optional[torch.Tensor], k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                  positions: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], interleaved: bool,
                  slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                  err: Optional[torch.Tensor]) -> None:
    """Rotates ``q [T, n_q * d]`` and ``k [T, n_kv * d]`` in place (when ``inv_freq`` is given)
    and stores ``k`` and ``v [T, n_kv * d]`` at ``slot_mapping`` in the paged cache
    ``[pages, n_kv, page_size, d]`` (when the caches are given).  The three inputs may be
    views with any row stride, e.g. sections of one fused row."""
    _cuda(q, k, v, positions, inv_freq, slot_mapping, k_cache, v_cache, err)
    ref = q if q is not None else k
    if ref is None:
        return
    T = ref.shape[0]
    for name, t, heads in (("q", q, n_q), ("k", k, n_kv), ("v", v, n_kv)):
        if t is None:
            continue
        if t.dim() == 3:
            ok = t.shape == (T, heads, head_dim) and t.stride(2) == 1 and t.stride(1) == head_dim
        else:
            ok = t.shape == (T, heads * head_dim) and t.stride(1) == 1
        if not ok or t.dtype != ref.dtype:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              f"rope_kv_write: {name} must be [T, {heads} * {head_dim}] with contiguous heads")
    rotate = inv_freq is not None
    write = k_cache is not None
    page_size, num_slots = 1, 0
    if rotate:
        _int32(positions, "positions")
        if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2 or head_dim % 2:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "rope_kv_write: inv_freq must be float32 [head_dim / 2]")
    if write:
        if k is None or v is None:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "rope_kv_write: storing needs k and v")
        _int32(slot_mapping, "slot_mapping")
        if k_cache.dtype != ref.dtype or v_cache.dtype != ref.dtype or k_cache.shape != v_cache.shape \
                or k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != head_dim \
                or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              "rope_kv_write: caches must be contiguous [pages, n_kv, page_size, head_dim] of the run dtype")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    f = _fn("rope_kv", "photon_rope_kv_write",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_long, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0) if q is not None else 0, _ptr(k), k.stride(0) if k is not None else 0,
             _ptr(v), v.stride(0) if v is not None else 0, _dtype_code(ref), _ptr(positions), _ptr(inv_freq),
             int(interleaved), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), T, n_q, n_kv, head_dim,
             page_size, num_slots, int(rotate), int(write), _ptr(err), _stream()), "rope_kv_write")


def qk_norm_rope_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_out: torch.Tensor,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dims: int,
                       slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, value_dim: int,
                       err: Optional[torch.Tensor]) -> None:
    """Per head ``y = x / sqrt(mean(x^2) + eps) [* weight]`` for ``q [T, n_q * d]`` and ``k [T, n_kv * d]``, then the
    rotation of the first ``rot_dims`` numbers of every head (number ``j`` with ``j + rot_dims / 2``, angle
    ``position * inv_freq[j]``, ``inv_freq`` float64), queries into ``q_out`` and keys and ``v [T, n_kv * dv]`` into the
    paged caches ``[pages, n_kv, page_size, d | dv]``.  The inputs are views with any row stride and may be 32-bit
    while ``q_out`` and the caches are bfloat16.  Caches None: only the queries (``k`` and ``v`` are not read)."""
    _cuda(q, k, v, q_out, q_weight, k_weight, positions, inv_freq, slot_mapping, k_cache, v_cache, err)
    T = q.shape[0]
    d, dv = head_dim, value_dim
    if q.shape != (T, n_q * d) or q.stride(1) != 1 or q_out.shape != (T, n_q * d) or q_out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "qk_norm_rope_write: q and q_out must be [T, n_q * head_dim]")
    write = k_cache is not None
    page_size, num_slots = 1, 0
    if write:
        if k is None or v is None or k.shape != (T, n_kv * d) or v.shape != (T, n_kv * dv) or k.stride(1) != 1 \
                or v.stride(1) != 1 or k.dtype != q.dtype or v.dtype != q.dtype:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "qk_norm_rope_write: k [T, n_kv * head_dim], v [T, n_kv * value_dim]")
        _int32(slot_mapping, "slot_mapping")
        if k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or v_cache.shape[:3] != k_cache.shape[:3] \
                or v_cache.shape[3] != dv or k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype \
                or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              "qk_norm_rope_write: caches must be contiguous [pages, n_kv, page_size, head_dim | value_dim]")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    _int32(positions, "positions")
    if inv_freq is not None and (inv_freq.dtype != torch.float64 or inv_freq.numel() != rot_dims // 2 or rot_dims % 2
                                 or rot_dims > d):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "qk_norm_rope_write: inv_freq must be float64 [rot_dims / 2], rot_dims even, <= head_dim")
    wt = q_weight if q_weight is not None else k_weight
    for w in (q_weight, k_weight):
        if w is not None and (w.numel() != d or w.dtype != wt.dtype or not w.is_contiguous()):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "qk_norm_rope_write: norm weights must be [head_dim] of one dtype")
    f = _fn("qk_norm", "photon_qk_norm_rope_write",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int,
             c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_long, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k) if write else None, k.stride(0) if write else 0, _ptr(v) if write else None,
             v.stride(0) if write else 0, _dtype_code(q), _ptr(q_out), q_out.stride(0), _dtype_code(q_out), _ptr(q_weight),
             _ptr(k_weight), _dtype_code(wt) if wt is not None else F32, float(eps), _ptr(positions),
             _ptr(inv_freq) if rot_dims else None, int(rot_dims) if inv_freq is not None else 0, _ptr(slot_mapping),
             _ptr(k_cache), _ptr(v_cache), T, n_q, n_kv, d, dv, page_size, num_slots, _ptr(err), _stream()),
           "qk_norm_rope_write")


# ----------------------------------------------------------------------------- attention

def _check_gate(gate: Optional[torch.Tensor], q: torch.Tensor, out: torch.Tensor) -> None:
    if gate is None:
        return
    _cuda(gate)
    if gate.shape != out.shape or gate.stride(1) != 1 or gate.dtype != q.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention: the gate must have the shape of the output and the type of q")


def gate_fusable(gate: torch.Tensor) -> bool:
    """Whether the tensor-core attention kernels can take this gate into their epilogue (16-byte aligned rows)."""
    return gate.stride(1) == 1 and gate.data_ptr() % 16 == 0 and (gate.stride(0) * gate.element_size()) % 16 == 0


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor,
                    n_q: int, n_kv: int, head_dim: int, window: Optional[int], scale: float,
                    err: Optional[torch.Tensor], value_dim: Optional[int] = None, splits: int = 1,
                    keep_first: int = 0, sink: bool = False, softcap: Optional[float] = None,
                    gate: Optional[torch.Tensor] = None) -> None:
    """General paged causal attention.  ``q`` is a ``[T, n_q * d]`` view (row stride free),
    ``out [T, n_q * dv]``; the token at position ``p`` of request ``token_seq[t]`` sees keys
    ``max(0, p - window + 1) .. p`` through ``block_table[seq]``.  ``value_dim`` (default ``head_dim``) is the
    width of a value; ``v_cache is k_cache`` means that a key's value is the first ``value_dim`` numbers of
    its own row (attention over a cached latent).  ``splits`` > 1 shares every token's keys out over that many
    blocks (for decoded tokens with long contexts; the order of the sums then depends on ``splits``).
    ``keep_first``: with a window, keys ``0 .. keep_first - 1`` stay visible as well.  ``sink``: the softmax has one
    more key with score 0 and no value (``p_j = exp(s_j) / (1 + sum exp(s_i))``).  ``softcap``: scores become
    ``softcap * tanh(score / softcap)`` after the scale.  ``gate`` (``[T, n_q * value_dim]`` of the type of ``q``, a
    view with any row stride): every output is multiplied by ``sigmoid(gate)`` before it is rounded."""
    _check_gate(gate, q, out)
    _cuda(q, out, k_cache, v_cache, block_table, token_seq, positions, err)
    T = q.shape[0]
    dv = head_dim if value_dim is None else int(value_dim)
    shared = v_cache is k_cache or v_cache.data_ptr() == k_cache.data_ptr()
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * dv) or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "paged_attention: q must be [T, n_q * head_dim], out [T, n_q * value_dim]")
    if q.dtype != out.dtype or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "paged_attention: q, out and the caches must share one dtype")
    if n_kv <= 0 or n_q % n_kv or dv <= 0 or (shared and dv > head_dim):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "paged_attention: n_q must be a multiple of n_kv, and a value that "
                          "lies in its key's row cannot be wider than the row")
    if k_cache.shape[3] != head_dim or (not shared and v_cache.shape[3] != dv):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "paged_attention: the caches' last dimension must be head_dim / value_dim")
    for name, t in (("block_table", block_table), ("token_seq", token_seq), ("positions", positions)):
        _int32(t, name)
    f = _fn("attention", "photon_paged_attention_ex",
            [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int,
             c_float, c_void_p, c_long, c_void_p])
    splits = max(1, min(int(splits), 64))
    part = torch.empty(T * n_q * splits * (dv + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _dtype_code(q), _ptr(k_cache), _ptr(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(positions), T, n_q, n_kv, head_dim, dv,
             k_cache.shape[2], k_cache.shape[0], int(window) if window else 0, float(scale), splits, _ptr(part), _ptr(err),
             int(keep_first or 0), int(bool(sink)), float(softcap or 0.0), _ptr(gate), gate.stride(0) if gate is not None else 0,
             _stream()), "paged_attention")
    if splits > 1:
        global _launch_count
        _launch_count += 1


_ticket_buffers = {}


def _attention_tickets(device) -> torch.Tensor:
    """Zeroed tickets, one per (token, key/value head); the kernel puts them back to zero."""
    key = (device.type, device.index)
    if key not in _ticket_buffers:
        _ticket_buffers[key] = torch.zeros(1 << 16, dtype=torch.int32, device=device)
    return _ticket_buffers[key]


def reset_tickets(device) -> None:
    """Puts the ticket counters of the split-key attention and of the split-K products back to zero.  The
    kernels do that themselves after every launch; a launch that gave up (the error word says so) may not."""
    key = (device.type, device.index)
    if key in _ticket_buffers:
        _ticket_buffers[key].zero_()
    if key in _skinny_buffers:
        _skinny_buffers[key][1].zero_()


def flash_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """The tensor-core kernel takes bfloat16 and head sizes that are a multiple of 16 up to 128."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def flash_attention_max_groups(head_dim: int) -> int:
    """Groups of four warps that the split-key kernel can run in one block at this head size (4, 2 or 1)."""
    lib = load_module("attention_flash", {"HEAD_DIM": head_dim})
    return int(lib.photon_flash_attention_max_groups())


def flash_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, cu_tokens: torch.Tensor, positions: torch.Tensor,
                    num_seqs: int, max_tokens_per_seq: int, n_q: int, n_kv: int, head_dim: int,
                    window: Optional[int], scale: float, num_splits: int, scratch: Optional[torch.Tensor],
                    rows_mode: bool, keys_mode: bool, err: Optional[torch.Tensor],
                    context_lens: Optional[torch.Tensor] = None, key_groups: int = 1, keep_first: int = 0,
                    sink: bool = False, softcap: Optional[float] = None, gate: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention on the tensor cores.  ``cu_tokens [S + 1]`` gives each request's
    tokens in the step.  ``rows_mode``: run requests with more than 16 rows (tokens x heads per
    group); ``keys_mode``: run the others, their keys split over ``num_splits`` blocks.
    ``scratch``: float32, at least ``T * n_q * num_splits * (head_dim + 2)`` when ``num_splits > 1``.
    ``context_lens [S]`` (optional): tokens of each request after this step; the split-key kernel then
    derives positions from it (a request's tokens of the step are its last ones) and saves a round trip.
    ``key_groups``: 1, 2 or 4 groups of four warps per block of the split-key kernel, each walking its own
    share of the block's keys (``flash_attention_max_groups`` bounds it); their results are merged in shared
    memory, which is far cheaper than the merge of ``num_splits`` blocks through global memory.
    ``keep_first``, ``sink``, ``softcap``, ``gate``: as in ``paged_attention``."""
    _check_gate(gate, q, out)
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, scratch, err, context_lens)
    if context_lens is not None:
        _int32(context_lens, "context_lens")
        if context_lens.numel() < num_seqs:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: context_lens must cover every request")
    T = q.shape[0]
    if not flash_attention_supported(q.dtype, head_dim) or n_kv <= 0 or n_q % n_kv:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, f"flash_attention: head_dim {head_dim} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "flash_attention: q, out and the caches must be bfloat16")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("positions", positions)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "flash_attention: cu_tokens and block_table must cover every request")
    part_acc = part_ml = tickets = None
    splits = int(num_splits) if keys_mode else 1
    if splits > 1:
        need = T * n_q * splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"flash_attention: scratch must hold {need} float32 values")
        part_acc = scratch
        part_ml = scratch[T * n_q * splits * head_dim:]
        tickets = _attention_tickets(q.device)
        if tickets.numel() < num_seqs * n_kv:
            raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "flash_attention: too many requests for the ticket buffer")
    mode = (1 if rows_mode else 0) | (2 if keys_mode else 0)
    f = _fn("attention_flash", "photon_flash_attention_ex",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
             c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_long, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(positions), _ptr(context_lens), _ptr(part_acc), _ptr(part_ml),
             _ptr(tickets),
             int(num_seqs), int(max_tokens_per_seq), n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0],
             int(window) if window else 0, float(scale), splits, int(key_groups) if keys_mode else 1, mode, _ptr(err),
             int(keep_first or 0), int(bool(sink)), float(softcap or 0.0), _ptr(gate), gate.stride(0) if gate is not None else 0,
             _stream()), "flash_attention")
    if rows_mode and keys_mode:
        global _launch_count
        _launch_count += 1


def attention_decode_supported(dtype: torch.dtype, head_dim: int, group: int, page_size: int, num_seqs: int) -> bool:
    """The persistent TMA kernel for decoded tokens: bfloat16, head size 64 or 128, up to 16 heads per
    key/value head, pages of 8, 16, 32 or a multiple of 64 tokens, up to 512 requests in the step."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 16 and num_seqs <= 512
            and page_size % 8 == 0 and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0))


def attention_decode_slots(head_dim: int) -> int:
    """Blocks of the persistent decode-attention kernel that the current device holds at once."""
    lib = load_module("attention_decode", {"HEAD_DIM": head_dim})
    return int(lib.photon_attention_decode_slots())


def attention_decode_plan(num_seqs: int, n_kv: int, max_keys: int, head_dim: int, page_size: int):
    """(tiles of 64 keys per work item, chunks to reserve scratch for, upper bound of the work items) for a step of
    ``num_seqs`` requests of at most ``max_keys`` visible keys; None when a request has more keys than the kernel
    takes (min(120, head size) chunks of 64 tiles of 64 keys: about 490,000 at heads of 128, 260,000 at heads of 64).

    A request's keys are cut into ``p`` chunks; a (chunk, key/value head) is a work item that one of the resident
    blocks draws.  ``p`` minimises ``rounds * (tiles per item + 5) + 0.3 * p`` with ``rounds = ceil(items / blocks)``:
    an item costs about five tile times beside its tiles (Q, the first round trip, the merge of its four warps), a
    chunk a partial result written and merged, and what decides most is how many items the busiest block gets.
    Measured on B200: 64 requests of 640 keys run best whole (26 us against 45 us in chunks of four tiles); 8
    requests x 8 heads of 16,500 keys: five chunks each are 320 items for 296 blocks, two rounds of 52 tiles (95
    us), chunks of four tiles 154 us."""
    slots = attention_decode_slots(head_dim)
    tiles = -(-max(max_keys, 1) // 64) + 1              # a window may start inside a tile
    most = 64                                           # tiles an item may have
    pairs = max(1, num_seqs * n_kv)
    best = None
    for p in range(-(-tiles // most), min(120, head_dim, tiles) + 1):     # the kernel merges up to min(120, head_dim) chunks
        chunk = -(-tiles // p)
        if -(-tiles // chunk) != p:
            continue                                    # the same chunk length as a smaller p
        rounds = -(-(pairs * p) // slots)
        cost = rounds * (chunk + 5) + (0.3 * p if p > 1 else 0.0)
        if best is None or cost < best[0]:
            best = (cost, chunk, p)
    if best is None:
        return None                                     # more keys than 120 chunks of 64 tiles hold
    _, chunk, per_seq = best
    return chunk, num_seqs * per_seq, num_seqs * per_seq * n_kv


_decode_scratch = {}


def attention_decode_scratch(device, floats: int) -> torch.Tensor:
    """The partial results of ``attention_decode``: one float32 buffer per device of at least ``floats`` elements.
    It grows by doubling and the buffers it outgrew are kept, because a captured CUDA graph holds the address it
    was captured with; a tensor that died with the step would leave the graph writing into memory that has a
    new owner."""
    key = (device.type, device.index)
    buffers = _decode_scratch.setdefault(key, [])
    if not buffers or buffers[-1].numel() < floats:
        size = max(int(floats), 2 * buffers[-1].numel() if buffers else 0, 1 << 20)
        buffers.append(torch.empty(size, dtype=torch.float32, device=device))
    return buffers[-1]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, cu_tokens: torch.Tensor, context_lens: torch.Tensor, num_seqs: int,
                     n_q: int, n_kv: int, head_dim: int, window: Optional[int], scale: float, chunk_tiles: int,
                     scratch: torch.Tensor, scratch_chunks: int, max_items: int, err: Optional[torch.Tensor]) -> None:
    """Attention of the requests that bring at most 16 rows (tokens x heads per group) in this step, by the
    persistent TMA kernel (``attention_decode.cu``); the rows of the other requests are left untouched.
    ``context_lens [S]``: tokens of each request after this step (a request's tokens of the step are its last).
    ``scratch``: float32, at least ``scratch_chunks * n_kv * 16 * (head_dim + 2)``; ``scratch_chunks`` at least the
    chunks of ``chunk_tiles`` tiles that all requests have together (``attention_decode_plan``)."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, context_lens, scratch, err)
    T = q.shape[0]
    if n_kv <= 0 or n_q % n_kv or not attention_decode_supported(q.dtype, head_dim, n_q // n_kv, k_cache.shape[2], num_seqs):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE,
                          f"attention_decode: head_dim {head_dim}, {n_q}/{n_kv} heads, pages of {k_cache.shape[2]} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_decode: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_decode: q, out and the caches must be bfloat16")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_decode: the caches must be contiguous [pages, n_kv, page, d]")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("context_lens", context_lens)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs or context_lens.numel() < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_decode: cu_tokens, context_lens and block_table must cover every request")
    need = scratch_chunks * n_kv * 16 * (head_dim + 2)
    if scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"attention_decode: scratch must hold {need} float32 values")
    tickets = _attention_tickets(q.device)
    if tickets.numel() < num_seqs * n_kv + 2:      # the tickets, then the kernel's two work counters
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "attention_decode: too many requests for the ticket buffer")
    part_ml = scratch[scratch_chunks * n_kv * 16 * head_dim:]
    f = _fn("attention_decode", "photon_attention_decode",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
             c_long, c_void_p, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(context_lens), _ptr(scratch), _ptr(part_ml), int(scratch_chunks),
             _ptr(tickets), int(num_seqs), T, n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0],
             int(window) if window else 0, float(scale), int(chunk_tiles), max(1, -(-int(scratch_chunks) // max(num_seqs, 1))),
             int(max_items), _ptr(err), _stream()),
           "attention_decode")


# PHOTON_ATTENTION_TC=0 keeps prompt portions on the mma.sync kernel (for comparisons)
USE_ATTENTION_TC = os.environ.get("PHOTON_ATTENTION_TC", "1") != "0"


def attention_tc_supported(dtype: torch.dtype, head_dim: int, group: int, page_size: int) -> bool:
    """The tcgen05 kernel for prompt portions: bfloat16, head size 64 or 128, up to 128 heads per
    key/value head and pages of 8, 16, 32 or a multiple of 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 128
            and page_size % 8 == 0 and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0))


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_tokens: torch.Tensor, positions: torch.Tensor,
                 num_seqs: int, max_tokens_per_seq: int, n_q: int, n_kv: int, head_dim: int,
                 window: Optional[int], scale: float, err: Optional[torch.Tensor], keep_first: int = 0,
                 sink: bool = False, softcap: Optional[float] = None, gate: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention of the requests that bring more than 16 rows (tokens x heads per
    group) in this step, on the tcgen05 tensor cores; the rows of the other requests are left
    untouched (``flash_attention`` with ``keys_mode`` takes them).  ``keep_first``, ``sink``, ``softcap``, ``gate``: as in
    ``paged_attention`` (the gate's rows must start on 16-byte boundaries: ``gate_fusable``)."""
    _check_gate(gate, q, out)
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, err)
    T = q.shape[0]
    if n_kv <= 0 or n_q % n_kv or not attention_tc_supported(q.dtype, head_dim, n_q // n_kv, k_cache.shape[2]):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE,
                          f"attention_tc: head_dim {head_dim}, {n_q}/{n_kv} heads, pages of {k_cache.shape[2]} in {q.dtype} is not supported")
    if q.shape[1] != n_q * head_dim or q.stride(1) != 1 or out.shape != (T, n_q * head_dim) or not out.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_tc: q and out must be [T, n_q * head_dim]")
    if out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_tc: q, out and the caches must be bfloat16")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "attention_tc: the caches must be contiguous [pages, n_kv, page, d]")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("positions", positions)):
        _int32(t, name)
    if cu_tokens.numel() < num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "attention_tc: cu_tokens and block_table must cover every request")
    f = _fn("attention_tc", "photon_attention_tc_ex",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_float,
             c_void_p, c_long, c_void_p],
            defines={"HEAD_DIM": head_dim})
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(positions), int(num_seqs), int(max_tokens_per_seq), T,
             n_q, n_kv, head_dim, k_cache.shape[2], k_cache.shape[0], int(window) if window else 0, float(scale),
             _ptr(err), int(keep_first or 0), int(bool(sink)), float(softcap or 0.0), _ptr(gate),
             gate.stride(0) if gate is not None else 0, _stream()), "attention_tc")


# ----------------------------------------------------------------------------- matrix products

SKINNY_MAX_ROWS = 8         # up to this many rows the weight-streaming kernel runs instead of the library


def skinny_gemm_supported(x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False) -> bool:
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 1 <= M <= (32 if swiglu else 64)
            and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


_skinny_buffers = {}


def _skinny_scratch(device):
    """One scratch buffer and one ticket array per device for the split of K over blocks; launches
    on one stream use them one after the other."""
    key = (device.type, device.index)
    if key not in _skinny_buffers:
        _skinny_buffers[key] = (torch.empty(1 << 20, dtype=torch.float32, device=device),
                                torch.zeros(8192, dtype=torch.int32, device=device))
    return _skinny_buffers[key]


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16") -> None:
    """``out = x @ weight^T`` for few rows, the weights streamed once.  ``epilogue``: ``"bf16"``,
    ``"f32"`` (float output), ``"swiglu"`` (``weight`` holds gate rows then up rows; ``out`` is
    ``[M, I]`` with ``silu(gate) * up``) or ``"gelu"`` (the exact gelu of every output, bfloat16)."""
    _cuda(x, weight, out)
    M, K = x.shape
    N = weight.shape[0]
    code = {"bf16": 0, "f32": 1, "swiglu": 2, "gelu": 4}[epilogue]
    cols = N // 2 if epilogue == "swiglu" else N
    want = torch.float32 if epilogue == "f32" else torch.bfloat16
    if not skinny_gemm_supported(x, weight, epilogue == "swiglu") or weight.shape[1] != K:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "skinny_gemm: needs bfloat16, K a multiple of 8, aligned rows, few rows of x")
    if out.shape != (M, cols) or out.dtype != want or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"skinny_gemm: out must be {want} [{M}, {cols}]")
    scratch, tickets = _skinny_scratch(x.device)
    f = _fn("gemm_skinny", "photon_skinny_gemm",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_long,
             c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             _ptr(scratch), scratch.numel(), _ptr(tickets), tickets.numel(), _stream()), "skinny_gemm")


def skinny_fused_supported(residual: torch.Tensor, weight: torch.Tensor) -> bool:
    """The decode-step product with the residual add and the norm folded in: up to 8 rows of a contiguous
    float32 residual stream, bfloat16 weights, K a multiple of 8."""
    M, K = residual.shape
    return (residual.dtype == torch.float32 and residual.is_contiguous() and weight.dtype == torch.bfloat16
            and weight.is_contiguous() and 1 <= M <= 8 and K % 8 == 0 and weight.shape[1] == K
            and weight.data_ptr() % 16 == 0 and residual.data_ptr() % 16 == 0)


def skinny_fused(residual: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                 weight: torch.Tensor, epilogue: str, rope: Optional[dict] = None,
                 err: Optional[torch.Tensor] = None):
    """``x = residual + delta``; ``out = epilogue(rmsnorm(x; norm_weight, eps) @ weight^T)`` in one kernel.
    Returns ``(out, new_residual)``; the input residual is left untouched (the sum goes to a new tensor).
    ``epilogue``: ``"bf16"``, ``"swiglu"`` (``weight`` = gate rows then up rows) or ``"qkv"`` with
    ``rope = dict(positions, inv_freq, slot_mapping, k_cache, v_cache, n_q, n_kv, head_dim)``: q and k are
    rotated (partners must be neighbouring rows of ``weight``), q is returned ``[M, n_q * d]`` wide in
    ``out[:, :n_q * d]``, k and v go into the paged cache."""
    _cuda(residual, delta, norm_weight, weight, err)
    M, K = residual.shape
    N = weight.shape[0]
    if not skinny_fused_supported(residual, weight):
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "skinny_fused: needs <= 8 float32 rows, bfloat16 weights, K % 8 == 0")
    if delta is not None and (delta.shape != residual.shape or delta.dtype != torch.bfloat16 or not delta.is_contiguous()
                              or delta.data_ptr() % 16):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: delta must be contiguous bfloat16 like the residual")
    if norm_weight.numel() != K or norm_weight.data_ptr() % 16:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: norm weight must be [K]")
    code = {"bf16": 0, "swiglu": 2, "qkv": 3}[epilogue]
    new_residual = torch.empty_like(residual) if delta is not None else residual
    r = rope or {}
    if epilogue == "qkv":
        n_q, n_kv, d = r["n_q"], r["n_kv"], r["head_dim"]
        if N != (n_q + 2 * n_kv) * d or d % 2:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: weight must hold q, k and v rows")
        k_cache, v_cache = r["k_cache"], r["v_cache"]
        if k_cache.dtype != torch.bfloat16 or k_cache.shape != v_cache.shape or k_cache.dim() != 4 \
                or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or not k_cache.is_contiguous() \
                or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "skinny_fused: caches must be contiguous bfloat16 [pages, n_kv, page, d]")
        _int32(r["positions"], "positions")
        _int32(r["slot_mapping"], "slot_mapping")
        out = torch.empty((M, n_q * d), dtype=torch.bfloat16, device=residual.device)
        page_size, num_slots = k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2]
    else:
        n_q = n_kv = d = 0
        k_cache = v_cache = None
        page_size, num_slots = 1, 0
        out = torch.empty((M, N // 2 if epilogue == "swiglu" else N), dtype=torch.bfloat16, device=residual.device)
    if err is None:
        err = _error_word(residual.device)
    f = _fn("gemm_skinny_fused", "photon_skinny_fused",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long,
             c_void_p, c_void_p])
    _check(f(_ptr(residual), _ptr(new_residual if delta is not None else None), _ptr(delta), _ptr(norm_weight),
             _dtype_code(norm_weight), float(eps), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
             code, _ptr(r.get("positions")), _ptr(r.get("inv_freq")), _ptr(r.get("slot_mapping")), _ptr(k_cache),
             _ptr(v_cache), n_q, n_kv, d, page_size, num_slots, _ptr(err), _stream()), "skinny_fused")
    return out, new_residual


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` with ``w_gate_up = [Wg; Wu]``: one kernel for few rows, else the
    product followed by the gated-activation kernel.  The fused epilogues compute silu; another
    activation takes the product followed by the activation kernel at every size."""
    M = x.shape[0]
    I = w_gate_up.shape[0] // 2
    out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    if activation != "silu":
        swiglu(linear(x, w_gate_up), out, activation)
        return out
    if M <= SKINNY_MAX_ROWS and skinny_gemm_supported(x, w_gate_up, swiglu=True):
        skinny_gemm(x, w_gate_up, out, "swiglu")
        return out
    if gemm_tc_supported(x, w_gate_up) and gemm_tc_tiles(M, 2 * I, swiglu=True) >= TC_MIN_TILES:
        gemm_tc(x, w_gate_up, out, "swiglu", pair=M >= TC_PAIR_MIN_ROWS)
        return out
    swiglu(linear(x, w_gate_up), out)
    return out


def linear_act(x: torch.Tensor, weight: torch.Tensor, act: str) -> torch.Tensor:
    """``act(x W^T)`` for an ungated feed-forward.  bfloat16 with the exact gelu: the activation rides in the
    epilogue of the product where this package's own kernels run it (few rows: the weight-streaming kernel; enough
    tiles: tcgen05); otherwise the product followed by the activation kernel."""
    M, N = x.shape[0], weight.shape[0]
    if act == "gelu" and x.dtype == torch.bfloat16:
        if M <= SKINNY_MAX_ROWS and skinny_gemm_supported(x, weight):
            out = torch.empty((M, N), dtype=x.dtype, device=x.device)
            skinny_gemm(x, weight, out, "gelu")
            return out
        if gemm_tc_supported(x, weight) and gemm_tc_tiles(M, N) >= TC_MIN_TILES:
            out = torch.empty((M, N), dtype=x.dtype, device=x.device)
            gemm_tc(x, weight, out, "gelu", pair=M >= TC_PAIR_MIN_ROWS)
            return out
    return activation(linear(x, weight), act)


_error_words = {}


def set_error_word(flag: torch.Tensor) -> None:
    """The int32[4] word in which kernels called without an explicit one report a wait that ran out."""
    _error_words[(flag.device.type, flag.device.index)] = flag


def _error_word(device) -> Optional[torch.Tensor]:
    return _error_words.get((device.type, device.index))


TC_MIN_TILES = 96           # below this many 128 x 256 tiles the tcgen05 product leaves too many SMs idle
TC_PAIR_MIN_ROWS = 256      # from here on tiles of 256 x 256 on pairs of SMs (gemm_tc2.cu): a third less operand traffic


def gemm_tc_tiles(M: int, N: int, swiglu: bool = False) -> int:
    """Tiles the tcgen05 product would run; 0 when a tile of 128 rows would be mostly padding."""
    if M < 128:
        return 0
    cols = N // 2 if swiglu else N
    return -(-M // 128) * -(-cols // (128 if swiglu else 256))


def gemm_tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tcgen05 product takes bfloat16, K a multiple of 8 and 16-byte aligned rows (TMA)."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16",
            err: Optional[torch.Tensor] = None, pair: bool = False) -> None:
    """``out = x @ weight^T`` on the tcgen05 tensor cores (TMA operands, accumulator in tensor memory).
    ``epilogue``: ``"bf16"``, ``"f32"``, ``"swiglu"`` (``weight`` holds gate rows then up rows; ``out``
    is ``[M, I]``) or ``"gelu"`` (the exact gelu of every output).  ``pair``: tiles of 256 x 256 on pairs of SMs (``gemm_tc2.cu``) instead of 128 x 256
    on one."""
    _cuda(x, weight, out, err)
    M, K = x.shape
    N = weight.shape[0]
    code = {"bf16": 0, "f32": 1, "swiglu": 2, "gelu": 4}[epilogue]
    cols = N // 2 if epilogue == "swiglu" else N
    want = torch.float32 if epilogue == "f32" else torch.bfloat16
    if not gemm_tc_supported(x, weight) or weight.shape[1] != K:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "gemm_tc: needs bfloat16, K a multiple of 8 and aligned rows")
    if out.shape != (M, cols) or out.dtype != want or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc: out must be {want} [{M}, {cols}]")
    module, entry = ("gemm_tc2", "photon_gemm_tc2") if pair else ("gemm_tc", "photon_gemm_tc")
    f = _fn(module, entry,
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    if err is None:
        err = _error_word(x.device)
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             _ptr(err), _stream()), module)


def rope_table(inv_freq: torch.Tensor, count: int) -> torch.Tensor:
    """``(cos, sin)`` of ``position * inv_freq[j]`` for positions below ``count``, float32
    ``[count, len(inv_freq), 2]``, computed on the device with the expression the rotary kernels use."""
    _cuda(inv_freq)
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "rope_table: inv_freq must be contiguous float32")
    half = inv_freq.numel()
    out = torch.empty((int(count), half, 2), dtype=torch.float32, device=inv_freq.device)
    f = _fn("rope_kv", "photon_rope_table", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(inv_freq), half, int(count), _ptr(out), _stream()), "rope_table")
    return out


def gemm_tc_qkv_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int) -> bool:
    """The q/k/v product with rotation and cache write in its epilogue: the tcgen05 kernel on pairs of SMs with
    enough tiles, heads that are a multiple of 32 wide."""
    M = x.shape[0]
    return (gemm_tc_supported(x, w_qkv) and M >= TC_PAIR_MIN_ROWS and head_dim % 32 == 0
            and gemm_tc_tiles(M, w_qkv.shape[0]) >= TC_MIN_TILES)


def gemm_tc_qkv(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                slot_mapping: torch.Tensor, inv_freq: torch.Tensor, table: Optional[torch.Tensor],
                k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                err: Optional[torch.Tensor] = None) -> None:
    """``x @ w_qkv^T`` (rows of q, then k, then v; rotation partners of q and k as neighbours) with the
    rotation and the cache write in the epilogue: rotated queries to ``q_out [M, n_q * d]``, rotated keys and
    the values to ``slot_mapping`` of the paged cache ``[pages, n_kv, page_size, d]``.  ``table``: from
    ``rope_table`` (positions beyond it are computed in place)."""
    _cuda(x, w_qkv, q_out, positions, slot_mapping, inv_freq, table, k_cache, v_cache, err)
    M, K = x.shape
    if not gemm_tc_supported(x, w_qkv) or w_qkv.shape != ((n_q + 2 * n_kv) * head_dim, K) or head_dim % 32:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "gemm_tc_qkv: needs bfloat16, K a multiple of 8, aligned rows, "
                          "head_dim a multiple of 32 and a weight of (n_q + 2 n_kv) * head_dim rows")
    if q_out.shape != (M, n_q * head_dim) or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc_qkv: q_out must be bfloat16 [{M}, {n_q * head_dim}]")
    for name, t in (("positions", positions), ("slot_mapping", slot_mapping)):
        _int32(t, name)
        if t.numel() < M:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gemm_tc_qkv: {name} must have an entry per row")
    if k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape or k_cache.shape[1] != n_kv \
            or k_cache.shape[3] != head_dim:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "gemm_tc_qkv: the caches must be contiguous bfloat16 [pages, n_kv, page, d]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gemm_tc_qkv: inv_freq must be float32 [head_dim / 2]")
    count = 0
    if table is not None:
        if table.dtype != torch.float32 or table.dim() != 3 or table.shape[1:] != (head_dim // 2, 2) or not table.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gemm_tc_qkv: table must be float32 [positions, head_dim / 2, 2]")
        count = table.shape[0]
    f = _fn("gemm_tc2", "photon_gemm_tc2_qkv",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_long, c_void_p, c_void_p])
    if err is None:
        err = _error_word(x.device)
    _check(f(_ptr(x), x.stride(0), _ptr(w_qkv), w_qkv.stride(0), _ptr(q_out), q_out.stride(0), M, K, _ptr(positions),
             _ptr(slot_mapping), _ptr(inv_freq), _ptr(table), count, _ptr(k_cache), _ptr(v_cache), n_q, n_kv, head_dim,
             k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2], _ptr(err), _stream()), "gemm_tc_qkv")


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] @ weight[N, K]^T``.  float32: this package's FMA kernel (true 32-bit).
    bfloat16: up to 8 rows the weight-streaming kernel; with enough 128 x 256 tiles to fill the
    GPU the tcgen05 kernel; in between the library product (cuBLAS through torch), where the
    reference's engine also calls the library (src/ops/kernels/cuda/matmul_dequant_cached.cu:193-207)."""
    _cuda(x, weight, out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or x.stride(1) != 1 or not weight.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"linear: x [M, {K}] against weight {tuple(weight.shape)}")
    if x.dtype != weight.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"linear: x is {x.dtype}, weight is {weight.dtype}")
    want = out_dtype or x.dtype
    if M <= SKINNY_MAX_ROWS and want in (torch.bfloat16, torch.float32) and skinny_gemm_supported(x, weight):
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        skinny_gemm(x, weight, out, "f32" if want == torch.float32 else "bf16")
        return out
    if want in (torch.bfloat16, torch.float32) and gemm_tc_supported(x, weight) \
            and gemm_tc_tiles(M, N) >= TC_MIN_TILES and (out is None or out.stride(1) == 1):
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        gemm_tc(x, weight, out, "f32" if want == torch.float32 else "bf16", pair=M >= TC_PAIR_MIN_ROWS)
        return out
    if x.dtype == torch.float32:
        if want != torch.float32:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "linear: a float32 product gives float32")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        f = _fn("gemm_f32", "photon_sgemm_nt",
                [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p])
        _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()),
               "sgemm")
        return out
    if want == torch.float32:
        res = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        return torch.mm(x, weight.t())
    torch.mm(x, weight.t(), out=out)
    return out


# ----------------------------------------------------------------------------- attention over a cached latent

def latent_prep(down: torch.Tensor, q_rank: int, kv_rank: int, rot: int, rot_dims: int, q_norm_w: torch.Tensor,
                kv_norm_w: torch.Tensor, eps: float, positions: torch.Tensor, inv_freq: torch.Tensor,
                slot_mapping: torch.Tensor, cq: torch.Tensor, cache: torch.Tensor, err: Optional[torch.Tensor]) -> None:
    """One pass over the fused down-projection rows ``down [T, q_rank + kv_rank + rot]``: the normed query latent
    goes to ``cq [T, q_rank]``, the normed key/value latent and the rotated shared key part to the cache row
    ``slot_mapping[t]`` of ``cache [pages, 1, page_size, kv_rank + rot]``."""
    _cuda(down, q_norm_w, kv_norm_w, positions, inv_freq, slot_mapping, cq, cache, err)
    T = down.shape[0]
    width = kv_rank + rot
    if down.shape[1] != q_rank + width or down.stride(1) != 1 or cq.shape != (T, q_rank) or cq.stride(1) != 1 \
            or cq.dtype != down.dtype or cache.dtype != down.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "latent_prep: down [T, q_rank + kv_rank + rot], cq [T, q_rank], one dtype")
    if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != width or not cache.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "latent_prep: the cache must be contiguous [pages, 1, page_size, kv_rank + rot]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2 or rot_dims % 2 or rot_dims > rot:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "latent_prep: inv_freq must be float32 [rot_dims / 2], rot_dims even and <= rot")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    f = _fn("latent", "photon_latent_prep",
            [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p,
             c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p])
    _check(f(_ptr(down), down.stride(0), _dtype_code(down), q_rank, kv_rank, rot, rot_dims, _ptr(q_norm_w),
             _dtype_code(q_norm_w), _ptr(kv_norm_w), _dtype_code(kv_norm_w), float(eps), _ptr(positions), _ptr(inv_freq),
             _ptr(slot_mapping), _ptr(cq), cq.stride(0), _ptr(cache), cache.shape[0] * cache.shape[2], T, _ptr(err),
             _stream()), "latent_prep")


def latent_q_rope(q: torch.Tensor, heads: int, dim: int, rot: int, rot_dims: int, positions: torch.Tensor,
                  inv_freq: torch.Tensor, out: torch.Tensor, out_off: int) -> None:
    """The last ``rot`` numbers of every head of ``q [T, heads * (dim + rot)]``, rotated, into
    ``out [T, heads, out_head]`` at offset ``out_off`` of every head."""
    _cuda(q, positions, inv_freq, out)
    T = q.shape[0]
    if q.shape[1] != heads * (dim + rot) or q.stride(1) != 1 or out.dim() != 3 or out.shape[:2] != (T, heads) \
            or out.stride(2) != 1 or out.stride(1) != out.shape[2] or out.dtype != q.dtype or out_off + rot > out.shape[2]:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "latent_q_rope: q [T, heads * (dim + rot)], out [T, heads, >= out_off + rot]")
    _int32(positions, "positions")
    f = _fn("latent", "photon_latent_q_rope",
            [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int,
             c_int, c_void_p])
    _check(f(_ptr(q), q.stride(0), _dtype_code(q), heads, dim, rot, rot_dims, _ptr(positions), _ptr(inv_freq), _ptr(out),
             out.stride(0), out.shape[2], out_off, T, _stream()), "latent_q_rope")


def latent_decode_supported(q: torch.Tensor, width: int, value_dim: int) -> bool:
    """The tensor-core kernel for decoded tokens over a cached latent: bfloat16, row and value widths multiples of 16."""
    return (q.dtype == torch.bfloat16 and width % 16 == 0 and value_dim % 16 == 0 and value_dim <= width
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and (80 * (width + 8) * 2 + 16384) <= 220 * 1024)


def latent_decode_attention(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                            token_seq: torch.Tensor, positions: torch.Tensor, heads: int, width: int, value_dim: int,
                            scale: float, max_context: int, err: Optional[torch.Tensor]) -> None:
    """Attention of decoded tokens (or of the few tokens of a short portion) over cached latent rows on the tensor
    cores: ``q [T, heads * width]``, ``cache [pages, 1, page_size, width]``, ``out [T, heads * value_dim]``; every token
    sees the rows up to its own position, a row's value is its first ``value_dim`` numbers.  ``max_context``: an upper
    bound of the tokens' contexts (sizes the grid: one block per token and 64 rows)."""
    _cuda(q, out, cache, block_table, token_seq, positions, err)
    T = q.shape[0]
    if not latent_decode_supported(q, width, value_dim) or q.shape[1] != heads * width or q.stride(1) != 1 \
            or out.shape != (T, heads * value_dim) or out.stride(1) != 1 or out.dtype != q.dtype or cache.dtype != q.dtype \
            or cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != width or not cache.is_contiguous():
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "latent_decode_attention: bfloat16, widths that are multiples of 16")
    for name, t in (("block_table", block_table), ("token_seq", token_seq), ("positions", positions)):
        _int32(t, name)
    splits = max(1, -(-int(max_context) // 64))
    part = torch.empty(T * heads * splits * (value_dim + 2), dtype=torch.float32, device=q.device)
    f = _fn("latent", "photon_latent_decode_attention",
            [c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_float, c_int, c_void_p, c_void_p, c_long, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(positions), T,
             heads, width, value_dim, cache.shape[2], cache.shape[0], float(scale), splits, _ptr(part), _ptr(out),
             out.stride(0), _ptr(err), _stream()), "latent_decode_attention")
    global _launch_count
    _launch_count += 1


#: From this many rows on the bfloat16 per-head products go to the library's batched product.
HEAD_LINEAR_LIBRARY_ROWS = 16


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, h, :] = weight[h] @ x[t, h, :]`` for all heads at once: ``x [T, heads, K]`` and
    ``out [T, heads, N]`` are views with free row and head strides, ``weight [heads, N, K]`` is contiguous.
    float32 and few rows: this package's kernel (one chain of fused multiply-adds per output); many bfloat16
    rows: the library's batched product."""
    _cuda(x, weight, out)
    T, heads, K = x.shape
    N = weight.shape[1]
    if weight.shape != (heads, N, K) or not weight.is_contiguous() or out.shape != (T, heads, N) \
            or x.stride(2) != 1 or out.stride(2) != 1 or x.dtype != weight.dtype or out.dtype != x.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "head_linear: x [T, heads, K], weight [heads, N, K], out [T, heads, N]")
    if x.dtype == torch.bfloat16 and T >= HEAD_LINEAR_LIBRARY_ROWS:
        torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
        return
    f = _fn("latent", "photon_head_linear",
            [c_void_p, c_long, c_long, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), x.stride(1), _ptr(weight), _ptr(out), out.stride(0), out.stride(1), _dtype_code(x),
             T, heads, N, K, _stream()), "head_linear")


def gather_rows(cache: torch.Tensor, table: torch.Tensor, count: int, err: Optional[torch.Tensor]) -> torch.Tensor:
    """The first ``count`` cached rows of the request whose pages are ``table`` (one row of a block table), as
    one dense matrix ``[count, width]``; ``cache [pages, 1, page_size, width]``."""
    _cuda(cache, table, err)
    _int32(table, "table")
    pages, _, page_size, width = cache.shape
    if count > table.numel() * page_size or not cache.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "gather_rows: more rows asked for than the table's pages hold")
    out = torch.empty((count, width), dtype=cache.dtype, device=cache.device)
    f = _fn("latent", "photon_gather_rows", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(cache), _dtype_code(cache), _ptr(table), page_size, pages, width, int(count), _ptr(out), _ptr(err), _stream()),
           "gather_rows")
    return out


def causal_softmax_rows(scores: torch.Tensor, probs: torch.Tensor, heads: int, first_pos: int, scale: float) -> None:
    """``probs = softmax(scale * scores)`` row by row over the keys each row may see: row ``r`` belongs to the token
    at position ``first_pos + r // heads`` and sees the keys up to that position; zero beyond."""
    _cuda(scores, probs)
    rows, cols = scores.shape
    if scores.dtype != torch.float32 or scores.stride(1) != 1 or probs.shape != scores.shape or probs.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "causal_softmax_rows: scores float32 [rows, cols], probs of the same shape")
    f = _fn("latent", "photon_causal_softmax_rows",
            [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(scores), scores.stride(0), _ptr(probs), probs.stride(0), _dtype_code(probs), rows, int(heads), int(first_pos),
             cols, float(scale), _stream()), "causal_softmax_rows")


# ----------------------------------------------------------------------------- gated delta rule

def delta_conv(x: torch.Tensor, taps_w: torch.Tensor, token_seq: torch.Tensor, cu_tokens: torch.Tensor,
               state_slots: torch.Tensor, state: torch.Tensor, conv_offset: int, y: torch.Tensor, num_seqs: int, qk_heads: int,
               heads: int, dim: int, vdim: int, err: Optional[torch.Tensor]) -> None:
    """Short causal convolution with silu over the projected ``[q | k | v]`` rows ``x [T, C]`` (a view with a row
    stride), ``taps_w [C, taps]`` float32; q and k heads become unit vectors (q also times ``dim^-0.5``); ``y [T, C]``
    float32.  The ``taps - 1`` rows before a request's first token of the step come from its state row (at
    ``conv_offset``), which is then brought up to date.  ``state [slots, row]`` float32."""
    _cuda(x, taps_w, token_seq, cu_tokens, state_slots, state, y, err)
    T = x.shape[0]
    C = 2 * qk_heads * dim + heads * vdim
    taps = taps_w.shape[1]
    if x.shape[1] != C or x.stride(1) != 1 or taps_w.shape != (C, taps) or taps_w.dtype != torch.float32 or not taps_w.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"delta_conv: x [T, {C}] and float32 taps [{C}, taps]")
    if y.shape != (T, C) or y.dtype != torch.float32 or not y.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_conv: y must be contiguous float32 [T, C]")
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < conv_offset + (taps - 1) * C:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_conv: state must be contiguous float32 [slots, row] with room for the taps")
    for t, what in ((token_seq, "token_seq"), (cu_tokens, "cu_tokens"), (state_slots, "state_slots")):
        _int32(t, what)
    f = _fn("delta", "photon_delta_conv",
            [c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _dtype_code(x), _ptr(taps_w), taps, _ptr(token_seq), _ptr(cu_tokens), _ptr(state_slots),
             _ptr(state), state.stride(0), int(conv_offset), state.shape[0], _ptr(y), T, int(num_seqs), qk_heads, heads, dim, vdim,
             _ptr(err), _stream()), "delta_conv")


def delta_recurrent(y: torch.Tensor, ab: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, cu_tokens: torch.Tensor,
                    state_slots: torch.Tensor, state: torch.Tensor, o: torch.Tensor, num_seqs: int, qk_heads: int, heads: int,
                    dim: int, vdim: int, err: Optional[torch.Tensor]) -> None:
    """The gated delta rule over the tokens of a step, request by request: ``y [T, C]`` from ``delta_conv``,
    ``ab [T, 2 heads]`` (a view with a row stride: the raw decay inputs, then the raw beta inputs), ``a_log``,
    ``dt_bias`` float32 ``[heads]``; ``o [T, heads * vdim]`` float32 receives the read-outs.  The state matrices are
    the first ``heads * dim * vdim`` numbers of a request's state row."""
    _cuda(y, ab, a_log, dt_bias, cu_tokens, state_slots, state, o, err)
    T = y.shape[0]
    if ab.shape != (T, 2 * heads) or ab.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_recurrent: ab must be [T, 2 * heads]")
    if o.shape != (T, heads * vdim) or o.dtype != torch.float32 or not o.is_contiguous() or y.dtype != torch.float32 or not y.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_recurrent: y and o must be contiguous float32")
    for t in (a_log, dt_bias):
        if t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_recurrent: a_log and dt_bias float32 [heads]")
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < heads * dim * vdim:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_recurrent: state must be contiguous float32 [slots, row]")
    _int32(cu_tokens, "cu_tokens")
    _int32(state_slots, "state_slots")
    f = _fn("delta", "photon_delta_recurrent",
            [c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(y), _ptr(ab), ab.stride(0), _dtype_code(ab), _ptr(a_log), _ptr(dt_bias), _ptr(cu_tokens), _ptr(state_slots),
             _ptr(state), state.stride(0), state.shape[0], _ptr(o), int(num_seqs), qk_heads, heads, dim, vdim, _ptr(err),
             _stream()), "delta_recurrent")


def delta_out(o: torch.Tensor, z: torch.Tensor, norm_w: torch.Tensor, eps: float, out: torch.Tensor, heads: int, vdim: int) -> None:
    """``out = o / sqrt(mean(o^2) + eps) * norm_w * silu(z)`` per head over ``vdim``; ``o`` float32, ``z`` a view."""
    _cuda(o, z, norm_w, out)
    T = o.shape[0]
    if z.shape != o.shape or z.stride(1) != 1 or out.shape != o.shape or out.stride(1) != 1 or norm_w.dtype != torch.float32 \
            or norm_w.numel() != vdim or o.dtype != torch.float32 or not o.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "delta_out: o float32 [T, heads * vdim], z and out alike, norm_w float32 [vdim]")
    f = _fn("delta", "photon_delta_out", [c_void_p, c_void_p, c_long, c_int, c_void_p, c_float, c_void_p, c_long, c_int, c_int,
                                          c_int, c_int, c_void_p])
    _check(f(_ptr(o), _ptr(z), z.stride(0), _dtype_code(z), _ptr(norm_w), float(eps), _ptr(out), out.stride(0), _dtype_code(out),
             T, heads, vdim, _stream()), "delta_out")


# ----------------------------------------------------------------------------- norms over parts of a row

GATE_MODES = {None: 0, "silu_before": 1, "sigmoid_after": 2}


def group_rmsnorm(x: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, groups: int,
                  out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                  gate: Optional[torch.Tensor] = None, gate_mode: Optional[str] = None,
                  x_bias: Optional[torch.Tensor] = None) -> None:
    """RMS norm in ``groups`` equal consecutive parts of a row: every part of ``x [T, H]`` (a view with a row stride) is
    divided by its own ``sqrt(mean(part^2) + eps)``, the whole times ``weight [H]``.  ``gate`` (float32 ``[T, H]`` view):
    ``gate_mode`` ``silu_before`` multiplies the row by ``silu(gate)`` before the norm, ``sigmoid_after`` the normed row by
    ``sigmoid(gate)``.  ``residual`` (contiguous float32 ``[T, H]``): the result is added to it in place, and ``out`` (may
    then be None) receives the stream's new rows in its own type; with ``x`` None ``out`` just receives the stream's rows.
    Without a residual ``out`` receives the result.  ``x_bias [H]``: added to every row of ``x`` first (the bias of the
    product that made ``x``, which then needs no pass of its own)."""
    _cuda(x, weight, out, residual, gate, x_bias)
    if x_bias is not None and (x is None or x_bias.numel() != x.shape[1] or not x_bias.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "group_rmsnorm: x_bias must be contiguous [H] and goes with x")
    ref = x if x is not None else residual
    if ref is None or (out is None and residual is None):
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "group_rmsnorm: nothing to read or nothing to write")
    T, H = ref.shape
    if x is not None and (x.stride(1) != 1 or weight is None or weight.numel() != H or not weight.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "group_rmsnorm: x [T, H] with unit column stride and weight [H]")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != (T, H) or not residual.is_contiguous()):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "group_rmsnorm: the residual stream must be contiguous float32 [T, H]")
    if out is not None and (out.shape != (T, H) or out.stride(1) != 1):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "group_rmsnorm: out must be [T, H]")
    if groups <= 0 or H % groups:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"group_rmsnorm: {H} numbers do not split into {groups} equal parts")
    if gate_mode not in GATE_MODES or (gate is None) != (gate_mode is None):
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "group_rmsnorm: a gate goes with a gate mode (silu_before, sigmoid_after)")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != (T, H) or gate.stride(1) != 1):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "group_rmsnorm: the gate must be a float32 [T, H] view")
    f = _fn("row_norms", "photon_group_rmsnorm",
            [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int,
             c_int, c_float, c_void_p, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0) if x is not None else 0, _dtype_code(x) if x is not None else F32, _ptr(gate),
             gate.stride(0) if gate is not None else 0, GATE_MODES[gate_mode], _ptr(residual), _ptr(weight),
             _dtype_code(weight) if weight is not None else F32, _ptr(out), out.stride(0) if out is not None else 0,
             _dtype_code(out) if out is not None else F32, T, H, int(groups), float(eps), _ptr(x_bias),
             _dtype_code(x_bias) if x_bias is not None else F32, _stream()), "group_rmsnorm")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = a N(z) + b N(z^2) + c N(z^3) + e`` per row, powers element by element, ``N(u) = u / sqrt(mean(u^2) + eps)``;
    ``coef [4] = (a, b, c, e)``."""
    _cuda(z, coef, out)
    T, F = z.shape
    if z.stride(1) != 1 or out.shape != (T, F) or out.stride(1) != 1 or coef.numel() != 4 or not coef.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "polynorm: z and out [T, F], coef [4]")
    f = _fn("row_norms", "photon_polynorm", [c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int,
                                             c_float, c_void_p])
    _check(f(_ptr(z), z.stride(0), _dtype_code(z), _ptr(coef), _dtype_code(coef), _ptr(out), out.stride(0), _dtype_code(out),
             T, F, float(eps), _stream()), "polynorm")


def softcap_(x: torch.Tensor, cap: float) -> None:
    """``x <- cap * tanh(x / cap)`` in place (contiguous float32)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "softcap: x must be contiguous float32")
    f = _fn("row_norms", "photon_softcap", [c_void_p, c_long, c_float, c_void_p])
    _check(f(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


# ----------------------------------------------------------------------------- attention with two score maps per head

def diff_prep(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_out: torch.Tensor,
              q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor], v_bias: Optional[torch.Tensor],
              q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
              inv_freq: Optional[torch.Tensor], rot_dims: int, slot_mapping: Optional[torch.Tensor],
              k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int,
              value_dim: int, err: Optional[torch.Tensor]) -> None:
    """Biases, the per-(head, map) RMS norm with a shared weight ``[dim]``, and the rotation of the first ``rot_dims``
    numbers for ``q [T, heads * 2 * dim]`` and ``k [T, kv_heads * 2 * dim]`` (views); queries into ``q_out``, keys into
    ``k_cache [pages, kv_heads, page_size, 2 * dim]`` and ``v [T, kv_heads * value_dim]`` (plus bias) into ``v_cache
    [pages, kv_heads, page_size, value_dim]``.  Caches None: queries only."""
    _cuda(q, k, v, q_out, q_bias, k_bias, v_bias, q_weight, k_weight, positions, inv_freq, slot_mapping, k_cache, v_cache, err)
    T = q.shape[0]
    d, dv = dim, value_dim
    if q.shape != (T, heads * 2 * d) or q.stride(1) != 1 or q_out.shape != q.shape or q_out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_prep: q and q_out must be [T, heads * 2 * dim]")
    write = k_cache is not None
    page_size, num_slots = 1, 0
    if write:
        if k is None or v is None or k.shape != (T, kv_heads * 2 * d) or v.shape != (T, kv_heads * dv) or k.stride(1) != 1 \
                or v.stride(1) != 1 or k.dtype != q.dtype or v.dtype != q.dtype:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_prep: k [T, kv_heads * 2 * dim], v [T, kv_heads * value_dim]")
        _int32(slot_mapping, "slot_mapping")
        if k_cache.dim() != 4 or k_cache.shape[1] != kv_heads or k_cache.shape[3] != 2 * d or v_cache.shape[:3] != k_cache.shape[:3] \
                or v_cache.shape[3] != dv or k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype \
                or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH,
                              "diff_prep: caches must be contiguous [pages, kv_heads, page_size, 2 * dim | value_dim]")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    _int32(positions, "positions")
    if inv_freq is not None and (inv_freq.dtype != torch.float64 or inv_freq.numel() != rot_dims // 2 or rot_dims % 2 or rot_dims > d):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_prep: inv_freq must be float64 [rot_dims / 2], rot_dims even, <= dim")
    biases = [b for b in (q_bias, k_bias, v_bias) if b is not None]
    weights = [w for w in (q_weight, k_weight) if w is not None]
    if any(b.dtype != biases[0].dtype or not b.is_contiguous() for b in biases) or \
            any(w.dtype != weights[0].dtype or w.numel() != d or not w.is_contiguous() for w in weights):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_prep: biases of one dtype, norm weights [dim] of one dtype")
    f = _fn("attention_diff", "photon_diff_prep",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_long, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k) if write else None, k.stride(0) if write else 0, _ptr(v) if write else None,
             v.stride(0) if write else 0, _dtype_code(q), _ptr(q_out), q_out.stride(0), _dtype_code(q_out), _ptr(q_bias),
             _ptr(k_bias) if write else None, _ptr(v_bias) if write else None, _dtype_code(biases[0]) if biases else F32,
             _ptr(q_weight), _ptr(k_weight), _dtype_code(weights[0]) if weights else F32, float(eps), _ptr(positions),
             _ptr(inv_freq) if rot_dims else None, int(rot_dims) if inv_freq is not None else 0,
             _ptr(slot_mapping) if write else None, _ptr(k_cache), _ptr(v_cache), T, heads, kv_heads, d, dv, page_size, num_slots,
             _ptr(err), _stream()), "diff_prep")


def diff_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                   token_seq: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int, dim: int, value_dim: int,
                   window: Optional[int], scale: float, lam: float, out_scale: float, eps: float,
                   err: Optional[torch.Tensor]) -> None:
    """Differential attention, the general kernel.  ``q [T, heads * 2 * dim]`` (view), ``out [T, heads * value_dim]``; per
    head two softmax maps over the keys ``max(0, p - window + 1) .. p`` share the values; ``o = a1 - lam * a2``, then
    ``o / sqrt(mean(o^2) + eps) * out_scale`` per head."""
    _cuda(q, out, k_cache, v_cache, block_table, token_seq, positions, err)
    T = q.shape[0]
    if q.shape[1] != heads * 2 * dim or q.stride(1) != 1 or out.shape != (T, heads * value_dim) or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_attention: q must be [T, heads * 2 * dim], out [T, heads * value_dim]")
    if q.dtype != out.dtype or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "diff_attention: q, out and the caches must share one dtype")
    if k_cache.dim() != 4 or k_cache.shape[1] != kv_heads or k_cache.shape[3] != 2 * dim or v_cache.shape[3] != value_dim \
            or v_cache.shape[:3] != k_cache.shape[:3] or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_attention: caches [pages, kv_heads, page_size, 2 * dim | value_dim]")
    for name, t in (("block_table", block_table), ("token_seq", token_seq), ("positions", positions)):
        _int32(t, name)
    f = _fn("attention_diff", "photon_diff_attention",
            [c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _dtype_code(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(token_seq), _ptr(positions), T, heads, kv_heads, dim, value_dim, k_cache.shape[2],
             k_cache.shape[0], int(window) if window else 0, float(scale), float(lam), float(out_scale), float(eps), _ptr(err),
             _stream()), "diff_attention")


def diff_mma_supported(dtype: torch.dtype, heads: int, kv_heads: int, dim: int, value_dim: int) -> bool:
    """The tensor-core kernel takes bfloat16, sizes that are multiples of 16, at most 64 query heads per key/value head,
    and what fits its shared memory (queries of 64 rows, two stages of 64 keys and values, the two maps' outputs)."""
    if dtype != torch.bfloat16 or dim % 16 or value_dim % 16 or heads // kv_heads > 64:
        return False
    stages, fin = 2 * 64 * (2 * dim + value_dim) * 2, 2 * 64 * value_dim * 4
    return 64 * 2 * dim * 2 + max(stages, fin) <= 220 * 1024 and value_dim <= 256


def diff_attention_mma(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                       cu_tokens: torch.Tensor, positions: torch.Tensor, query_lens, heads: int, kv_heads: int, dim: int,
                       value_dim: int, window: Optional[int], scale: float, lam: float, out_scale: float, eps: float,
                       err: Optional[torch.Tensor], splits: int = 1) -> None:
    """``diff_attention`` on the tensor cores (bfloat16): a block owns the query heads of one key/value head for up to
    ``64 / (heads / kv_heads)`` neighbouring tokens of a request.  ``query_lens``: the requests' token counts (host).
    ``splits`` > 1 shares every block's key tiles out over that many blocks (decode steps); a second kernel puts the
    shares together in their order."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, err)
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "diff_attention_mma: bfloat16 only")
    if q.shape[1] != heads * 2 * dim or q.stride(1) != 1 or out.shape != (T, heads * value_dim) or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_attention_mma: q must be [T, heads * 2 * dim], out [T, heads * value_dim]")
    if k_cache.dim() != 4 or k_cache.shape[1] != kv_heads or k_cache.shape[3] != 2 * dim or v_cache.shape[3] != value_dim \
            or v_cache.shape[:3] != k_cache.shape[:3] or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "diff_attention_mma: caches [pages, kv_heads, page_size, 2 * dim | value_dim]")
    for name, t in (("block_table", block_table), ("cu_tokens", cu_tokens), ("positions", positions)):
        _int32(t, name)
    per_block = 64 // (heads // kv_heads)
    tiles = sum(-(-int(n) // per_block) for n in query_lens)
    f = _fn("attention_diff_mma", "photon_diff_mma",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p],
            defines={"DIFF_D": dim, "DIFF_DV": value_dim})
    splits = max(1, min(int(splits), 64))
    part = talk_scratch(q.device, T * heads * 2 * splits * (value_dim + 2)) if splits > 1 else None
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(cu_tokens), _ptr(positions), len(query_lens), tiles, heads, kv_heads, k_cache.shape[2], k_cache.shape[0],
             int(window) if window else 0, float(scale), float(lam), float(out_scale), float(eps), splits, _ptr(part), T, _ptr(err),
             _stream()), "diff_attention_mma")
    if splits > 1:
        global _launch_count
        _launch_count += 1


# ----------------------------------------------------------------------------- recurrences with one decay per head and token

def conv_silu(x: torch.Tensor, taps_w: torch.Tensor, bias: Optional[torch.Tensor], token_seq: torch.Tensor,
              cu_tokens: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, conv_offset: int, y: torch.Tensor,
              num_seqs: int, err: Optional[torch.Tensor]) -> None:
    """``y = silu(bias + causal convolution per channel)`` of ``x [T, C]`` (a view), ``taps_w`` float32 ``[C, taps]`` (the last
    column weighs the current token), ``y`` float32 ``[T, C]``.  The ``taps - 1`` rows before a request's first token of the
    step come from its state row at ``conv_offset``; afterwards the state gets the request's last ``taps - 1`` input rows."""
    _cuda(x, taps_w, bias, token_seq, cu_tokens, state_slots, state, y, err)
    T, C = x.shape
    taps = taps_w.shape[1]
    if x.stride(1) != 1 or taps_w.shape != (C, taps) or taps_w.dtype != torch.float32 or not taps_w.is_contiguous() or \
            (bias is not None and (bias.dtype != torch.float32 or bias.numel() != C or not bias.is_contiguous())):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"conv_silu: x [T, {C}], float32 taps [{C}, taps] and bias [{C}]")
    if y.shape != (T, C) or y.dtype != torch.float32 or not y.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "conv_silu: y must be contiguous float32 [T, C]")
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < conv_offset + (taps - 1) * C:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "conv_silu: state must be contiguous float32 [slots, row] with room for the taps")
    for t, what in ((token_seq, "token_seq"), (cu_tokens, "cu_tokens"), (state_slots, "state_slots")):
        _int32(t, what)
    f = _fn("linrec", "photon_conv_silu",
            [c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long, c_int,
             c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _dtype_code(x), _ptr(taps_w), _ptr(bias), taps, _ptr(token_seq), _ptr(cu_tokens),
             _ptr(state_slots), _ptr(state), state.stride(0), int(conv_offset), state.shape[0], _ptr(y), T, C, _ptr(err),
             _stream()), "conv_silu")
    if taps > 1:
        g = _fn("linrec", "photon_conv_state",
                [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_void_p])
        _check(g(_ptr(x), x.stride(0), _dtype_code(x), taps, _ptr(cu_tokens), _ptr(state_slots), _ptr(state), state.stride(0),
                 int(conv_offset), state.shape[0], int(num_seqs), C, _stream()), "conv_state")


LINREC_MODES = {"state_space": 0, "matrix_memory": 1}


def linrec(mode: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate_a: torch.Tensor, gate_b: Optional[torch.Tensor],
           p0: torch.Tensor, p1: torch.Tensor, p2: Optional[torch.Tensor], cap: float, q_scale: float, cu_tokens: torch.Tensor,
           state_slots: torch.Tensor, state: torch.Tensor, out: torch.Tensor, num_seqs: int, heads: int, qk_heads: int,
           dim: int, vdim: int, err: Optional[torch.Tensor]) -> None:
    """The recurrence ``S <- keep S + take k v^T, o = S^T q`` over the tokens of a step, per request and head, with the
    state ``[heads, dim, vdim]`` (then, for ``matrix_memory``, ``n [heads, dim]`` and ``m [heads]``) at the start of the
    request's float32 state row.  ``state_space``: ``gate_a`` = raw step sizes ``[T, heads]``, ``p0, p1, p2`` = ``A_log``,
    ``dt_bias``, ``D``; the output is ``o + D v``.  ``matrix_memory``: ``gate_a, gate_b`` = raw input and forget gates, ``p0,
    p1`` their biases, ``cap`` their bound; the output is ``o / (max(|n . q|, exp(-m)) + 1e-6)``.  All inputs float32 views
    with unit column stride; ``out`` float32 ``[T, heads * vdim]``."""
    _cuda(q, k, v, gate_a, gate_b, p0, p1, p2, cu_tokens, state_slots, state, out, err)
    if mode not in LINREC_MODES:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"linrec: unknown mode {mode!r}")
    T = q.shape[0]
    for t, w, what in ((q, qk_heads * dim, "q"), (k, qk_heads * dim, "k"), (v, heads * vdim, "v"), (gate_a, heads, "gate_a"),
                       (gate_b, heads, "gate_b"), (out, heads * vdim, "out")):
        if t is not None and (t.dtype != torch.float32 or t.shape != (T, w) or t.stride(1) != 1):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"linrec: {what} must be a float32 [T, {w}] view")
    if gate_b is not None and gate_b.stride(0) != gate_a.stride(0):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "linrec: both gates must have one row stride")
    if (mode == "matrix_memory") != (gate_b is not None):
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "linrec: the matrix memory has two gates, the state-space layer one")
    for t, what in ((p0, "p0"), (p1, "p1"), (p2, "p2")):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous()):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"linrec: {what} must be float32 [heads]")
    need = heads * dim * vdim + (heads * dim + heads if mode == "matrix_memory" else 0)
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < need:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "linrec: state must be contiguous float32 [slots, row]")
    _int32(cu_tokens, "cu_tokens")
    _int32(state_slots, "state_slots")
    f = _fn("linrec", "photon_linrec",
            [c_int, c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p,
             c_float, c_float, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p])
    _check(f(LINREC_MODES[mode], _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(gate_a), _ptr(gate_b),
             gate_a.stride(0), _ptr(p0), _ptr(p1), _ptr(p2), float(cap), float(q_scale), _ptr(cu_tokens), _ptr(state_slots),
             _ptr(state), state.stride(0), state.shape[0], _ptr(out), out.stride(0), int(num_seqs), heads, qk_heads, dim, vdim,
             _ptr(err), _stream()), "linrec")


# ----------------------------------------------------------------------------- attention whose heads' scores are mixed

def talk_prep(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor],
              q_out: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dims: int,
              slot_mapping: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
              n_q: int, n_kv: int, d: int, err: Optional[torch.Tensor]) -> None:
    """Bias and rotation of the projected ``q [T, n_q * d]`` and ``k [T, n_kv * d]`` (views with row strides) in
    32-bit; ``q_out`` gets the queries, ``k_cache`` the rotated keys and ``v_cache`` (may be None) the values:
    ``v [T, n_kv * d]`` or, with ``v`` None, the keys before their rotation; all at ``slot_mapping``.  ``k_cache``
    None: nothing is stored."""
    _cuda(q, k, v, q_bias, k_bias, q_out, positions, inv_freq, slot_mapping, k_cache, v_cache, err)
    T = q.shape[0]
    if q.shape != (T, n_q * d) or q.stride(1) != 1 or q_out.shape != (T, n_q * d) or q_out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_prep: q and q_out must be [T, n_q * d]")
    store = k_cache is not None
    if v is not None and (v.shape != (T, n_kv * d) or v.stride(1) != 1 or v.dtype != q.dtype or v_cache is None):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_prep: v must be [T, n_kv * d] of q's type, with a value cache")
    if store and (k is None or k.shape != (T, n_kv * d) or k.stride(1) != 1 or k.dtype != q.dtype or slot_mapping is None
                  or k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or not k_cache.is_contiguous()
                  or k_cache.dtype != q_out.dtype or (v_cache is not None and (v_cache.shape != k_cache.shape or not v_cache.is_contiguous()
                                                                                  or v_cache.dtype != k_cache.dtype))):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_prep: k [T, n_kv * d] and caches [pages, n_kv, page, d] of q_out's type")
    for b, n in ((q_bias, n_q * d), (k_bias, n_kv * d)):
        if b is not None and (b.dtype != torch.float32 or b.numel() != n or not b.is_contiguous()):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_prep: biases must be contiguous float32")
    if inv_freq is not None and (inv_freq.dtype != torch.float64 or inv_freq.numel() != rot_dims // 2):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_prep: inv_freq must be float64 [rot_dims / 2]")
    _int32(positions, "positions")
    page_size = k_cache.shape[2] if store else 1
    num_slots = k_cache.shape[0] * page_size if store else 0
    f = _fn("attention_talk", "photon_talk_prep",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p,
             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_long, c_void_p, c_void_p])
    v_in = v if store and v is not None else None
    _check(f(_ptr(q), q.stride(0), _ptr(k if store else None), k.stride(0) if store else 0, _ptr(v_in),
             v_in.stride(0) if v_in is not None else 0, _dtype_code(q), _ptr(q_bias),
             _ptr(k_bias), _ptr(q_out), q_out.stride(0), _dtype_code(q_out), _ptr(positions), _ptr(inv_freq),
             int(rot_dims) if inv_freq is not None else 0, _ptr(slot_mapping if store else None), _ptr(k_cache if store else None),
             _ptr(v_cache if store else None), T, n_q, n_kv, d, page_size, num_slots, _ptr(err), _stream()), "talk_prep")


_talk_scratch = {}


def talk_scratch(device, floats: int) -> torch.Tensor:
    """Partial results of split attention: one buffer per device that only grows; a buffer it outgrows is kept,
    because a captured step may hold its address."""
    key = (device.type, device.index)
    kept = _talk_scratch.setdefault(key, [])
    if not kept or kept[-1].numel() < floats:
        kept.append(torch.empty((max(floats, 1 << 20),), dtype=torch.float32, device=device))
    return kept[-1]


def talk_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                   token_seq: torch.Tensor, positions: torch.Tensor, n_q: int, n_kv: int, d: int, window: Optional[int],
                   qmul: torch.Tensor, talk: Optional[torch.Tensor], sink: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                   err: Optional[torch.Tensor], splits: int = 1) -> None:
    """Paged causal attention over all heads of a token at once: raw scores times ``qmul [n_q]``, mixed across the heads
    by ``talk [n_q, n_q]``, a window, ``exp(sink[h])`` in the softmax's denominator, outputs times ``sigmoid(gate)``
    (``gate [T, n_q]`` float32, a view).  The general kernel: 32-bit arithmetic on any sizes, a sum's order depends on
    the token's position alone (``splits`` 1)."""
    _cuda(q, out, k_cache, v_cache, block_table, token_seq, positions, qmul, talk, sink, gate, err)
    T = q.shape[0]
    if q.shape != (T, n_q * d) or q.stride(1) != 1 or out.shape != (T, n_q * d) or out.stride(1) != 1 or out.dtype != q.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention: q and out must be [T, n_q * d] of one type")
    if k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or v_cache.shape != k_cache.shape \
            or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention: caches must be [pages, n_kv, page, d] of q's type")
    for t_, n in ((qmul, n_q), (talk, n_q * n_q), (sink, n_q)):
        if t_ is not None and (t_.dtype != torch.float32 or t_.numel() != n or not t_.is_contiguous()):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention: qmul, talk and sink must be contiguous float32")
    if gate is not None and (gate.shape != (T, n_q) or gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention: gate must be float32 [T, n_q]")
    for t_, what in ((block_table, "block_table"), (token_seq, "token_seq"), (positions, "positions")):
        _int32(t_, what)
    part = talk_scratch(q.device, T * splits * n_q * (d + 2)) if splits > 1 else None
    f = _fn("attention_talk", "photon_talk_attention",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p,
             c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _dtype_code(q), _ptr(block_table),
             block_table.shape[1], _ptr(token_seq), _ptr(positions), T, n_q, n_kv, d, k_cache.shape[2], k_cache.shape[0],
             int(window or 0), _ptr(qmul), _ptr(talk), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
             int(splits), _ptr(part), _ptr(err), _stream()), "talk_attention")


def talk_mma_supported(n_q: int, n_kv: int, d: int) -> bool:
    """Whether the tensor-core kernel of ``talk_attention_mma`` can be compiled for these sizes: the head size a
    multiple of 16 up to 256, the accumulators of a warp's heads within its registers, shared memory for a tile of 32
    keys.  Mirrors the static checks of ``attention_talk_mma.cu``."""
    if d % 16 or not 16 <= d <= 256 or n_kv <= 0 or n_q % n_kv:
        return False
    warps = max(4, n_q) if n_q <= 8 else 16
    heads_per_warp = -(-n_q // warps)
    if heads_per_warp * d > (128 if warps > 8 else 256):
        return False
    smem = lambda bn: n_q * 16 * (d + 8) * 2 + 2 * n_kv * bn * (d + 8) * 2 + n_q * 16 * (bn + 8) * 4 + n_q * ((n_q + 3) & ~3) * 8 + 128
    return smem(32) <= 226 * 1024


def talk_attention_mma(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                       cu_tokens: torch.Tensor, positions: torch.Tensor, num_seqs: int, max_tokens: int, n_q: int, n_kv: int,
                       d: int, window: Optional[int], qmul: torch.Tensor, talk: Optional[torch.Tensor],
                       sink: Optional[torch.Tensor], gate: Optional[torch.Tensor], err: Optional[torch.Tensor],
                       splits: int = 1) -> None:
    """``talk_attention`` on the tensor cores (bfloat16): one block per 16 neighbouring tokens of a request with all
    heads; raw scores and weighted sums as mma.m16n8k16 with 32-bit sums, the mixing of the heads' scores and the
    softmax in 32-bit.  ``splits`` > 1 shares a token's key tiles out over that many blocks, merged in split order."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, positions, qmul, talk, sink, gate, err)
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or not talk_mma_supported(n_q, n_kv, d):
        raise PhotonError(ErrorCode.UNSUPPORTED, "talk_attention_mma: bfloat16 and sizes that talk_mma_supported accepts")
    if q.shape != (T, n_q * d) or q.stride(1) != 1 or out.shape != (T, n_q * d) or out.stride(1) != 1 or out.dtype != q.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention_mma: q and out must be [T, n_q * d] of one type")
    if k_cache.dim() != 4 or k_cache.shape[1] != n_kv or k_cache.shape[3] != d or v_cache.shape != k_cache.shape \
            or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention_mma: caches must be [pages, n_kv, page, d] of q's type")
    for t_, n in ((qmul, n_q), (talk, n_q * n_q), (sink, n_q)):
        if t_ is not None and (t_.dtype != torch.float32 or t_.numel() != n or not t_.is_contiguous()):
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention_mma: qmul, talk and sink must be contiguous float32")
    if gate is not None and (gate.shape != (T, n_q) or gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "talk_attention_mma: gate must be float32 [T, n_q]")
    for t_, what in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (positions, "positions")):
        _int32(t_, what)
    part = talk_scratch(q.device, T * splits * n_q * (d + 2)) if splits > 1 else None
    defines = {"HEAD_DIM": d, "TALK_H": n_q, "TALK_G": n_kv}
    f = _fn("attention_talk_mma", "photon_talk_mma",
            [c_void_p, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_void_p,
             c_void_p], defines=defines)
    gate_stride = gate.stride(0) if gate is not None else 0
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(cu_tokens), _ptr(positions), int(num_seqs), int(max_tokens), n_q, n_kv, d,
             k_cache.shape[2], k_cache.shape[0], int(window or 0), _ptr(qmul), _ptr(talk), _ptr(sink), _ptr(gate), gate_stride,
             int(splits), _ptr(part), _ptr(err), _stream()), "talk_attention_mma")
    if splits > 1:
        m = _fn("attention_talk", "photon_talk_merge",
                [c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_long, c_void_p])
        _check(m(_ptr(part), int(splits), _ptr(out), out.stride(0), _dtype_code(out), T, n_q, d, _ptr(sink), _ptr(gate),
                 gate_stride, _stream()), "talk_merge")


# ----------------------------------------------------------------------------- gated linear attention

def gla_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, low: torch.Tensor,
                  w_a2: torch.Tensor, b_a2: torch.Tensor, norm_w: torch.Tensor, eps: float, tau: float, qscale: float,
                  cu_tokens: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                  num_seqs: int, heads: int, dim: int, vdim: int, err: Optional[torch.Tensor], skip_from: int = 0) -> None:
    """The recurrence of gated linear attention over the tokens of a step, request by request, with the decay
    logits ``w_a2 low + b_a2``, the per-head norm and the output gate.  ``q, k [T, heads * dim]``,
    ``v, g [T, heads * vdim]`` and ``low [T, rank]`` are sections of one fused row (same row stride),
    ``w_a2 [heads * dim, rank]``, ``state [slots, heads, dim, vdim]`` float32, ``out [T, heads * vdim]``.
    ``skip_from`` > 0: requests that bring that many tokens or more are left alone (``gla_chunked`` runs them)."""
    _cuda(q, k, v, g, low, w_a2, b_a2, norm_w, cu_tokens, state_slots, state, out, err)
    T = q.shape[0]
    rank = low.shape[1]
    for name, t, w in (("q", q, heads * dim), ("k", k, heads * dim), ("v", v, heads * vdim), ("g", g, heads * vdim),
                       ("low", low, rank)):
        if t.shape != (T, w) or t.stride(1) != 1 or t.stride(0) != q.stride(0) or t.dtype != q.dtype:
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, f"gla_recurrent: {name} must be [T, {w}] with the row stride of q")
    if w_a2.shape != (heads * dim, rank) or not w_a2.is_contiguous() or w_a2.dtype != q.dtype or b_a2.numel() != heads * dim:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gla_recurrent: w_a2 [heads * dim, rank] of q's dtype, b_a2 [heads * dim]")
    if state.dtype != torch.float32 or state.dim() != 4 or state.shape[1:] != (heads, dim, vdim) or not state.is_contiguous():
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gla_recurrent: state must be contiguous float32 [slots, heads, dim, vdim]")
    if out.shape != (T, heads * vdim) or out.stride(1) != 1 or out.dtype != q.dtype or norm_w.numel() != vdim:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "gla_recurrent: out [T, heads * vdim] of q's dtype, norm weight [vdim]")
    _int32(cu_tokens, "cu_tokens")
    _int32(state_slots, "state_slots")
    f = _fn("gla", "photon_gla_recurrent",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_float, c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(low), q.stride(0), _dtype_code(q), rank, _ptr(w_a2), _ptr(b_a2),
             _dtype_code(b_a2), _ptr(norm_w), _dtype_code(norm_w), float(eps), float(tau), float(qscale), _ptr(cu_tokens),
             _ptr(state_slots), _ptr(state), state.shape[0], _ptr(out), out.stride(0), int(num_seqs), heads, dim, vdim,
             int(skip_from), _ptr(err), _stream()), "gla_recurrent")


GLA_CHUNK = 32              # tokens of a chunk of the chunk-parallel recurrence (measured: 64 -> 521 us, 32 -> 420 us, 16 -> 515 us at 2,048 tokens, 16 heads of 128 x 128)


def gla_chunked_supported(dim: int, vdim: int, rank: int = 64) -> bool:
    """A block shape of the chunk kernel exists (columns x row groups within 512 threads, the groups a power of two),
    and the shared memory of the two chunk kernels fits."""
    for rpt in (8, 16, 32, 64):
        groups = -(-dim // rpt)
        p = 1
        while p < groups:
            p *= 2
        if p <= 32 and vdim * p <= 512 and dim <= 512:
            local = (3 * GLA_CHUNK * groups * (rpt + 4) + GLA_CHUNK * vdim + dim * (rank + 2)) * 4
            out = (dim * vdim + 4 + (GLA_CHUNK + 4) * dim + GLA_CHUNK * vdim) * 4
            return local <= 220 * 1024 and out <= 200 * 1024
    return False


def gla_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, low: torch.Tensor, w_a2: torch.Tensor,
                b_a2: torch.Tensor, norm_w: torch.Tensor, eps: float, tau: float, qscale: float, first: int, count: int,
                slot: int, state: torch.Tensor, out: torch.Tensor, heads: int, dim: int, vdim: int,
                err: Optional[torch.Tensor]) -> None:
    """One long prompt portion (tokens ``first .. first + count - 1`` of the step's rows, state slot ``slot``) with its
    chunks of ``GLA_CHUNK`` tokens side by side: each chunk's own recurrence from zero, a scan over the chunks' end
    states, and the start states' share of the outputs with the norm and the gate.  Same tensors as
    ``gla_recurrent``; the sums differ from its sums in their order only."""
    _cuda(q, k, v, g, low, w_a2, b_a2, norm_w, state, out, err)
    rank = low.shape[1]
    chunks = -(-count // GLA_CHUNK)
    scratch = torch.empty(count * heads * (vdim + dim) + 4 + chunks * heads * dim * vdim, dtype=torch.float32, device=q.device)
    f = _fn("gla", "photon_gla_chunked",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_float, c_float, c_float, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long,
             c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(low), q.stride(0), _dtype_code(q), rank, _ptr(w_a2), _ptr(b_a2),
             _dtype_code(b_a2), _ptr(norm_w), _dtype_code(norm_w), float(eps), float(tau), float(qscale), int(first),
             int(count), GLA_CHUNK, int(slot), _ptr(state), state.shape[0], _ptr(scratch), _ptr(out), out.stride(0), heads,
             dim, vdim, _ptr(err), _stream()), "gla_chunked")
    global _launch_count
    _launch_count += 2


# ----------------------------------------------------------------------------- routed experts

def moe_tile_rows() -> int:
    return int(load_module("moe").photon_moe_tile_rows())


def moe_route(h: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int,
              scoring: str = "softmax_chosen", groups: int = 1, keep_groups: int = 1, route_scale: float = 1.0,
              w_shared_gate: Optional[torch.Tensor] = None):
    """Router logits in 32-bit and the ``top`` experts of every token.  ``scoring`` ``softmax_chosen``: the largest
    logits win and the weights are the softmax over the chosen logits.  ``softmax_all``: scores are the softmax
    over all experts; the experts form ``groups`` equal groups of neighbours, a group's score is its largest
    score and only experts of the ``keep_groups`` best groups can be chosen; the weights are the chosen scores
    over their sum (+ 1e-20) times ``route_scale``.  ``sigmoid``: scores are ``sigmoid(logit)``, a group's score is the
    sum of its two largest scores, and the weights are the chosen scores times ``route_scale`` (not divided by their
    sum).  ``w_shared_gate [1, H]``: also returns ``sigmoid(w . h)``
    per token.  Returns ``(ids int32 [T, top], weights float32 [T, top], counts int32 [E])`` or, with a gate,
    those and ``gate float32 [T]``."""
    _cuda(h, w_router, bias, w_shared_gate)
    if scoring not in ROUTER_SCORING:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, f"moe_route: unknown scoring {scoring!r} ({', '.join(ROUTER_SCORING)})")
    T, H = h.shape
    E = w_router.shape[0]
    if w_router.shape != (E, H) or not w_router.is_contiguous() or h.stride(1) != 1 or h.dtype != w_router.dtype:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_route: h [T, H] and the router [E, H] of one dtype")
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
    counts = torch.empty(E, dtype=torch.int32, device=h.device)
    gate = None
    if w_shared_gate is not None:
        if w_shared_gate.numel() != H or w_shared_gate.dtype != w_router.dtype or not w_shared_gate.is_contiguous():
            raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_route: the shared expert's gate must be [1, H] of the router's dtype")
        gate = torch.empty(T, dtype=torch.float32, device=h.device)
    f = _fn("moe", "photon_moe_route_ex",
            [c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(h), h.stride(0), _dtype_code(h), _ptr(w_router), _ptr(bias),
             _dtype_code(bias) if bias is not None else F32, T, H, E, int(top), _ptr(ids), _ptr(weights), _ptr(counts),
             ROUTER_SCORING[scoring], int(groups), int(keep_groups), float(route_scale), _ptr(w_shared_gate), _ptr(gate),
             _stream()), "moe_route")
    if gate is not None:
        return ids, weights, counts, gate
    return ids, weights, counts


ROUTER_SCORING = {"softmax_chosen": 0, "softmax_all": 1, "sigmoid": 2}


def moe_align(ids: torch.Tensor, counts: torch.Tensor):
    """Sorts the (token, choice) pairs by expert on the device.  Returns ``(offsets [E + 1], sorted [n], place
    [n], tiles [max_tiles, 3], num_tiles [1], max_tiles)``."""
    _cuda(ids, counts)
    n, E = ids.numel(), counts.numel()
    max_tiles = n // moe_tile_rows() + E
    dev = ids.device
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    srt = torch.empty(n, dtype=torch.int32, device=dev)
    place = torch.empty(n, dtype=torch.int32, device=dev)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    f = _fn("moe", "photon_moe_align",
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(ids), _ptr(counts), n, E, _ptr(offsets), _ptr(srt), _ptr(place), _ptr(tiles), _ptr(num_tiles),
             _stream()), "moe_align")
    return offsets, srt, place, tiles, num_tiles, max_tiles


def moe_gemm(a: torch.Tensor, gather: Optional[torch.Tensor], gather_div: int, weight: torch.Tensor, out: torch.Tensor,
             tiles: torch.Tensor, num_tiles: torch.Tensor, max_tiles: int, glu: bool = False,
             activation: Optional[str] = None) -> None:
    """Grouped product over rows sorted by expert: ``weight [E, N, K]``; sorted row ``r`` reads row
    ``gather[r] // gather_div`` of ``a`` (``gather`` None: row ``r``).  ``glu``: ``weight`` holds gate rows
    then up rows and ``out [n, N / 2] = act(gate) * up`` (silu unless named).  Without ``glu`` an ``activation`` is
    applied to every output (None: the plain product)."""
    _cuda(a, gather, weight, out, tiles, num_tiles)
    act = ACTIVATIONS[activation or "silu"] if glu or activation else ACT_NONE
    E, N, K = weight.shape
    if a.shape[1] != K or a.stride(1) != 1 or not weight.is_contiguous() or a.dtype != weight.dtype \
            or out.stride(1) != 1 or out.shape[1] != (N // 2 if glu else N) or out.dtype not in (a.dtype, torch.float32):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_gemm: a [*, K], weight [E, N, K], out [n, N or N / 2]")
    f = _fn("moe", "photon_moe_gemm",
            [c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), a.stride(0), _dtype_code(a), _ptr(gather), int(gather_div), _ptr(weight), _ptr(out), out.stride(0),
             _dtype_code(out), N, K, _ptr(tiles), _ptr(num_tiles), int(max_tiles), int(glu), act,
             _stream()), "moe_gemm")


def moe_combine(y: torch.Tensor, place: Optional[torch.Tensor], weights: torch.Tensor, shared_out: Optional[torch.Tensor],
                out: torch.Tensor, shared_gate: Optional[torch.Tensor] = None) -> None:
    """``out[t] = sum_j weights[t, j] * y[place[t, j]] (+ shared_out[t])``, summed in 32-bit in the order of ``j``;
    ``place`` None: the rows of ``y`` stand in the order of the pairs.  ``shared_gate`` float32 ``[T]``: the shared
    expert's row of token ``t`` is multiplied by ``shared_gate[t]``."""
    _cuda(y, place, weights, shared_out, out, shared_gate)
    if shared_gate is not None and (shared_out is None or shared_gate.dtype != torch.float32 or shared_gate.numel() != weights.shape[0]):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_combine: shared_gate float32 [T] goes with shared_out")
    T, top = weights.shape
    H = y.shape[1]
    if y.stride(1) != 1 or out.shape != (T, H) or not out.is_contiguous() \
            or (shared_out is not None and (shared_out.shape != (T, H) or not shared_out.is_contiguous()
                                            or shared_out.dtype != out.dtype)):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_combine: y [n, H], out and shared_out contiguous [T, H]")
    f = _fn("moe", "photon_moe_combine_ex",
            [c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(y), y.stride(0), _dtype_code(y), _ptr(place), _ptr(weights), top, _ptr(shared_out), _ptr(shared_gate),
             _ptr(out), _dtype_code(out), T, H, _stream()), "moe_combine")


def moe_gather(x: torch.Tensor, srt: torch.Tensor, div: int) -> torch.Tensor:
    """``out[r] = x[srt[r] // div]``: the pairs' input rows in sorted order."""
    _cuda(x, srt)
    n, H = srt.numel(), x.shape[1]
    out = torch.empty((n, H), dtype=x.dtype, device=x.device)
    f = _fn("moe", "photon_moe_gather", [c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _dtype_code(x), _ptr(srt), int(div), _ptr(out), n, H, _stream()), "moe_gather")
    return out


def moe_gemv_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K = weight.shape[2]
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.is_contiguous() and K * 2 <= 96 * 1024)


def moe_gemv(x: torch.Tensor, x_div: int, ids: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, glu: bool = False,
             activation: Optional[str] = None) -> None:
    """A decode step's few (token, choice) pairs: ``out[p] = weight[ids[p]] @ x[p // x_div]``, one matrix-vector
    product per pair in the order of the pairs, the expert's rows streamed once.  bfloat16 in, bfloat16 or float32 out."""
    _cuda(x, ids, weight, out)
    act = ACTIVATIONS[activation or "silu"] if glu or activation else ACT_NONE
    E, N, K = weight.shape
    n = ids.numel()
    if not moe_gemv_supported(x, weight) or x.shape[1] != K:
        raise PhotonError(ErrorCode.UNSUPPORTED_SIZE, "moe_gemv: bfloat16, K a multiple of 8, aligned rows")
    if out.shape != (n, N // 2 if glu else N) or out.stride(1) != 1:
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "moe_gemv: out [pairs, N or N / 2]")
    f = _fn("moe", "photon_moe_gemv",
            [c_void_p, c_long, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), int(x_div), _ptr(ids), n, _ptr(weight), _ptr(out), out.stride(0), _dtype_code(out), N, K,
             int(glu), act, _stream()), "moe_gemv")


# ----------------------------------------------------------------------------- sampling

def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], u: Optional[torch.Tensor],
           out: torch.Tensor) -> None:
    """Row-wise: first-maximum argmax where ``temperature <= 0`` (or None), else the first
    index whose running sum of ``softmax(logits / temperature)`` reaches ``u``."""
    _cuda(logits, temperature, u, out)
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise PhotonError(ErrorCode.INVALID_ARGUMENT, "sample: logits must be float32 with unit inner stride")
    _int32(out, "out")
    if temperature is not None and (temperature.dtype != torch.float32 or temperature.numel() != rows
                                    or u is None or u.dtype != torch.float32 or u.numel() != rows):
        raise PhotonError(ErrorCode.SHAPE_MISMATCH, "sample: temperature and u must be float32 [rows]")
    scratch = None
    if V > 16384:
        # long rows are cut into 32 spans that separate blocks reduce; their results meet here
        scratch = torch.empty(rows * 32 * 4, dtype=torch.float32, device=logits.device)
    f = _fn("sampling", "photon_sample", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), _ptr(temperature), _ptr(u), _ptr(out), rows, V, _ptr(scratch), _stream()),
           "sample")
    if scratch is not None:
        global _launch_count
        _launch_count += 1
