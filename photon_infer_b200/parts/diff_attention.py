"""Differential attention over the paged cache: every query head has two score maps over the same values.

``q = W_q h + b_q`` has ``heads * 2 * dim`` rows and ``k = W_k h + b_k`` has ``kv_heads * 2 * dim`` rows, laid out head
by head as (map 1, map 2); ``v = W_v h + b_v`` has ``kv_heads * value_dim``.  Query head ``h`` uses key/value head
``h // (heads / kv_heads)``.  Every (head, map) of q and k is divided by its root mean square (``eps`` inside the root) and
multiplied by a weight ``[dim]`` that all heads and maps share; then its first ``rot_dims`` numbers are rotated by the
token's position (number ``j`` paired with ``j + rot_dims / 2``, angle ``p * rot_base^(-2j / rot_dims)``).  Each map is
an attention of its own, ``softmax((q_m . k_m) * scale)`` over the keys ``0 <= i - j < window`` (no window: every
earlier key); with the maps' outputs ``a_1, a_2`` (both over the same values) and

    lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff        (one number per layer),

a head's output is ``o = a_1 - lambda a_2``, divided by its root mean square over ``value_dim`` (no weight), times
``1 - diff``.  The heads are concatenated and projected by ``W_o`` (with a bias).

``own_kv`` False: the layer has no key and value tensors; it reads the cache pages of an earlier layer (the run list's
``kv_from``) with its own queries, window and everything else.  ``cache_window``: how many keys the cache must keep for
this layer AND the layers that read its pages (``"own"``: this layer's window; None: everything).

Kernels of a step: ONE product for q, k, v with 32-bit rows; one pass that adds the biases, norms and rotates in
32-bit (angles in 64-bit) and writes queries, keys (both maps of a head side by side) and values
(``attention_diff.cu``); attention; the output product.  Prompt portions, decoded tokens and mixed batches take the
same path.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedCacheSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                 "q_norm": "q.norm", "k_norm": "k.norm", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}


class DifferentialAttention(Mixer):
    kernel_modules = ("attention_diff", "elementwise")

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, value_dim: int, eps: float,
                 scale: float, diff: float, rot_dims: int = 0, rot_base: float = 10000.0, window: Optional[int] = None,
                 cache_window="own", own_kv: bool = True, bias: bool = True, names: Optional[Dict[str, str]] = None):
        if n_kv_heads <= 0 or n_q_heads % n_kv_heads:
            raise ValueError("the number of query heads must be a multiple of the number of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
            raise ValueError("rot_dims must be even and at most head_dim")
        self.hidden_size, self.n_q, self.n_kv, self.head_dim, self.value_dim = hidden_size, n_q_heads, n_kv_heads, head_dim, value_dim
        self.eps, self.scale, self.diff = float(eps), float(scale), float(diff)
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.window = int(window) if window else None
        self.cache_window = self.window if cache_window == "own" else (int(cache_window) if cache_window else None)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError("the cache must keep at least the keys that this layer's window sees")
        self.own_kv, self.bias = bool(own_kv), bool(bias)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.inv_freq = None
        self.q_bias = self.k_bias = self.v_bias = self.o_bias = None
        self.lam: Optional[float] = None

    @property
    def _sections(self):
        q = self.n_q * 2 * self.head_dim
        return (q, self.n_kv * 2 * self.head_dim, self.n_kv * self.value_dim) if self.own_kv else (q, 0, 0)

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])
        if self._mma_ok(dtype):
            mods.append(("attention_diff_mma", {"DIFF_D": self.head_dim, "DIFF_DV": self.value_dim}))
        return mods

    def _mma_ok(self, dtype) -> bool:
        return USE_DIFF_MMA and ops.diff_mma_supported(dtype, self.n_q, self.n_kv, self.head_dim, self.value_dim)

    def tensor_specs(self) -> List[TensorSpec]:
        n, H, d = self.names, self.hidden_size, self.head_dim
        nq, nk, nv = self._sections
        vec = lambda name, size, init="normal": TensorSpec(n[name], (size,), role="vector", init=init)
        specs = [TensorSpec(n["q"], (nq, H)), TensorSpec(n["o"], (H, self.n_q * self.value_dim)), vec("q_norm", d, "norm")]
        specs += [vec(x, d) for x in ("lq1", "lk1", "lq2", "lk2")]
        if self.bias:
            specs += [vec("q_bias", nq), vec("o_bias", H)]
        if self.own_kv:
            specs += [TensorSpec(n["k"], (nk, H)), TensorSpec(n["v"], (nv, H)), vec("k_norm", d, "norm")]
            if self.bias:
                specs += [vec("k_bias", nk), vec("v_bias", nv)]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        mats = [tensors[n["q"]]] + ([tensors[n["k"]], tensors[n["v"]]] if self.own_kv else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        f32 = lambda name: tensors[n[name]].to(torch.float32).contiguous()
        self.q_norm = f32("q_norm")
        self.k_norm = f32("k_norm") if self.own_kv else None
        if self.bias:
            self.q_bias, self.o_bias = f32("q_bias"), f32("o_bias")
            if self.own_kv:
                self.k_bias, self.v_bias = f32("k_bias"), f32("v_bias")
        # the weight of the second map, one number per layer, in 32-bit
        lam = torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum()) + \
            torch.tensor(self.diff, dtype=torch.float32, device=self.w_in.device)
        self.lam = float(lam.item())
        if self.rot_dims:
            j = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * j / self.rot_dims).to(self.w_in.device)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        # both maps of a head's key lie side by side in one cached row
        return PagedCacheSpec(self.n_kv, 2 * self.head_dim, self.cache_window, value_dim=self.value_dim)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        out, bias = self.forward_deferred_bias(h, ctx, cache)
        if bias is not None:
            ops.scale_bias_rows(out, 1.0, bias)
        return out

    def forward_deferred_bias(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache):
        T = h.shape[0]
        nq, nk, nv = self._sections
        rows = project(h, self.w_in, out_dtype=torch.float32)       # unrounded sums go into bias, norm and rotation
        q = torch.empty((T, nq), dtype=h.dtype, device=h.device)
        group = ctx.groups[cache.group]
        store = self.own_kv and not cache.shared and cache.k is not None
        ops.diff_prep(rows[:, :nq], rows[:, nq:nq + nk] if store else None, rows[:, nq + nk:] if store else None, q,
                      self.q_bias, self.k_bias, self.v_bias, self.q_norm, self.k_norm, self.eps, ctx.positions, self.inv_freq,
                      self.rot_dims, group.slot_mapping if store else None, cache.k if store else None,
                      cache.v if store else None, self.n_q, self.n_kv, self.head_dim, self.value_dim, ctx.error_flag)
        attn = torch.empty((T, self.n_q * self.value_dim), dtype=h.dtype, device=h.device)
        self.attend(q, attn, ctx, cache)
        return project(attn, self.w_o, out_dtype=torch.float32), self.o_bias

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        """bfloat16 with sizes that are multiples of 16: the tensor-core kernel, for prompt portions and decoded tokens
        alike.  float32 and other sizes: the general kernel, whose sums depend on a token's position alone."""
        group = ctx.groups[cache.group]
        if self._mma_ok(q.dtype) and q.stride(0) % 8 == 0 and ctx.host_query_lens:
            splits = 1
            if ctx.max_query_len == 1:
                # a decode step: a block per (request, key/value head) leaves most SMs empty, so the keys are shared out
                keys = ctx.max_context_len if self.window is None else min(self.window + 1, ctx.max_context_len)
                blocks = max(1, ctx.num_seqs * self.n_kv)
                splits = max(1, min(-(-keys // 128), ops.sm_count(q.device) // blocks, 16))
            ops.diff_attention_mma(q, out, cache.k, cache.v, group.block_table, ctx.cu_tokens, ctx.positions, ctx.host_query_lens,
                                   self.n_q, self.n_kv, self.head_dim, self.value_dim, self.window, self.scale, self.lam,
                                   1.0 - self.diff, self.eps, ctx.error_flag, splits=splits)
            return
        ops.diff_attention(q, out, cache.k, cache.v, group.block_table, ctx.token_seq, ctx.positions, self.n_q, self.n_kv,
                           self.head_dim, self.value_dim, self.window, self.scale, self.lam, 1.0 - self.diff, self.eps,
                           ctx.error_flag)


#: The tensor-core kernel for bfloat16 (``PHOTON_DIFF_MMA=0``: the general kernel everywhere).
USE_DIFF_MMA = os.environ.get("PHOTON_DIFF_MMA", "1") != "0"

register_mixer("diff_attention", DifferentialAttention)
