"""Grouped-query attention whose heads' scores are mixed before the softmax ("talking heads"), over the paged cache.

``q = W_q h (+ b_q)``, ``k = W_k h (+ b_k)``; optionally the first ``rot_dims`` numbers of every head are rotated by
the token's position (number ``j`` paired with ``j + rot_dims / 2``, angle ``p * rot_base^(-2j / rot_dims)``).  Per
head ``raw_g = (q_g . k) * scale * temperature[g]``; then every head's score is a weighted sum of ALL heads' scores
for the same pair of tokens, ``s_h = sum_g talk[h, g] raw_g``.  A token at position ``i`` sees key ``j <= i`` when
``i - j < window`` (no window: every earlier key).  The softmax may have a learned sink per head: ``exp(sink[h])``
joins the denominator, with no key and no value.  The heads' outputs may be multiplied by ``sigmoid(W_g h)``, one
number per head, before the output projection.  With ``values_are_keys`` there is no value projection: a value is
its key as projected, before the rotation.

Kernels of a step: ONE product for q, k (v) and the gate with 32-bit rows; one pass that adds the biases, rotates and
writes queries, keys and values (``attention_talk.cu``); attention over all heads of a token at once; the output
product.  Prompt portions, decoded tokens and mixed batches take the same path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedCacheSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b", "talk": "talk",
                 "temperature": "temp", "sink": "sink"}


class TalkingAttention(Mixer):
    kernel_modules = ("attention_talk", "elementwise")

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                 window: Optional[int] = None, rot_dims: int = 0, rot_base: float = 10000.0, bias: bool = False,
                 temperature: bool = False, talk: bool = True, sink: bool = False, output_gate: bool = False,
                 values_are_keys: bool = False, names: Optional[Dict[str, str]] = None):
        if n_kv_heads <= 0 or n_q_heads % n_kv_heads:
            raise ValueError("the number of query heads must be a multiple of the number of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
            raise ValueError("rot_dims must be even and at most head_dim")
        self.hidden_size, self.n_q, self.n_kv, self.head_dim = hidden_size, n_q_heads, n_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = int(window) if window else None
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.bias, self.temperature, self.talk, self.sink = bool(bias), bool(temperature), bool(talk), bool(sink)
        self.output_gate, self.values_are_keys = bool(output_gate), bool(values_are_keys)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in: Optional[torch.Tensor] = None        # [W_q; W_k; (W_v); (W_g)]
        self.w_o: Optional[torch.Tensor] = None
        self.q_bias = self.k_bias = self.qmul = self.talk_w = self.sink_w = self.inv_freq = None
        # bfloat16 steps run on the tensor cores when the sizes allow it, else (and in 32-bit) the general kernel
        self._tensor_cores = ops.talk_mma_supported(n_q_heads, n_kv_heads, head_dim)

    @property
    def _sections(self):
        q, k = self.n_q * self.head_dim, self.n_kv * self.head_dim
        return q, k, (0 if self.values_are_keys else k), (self.n_q if self.output_gate else 0)

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_tc", "gemm_tc2"])
            if self._tensor_cores:
                mods.append(("attention_talk_mma", {"HEAD_DIM": self.head_dim, "TALK_H": self.n_q, "TALK_G": self.n_kv}))
        return mods

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden_size
        q, k, v, g = self._sections
        specs = [TensorSpec(n["q"], (q, H)), TensorSpec(n["k"], (k, H)), TensorSpec(n["o"], (H, q))]
        if v:
            specs.append(TensorSpec(n["v"], (v, H)))
        if g:
            specs.append(TensorSpec(n["g"], (g, H)))
        if self.bias:
            specs += [TensorSpec(n["q_bias"], (q,), role="vector", init="normal"),
                      TensorSpec(n["k_bias"], (k,), role="vector", init="normal")]
        if self.talk:
            specs.append(TensorSpec(n["talk"], (self.n_q, self.n_q), role="vector", init="normal"))
        if self.temperature:
            specs.append(TensorSpec(n["temperature"], (self.n_q,), role="vector", init="norm"))
        if self.sink:
            specs.append(TensorSpec(n["sink"], (self.n_q,), role="vector", init="normal"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        f32 = lambda name: tensors[n[name]].to(torch.float32).contiguous()
        parts = [tensors[n["q"]], tensors[n["k"]]]
        if not self.values_are_keys:
            parts.append(tensors[n["v"]])
        if self.output_gate:
            parts.append(tensors[n["g"]])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        dev = self.w_in.device
        if self.bias:
            self.q_bias, self.k_bias = f32("q_bias"), f32("k_bias")
        # scale and the heads' temperatures are one factor per head, applied to the query in 32-bit
        self.qmul = torch.full((self.n_q,), self.scale, dtype=torch.float32, device=dev)
        if self.temperature:
            self.qmul = (self.qmul * f32("temperature")).contiguous()
        self.talk_w = f32("talk") if self.talk else None
        self.sink_w = f32("sink") if self.sink else None
        if self.rot_dims:
            j = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * j / self.rot_dims).to(dev)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(self.n_kv, self.head_dim, self.window)

    # -- one step
    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        nq, nk, nv, ng = self._sections
        rows = project(h, self.w_in, out_dtype=torch.float32)           # biases and rotation work on unrounded sums
        q = torch.empty((T, nq), dtype=h.dtype, device=h.device)
        group = ctx.groups[cache.group]
        store = not cache.shared and cache.k is not None
        ops.talk_prep(rows[:, :nq], rows[:, nq:nq + nk], rows[:, nq + nk:nq + nk + nv] if nv else None, self.q_bias,
                      self.k_bias, q, ctx.positions, self.inv_freq, self.rot_dims, group.slot_mapping if store else None,
                      cache.k if store else None, cache.v if store else None, self.n_q, self.n_kv, self.head_dim,
                      ctx.error_flag)
        attn = torch.empty((T, nq), dtype=h.dtype, device=h.device)
        gate = rows[:, nq + nk + nv:] if self.output_gate else None
        self.attend(q, attn, ctx, cache, gate)
        return project(attn, self.w_o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, cache: LayerCache,
               gate: Optional[torch.Tensor]) -> None:
        group = ctx.groups[cache.group]
        splits = 1
        if q.dtype == torch.bfloat16 and ctx.max_query_len == 1:
            # decode steps: few tokens, so a token's key tiles are shared out over blocks (bfloat16 only; the 32-bit
            # run keeps one order of sums whatever the step)
            keys = ctx.max_context_len if self.window is None else min(self.window + 1, ctx.max_context_len)
            splits = max(1, min(keys // 128, (2 * ops.sm_count(q.device)) // max(1, ctx.num_tokens), 64))
        if q.dtype == torch.bfloat16 and self._tensor_cores:
            ops.talk_attention_mma(q, out, cache.k, cache.v, group.block_table, ctx.cu_tokens, ctx.positions, ctx.num_seqs,
                                   ctx.max_query_len, self.n_q, self.n_kv, self.head_dim, self.window, self.qmul, self.talk_w,
                                   self.sink_w, gate, ctx.error_flag, splits=splits)
            return
        ops.talk_attention(q, out, cache.k, cache.v, group.block_table, ctx.token_seq, ctx.positions, self.n_q, self.n_kv,
                           self.head_dim, self.window, self.qmul, self.talk_w, self.sink_w, gate, ctx.error_flag, splits=splits)


register_mixer("talking_attention", TalkingAttention)
