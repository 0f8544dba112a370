"""Gated delta rule: a recurrent mixer with a matrix-valued state per head and short convolutions in front of it.

``q = W_q h``, ``k = W_k h`` (``qk_heads x dim``), ``v = W_v h`` (``heads x vdim``); value head ``h`` uses query/key
head ``h // (heads / qk_heads)``.  Each channel of q, k and v passes a causal convolution over the last ``taps``
tokens (zeros before the start of the sequence) and silu; q and k heads are then made unit vectors
(``x / sqrt(sum(x^2) + 1e-6)``), q also times ``dim^(-1/2)``.  Per head and token ``beta = sigmoid(W_b h)`` and a decay
``g = exp(-exp(A_log) * softplus(W_a h + dt_bias))``, and

    S <- g S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q,

so the read-out sees the token's own write.  ``o`` is RMS-normed per head over vdim with a weight that the heads
share, multiplied by ``silu(W_g h)`` and projected by ``W_o``.  The state (``S`` and the last ``taps - 1`` projected
rows) starts at zero, is 32-bit, and lives in the request's state slot between steps; everything after the
projections is 32-bit.

One fused product gives ``[q | k | v | W_g h | W_a h | W_b h]`` as 32-bit rows; then the convolution kernel, the
recurrence over the tokens of the step (one block per request and head), and norm and gate.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a": "a", "b": "b", "A_log": "A_log", "dt_bias": "dt_bias",
                 "norm": "norm", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}


class GatedDeltaRule(Mixer):
    kernel_modules = ("delta",)
    state_skips_negative_slots = True

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, taps: int, eps: float,
                 qk_heads: Optional[int] = None, names: Optional[Dict[str, str]] = None):
        qk_heads = heads if qk_heads is None else qk_heads
        if qk_heads <= 0 or heads % qk_heads:
            raise ValueError("the number of value heads must be a multiple of the number of query/key heads")
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.hidden_size, self.heads, self.qk_heads, self.dim, self.vdim = hidden_size, heads, qk_heads, dim, vdim
        self.taps, self.eps = int(taps), float(eps)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in = self.w_o = self.taps_w = self.a_log = self.dt_bias = self.norm = None

    @property
    def channels(self) -> int:
        """Channels that pass the convolution: q, k and v side by side."""
        return 2 * self.qk_heads * self.dim + self.heads * self.vdim

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_tc", "gemm_tc2"])
        return mods

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden_size
        qk, nv = self.qk_heads * self.dim, self.heads * self.vdim
        return [TensorSpec(n["q"], (qk, H)), TensorSpec(n["k"], (qk, H)), TensorSpec(n["v"], (nv, H)),
                TensorSpec(n["g"], (nv, H)), TensorSpec(n["o"], (H, nv)),
                TensorSpec(n["a"], (self.heads, H)), TensorSpec(n["b"], (self.heads, H)),
                TensorSpec(n["q_conv"], (qk, self.taps), role="vector", init="normal"),
                TensorSpec(n["k_conv"], (qk, self.taps), role="vector", init="normal"),
                TensorSpec(n["v_conv"], (nv, self.taps), role="vector", init="normal"),
                TensorSpec(n["A_log"], (self.heads,), role="vector", init="normal"),
                TensorSpec(n["dt_bias"], (self.heads,), role="vector", init="normal"),
                TensorSpec(n["norm"], (self.vdim,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        f32 = lambda name: tensors[n[name]].to(torch.float32).contiguous()
        self.w_in = torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g", "a", "b")], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.taps_w = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = f32("A_log"), f32("dt_bias"), f32("norm")

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.heads * self.dim * self.vdim + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        C, nv, H = self.channels, self.heads * self.vdim, self.heads
        rows = project(h, self.w_in, out_dtype=torch.float32)       # [T, C + nv + 2 H]: what enters the recurrence stays 32-bit
        y = torch.empty((T, C), dtype=torch.float32, device=h.device)
        state = cache.state
        ops.delta_conv(rows[:, :C], self.taps_w, ctx.token_seq, ctx.cu_tokens, ctx.state_slots, state,
                       self.heads * self.dim * self.vdim, y, ctx.num_seqs, self.qk_heads, H, self.dim, self.vdim, ctx.error_flag)
        o = torch.empty((T, nv), dtype=torch.float32, device=h.device)
        ops.delta_recurrent(y, rows[:, C + nv:C + nv + 2 * H], self.a_log, self.dt_bias, ctx.cu_tokens, ctx.state_slots, state,
                            o, ctx.num_seqs, self.qk_heads, H, self.dim, self.vdim, ctx.error_flag)
        out = torch.empty((T, nv), dtype=h.dtype, device=h.device)
        ops.delta_out(o, rows[:, C:C + nv], self.norm, self.eps, out, H, self.vdim)
        return project(out, self.w_o)


register_mixer("delta_rule", GatedDeltaRule)
