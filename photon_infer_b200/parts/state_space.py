"""State-space mixer with a scalar decay per head (the state-space duality form): a recurrent mixer whose state is
one matrix per head, with a short causal convolution in front of it.

``W_in h`` is laid out as ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]`` with
``inner = heads * vdim``.  x, B and C together pass a causal convolution per channel over the last ``taps`` tokens
(with a bias; zeros before the start of the sequence) and silu.  ``dt = softplus(dt + dt_bias)``; per head (head ``h``
uses group ``h // (heads / groups)``)

    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T        (S is state x vdim),      y_t = S_t^T C_t + D_h x_t.

``y`` (heads side by side) is multiplied by ``silu(z)``, then RMS-normed in ``norm_groups`` equal parts (each part by its
own root mean square), times the weight ``norm``, then projected by ``W_o``.  The state (``S`` in 32-bit and the last
``taps - 1`` rows that entered the convolution) starts at zero and lives in the request's state slot between steps;
everything after the input product is 32-bit.

Kernels of a step: the input product with 32-bit rows; the convolution (``linrec.cu``); the recurrence over the tokens
of the step; gate and norm in one pass (``row_norms.cu``); the output product.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
                 "norm": "norm", "o": "o"}


class StateSpaceMixer(Mixer):
    kernel_modules = ("linrec", "row_norms")
    state_skips_negative_slots = True

    def __init__(self, hidden_size: int, heads: int, vdim: int, state: int, taps: int, eps: float, groups: int = 1,
                 norm_groups: int = 1, names: Optional[Dict[str, str]] = None):
        if groups <= 0 or heads % groups:
            raise ValueError("the number of heads must be a multiple of the number of groups")
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        if norm_groups <= 0 or (heads * vdim) % norm_groups:
            raise ValueError("the heads' outputs must split into equal parts for the norm")
        self.hidden_size, self.heads, self.vdim, self.state, self.groups = hidden_size, heads, vdim, state, groups
        self.taps, self.eps, self.norm_groups = int(taps), float(eps), int(norm_groups)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in = self.w_o = self.taps_w = self.conv_bias = self.dt_bias = self.a_log = self.d_skip = self.norm = None

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:
        """Channels that pass the convolution: x, B and C side by side."""
        return self.inner + 2 * self.groups * self.state

    def required_kernels(self, dtype):
        return list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])

    def tensor_specs(self) -> List[TensorSpec]:
        n, H, C = self.names, self.hidden_size, self.channels
        vec = lambda name, size, init="normal": TensorSpec(n[name], (size,), role="vector", init=init)
        return [TensorSpec(n["in"], (self.inner + C + self.heads, H)), TensorSpec(n["o"], (H, self.inner)),
                TensorSpec(n["conv"], (C, self.taps), role="vector", init="normal"), vec("conv_bias", C),
                vec("dt_bias", self.heads), vec("A_log", self.heads), vec("D", self.heads), vec("norm", self.inner, "norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        f32 = lambda name: tensors[n[name]].to(torch.float32).contiguous()
        self.w_in, self.w_o = tensors[n["in"]].contiguous(), tensors[n["o"]].contiguous()
        self.taps_w, self.conv_bias = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.d_skip, self.norm = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.heads * self.state * self.vdim + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        inner, C, GN = self.inner, self.channels, self.groups * self.state
        rows = project(h, self.w_in, out_dtype=torch.float32)       # [z | x B C | dt]: what enters the recurrence stays 32-bit
        y = torch.empty((T, C), dtype=torch.float32, device=h.device)
        ops.conv_silu(rows[:, inner:inner + C], self.taps_w, self.conv_bias, ctx.token_seq, ctx.cu_tokens, ctx.state_slots,
                      cache.state, self.heads * self.state * self.vdim, y, ctx.num_seqs, ctx.error_flag)
        o = torch.empty((T, inner), dtype=torch.float32, device=h.device)
        ops.linrec("state_space", y[:, inner + GN:], y[:, inner:inner + GN], y[:, :inner], rows[:, inner + C:], None,
                   self.a_log, self.dt_bias, self.d_skip, 0.0, 1.0, ctx.cu_tokens, ctx.state_slots, cache.state, o,
                   ctx.num_seqs, self.heads, self.groups, self.state, self.vdim, ctx.error_flag)
        out = torch.empty((T, inner), dtype=h.dtype, device=h.device)
        ops.group_rmsnorm(o, self.norm, self.eps, self.norm_groups, out=out, gate=rows[:, :inner], gate_mode="silu_before")
        return project(out, self.w_o, out_dtype=torch.float32)


register_mixer("state_space", StateSpaceMixer)
