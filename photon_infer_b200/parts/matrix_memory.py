"""Matrix memory with exponential gates (the mLSTM cell): a recurrent mixer whose state is one matrix per head, a
vector that follows the keys, and a running maximum that keeps the exponentials in range.

``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim).  Per head a log input gate
``i = cap tanh((W_i h + b_i) / cap)`` and a log forget gate ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))``.  With
``S``, ``n`` and the running maximum ``m`` all starting at zero,

    m_t = max(f + m_(t-1), i);   S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;   n_t likewise with k alone;
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6).

Each head's ``o`` is divided by its root mean square; the heads are concatenated, multiplied by the weight ``norm``
(all heads' size) and by ``sigmoid(W_g h)``, and projected by ``W_o``.  The state (``S``, ``n``, ``m``) is 32-bit and lives in
the request's state slot between steps; everything after the input product is 32-bit.

Kernels of a step: ONE product ``[q | k | v | g | i | f]`` with 32-bit rows; the recurrence over the tokens of the step
(``linrec.cu``; the vector ``n`` rides along as one more column of ``S``); norm and gate in one pass (``row_norms.cu``);
the output product.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "i_bias": "i.b", "f": "f",
                 "f_bias": "f.b"}


class MatrixMemoryMixer(Mixer):
    kernel_modules = ("linrec", "row_norms")
    state_skips_negative_slots = True

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 names: Optional[Dict[str, str]] = None):
        if not gate_cap > 0:
            raise ValueError("the gates' bound must be positive")
        self.hidden_size, self.heads, self.dim, self.vdim = hidden_size, heads, dim, vdim
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in = self.w_o = self.norm = self.i_bias = self.f_bias = None

    def required_kernels(self, dtype):
        return list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden_size
        nd, nv = self.heads * self.dim, self.heads * self.vdim
        vec = lambda name, size, init="normal": TensorSpec(n[name], (size,), role="vector", init=init)
        return [TensorSpec(n["q"], (nd, H)), TensorSpec(n["k"], (nd, H)), TensorSpec(n["v"], (nv, H)), TensorSpec(n["g"], (nv, H)),
                TensorSpec(n["o"], (H, nv)), vec("norm", nv, "norm"), TensorSpec(n["i"], (self.heads, H)), vec("i_bias", self.heads),
                TensorSpec(n["f"], (self.heads, H)), vec("f_bias", self.heads)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        f32 = lambda name: tensors[n[name]].to(torch.float32).contiguous()
        self.w_in = torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.norm, self.i_bias, self.f_bias = f32("norm"), f32("i_bias"), f32("f_bias")

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.heads * self.dim * self.vdim + self.heads * self.dim + self.heads,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        nd, nv, H = self.heads * self.dim, self.heads * self.vdim, self.heads
        rows = project(h, self.w_in, out_dtype=torch.float32)       # [q | k | v | g | i | f]
        o = torch.empty((T, nv), dtype=torch.float32, device=h.device)
        g0 = 2 * nd + nv
        ops.linrec("matrix_memory", rows[:, :nd], rows[:, nd:2 * nd], rows[:, 2 * nd:g0], rows[:, g0 + nv:g0 + nv + H],
                   rows[:, g0 + nv + H:], self.i_bias, self.f_bias, None, self.gate_cap, self.dim ** -0.5, ctx.cu_tokens,
                   ctx.state_slots, cache.state, o, ctx.num_seqs, H, H, self.dim, self.vdim, ctx.error_flag)
        out = torch.empty((T, nv), dtype=h.dtype, device=h.device)
        ops.group_rmsnorm(o, self.norm, self.eps, H, out=out, gate=rows[:, g0:g0 + nv], gate_mode="sigmoid_after")
        return project(out, self.w_o, out_dtype=torch.float32)


register_mixer("matrix_memory", MatrixMemoryMixer)
