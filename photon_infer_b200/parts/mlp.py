"""Dense gated feed-forward: ``down(act(gate(h)) * up(h))``; with ``act`` silu it is SwiGLU
(src/arch/transformer_block.cpp:282-291; include/photon/ops/kernels/swiglu_kernel.hpp:
67-76), with the tanh form of gelu it is GeGLU, with relu a ReLU-gated unit.  Gate and up are one fused matrix on the
device, so ``h`` is read once.  The tensor names are parameters."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, TensorSpec
from .linear import project
from .registry import register_feed_forward


class SwiGLUFeedForward(FeedForward):
    kernel_modules = ("elementwise",)

    def required_kernels(self, dtype):
        if dtype != torch.bfloat16:
            return ["elementwise"]
        return ["elementwise", "gemm_skinny", "gemm_tc", "gemm_tc2"] + (["gemm_skinny_fused"] if self.fuse_norm else [])

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (one of {sorted(ops.ACTIVATIONS)})")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation
        self.names = tuple(names)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        g, u, d = self.names
        return [TensorSpec(g, (I, H)), TensorSpec(u, (I, H)), TensorSpec(d, (H, I))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, d = self.names
        self.w_gate_up = torch.cat([tensors[g], tensors[u]], dim=0).contiguous()
        self.w_down = tensors[d].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    #: Taking the norm into the gate/up kernel is implemented but off: at the Llama 3.2 1B shape it measured
    #: 18.9 us against 15.4 us for norm kernel + product, because every one of the 512 blocks re-reads the
    #: 8 x 2048 residual rows (the product itself is bound by streaming its 67 MB of weights).
    fuse_norm = False

    def fuses_norm(self, norm, residual, ctx) -> bool:
        from .norm import RMSNorm
        return (self.fuse_norm and self.activation == "silu" and isinstance(norm, RMSNorm) and ctx is not None and ctx.dtype == torch.bfloat16
                and ops.skinny_fused_supported(residual, self.w_gate_up))

    def forward_with_norm(self, residual, delta, norm, ctx):
        """Residual sum, RMSNorm, gate/up products and SwiGLU in one kernel; then the down product."""
        act, residual = ops.skinny_fused(residual, delta, norm.weight, norm.eps, self.w_gate_up, "swiglu",
                                         err=ctx.error_flag)
        return project(act, self.w_down), residual

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ops.linear_swiglu(h, self.w_gate_up, self.activation)
        return project(act, self.w_down)


class PolyNormFeedForward(FeedForward):
    """``W_down act(W_up h)`` with the PolyNorm activation ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e``: powers element by
    element, ``N`` divides a token's vector of ff values by its root mean square (``eps`` inside the root), and the four
    numbers ``(a, b, c, e)`` are a tensor of the layer.  The up product keeps 32-bit rows, which the activation reads
    (its three norms are 32-bit) and rounds once."""
    kernel_modules = ("row_norms",)

    def required_kernels(self, dtype):
        return list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, names=("up", "down", "act")):
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, float(eps)
        self.names = tuple(names)
        self.w_up = self.w_down = self.coef = None

    def tensor_specs(self) -> List[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        u, d, a = self.names
        return [TensorSpec(u, (I, H)), TensorSpec(d, (H, I)), TensorSpec(a, (4,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        u, d, a = self.names
        self.w_up, self.w_down = tensors[u].contiguous(), tensors[d].contiguous()
        self.coef = tensors[a].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        z = project(h, self.w_up, out_dtype=torch.float32)
        act = torch.empty(z.shape, dtype=h.dtype, device=h.device)
        ops.polynorm(z, self.coef, self.eps, act)
        return project(act, self.w_down, out_dtype=torch.float32)


register_feed_forward("swiglu", SwiGLUFeedForward)
register_feed_forward("polynorm", PolyNormFeedForward)
register_feed_forward("gated", SwiGLUFeedForward)
