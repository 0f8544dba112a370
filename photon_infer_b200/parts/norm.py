"""Norms of the residual stream.  RMSNorm: ``y = w * (x / sqrt(mean(x^2) + eps))`` in 32-bit
(include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86), fused with the residual sum
that precedes it (the reference runs a separate add kernel,
src/arch/transformer_block.cpp:270,295)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import ChannelScalePart, Norm, Normed, TensorSpec, delta_pair, delta_terms
from .registry import register_norm, register_scale


class RMSNorm(Norm):
    kernel_modules = ("elementwise",)

    def __init__(self, size: int, eps: float, weight_name: str = "weight", scalar: bool = False):
        self.size = size
        self.eps = float(eps)
        self.weight_name = weight_name
        self.scalar = bool(scalar)              # the weight is ONE number for all coordinates (a tensor without axes)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, () if self.scalar else (self.size,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        # one number: the kernel reads a weight per coordinate, so the number is repeated (32-bit, exact)
        self.weight = w.to(torch.float32).reshape(1).expand(self.size).contiguous() if self.scalar else w

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(None, x, out_dtype)

    def add_forward(self, delta, residual, out_dtype):
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        d1, d2, sc = delta_terms(delta)
        ops.add_rmsnorm(d1, residual, self.weight, self.eps, out, delta2=d2, delta_scale=sc)
        return out

    def add_forward_rows(self, delta, residual, rows, out_dtype):
        out = torch.empty((rows.numel(), residual.shape[1]), dtype=out_dtype, device=residual.device)
        d1, d2, sc = delta_terms(delta)
        ops.add_rmsnorm(d1, residual, self.weight, self.eps, out, rows=rows, delta2=d2, delta_scale=sc)
        return out


class LayerNorm(Norm):
    """``y = (x - mean(x)) / sqrt(var(x) + eps) * w + b`` in 32-bit, the variance being the mean of the squared
    deviations; fused with the residual sum before it like ``RMSNorm``.  ``bias_name`` None: no bias."""
    kernel_modules = ("elementwise",)

    def __init__(self, size: int, eps: float, weight_name: str = "weight", bias_name: Optional[str] = "bias"):
        self.size = size
        self.eps = float(eps)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.weight_name, (self.size,), role="vector", init="norm")]
        if self.bias_name is not None:
            specs.append(TensorSpec(self.bias_name, (self.size,), role="vector", init="normal"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]
        self.bias = tensors[self.bias_name] if self.bias_name is not None else None

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.bias) if t is not None)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(None, x, out_dtype)

    def add_forward(self, delta, residual, out_dtype):
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        d1, d2, sc = delta_terms(delta)
        ops.add_layernorm(d1, residual, self.weight, self.bias, self.eps, out, delta2=d2, delta_scale=sc)
        return out

    def add_forward_rows(self, delta, residual, rows, out_dtype):
        out = torch.empty((rows.numel(), residual.shape[1]), dtype=out_dtype, device=residual.device)
        d1, d2, sc = delta_terms(delta)
        ops.add_layernorm(d1, residual, self.weight, self.bias, self.eps, out, rows=rows, delta2=d2, delta_scale=sc)
        return out


class GroupRMSNorm(Norm):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive parts, each is divided by its own
    ``sqrt(mean(part^2) + eps)``, and the whole is multiplied by the weight ``[size]``, in 32-bit.  As the norm of a
    sublayer's output (``add_normed``) it also does the residual sum and hands back the stream's new rows in the run
    type, all in one kernel; as a norm of the stream (``forward``, the model's last norm) it normalises the rows it is
    given."""
    kernel_modules = ("row_norms",)

    def __init__(self, size: int, eps: float, groups: int = 1, weight_name: str = "weight"):
        if groups <= 0 or size % groups:
            raise ValueError(f"{size} numbers do not split into {groups} equal parts")
        self.size, self.eps, self.groups, self.weight_name = size, float(eps), int(groups), weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out=out)
        return out

    def add_normed(self, x, residual, out_dtype, bias=None):
        if x is None and (out_dtype is None or out_dtype == residual.dtype):
            return residual if out_dtype is not None else None
        # the 32-bit run reads the stream itself; the bfloat16 run gets a rounded copy from the same kernel
        out = None if out_dtype in (None, residual.dtype) else torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out=out, residual=residual, x_bias=bias if x is not None else None)
        if out_dtype is None:
            return None
        return residual if out is None else out

    def add_forward(self, delta, residual, out_dtype):
        if isinstance(delta, Normed):
            delta.norm.add_normed(delta.tensor, residual, None, bias=delta.bias)
        else:
            d1, d2 = delta_pair(delta)
            if d1 is not None:
                residual.add_(d1.to(residual.dtype) + d2.to(residual.dtype) if d2 is not None else d1.to(residual.dtype))
        return self.forward(residual, out_dtype)

    def add_forward_rows(self, delta, residual, rows, out_dtype):
        idx = rows.long()
        r = residual.index_select(0, idx)
        if isinstance(delta, Normed):
            delta.norm.add_normed(delta.tensor.index_select(0, idx), r, None, bias=delta.bias)
        else:
            d = [x.index_select(0, idx) for x in delta_pair(delta) if x is not None]
            for x in d:
                r.add_(x.to(r.dtype))
        return self.forward(r, out_dtype)


class ChannelScale(ChannelScalePart):
    """``y = s * x`` with a learned vector ``s [size]`` (layer scale).  The product is formed in 32-bit inside the
    norm kernel that adds the sublayer's output to the residual stream."""
    kernel_modules = ("elementwise",)

    def __init__(self, size: int, name: str = "scale"):
        self.size, self.name = size, name

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), role="vector", init="norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.vector = tensors[self.name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.vector.numel() * self.vector.element_size()


register_scale("channel_scale", ChannelScale)
register_norm("rms_norm", RMSNorm)
register_norm("layer_norm", LayerNorm)
register_norm("group_rms_norm", GroupRMSNorm)
