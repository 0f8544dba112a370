"""Mixture of experts: ``experts`` small gated feed-forward layers, of which every token uses ``top``, and an
optional shared expert of the same form that every token uses.

Router logits ``z = W_r h + b`` in 32-bit; the ``top`` experts with the largest logits are chosen and weighted
with the softmax over the chosen logits only; the output is the weighted sum of their outputs plus the shared
expert's.  An expert is ``W_down (act(W_gate h) * (W_up h))`` without biases.

On the device the (token, choice) pairs are sorted by expert without a round trip to the host; two grouped
products walk the sorted rows (the first gathers its rows of ``h`` and applies the gated activation in its
epilogue, the second leaves 32-bit rows), and one kernel forms every token's weighted sum in the order of its
choices and adds the shared expert's output.  That is the float32 path and the one for a middling number of
rows.  A bfloat16 decode step (a handful of pairs) skips the sort and runs one matrix-vector product per pair;
a bfloat16 step with many rows hands the sorted rows to the library's grouped product.  The experts' matrices are stacked into ``[E, 2 ff, H]`` and
``[E, H, ff]`` when loaded.

Variants, all by parameter.  ``gated`` False: an expert is ``W_down act(W_up h)`` (tensors ``e<i>.up``, ``e<i>.down``;
the stack is ``[E, ff, H]``), and so is the shared expert.  ``router_bias`` False: no ``router.b``.  ``scoring``
``softmax_all``: scores are the softmax over all experts, the experts form ``groups`` equal groups of neighbours of
which only the ``keep_groups`` with the largest best score may be chosen from, and the weights are the chosen scores
over their sum times ``route_scale``.  ``shared_gate``: the shared expert's output is multiplied by
``sigmoid(W_sg h)``, one number per token (``shared.sg [1, H]``), computed with the router's logits in 32-bit.
``scoring`` ``sigmoid``: scores are ``sigmoid(logit)``, each expert by itself; a group's score is the sum of its two largest
scores; the weights are the chosen scores times ``route_scale``, not divided by their sum.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, TensorSpec
from .linear import project
from .registry import register_feed_forward


class MoEFeedForward(FeedForward):
    kernel_modules = ("moe", "elementwise")

    def required_kernels(self, dtype):
        return list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, shared_size: Optional[int] = None,
                 activation: str = "silu", shared_activation: Optional[str] = None, gated: bool = True,
                 router_bias: bool = True, scoring: str = "softmax_chosen", groups: int = 1, keep_groups: Optional[int] = None,
                 route_scale: float = 1.0, shared_gate: bool = False):
        if not 1 <= top <= experts:
            raise ValueError("a token uses between one and all of the experts")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        self.hidden_size, self.experts, self.top = hidden_size, experts, top
        self.expert_size, self.shared_size = expert_size, shared_size
        self.activation = activation
        self.shared_activation = shared_activation or activation
        if scoring not in ops.ROUTER_SCORING:
            raise ValueError(f"unknown router scoring {scoring!r}")
        self.gated, self.router_bias, self.scoring = bool(gated), bool(router_bias), scoring
        self.groups = int(groups or 1)
        self.keep_groups = int(keep_groups) if keep_groups else self.groups
        if experts % self.groups or not 1 <= self.keep_groups <= self.groups or self.keep_groups * (experts // self.groups) < top:
            raise ValueError("the experts must split into equal groups, and the kept groups must hold at least `top` experts")
        self.route_scale = float(route_scale)
        self.shared_gate = bool(shared_gate) and bool(shared_size)
        self.w_shared_gate = None
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None
        self.shared_gate_up = self.shared_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        H, F = self.hidden_size, self.expert_size
        specs = [TensorSpec("router", (self.experts, H))]
        if self.router_bias:
            specs.append(TensorSpec("router.b", (self.experts,), role="vector", init="normal"))
        for e in range(self.experts):
            specs += ([TensorSpec(f"e{e}.gate", (F, H))] if self.gated else []) + \
                     [TensorSpec(f"e{e}.up", (F, H)), TensorSpec(f"e{e}.down", (H, F))]
        if self.shared_size:
            S = self.shared_size
            specs += ([TensorSpec("shared.gate", (S, H))] if self.gated else []) + \
                     [TensorSpec("shared.up", (S, H)), TensorSpec("shared.down", (H, S))]
            if self.shared_gate:
                specs.append(TensorSpec("shared.sg", (1, H)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = self.experts
        self.w_router = tensors["router"].contiguous()
        self.b_router = tensors["router.b"].contiguous() if self.router_bias else None
        # the first matrix of every expert: [gate rows; up rows] of a gated expert, the up rows of a plain one
        first = (lambda p: torch.cat([tensors[p + "gate"], tensors[p + "up"]], dim=0)) if self.gated else (lambda p: tensors[p + "up"])
        self.w_gate_up = torch.stack([first(f"e{e}.") for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared_size:
            self.shared_gate_up = first("shared.").contiguous()
            self.shared_down = tensors["shared.down"].contiguous()
            if self.shared_gate:
                self.w_shared_gate = tensors["shared.sg"].contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router, the shared expert and every expert once."""
        ws = [self.w_router, self.w_gate_up, self.w_down] + ([self.shared_gate_up, self.shared_down] if self.shared_size else [])
        return sum(w.numel() * w.element_size() for w in ws)

    def _shared(self, h: torch.Tensor) -> torch.Tensor:
        if self.gated:
            return project(ops.linear_swiglu(h, self.shared_gate_up, self.shared_activation), self.shared_down)
        return project(ops.linear_act(h, self.shared_gate_up, self.shared_activation), self.shared_down)

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, H = h.shape
        n = T * self.top
        # A long portion: the shared expert's two products run on a second stream beside the router, the sort, the
        # gather and the passes between the grouped products, which leave most of the GPU idle.  The weighted sum
        # waits for them.  Not while a stream is captured, and not for few rows (their products share scratch
        # memory with others of their kind).
        shared_done = None
        if SHARED_EXPERT_STREAM and self.shared_size and n >= GROUPED_LIBRARY_PAIRS and T >= 64 and h.dtype == torch.bfloat16 \
                and not torch.cuda.is_current_stream_capturing():
            side = _side_stream(h.device)
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                shared_early = self._shared(h)
                shared_done = torch.cuda.Event()
                shared_done.record(side)
        routed = ops.moe_route(h, self.w_router, self.b_router, self.top, self.scoring, self.groups, self.keep_groups,
                               self.route_scale, self.w_shared_gate)
        ids, weights, counts = routed[:3]
        sgate = routed[3] if self.w_shared_gate is not None else None
        if shared_done is not None:
            shared = shared_early
        else:
            shared = self._shared(h) if self.shared_size else None
        glu, act_name = self.gated, self.activation
        out = torch.empty((T, H), dtype=h.dtype, device=h.device)

        def combine(y, place):
            if shared_done is not None:
                torch.cuda.current_stream().wait_event(shared_done)      # the shared expert's rows are there
            ops.moe_combine(y, place, weights, shared, out, sgate)

        if n <= GEMV_MAX_PAIRS and ops.moe_gemv_supported(h, self.w_gate_up) and self.expert_size % 8 == 0:
            # a decode step: nothing is sorted, every pair streams its expert's matrices once
            act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
            ops.moe_gemv(h, self.top, ids, self.w_gate_up, act, glu=glu, activation=act_name)
            y = torch.empty((n, H), dtype=torch.float32, device=h.device)
            ops.moe_gemv(act, 1, ids, self.w_down, y)
            combine(y, None)
            return out
        offsets, srt, place, tiles, num_tiles, max_tiles = ops.moe_align(ids, counts)
        if h.dtype == torch.bfloat16 and n >= GROUPED_LIBRARY_PAIRS and H % 8 == 0 and self.expert_size % 8 == 0:
            # many bfloat16 rows: the library's grouped product over the rows gathered in sorted order
            xs = ops.moe_gather(h, srt, self.top)
            gate_up = torch._grouped_mm(xs, self.w_gate_up.transpose(1, 2), offs=offsets[1:])
            if glu:
                act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
                ops.swiglu(gate_up, act, act_name)
            else:
                act = ops.activation(gate_up, act_name)
            y = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=offsets[1:])
            combine(y, place)
            return out
        act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
        ops.moe_gemm(h, srt, self.top, self.w_gate_up, act, tiles, num_tiles, max_tiles, glu=glu, activation=act_name)
        y = torch.empty((n, H), dtype=torch.float32, device=h.device)
        ops.moe_gemm(act, None, 1, self.w_down, y, tiles, num_tiles, max_tiles)
        combine(y, place)
        return out


#: The shared expert of a long portion on a second stream (``PHOTON_MOE_SHARED_STREAM=0``: in line).
SHARED_EXPERT_STREAM = os.environ.get("PHOTON_MOE_SHARED_STREAM", "1") != "0"
_side_streams: Dict[tuple, "torch.cuda.Stream"] = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = (device.type, device.index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


#: Up to this many (token, choice) pairs a bfloat16 step runs one matrix-vector product per pair.
GEMV_MAX_PAIRS = 64
#: From this many pairs on a bfloat16 step hands the sorted rows to the library's grouped product.
GROUPED_LIBRARY_PAIRS = 256

register_feed_forward("moe", MoEFeedForward)
