"""Interfaces of the parts a layer is put together from.

A layer is a *block* that arranges a *mixer* (attention here), a *feed-forward* and
*norms*; a mixer may use a *position encoding*.  Every part gets its sizes and
constants as constructor parameters, declares the weight tensors it needs
(``tensor_specs``) and receives them by local name (``load``).  No part knows which
model it is in: the weight-name prefix, the layer index and the cache it reads are
handed to it from outside.

The reference builds each block from fixed operator members
(include/photon/arch/transformer_block.hpp:53-218); the split into exchangeable
parts has no counterpart there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------- weights

@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One weight tensor of a part.

    ``role``: ``"matrix"`` tensors are operands of matrix products or lookup tables
    and are held in the run dtype; ``"vector"`` tensors (norm weights) keep 32-bit
    storage when the file has it; ``"int"`` tensors are integer tables, held as int32.
    ``init`` tells the random-weights mode how to fill it: ``"normal"`` (N(0, std)),
    ``"norm"`` (ones, or 1 + N(0, norm_std)), ``"zeros"``.
    A dimension of ``-1`` in ``shape`` is a size that the configuration does not give: the weight file decides it
    (the loader accepts any size there), and the random-weights mode uses ``free_size``.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    free_size: int = 16

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(a == -1 or a == b for a, b in zip(self.shape, shape))

    def concrete_shape(self) -> Tuple[int, ...]:
        return tuple(self.free_size if a == -1 else a for a in self.shape)


# ----------------------------------------------------------------------------- caches

@dataclasses.dataclass(frozen=True)
class PagedCacheSpec:
    """What a mixer needs of the paged cache, per token: keys and values of
    ``n_kv_heads * head_dim`` each.  ``window`` None: every earlier key stays
    visible; an integer: only the last ``window`` keys do, and pages behind the
    window are given back.  Layers with equal specs share one group of pages.
    ``values`` False: one row of ``n_kv_heads * head_dim`` per token and no value rows (a
    mixer that caches a latent from which it derives keys and values alike).
    ``value_dim``: width of a value where it differs from a key's (None: ``head_dim``); keys and
    values then live in two tensors.  ``keep_first``: with a window, the first ``keep_first`` tokens
    of a request stay visible for good, so the pages that hold them are not given back."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    values: bool = True
    value_dim: Optional[int] = None
    keep_first: int = 0

    @property
    def planes(self) -> int:
        return 2 if self.values else 1

    @property
    def split_planes(self) -> bool:
        """Keys and values of different widths: one tensor each instead of two planes of one."""
        return self.values and self.value_dim is not None and self.value_dim != self.head_dim

    @property
    def row_width(self) -> int:
        """Numbers cached per token and key/value head."""
        if not self.values:
            return self.head_dim
        return self.head_dim + (self.value_dim if self.value_dim is not None else self.head_dim)


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """Fixed-size state of one request in one layer (shape without the slot axis)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass
class GroupView:
    """Device-side view of one cache group for the current step."""
    block_table: torch.Tensor       # int32 [S, max_pages]; -1 where no page is held
    slot_mapping: torch.Tensor      # int32 [T]; page * page_size + offset of each token of the step
    page_size: int
    num_pages: int
    max_pages_per_seq: int


@dataclasses.dataclass
class LayerCache:
    """What one entry of the run list gets for its mixer."""
    group: Optional[int] = None             # index into StepContext.groups
    k: Optional[torch.Tensor] = None        # [num_pages, n_kv, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    shared: bool = False                    # true: another entry wrote these pages; do not write
    state: Optional[torch.Tensor] = None    # [max_sequences, *StateSpec.shape]


@dataclasses.dataclass
class StepContext:
    """Everything a part may read about the current step.

    Token-major arrays have one entry per token of the step (``T``); sequence-major
    arrays one per request in the step (``S``), in batch order.
    """
    num_tokens: int
    num_seqs: int
    dtype: torch.dtype                      # run dtype of activations and caches
    token_ids: torch.Tensor                 # int32 [T]
    positions: torch.Tensor                 # int32 [T] position of each token in its request
    token_seq: torch.Tensor                 # int32 [T] index of the token's request in the batch
    cu_tokens: torch.Tensor                 # int32 [S+1] first token of each request in the step
    context_lens: torch.Tensor              # int32 [S] tokens of the request after this step
    state_slots: torch.Tensor               # int32 [S] slot of the request's fixed-size state
    groups: List[GroupView]
    # host copies, for choosing kernels and grids
    host_query_lens: Sequence[int] = ()
    host_context_lens: Sequence[int] = ()
    host_start_positions: Sequence[int] = ()
    max_query_len: int = 0
    max_context_len: int = 0
    error_flag: Optional[torch.Tensor] = None   # int32 [4] written by kernels on bad indices
    scratch: Optional[object] = None            # engine.workspace.Workspace
    host_state_slots: Sequence[int] = ()        # host copy of state_slots


# ----------------------------------------------------------------------------- parts

class Part:
    """Base of all parts: declared tensors in, device tensors held."""

    #: names of the CUDA modules (files under csrc/) the part launches
    kernel_modules: Tuple[str, ...] = ()

    def required_kernels(self, dtype: torch.dtype) -> List[object]:
        """Modules to compile before the first step: names, or (name, definitions) pairs."""
        return list(self.kernel_modules)

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors of ``tensor_specs`` by local name, on the device."""

    def weight_bytes(self) -> int:
        """Bytes a step reads of this part's weights (for the roofline)."""
        return 0


@dataclasses.dataclass
class Scaled:
    """A pending output whose channels are multiplied by a learned vector before the sum:
    ``residual += scale * tensor`` (``scale [H]``, 32-bit); the norm that follows does both in its kernel."""
    tensor: torch.Tensor
    scale: torch.Tensor

    def materialize(self) -> torch.Tensor:
        """The scaled rows as a 32-bit tensor, for a consumer that cannot take the vector into its own kernel."""
        return self.tensor.to(torch.float32) * self.scale.to(torch.float32)


@dataclasses.dataclass
class Normed:
    """A pending output that passes a norm before the sum: ``residual += norm(tensor)`` (a layer whose norms sit on
    its sublayers' outputs).  A consumer that knows the kind does norm and sum in one kernel (``Norm.add_normed``)."""
    tensor: torch.Tensor
    norm: "Norm"
    bias: Optional[torch.Tensor] = None     # [H]: still to be added to ``tensor`` before the norm (a product's bias)

    def materialize(self) -> torch.Tensor:
        """The normed rows as a 32-bit tensor, for a consumer that cannot take the norm into its own kernel."""
        x = self.tensor if self.bias is None else self.tensor.to(torch.float32) + self.bias.to(torch.float32)
        return self.norm.forward(x, torch.float32)


def delta_terms(delta) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``(d1, d2, scale)``: what is pending on the stream as ``scale * d1 + d2`` (each may be None)."""
    if isinstance(delta, Scaled):
        return delta.tensor, None, delta.scale
    d1, d2 = delta_pair(delta)
    return d1, d2, None


def delta_pair(delta) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """What a block hands on to be added to the residual stream: nothing, one tensor, or the two outputs of a
    parallel block (mixer and feed-forward), which are summed with each other first and then into the stream."""
    if delta is None:
        return None, None
    if isinstance(delta, (Scaled, Normed)):
        return delta.materialize(), None
    if isinstance(delta, (tuple, list)):
        parts = [d for d in delta if d is not None]
        if len(parts) > 2:
            raise ValueError("at most two pending outputs can be added to the residual stream")
        return (parts + [None, None])[0], (parts + [None, None])[1]
    return delta, None


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``x`` is the 32-bit residual stream ``[T, H]``; returns the normed rows."""
        raise NotImplementedError

    def add_forward(self, delta, residual: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``residual += delta`` (in 32-bit, in place), then ``forward(residual)``.  ``delta``: a tensor, a pair
        of tensors (``delta_pair``) or None."""
        d1, d2 = delta_pair(delta)
        if d1 is not None:
            residual.add_(d1.to(residual.dtype) + d2.to(residual.dtype) if d2 is not None else d1.to(residual.dtype))
        return self.forward(residual, out_dtype)

    def add_normed(self, x: Optional[torch.Tensor], residual: torch.Tensor, out_dtype: Optional[torch.dtype],
                   bias: Optional[torch.Tensor] = None):
        """``residual += forward(x + bias)`` in 32-bit, in place (``x`` None: nothing is added; ``bias [H]`` may be None);
        returns the stream's new rows in ``out_dtype`` (None: nothing is returned).  A norm that sits on a sublayer's
        output fuses them all."""
        if x is not None:
            if bias is not None:
                x = x.to(torch.float32) + bias.to(torch.float32)
            residual.add_(self.forward(x, torch.float32))
        if out_dtype is None:
            return None
        return residual if out_dtype == residual.dtype else residual.to(out_dtype)

    def add_forward_rows(self, delta, residual: torch.Tensor, rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """Same as ``add_forward`` for the listed rows only; returns ``[len(rows), H]``."""
        r = residual.index_select(0, rows.long())
        d = tuple(x.index_select(0, rows.long()) for x in delta_pair(delta) if x is not None)
        return self.add_forward(d or None, r, out_dtype)


class PositionEncoding(Part):
    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        """Encode in place: ``q [T, n_q, d]``, ``k [T, n_kv, d]`` (views with a row stride)."""
        raise NotImplementedError


class Mixer(Part):
    #: True when the mixer treats a negative state slot as "start from a zero state and store nothing"; decode
    #: steps of a model whose stateful mixers all do are replayed as CUDA graphs.
    state_skips_negative_slots = False

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """``h [T, H]`` normed input in the run dtype; returns ``[T, H]`` to add to the residual."""
        raise NotImplementedError

    def forward_deferred_bias(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache):
        """``(output, bias)``: like ``forward``, but a mixer whose output product has a bias may leave it out of the
        output and hand it over, for a block whose next kernel adds it (``bias`` None: nothing is left out)."""
        return self.forward(h, ctx, cache), None

    # Optional fast path.  A mixer that can take the residual sum and the norm into its first kernel
    # answers True and implements forward_with_norm; the block then skips the separate norm pass.
    def fuses_norm(self, norm: Norm, residual: torch.Tensor, ctx: StepContext, cache: LayerCache) -> bool:
        return False

    def forward_with_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], norm: Norm,
                          ctx: StepContext, cache: LayerCache) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(output, new residual)`` where the new residual is ``residual + delta``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def fuses_norm(self, norm: Norm, residual: torch.Tensor, ctx: StepContext) -> bool:
        return False

    def forward_with_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], norm: Norm,
                          ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError


class ChannelScalePart(Part):
    """A learned vector ``[H]`` that multiplies a sublayer's output channel by channel (``vector`` below, 32-bit)."""
    vector: Optional[torch.Tensor] = None

    def apply(self, x: torch.Tensor) -> "Scaled":
        return Scaled(x, self.vector)


class StreamPart(Part):
    """A step between two layers that works on the residual stream itself (a projection that mixes the running
    stream with the embedding output, for instance).  The model calls it before the run-list entries that name it."""

    def forward(self, residual: torch.Tensor, delta, first: torch.Tensor, index: int, ctx: StepContext) -> torch.Tensor:
        """``residual`` (32-bit) with the pending output ``delta`` of the block before, ``first``: the embedding
        output of the step (32-bit), ``index``: which of its uses this is.  Returns the new 32-bit stream; nothing
        stays pending."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of parts in a layer.  ``forward`` gets the 32-bit residual stream
    and the not-yet-added output of the previous block, and returns the same pair, so
    that every residual sum is fused with the norm that follows it."""

    def parts(self) -> Dict[str, Part]:
        raise NotImplementedError

    def mixer(self) -> Mixer:
        raise NotImplementedError

    def forward(self, residual: torch.Tensor, delta, ctx: StepContext, cache: LayerCache):
        """``delta``: what the block before left to be added (a tensor, a pair, or None); returns the stream and
        what this block leaves to be added."""
        raise NotImplementedError
