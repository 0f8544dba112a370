"""A model as data: which parts each layer has, and in which order layers run.

An architecture's ``build_spec(config)`` returns a ``ModelSpec``; ``CausalLM`` builds
the parts from it, the weight loader and the random-weights mode read the tensor
list from it, and the cache manager reads the cache needs from it.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional


@dataclasses.dataclass
class PartSpec:
    kind: str                               # a name in the matching registry of parts.registry
    params: Dict[str, Any]                  # constructor parameters (sizes and constants)
    prefix: str = ""                        # weight-name prefix inside the layer, e.g. "self_attn."


@dataclasses.dataclass
class LayerSpec:
    block: PartSpec                         # arrangement, e.g. kind "pre_norm" or "parallel"
    norm1: PartSpec
    mixer: PartSpec
    norm2: Optional[PartSpec]               # None: the arrangement has one norm
    feed_forward: Optional[PartSpec]        # None: a layer without a feed-forward
    prefix: str                             # e.g. "model.layers.3."
    # optional learned vectors (kind "channel_scale") that multiply the mixer's and the feed-forward's output channel
    # by channel before it is added to the residual stream
    scale1: Optional[PartSpec] = None
    scale2: Optional[PartSpec] = None


@dataclasses.dataclass
class RunEntry:
    """One step of the run list.  ``layer`` indexes ``ModelSpec.layers`` and may occur in
    several entries (shared weights, a cache of its own for each entry).  ``kv_from``
    names an EARLIER entry of the run list whose cache this entry reads instead of
    writing one.  ``before``: ``(name, index)`` of a stream part (``ModelSpec.stream_parts``)
    that works on the residual stream right before this entry, e.g. the entrance of a block
    of layers that is run several times, with the number of the pass."""
    layer: int
    kv_from: Optional[int] = None
    before: Optional[tuple] = None


@dataclasses.dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding_name: str                     # e.g. "model.embed_tokens.weight"
    head_name: Optional[str]                # None: the output head is the embedding table (tied)
    final_norm: PartSpec
    position_encodings: Dict[str, PartSpec]  # shared by name between the mixers that ask for one
    layers: List[LayerSpec]
    run: List[RunEntry]
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    # name patterns of tensors that weight files of this architecture may carry and the model does not use
    ignored_tensors: tuple = ()
    # optional factors: the embedded rows are multiplied by ``embedding_scale`` before the first block, the
    # logits by ``logit_scale`` after the head (architectures that scale either; None: untouched)
    embedding_scale: Optional[float] = None
    logit_scale: Optional[float] = None
    # logits <- logit_softcap * tanh(logits / logit_softcap) after the head (None: unbounded)
    logit_softcap: Optional[float] = None
    # a norm that the embedded rows pass before the first block (None: they enter the stream as they are)
    embedding_norm: Optional[PartSpec] = None
    # parts that work on the residual stream between layers, by name (see RunEntry.before)
    stream_parts: Dict[str, PartSpec] = dataclasses.field(default_factory=dict)

    def validate(self) -> None:
        from ..errors import ErrorCode, PhotonError
        for i, e in enumerate(self.run):
            if not 0 <= e.layer < len(self.layers):
                raise PhotonError(ErrorCode.INVALID_CONFIG, f"run entry {i} names layer {e.layer}, which does not exist")
            if e.before is not None and e.before[0] not in self.stream_parts:
                raise PhotonError(ErrorCode.INVALID_CONFIG, f"run entry {i} names the stream part {e.before[0]!r}, which the model does not define")
            if e.kv_from is not None:
                if not 0 <= e.kv_from < i:
                    raise PhotonError(ErrorCode.INVALID_CONFIG,
                                      f"run entry {i} reads the cache of entry {e.kv_from}, which does not run before it")
                if self.run[e.kv_from].kv_from is not None:
                    raise PhotonError(ErrorCode.INVALID_CONFIG,
                                      f"run entry {i} reads the cache of entry {e.kv_from}, which has none of its own")
