"""A causal language model built from a ``ModelSpec``: embedding, the run list of
blocks, final norm and output head.  It knows nothing of Llama; the spec does.

``forward`` runs exactly the tokens of one step (``StepContext``) against the cache
and returns 32-bit logits for the wanted rows only; the reference computes logits
for every token of the step (include/photon/scheduler/continuous_batch_engine.hpp:
226-237).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..errors import ErrorCode, PhotonError
from ..kernels import ops
from ..parts.base import (Block, LayerCache, Mixer, PagedCacheSpec, Part, StateSpec, StepContext,
                          TensorSpec)
from ..parts.registry import create_part
from .spec import LayerSpec, ModelSpec


def _build_position_encodings(spec: ModelSpec) -> Dict[str, Part]:
    return {name: create_part("position_encoding", ps.kind, ps.params)
            for name, ps in spec.position_encodings.items()}


def _build_layer(ls: LayerSpec, encodings: Dict[str, Part]) -> Block:
    mixer_params = dict(ls.mixer.params)
    if "position_encoding" in mixer_params and isinstance(mixer_params["position_encoding"], str):
        key = mixer_params["position_encoding"]
        if key not in encodings:
            raise PhotonError(ErrorCode.INVALID_CONFIG, f"mixer asks for position encoding {key!r}, which the model does not define")
        mixer_params["position_encoding"] = encodings[key]
    norm1 = create_part("norm", ls.norm1.kind, ls.norm1.params)
    mixer = create_part("mixer", ls.mixer.kind, mixer_params)
    norm2 = create_part("norm", ls.norm2.kind, ls.norm2.params) if ls.norm2 is not None else None
    ff = create_part("feed_forward", ls.feed_forward.kind, ls.feed_forward.params) if ls.feed_forward is not None else None
    params = dict(ls.block.params, norm1=norm1, mixer=mixer, norm2=norm2, feed_forward=ff)
    for key, ps in (("scale1", ls.scale1), ("scale2", ls.scale2)):
        if ps is not None:
            params[key] = create_part("scale", ps.kind, ps.params)
    return create_part("block", ls.block.kind, params)


def _layer_part_prefixes(ls: LayerSpec) -> Dict[str, str]:
    out = {"norm1": ls.prefix + ls.norm1.prefix, "mixer": ls.prefix + ls.mixer.prefix}
    if ls.norm2 is not None:
        out["norm2"] = ls.prefix + ls.norm2.prefix
    if ls.feed_forward is not None:
        out["feed_forward"] = ls.prefix + ls.feed_forward.prefix
    for key, ps in (("scale1", ls.scale1), ("scale2", ls.scale2)):
        if ps is not None:
            out[key] = ls.prefix + ps.prefix
    return out


class _Skeleton:
    """Parts of a model built without weights or a device: enough to list tensors and cache needs."""

    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.encodings = _build_position_encodings(spec)
        self.blocks: List[Block] = [_build_layer(ls, self.encodings) for ls in spec.layers]
        self.stream_parts: Dict[str, Part] = {name: create_part("stream", ps.kind, ps.params)
                                              for name, ps in spec.stream_parts.items()}
        self.final_norm = create_part("norm", spec.final_norm.kind, spec.final_norm.params)
        self.embedding_norm = (create_part("norm", spec.embedding_norm.kind, spec.embedding_norm.params)
                               if spec.embedding_norm is not None else None)

    def named_parts(self) -> List[Tuple[str, Part]]:
        out: List[Tuple[str, Part]] = []
        for name, pe in self.encodings.items():
            out.append((self.spec.position_encodings[name].prefix, pe))
        for name, sp in self.stream_parts.items():
            out.append((self.spec.stream_parts[name].prefix, sp))
        for ls, block in zip(self.spec.layers, self.blocks):
            prefixes = _layer_part_prefixes(ls)
            for key, part in block.parts().items():
                out.append((prefixes[key], part))
        out.append((self.spec.final_norm.prefix, self.final_norm))
        if self.embedding_norm is not None:
            out.append((self.spec.embedding_norm.prefix, self.embedding_norm))
        return out

    def declared(self) -> Dict[str, TensorSpec]:
        s = self.spec
        d: Dict[str, TensorSpec] = {s.embedding_name: TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size))}
        for prefix, part in self.named_parts():
            for ts in part.tensor_specs():
                full = prefix + ts.name
                if full in d:
                    raise PhotonError(ErrorCode.INVALID_CONFIG, f"two parts declare the tensor {full!r}")
                d[full] = ts
        if s.head_name is not None:
            d[s.head_name] = TensorSpec(s.head_name, (s.vocab_size, s.hidden_size))
        return d


def declared_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Full tensor name -> spec, for the loader and the random-weights mode."""
    return _Skeleton(spec).declared()


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        sk = _Skeleton(spec)
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.encodings = sk.encodings
        self.blocks = sk.blocks
        self.stream_parts = sk.stream_parts
        self.final_norm = sk.final_norm
        self.embedding_norm = sk.embedding_norm
        self._skeleton = sk
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ weights
    def declared(self) -> Dict[str, TensorSpec]:
        return self._skeleton.declared()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name]
        self.head = self.embedding if s.head_name is None else tensors[s.head_name]   # tied: alias, no copy
        for prefix, part in self._skeleton.named_parts():
            local = {ts.name: tensors[prefix + ts.name] for ts in part.tensor_specs()}
            part.load(local)
        for pe in self.encodings.values():
            if hasattr(pe, "to_device"):
                pe.to_device(self.device)

    def kernel_modules(self) -> List[object]:
        """What this model launches in this dtype: module names and (name, definitions) pairs."""
        mods: List[object] = ["elementwise", "sampling"] + (["row_norms"] if self.spec.logit_softcap is not None else [])
        if self.dtype == torch.float32:
            mods.append("gemm_f32")
        for _, part in self._skeleton.named_parts():
            for m in part.required_kernels(self.dtype):
                if m not in mods:
                    mods.append(m)
        return mods

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every matrix of every run-list entry once, the output
        head, no embedding rows."""
        total = self.head.numel() * self.head.element_size() + self.final_norm.weight_bytes()
        for e in self.spec.run:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts().values())
            if e.before is not None:
                total += self.stream_parts[e.before[0]].weight_bytes()
        return total

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> List[Tuple[Optional[PagedCacheSpec], Optional[StateSpec]]]:
        """One pair per entry of the run list; entries that read another entry's cache report None pages."""
        out = []
        for e in self.spec.run:
            m: Mixer = self.blocks[e.layer].mixer()
            out.append((m.cache_spec() if e.kv_from is None else None, m.state_spec()))
        return out

    # ------------------------------------------------------------------ one step
    def forward(self, ctx: StepContext, caches: List[LayerCache], logit_rows: torch.Tensor) -> torch.Tensor:
        """``caches[i]`` belongs to entry ``i`` of the run list.  ``logit_rows``: int32 indices of the
        tokens of the step whose logits are wanted.  Returns float32 ``[len(logit_rows), vocab]``."""
        T = ctx.num_tokens
        residual = torch.empty((T, self.spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.embedding(ctx.token_ids, self.embedding, residual, ctx.error_flag)
        if self.spec.embedding_scale is not None:
            ops.scale_bias_rows(residual, self.spec.embedding_scale)
        if self.embedding_norm is not None:
            residual = self.embedding_norm.forward(residual, torch.float32)        # the normed rows are the stream
        # the embedding output is kept when a stream part will read it again (the blocks add into `residual` in place)
        first = residual.clone() if any(e.before is not None for e in self.spec.run) else None
        delta = None
        for entry, cache in zip(self.spec.run, caches):
            if entry.before is not None:
                name, index = entry.before
                residual, delta = self.stream_parts[name].forward(residual, delta, first, index, ctx), None
            residual, delta = self.blocks[entry.layer].forward(residual, delta, ctx, cache)
        n = logit_rows.numel()
        if n == 0:
            # the blocks still ran: their cache writes are the step's effect
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        y = self.final_norm.add_forward_rows(delta, residual, logit_rows, self.dtype)
        logits = ops.linear(y, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale is not None:
            logits.mul_(self.spec.logit_scale)
        if self.spec.logit_softcap is not None:
            ops.softcap_(logits, self.spec.logit_softcap)
        return logits
