"""The Pebodra decoder as a ``ModelSpec``.

Layers with the norm on the sublayer's output only: ``x <- x + norm1(mixer(x)); x <- x + norm2(ff(x))``; the sublayers read
the stream itself.  The norms are RMS norms in groups (``parts/norm.py: GroupRMSNorm``).  The mixer is differential
attention (``parts/diff_attention.py``; a layer may read an earlier layer's keys and values), a state-space layer with a
scalar decay per head (``parts/state_space.py``) or a matrix memory with exponential gates (``parts/matrix_memory.py``).
The feed-forward is dense with the PolyNorm activation (``parts/mlp.py``), a mixture of gated experts behind a sigmoid
router with groups (``parts/moe.py``), or absent.  A final norm of the same kind, an untied output head, and logits
bounded by ``logit_softcap * tanh(logits / logit_softcap)``.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from typing import Optional

from ..config.pebodra_config import PebodraConfig
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _window(m: dict) -> Optional[int]:
    return (m.get("mask") or {}).get("size")


def _cache_window(cfg: PebodraConfig, index: int) -> Optional[int]:
    """Keys that layer ``index`` must keep: the largest window among itself and the layers that read its pages."""
    sizes = [_window(cfg.layers[index].mixer)]
    sizes += [_window(l.mixer) for l in cfg.layers if l.type == "attention" and l.mixer.get("kv_from") == index]
    return None if any(s is None for s in sizes) else max(sizes)


def _mixer(cfg: PebodraConfig, index: int) -> PartSpec:
    l = cfg.layers[index]
    m = l.mixer
    if l.type == "attention":
        rot = m.get("rot") or {}
        own = m.get("kv_from") is None
        return PartSpec("diff_attention",
                        dict(hidden_size=cfg.width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                             value_dim=m["vdim"], eps=cfg.norm_eps, scale=m["scale"], diff=m["diff"], rot_dims=rot.get("dims", 0),
                             rot_base=rot.get("base", 10000.0), window=_window(m),
                             cache_window=_cache_window(cfg, index) if own else "own", own_kv=own, bias=True), "mix.")
    if l.type == "mamba2":
        return PartSpec("state_space", dict(hidden_size=cfg.width, heads=m["heads"], vdim=m["vdim"], state=m["state"],
                                            taps=m["conv"], eps=cfg.norm_eps, groups=m["groups"], norm_groups=m["norm_groups"]),
                        "mix.")
    return PartSpec("matrix_memory", dict(hidden_size=cfg.width, heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                                          gate_cap=m["gate_cap"], eps=cfg.norm_eps), "mix.")


def _feed_forward(cfg: PebodraConfig, mlp: Optional[dict]) -> Optional[PartSpec]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("polynorm", dict(hidden_size=cfg.width, intermediate_size=mlp["ff"], eps=cfg.norm_eps,
                                         names=("up", "down", "act")), "mlp.")
    r = mlp["router"]
    g = r.get("groups") or {}
    return PartSpec("moe", dict(hidden_size=cfg.width, experts=r["experts"], top=r["top"], expert_size=mlp["expert"]["ff"],
                                activation="silu", gated=True, router_bias=False, scoring="sigmoid", groups=g.get("count", 1),
                                keep_groups=g.get("keep"), route_scale=1.0), "mlp.")


def build_pebodra_spec(cfg: PebodraConfig) -> ModelSpec:
    norm = lambda name: PartSpec("group_rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups,
                                                    "weight_name": name})
    layers, run = [], []
    for i, l in enumerate(cfg.layers):
        ff = _feed_forward(cfg, l.mlp)
        layers.append(LayerSpec(block=PartSpec("output_norm", {}), norm1=norm("norm1"), mixer=_mixer(cfg, i),
                                norm2=norm("norm2") if ff is not None else None, feed_forward=ff, prefix=f"l{i}."))
        run.append(RunEntry(i, kv_from=l.mixer.get("kv_from") if l.type == "attention" else None))
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions, embedding_name="embed",
                     head_name="head", final_norm=norm("final.norm"), position_encodings={}, layers=layers, run=run,
                     logit_softcap=cfg.logit_softcap)


register_architecture("Pebodra", PebodraConfig, build_pebodra_spec, replace=True)
