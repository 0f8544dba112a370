"""The Lerosun decoder as a ``ModelSpec``.

The embedded rows pass an RMS norm whose weight is one number (``embed.norm``).  Pre-norm layers with such norms:
``x += ls1 * mixer(norm1(x)); x += ls2 * ff(norm2(x))``, the outputs of both sublayers multiplied channel by channel
by a learned vector before they are added.  The mixer is attention whose heads' scores are mixed before the softmax
and whose values are its keys (``parts/talking_attention.py``), or a gated delta rule with short convolutions
(``parts/delta_rule.py``).  The feed-forward is ``W_down (relu(W_gate h) * (W_up h))`` or absent.  A block of layers
may run several times with the same weights, each pass with a cache or state of its own; nothing happens between
the passes.  A final norm of the same kind and an untied output head.

Tensor names: ``embed``, ``embed.norm``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.lerosun_config import LerosunConfig
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(cfg: LerosunConfig, kind: str, m: dict) -> PartSpec:
    if kind == "attention":
        rot = m.get("rot") or {}
        return PartSpec("talking_attention",
                        dict(hidden_size=cfg.width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                             scale=m["scale"], window=(m.get("mask") or {}).get("size"), rot_dims=rot.get("dims", 0),
                             rot_base=rot.get("base", 10000.0), bias=True, temperature=True, talk=True, sink=True,
                             output_gate=True, values_are_keys=True), "mix.")
    return PartSpec("delta_rule", dict(hidden_size=cfg.width, heads=m["heads"], qk_heads=m["kv_heads"], dim=m["dim"],
                                       vdim=m["vdim"], taps=m["conv"], eps=cfg.norm_eps), "mix.")


def build_lerosun_spec(cfg: LerosunConfig) -> ModelSpec:
    norm = lambda name: PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": name, "scalar": True})
    scale = lambda name: PartSpec("channel_scale", {"size": cfg.width, "name": name})
    layers = []
    for i, l in enumerate(cfg.layers):
        ff = None
        if l.mlp is not None:
            ff = PartSpec("gated", dict(hidden_size=cfg.width, intermediate_size=l.mlp["ff"], activation="relu",
                                        names=("gate", "up", "down")), "mlp.")
        layers.append(LayerSpec(block=PartSpec("pre_norm", {}), norm1=norm("norm1"), mixer=_mixer(cfg, l.type, l.mixer),
                                norm2=norm("norm2") if ff is not None else None, feed_forward=ff, prefix=f"l{i}.",
                                scale1=scale("ls1"), scale2=scale("ls2") if ff is not None else None))
    n = len(layers)
    if cfg.loop is None:
        run = [RunEntry(i) for i in range(n)]
    else:
        lp = cfg.loop
        run = [RunEntry(i) for i in range(lp.start)]
        for _ in range(lp.times):
            run += [RunEntry(i) for i in range(lp.start, lp.stop)]
        run += [RunEntry(i) for i in range(lp.stop, n)]
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions,
                     embedding_name="embed", head_name="head", final_norm=norm("final.norm"), position_encodings={},
                     layers=layers, run=run, embedding_norm=norm("embed.norm"))


register_architecture("Lerosun", LerosunConfig, build_lerosun_spec, replace=True)
