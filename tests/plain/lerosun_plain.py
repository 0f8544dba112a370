"""The Lerosun decoder, written plainly: one function per mechanism, float64 torch on the CPU, whole sequences
at once, no cache and no state (the recurrence is a loop over the tokens).  It shares no code with the package;
the tests compare the package against it.

A model is ``(config, tensors)``: the dictionary of config.json and the tensors by name.

Notation: ``x [n, width]`` the residual stream of one sequence, position ``i`` of a query, ``j`` of a key,
``H`` query heads, ``G`` key/value heads.
"""
import json
import math
import os
import struct

import torch

F = torch.float64


def t64(t):
    return t.to(F)


# ----------------------------------------------------------------------------- norms

def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_rms_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(x, eps) * g


# ----------------------------------------------------------------------------- positions

def rotate_first_dims(x, pos, dims, base):
    """x [n, heads, d]; the first ``dims`` numbers of a head are rotated, number i with number i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = pos.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- attention with mixed heads

def window_visible(n, size=None):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & (i - j < size)
    return ok


def mixed_head_scores(q, k, scale, temp, talk):
    """q [n, H, d], k [n, G, d] -> [H, n, n]: per-head scores times scale and the head's temperature, then every
    head's score becomes a weighted sum of all heads' scores, ``talk [H, H]`` (row: the head that receives)."""
    n, H, _ = q.shape
    G = k.shape[1]
    raw = torch.stack([q[:, h, :] @ k[:, h // (H // G), :].T for h in range(H)]) * scale * temp[:, None, None]
    return torch.einsum("hg,gij->hij", talk, raw)


def softmax_with_sink(s, ok, sink):
    """s [H, n, n]; the denominator also holds exp(sink[h]), which has no key and no value."""
    s = s.masked_fill(~ok, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def attention_mixer(h, w, p, m, pos):
    """``w``: the layer's tensors by local name; ``m``: the mixer's sizes and constants."""
    n = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, d)
    k = (h @ w["k"].T + w["k.b"]).reshape(n, G, d)
    v = k                                                  # the values are the keys, before the rotation
    rot = m.get("rot") or {}
    qr = rotate_first_dims(q, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    kr = rotate_first_dims(k, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    s = mixed_head_scores(qr, kr, m["scale"], w["temp"], w["talk"])
    ok = window_visible(n, (m.get("mask") or {}).get("size"))
    pr = softmax_with_sink(s, ok, w["sink"])
    o = torch.stack([pr[hh] @ v[:, hh // (H // G), :] for hh in range(H)], dim=1)      # [n, H, d]
    gate = torch.sigmoid(h @ w["g"].T)                     # [n, H]
    return (o * gate[:, :, None]).reshape(n, H * d) @ w["o"].T


# ----------------------------------------------------------------------------- gated delta rule

def short_conv_silu(x, taps_w):
    """x [n, C]; ``taps_w [C, taps]``, the last column weighs the current token; zeros before the start."""
    n, C = x.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    y = torch.zeros(n, C, dtype=F)
    for i in range(taps):
        y = y + pad[i:i + n] * taps_w[:, i][None, :]
    return y * torch.sigmoid(y)


def unit_vectors(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [n, H, d], v [n, H, dv], beta, g [n, H] -> [n, H, dv].  Per head, with the state S [d, dv] from zero:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=F)
    out = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def delta_mixer(h, w, m, eps):
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_vectors(short_conv_silu(h @ w["q"].T, w["q.conv"]).reshape(n, G, d)) * d ** -0.5
    k = unit_vectors(short_conv_silu(h @ w["k"].T, w["k.conv"]).reshape(n, G, d))
    v = short_conv_silu(h @ w["v"].T, w["v.conv"]).reshape(n, H, dv)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w["b"].T)
    g = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * w["norm"]
    z = (h @ w["g"].T).reshape(n, H, dv)
    return (o * z * torch.sigmoid(z)).reshape(n, H * dv) @ w["o"].T


# ----------------------------------------------------------------------------- feed-forward

def relu_gated(h, w):
    return (torch.relu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# ----------------------------------------------------------------------------- the whole model

def run_list(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def local(tensors, prefix):
    return {k[len(prefix):]: t64(v) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, ids, layers_out=None):
    """Logits [n, vocab] (float64) of one sequence.  ``layers_out``: a list that receives the stream after every
    layer run."""
    eps = cfg["norm"]["eps"]
    pos = torch.arange(len(ids))
    x = scalar_rms_norm(t64(tensors["embed"])[torch.tensor(ids)], t64(tensors["embed.norm"]), eps)
    for li in run_list(cfg):
        l = cfg["layers"][li]
        p = f"l{li}."
        h = scalar_rms_norm(x, t64(tensors[p + "norm1"]), eps)
        w = local(tensors, p + "mix.")
        if l["type"] == "attention":
            a = attention_mixer(h, w, p, l["mixer"], pos)
        else:
            a = delta_mixer(h, w, l["mixer"], eps)
        x = x + a * t64(tensors[p + "ls1"])
        if l.get("mlp") is not None:
            h = scalar_rms_norm(x, t64(tensors[p + "norm2"]), eps)
            x = x + relu_gated(h, local(tensors, p + "mlp.")) * t64(tensors[p + "ls2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = scalar_rms_norm(x, t64(tensors["final.norm"]), eps)
    return x @ t64(tensors["head"]).T


# ----------------------------------------------------------------------------- reading a folder

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "F64": torch.float64}


def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=_DT[info["dtype"]]) if b > a else torch.zeros(0, dtype=_DT[info["dtype"]])
        tensors[name] = t.reshape(info["shape"]).clone()
    return cfg, tensors


def greedy(config, tensors, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(forward(config, tensors, ids)[-1])))
    return ids[len(prompt):]
