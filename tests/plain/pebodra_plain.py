"""The Pebodra decoder, written plainly: one function per mechanism, float64 torch on the CPU, whole sequences
at once, no cache and no state (recurrences are loops over the tokens).  It shares no code with the package;
the tests compare the package against it.

A model is ``(config, tensors)``: the dictionary of config.json and the tensors by name.

Notation: ``x [n, width]`` the residual stream of one sequence, position ``i`` of a query, ``j`` of a key,
``H`` query heads, ``G`` key/value heads (or groups), ``d`` a query's or key's size, ``dv`` a value's.
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


def group_rms_norm(x, w, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each divided by its own root mean square; then times w."""
    shape = x.shape
    y = unit_rms(x.reshape(*shape[:-1], groups, shape[-1] // groups), eps).reshape(shape)
    return y * w


# ----------------------------------------------------------------------------- positions

def rotate_first_dims(x, pos, dims, base):
    """x [n, ..., d]; the first ``dims`` numbers of the last axis are rotated, number i with number i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = pos.to(F)[:, None] * freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- differential attention

def window_visible(n, size=None):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & (i - j < size)
    return ok


def difference_weight(w, diff):
    """One number per layer: exp(lq1 . lk1) - exp(lq2 . lk2) + diff."""
    return torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff


def attention_keys_values(h, w, m, pos, eps):
    """Keys after norm and rotation ``[n, G, 2, d]`` and values ``[n, G, dv]`` of a layer that owns them."""
    n = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    k = (h @ w["k"].T + w["k.b"]).reshape(n, G, 2, d)
    k = rotate_first_dims(unit_rms(k, eps) * w["k.norm"], pos, rot.get("dims", 0), rot.get("base", 10000.0))
    v = (h @ w["v"].T + w["v.b"]).reshape(n, G, dv)
    return k, v


def difference_of_maps(q, k, v, ok, scale, lam, diff, eps):
    """q [n, H, 2, d], k [L, G, 2, d], v [L, G, dv], ok [n, L] (who sees whom) -> [n, H * dv].  Each map is a softmax
    attention of its own over the same values; a head's output is a_1 - lam a_2, divided by its root mean square, times
    1 - diff."""
    H, G = q.shape[1], k.shape[1]
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hh, mp, :] @ k[:, g, mp, :].T) * scale
            maps.append(torch.softmax(s.masked_fill(~ok, -math.inf), dim=-1) @ v[:, g, :])
        heads.append(unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1)


def differential_attention(h, w, m, pos, eps, kv):
    """``kv``: (keys, values) as ``attention_keys_values`` gives them, of this layer or of the layer it reads."""
    n = h.shape[0]
    H, d = m["heads"], m["dim"]
    rot = m.get("rot") or {}
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, 2, d)
    q = rotate_first_dims(unit_rms(q, eps) * w["q.norm"], pos, rot.get("dims", 0), rot.get("base", 10000.0))
    k, v = kv
    ok = window_visible(n, (m.get("mask") or {}).get("size"))
    o = difference_of_maps(q, k, v, ok, m["scale"], difference_weight(w, m["diff"]), m["diff"], eps)
    return o @ w["o"].T + w["o.b"]


# ----------------------------------------------------------------------------- state-space mixer

def short_conv_silu(x, taps_w, bias):
    """x [n, C]; ``taps_w [C, taps]``, the last column weighs the current token; zeros before the start."""
    n, C = x.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    y = bias[None, :].expand(n, C).clone()
    for i in range(taps):
        y = y + pad[i:i + n] * taps_w[:, i][None, :]
    return y * torch.sigmoid(y)


def selective_scan(x, B, C, dt, a, D):
    """x [n, H, dv], B, C [n, H, N], dt [n, H], a [H] (positive decay rates), D [H] -> [n, H, dv].  Per head, with
    the state S [N, dv] from zero: S <- exp(-a dt) S + dt B x^T; y = S^T C + D x."""
    n, H, dv = x.shape
    N = B.shape[-1]
    S = torch.zeros(H, N, dv, dtype=F)
    out = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        S = S * torch.exp(-a * dt[t])[:, None, None] + (dt[t][:, None] * B[t])[:, :, None] * x[t][:, None, :]
        out[t] = torch.einsum("hnv,hn->hv", S, C[t]) + D[:, None] * x[t]
    return out


def mamba_mixer(h, w, m, eps):
    n = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    row = h @ w["in"].T
    z, xbc, dt = row[:, :inner], row[:, inner:2 * inner + 2 * G * N], row[:, 2 * inner + 2 * G * N:]
    xbc = short_conv_silu(xbc, w["conv"], w["conv.b"])
    x = xbc[:, :inner].reshape(n, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].reshape(n, G, N).repeat_interleave(H // G, dim=1)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"])
    y = selective_scan(x, B, C, dt, torch.exp(w["A_log"]), w["D"]).reshape(n, inner)
    y = y * (z * torch.sigmoid(z))
    return group_rms_norm(y, w["norm"], m["norm_groups"], eps) @ w["o"].T


# ----------------------------------------------------------------------------- matrix memory

def capped(x, cap):
    return cap * torch.tanh(x / cap)


def matrix_memory(q, k, v, i_log, f_log):
    """q, k [n, H, d], v [n, H, dv], log gates [n, H] -> [n, H, dv].  S [d, dv], n [d] and the running maximum m
    start at zero: m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T; n likewise with k;
    o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)."""
    n, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=F)
    nv = torch.zeros(H, d, dtype=F)
    m = torch.zeros(H, dtype=F)
    out = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        keep, take = torch.exp(f_log[t] + m - m_new), torch.exp(i_log[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        nv = keep[:, None] * nv + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((nv * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm_mixer(h, w, m, eps):
    n = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).reshape(n, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(n, H, d)
    v = (h @ w["v"].T).reshape(n, H, dv)
    i_log = capped(h @ w["i"].T + w["i.b"], cap)
    f_log = torch.nn.functional.logsigmoid(capped(h @ w["f"].T + w["f.b"], cap))
    o = unit_rms(matrix_memory(q, k, v, i_log, f_log), eps).reshape(n, H * dv)
    return (o * w["norm"] * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


# ----------------------------------------------------------------------------- feed-forwards

def polynorm(z, coef, eps):
    a, b, c, e = coef
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def dense_ff(h, w, eps):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def route(h, w_router, r):
    """Chosen experts [n, top] and their weights: sigmoid scores; a group's score is the sum of its two largest;
    only experts of the best ``keep`` groups can be chosen; the weights are the chosen scores as they are."""
    s = torch.sigmoid(h @ w_router.T)
    n, E = s.shape
    allowed = torch.ones(n, E, dtype=torch.bool)
    gr = r.get("groups")
    if gr:
        per = E // gr["count"]
        gs = s.reshape(n, gr["count"], per).topk(min(2, per), dim=-1).values.sum(-1)
        best = gs.topk(gr["keep"], dim=-1).indices
        allowed = torch.zeros(n, gr["count"], dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
    chosen = s.masked_fill(~allowed, -1.0).topk(r["top"], dim=-1).indices
    return chosen, s.gather(1, chosen)


def moe_ff(h, w, mlp, chosen=None):
    """``chosen [n, top]``: experts to use instead of the router's own choice (their weights are still their scores)."""
    r = mlp["router"]
    if chosen is None:
        chosen, weight = route(h, w["router"], r)
    else:
        weight = torch.sigmoid(h @ w["router"].T).gather(1, chosen)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for c, wt in zip(chosen[t].tolist(), weight[t]):
            g = h[t] @ w[f"e{c}.gate"].T
            out[t] += wt * ((g * torch.sigmoid(g) * (h[t] @ w[f"e{c}.up"].T)) @ w[f"e{c}.down"].T)
    return out


# ----------------------------------------------------------------------------- the whole model

def local(tensors, prefix):
    return {k[len(prefix):]: t64(v) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, ids, layers_out=None, forced=None):
    """Logits [n, vocab] (float64) of one sequence.  ``layers_out``: a list that receives the stream after every
    layer.  ``forced``: for every mixture-of-experts layer in order, the experts ``[n, top]`` to use instead of the
    router's choice."""
    forced = list(forced) if forced is not None else None
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    pos = torch.arange(len(ids))
    x = t64(tensors["embed"])[torch.tensor(ids)]
    kept = {}                                                   # keys and values of the attention layers that own them
    for li, l in enumerate(cfg["layers"]):
        p = f"l{li}."
        w, m = local(tensors, p + "mix."), l["mixer"]
        if l["type"] == "attention":
            if m.get("kv_from") is None:
                kept[li] = attention_keys_values(x, w, m, pos, eps)
            a = differential_attention(x, w, m, pos, eps, kept[li if m.get("kv_from") is None else m["kv_from"]])
        elif l["type"] == "mamba2":
            a = mamba_mixer(x, w, m, eps)
        else:
            a = mlstm_mixer(x, w, m, eps)
        x = x + group_rms_norm(a, t64(tensors[p + "norm1"]), groups, eps)
        mlp = l.get("mlp")
        if mlp is not None:
            wf = local(tensors, p + "mlp.")
            d = dense_ff(x, wf, eps) if mlp["kind"] == "dense" else moe_ff(x, wf, mlp, forced.pop(0) if forced else None)
            x = x + group_rms_norm(d, t64(tensors[p + "norm2"]), groups, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    y = group_rms_norm(x, t64(tensors["final.norm"]), groups, eps) @ t64(tensors["head"]).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(y / cap) if cap else y


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
