"""Each mechanism of the Lerosun decoder alone, on the device, against its plain function: the RMS norm whose weight is
one number, fused with the residual sum of an output that waits with a channel scale; the feed-forward with a relu
gate on each path of the products; bias, partial rotation and the cache write of an attention whose values are its
keys; attention with mixed heads, a window, a sink and an output gate over a paged cache (pages scattered, stale
numbers in unused slots), with keys made to stand out far back, just inside and just outside the window, at both
sides of a page border and at the start of the sequence, in prompts and in decoding, whole and with the keys split
over blocks; the short convolution with its rows carried between steps; the gated delta rule with its state carried
between steps, in slots that are used again; both mixers in portions down to one token and in batches of unequal
requests."""
import math

import pytest
import torch

from helpers import rel_err
from plain import lerosun_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)


def _weights(part, dtype, std, seed, overrides=None):
    g = torch.Generator().manual_seed(seed)
    w = {}
    for t in part.tensor_specs():
        x = std * torch.randn(t.concrete_shape(), generator=g)
        if t.init == "norm":
            x = 1.0 + x
        w[t.name] = x.to(dtype)
    for k, v in (overrides or {}).items():
        w[k] = v.to(dtype)
    part.load({k: v.to(DEV) for k, v in w.items()})
    return {k: v.double() for k, v in w.items()}


# ----------------------------------------------------------------------------- norm, layer scale, feed-forward

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 50, 1024])
def test_scalar_norm_with_a_scaled_pending_output(dtype, width):
    from photon_infer_b200.parts.registry import create_part
    g = torch.Generator().manual_seed(width)
    norm = create_part("norm", "rms_norm", {"size": width, "eps": 1e-5, "weight_name": "w", "scalar": True})
    scale = create_part("scale", "channel_scale", {"size": width, "name": "ls"})
    w = torch.tensor(1.37).to(dtype)
    ls = (0.5 * torch.randn(width, generator=g)).to(dtype)
    norm.load({"w": w.to(DEV)})
    scale.load({"ls": ls.to(DEV)})
    x = 2 * torch.randn(6, width, generator=g)
    a = torch.randn(6, width, generator=g).to(dtype)
    res = x.to(DEV).clone()
    out = norm.add_forward(scale.apply(a.to(DEV)), res, dtype)
    want_x = x.double() + a.double() * ls.double()
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    assert rel_err(res.cpu(), want_x) < 1e-6
    assert rel_err(out.float().cpu(), plain.scalar_rms_norm(want_x, w.double(), 1e-5)) < tol
    rows = i32([4, 1])
    res2 = x.to(DEV).clone()
    out2 = norm.add_forward_rows(scale.apply(a.to(DEV)), res2, rows, dtype)
    assert torch.equal(res2.cpu(), x) and torch.equal(out2, out[[4, 1]])
    # the norm alone, with a 32-bit result: the entrance of the embedded rows into the stream
    alone = norm.forward(x.to(DEV).clone(), torch.float32)
    assert alone.dtype == torch.float32 and rel_err(alone.cpu(), plain.scalar_rms_norm(x.double(), w.double(), 1e-5)) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H,ff", [(3, 64, 96), (40, 50, 70), (300, 128, 512), (1, 256, 1024)])
def test_relu_gated_feed_forward(dtype, rows, H, ff):
    from photon_infer_b200.parts.registry import create_part
    part = create_part("feed_forward", "gated", dict(hidden_size=H, intermediate_size=ff, activation="relu", names=("gate", "up", "down")))
    w = _weights(part, dtype, 0.2, rows)
    h = torch.randn(rows, H, generator=torch.Generator().manual_seed(1)).to(dtype)
    got = part.forward(h.to(DEV), None).float().cpu()
    assert rel_err(got, plain.relu_gated(h.double(), w)) < (1e-5 if dtype == torch.float32 else 2e-2)


# ----------------------------------------------------------------------------- attention: bias, rotation, cache write

@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("shape", [dict(H=4, G=2, d=64, rot=32), dict(H=3, G=1, d=10, rot=6), dict(H=2, G=2, d=128, rot=128), dict(H=5, G=5, d=24, rot=0)])
def test_bias_rotation_and_cache_write(in_dtype, out_dtype, shape):
    from photon_infer_b200.kernels import ops
    H, G, d, rot = shape["H"], shape["G"], shape["d"], shape["rot"]
    g = torch.Generator().manual_seed(d)
    T, page, pages = 9, 4, 6
    rows = torch.randn(T, (H + G) * d + 8, generator=g).to(in_dtype)             # sections of a wider row
    qb, kb = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
    pos = [0, 1, 2, 700, 3, 4, 12345, 5, 6]
    slots = [3, 7, -1, 20, 0, 23, 9, 10, 15]
    inv = torch.tensor([1e4 ** (-2.0 * j / rot) for j in range(rot // 2)], dtype=torch.float64) if rot else None
    kc = torch.zeros(pages, G, page, d, dtype=out_dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, H * d, dtype=out_dtype, device=DEV)
    rd = rows.to(DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.talk_prep(rd[:, :H * d], rd[:, H * d:(H + G) * d], None, qb.to(DEV), kb.to(DEV), q_out, i32(pos), inv.to(DEV) if rot else None,
                  rot, i32(slots), kc, vc, H, G, d, err)
    assert err.cpu().tolist()[0] == 0
    q = (rows[:, :H * d].double() + qb.double()).reshape(T, H, d)
    k = (rows[:, H * d:(H + G) * d].double() + kb.double()).reshape(T, G, d)
    qr = plain.rotate_first_dims(q, torch.tensor(pos), rot, 1e4)
    kr = plain.rotate_first_dims(k, torch.tensor(pos), rot, 1e4)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    assert rel_err(q_out.float().cpu().reshape(T, H, d), qr) < tol
    for t, s in enumerate(slots):
        if s < 0:
            continue
        assert rel_err(kc[s // page, :, s % page].float().cpu(), kr[t]) < tol
        assert rel_err(vc[s // page, :, s % page].float().cpu(), k[t]) < tol       # the value: the key before its rotation
    used = {s for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in used:
            assert float(kc[s // page, :, s % page].abs().max()) == 0.0 and float(vc[s // page, :, s % page].abs().max()) == 0.0


# ----------------------------------------------------------------------------- attention with mixed heads

def _oracle(q, k, v, pos, qmul, talk, sink, window, gate):
    """q [n, H, d] (the last n tokens), k, v [L, G, d], pos [n] -> [n, H * d]."""
    L, (n, H, d), G = k.shape[0], q.shape, k.shape[1]
    raw = torch.stack([q[:, h] @ k[:, h // (H // G)].T for h in range(H)]) * qmul[:, None, None]
    s = torch.einsum("hg,gij->hij", talk, raw) if talk is not None else raw
    i, j = torch.tensor(pos)[:, None], torch.arange(L)[None, :]
    ok = (j <= i) & ((i - j < window) if window else True)
    sk = sink if sink is not None else torch.full((H,), -math.inf, dtype=torch.float64)
    p = plain.softmax_with_sink(s, ok, sk)
    o = torch.stack([p[h] @ v[:, h // (H // G)] for h in range(H)], dim=1)
    if gate is not None:
        o = o * torch.sigmoid(gate)[:, :, None]
    return o.reshape(n, H * d)


class _Step:
    """Requests with keys and values already in a paged cache (pages scattered over the pool, stale numbers in the
    pages' unused slots), and a step that brings the last ``n`` tokens of each."""

    def __init__(self, lengths, counts, H, G, d, page, dtype, seed, std=1.0):
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.counts, self.dims, self.page, self.dtype = lengths, counts, (H, G, d), page, dtype
        S = len(lengths)
        per = max(-(-L // page) for L in lengths) + 1
        order = torch.randperm(S * per, generator=g).tolist()
        self.k = [(std * torch.randn(L, G, d, generator=g)).to(dtype) for L in lengths]
        self.v = [torch.randn(L, G, d, generator=g).to(dtype) for L in lengths]
        self.q = [(std * torch.randn(n, H, d, generator=g)).to(dtype) for n in counts]
        self.gate = [2 * torch.randn(n, H, generator=g) for n in counts]
        self.kc = (100.0 * torch.randn(S * per, G, page, d, generator=g)).to(dtype)
        self.vc = (100.0 * torch.randn(S * per, G, page, d, generator=g)).to(dtype)
        self.table = [[order[s * per + i] if i * page < lengths[s] else -1 for i in range(per)] for s in range(S)]
        self.pos = [list(range(L - n, L)) for L, n in zip(lengths, counts)]

    def run(self, window, qmul, talk, sink, use_gate, splits=1, mma=False):
        from photon_infer_b200.kernels import ops
        H, G, d = self.dims
        for s, L in enumerate(self.lengths):
            for p in range(L):
                pg = self.table[s][p // self.page]
                self.kc[pg, :, p % self.page] = self.k[s][p]
                self.vc[pg, :, p % self.page] = self.v[s][p]
        width = max(8, -(-len(self.table[0]) // 8) * 8)
        bt = i32([row + [-1] * (width - len(row)) for row in self.table])
        pos = i32([p for ps in self.pos for p in ps])
        seq = i32([s for s, n in enumerate(self.counts) for _ in range(n)])
        q = torch.cat(self.q).reshape(-1, H * d).to(DEV)
        out = torch.full(q.shape, float("nan"), dtype=self.dtype, device=DEV)
        gate = None
        if use_gate:
            wide = torch.zeros(q.shape[0], H + 5, dtype=torch.float32, device=DEV)       # a view with a row stride
            wide[:, 3:3 + H] = torch.cat(self.gate).to(DEV)
            gate = wide[:, 3:3 + H]
        err = torch.zeros(4, dtype=torch.int32, device=DEV)
        f = lambda t: None if t is None else t.float().contiguous().to(DEV)
        if mma:
            assert ops.talk_mma_supported(H, G, d)
            cu = i32([sum(self.counts[:s]) for s in range(len(self.counts) + 1)])
            ops.talk_attention_mma(q, out, self.kc.to(DEV), self.vc.to(DEV), bt, cu, pos, len(self.counts), max(self.counts), H, G, d,
                                   window, f(qmul), f(talk), f(sink), gate, err, splits=splits)
        else:
            ops.talk_attention(q, out, self.kc.to(DEV), self.vc.to(DEV), bt, seq, pos, H, G, d, window, f(qmul), f(talk), f(sink), gate,
                               err, splits=splits)
        torch.cuda.synchronize()
        assert err.cpu().tolist()[0] == 0
        return out.float().cpu()

    def want(self, window, qmul, talk, sink, use_gate):
        d64 = lambda t: None if t is None else t.double()
        return torch.cat([_oracle(self.q[s].double(), self.k[s].double(), self.v[s].double(), self.pos[s], qmul.double(), d64(talk),
                                  d64(sink), window, self.gate[s].double() if use_gate else None) for s in range(len(self.lengths))])


# a whole short prompt, the end of a long one, single decoded tokens near and far, two tokens, the very first token
LENGTHS, COUNTS = [33, 150, 97, 200, 1, 300], [33, 50, 1, 2, 1, 1]
RULES = [dict(window=None, talk=True, sink=True, gate=True), dict(window=24, talk=True, sink=False, gate=False),
         dict(window=3, talk=False, sink=True, gate=True), dict(window=70, talk=True, sink=True, gate=False),
         dict(window=64, talk=True, sink=True, gate=True), dict(window=1, talk=True, sink=True, gate=True)]


@pytest.mark.parametrize("rule", RULES, ids=lambda r: f"w{r['window']}t{int(r['talk'])}s{int(r['sink'])}g{int(r['gate'])}")
@pytest.mark.parametrize("heads", [(2, 1), (6, 2), (2, 2), (8, 1), (5, 5), (1, 1)])
@pytest.mark.parametrize("dtype,d,page", [(torch.float32, 10, 8), (torch.float32, 64, 16), (torch.bfloat16, 24, 16), (torch.bfloat16, 128, 32),
                                          (torch.float32, 256, 16)])
def test_attention_with_mixed_heads(rule, heads, dtype, d, page):
    H, G = heads
    st = _Step(LENGTHS, COUNTS, H, G, d, page, dtype, seed=H * 100 + d, std=1.0 if d < 64 else 0.5)
    g = torch.Generator().manual_seed(H)
    qmul = (0.5 + torch.rand(H, generator=g)) / math.sqrt(d)
    talk = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)) if rule["talk"] else None
    sink = torch.randn(H, generator=g) if rule["sink"] else None
    got = st.run(rule["window"], qmul, talk, sink, rule["gate"])
    want = st.want(rule["window"], qmul, talk, sink, rule["gate"])
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("rule", RULES, ids=lambda r: f"w{r['window']}t{int(r['talk'])}s{int(r['sink'])}g{int(r['gate'])}")
@pytest.mark.parametrize("heads", [(2, 1), (6, 2), (8, 1), (5, 5), (1, 1), (16, 2), (12, 4), (20, 5)])
@pytest.mark.parametrize("d,page", [(16, 8), (64, 16), (128, 32), (48, 24)])
def test_attention_with_mixed_heads_on_the_tensor_cores(rule, heads, d, page):
    """The bfloat16 kernel that owns 16 tokens with all their heads: portions that end inside a tile of 16 rows, single
    tokens, the first token, pages smaller than a key tile and pages that do not divide it."""
    from photon_infer_b200.kernels import ops
    H, G = heads
    if not ops.talk_mma_supported(H, G, d):
        pytest.skip("the general kernel takes these sizes")
    st = _Step(LENGTHS, COUNTS, H, G, d, page, torch.bfloat16, seed=H * 100 + d, std=1.0 if d < 64 else 0.5)
    g = torch.Generator().manual_seed(H)
    qmul = (0.5 + torch.rand(H, generator=g)) / math.sqrt(d)
    talk = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)) if rule["talk"] else None
    sink = torch.randn(H, generator=g) if rule["sink"] else None
    got = st.run(rule["window"], qmul, talk, sink, rule["gate"], mma=True)
    assert rel_err(got, st.want(rule["window"], qmul, talk, sink, rule["gate"])) < 2e-2


def test_the_tensor_core_kernel_accepts_what_it_can_hold():
    from photon_infer_b200.kernels import ops
    assert ops.talk_mma_supported(16, 2, 128) and ops.talk_mma_supported(8, 2, 256) and ops.talk_mma_supported(32, 4, 64)
    assert not ops.talk_mma_supported(4, 2, 24) and not ops.talk_mma_supported(32, 4, 128) and not ops.talk_mma_supported(6, 4, 64)


@pytest.mark.parametrize("dtype,mma", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("splits", [2, 5, 64])
@pytest.mark.parametrize("window", [None, 130, 40])
def test_attention_with_keys_split_over_blocks(dtype, mma, splits, window):
    st = _Step([300, 7, 129, 1], [1, 1, 1, 1], 6, 3, 32, 16, dtype, seed=splits)
    g = torch.Generator().manual_seed(3)
    qmul, talk, sink = torch.full((6,), 0.2), torch.eye(6) + 0.3 * torch.randn(6, 6, generator=g), torch.randn(6, generator=g)
    got = st.run(window, qmul, talk, sink, True, splits=splits, mma=mma)
    assert rel_err(got, st.want(window, qmul, talk, sink, True)) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype,d,page,mma", [(torch.float32, 12, 8, False), (torch.bfloat16, 64, 16, False), (torch.bfloat16, 64, 16, True),
                                              (torch.bfloat16, 32, 8, True)])
@pytest.mark.parametrize("count,splits", [(1, 1), (40, 1), (1, 4)])
def test_keys_that_stand_out_at_every_edge(dtype, d, page, mma, count, splits):
    """Random keys score about 0.  One key at a time is made to score high in head 1 for the LAST token of a request of
    333 tokens (decoded alone, or the end of a portion of 40).  Head 0 listens to head 1 alone (``talk``), so it must
    bring that key's value where the window lets the token see it, and must not where it does not."""
    L, window = 333, 96
    i = L - 1
    places = {"far": (1, None), "first_token": (0, None), "window_first": (i - window + 1, window), "window_behind": (i - window, window),
              "self": (i, window), "page_low": ((i - 40) // page * page - 1, window), "page_high": ((i - 40) // page * page, window)}
    talk = torch.tensor([[0.0, 1.0], [0.0, 1.0]])                     # both heads take head 1's score
    for name, (j, w) in places.items():
        st = _Step([L, 50], [count, 1], 2, 2, d, page, dtype, seed=len(name), std=0.05)
        qdir = st.q[0][-1, 1].double()
        st.k[0][j, 1] = (qdir / qdir.norm() * 40.0).to(dtype)          # this key's score with head 1 of the last token: large
        st.v[0][j, 0] = torch.full((d,), 7.0).to(dtype)                # head 0 reads its own key/value head's value there
        qmul = torch.full((2,), 1.0 / float(qdir.norm()))
        sink = torch.tensor([0.5, -0.5])
        got = st.run(w, qmul, talk, sink, False, splits=splits, mma=mma)
        want = st.want(w, qmul, talk, sink, False)
        assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 2e-2), name
        row = got[count - 1, :d]
        if w is None or i - j < w:
            assert float((row - 7.0).abs().max()) < 0.1, f"{name}: key {j} must be seen"
        else:
            assert float(row.abs().max()) < 3.0, f"{name}: key {j} must not be seen"


def test_a_sink_that_outweighs_every_key():
    """A large sink takes nearly all of the softmax's mass and has no value: the output shrinks towards zero."""
    st = _Step([40], [40], 2, 1, 16, 8, torch.float32, seed=1)
    qmul = torch.full((2,), 0.25)
    got = st.run(None, qmul, None, torch.tensor([30.0, -30.0]), False)
    assert rel_err(got, st.want(None, qmul, None, torch.tensor([30.0, -30.0]), False)) < 1e-5
    assert float(got[:, :16].abs().max()) < 1e-6 and float(got[:, 16:].abs().max()) > 0.05


# ----------------------------------------------------------------------------- the mixers in portions and batches

def _ctx(dtype, pos_lists, slots, tables, page, num_pages):
    """A step that brings the tokens at ``pos_lists[s]`` of request s (state slot ``slots[s]``, pages ``tables[s]``)."""
    from photon_infer_b200.parts.base import GroupView, StepContext
    counts = [len(p) for p in pos_lists]
    T, S = sum(counts), len(counts)
    cu = [0]
    for n in counts:
        cu.append(cu[-1] + n)
    pos = [p for ps in pos_lists for p in ps]
    seq = [s for s, n in enumerate(counts) for _ in range(n)]
    width = max(8, max(len(t) for t in tables))
    bt = [list(t) + [-1] * (width - len(t)) for t in tables]
    slot_map = [tables[s][p // page] * page + p % page for s, ps in enumerate(pos_lists) for p in ps]
    ends = [ps[-1] + 1 for ps in pos_lists]
    return StepContext(T, S, dtype, i32([0] * T), i32(pos), i32(seq), i32(cu), i32(ends), i32(slots),
                       [GroupView(i32(bt), i32(slot_map), page, num_pages, width)], counts, ends, [ps[0] for ps in pos_lists],
                       max(counts), max(ends), torch.zeros(4, dtype=torch.int32, device=DEV), host_state_slots=list(slots))


ATT_SHAPES = [dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.11, mask=dict(size=24), rot=dict(base=5000.0, dims=16)),
              dict(heads=3, kv_heads=1, dim=10, vdim=10, scale=0.3, mask=dict(size=7), rot=dict(base=100.0, dims=10)),
              dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.08)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", ATT_SHAPES, ids=lambda m: f"h{m['heads']}d{m['dim']}")
def test_attention_mixer_in_portions_and_batches(dtype, m):
    """Two requests of unequal length through the mixer, cut differently (one in portions of 30, 2, 1, 1, 17, 1 tokens,
    the other whole in the second step and then left out), against the plain mixer over each whole sequence."""
    import types
    from photon_infer_b200.models.lerosun import _mixer
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    W = 48
    spec = _mixer(types.SimpleNamespace(width=W, norm_eps=1e-5), "attention", m)
    att = create_part("mixer", spec.kind, spec.params)
    g = torch.Generator().manual_seed(5)
    H = m["heads"]
    w = _weights(att, dtype, 0.3, 5, overrides={"talk": torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)})
    n, n2, page = 52, 21, 16
    h = [torch.randn(n, W, generator=g).to(dtype), torch.randn(n2, W, generator=g).to(dtype)]
    want = [plain.attention_mixer(x.double(), w, "", m, torch.arange(x.shape[0])) for x in h]
    tables = [[5, 0, 3, 6], [2, 4]]
    cs = att.cache_spec()
    kc = torch.zeros(8, cs.n_kv_heads, page, cs.head_dim, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    got, p = [[], []], 0
    for step, cnt in enumerate((30, 2, 1, 1, 17, 1)):
        pos_lists, slots, tabs, xs = [list(range(p, p + cnt))], [0], [tables[0]], [h[0][p:p + cnt]]
        if step == 1:                                               # the second request joins for one step, first in the batch
            pos_lists, slots, tabs, xs = [list(range(n2))] + pos_lists, [1, 0], [tables[1], tables[0]], [h[1]] + xs
        ctx = _ctx(dtype, pos_lists, slots, tabs, page, 8)
        out = att.forward(torch.cat(xs).to(DEV), ctx, LayerCache(group=0, k=kc, v=vc)).float().cpu()
        assert ctx.error_flag.cpu().tolist()[0] == 0
        if step == 1:
            got[1].append(out[:n2])
            out = out[n2:]
        got[0].append(out)
        p += cnt
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    assert rel_err(torch.cat(got[0]), want[0]) < tol and rel_err(torch.cat(got[1]), want[1]) < tol


DELTA_SHAPES = [dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=4), dict(heads=3, kv_heads=3, dim=9, vdim=33, conv=7),
                dict(heads=2, kv_heads=1, dim=128, vdim=128, conv=2), dict(heads=1, kv_heads=1, dim=72, vdim=40, conv=1),
                dict(heads=2, kv_heads=2, dim=64, vdim=8, conv=3), dict(heads=1, kv_heads=1, dim=256, vdim=16, conv=4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m", DELTA_SHAPES, ids=lambda m: f"h{m['heads']}d{m['dim']}v{m['vdim']}c{m['conv']}")
def test_delta_mixer_in_portions_batches_and_reused_slots(dtype, m):
    """Three requests through the mixer in one state tensor of two slots.  The first runs in portions of 30, 2, 1, 1,
    17, 1 tokens (portions shorter than the convolution's reach among them); the second runs whole beside the first's
    second portion and ends; the third then takes the second's slot, which the pool hands out cleared, and runs
    token by token.  Each must equal the plain mixer over its whole sequence."""
    import types
    from photon_infer_b200.cache.state_slots import StateSlotPool
    from photon_infer_b200.models.lerosun import _mixer
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    W = 40
    spec = _mixer(types.SimpleNamespace(width=W, norm_eps=1e-5), "delta", m)
    mix = create_part("mixer", spec.kind, spec.params)
    g = torch.Generator().manual_seed(7)
    w = _weights(mix, dtype, 0.4, 7)
    lens = (52, 21, 4)
    h = [torch.randn(n, W, generator=g).to(dtype) for n in lens]
    want = [plain.delta_mixer(x.double(), w, m, 1e-5) for x in h]
    pool = StateSlotPool(2, {0: mix.state_spec()}, torch.device(DEV))
    state = pool.tensors[0]
    slot_a = pool.allocate("a")
    got, p = [[], [], []], 0
    for step, cnt in enumerate((30, 2, 1, 1, 17, 1)):
        pos_lists, slots, xs, who = [list(range(p, p + cnt))], [slot_a], [h[0][p:p + cnt]], [0]
        if step == 1:
            slot_b = pool.allocate("b")
            pos_lists, slots, xs, who = [list(range(lens[1]))] + pos_lists, [slot_b, slot_a], [h[1]] + xs, [1, 0]
        if step >= 2 and step - 2 < lens[2]:
            if step == 2:
                pool.free("b")
                assert pool.allocate("c") == slot_b               # the slot of the request that ended, cleared
            t = step - 2
            pos_lists, slots, xs, who = pos_lists + [[t]], slots + [slot_b], xs + [h[2][t:t + 1]], who + [2]
        ctx = _ctx(dtype, pos_lists, slots, [[0]] * len(slots), 64, 1)
        out = mix.forward(torch.cat(xs).to(DEV), ctx, LayerCache(state=state)).float().cpu()
        assert ctx.error_flag.cpu().tolist()[0] == 0
        at = 0
        for r, ps in zip(who, pos_lists):
            got[r].append(out[at:at + len(ps)])
            at += len(ps)
        p += cnt
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for r in range(3):
        assert rel_err(torch.cat(got[r]), want[r]) < tol, f"request {r}"


def test_a_negative_state_slot_starts_from_zero_and_stores_nothing():
    import types
    from photon_infer_b200.models.lerosun import _mixer
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    m = dict(heads=2, kv_heads=1, dim=16, vdim=8, conv=3)
    spec = _mixer(types.SimpleNamespace(width=24, norm_eps=1e-5), "delta", m)
    mix = create_part("mixer", spec.kind, spec.params)
    w = _weights(mix, torch.float32, 0.4, 2)
    h = torch.randn(5, 24, generator=torch.Generator().manual_seed(2))
    state = torch.full((2, mix.state_spec().shape[0]), 3.0, device=DEV)
    ctx = _ctx(torch.float32, [list(range(5))], [-1], [[0]], 64, 1)
    out = mix.forward(h.to(DEV), ctx, LayerCache(state=state)).cpu()
    assert rel_err(out, plain.delta_mixer(h.double(), w, m, 1e-5)) < 3e-5
    assert bool((state == 3.0).all())


def test_a_write_far_back_is_read_after_hundreds_of_tokens():
    """The delta rule with decay 1 and beta 1 stores v under the unit key k and reads it back with q = k: one token
    writes a marker, 300 tokens with other (orthogonal) keys follow, and the last token asks for the marker."""
    from photon_infer_b200.kernels import ops
    T, dim, vdim = 302, 32, 16
    y = torch.zeros(T, 2 * dim + vdim)
    e = torch.eye(dim)
    for t in range(T):
        y[t, dim:2 * dim] = e[1 + t % (dim - 1)]                   # keys: unit vectors 1 .. dim - 1, never 0
        y[t, :dim] = e[1 + (t + 5) % (dim - 1)]
        y[t, 2 * dim:] = 0.01 * t
    y[3, dim:2 * dim] = e[0]
    y[3, 2 * dim:] = 7.0                                           # the marker, under key 0
    y[T - 1, :dim] = e[0]                                          # the last token asks for key 0
    ab = torch.zeros(T, 2)
    ab[:, 0] = -100.0                                              # softplus(-100 + 0) = 0: no decay
    ab[:, 1] = 100.0                                               # beta = 1
    state = torch.zeros(1, dim * vdim, device=DEV)
    o = torch.empty(T, vdim, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.delta_recurrent(y.to(DEV), ab.to(DEV), torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), i32([0, T]), i32([0]), state, o,
                        1, 1, 1, dim, vdim, err)
    assert err.cpu().tolist()[0] == 0
    assert float((o[T - 1].cpu() - 7.0).abs().max()) < 1e-4
    want = plain.delta_rule(y[:, None, :dim].double(), y[:, None, dim:2 * dim].double(), y[:, None, 2 * dim:].double(),
                            torch.ones(T, 1, dtype=torch.float64), torch.ones(T, 1, dtype=torch.float64))
    assert rel_err(o.cpu(), want[:, 0]) < 1e-5
