"""Each mechanism of the Pebodra decoder alone, on the device, against its plain function: the RMS norm in groups (as
a norm of rows, and on a sublayer's output with the residual sum and the rounded copy of the stream); the gate before
and behind a norm; the PolyNorm feed-forward; the sigmoid router with groups scored by their two best experts; bias,
per-map norm, partial rotation and the cache write of differential attention; the attention itself over a paged
cache (pages scattered, stale numbers in unused slots) with keys made to stand out far back, just inside and just
outside the window, at both sides of a page border and at the start of the sequence, in prompts and in decoding, for
each of the two maps; the short convolution with its rows carried between steps; the two recurrences with their
state carried between steps in portions down to one token, in batches of unequal requests, and in slots that are
used again; and the block that puts the norms on the sublayers' outputs."""
import math

import pytest
import torch

from helpers import rel_err
from plain import pebodra_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
F64 = torch.float64


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


# ----------------------------------------------------------------------------- norms

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups", [(72, 4), (50, 5), (1024, 1), (96, 16), (60, 60), (336, 2)])
def test_group_norm_of_rows_and_on_a_sublayer_s_output(dtype, width, groups):
    from photon_infer_b200.parts.registry import create_part
    g = torch.Generator().manual_seed(width + groups)
    norm = create_part("norm", "group_rms_norm", {"size": width, "eps": 1e-5, "groups": groups, "weight_name": "w"})
    w = (1.0 + 0.3 * torch.randn(width, generator=g)).to(dtype)
    norm.load({"w": w.to(DEV)})
    x = 2 * torch.randn(6, width, generator=g)
    a = (3 * torch.randn(6, width, generator=g)).to(dtype)
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    alone = norm.forward(a.to(DEV), torch.float32)
    want = plain.group_rms_norm(a.double(), w.double(), groups, 1e-5)
    assert alone.dtype == torch.float32 and rel_err(alone.cpu(), want) < 3e-6
    res = x.to(DEV).clone()
    h = norm.add_normed(a.to(DEV), res, dtype)
    assert rel_err(res.cpu(), x.double() + want) < 3e-6
    assert h.dtype == dtype and rel_err(h.float().cpu(), x.double() + want) < tol
    if dtype == torch.float32:
        assert h.data_ptr() == res.data_ptr()              # the 32-bit run reads the stream itself
    # nothing pending: the stream's rows in the run type
    h0 = norm.add_normed(None, x.to(DEV).clone(), dtype)
    assert torch.equal(h0.cpu(), x.to(dtype))
    # the model's last norm on chosen rows, with an output that still waits for its own norm
    from photon_infer_b200.parts.base import Normed
    res2 = x.to(DEV).clone()
    out = norm.add_forward_rows(Normed(a.to(DEV), norm), res2, i32([4, 1]), dtype)
    assert torch.equal(res2.cpu(), x)
    want_rows = plain.group_rms_norm((x.double() + want)[[4, 1]], w.double(), groups, 1e-5)
    assert rel_err(out.float().cpu(), want_rows) < tol


@pytest.mark.parametrize("mode", ["silu_before", "sigmoid_after"])
@pytest.mark.parametrize("width,groups", [(64, 2), (33, 3), (512, 16), (192, 1)])
def test_gate_before_and_behind_the_norm(mode, width, groups):
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    o, w = torch.randn(5, width, generator=g), 1.0 + 0.2 * torch.randn(width, generator=g)
    rows = torch.randn(5, width + 10, generator=g)          # the gate is a section of a wider row
    z = rows[:, 3:3 + width]
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
        out = torch.empty(5, width, dtype=dtype, device=DEV)
        ops.group_rmsnorm(o.to(DEV), w.to(DEV), 1e-6, groups, out=out, gate=rows.to(DEV)[:, 3:3 + width], gate_mode=mode)
        if mode == "silu_before":
            want = plain.group_rms_norm(o.double() * z.double() * torch.sigmoid(z.double()), w.double(), groups, 1e-6)
        else:
            want = plain.group_rms_norm(o.double(), w.double(), groups, 1e-6) * torch.sigmoid(z.double())
        assert rel_err(out.float().cpu(), want) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H,ff", [(3, 64, 96), (40, 50, 70), (300, 128, 512), (1, 256, 1024)])
def test_polynorm_feed_forward(dtype, rows, H, ff):
    from photon_infer_b200.parts.registry import create_part
    part = create_part("feed_forward", "polynorm", dict(hidden_size=H, intermediate_size=ff, eps=1e-6))
    w = _weights(part, dtype, 0.2, rows, {"act": torch.tensor([0.7, -0.4, 0.25, 0.1])})
    h = torch.randn(rows, H, generator=torch.Generator().manual_seed(1)).to(dtype)
    got = part.forward(h.to(DEV), None).float().cpu()
    assert rel_err(got, plain.dense_ff(h.double(), w, 1e-6)) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_polynorm_alone():
    from photon_infer_b200.kernels import ops
    z = 3 * torch.randn(7, 45, generator=torch.Generator().manual_seed(3))
    coef = torch.tensor([1.5, 0.5, -0.125, 2.0])
    out = torch.empty(7, 45, dtype=torch.float32, device=DEV)
    ops.polynorm(z.to(DEV), coef.to(DEV), 1e-5, out)
    assert rel_err(out.cpu(), plain.polynorm(z.double(), coef.double(), 1e-5)) < 3e-6


def test_bounded_logits():
    from photon_infer_b200.kernels import ops
    x = torch.linspace(-200, 200, 1001)
    y = x.to(DEV).clone()
    ops.softcap_(y, 25.0)
    assert rel_err(y.cpu(), 25.0 * torch.tanh(x.double() / 25.0)) < 1e-6


# ----------------------------------------------------------------------------- router

@pytest.mark.parametrize("E,top,groups", [(8, 2, (2, 1)), (6, 2, (3, 2)), (5, 3, (5, 3)), (40, 4, (8, 3)), (4, 1, None), (12, 3, (2, 2))])
def test_sigmoid_router_with_groups(E, top, groups):
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(E)
    h, wr = torch.randn(200, 48, generator=g), 0.5 * torch.randn(E, 48, generator=g)
    r = dict(experts=E, top=top)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    ids, weights, counts = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, "sigmoid", groups[0] if groups else 1,
                                         groups[1] if groups else 1, 1.0)
    chosen, weight = plain.route(h.double(), wr.double(), r)
    assert torch.equal(ids.long().cpu().sort(dim=1).values, chosen.sort(dim=1).values)
    got = torch.zeros(200, E, dtype=F64).scatter_(1, ids.long().cpu(), weights.double().cpu())
    want = torch.zeros(200, E, dtype=F64).scatter_(1, chosen, weight)
    assert rel_err(got, want) < 1e-6                       # the scores themselves, not divided by their sum
    assert counts.cpu().tolist() == torch.bincount(chosen.flatten(), minlength=E).tolist()


def test_a_group_is_scored_by_its_two_best_experts():
    """Group 0 holds the single best expert, group 1 the better pair: the pair wins."""
    from photon_infer_b200.kernels import ops
    wr = torch.zeros(6, 4)
    wr[0, 0], wr[1, 0], wr[2, 0] = 3.0, -3.0, -3.0          # group 0: one high score, two low ones
    wr[3, 0], wr[4, 0], wr[5, 0] = 1.5, 1.4, -3.0           # group 1: two good ones
    h = torch.tensor([[1.0, 0, 0, 0]])
    ids, weights, _ = ops.moe_route(h.to(DEV), wr.to(DEV), None, 2, "sigmoid", 2, 1, 1.0)
    assert sorted(ids.cpu().tolist()[0]) == [3, 4]
    assert rel_err(weights.cpu().sort().values, torch.sigmoid(torch.tensor([[1.4, 1.5]], dtype=F64))) < 1e-6


# ----------------------------------------------------------------------------- differential attention: what is cached

@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [dict(H=4, G=2, d=16, dv=24, rot=8), dict(H=3, G=1, d=10, dv=10, rot=10), dict(H=2, G=2, d=64, dv=128, rot=32),
                                   dict(H=5, G=5, d=6, dv=3, rot=0)])
def test_bias_norm_rotation_and_cache_write(out_dtype, shape):
    from photon_infer_b200.kernels import ops
    H, G, d, dv, rot = (shape[k] for k in ("H", "G", "d", "dv", "rot"))
    g = torch.Generator().manual_seed(d)
    T, page, pages = 9, 4, 6
    nq, nk, nv = H * 2 * d, G * 2 * d, G * dv
    rows = torch.randn(T, nq + nk + nv + 5, generator=g)                             # sections of a wider row
    qb, kb, vb = (torch.randn(n, generator=g) for n in (nq, nk, nv))
    qw, kw = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    pos = [0, 1, 2, 700, 3, 4, 12345, 5, 6]
    slots = [3, 7, -1, 20, 0, 23, 9, 10, 15]
    inv = torch.tensor([1e4 ** (-2.0 * j / rot) for j in range(rot // 2)], dtype=F64) if rot else None
    kc = torch.zeros(pages, G, page, 2 * d, dtype=out_dtype, device=DEV)
    vc = torch.zeros(pages, G, page, dv, dtype=out_dtype, device=DEV)
    q_out = torch.empty(T, nq, dtype=out_dtype, device=DEV)
    rd = rows.to(DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.diff_prep(rd[:, :nq], rd[:, nq:nq + nk], rd[:, nq + nk:nq + nk + nv], q_out, qb.to(DEV), kb.to(DEV), vb.to(DEV), qw.to(DEV),
                  kw.to(DEV), 1e-5, i32(pos), inv.to(DEV) if rot else None, rot, i32(slots), kc, vc, H, G, d, dv, err)
    assert err.cpu().tolist()[0] == 0
    P = torch.tensor(pos)
    q = plain.rotate_first_dims(plain.unit_rms((rows[:, :nq].double() + qb.double()).reshape(T, H, 2, d), 1e-5) * qw.double(), P, rot, 1e4)
    k = plain.rotate_first_dims(plain.unit_rms((rows[:, nq:nq + nk].double() + kb.double()).reshape(T, G, 2, d), 1e-5) * kw.double(), P, rot, 1e4)
    v = (rows[:, nq + nk:nq + nk + nv].double() + vb.double()).reshape(T, G, dv)
    tol = 3e-6 if out_dtype == torch.float32 else 5e-3
    assert rel_err(q_out.float().cpu().reshape(T, H, 2, d), q) < tol
    for t, s in enumerate(slots):
        if s < 0:
            continue
        assert rel_err(kc[s // page, :, s % page].float().cpu().reshape(G, 2, d), k[t]) < tol
        assert rel_err(vc[s // page, :, s % page].float().cpu(), v[t]) < tol
    used = {s for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in used:
            assert float(kc[s // page, :, s % page].abs().max()) == 0.0 and float(vc[s // page, :, s % page].abs().max()) == 0.0
    # a layer that reads another layer's pages: queries only
    q2 = torch.empty_like(q_out)
    ops.diff_prep(rd[:, :nq], None, None, q2, qb.to(DEV), None, None, qw.to(DEV), None, 1e-5, i32(pos), inv.to(DEV) if rot else None, rot,
                  None, None, None, H, G, d, dv, err)
    assert torch.equal(q2, q_out)


# ----------------------------------------------------------------------------- differential attention over the cache

class _Cached:
    """Requests whose keys and values lie in a paged cache (pages scattered over the pool, stale numbers in the unused
    slots), and a step that brings the last ``counts[s]`` tokens of each."""

    def __init__(self, lengths, counts, H, G, d, dv, page, dtype, seed, std=1.0):
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.counts, self.dims, self.page, self.dtype = lengths, counts, (H, G, d, dv), page, dtype
        self.k = [(std * torch.randn(L, G, 2, d, generator=g)).to(dtype) for L in lengths]
        self.v = [torch.randn(L, G, dv, generator=g).to(dtype) for L in lengths]
        self.q = [(std * torch.randn(n, H, 2, d, generator=g)).to(dtype) for n in counts]

    def run(self, window, scale, lam, diff, eps=1e-5, mma=False, splits=1):
        from photon_infer_b200.kernels import ops
        H, G, d, dv = self.dims
        page = self.page
        per = [-(-L // page) for L in self.lengths]
        total = sum(per) + 3
        order = torch.randperm(total, generator=torch.Generator().manual_seed(7)).tolist()
        kc = (9 * torch.randn(total, G, page, 2 * d)).to(self.dtype)
        vc = (9 * torch.randn(total, G, page, dv)).to(self.dtype)
        table = torch.full((len(self.lengths), max(per) + 2), -1, dtype=torch.int32)
        at = 0
        for s, L in enumerate(self.lengths):
            for i in range(per[s]):
                table[s, i] = order[at]
                at += 1
            for j in range(L):
                kc[table[s, j // page], :, j % page] = self.k[s][j].reshape(G, 2 * d)
                vc[table[s, j // page], :, j % page] = self.v[s][j]
        q = torch.cat([x.reshape(x.shape[0], H * 2 * d) for x in self.q]).to(DEV)
        tseq = [s for s, n in enumerate(self.counts) for _ in range(n)]
        pos = [L - n + i for L, n in zip(self.lengths, self.counts) for i in range(n)]
        out = torch.empty(q.shape[0], H * dv, dtype=self.dtype, device=DEV)
        err = torch.zeros(4, dtype=torch.int32, device=DEV)
        if mma:
            assert ops.diff_mma_supported(self.dtype, H, G, d, dv)
            cu = [0]
            for n in self.counts:
                cu.append(cu[-1] + n)
            ops.diff_attention_mma(q, out, kc.to(DEV), vc.to(DEV), table.to(DEV), i32(cu), i32(pos), self.counts, H, G, d, dv, window,
                                   scale, lam, 1.0 - diff, eps, err, splits=splits)
        else:
            ops.diff_attention(q, out, kc.to(DEV), vc.to(DEV), table.to(DEV), i32(tseq), i32(pos), H, G, d, dv, window, scale, lam,
                               1.0 - diff, eps, err)
        assert err.cpu().tolist()[0] == 0
        want = []
        for s, (L, n) in enumerate(zip(self.lengths, self.counts)):
            i, j = torch.arange(L - n, L)[:, None], torch.arange(L)[None, :]
            ok = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
            want.append(plain.difference_of_maps(self.q[s].double(), self.k[s].double(), self.v[s].double(), ok, scale, lam, diff, eps))
        return out.float().cpu(), torch.cat(want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,page,window", [(4, 2, 16, 24, 16, 40), (3, 1, 48, 80, 8, None), (2, 2, 64, 128, 32, 100), (5, 5, 6, 10, 16, 3),
                                                  (8, 1, 128, 128, 16, 130), (2, 1, 10, 7, 4, 33)])
def test_attention_prompts_decoding_and_batches(dtype, H, G, d, dv, page, window):
    lengths, counts = [150, 37, 64, 1, 200], [150, 1, 20, 1, 2]
    c = _Cached(lengths, counts, H, G, d, dv, page, dtype, seed=H * d, std=0.7)
    got, want = c.run(window, d ** -0.5, 0.37, 0.2)
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("H,G,d,dv,page,window", [(4, 2, 16, 32, 16, 40), (3, 1, 48, 80, 8, None), (2, 2, 64, 128, 32, 100), (5, 5, 32, 16, 16, 3),
                                                  (8, 1, 128, 128, 16, 130), (8, 2, 128, 256, 16, 70), (6, 2, 16, 48, 4, 33)])
def test_attention_on_the_tensor_cores(H, G, d, dv, page, window):
    lengths, counts = [150, 37, 64, 1, 200, 300], [150, 1, 20, 1, 2, 129]
    c = _Cached(lengths, counts, H, G, d, dv, page, torch.bfloat16, seed=H * d + 1, std=0.7)
    got, want = c.run(window, d ** -0.5, 0.37, 0.2, mma=True)
    assert rel_err(got, want) < 2e-2
    general, _ = c.run(window, d ** -0.5, 0.37, 0.2)
    assert rel_err(got, general.double()) < 2e-2


@pytest.mark.parametrize("splits", [2, 3, 7, 16])
@pytest.mark.parametrize("H,G,d,dv,page,window", [(4, 2, 16, 32, 16, 40), (8, 2, 128, 256, 16, None), (3, 1, 48, 80, 8, 300), (2, 2, 64, 128, 32, 100)])
def test_decoded_tokens_with_their_keys_shared_out_over_blocks(splits, H, G, d, dv, page, window):
    """Single tokens of requests of very different lengths (one key, a page, many tiles): shares without any key, shares
    of one tile and the merge in the order of the shares."""
    lengths = [700, 1, 64, 65, 17, 400, 129]
    c = _Cached(lengths, [1] * len(lengths), H, G, d, dv, page, torch.bfloat16, seed=splits + d, std=0.7)
    got, want = c.run(window, d ** -0.5, 0.4, 0.25, mma=True, splits=splits)
    assert rel_err(got, want) < 2e-2
    whole, _ = c.run(window, d ** -0.5, 0.4, 0.25, mma=True)
    assert rel_err(got, whole.double()) < 1e-2


@pytest.mark.parametrize("which_map", [0, 1])
def test_a_key_that_stands_out_when_the_keys_are_shared_out(which_map):
    H, G, d, dv, page, window, L = 2, 1, 32, 16, 16, 150, 430
    for place in (L - 1, L - window, L - window - 1, L - window + 1, 0, 300, 319, 320, 383, 384, 385):
        c = _Cached([L], [1], H, G, d, dv, page, torch.bfloat16, seed=place + 1, std=0.05)
        direction = torch.zeros(d)
        direction[3] = 4.0
        c.k[0][place, 0, which_map] = direction.bfloat16()
        c.q[0][-1, :, which_map] = (3 * direction).bfloat16()
        c.v[0][place] = 25.0
        got, want = c.run(window, 1.0, 0.6, 0.1, mma=True, splits=3)
        assert rel_err(got, want) < 3e-2, place


@pytest.mark.parametrize("which_map", [0, 1])
@pytest.mark.parametrize("count", [1, 30, 100])
def test_a_key_that_stands_out_at_every_edge_on_the_tensor_cores(which_map, count):
    H, G, d, dv, page, window, L = 2, 1, 32, 16, 16, 48, 230
    for place in (L - 1, L - 2, L - window, L - window - 1, L - window + 1, 0, 1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 181, 182, 183, 191, 192, 100):
        c = _Cached([L], [count], H, G, d, dv, page, torch.bfloat16, seed=place + 1, std=0.05)
        direction = torch.zeros(d)
        direction[3] = 4.0
        c.k[0][place, 0, which_map] = direction.bfloat16()
        c.q[0][-1, :, which_map] = (3 * direction).bfloat16()
        c.v[0][place] = 25.0
        got, want = c.run(window, 1.0, 0.6, 0.1, mma=True)
        assert rel_err(got, want) < 3e-2, place


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which_map", [0, 1])
@pytest.mark.parametrize("count", [1, 30])
def test_a_key_that_stands_out_at_every_edge(dtype, which_map, count):
    """One key of ONE map is made to match the last token's query of that map (all others are small), and its value is
    large.  Placed far back, just inside the window, just outside it, on both sides of a page border, and at the first
    positions of the sequence: the output must follow the oracle in every place, when the last tokens come as a prompt
    portion and when the last token is decoded alone."""
    H, G, d, dv, page, window, L = 2, 1, 32, 16, 16, 48, 230
    for place in (L - 1, L - 2, L - window, L - window - 1, L - window + 1, 0, 1, 2, 15, 16, 17, L - 33, L - 32, L - 31, 181, 182, 183, 100):
        c = _Cached([L], [count], H, G, d, dv, page, dtype, seed=place + 1, std=0.05)
        direction = torch.zeros(d)
        direction[3] = 4.0
        c.k[0][place, 0, which_map] = direction.to(dtype)
        c.q[0][-1, :, which_map] = (3 * direction).to(dtype)
        c.v[0][place] = 25.0
        got, want = c.run(window, 1.0, 0.6, 0.1)
        seen = 0 <= (L - 1) - place < window
        # the oracle's last row is dominated by the marked value exactly when the key is seen
        assert (float(want[-1].abs().max()) > 0) and rel_err(got, want) < (3e-5 if dtype == torch.float32 else 3e-2), (place, seen)


def test_the_two_maps_are_weighed_by_lambda():
    """With equal maps the head's output before its norm is (1 - lambda) a; lambda = 1 would leave nothing but rounding,
    so the kernel's use of lambda shows in the sign: lambda > 1 flips it."""
    H, G, d, dv = 1, 1, 8, 4
    c = _Cached([20], [20], H, G, d, dv, 4, torch.float32, seed=3)
    c.k[0][:, :, 1] = c.k[0][:, :, 0]
    c.q[0][:, :, 1] = c.q[0][:, :, 0]
    a, _ = c.run(None, 0.3, 0.25, 0.0)
    b, _ = c.run(None, 0.3, 1.75, 0.0)
    assert rel_err(a, -b.double()) < 1e-5


# ----------------------------------------------------------------------------- short convolution

@pytest.mark.parametrize("taps,C", [(4, 100), (1, 33), (7, 260), (2, 5)])
def test_convolution_carries_its_rows_between_steps(taps, C):
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(taps * C)
    lengths = [23, 9, 40]
    x = [torch.randn(L, C + 6, generator=g) for L in lengths]
    w, b = 0.5 * torch.randn(C, taps, generator=g), 0.2 * torch.randn(C, generator=g)
    want = [plain.short_conv_silu(xx[:, 2:2 + C].double(), w.double(), b.double()) for xx in x]
    offset = 17
    state = torch.zeros(4, offset + (taps - 1) * C + 3, device=DEV)
    state[:, :offset] = 5.0                                     # what lies before the rows is someone else's
    slots = [2, 0, 3]
    done = [0, 0, 0]
    got = [[] for _ in lengths]
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    for sizes in ([5, 9, 1], [1, 0, 2], [2, 0, 30], [15, 0, 7]):
        live = [s for s in range(3) if sizes[s] > 0]
        rows = torch.cat([x[s][done[s]:done[s] + sizes[s]] for s in live]).to(DEV)
        cu = [0]
        for s in live:
            cu.append(cu[-1] + sizes[s])
        tseq = [i for i, s in enumerate(live) for _ in range(sizes[s])]
        y = torch.empty(rows.shape[0], C, dtype=torch.float32, device=DEV)
        ops.conv_silu(rows[:, 2:2 + C], w.to(DEV), b.to(DEV), i32(tseq), i32(cu), i32([slots[s] for s in live]), state, offset, y,
                      len(live), err)
        for i, s in enumerate(live):
            got[s].append(y[cu[i]:cu[i + 1]].cpu())
            done[s] += sizes[s]
    assert err.cpu().tolist()[0] == 0 and done == lengths
    for s in range(3):
        assert rel_err(torch.cat(got[s]), want[s]) < 3e-6
    assert float((state[:, :offset] - 5.0).abs().max()) == 0.0 and float(state[1].abs()[offset:].max()) == 0.0


# ----------------------------------------------------------------------------- the two recurrences

def _portions(total, sizes):
    out, p, i = [], 0, 0
    while p < total:
        n = min(sizes[i % len(sizes)], total - p)
        out.append(n)
        p += n
        i += 1
    return out


def _run_recurrence(mode, H, Gq, N, dv, lengths, cuts, seed, slots_total=3):
    """Three requests walk through ``ops.linrec`` in portions (a request with nothing left drops out; when one ends, its
    slot goes to the next request, cleared as the state pool does); returns what the kernel gave and the inputs."""
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    data = []
    for L in lengths:
        rows = torch.randn(L, 2 * Gq * N + H * dv + 2 * H + 3, generator=g)        # q | k | v | gate a | gate b | spare
        data.append(rows)
    p0, p1, p2 = (0.5 * torch.randn(H, generator=g) for _ in range(3))
    extra = H * N + H if mode == "matrix_memory" else 0
    state = torch.zeros(slots_total, H * N * dv + extra + 4, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    waiting = list(range(len(lengths)))
    live, slot_of, free = [], {}, list(range(slots_total))
    done = [0] * len(lengths)
    plans = [_portions(L, cuts[i % len(cuts)]) for i, L in enumerate(lengths)]
    got = [[] for _ in lengths]
    a, b, c = Gq * N, 2 * Gq * N, 2 * Gq * N + H * dv
    while waiting or live:
        while waiting and free:
            r = waiting.pop(0)
            slot_of[r] = free.pop()
            state[slot_of[r]].zero_()
            live.append(r)
        sizes = [plans[r].pop(0) for r in live]
        rows = torch.cat([data[r][done[r]:done[r] + n] for r, n in zip(live, sizes)]).to(DEV)
        cu = [0]
        for n in sizes:
            cu.append(cu[-1] + n)
        out = torch.empty(rows.shape[0], H * dv, dtype=torch.float32, device=DEV)
        ops.linrec(mode, rows[:, :a], rows[:, a:b], rows[:, b:c], rows[:, c:c + H], rows[:, c + H:c + 2 * H] if mode == "matrix_memory" else None,
                   p0.to(DEV), p1.to(DEV), p2.to(DEV) if mode == "state_space" else None, 6.0 if mode == "matrix_memory" else 0.0,
                   N ** -0.5 if mode == "matrix_memory" else 1.0, i32(cu), i32([slot_of[r] for r in live]), state, out, len(live), H, Gq, N, dv, err)
        for i, r in enumerate(live):
            got[r].append(out[cu[i]:cu[i + 1]].cpu())
            done[r] += sizes[i]
        for r in [r for r in live if done[r] == lengths[r]]:
            live.remove(r)
            free.append(slot_of.pop(r))
    assert err.cpu().tolist()[0] == 0
    return [torch.cat(x) for x in got], data, (p0.double(), p1.double(), p2.double())


SHAPES = [(4, 2, 16, 8), (3, 3, 7, 11), (2, 1, 56, 24), (1, 1, 128, 40), (2, 2, 40, 15), (6, 2, 12, 4), (1, 1, 200, 17), (1, 1, 300, 9),
          (1, 1, 512, 16)]


@pytest.mark.parametrize("H,Gq,N,dv", SHAPES)
def test_state_space_recurrence_in_portions_batches_and_reused_slots(H, Gq, N, dv):
    lengths = [70, 33, 121, 18, 50]
    got, data, (A_log, dt_bias, D) = _run_recurrence("state_space", H, Gq, N, dv, lengths, [[70], [1, 2, 16, 5], [17, 31, 3], [2], [1]], seed=N + dv)
    a, b, c = Gq * N, 2 * Gq * N, 2 * Gq * N + H * dv
    whole, _, _ = _run_recurrence("state_space", H, Gq, N, dv, lengths, [[1000]], seed=N + dv)
    for r, L in enumerate(lengths):
        rows = data[r].double()
        C = rows[:, :a].reshape(L, Gq, N).repeat_interleave(H // Gq, dim=1)
        B = rows[:, a:b].reshape(L, Gq, N).repeat_interleave(H // Gq, dim=1)
        x = rows[:, b:c].reshape(L, H, dv)
        dt = torch.nn.functional.softplus(rows[:, c:c + H] + dt_bias)
        want = plain.selective_scan(x, B, C, dt, torch.exp(A_log), D).reshape(L, H * dv)
        assert rel_err(got[r], want) < 2e-5, r
        assert torch.equal(got[r], whole[r]), r                 # the cut changes no bit


@pytest.mark.parametrize("H,Gq,N,dv", [s for s in SHAPES if s[0] == s[1]] + [(4, 4, 16, 8), (2, 2, 72, 24)])
def test_matrix_memory_recurrence_in_portions_batches_and_reused_slots(H, Gq, N, dv):
    lengths = [70, 33, 121, 18, 50]
    got, data, (bi, bf, _) = _run_recurrence("matrix_memory", H, Gq, N, dv, lengths, [[70], [1, 2, 16, 5], [17, 31, 3], [2], [1]], seed=N * dv)
    whole, _, _ = _run_recurrence("matrix_memory", H, Gq, N, dv, lengths, [[1000]], seed=N * dv)
    a, b, c = H * N, 2 * H * N, 2 * H * N + H * dv
    for r, L in enumerate(lengths):
        rows = data[r].double()
        q, k, v = rows[:, :a].reshape(L, H, N) * N ** -0.5, rows[:, a:b].reshape(L, H, N), rows[:, b:c].reshape(L, H, dv)
        i_log = plain.capped(rows[:, c:c + H] + bi, 6.0)
        f_log = torch.nn.functional.logsigmoid(plain.capped(rows[:, c + H:c + 2 * H] + bf, 6.0))
        want = plain.matrix_memory(q, k, v, i_log, f_log).reshape(L, H * dv)
        assert rel_err(got[r], want) < 5e-5, r
        assert torch.equal(got[r], whole[r]), r


def test_matrix_memory_keeps_its_exponentials_in_range():
    """Input gates at their bound for hundreds of tokens: the running maximum grows and the outputs stay finite and right."""
    from photon_infer_b200.kernels import ops
    H, N, dv, L = 2, 16, 8, 400
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(L, 2 * H * N + H * dv + 2 * H, generator=g)
    c = 2 * H * N + H * dv
    rows[:, :2 * H * N] = rows[:, :2 * H * N].abs()             # n . q stays away from zero, where the quotient is ill-conditioned
    rows[:, c:c + H] = 500.0                                    # capped to +cap
    rows[:, c + H:] = 500.0                                     # the forget gate near one
    bias = torch.zeros(H)
    state = torch.zeros(1, H * N * dv + H * N + H, device=DEV)
    out = torch.empty(L, H * dv, dtype=torch.float32, device=DEV)
    rd = rows.to(DEV)
    ops.linrec("matrix_memory", rd[:, :H * N], rd[:, H * N:2 * H * N], rd[:, 2 * H * N:c], rd[:, c:c + H], rd[:, c + H:], bias.to(DEV),
               bias.to(DEV), None, 9.0, 0.25, i32([0, L]), i32([0]), state, out, 1, H, H, N, dv, None)
    r = rows.double()
    want = plain.matrix_memory(r[:, :H * N].reshape(L, H, N) * 0.25, r[:, H * N:2 * H * N].reshape(L, H, N), r[:, 2 * H * N:c].reshape(L, H, dv),
                               plain.capped(r[:, c:c + H], 9.0), torch.nn.functional.logsigmoid(plain.capped(r[:, c + H:], 9.0)))
    assert torch.isfinite(out).all() and rel_err(out.cpu(), want.reshape(L, H * dv)) < 5e-5
    assert abs(float(state[0, -1]) - 9.0) < 1e-3               # the running maximum is kept with the state


def test_a_negative_slot_starts_from_zero_and_stores_nothing():
    from photon_infer_b200.kernels import ops
    H, N, dv = 2, 8, 4
    rows = torch.randn(3, 2 * H * N + H * dv + 2 * H, generator=torch.Generator().manual_seed(1)).to(DEV)
    c = 2 * H * N + H * dv
    state = torch.full((2, H * N * dv + H * N + H), 3.0, device=DEV)
    out = torch.empty(3, H * dv, dtype=torch.float32, device=DEV)
    z = torch.zeros(H, device=DEV)
    args = lambda slot, st, o: ops.linrec("matrix_memory", rows[:, :H * N], rows[:, H * N:2 * H * N], rows[:, 2 * H * N:c], rows[:, c:c + H],
                                          rows[:, c + H:], z, z, None, 5.0, 1.0, i32([0, 3]), i32([slot]), st, o, 1, H, H, N, dv, None)
    args(-1, state, out)
    assert float((state - 3.0).abs().max()) == 0.0
    fresh = torch.zeros_like(state)
    out2 = torch.empty_like(out)
    args(1, fresh, out2)
    assert torch.equal(out, out2) and float(fresh[0].abs().max()) == 0.0 and float(fresh[1].abs().max()) > 0.0


# ----------------------------------------------------------------------------- the block

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_with_norms_on_the_sublayers_outputs(dtype):
    """x <- x + norm1(mixer(x)); x <- x + norm2(ff(x)) with a mixer and a feed-forward that are plain functions of the rows
    they are given: the sublayers must see the stream itself, and the second sum stays pending with its norm."""
    from photon_infer_b200.parts.base import FeedForward, Mixer, Normed
    from photon_infer_b200.parts.registry import create_part
    from photon_infer_b200.parts.base import StepContext

    class Twice(Mixer):
        def forward(self, h, ctx, cache):
            return (2 * h.float() + 1).to(h.dtype)

    class Square(FeedForward):
        def forward(self, h, ctx):
            return (h.float() ** 2 - 0.5).to(h.dtype)

    W = 24
    g = torch.Generator().manual_seed(2)
    norms = [create_part("norm", "group_rms_norm", {"size": W, "eps": 1e-5, "groups": 3, "weight_name": "w"}) for _ in range(2)]
    ws = [(1 + 0.2 * torch.randn(W, generator=g)) for _ in range(2)]
    for n, w in zip(norms, ws):
        n.load({"w": w.to(DEV)})
    block = create_part("block", "output_norm", dict(norm1=norms[0], mixer=Twice(), norm2=norms[1], feed_forward=Square()))
    x = torch.randn(5, W, generator=g)
    ctx = StepContext(num_tokens=5, num_seqs=1, dtype=dtype, token_ids=None, positions=None, token_seq=None, cu_tokens=None,
                      context_lens=None, state_slots=None, groups=[])
    res, pending = block.forward(x.to(DEV).clone(), None, ctx, None)
    rnd = lambda t: t.to(dtype).double()                        # what a sublayer reads and returns is in the run type
    x1 = x.double() + plain.group_rms_norm(rnd(2 * rnd(x) + 1), ws[0].double(), 3, 1e-5)
    d = rnd(rnd(x1) ** 2 - 0.5)
    assert isinstance(pending, Normed) and pending.norm is norms[1]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(res.cpu(), x1) < tol and rel_err(pending.tensor.float().cpu(), d) < 3 * tol
    # the next block (or the model's last norm) adds what is pending
    res2, _ = block.forward(res, pending, ctx, None)
    x2 = x1 + plain.group_rms_norm(d, ws[1].double(), 3, 1e-5)
    x3 = x2 + plain.group_rms_norm(rnd(2 * rnd(x2) + 1), ws[0].double(), 3, 1e-5)
    assert rel_err(res2.cpu(), x3) < 5 * tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_mixer_s_output_bias_rides_in_the_norm_kernel(dtype):
    """A mixer may hand its output product's bias over instead of adding it: the block's norm kernel adds it before the norm,
    also when the output stays pending and when the model's last norm takes it on chosen rows."""
    from photon_infer_b200.parts.base import Mixer, Normed, StepContext
    from photon_infer_b200.parts.registry import create_part
    W = 40
    g = torch.Generator().manual_seed(4)
    b = torch.randn(W, generator=g)

    class WithBias(Mixer):
        def forward(self, h, ctx, cache):
            return 3 * h.float() + b.to(DEV)

        def forward_deferred_bias(self, h, ctx, cache):
            return 3 * h.float(), b.to(DEV)

    norm = create_part("norm", "group_rms_norm", {"size": W, "eps": 1e-5, "groups": 4, "weight_name": "w"})
    w = 1 + 0.2 * torch.randn(W, generator=g)
    norm.load({"w": w.to(DEV)})
    block = create_part("block", "output_norm", dict(norm1=norm, mixer=WithBias(), norm2=None, feed_forward=None))
    x = torch.randn(6, W, generator=g)
    ctx = StepContext(num_tokens=6, num_seqs=1, dtype=dtype, token_ids=None, positions=None, token_seq=None, cu_tokens=None,
                      context_lens=None, state_slots=None, groups=[])
    res, pending = block.forward(x.to(DEV).clone(), None, ctx, None)
    assert isinstance(pending, Normed) and pending.bias is not None
    want = x.double() + plain.group_rms_norm(3 * x.to(dtype).double() + b.double(), w.double(), 4, 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err((res + pending.materialize()).cpu(), want) < tol
    res2 = res.clone()
    block._enter(res2, pending, ctx)
    assert rel_err(res2.cpu(), want) < tol
    rows = norm.add_forward_rows(pending, res, i32([5, 0]), torch.float32)
    assert rel_err(rows.cpu(), plain.group_rms_norm(want[[5, 0]], w.double(), 4, 1e-5)) < tol
