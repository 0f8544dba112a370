"""Whole Pebodra models through ``bin/trace_run`` and through the engine, against the plain implementation: each
request whole; a prompt and then its tail token by token; portions of changing size down to two tokens; up to four
live requests in mixed batches with so few pages and state slots that they are used again; long decoding past every
window; greedy generation through the engine's own entry point and scheduler.  Five tiny configurations that differ
in every size and in the order of their layers (attention, state-space or matrix memory first; layers that read an
earlier layer's keys and values through a longer, a shorter or no window; values narrower than, as wide as and wider
than two maps of keys; one to seven taps; heads of 6 to 128; one with sizes that are multiples of nothing; routers
with groups of one, two and more experts or none; one or several norm groups; with and without a bound on the logits),
in float32 and in bfloat16.  Their windows are short (3 to 100 keys), so prompts and decoded tokens pass the window's
edge and page borders at most positions, and a portion often starts inside a convolution's reach.

float32 must match the plain implementation at every position.  How a request is cut must not matter in either dtype.
"""
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import (TINY_PEBODRA, TOL, TraceSession, pebodra_plain_logits, pebodra_plain_model, make_pebodra_folder,
                     random_ids, rel_err, round64)

pytestmark = pytest.mark.gpu

LENGTHS = {"pb_a": [75, 150, 33, 200, 97, 1], "pb_b": [45, 130, 64, 170, 31, 99],
           "pb_c": [90, 140, 40, 2, 65, 210], "pb_d": [120, 190, 36, 180, 75, 3], "pb_e": [150, 33, 300, 64, 5, 131]}
PORTIONS = [7, 2, 16, 3, 2, 33, 5, 2, 64, 11, 2, 17]


def _requests(name):
    vocab = TINY_PEBODRA[name]["config"]["vocab"]
    return {f"r{i}": random_ids(n, vocab, seed=100 * i + len(name) + 7) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in TINY_PEBODRA for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def session(request, tmp_path_factory):
    name, dtype = request.param
    folder = str(tmp_path_factory.mktemp(f"model_{name}"))
    make_pebodra_folder(folder, name)
    out = str(tmp_path_factory.mktemp(f"out_{name}_{dtype}"))
    reqs = _requests(name)
    max_tokens = sum(sorted((round64(len(v)) for v in reqs.values()), reverse=True)[:4])
    s = TraceSession(folder, dtype, out, max_tokens, TINY_PEBODRA[name]["block_size"], TINY_PEBODRA[name]["config"]["vocab"])
    s.name, s.dtype, s.folder, s.requests = name, dtype, folder, reqs
    s.collected = {}
    yield s
    assert s.close() == 0


def _check(session, rid, got, label):
    want = pebodra_plain_logits(session.folder, session.requests[rid])
    got_t = torch.from_numpy(np.ascontiguousarray(got)).double()
    scale = float(want.abs().max())
    per_row = (got_t - want).abs().amax(dim=1) / scale
    tol = TOL[session.dtype] if session.dtype != "float32" else 5e-5
    bad = (per_row > tol).nonzero().flatten().tolist()
    # bfloat16: a router's close call may fall the other way for a token, and the norm on the feed-forward's output then
    # gives the other expert's output the same size; and a norm on a sublayer's output magnifies the rounding of an
    # output that happens to be small, more so in models as narrow as these.  So the bound holds for the typical
    # position and a minority may be off (test_bfloat16_with_the_router_s_own_choices takes the choices out; the
    # float32 runs hold at every position).
    allowed = 0 if session.dtype == "float32" else max(2, int(0.3 * len(per_row)))
    assert session.dtype == "float32" or float(per_row.median()) < 2e-2, f"{label}: request {rid}: median {float(per_row.median()):.3g}"
    assert len(bad) <= allowed, f"{label}: request {rid}: {len(bad)} of {len(per_row)} positions off, first {bad[0]}, " \
        f"worst {float(per_row.max()):.3g}"
    session.collected.setdefault(label, {})[rid] = np.array(got)


def test_whole(session):
    for rid, ids in session.requests.items():
        got = session.step([{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], end=[rid])
        _check(session, rid, got, "whole")


def test_tail_one_by_one(session):
    """The last 60 tokens one by one: more than most windows, so decoded tokens drop out of them again."""
    for rid, ids in session.requests.items():
        head = max(1, len(ids) - 60)
        got = [session.step([{"id": rid, "tokens": ids[:head], "want": list(range(head))}],
                            end=[rid] if head == len(ids) else [])]
        for p in range(head, len(ids)):
            got.append(session.step([{"id": rid, "tokens": [ids[p]], "want": [0]}], end=[rid] if p == len(ids) - 1 else []))
        _check(session, rid, np.concatenate(got), "tail")


def test_portions(session):
    for k, (rid, ids) in enumerate(session.requests.items()):
        got, p, j = [], 0, k
        while p < len(ids):
            n = min(PORTIONS[j % len(PORTIONS)], len(ids) - p)
            j += 1
            got.append(session.step([{"id": rid, "tokens": ids[p:p + n], "want": list(range(n))}],
                                    end=[rid] if p + n == len(ids) else []))
            p += n
        _check(session, rid, np.concatenate(got), "portions")


def test_mixed(session):
    """Pages for the four longest requests only; six requests run, so the pages of the ones that end, and the pages
    that a window has passed, go to the ones that start later.  A request is left out of a step now and then."""
    rng = random.Random(5)
    pending = list(session.requests.items())
    live, got, steps = {}, {rid: [] for rid, _ in pending}, 0
    while pending or live:
        while pending and len(live) < 4:
            live[pending.pop(0)[0]] = 0
        entries, ending = [], []
        for rid in list(live):
            ids, p = session.requests[rid], live[rid]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            tail = len(ids) - 24
            n = 1 if p >= tail else min(rng.choice([2, 3, 5, 9, 17, 30]), tail - p)
            entries.append({"id": rid, "tokens": ids[p:p + n], "want": list(range(n))})
            live[rid] = p + n
            if p + n == len(ids):
                ending.append(rid)
        if not entries:
            continue
        out = session.step(entries, end=ending)
        row = 0
        for e in entries:
            got[e["id"]].append(out[row:row + len(e["tokens"])])
            row += len(e["tokens"])
        for rid in ending:
            del live[rid]
        steps += 1
    assert steps > 20
    for rid in session.requests:
        _check(session, rid, np.concatenate(got[rid]), "mixed")


def test_cuts_agree(session):
    """In float32 every sum on the path has an order that depends only on the token's place in its request (products:
    one chain of multiply-adds per output; attention: key tiles from the window's first tile; the recurrences: the same
    chain per token whatever the step brought before it; norms: one row at a time), so all ways of cutting a request
    give the same bits."""
    for label, fn in (("whole", test_whole), ("tail", test_tail_one_by_one), ("portions", test_portions), ("mixed", test_mixed)):
        if label not in session.collected:
            fn(session)
    for label in ("tail", "portions", "mixed"):
        for rid, ref in session.collected["whole"].items():
            other = session.collected[label][rid]
            if session.dtype == "float32":
                same = np.array_equal(other, ref)
                where = None if same else int(np.argwhere((other != ref).any(axis=1))[0, 0])
                assert same, f"{label} against whole, request {rid}: first position that differs {where}, " \
                    f"largest difference {float(np.abs(other - ref).max()):.3g}"
            else:
                scale = float(np.abs(ref).max())
                per_row = np.abs(other - ref).max(axis=1) / scale
                assert (per_row > 4e-2).sum() <= max(2, int(0.3 * len(per_row))) and float(np.median(per_row)) < 2e-2, \
                    f"{label} against whole, request {rid}: worst {float(per_row.max()):.3g}"


def test_long_decoding(session):
    """A short prompt, then 230 tokens one by one: every window slides over decoded tokens only, pages behind it are
    given back, and the recurrent state is carried through 230 steps."""
    if session.name not in ("pb_a", "pb_b", "pb_e"):
        pytest.skip("three configurations are enough")
    ids = random_ids(240, TINY_PEBODRA[session.name]["config"]["vocab"], seed=77)
    got = [session.step([{"id": "long", "tokens": ids[:10], "want": list(range(10))}])]
    for p in range(10, len(ids)):
        got.append(session.step([{"id": "long", "tokens": [ids[p]], "want": [0]}], end=["long"] if p == len(ids) - 1 else []))
    session.requests["long"] = ids
    try:
        _check(session, "long", np.concatenate(got), "long")
    finally:
        del session.requests["long"]
        session.collected.pop("long", None)


@pytest.mark.parametrize("name", list(TINY_PEBODRA))
def test_bfloat16_with_the_router_s_own_choices(tmp_path, name):
    """A bfloat16 step with the experts it chose handed to the plain implementation: with the routers' close calls
    taken out, the typical position is within a few roundings and hardly any is far off (the choice itself is checked
    by the float32 runs)."""
    from photon_infer_b200 import EngineOptions
    from photon_infer_b200.engine.loading import build_runner
    from photon_infer_b200.engine.runner import StepEntry
    from photon_infer_b200.kernels import ops
    from plain import pebodra_plain
    folder = make_pebodra_folder(str(tmp_path / name), name)
    ids = random_ids(160, TINY_PEBODRA[name]["config"]["vocab"], seed=9)
    runner = build_runner(folder, EngineOptions(dtype="bfloat16", block_size=TINY_PEBODRA[name]["block_size"], max_cache_tokens=256,
                                                max_sequences=2, use_cuda_graphs=False))
    chosen, route = [], ops.moe_route

    def recording(*args, **kw):
        out = route(*args, **kw)
        chosen.append(out[0].long().cpu())
        return out
    ops.moe_route = recording
    try:
        runner.cache.add_request("r")
        got = runner.step([StepEntry("r", ids, list(range(len(ids))))]).logits.double().cpu()
        runner.check_device_errors()
    finally:
        ops.moe_route = route
    cfg, tensors = pebodra_plain_model(folder)
    assert len(chosen) == sum(1 for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    want = pebodra_plain.forward(cfg, tensors, ids, forced=chosen)
    per_row = (got - want).abs().amax(dim=1) / float(want.abs().max())
    assert float(per_row.median()) < 1.25e-2 and int((per_row > 5e-2).sum()) <= max(2, int(0.05 * len(per_row))), \
        f"median {float(per_row.median()):.3g}, worst {float(per_row.max()):.3g} at {int(per_row.argmax())}"


@pytest.mark.parametrize("name,lengths,slots,dtype", [("pb_a", (37, 5, 18), 2, "float32"), ("pb_b", (37, 5, 18), 2, "float32"),
                                                      ("pb_e", (9, 30, 4, 21, 13), 5, "float32"), ("pb_c", (3, 12, 7), 3, "float32"),
                                                      ("pb_d", (20, 2, 33), 3, "float32")])
def test_greedy_generation_through_the_engine(tmp_path, name, lengths, slots, dtype):
    """Requests of unequal length through ``ContinuousBatchEngine`` (scheduler, portions of 16 tokens, fewer live
    requests than there are requests, or as many): the tokens are those of the plain implementation's greedy loop.
    The decode steps replay CUDA graphs (padding rows carry state slot -1, which stores nothing); 40 new tokens take
    every request past its shortest windows."""
    from photon_infer_b200 import ContinuousBatchEngine, EngineOptions
    from plain import pebodra_plain
    folder = make_pebodra_folder(str(tmp_path / name), name)
    vocab = TINY_PEBODRA[name]["config"]["vocab"]
    prompts = [random_ids(n, vocab, seed=n) for n in lengths]
    engine = ContinuousBatchEngine(folder, EngineOptions(dtype=dtype, block_size=TINY_PEBODRA[name]["block_size"],
                                                         max_cache_tokens=128 * slots + 128, max_sequences=slots, chunk_size=16,
                                                         max_num_batched_tokens=24, max_model_len=128))
    assert engine.runner.use_cuda_graphs
    rids = [engine.add_request(p, max_new_tokens=40, temperature=0.0, ignore_eos=True) for p in prompts]
    out = engine.run_until_complete()
    cfg, tensors = pebodra_plain_model(folder)
    for rid, p in zip(rids, prompts):
        assert list(out[rid]) == pebodra_plain.greedy(cfg, tensors, p, 40)


def test_command_line(tmp_path):
    """``bin/llama_infer`` picks the model class by config.json: the same command line serves a Pebodra folder."""
    from plain import pebodra_plain
    folder = make_pebodra_folder(str(tmp_path / "m"), "pb_d")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = random_ids(11, TINY_PEBODRA["pb_d"]["config"]["vocab"], seed=5)
    cmd = [sys.executable, os.path.join(root, "bin", "llama_infer"), folder, "cuda", "--dtype", "fp32", "--prompt-ids",
           ",".join(map(str, prompt)), "--prompt-ids", "7 8 9", "--max-new-tokens", "6", "--temperature", "0", "--ignore-eos",
           "--num-blocks", "32", "--max-sequences", "4", "--max-model-len", "128"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("request")]
    cfg, tensors = pebodra_plain_model(folder)
    assert lines[0].split(": ")[1].split() == [str(t) for t in pebodra_plain.greedy(cfg, tensors, prompt, 6)]
    assert lines[1].split(": ")[1].split() == [str(t) for t in pebodra_plain.greedy(cfg, tensors, [7, 8, 9], 6)]
