"""Whole Lerosun models through ``bin/trace_run`` and through the engine, against the plain implementation: each
request whole; a prompt and then its tail token by token; portions of changing size down to two tokens; up to four
live requests in mixed batches with so few pages and state slots that they are used again; long decoding past every
window; greedy generation through the engine's own entry point and scheduler.  Five tiny configurations that differ
in every size (query/key heads shared by several value heads or not, convolutions of one to seven taps, heads of 6 to
128, one with sizes that are multiples of nothing, looped blocks at the start, in the middle, at the end, or none),
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

from helpers import (TINY_LEROSUN, TOL, TraceSession, lerosun_plain_logits, lerosun_plain_model, make_lerosun_folder,
                     random_ids, rel_err, round64)

pytestmark = pytest.mark.gpu

LENGTHS = {"ls_a": [75, 150, 33, 200, 97, 1], "ls_b": [45, 130, 64, 170, 31, 99],
           "ls_c": [90, 140, 40, 2, 65, 210], "ls_d": [120, 190, 36, 180, 75, 3], "ls_e": [150, 33, 300, 64, 5, 131]}
PORTIONS = [7, 2, 16, 3, 2, 33, 5, 2, 64, 11, 2, 17]


def _requests(name):
    vocab = TINY_LEROSUN[name]["config"]["vocab"]
    return {f"r{i}": random_ids(n, vocab, seed=100 * i + len(name) + 7) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in TINY_LEROSUN for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def session(request, tmp_path_factory):
    name, dtype = request.param
    folder = str(tmp_path_factory.mktemp(f"model_{name}"))
    make_lerosun_folder(folder, name)
    out = str(tmp_path_factory.mktemp(f"out_{name}_{dtype}"))
    reqs = _requests(name)
    max_tokens = sum(sorted((round64(len(v)) for v in reqs.values()), reverse=True)[:4])
    s = TraceSession(folder, dtype, out, max_tokens, TINY_LEROSUN[name]["block_size"], TINY_LEROSUN[name]["config"]["vocab"])
    s.name, s.dtype, s.folder, s.requests = name, dtype, folder, reqs
    s.collected = {}
    yield s
    assert s.close() == 0


def _check(session, rid, got, label):
    want = lerosun_plain_logits(session.folder, session.requests[rid])
    got_t = torch.from_numpy(np.ascontiguousarray(got)).double()
    scale = float(want.abs().max())
    per_row = (got_t - want).abs().amax(dim=1) / scale
    tol = TOL[session.dtype] if session.dtype != "float32" else 5e-5
    bad = (per_row > tol).nonzero().flatten().tolist()
    allowed = 0
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
    one chain of multiply-adds per output; attention: key tiles from the window's first tile; the recurrence: the same
    chain per token whatever the step brought before it), so all ways of cutting a request give the same bits."""
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
                assert (per_row > 4e-2).sum() <= max(1, int(0.03 * len(per_row))), \
                    f"{label} against whole, request {rid}: worst {float(per_row.max()):.3g}"


def test_long_decoding(session):
    """A short prompt, then 230 tokens one by one: every window slides over decoded tokens only, pages behind it are
    given back, and the recurrent state is carried through 230 steps."""
    if session.name not in ("ls_a", "ls_b", "ls_e"):
        pytest.skip("three configurations are enough")
    ids = random_ids(240, TINY_LEROSUN[session.name]["config"]["vocab"], seed=77)
    got = [session.step([{"id": "long", "tokens": ids[:10], "want": list(range(10))}])]
    for p in range(10, len(ids)):
        got.append(session.step([{"id": "long", "tokens": [ids[p]], "want": [0]}], end=["long"] if p == len(ids) - 1 else []))
    session.requests["long"] = ids
    try:
        _check(session, "long", np.concatenate(got), "long")
    finally:
        del session.requests["long"]
        session.collected.pop("long", None)


@pytest.mark.parametrize("name,lengths,slots,dtype", [("ls_a", (37, 5, 18), 2, "float32"), ("ls_b", (37, 5, 18), 2, "float32"),
                                                      ("ls_e", (9, 30, 4, 21, 13), 5, "float32"), ("ls_c", (3, 12, 7), 3, "float32"),
                                                      ("ls_d", (20, 2, 33), 3, "float32")])
def test_greedy_generation_through_the_engine(tmp_path, name, lengths, slots, dtype):
    """Requests of unequal length through ``ContinuousBatchEngine`` (scheduler, portions of 16 tokens, fewer live
    requests than there are requests, or as many): the tokens are those of the plain implementation's greedy loop.
    The decode steps replay CUDA graphs (padding rows carry state slot -1, which stores nothing); 40 new tokens take
    every request past its shortest windows."""
    from photon_infer_b200 import ContinuousBatchEngine, EngineOptions
    from plain import lerosun_plain
    folder = make_lerosun_folder(str(tmp_path / name), name)
    vocab = TINY_LEROSUN[name]["config"]["vocab"]
    prompts = [random_ids(n, vocab, seed=n) for n in lengths]
    engine = ContinuousBatchEngine(folder, EngineOptions(dtype=dtype, block_size=TINY_LEROSUN[name]["block_size"],
                                                         max_cache_tokens=128 * slots + 128, max_sequences=slots, chunk_size=16,
                                                         max_num_batched_tokens=24, max_model_len=128))
    assert engine.runner.use_cuda_graphs
    rids = [engine.add_request(p, max_new_tokens=40, temperature=0.0, ignore_eos=True) for p in prompts]
    out = engine.run_until_complete()
    cfg, tensors = lerosun_plain_model(folder)
    for rid, p in zip(rids, prompts):
        assert list(out[rid]) == lerosun_plain.greedy(cfg, tensors, p, 40)


def test_command_line(tmp_path):
    """``bin/llama_infer`` picks the model class by config.json: the same command line serves a Lerosun folder."""
    from plain import lerosun_plain
    folder = make_lerosun_folder(str(tmp_path / "m"), "ls_d")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = random_ids(11, TINY_LEROSUN["ls_d"]["config"]["vocab"], seed=5)
    cmd = [sys.executable, os.path.join(root, "bin", "llama_infer"), folder, "cuda", "--dtype", "fp32", "--prompt-ids",
           ",".join(map(str, prompt)), "--prompt-ids", "7 8 9", "--max-new-tokens", "6", "--temperature", "0", "--ignore-eos",
           "--num-blocks", "32", "--max-sequences", "4", "--max-model-len", "128"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("request")]
    cfg, tensors = lerosun_plain_model(folder)
    assert lines[0].split(": ")[1].split() == [str(t) for t in lerosun_plain.greedy(cfg, tensors, prompt, 6)]
    assert lines[1].split(": ")[1].split() == [str(t) for t in lerosun_plain.greedy(cfg, tensors, [7, 8, 9], 6)]
