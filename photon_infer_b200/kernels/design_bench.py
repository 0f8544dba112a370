"""Prefill and decode throughput of another design (the Finelix, the Fekopel, the Lerosun or the Pebodra decoder) beside
a Llama decoder of equal width, depth and feed-forward size (``python bench.py --design finelix|fekopel|lerosun|pebodra``),
with the parts of a layer timed alone against their rooflines.  The Lerosun and the Pebodra decoder also run beside the
Finelix decoder, the other design with a recurrent mixer (a matrix of state per head) and routed experts next to
attention.

Random weights drawn on the device, synthetic token ids, bfloat16.  Per size:

* prefill: one request, one portion of 2,048 tokens, the best of three timed steps after a warm-up;
* decode: 8 requests with 512 tokens in the cache, single-token steps (replayed CUDA graphs);
* parts: the mixer and the feed-forward of one layer of each kind, alone.  Prefill rows are timed with CUDA
  events around the call; decode rows as a CUDA graph of the part alone, a buffer larger than L2 written before
  every replay.  ``frac`` is the part's share of its roofline: for decode rows the bytes it must move (the
  weights it reads, the cache rows or state it reads and writes) over the measured copy bandwidth; for prefill rows
  its arithmetic (the products and the attention or recurrence) over the measured bfloat16 tensor throughput.
"""
from __future__ import annotations

import sys
from typing import Dict

import torch

PREFILL, PROMPT, BATCH = 2048, 512, 8


def finelix_config(width: int, layers: int) -> dict:
    """Alternating gated-linear-attention and latent-attention layers; heads of 128; a latent of 512 + 64; dense
    feed-forwards of 4 x width and routed ones (16 experts, 2 per token, one shared) of the same active size."""
    heads = width // 128
    gla = dict(type="gla", mixer=dict(heads=heads, dim=128, vdim=128, tau=16.0), mlp=dict(kind="dense", ff=4 * width))
    lat = dict(type="latent_attention",
               mixer=dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=max(768, width * 3 // 8),
                          scale=192 ** -0.5, rot=dict(base=10000.0, dims=64)),
               mlp=dict(kind="moe", router=dict(experts=16, top=2), expert=dict(ff=width), shared=dict(ff=2 * width)))
    return dict(architecture="Finelix", vocab=32000, width=width, embedding=dict(scale=1.0), norm=dict(eps=1e-5),
                layers=[gla if i % 2 == 0 else lat for i in range(layers)], loop=None)


FEKOPEL_WINDOW = 1024


def fekopel_config(width: int, layers: int) -> dict:
    """Alternating layers of the two attention mixers, heads of 128, four query heads per key/value head, a window of
    1,024 keys (the second kind keeps its first 4 keys, rotates half of a head and bounds its scores); 16 plain experts
    of 2 x width, 2 per token from the best 2 of 4 groups, and a shared expert of 2 x width: 12 x width^2 active
    weights per token, as a gated feed-forward of 4 x width has."""
    heads, kv = width // 128, max(1, width // 512)
    mlp = dict(kind="moe", router=dict(experts=16, top=2, scale=1.0, groups=dict(count=4, keep=2)), expert=dict(ff=2 * width),
               shared=dict(ff=2 * width))
    a1 = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=128, vdim=128, scale=128 ** -0.5,
                                           mask=dict(size=FEKOPEL_WINDOW)), mlp=mlp)
    a2 = dict(type="attention_2", mixer=dict(heads=heads, kv_heads=kv, dim=128, vdim=128, scale=128 ** -0.5,
                                             mask=dict(size=FEKOPEL_WINDOW, keep_first=4), rot=dict(base=10000.0, dims=64),
                                             softcap=30.0), mlp=mlp)
    return dict(architecture="Fekopel", vocab=32000, width=width, norm=dict(eps=1e-5),
                layers=[a2 if i % 2 == 0 else a1 for i in range(layers)], loop=None)


LEROSUN_WINDOW = 1024


def lerosun_config(width: int, layers: int) -> dict:
    """Alternating layers of attention with mixed heads (at most 16 heads of 128, since every head's score is a sum over
    all heads and the tensor-core kernel keeps 16 tokens with all their heads in one block; a window of 1,024 keys, half
    of a head rotated, a sink, an output gate; the values are the keys) and of the gated delta rule (heads of 128 x
    128, two value heads per query/key head, convolutions of four taps); dense feed-forwards of 4 x width with a relu
    gate."""
    heads = width // 128
    att_heads = min(16, heads)
    mlp = dict(kind="dense", ff=4 * width)
    att = dict(type="attention", mixer=dict(heads=att_heads, kv_heads=max(1, att_heads // 8), dim=128, vdim=128, scale=128 ** -0.5,
                                            mask=dict(size=LEROSUN_WINDOW), rot=dict(base=10000.0, dims=64)), mlp=mlp)
    delta = dict(type="delta", mixer=dict(heads=heads, kv_heads=heads // 2, dim=128, vdim=128, conv=4), mlp=mlp)
    return dict(architecture="Lerosun", vocab=32000, width=width, norm=dict(eps=1e-5),
                layers=[delta if i % 2 == 0 else att for i in range(layers)], loop=None)


PEBODRA_WINDOW = 1024


def pebodra_config(width: int, layers: int) -> dict:
    """Layers in the order matrix memory, differential attention, state-space, differential attention that reads the
    keys and values of the attention layer before it.  Recurrent heads of 128 x 128 (state-space: four taps, one group of B
    and C per eight heads); attention with two maps of 128 per head and values of 256, so that queries and outputs are as
    wide as the model, four query heads per key/value head, a window of 1,024 keys, half of a map rotated.  Dense
    feed-forwards of 4 x width (PolyNorm) alternate with 16 gated experts of width, 2 per token from the best 2 of 4
    groups."""
    heads = width // 128
    att_heads = max(1, width // 256)
    dense = dict(kind="dense", ff=4 * width)
    moe = dict(kind="moe", expert=dict(ff=width), router=dict(experts=16, top=2, groups=dict(count=4, keep=2)))
    att = lambda extra: dict(heads=att_heads, kv_heads=max(1, att_heads // 4), dim=128, vdim=256, scale=128 ** -0.5, diff=0.2,
                             mask=dict(size=PEBODRA_WINDOW), rot=dict(base=10000.0, dims=64), **extra)
    kinds = [lambda i: dict(type="mlstm", mixer=dict(heads=heads, dim=128, vdim=128, gate_cap=15.0), mlp=dense),
             lambda i: dict(type="attention", mixer=att({}), mlp=moe),
             lambda i: dict(type="mamba2", mixer=dict(heads=heads, vdim=128, state=128, groups=max(1, heads // 8), conv=4,
                                                      norm_groups=max(1, heads // 8)), mlp=moe),
             lambda i: dict(type="attention", mixer=att(dict(kv_from=i - 2)), mlp=dense)]
    return dict(architecture="Pebodra", vocab=32000, width=width, norm=dict(eps=1e-5, groups=8), logit_softcap=50.0,
                layers=[kinds[i % 4](i) for i in range(layers)])


def llama_config(width: int, layers: int, window=None) -> dict:
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=width, intermediate_size=4 * width, num_hidden_layers=layers,
               num_attention_heads=width // 128, num_key_value_heads=max(1, width // 512), head_dim=128, vocab_size=32000,
               max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    if window:
        cfg.update(sliding_window=window, layer_types=["sliding_attention"] * layers)
    return cfg


def _time_events(fn, reps: int = 3) -> float:
    fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best * 1e3


_flush = None


def _time_graph(fn, reps: int = 8) -> float:
    """Microseconds of ``fn()`` replayed as a CUDA graph, with L2 written over before every replay."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    times = []
    for _ in range(reps):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return min(times) * 1e3


def _part_bytes(part, kind: str, rows: int) -> int:
    if kind == "moe":
        # a step reads the router, the shared expert and the experts that were chosen (all of them at most)
        expert = (part.w_gate_up[0].numel() + part.w_down[0].numel()) * part.w_down.element_size()
        used = min(part.experts, rows * part.top)
        rest = part.weight_bytes() - part.experts * expert
        return rest + used * expert
    return part.weight_bytes()


def _mixer_numbers(m, kind: str, tokens: int, contexts) -> tuple:
    """(bytes of cache or state a step over ``contexts`` moves, floating-point operations of ``tokens`` rows)."""
    w = m.weight_bytes()
    if kind == "gla":
        state = len(contexts) * m.heads * m.dim * m.vdim * 4 * 2
        flops = tokens * (w // 2) * 2 + 5 * tokens * m.heads * m.dim * m.vdim
        return state, flops
    if kind == "delta":
        # the state is read and written once a step; per token and state element: two read-outs, the decay and the write
        state = len(contexts) * (m.heads * m.dim * m.vdim + (m.taps - 1) * m.channels) * 4 * 2
        flops = tokens * (w // 2) * 2 + 7 * tokens * m.heads * m.dim * m.vdim
        return state, flops
    if kind == "ssm":
        # the state and the convolution's rows are read and written once a step; per token and state element: the decay, the
        # write and the read-out
        state = len(contexts) * (m.heads * m.state * m.vdim + (m.taps - 1) * m.channels) * 4 * 2
        return state, tokens * (w // 2) * 2 + 5 * tokens * m.heads * m.state * m.vdim
    if kind == "memory":
        state = len(contexts) * (m.heads * m.dim * m.vdim + m.heads * m.dim + m.heads) * 4 * 2
        return state, tokens * (w // 2) * 2 + 5 * tokens * m.heads * m.dim * (m.vdim + 1)
    reach = getattr(m, "window", None)
    reach = None if reach is None else reach + getattr(m, "keep_first", 0)
    seen_by = lambda p: p + 1 if reach is None else min(p + 1, reach)      # keys the token at position p reads
    if kind == "diff":
        # two maps per head: two score products over 128 numbers and two weighted sums of the same values
        pairs = sum(sum(seen_by(p) for p in range(c)) for c in contexts) if tokens > len(contexts) else sum(seen_by(c - 1) for c in contexts)
        held = sum(seen_by(c - 1) for c in contexts)
        return held * m.n_kv * (2 * m.head_dim + m.value_dim) * 2, \
            tokens * (w // 2) * 2 + 2 * m.n_q * (2 * m.head_dim + 2 * m.value_dim) * pairs
    if kind in ("attention", "normed", "talking"):
        pairs = sum(sum(seen_by(p) for p in range(c)) for c in contexts) if tokens > len(contexts) else sum(seen_by(c - 1) for c in contexts)
        held = sum(seen_by(c - 1) for c in contexts)
        dv = getattr(m, "value_dim", m.head_dim)
        mix = 2 * m.n_q * m.n_q * pairs if kind == "talking" and m.talk else 0       # every head's score from all heads'
        return held * m.n_kv * (m.head_dim + dv) * 2, tokens * (w // 2) * 2 + 2 * m.n_q * (m.head_dim + dv) * pairs + mix
    pairs = sum(c * (c + 1) // 2 for c in contexts) if tokens > len(contexts) else sum(contexts)
    if kind == "latent":
        rows = sum(contexts) * m.width * 2
        flops = tokens * (w // 2) * 2 + 2 * m.heads * (m.width + m.kv_rank) * pairs
        return rows, flops
    raise ValueError(kind)


def _parts(runner, hbm_peak: float, tf_peak: float) -> Dict[str, dict]:
    """The mixer and the feed-forward of the first layer of every kind, alone, in a prefill step and a decode step."""
    from ..parts.attention import PagedAttention
    from ..parts.delta_rule import GatedDeltaRule
    from ..parts.diff_attention import DifferentialAttention
    from ..parts.matrix_memory import MatrixMemoryMixer
    from ..parts.state_space import StateSpaceMixer
    from ..parts.gla import GatedLinearAttention
    from ..parts.latent_attention import LatentAttention
    from ..parts.moe import MoEFeedForward
    from ..parts.normed_attention import NormedAttention
    from ..parts.talking_attention import TalkingAttention
    model, cache = runner.model, runner.cache
    H = model.spec.hidden_size
    out: Dict[str, dict] = {}
    seen = set()
    for phase in ("prefill", "decode"):
        rids = ["x"] if phase == "prefill" else [("y", i) for i in range(BATCH)]
        from ..engine.runner import StepEntry
        for r in rids:
            cache.add_request(r)
        if phase == "decode":
            for r in rids:
                cache.extend(r, PROMPT); cache.commit(r, PROMPT)
        n = PREFILL if phase == "prefill" else 1
        entries = [StepEntry(r, [1] * n, []) for r in rids]
        for e in entries:
            cache.extend(e.request_id, n)
        ctx, _, _ = runner._build_context(entries)
        T = ctx.num_tokens
        contexts = [PREFILL] if phase == "prefill" else [PROMPT + 1] * BATCH
        h = torch.randn(T, H, device=model.device).to(model.dtype)
        timer = _time_events if phase == "prefill" else _time_graph
        for i, e in enumerate(model.spec.run):
            block = model.blocks[e.layer]
            m = block.mixer()
            kind = {GatedLinearAttention: "gla", LatentAttention: "latent", PagedAttention: "attention",
                    NormedAttention: "normed", TalkingAttention: "talking", GatedDeltaRule: "delta",
                    DifferentialAttention: "diff", StateSpaceMixer: "ssm", MatrixMemoryMixer: "memory"}.get(type(m))
            if kind == "normed":                     # the two kinds of layer are timed apart
                kind_name = "normed_gated" if m.output_gate else "normed_sink"
            elif kind == "diff":                     # a layer that owns its keys and values, and one that reads another's
                kind_name = "diff" if m.own_kv else "diff_reader"
            else:
                kind_name = kind
            ff = block.parts().get("feed_forward")
            fkind = None if ff is None else ("moe" if isinstance(ff, MoEFeedForward) else "dense")
            if fkind == "dense" and not hasattr(ff, "w_gate_up"):
                fkind = "polynorm"
            lc = runner._layer_caches[i]
            if kind and (kind_name, phase) not in seen:
                seen.add((kind_name, phase))
                us = timer(lambda: m.forward(h, ctx, lc))
                moved, flops = _mixer_numbers(m, kind, T, contexts)
                frac = (m.weight_bytes() + moved) / (us * 1e-6) / (hbm_peak * 1e9) if phase == "decode" \
                    else flops / (us * 1e-6) / (tf_peak * 1e12)
                out[f"{kind_name}.{phase}"] = {"us": round(us, 1), "frac": round(frac, 4)}
            if fkind and (fkind, phase) not in seen:
                seen.add((fkind, phase))
                us = timer(lambda: ff.forward(h, ctx))
                wb = _part_bytes(ff, fkind, T)
                if fkind == "moe":
                    expert = (ff.w_gate_up[0].numel() + ff.w_down[0].numel())
                    active = (ff.weight_bytes() // ff.w_down.element_size() - ff.experts * expert) + ff.top * expert
                else:
                    active = ff.weight_bytes() // ff.w_down.element_size()
                frac = wb / (us * 1e-6) / (hbm_peak * 1e9) if phase == "decode" else 2 * T * active / (us * 1e-6) / (tf_peak * 1e12)
                out[f"{fkind}_ff.{phase}"] = {"us": round(us, 1), "frac": round(frac, 4)}
        runner.check_device_errors()
        for r in rids:
            cache.free_request(r)
    return out


def _throughput(runner, vocab: int, steps: int, warmup: int) -> dict:
    from ..engine.runner import StepEntry
    cache = runner.cache
    gen = torch.Generator().manual_seed(3)
    ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
    prompt = ids(PREFILL)

    def prefill_once():
        cache.add_request("p")
        runner.step([StepEntry("p", prompt, [PREFILL - 1])])
        cache.free_request("p")
    pf_us = _time_events(prefill_once)
    for i in range(BATCH):
        cache.add_request(("d", i))
    runner.step([StepEntry(("d", i), ids(PROMPT), []) for i in range(BATCH)])
    greedy = ([0.0] * BATCH, [0.0] * BATCH)
    toks = [ids(BATCH) for _ in range(steps + warmup)]
    one = lambda k: runner.step([StepEntry(("d", i), [toks[k][i]], [0]) for i in range(BATCH)], sampling=greedy)
    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(warmup, warmup + steps):
        one(k)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    runner.check_device_errors()
    for i in range(BATCH):
        cache.free_request(("d", i))
    return {"prefill_tokens_per_s": round(PREFILL / (pf_us * 1e-6), 1), "prefill_ms": round(pf_us / 1e3, 3),
            "decode_tokens_per_s": round(BATCH / (ms * 1e-3), 1), "decode_ms_per_step": round(ms, 4),
            "decode_graphs": bool(runner.use_cuda_graphs)}


def run_finelix_comparison(args, hbm_peak: float, tf_peak: float, peak_src: str) -> dict:
    return run_design_comparison("finelix", args, hbm_peak, tf_peak, peak_src)


def run_design_comparison(design: str, args, hbm_peak: float, tf_peak: float, peak_src: str) -> dict:
    from ..cache.manager import CacheManager  # noqa: F401  (import order: the engine pulls in the CUDA side)
    from ..config.engine_options import EngineOptions
    from ..engine.loading import build_cache, random_model
    from ..engine.runner import ModelRunner
    steps, warmup = max(8, min(args.steps, 64)), max(args.warmup, 3)
    layers = {2048: 8, 4096: 4}
    make, window = {"finelix": (finelix_config, None), "fekopel": (fekopel_config, FEKOPEL_WINDOW),
                    "lerosun": (lerosun_config, LEROSUN_WINDOW), "pebodra": (pebodra_config, PEBODRA_WINDOW)}[design]
    line = {"design": design, "dtype": args.dtype, "data": "synthetic", "peaks": peak_src,
            "workload": {"prefill_tokens": PREFILL, "decode_batch": BATCH, "decode_context": PROMPT, "steps": steps,
                         "warmup": warmup}, "sizes": {}}
    for width in [int(w) for w in args.design_sizes.split(",") if w]:
        n_layers = layers.get(width, 4)
        point = {"layers": n_layers}
        models = [(design, make(width, n_layers)), ("llama", llama_config(width, n_layers, window))]
        if design in ("lerosun", "pebodra"):
            models.append(("finelix", finelix_config(width, n_layers)))
        for name, cfg in models:
            print(f"[bench] {name} width {width}, {n_layers} layers", file=sys.stderr, flush=True)
            model = random_model(cfg, args.dtype, seed=0)
            options = EngineOptions(dtype=args.dtype, block_size=args.block_size,
                                    max_cache_tokens=BATCH * (PROMPT + 128) + PREFILL + 64, max_sequences=BATCH + 1,
                                    max_batch_size=BATCH + 1, max_num_batched_tokens=max(PREFILL, BATCH * PROMPT),
                                    max_model_len=4096, use_cuda_graphs=not args.no_graphs)
            runner = ModelRunner(model, build_cache(model, options, 4096), 4096, use_cuda_graphs=options.use_cuda_graphs)
            point[name] = _throughput(runner, cfg.get("vocab", cfg.get("vocab_size")), steps, warmup)
            point[name]["parts"] = _parts(runner, hbm_peak, tf_peak)
            del runner, model
            torch.cuda.empty_cache()
        line["sizes"][str(width)] = point
    return line
