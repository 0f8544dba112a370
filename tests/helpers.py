"""Shared pieces of the tests: tiny configurations, model folders in temporary
places, the plain implementation as oracle, and a driver for ``bin/trace_run``."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Tiny configurations that differ in every size and option.
TINY: Dict[str, dict] = {
    # the reference's own constants: rope base 10000, neighbouring pairs, eps 1e-5, tied head
    "tiny_a": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=256,
                    max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
                    rope_interleaved=True, tie_word_embeddings=True, bos_token_id=1, eos_token_id=2),
        seed=0, init_std=0.02, norm_std=0.1, block_size=16),
    # one key/value head for three query heads, llama3 frequency scaling, untied head
    "tiny_b": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=200,
                    num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, vocab_size=384,
                    max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                      original_max_position_embeddings=64),
                    tie_word_embeddings=False, bos_token_id=0, eos_token_id=[5, 7]),
        seed=1, init_std=0.05, norm_std=0.1, block_size=8),
    # head_dim not hidden/heads, odd vocabulary, a window on every other layer
    "tiny_c": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=120, intermediate_size=176,
                    num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
                    vocab_size=389, max_position_embeddings=1024, rms_norm_eps=3e-6, rope_theta=250000.0,
                    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=2.0,
                                      original_max_position_embeddings=32),
                    tie_word_embeddings=False, sliding_window=24,
                    layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                    bos_token_id=3, eos_token_id=4),
        seed=2, init_std=0.08, norm_std=0.2, block_size=16),
    # heads of 64 (the size the tensor-memory attention kernel takes), three query heads per key/value
    # head, a window on the first layer, half-split rotation pairs, pages of 32
    "tiny_d": dict(
        config=dict(architectures=["LlamaForCausalLM"], hidden_size=160, intermediate_size=208,
                    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                    vocab_size=301, max_position_embeddings=1024, rms_norm_eps=2e-5, rope_theta=100000.0,
                    rope_scaling=None, tie_word_embeddings=True, sliding_window=40,
                    layer_types=["sliding_attention", "full_attention"], bos_token_id=1, eos_token_id=2),
        seed=3, init_std=0.06, norm_std=0.15, block_size=32),
}


def make_model_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_plain_cache: Dict[tuple, torch.Tensor] = {}


def plain_logits(folder: str, ids: Sequence[int], dtype=torch.float32, **kw) -> torch.Tensor:
    from plain.llama_plain import PlainLlama
    key = (folder, tuple(ids), dtype, repr(sorted(kw.items())))
    if key not in _plain_cache:
        _plain_cache[key] = PlainLlama.from_folder(folder, dtype=dtype, **kw).logits(ids)
    return _plain_cache[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest absolute difference over the largest absolute wanted value."""
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


# float32: both sides are 32-bit with different summation orders.
# bfloat16: activations are rounded to 8 bits of mantissa at every matrix product; the bound is a few
# roundings' worth (2^-8 each) relative to the largest logit.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


class TraceSession:
    """Drives one ``bin/trace_run`` process: a step goes in, ``done`` comes back, logits are read."""

    def __init__(self, model: str, dtype: str, out_dir: str, max_tokens: int, block_size: int, vocab: int):
        self.out_dir = out_dir
        self.vocab = vocab
        self.step_no = 0
        env = dict(os.environ)
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens), "--block-size", str(block_size)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)

    def step(self, entries: List[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_no} (exit code {rc})")
        path = os.path.join(self.out_dir, f"{self.step_no}.f32")
        self.step_no += 1
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        os.remove(path)
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc


def round64(n: int) -> int:
    return (n + 63) // 64 * 64


# ----------------------------------------------------------------------------- Finelix

def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
                scale=(dim + rot_dim) ** -0.5, rot=dict(base=base, dims=rot_dim))


def _moe(experts, top, ff, shared=None):
    m = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


# Tiny Finelix configurations that differ in every size, in the order of the layers and in which optional pieces
# they have.
TINY_FINELIX: Dict[str, dict] = {
    # a looped block in the middle (two passes), every kind of mixer and feed-forward, a layer without feed-forward
    "fx_a": dict(
        config=dict(architecture="Finelix", vocab=160, width=64, embedding=dict(scale=4.0), norm=dict(eps=1e-5),
                    layers=[dict(type="gla", mixer=dict(heads=2, dim=16, vdim=24, tau=4.0), mlp=dict(kind="dense", ff=96)),
                            dict(type="latent_attention", mixer=_latent(3, 16, 8, 20, 32, 24), mlp=_moe(4, 2, 32, 48)),
                            dict(type="gla_2", mixer=dict(heads=1, dim=32, vdim=16, tau=8.0), mlp=None),
                            dict(type="latent_attention", mixer=_latent(2, 8, 16, 12, 24, 40, base=500.0),
                                 mlp=dict(kind="dense", ff=80))],
                    loop=dict(start=1, stop=3, times=2)),
        seed=11, init_std=0.1, norm_std=0.1, block_size=16),
    # no loop; one attention head; every expert chosen and no shared expert; one expert of five with a shared one;
    # a strong decay (tau 1); pages of 8
    "fx_b": dict(
        config=dict(architecture="Finelix", vocab=200, width=96, embedding=dict(scale=1.0), norm=dict(eps=1e-6),
                    layers=[dict(type="latent_attention", mixer=_latent(1, 24, 16, 24, 40, 16, base=1e6), mlp=_moe(3, 3, 40)),
                            dict(type="gla", mixer=dict(heads=4, dim=8, vdim=8, tau=1.0), mlp=_moe(5, 1, 24, 16))],
                    loop=None),
        seed=12, init_std=0.08, norm_std=0.15, block_size=8),
    # the whole model is the looped block (three passes); pages of 32; a wide gla head
    "fx_c": dict(
        config=dict(architecture="Finelix", vocab=131, width=48, embedding=dict(scale=7.5), norm=dict(eps=2e-5),
                    layers=[dict(type="latent_attention", mixer=_latent(4, 4, 4, 6, 16, 8), mlp=None),
                            dict(type="gla_2", mixer=dict(heads=1, dim=72, vdim=40, tau=16.0, decay_rank=6),
                                 mlp=dict(kind="dense", ff=56))],
                    loop=dict(start=0, stop=2, times=3)),
        seed=13, init_std=0.12, norm_std=0.05, block_size=32),
    # a block that is "looped" once, at the end of the model
    "fx_d": dict(
        config=dict(architecture="Finelix", vocab=90, width=32, embedding=dict(scale=2.0), norm=dict(eps=1e-5),
                    layers=[dict(type="gla", mixer=dict(heads=2, dim=12, vdim=10, tau=2.0), mlp=_moe(2, 1, 16, 8)),
                            dict(type="latent_attention", mixer=_latent(2, 12, 4, 8, 20, 12), mlp=dict(kind="dense", ff=40))],
                    loop=dict(start=1, stop=2, times=1)),
        seed=14, init_std=0.15, norm_std=0.1, block_size=16),
    # sizes that are multiples of nothing: no 16-byte rows anywhere, so every kernel takes its unaligned path
    "fx_e": dict(
        config=dict(architecture="Finelix", vocab=77, width=50, embedding=dict(scale=3.0), norm=dict(eps=1e-5),
                    layers=[dict(type="latent_attention", mixer=_latent(3, 10, 6, 14, 36, 26), mlp=dict(kind="dense", ff=70)),
                            dict(type="gla", mixer=dict(heads=1, dim=9, vdim=33, tau=5.0, decay_rank=3), mlp=None),
                            dict(type="gla_2", mixer=dict(heads=3, dim=18, vdim=14, tau=3.0), mlp=_moe(6, 2, 30, 22))],
                    loop=dict(start=0, stop=2, times=2)),
        seed=15, init_std=0.1, norm_std=0.1, block_size=16),
}


def make_finelix_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY_FINELIX[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


_finelix_cache: Dict[tuple, torch.Tensor] = {}


def finelix_plain_logits(folder: str, ids: Sequence[int]) -> torch.Tensor:
    from plain.finelix_plain import PlainFinelix
    key = (folder, tuple(ids))
    if key not in _finelix_cache:
        _finelix_cache[key] = PlainFinelix.from_folder(folder).logits(ids)
    return _finelix_cache[key]


# ----------------------------------------------------------------------------- Fekopel

def _att(heads, kv_heads, dim, vdim, scale, size=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if size:
        m["mask"] = dict(size=size)
    return m


def _att2(heads, kv_heads, dim, vdim, scale, size=None, keep_first=None, rot=None, softcap=None):
    m = _att(heads, kv_heads, dim, vdim, scale, size)
    if keep_first is not None:
        m["mask"]["keep_first"] = keep_first
    if rot:
        m["rot"] = dict(base=rot[0], dims=rot[1])
    if softcap:
        m["softcap"] = softcap
    return m


def _fmoe(experts, top, ff, shared=None, groups=None, scale=1.0):
    r = dict(experts=experts, top=top, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    m = dict(kind="moe", router=r, expert=dict(ff=ff))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


# Tiny Fekopel configurations that differ in every size, in the order of the layers and in which optional pieces they
# have.  Windows are short, so that prompts and decoded tokens alike pass their edges many times.
TINY_FEKOPEL: Dict[str, dict] = {
    # heads of 64 with pages of 16: the tensor-core attention kernels in bfloat16; a looped block at the start
    "fk_a": dict(
        config=dict(architecture="Fekopel", vocab=150, width=64, norm=dict(eps=1e-5),
                    layers=[dict(type="attention_2", mixer=_att2(2, 1, 64, 64, 0.2, 40, 5, (5000.0, 16), 6.0), mlp=_fmoe(6, 2, 24, 40, (3, 2), 0.06)),
                            dict(type="attention", mixer=_att(4, 2, 64, 64, 0.15, 24), mlp=_fmoe(4, 4, 16, None, None, 0.1)),
                            dict(type="attention", mixer=_att(2, 2, 64, 64, 0.1, 70), mlp=None)],
                    loop=dict(start=0, stop=2, times=2)),
        seed=21, init_std=0.1, norm_std=0.1, block_size=16),
    # values wider and narrower than keys, one key/value head, no loop, rotation of the whole head, a window of one
    # page and kept keys that fill more than a page, pages of 8
    "fk_b": dict(
        config=dict(architecture="Fekopel", vocab=210, width=96, norm=dict(eps=1e-6),
                    layers=[dict(type="attention", mixer=_att(3, 1, 16, 40, 0.3, 8), mlp=_fmoe(8, 3, 32, 16, (2, 1), 0.05)),
                            dict(type="attention_2", mixer=_att2(4, 2, 24, 8, 0.25, 19, 11, (100.0, 24), None), mlp=_fmoe(3, 1, 40, 24, None, 0.08)),
                            dict(type="attention_2", mixer=_att2(2, 2, 32, 48, 0.2, 33, 0, (1e6, 8), 30.0), mlp=None)],
                    loop=None),
        seed=22, init_std=0.08, norm_std=0.15, block_size=8),
    # the whole model is the looped block (three passes); no windows at all; no rotation; pages of 32
    "fk_c": dict(
        config=dict(architecture="Fekopel", vocab=131, width=48, norm=dict(eps=2e-5),
                    layers=[dict(type="attention_2", mixer=_att2(3, 3, 16, 16, 0.25, None, None, None, 4.0), mlp=_fmoe(5, 2, 20, 12, None, 0.04)),
                            dict(type="attention", mixer=_att(2, 1, 8, 12, 0.5), mlp=None)],
                    loop=dict(start=0, stop=2, times=3)),
        seed=23, init_std=0.12, norm_std=0.05, block_size=32),
    # a block that is "looped" once, in the middle; heads of 128; a window longer than most requests
    "fk_d": dict(
        config=dict(architecture="Fekopel", vocab=90, width=32, norm=dict(eps=1e-5),
                    layers=[dict(type="attention", mixer=_att(1, 1, 128, 128, 0.08, 100), mlp=_fmoe(2, 1, 16, 8, (2, 2), 0.07)),
                            dict(type="attention_2", mixer=_att2(2, 1, 128, 128, 0.09, 48, 2, (300000.0, 64), 15.0), mlp=_fmoe(4, 2, 8, None, (4, 3), 0.03)),
                            dict(type="attention", mixer=_att(2, 1, 12, 12, 0.3, 17), mlp=_fmoe(2, 2, 24, 24, None, 0.09))],
                    loop=dict(start=1, stop=2, times=1)),
        seed=24, init_std=0.15, norm_std=0.1, block_size=16),
    # sizes that are multiples of nothing: no 16-byte rows anywhere; a window of three keys
    "fk_e": dict(
        config=dict(architecture="Fekopel", vocab=77, width=50, norm=dict(eps=1e-5),
                    layers=[dict(type="attention_2", mixer=_att2(3, 1, 10, 14, 0.3, 3, 1, (777.0, 6), 9.0), mlp=_fmoe(6, 2, 30, 22, (3, 1), 0.05)),
                            dict(type="attention", mixer=_att(5, 5, 6, 9, 0.4, 37), mlp=None),
                            dict(type="attention_2", mixer=_att2(2, 2, 18, 6, 0.2, 21, 30, None, None), mlp=_fmoe(7, 7, 10, 14, None, 0.11))],
                    loop=dict(start=1, stop=3, times=2)),
        seed=25, init_std=0.1, norm_std=0.1, block_size=16),
}


def make_fekopel_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY_FEKOPEL[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


_fekopel_cache: Dict[tuple, torch.Tensor] = {}
_fekopel_models: Dict[str, tuple] = {}


def fekopel_plain_model(folder: str):
    from plain import fekopel_plain
    if folder not in _fekopel_models:
        _fekopel_models[folder] = fekopel_plain.read_folder(folder)
    return _fekopel_models[folder]


def fekopel_plain_logits(folder: str, ids: Sequence[int]) -> torch.Tensor:
    from plain import fekopel_plain
    key = (folder, tuple(ids))
    if key not in _fekopel_cache:
        cfg, tensors = fekopel_plain_model(folder)
        _fekopel_cache[key] = fekopel_plain.forward(cfg, tensors, list(ids))
    return _fekopel_cache[key]


# ----------------------------------------------------------------------------- Lerosun

def _latt(heads, kv_heads, dim, scale, size=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if size:
        m["mask"] = dict(size=size)
    if rot:
        m["rot"] = dict(base=rot[0], dims=rot[1])
    return m


def _ldelta(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


_dense = lambda ff: dict(kind="dense", ff=ff)

# Tiny Lerosun configurations that differ in every size, in the order of the layers and in which optional pieces they
# have.  Windows are short, so that prompts and decoded tokens alike pass their edges many times.
TINY_LEROSUN: Dict[str, dict] = {
    # a looped block in the middle; delta first; rotation of half a head; two windows
    "ls_a": dict(
        config=dict(architecture="Lerosun", vocab=150, width=64, norm=dict(eps=1e-5),
                    layers=[dict(type="delta", mixer=_ldelta(4, 2, 16, 24, 4), mlp=_dense(96)),
                            dict(type="attention", mixer=_latt(4, 2, 32, 0.2, 40, (5000.0, 16)), mlp=_dense(80)),
                            dict(type="delta", mixer=_ldelta(2, 2, 32, 16, 3), mlp=None),
                            dict(type="attention", mixer=_latt(2, 1, 64, 0.15, 24, (100.0, 64)), mlp=None)],
                    loop=dict(start=1, stop=3, times=2)),
        seed=31, init_std=0.1, norm_std=0.1, block_size=16),
    # no loop; one key/value head for three query heads; a window of one page; a convolution of two taps; no rotation;
    # one query/key head for four value heads; pages of 8
    "ls_b": dict(
        config=dict(architecture="Lerosun", vocab=210, width=96, norm=dict(eps=1e-6),
                    layers=[dict(type="attention", mixer=_latt(3, 1, 16, 0.3, 8), mlp=_dense(40)),
                            dict(type="delta", mixer=_ldelta(4, 1, 8, 8, 2), mlp=_dense(56)),
                            dict(type="attention", mixer=_latt(4, 4, 24, 0.25, 19, (1e6, 8)), mlp=None)],
                    loop=None),
        seed=32, init_std=0.08, norm_std=0.15, block_size=8),
    # the whole model is the looped block (three passes); no window at all; a wide delta head; a convolution of one
    # tap (no rows to keep); pages of 32
    "ls_c": dict(
        config=dict(architecture="Lerosun", vocab=131, width=48, norm=dict(eps=2e-5),
                    layers=[dict(type="attention", mixer=_latt(3, 3, 16, 0.25, None, (777.0, 4)), mlp=_dense(72)),
                            dict(type="delta", mixer=_ldelta(1, 1, 72, 40, 1), mlp=None)],
                    loop=dict(start=0, stop=2, times=3)),
        seed=33, init_std=0.12, norm_std=0.05, block_size=32),
    # a block that is "looped" once, at the end; heads of 128; a window longer than most requests; five taps
    "ls_d": dict(
        config=dict(architecture="Lerosun", vocab=90, width=32, norm=dict(eps=1e-5),
                    layers=[dict(type="delta", mixer=_ldelta(2, 1, 128, 128, 5), mlp=_dense(24)),
                            dict(type="attention", mixer=_latt(2, 1, 128, 0.09, 100, (300000.0, 32)), mlp=_dense(48))],
                    loop=dict(start=1, stop=2, times=1)),
        seed=34, init_std=0.15, norm_std=0.1, block_size=16),
    # sizes that are multiples of nothing; a window of three keys; one head
    "ls_e": dict(
        config=dict(architecture="Lerosun", vocab=77, width=50, norm=dict(eps=1e-5),
                    layers=[dict(type="attention", mixer=_latt(5, 5, 6, 0.4, 3, (50.0, 6)), mlp=_dense(30)),
                            dict(type="delta", mixer=_ldelta(3, 3, 9, 33, 7), mlp=None),
                            dict(type="attention", mixer=_latt(1, 1, 18, 0.2, 37), mlp=_dense(22)),
                            dict(type="delta", mixer=_ldelta(6, 2, 18, 14, 4), mlp=_dense(70))],
                    loop=dict(start=1, stop=4, times=2)),
        seed=35, init_std=0.1, norm_std=0.1, block_size=16),
}


def make_lerosun_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY_LEROSUN[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


_lerosun_cache: Dict[tuple, torch.Tensor] = {}
_lerosun_models: Dict[str, tuple] = {}


def lerosun_plain_model(folder: str):
    from plain import lerosun_plain
    if folder not in _lerosun_models:
        _lerosun_models[folder] = lerosun_plain.read_folder(folder)
    return _lerosun_models[folder]


def lerosun_plain_logits(folder: str, ids: Sequence[int]) -> torch.Tensor:
    from plain import lerosun_plain
    key = (folder, tuple(ids))
    if key not in _lerosun_cache:
        cfg, tensors = lerosun_plain_model(folder)
        _lerosun_cache[key] = lerosun_plain.forward(cfg, tensors, list(ids))
    return _lerosun_cache[key]


# ----------------------------------------------------------------------------- Pebodra

def _patt(heads, kv_heads, dim, vdim, scale, diff, size=None, rot=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if size:
        m["mask"] = dict(size=size)
    if rot:
        m["rot"] = dict(base=rot[0], dims=rot[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _pssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def _pmem(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def _pmoe(experts, top, ff, groups=None):
    r = dict(experts=experts, top=top)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff), router=r)


# Tiny Pebodra configurations that differ in every size, in the order of the layers and in which optional pieces they
# have.  Windows are short, so that prompts and decoded tokens alike pass their edges many times.
TINY_PEBODRA: Dict[str, dict] = {
    # attention first; a later layer reads its keys and values through a LONGER window; two of three router groups;
    # values neither as wide as a key nor twice as wide; rotation of half a map
    "pb_a": dict(
        config=dict(architecture="Pebodra", vocab=150, width=64, norm=dict(eps=1e-5, groups=2), logit_softcap=20.0,
                    layers=[dict(type="attention", mixer=_patt(4, 2, 16, 24, 0.3, 0.2, 40, (5000.0, 8)), mlp=_pmoe(6, 2, 32, (3, 2))),
                            dict(type="mlstm", mixer=_pmem(2, 24, 16, 8.0), mlp=_dense(96)),
                            dict(type="attention", mixer=_patt(4, 2, 16, 24, 0.25, 0.35, 56, (5000.0, 8), kv_from=0), mlp=None),
                            dict(type="mamba2", mixer=_pssm(4, 8, 16, 2, 3, 4), mlp=_pmoe(4, 1, 48))]),
        seed=41, init_std=0.1, norm_std=0.1, block_size=16),
    # the state-space layer first; attention that sees every earlier key, without rotation, read by a layer with a
    # window; one norm group; no bound on the logits; values as wide as a map's keys; pages of 8
    "pb_b": dict(
        config=dict(architecture="Pebodra", vocab=210, width=96, norm=dict(eps=1e-6, groups=1),
                    layers=[dict(type="mamba2", mixer=_pssm(2, 24, 8, 1, 2, 1), mlp=_dense(40)),
                            dict(type="attention", mixer=_patt(3, 1, 16, 16, 0.3, 0.5), mlp=_dense(56)),
                            dict(type="mlstm", mixer=_pmem(4, 8, 8, 3.0), mlp=None),
                            dict(type="attention", mixer=_patt(3, 1, 16, 16, 0.2, 0.1, 19, kv_from=1), mlp=_pmoe(8, 3, 24, (4, 3)))]),
        seed=42, init_std=0.08, norm_std=0.15, block_size=8),
    # sizes that are multiples of nothing; a window of three keys; router groups of one expert each; seven taps;
    # as many state groups as heads
    "pb_c": dict(
        config=dict(architecture="Pebodra", vocab=77, width=50, norm=dict(eps=2e-5, groups=5), logit_softcap=7.5,
                    layers=[dict(type="mlstm", mixer=_pmem(3, 9, 33, 15.0), mlp=_pmoe(5, 3, 14, (5, 3))),
                            dict(type="attention", mixer=_patt(5, 5, 6, 10, 0.4, 0.0, 3, (50.0, 6)), mlp=_dense(30)),
                            dict(type="mamba2", mixer=_pssm(3, 11, 7, 3, 7, 3), mlp=None)]),
        seed=43, init_std=0.12, norm_std=0.05, block_size=16),
    # heads of 64 and 128; a window longer than most requests; pages of 32; one head
    "pb_d": dict(
        config=dict(architecture="Pebodra", vocab=90, width=32, norm=dict(eps=1e-5, groups=2), logit_softcap=50.0,
                    layers=[dict(type="attention", mixer=_patt(2, 1, 64, 128, 0.09, 0.45, 100, (300000.0, 64)), mlp=_dense(24)),
                            dict(type="mamba2", mixer=_pssm(2, 64, 128, 1, 4, 2), mlp=_pmoe(2, 2, 16)),
                            dict(type="mlstm", mixer=_pmem(1, 128, 128, 10.0), mlp=_dense(48))]),
        seed=44, init_std=0.15, norm_std=0.1, block_size=16),
    # two layers read the first one's keys and values, one of them without a window (so everything is kept); a
    # convolution of one tap (no rows to carry); a small bound on the gates; groups of two experts, one kept
    "pb_e": dict(
        config=dict(architecture="Pebodra", vocab=131, width=48, norm=dict(eps=1e-5, groups=3),
                    layers=[dict(type="attention", mixer=_patt(2, 2, 24, 40, 0.2, 0.4, 24, (777.0, 4)), mlp=_pmoe(4, 2, 20, (2, 1))),
                            dict(type="attention", mixer=_patt(2, 2, 24, 40, 0.3, 0.25, None, (777.0, 4), kv_from=0), mlp=None),
                            dict(type="mamba2", mixer=_pssm(6, 4, 12, 2, 1, 1), mlp=_dense(72)),
                            dict(type="attention", mixer=_patt(2, 2, 24, 40, 0.15, 0.6, 8, (777.0, 4), kv_from=0), mlp=_dense(36)),
                            dict(type="mlstm", mixer=_pmem(2, 40, 12, 1.5), mlp=None)]),
        seed=45, init_std=0.1, norm_std=0.1, block_size=16),
}


def make_pebodra_folder(path: str, name: str, dtype: str = "bfloat16") -> str:
    from photon_infer_b200.weights import write_random_model
    t = TINY_PEBODRA[name]
    write_random_model(path, t["config"], seed=t["seed"], init_std=t["init_std"], norm_std=t["norm_std"], dtype=dtype)
    return path


_pebodra_cache: Dict[tuple, torch.Tensor] = {}
_pebodra_models: Dict[str, tuple] = {}


def pebodra_plain_model(folder: str):
    from plain import pebodra_plain
    if folder not in _pebodra_models:
        _pebodra_models[folder] = pebodra_plain.read_folder(folder)
    return _pebodra_models[folder]


def pebodra_plain_logits(folder: str, ids: Sequence[int]) -> torch.Tensor:
    from plain import pebodra_plain
    key = (folder, tuple(ids))
    if key not in _pebodra_cache:
        cfg, tensors = pebodra_plain_model(folder)
        _pebodra_cache[key] = pebodra_plain.forward(cfg, tensors, list(ids))
    return _pebodra_cache[key]
