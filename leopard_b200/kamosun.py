"""Kamosun: a decoder-only language model of PARALLEL layers — x <- x + m * (gate1 * mixer(norm1 x) + gate2 * ff(norm2 x)), both
sublayers on the same stream — whose norms are Dynamic Tanh (tanh(alpha x) * w + b, no statistics), whose sublayer outputs pass a
learned sigmoid gate of the sublayer's input, and whose layers read a learned weighted sum of ALL earlier results (depth average).
Mixers: grouped-query attention with biased projections, per-head query / key norm, rotate-half positions and BLOCK-LOCAL visibility
(a position sees only its own block of mask.size positions), optionally on the keys and values of an earlier layer (kv_from); and a
PARALLEL mixer of capped causal attention (interleaved rotation with band-rescaled frequencies) beside lightning attention (a decayed
matrix state read without softmax), each output RMS-normed and the two averaged.  Feed-forwards: a clamped gated unit, dense or as a
mixture of experts whose sigmoid router weights an expert's INPUT, plus a shared expert.  This module only reads the checkpoint's
config.json into the generic layer list of leopard_b200/seqlm.py and names its tensors; the mechanisms themselves are the shared ones.

config.json keys: architecture, vocab, width, norm.eps, residual_mult, layers[] = {type: "attention" | "parallel", mixer: {...},
mlp: null | {kind: "dense", ff, limit} | {kind: "moe", expert.{ff, limit}, router.{experts, top}, shared.{ff, limit} (optional)}}.
  attention mixer: heads, kv_heads, dim, vdim, scale, rot.{base, dims}, mask.size, kv_from (optional), softcap (optional).
  parallel mixer: left = {heads, kv_heads, dim, vdim, scale, softcap, rot.{base, dims, scaling.{factor, low, high, original}}, mask.size
  (optional)}, right = {heads, dim, vdim, decay[heads]}.
Tensor names: embed, head, final.norm (+ .alpha, .b), and per layer l<i>.{norm1, norm2 (+ .alpha, .b), rg1, rg1.b, rg2, rg2.b, dwa,
mix.{q, k, v, o (+ .b), q.norm, k.norm} | mix.left.{q, k, v, o, q.norm, k.norm, out}, mix.right.{q, k, v, g, o, norm, out},
mlp.{gate, up, down} | mlp.{router, e<j>.{gate, up, down}, shared.{gate, up, down}}}.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

from .safetensors_io import SafetensorsFile
from .seqlm import (BandScaling, DenseFFConfig, LayerConfig, MoEConfig, ParallelMixerConfig, RetentionConfig, RotaryConfig, SeqLMConfig,
                    SeqLMEngine, SeqLMWeights, WindowAttentionConfig)

ARCHITECTURE = "Kamosun"
NO_ROTATION = RotaryConfig(dims=0, base=10000.0)


def _rotary(d: Optional[dict], layout: str) -> RotaryConfig:
    if not d or not d.get("dims"):
        return RotaryConfig(dims=0, base=10000.0, layout=layout)
    s = d.get("scaling")
    scaling = BandScaling(factor=float(s["factor"]), original=float(s["original"]), low=float(s["low"]), high=float(s["high"])) if s else None
    return RotaryConfig(dims=int(d["dims"]), base=float(d["base"]), layout=layout, scaling=scaling)


def _attention(m: dict, layout: str, bias: bool) -> WindowAttentionConfig:
    """softmax attention with per-head query / key norm; `mask.size` makes it block-local, `softcap` caps the scores"""
    heads = int(m["heads"])
    size = (m.get("mask") or {}).get("size")
    kv_from = m.get("kv_from")
    return WindowAttentionConfig(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                 scale=float(m["scale"]), rot=_rotary(m.get("rot"), layout), qk_norm="head", softcap=float(m.get("softcap") or 0.0),
                                 bias=bias, out_bias=bias, chunk=int(size) if size else None,
                                 kv_from=int(kv_from) if kv_from is not None else None)


def _lightning(m: dict) -> RetentionConfig:
    heads = int(m["heads"])
    return RetentionConfig(heads=heads, dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])), decay=tuple(float(x) for x in m["decay"]),
                           rot=NO_ROTATION, form="lightning")


def _mixer(kind: str, m: dict):
    if kind == "attention":      # biased projections, rotate-half pairing
        return _attention(m, "half", bias=True)
    if kind == "parallel":       # left: no biases, interleaved pairing; right: lightning attention
        return ParallelMixerConfig(left=_attention(m["left"], "interleaved", bias=False), right=_lightning(m["right"]))
    raise ValueError(f"unknown mixer type {kind!r}")


def _ff(f: Optional[dict]):
    if f is None:
        return None
    if f["kind"] == "dense":
        return DenseFFConfig(ff=int(f["ff"]), act="clamp_glu", limit=float(f["limit"]))
    if f["kind"] == "moe":
        r, sh = f["router"], f.get("shared")
        return MoEConfig(experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(f["expert"]["ff"]), router="sigmoid_input",
                         act="clamp_glu", limit=float(f["expert"]["limit"]), shared_ff=int(sh["ff"]) if sh else 0,
                         shared_limit=float(sh["limit"]) if sh else 0.0, shared_gate=False)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


def config_from_dict(d: dict) -> SeqLMConfig:
    if d.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {d.get('architecture')!r}")
    layers = tuple(LayerConfig(mixer=_mixer(l["type"], l["mixer"]), ff=_ff(l.get("mlp"))) for l in d["layers"])
    return SeqLMConfig(architecture=ARCHITECTURE, vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=layers,
                       norm="parallel_dyt", residual_mult=float(d.get("residual_mult", 1.0)), residual_gate=True, depth_average=True)


def tensor_name(layer: Optional[int], key: str) -> str:
    return key if layer is None else f"l{layer}.{key}"


def load(path, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    """A folder with config.json and model.safetensors -> an engine ready to step."""
    path = Path(path)
    cfg = config_from_dict(json.loads((path / "config.json").read_text()))
    st = SafetensorsFile(path / "model.safetensors")
    try:
        weights = SeqLMWeights(cfg, lambda n: st[n], tensor_name, device)
    finally:
        st.close()
    return SeqLMEngine(cfg, weights, dtype=dtype, lib=lib, **engine_kw)


def from_state_dict(d: dict, tensors: dict, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    """d: the parsed config.json; tensors: {checkpoint name: tensor}"""
    cfg = config_from_dict(d)
    return SeqLMEngine(cfg, SeqLMWeights(cfg, lambda n: tensors[n], tensor_name, device), dtype=dtype, lib=lib, **engine_kw)
