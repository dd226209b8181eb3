"""Gavatar: a decoder-only language model whose layers mix three kinds of sequence mixer — grouped-query attention with a sliding
window, unit-RMS queries, keys and values, softmax weights MIXED OVER THE HEADS (talking heads) and a sigmoid output gate; sliding-window
LATENT attention without positions (queries and keys / values through normed latents, a learned SINK per head in the softmax
denominator, one gate per head); and an mLSTM matrix memory with capped exponential gates — each followed by a mixture of experts
whose router takes the largest logits and weights them by a softmax over the chosen ones.  Every sublayer sits between two RMS norms
with vector gains stored around zero; the mixer reads its input SHIFTED towards the previous token's; absolute sinusoidal positions
are added to the scaled embedding; a run of layers may LOOP several times over the same weights, each pass with a cache and state of
its own and a learned vector added to the stream before it.  This module only reads the checkpoint's config.json into the generic
layer list of leopard_b200/seqlm.py and names its tensors; the mechanisms themselves are the shared ones.

config.json keys: architecture, vocab, width, norm.eps, embedding.scale, loop.{start, stop, times} (optional), layers[] = {type:
"attention" | "latent_attention" | "mlstm", mixer: {...}, mlp: null | {kind: "moe", expert.ff, router.{experts, top}}}.
  attention mixer: heads, kv_heads, dim, vdim, scale, mask.size.   latent_attention mixer: heads, dim, vdim, q_rank, kv_rank, scale,
  mask.size.   mlstm mixer: heads, dim, vdim, gate_cap.
Tensor names: embed, head, final.norm, loop.step [times, width], and per layer l<i>.{norm1, norm1b, norm2, norm2b, shift, mix.*, mlp.*}.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, Tuple

from .safetensors_io import SafetensorsFile
from .seqlm import (LatentAttentionConfig, LayerConfig, MLSTMConfig, MoEConfig, RotaryConfig, SeqLMConfig, SeqLMEngine, SeqLMWeights,
                    WindowAttentionConfig)

ARCHITECTURE = "Gavatar"
POSITION_BASE = 10000.0          # the design fixes the base of its sinusoidal positions
NO_ROTATION = RotaryConfig(dims=0, base=POSITION_BASE)


def _window(m: dict) -> Optional[int]:
    size = (m.get("mask") or {}).get("size")
    return int(size) if size else None


def _mixer(kind: str, m: dict):
    if kind == "attention":
        heads = int(m["heads"])
        return WindowAttentionConfig(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                     scale=float(m["scale"]), rot=NO_ROTATION, qk_norm="unit", window=_window(m), bias=True, value_norm=True,
                                     talking_heads=True, out_gate=True)
    if kind == "latent_attention":
        return LatentAttentionConfig(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=0, vdim=int(m.get("vdim", m["dim"])),
                                     kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot=NO_ROTATION, window=_window(m),
                                     q_rank=int(m["q_rank"]), sink=True, head_gate=True)
    if kind == "mlstm":
        return MLSTMConfig(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])), gate_cap=float(m["gate_cap"]))
    raise ValueError(f"unknown mixer type {kind!r}")


def _ff(f: Optional[dict]):
    if f is None:
        return None
    if f["kind"] == "moe":
        r = f["router"]
        return MoEConfig(experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(f["expert"]["ff"]), router="softmax_top")
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


def layer_runs(d: dict) -> List[Tuple[int, Optional[int]]]:
    """The order in which the checkpoint's layers run: (layer, pass) pairs, `pass` set on the first layer of every pass of the loop."""
    n = len(d["layers"])
    loop = d.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not 0 <= start <= stop <= n or times < 0:
        raise ValueError(f"loop {loop!r} does not fit {n} layers")
    if stop == start:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def config_from_dict(d: dict) -> Tuple[SeqLMConfig, List[int]]:
    """(the layer list as it RUNS — a looped layer once per pass, later passes on the first pass's weights —, checkpoint layer of
    every entry of that list)"""
    if d.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {d.get('architecture')!r}")
    layers, source, first_run = [], [], {}
    for i, t in layer_runs(d):
        l = d["layers"][i]
        owner = first_run.setdefault(i, len(layers))
        layers.append(LayerConfig(mixer=_mixer(l["type"], l["mixer"]), ff=_ff(l.get("mlp")), weights_of=owner if owner != len(layers) else None,
                                  token_shift=True, add_before=("loop.step", t) if t is not None else None))
        source.append(i)
    cfg = SeqLMConfig(architecture=ARCHITECTURE, vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=tuple(layers),
                      norm="sandwich_vector", embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), position_base=POSITION_BASE)
    return cfg, source


def tensor_namer(source: List[int]):
    """generic key of entry `layer` of the run list -> checkpoint tensor name"""
    def name(layer: Optional[int], key: str) -> str:
        return key if layer is None else f"l{source[layer]}.{key}"
    return name


def load(path, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    """A folder with config.json and model.safetensors -> an engine ready to step."""
    path = Path(path)
    cfg, source = config_from_dict(json.loads((path / "config.json").read_text()))
    st = SafetensorsFile(path / "model.safetensors")
    try:
        weights = SeqLMWeights(cfg, lambda n: st[n], tensor_namer(source), device)
    finally:
        st.close()
    return SeqLMEngine(cfg, weights, dtype=dtype, lib=lib, **engine_kw)


def from_state_dict(d: dict, tensors: dict, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    """d: the parsed config.json; tensors: {checkpoint name: tensor}"""
    cfg, source = config_from_dict(d)
    return SeqLMEngine(cfg, SeqLMWeights(cfg, lambda n: tensors[n], tensor_namer(source), device), dtype=dtype, lib=lib, **engine_kw)
