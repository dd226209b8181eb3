"""Plain, slow float64 implementation of the Gavatar layers: what the tests compare the token-shift, talking-heads attention, sink
latent attention, mLSTM, softmax-of-the-chosen router and looped-layer paths of leopard_b200/seqlm.py with.  One function per
mechanism, whole sequences from position 0 only, explicit loops over tokens, nothing shared with the product path: it takes the
parsed config.json and a {name: tensor} dict.

Notation: T tokens, D width, H query heads, G key / value heads (query head h reads group h // (H // G)), d key size, e value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    """the gain is stored around zero"""
    return unit_rms(x, eps) * (1.0 + w)


def position_vectors(T: int, D: int) -> torch.Tensor:
    """row p: entries (2i, 2i + 1) = (sin, cos) of p * 10000^(-2i / D)"""
    out = torch.zeros(T, D, dtype=DT)
    for p in range(T):
        for c in range(D):
            ang = p * 10000.0 ** (-2.0 * (c // 2) / D)
            out[p, c] = math.cos(ang) if c % 2 else math.sin(ang)
    return out


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """row t becomes h_t + (h_(t-1) - h_t) * mu with the rows as they came in; row -1 is zero"""
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        prev = h[t - 1] if t > 0 else torch.zeros_like(h[0])
        out[t] = h[t] + (prev - h[t]) * mu
    return out


def _visible(i: int, size) -> List[int]:
    return [j for j in range(i + 1) if not size or i - j < size]


def talking_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """mixer 'attention': biased projections, unit-RMS q, k and v per head, windowed softmax, softmax weights mixed over the heads
    by `talk`, sigmoid output gate"""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads", H)
    q = unit_rms((h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d), eps)
    k = unit_rms((h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d), eps)
    v = unit_rms((h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, e), eps)
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, e, dtype=DT)
    for i in range(T):
        js = _visible(i, size)
        weights = torch.zeros(H, len(js), dtype=DT)
        for hd in range(H):
            g = hd // (H // G)
            sc = torch.stack([q[i, hd] @ k[j, g] for j in js]) * m["scale"]
            weights[hd] = torch.softmax(sc, 0)
        mixed = w[p + "talk"] @ weights                       # mixed[h, j] = sum_g talk[h, g] weights[g, j]
        for hd in range(H):
            g = hd // (H // G)
            out[i, hd] = mixed[hd] @ torch.stack([v[j, g] for j in js])
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * e) * gate) @ w[p + "o"].T


def sink_latent_attention(h, w, p: str, m: dict, eps: float):
    """mixer 'latent_attention': queries through a normed latent, keys and values from one normed latent per token, windowed softmax
    whose denominator also holds exp(sink) per head, one sigmoid gate per head"""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d)
    c = unit_rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, e)
    size = (m.get("mask") or {}).get("size")
    gate = torch.sigmoid(h @ w[p + "g"].T)                    # [T, H]
    out = torch.zeros(T, H, e, dtype=DT)
    for i in range(T):
        js = _visible(i, size)
        for hd in range(H):
            sc = torch.stack([q[i, hd] @ k[j, hd] for j in js]) * m["scale"]
            top = max(float(sc.max()), float(w[p + "sink"][hd]))
            ex = torch.exp(sc - top)
            wts = ex / (ex.sum() + math.exp(float(w[p + "sink"][hd]) - top))
            out[i, hd] = (wts @ torch.stack([v[j, hd] for j in js])) * gate[i, hd]
    return out.reshape(T, H * e) @ w[p + "o"].T


def mlstm(h, w, p: str, m: dict, eps: float):
    """mixer 'mlstm': per head a matrix memory S [d, e], a normaliser n [d] and a running maximum m that starts at 0"""
    T = h.shape[0]
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, e)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, e, dtype=DT)
    for hd in range(H):
        S = torch.zeros(d, e, dtype=DT)
        n = torch.zeros(d, dtype=DT)
        mx = 0.0
        for t in range(T):
            new = max(float(gf[t, hd]) + mx, float(gi[t, hd]))
            keep, take = math.exp(float(gf[t, hd]) + mx - new), math.exp(float(gi[t, hd]) - new)
            S = keep * S + take * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + take * k[t, hd]
            mx = new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * e) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def chosen_softmax_experts(h, w, p: str, f: dict):
    """feed-forward 'moe': the `top` largest router logits are chosen, weights = softmax over the chosen logits only"""
    r = f["router"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(r["experts"]), key=lambda e: (-float(z[t, e]), e))[: r["top"]]
        wts = torch.softmax(torch.stack([z[t, e] for e in order]), 0)
        for wt, e in zip(wts, order):
            a = h[t] @ w[f"{p}e{e}.gate"].T
            out[t] += wt * ((a * torch.sigmoid(a) * (h[t] @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T)
    return out


MIXERS = {"attention": talking_attention, "latent_attention": sink_latent_attention, "mlstm": mlstm}


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer index, pass number or None): the order in which layers run; a pass number marks the first layer of a pass of the loop"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of one sequence from position 0; `residuals` collects the stream after every layer run"""
    w = {k: v.to(DT) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T, D = len(tokens), cfg["width"]
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0) + position_vectors(T, D)
    for i, t in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if t is not None:
            x = x + w["loop.step"][t]
        hn = token_shift(one_plus_norm(x, w[p + "norm1"], eps), w[p + "shift"])
        x = x + one_plus_norm(MIXERS[layer["type"]](hn, w, p + "mix.", layer["mixer"], eps), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = chosen_softmax_experts(one_plus_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
            x = x + one_plus_norm(y, w[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return one_plus_norm(x, w["final.norm"], eps) @ w["head"].T


def random_weights(cfg: dict, seed: int = 0, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-representable random tensors under the checkpoint's names"""
    gen = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def mat(name, n, k, s=1.0):
        out[name] = (torch.randn(n, k, generator=gen) * s * scale / math.sqrt(k)).to(torch.bfloat16).float()

    def vec(name, n, s=0.3, mean=0.0):
        out[name] = (torch.randn(n, generator=gen) * s + mean).to(torch.bfloat16).float()

    mat("embed", cfg["vocab"], D, math.sqrt(D) * 0.5)
    mat("head", cfg["vocab"], D)
    vec("final.norm", D)
    loop = cfg.get("loop")
    if loop:
        out["loop.step"] = (torch.randn(loop["times"], D, generator=gen) * 0.5).to(torch.bfloat16).float()
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for k in ("norm1", "norm1b", "norm2", "norm2b"):
            vec(p + k, D)
        out[p + "shift"] = torch.rand(D, generator=gen).to(torch.bfloat16).float()
        H, d, e = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m.get("kv_heads", H)
            for k, n in (("q", H * d), ("k", G * d), ("v", G * e)):
                mat(p + "mix." + k, n, D)
                vec(p + "mix." + k + ".b", n)
            out[p + "mix.talk"] = (torch.eye(H) * 0.6 + torch.randn(H, H, generator=gen) * 0.3).to(torch.bfloat16).float()
            mat(p + "mix.g", H * e, D)
            mat(p + "mix.o", D, H * e)
        elif layer["type"] == "latent_attention":
            mat(p + "mix.dq", m["q_rank"], D)
            vec(p + "mix.dq.norm", m["q_rank"], mean=1.0)
            mat(p + "mix.uq", H * d, m["q_rank"], 2.0)
            mat(p + "mix.dkv", m["kv_rank"], D)
            vec(p + "mix.dkv.norm", m["kv_rank"], mean=1.0)
            mat(p + "mix.uk", H * d, m["kv_rank"], 2.0)
            mat(p + "mix.uv", H * e, m["kv_rank"])
            vec(p + "mix.sink", H, s=1.0)
            mat(p + "mix.g", H, D)
            mat(p + "mix.o", D, H * e)
        elif layer["type"] == "mlstm":
            for k, n in (("q", H * d), ("k", H * d), ("v", H * e), ("g", H * e)):
                mat(p + "mix." + k, n, D, 2.0 if k in "qk" else 1.0)
            mat(p + "mix.o", D, H * e)
            vec(p + "mix.norm", H * e, mean=1.0)
            for k in "if":
                mat(p + "mix." + k, H, D, 3.0)
                vec(p + "mix." + k + ".b", H, s=1.0, mean=2.0 if k == "f" else 0.0)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            mat(p + "mlp.router", E, D, 2.0)
            vec(p + "mlp.router.b", E, s=0.5)
            for e_ in range(E):
                mat(f"{p}mlp.e{e_}.gate", ff, D)
                mat(f"{p}mlp.e{e_}.up", ff, D)
                mat(f"{p}mlp.e{e_}.down", D, ff)
    return out
