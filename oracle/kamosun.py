"""Plain, slow float64 implementation of the Kamosun layers: what the tests compare the Dynamic-Tanh norm, parallel gated layers,
depth average, chunked and key/value-sharing attention, capped causal attention with rescaled interleaved rotation, lightning
attention, the clamped gated feed-forward and the input-weighted sigmoid router of leopard_b200/seqlm.py with.  One function per
mechanism, whole sequences from position 0 only, explicit loops over tokens, nothing shared with the product path: it takes the
parsed config.json and a {name: tensor} dict.

Notation: T tokens, D width, H query heads, G key / value heads (query head h reads group h // (H // G)), d key size, e value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

DT = torch.float64
GLU_ALPHA = 1.702


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x, w: Dict[str, torch.Tensor], name: str):
    """tanh(alpha x) * gain + shift: a norm without statistics"""
    return torch.tanh(w[name + ".alpha"].reshape(()) * x) * w[name] + w[name + ".b"]


def frequencies(rot: dict) -> List[float]:
    """f_i = base^(-2i / dims); with `scaling`: long wavelengths are divided by `factor`, short ones kept, a linear blend between"""
    n = rot["dims"] // 2
    f = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(n)]
    s = rot.get("scaling")
    if s:
        out = []
        for fi in f:
            wavelength = 2 * math.pi / fi
            if wavelength < s["original"] / s["high"]:
                out.append(fi)
            elif wavelength > s["original"] / s["low"]:
                out.append(fi / s["factor"])
            else:
                t = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
                out.append((1 - t) * fi / s["factor"] + t * fi)
        f = out
    return f


def rotate(x: torch.Tensor, pos: int, rot: Optional[dict], interleaved: bool) -> torch.Tensor:
    """one head's vector at position pos; only the first rot.dims entries turn"""
    if not rot or not rot.get("dims"):
        return x.clone()
    out = x.clone()
    n = rot["dims"] // 2
    for i, fi in enumerate(frequencies(rot)):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + n)
        c, s = math.cos(pos * fi), math.sin(pos * fi)
        out[a] = x[a] * c - x[b] * s
        out[b] = x[b] * c + x[a] * s
    return out


def keys_and_values(h, w, p: str, m: dict, eps: float, bias: bool, interleaved: bool):
    """what an attention layer caches: keys after norm and rotation [T, G, d], values [T, G, e]"""
    T = h.shape[0]
    G, d, e = m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    k = h @ w[p + "k"].T
    v = h @ w[p + "v"].T
    if bias:
        k = k + w[p + "k.b"]
        v = v + w[p + "v.b"]
    k = unit_rms(k.view(T, G, d), eps) * w[p + "k.norm"]
    k = torch.stack([torch.stack([rotate(k[t, g], t, m.get("rot"), interleaved) for g in range(G)]) for t in range(T)])
    return k, v.view(T, G, e)


def softmax_attention(h, w, p: str, m: dict, eps: float, bias: bool, interleaved: bool, kv: Optional[Tuple] = None):
    """grouped-query softmax attention; mask.size = c: position i sees j <= i of its own block of c positions (blocks counted from
    position 0); softcap: score <- cap tanh(score / cap).  Returns (output [T, D], (keys, values))."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m.get("vdim", m["dim"])
    G = m.get("kv_heads", H)
    if kv is None:
        kv = keys_and_values(h, w, p, m, eps, bias, interleaved)
    k, v = kv
    q = h @ w[p + "q"].T
    if bias:
        q = q + w[p + "q.b"]
    q = unit_rms(q.view(T, H, d), eps) * w[p + "q.norm"]
    chunk = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    out = torch.zeros(T, H, e, dtype=DT)
    for i in range(T):
        js = [j for j in range(i + 1) if not chunk or j // chunk == i // chunk]
        for hd in range(H):
            g = hd // (H // G)
            qi = rotate(q[i, hd], i, m.get("rot"), interleaved)
            sc = torch.stack([qi @ k[j, g] for j in js]) * m["scale"]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            out[i, hd] = torch.softmax(sc, 0) @ torch.stack([v[j, g] for j in js])
    y = out.reshape(T, H * e) @ w[p + "o"].T
    if bias:
        y = y + w[p + "o.b"]
    return y, kv


def lightning_attention(h, w, p: str, m: dict, eps: float):
    """per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu(projection); the concatenated heads are
    RMS-normed with a gain, gated by sigmoid(W_g h) and projected"""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m.get("vdim", m["dim"])
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, e)
    out = torch.zeros(T, H, e, dtype=DT)
    for hd in range(H):
        S = torch.zeros(d, e, dtype=DT)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = unit_rms(out.reshape(T, H * e), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p: str, m: dict, eps: float):
    """half the sum of the two branches, each RMS-normed over the width with its own gain"""
    left, _ = softmax_attention(h, w, p + "left.", m["left"], eps, bias=False, interleaved=True)
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * w[p + "left.out"] + unit_rms(right, eps) * w[p + "right.out"])


def clamped_glu(h, w, p: str, limit: float):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GLU_ALPHA * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p: str, top: int):
    """(chosen experts, their sigmoid scores) per token; the largest scores win, ties to the lower index"""
    s = torch.sigmoid(h @ w[p + "router"].T)
    idx, wts = [], []
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:top]
        idx.append(order)
        wts.append([float(s[t, e]) for e in order])
    return idx, wts


def feed_forward(h, w, p: str, f: dict):
    if f["kind"] == "dense":
        return clamped_glu(h, w, p, f["limit"])
    idx, wts = route(h, w, p, f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t], wts[t]):      # the score multiplies the expert's INPUT
            out[t] += clamped_glu((s * h[t]).unsqueeze(0), w, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + clamped_glu(h, w, p + "shared.", f["shared"]["limit"])
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, taps: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of one whole sequence from position 0; taps (a list) receives the stream after every layer"""
    w = {k: v.to(DT) for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    results = [x]                       # X_0 and every layer's own result
    caches = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h1 = dynamic_tanh(x, w, p + "norm1")
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, caches[i] = softmax_attention(h1, w, p + "mix.", m, eps, bias=True, interleaved=False,
                                             kv=caches[src] if src is not None else None)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h1, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        delta = y * torch.sigmoid(h1 @ w[p + "rg1"].T + w[p + "rg1.b"])
        if layer.get("mlp") is not None:
            h2 = dynamic_tanh(x, w, p + "norm2")
            delta = delta + feed_forward(h2, w, p + "mlp.", layer["mlp"]) * torch.sigmoid(h2 @ w[p + "rg2"].T + w[p + "rg2.b"])
        results.append(x + mult * delta)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        if taps is not None:
            taps.append(x.clone())
    return dynamic_tanh(x, w, "final.norm") @ w["head"].T


def random_weights(cfg: dict, seed: int = 0, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-representable random tensors under the checkpoint's names"""
    gen = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def mat(name, n, k, s=1.0):
        out[name] = (torch.randn(n, k, generator=gen) * s * scale / math.sqrt(k)).to(torch.bfloat16).float()

    def vec(name, n, s=0.3, mean=0.0):
        out[name] = (torch.randn(n, generator=gen) * s + mean).to(torch.bfloat16).float()

    def dyt(name):
        vec(name, D, mean=1.0)
        vec(name + ".b", D, s=0.2)
        out[name + ".alpha"] = (torch.rand((), generator=gen) * 0.8 + 0.4).to(torch.bfloat16).float()

    def glu(p, ff):
        mat(p + "gate", ff, D, 2.0)
        mat(p + "up", ff, D, 2.0)
        mat(p + "down", D, ff)

    def attention(p, m, bias):
        H, d, e = m["heads"], m["dim"], m.get("vdim", m["dim"])
        G = m.get("kv_heads", H)
        own = m.get("kv_from") is None
        for k, n in (("q", H * d), ("k", G * d), ("v", G * e)):
            if k == "q" or own:
                mat(p + k, n, D)
                if bias:
                    vec(p + k + ".b", n)
        vec(p + "q.norm", d, mean=1.0)
        if own:
            vec(p + "k.norm", d, mean=1.0)
        mat(p + "o", D, H * e)
        if bias:
            vec(p + "o.b", D)

    mat("embed", cfg["vocab"], D, math.sqrt(D))
    mat("head", cfg["vocab"], D)
    dyt("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        dyt(p + "norm1")
        mat(p + "rg1", D, D)
        vec(p + "rg1.b", D, s=0.5)
        out[p + "dwa"] = (torch.randn(i + 2, generator=gen) * 0.3 + torch.tensor([0.0] * (i + 1) + [1.0])).to(torch.bfloat16).float()
        if layer["type"] == "attention":
            attention(p + "mix.", m, True)
        elif layer["type"] == "parallel":
            attention(p + "mix.left.", m["left"], False)
            r = m["right"]
            H, d, e = r["heads"], r["dim"], r.get("vdim", r["dim"])
            for k, n in (("q", H * d), ("k", H * d), ("v", H * e), ("g", H * e)):
                mat(p + "mix.right." + k, n, D, 2.0)
            mat(p + "mix.right.o", D, H * e)
            vec(p + "mix.right.norm", H * e, mean=1.0)
            vec(p + "mix.left.out", D, mean=1.0)
            vec(p + "mix.right.out", D, mean=1.0)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is None:
            continue
        dyt(p + "norm2")
        mat(p + "rg2", D, D)
        vec(p + "rg2.b", D, s=0.5)
        if f["kind"] == "dense":
            glu(p + "mlp.", f["ff"])
        else:
            mat(p + "mlp.router", f["router"]["experts"], D, 3.0)
            for e_ in range(f["router"]["experts"]):
                glu(f"{p}mlp.e{e_}.", f["expert"]["ff"])
            if f.get("shared"):
                glu(p + "mlp.shared.", f["shared"]["ff"])
    return out
