"""Decoder-only language models described as a LIST OF LAYERS, on the 32-bit residual-stream kernels.

A model is a `SeqLMConfig`: vocabulary, width, norm epsilon and style, and a tuple of `LayerConfig`s, each naming its sequence mixer
(`RetentionConfig`, `LatentAttentionConfig`, `WindowAttentionConfig`, `MinGRUConfig`, `MLSTMConfig`, or a `ParallelMixerConfig` of
two of them side by side) and its feed-forward
(`DenseFFConfig`, `MoEConfig` or none); a layer may run on another layer's weights with a cache or state of its own (a looped stack
is such a list), shift its mixer's input towards the previous token's, and add a learned vector to the stream before it runs.  Every mechanism is a
separate native entry point with its constants as arguments (include/leopard_b200.h, "32-BIT RESIDUAL-STREAM MODELS"), so another
design is another list.  The residual stream, norms, routers, rotary angles, attention scores and recurrent state are fp32; matrix
products take bf16 weights and, in the serving precision, bf16 activations with fp32 accumulation ("bfloat16"), or fp32 activations
on fp32 FMAs ("float32": a true 32-bit forward, no tensor-core rounding).

`SeqLMEngine.step(entries)` is THE step function: a packed batch of requests, each bringing its next tokens (a whole prompt, a
portion of one, or one token), runs from the cache and state that earlier steps left (leopard_b200/seqcache.py) and returns the
logits of the rows asked for.  The scheduler (leopard_b200/scheduler.py), greedy generation and the trace replayer
(leopard_b200/cli.py) all drive this function.  Host code does allocation, shapes and index tables only; there is no CPU fallback
(a CPU device is accepted only together with an injected library: the tests run the kernel sources under their CPU emulator).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib
from .seqcache import SequenceCache

F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32
TENSOR_CORE_MIN_ROWS = 64
MOE_PAIRS_MAX = 64             # up to this many (token, choice) pairs the experts run as one-row weight-streaming problems
MAX_DECODE_GRAPHS = 32         # captured decode layouts kept at a time
PAGE_TABLE_STEP = 16           # decode batches round their page-table width up to a multiple of this


# ---------------------------------------------------------------------------------------------------------------- configuration
@dataclass(frozen=True)
class YarnScaling:
    """Frequency rescale for context extension: high-frequency pairs keep their frequency, low-frequency pairs are divided by
    `factor`, with a linear ramp between the pair indices at which `original` positions make `fast` / `slow` full turns; cos and sin
    are multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LinearScaling:
    """Position interpolation: every frequency is divided by `factor`."""
    factor: float


@dataclass(frozen=True)
class BandScaling:
    """Frequency rescale by wavelength bands: a pair whose wavelength is shorter than original / high keeps its frequency f, one
    whose wavelength is longer than original / low gets f / factor, and between the two the blend (1 - s) f / factor + s f with
    s = (original / wavelength - low) / (high - low)."""
    factor: float
    original: float
    low: float
    high: float


@dataclass(frozen=True)
class RotaryConfig:
    dims: int                      # leading dimensions of a head that are rotated
    base: float
    layout: str = "half"           # "half": i pairs with i + dims/2; "interleaved": 2i pairs with 2i + 1
    scaling: Union[YarnScaling, LinearScaling, BandScaling, None] = None


def rotary_table(rot: RotaryConfig) -> Tuple[torch.Tensor, float]:
    """(inv_freq fp32 [dims/2], magnitude factor) — computed in float64, rounded once."""
    if rot.dims % 2:
        raise ValueError("rotary dims must be even")
    n = rot.dims // 2
    i = np.arange(n, dtype=np.float64)
    f = rot.base ** (-2.0 * i / rot.dims) if n else np.zeros(0)
    mag = 1.0
    s = rot.scaling
    if isinstance(s, LinearScaling):
        f = f / s.factor
    elif isinstance(s, BandScaling):
        wavelength = 2 * math.pi / f
        blend = (s.original / wavelength - s.low) / (s.high - s.low) if s.high != s.low else np.ones_like(f)
        mixed = (1.0 - blend) * f / s.factor + blend * f
        f = np.where(wavelength < s.original / s.high, f, np.where(wavelength > s.original / s.low, f / s.factor, mixed))
    elif s is not None:
        def pair_index(turns):      # the (fractional) pair index whose wavelength fits `turns` times into the original context
            return rot.dims * math.log(s.original / (2 * math.pi * turns)) / (2 * math.log(rot.base))
        lo = max(math.floor(pair_index(s.fast)), 0)
        hi = min(math.ceil(pair_index(s.slow)), rot.dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / s.factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(s.factor) + 1.0
    return torch.from_numpy(f.astype(np.float32)), float(mag)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: RotaryConfig
    # "retention": rotated q and k, k scaled by dim^-1/2, every head's output divided by its root mean square and gated by silu(mix.g h);
    # "lightning": q, k and v are silu(projection), no rotation and no scale, the concatenated heads are RMS-normed together with the
    # gain mix.norm and gated by sigmoid(mix.g h)
    form: str = "retention"

    @property
    def k_scale(self) -> float:
        return self.dim ** -0.5 if self.form == "retention" else 1.0


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                       # unrotated query / key dimensions per head
    rot_dim: int                   # rotated dimensions per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    window: Optional[int] = None   # position i sees j with 0 <= i - j < window; None: every earlier position
    q_rank: int = 0                # > 0: queries go through a normed latent of this size (mix.dq, mix.dq.norm, mix.uq) instead of mix.q
    sink: bool = False             # exp(mix.sink[h]) joins head h's softmax denominator
    head_gate: bool = False        # head h's output is multiplied by sigmoid(mix.g h)[h]


@dataclass(frozen=True)
class WindowAttentionConfig:
    """Grouped-query softmax attention over cached keys and values with sliding-window visibility (csrc/lp_winattn.cu)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig
    # RMS norm of q and k before rotation: "head" (per head, gain [dim]), "unit" (per head, no gain), "full" (whole projection), "none"
    qk_norm: str = "none"
    window: Optional[int] = None   # position i sees j with 0 <= i - j < window; None: every earlier position
    keep_first: int = 0            # the first tokens of a request stay visible beyond the window
    pool: int = 0                  # > 0: blocks of this many tokens wholly before the window are seen as one mean key / value
    softcap: float = 0.0           # > 0: score <- softcap tanh(score / softcap)
    sink: bool = False             # one added to the softmax denominator
    value_rot: Optional[RotaryConfig] = None   # values rotated by their position, outputs turned back by the query's
    bias: bool = False             # q, k and v projections have biases (mix.q.b, mix.k.b, mix.v.b)
    value_norm: bool = False       # every value head is divided by its root mean square before it is cached
    talking_heads: bool = False    # softmax weights mixed over the heads by mix.talk [heads, heads] before they meet the values
    out_gate: bool = False         # the concatenated heads are multiplied by sigmoid(mix.g h)
    chunk: Optional[int] = None    # position i sees only j <= i of its own block, floor(j / chunk) = floor(i / chunk), counted from position 0
    out_bias: bool = False         # the output projection has a bias (mix.o.b)
    # the layer has no key / value tensors: it reads the cache rows of that layer (keys after norm and rotation, values), written
    # earlier in the same step, with its own queries, visibility and everything else
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class MinGRUConfig:
    """Gated recurrence whose gates read only the current token (csrc/lp_mingru.cu)."""
    width: int


@dataclass(frozen=True)
class MLSTMConfig:
    """Matrix memory with exponential gates and a running stabiliser (csrc/lp_mlstm.cu); the gates' pre-activations are capped by
    gate_cap * tanh(. / gate_cap)."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelMixerConfig:
    """Two mixers side by side on the same input (tensors under mix.left.* and mix.right.*); the result is half the sum of the two
    outputs, each first RMS-normed over the model width with its own plain gain (mix.left.out, mix.right.out)."""
    left: Union[RetentionConfig, LatentAttentionConfig, WindowAttentionConfig, MinGRUConfig, MLSTMConfig]
    right: Union[RetentionConfig, LatentAttentionConfig, WindowAttentionConfig, MinGRUConfig, MLSTMConfig]


GLU_SLOPE = 1.702                  # the sigmoid's slope in the clamped gated unit


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int
    # "xielu" (two learned constants in mlp.act), "relu2" (the square of relu), or "clamp_glu": with g = min(mlp.gate h, limit) and
    # u = clamp(mlp.up h, -limit, limit) the hidden vector is g sigmoid(1.702 g) (u + 1)
    act: str = "xielu"
    limit: float = 0.0


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    expert_ff: int
    n_groups: int = 1
    keep_groups: int = 1
    shared_ff: int = 0             # 0: no shared expert
    # "grouped_sigmoid": sigmoid scores, choice bias, best groups, weights = chosen scores / their sum;
    # "softmax_top": logits + mlp.router.b, the largest are chosen, weights = softmax over the chosen logits;
    # "sigmoid_input": sigmoid scores, the largest are chosen, and a chosen expert runs on score * h (its output is not weighted)
    router: str = "grouped_sigmoid"
    act: str = "silu_glu"          # the experts' unit: "silu_glu" (silu(gate) * up) or "clamp_glu" (DenseFFConfig) with the limits below
    limit: float = 0.0
    shared_limit: float = 0.0
    shared_gate: bool = True       # the shared expert's output is multiplied by sigmoid(mlp.shared.sg h); False: added as it is


@dataclass(frozen=True)
class LayerConfig:
    mixer: Union[RetentionConfig, LatentAttentionConfig, WindowAttentionConfig, MinGRUConfig, MLSTMConfig, ParallelMixerConfig]
    ff: Union[DenseFFConfig, MoEConfig, None]
    weights_of: Optional[int] = None   # run on that layer's tensors (mixer, feed-forward, norms); cache and state stay this layer's own
    # the mixer reads h_t + (h_(t-1) - h_t) * shift per channel instead of h_t (h: the normed stream; the previous token's h is part of
    # the request's state, zeros before the first token); the vector is the layer's tensor `shift`
    token_shift: bool = False
    add_before: Optional[Tuple[str, int]] = None   # (tensor, row): that row is added to the stream right before this layer runs


@dataclass(frozen=True)
class SeqLMConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[LayerConfig, ...]
    # "sandwich": x <- x + norm_b(sublayer(norm_a(x))), every norm with ONE gain; "pre": x <- x + residual_mult * sublayer(norm(x)),
    # the norm's gain a vector stored around zero (x / rms * (1 + w)); "sandwich_vector": the sandwich form with such vector gains;
    # "parallel_dyt": x <- x + residual_mult * (mixer(norm1(x)) + ff(norm2(x))), both sublayers on the same x, every norm (the final
    # one too) a Dynamic Tanh tanh(alpha x) * w + b with the tensors <name>, <name>.alpha, <name>.b
    norm: str = "sandwich"
    residual_mult: float = 1.0
    embed_scale: float = 1.0
    # > 0: absolute sinusoidal positions are added to the embedding, entries (2i, 2i + 1) = (sin, cos)(p * base^(-2i / width))
    position_base: float = 0.0
    # every sublayer's output is multiplied element by element by sigmoid(W h + b) of the sublayer's own input h (rg1, rg1.b for the
    # mixer, rg2, rg2.b for the feed-forward) before it joins the stream
    residual_gate: bool = False
    # what goes on to the next layer (and to the output) is sum_j dwa[j] X_j over the embedding output X_0 and the results X_1 ..
    # X_(i+1) of the layers so far (the layer's tensor dwa [i + 2])
    depth_average: bool = False


# the weight of every mixer's first product of its operand (SeqLMWeights)
FIRST_PRODUCT = {RetentionConfig: "w_qkvg", LatentAttentionConfig: "w_qdkv", WindowAttentionConfig: "w_qkv", MinGRUConfig: "w_zxg",
                 MLSTMConfig: "w_proj"}


def softplus(x: float) -> float:
    return math.log1p(math.exp(-abs(x))) + max(x, 0.0)


# ---------------------------------------------------------------------------------------------------------------- weights
class SeqLMWeights:
    """Device tensors in the layout the kernels read.  `get(name)` returns a checkpoint tensor; `name(layer, key)` maps the generic
    keys used here (norm1, norm1b, norm2, norm2b, mix.*, mlp.*; embed, final.norm, head with layer None) to checkpoint names."""

    def __init__(self, cfg: SeqLMConfig, get: Callable[[str], torch.Tensor], name: Callable[[Optional[int], str], str], device):
        self.cfg, self.device = cfg, torch.device(device)
        dev = self.device

        def w(layer, key, shape=None):
            t = get(name(layer, key))
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name(layer, key)}: shape {tuple(t.shape)}, expected {tuple(shape)}")
            return t

        def mat(t):
            return t.to(BF16).contiguous().to(dev)

        def num(layer, key):
            return float(w(layer, key).float().reshape(-1)[0])

        def vec(t):
            return t.float().contiguous().to(dev)

        def one_plus(layer, key):           # a gain stored around zero
            return (1.0 + w(layer, key, (cfg.width,)).float()).contiguous().to(dev)

        if cfg.norm not in ("sandwich", "pre", "sandwich_vector", "parallel_dyt"):
            raise ValueError(f"unknown norm style {cfg.norm!r}")
        pre = cfg.norm == "pre"
        dyt = cfg.norm == "parallel_dyt"
        if (cfg.residual_gate or cfg.depth_average) and not dyt:
            raise ValueError("gated residual branches and the depth average belong to the parallel layer form")
        vector = cfg.norm != "sandwich"

        def dyt_norm(layer, key):           # (alpha, gain, shift) of a Dynamic Tanh
            return (num(layer, key + ".alpha"), vec(w(layer, key, (cfg.width,))), vec(w(layer, key + ".b", (cfg.width,))))

        D = cfg.width
        self.embed = mat(w(None, "embed", (cfg.vocab, D)))
        self.head = mat(w(None, "head", (cfg.vocab, D)))
        self.final_gain = dyt_norm(None, "final.norm") if dyt else one_plus(None, "final.norm") if vector else num(None, "final.norm")
        if cfg.position_base > 0:      # frequencies in float64, split into two floats hi + lo
            f64 = cfg.position_base ** (-2.0 * np.arange((D + 1) // 2, dtype=np.float64) / D)
            hi = f64.astype(np.float32)
            lo = (f64 - hi.astype(np.float64)).astype(np.float32)
            self.position_freq = torch.from_numpy(np.concatenate([hi, lo])).to(dev)
        # vectors added to the stream before a layer: per layer of the list, also for one that runs on another layer's tensors
        self.add_before: List[Optional[torch.Tensor]] = []
        for lc in cfg.layers:
            if lc.add_before is None:
                self.add_before.append(None)
            else:
                key, row = lc.add_before
                t = w(None, key)
                if t.dim() != 2 or t.shape[1] != D or not 0 <= row < t.shape[0]:
                    raise ValueError(f"{name(None, key)}: shape {tuple(t.shape)} has no row {row} of width {D}")
                self.add_before.append(vec(t[row]))
        self.layers: List[Dict[str, object]] = []
        for i, lc in enumerate(cfg.layers):
            if lc.weights_of is not None:
                j = lc.weights_of
                if not 0 <= j < len(cfg.layers) or cfg.layers[j].weights_of is not None:
                    raise ValueError(f"layer {i}: weights_of = {j} must name a layer that has tensors of its own")
                if (cfg.layers[j].mixer, cfg.layers[j].ff, cfg.layers[j].token_shift) != (lc.mixer, lc.ff, lc.token_shift):
                    raise ValueError(f"layer {i} differs from layer {j}, whose weights it uses")
                self.layers.append(None)              # linked below, once every owner is loaded
                continue
            if dyt:
                lw: Dict[str, object] = {"norm1": dyt_norm(i, "norm1")}
            elif pre:
                lw = {"norm1": one_plus(i, "norm1")}
            elif vector:
                lw = {k: one_plus(i, k) for k in ("norm1", "norm1b")}
            else:
                lw = {k: num(i, k) for k in ("norm1", "norm1b")}
            if lc.token_shift:
                lw["shift"] = vec(w(i, "shift", (D,)))
            def mixer_weights(m, pfx: str) -> Dict[str, object]:
                """the tensors of one mixer, named <pfx><key> in the checkpoint"""
                mw: Dict[str, object] = {}
                if not isinstance(m, (MinGRUConfig, MLSTMConfig)):
                    inv_freq, mag = rotary_table(m.rot)
                    mw["inv_freq"], mw["rot_mag"] = inv_freq.to(dev), mag
                if isinstance(m, MLSTMConfig):
                    hd, hv = m.heads * m.dim, m.heads * m.vdim
                    mw["w_proj"] = mat(torch.cat([w(i, pfx + "q", (hd, D)), w(i, pfx + "k", (hd, D)), w(i, pfx + "v", (hv, D)), w(i, pfx + "g", (hv, D)),
                                                  w(i, pfx + "i", (m.heads, D)), w(i, pfx + "f", (m.heads, D))], 0))
                    mw["i_bias"], mw["f_bias"] = vec(w(i, pfx + "i.b", (m.heads,))), vec(w(i, pfx + "f.b", (m.heads,)))
                    mw["out_gain"] = vec(w(i, pfx + "norm", (hv,)))
                    mw["w_o"] = mat(w(i, pfx + "o", (D, hv)))
                elif isinstance(m, MinGRUConfig):
                    mw["w_zxg"] = mat(torch.cat([w(i, pfx + "z", (m.width, D)), w(i, pfx + "x", (m.width, D)), w(i, pfx + "g", (m.width, D))], 0))
                    mw["z_bias"], mw["x_bias"] = vec(w(i, pfx + "z.b", (m.width,))), vec(w(i, pfx + "x.b", (m.width,)))
                    mw["w_o"] = mat(w(i, pfx + "o", (D, m.width)))
                elif isinstance(m, WindowAttentionConfig):
                    if m.heads % m.kv_heads:
                        raise ValueError(f"layer {i}: {m.heads} query heads over {m.kv_heads} key / value heads")
                    parts = [w(i, pfx + "q", (m.heads * m.dim, D))]
                    if m.kv_from is None:
                        parts += [w(i, pfx + "k", (m.kv_heads * m.dim, D)), w(i, pfx + "v", (m.kv_heads * m.vdim, D))]
                    if m.out_gate:
                        parts.append(w(i, pfx + "g", (m.heads * m.vdim, D)))
                    mw["w_qkv"] = mat(torch.cat(parts, 0))
                    if m.bias:
                        mw["q_bias"] = vec(w(i, pfx + "q.b", (m.heads * m.dim,)))
                        if m.kv_from is None:
                            mw["k_bias"], mw["v_bias"] = vec(w(i, pfx + "k.b", (m.kv_heads * m.dim,))), vec(w(i, pfx + "v.b", (m.kv_heads * m.vdim,)))
                    if m.out_bias:
                        mw["o_bias"] = vec(w(i, pfx + "o.b", (D,)))
                    if m.talking_heads:
                        mw["talk"] = vec(w(i, pfx + "talk", (m.heads, m.heads)))
                    elif m.out_gate:      # the gate rides on the mixing kernel: no mixing is the unit matrix
                        mw["talk"] = torch.eye(m.heads, dtype=F32).to(dev)
                    if (m.talking_heads or m.out_gate) and m.value_rot is not None:
                        raise ValueError(f"layer {i}: mixed or gated heads with rotated values are not supported")
                    if m.qk_norm == "head":      # a layer without keys of its own hands the kernel its query gain twice (the second is unused)
                        mw["q_gain"] = vec(w(i, pfx + "q.norm", (m.dim,)))
                        mw["k_gain"] = vec(w(i, pfx + "k.norm", (m.dim,))) if m.kv_from is None else mw["q_gain"]
                    elif m.qk_norm == "full":
                        mw["q_gain"] = vec(w(i, pfx + "q.norm", (m.heads * m.dim,)))
                        mw["k_gain"] = vec(w(i, pfx + "k.norm", (m.kv_heads * m.dim,))) if m.kv_from is None else mw["q_gain"]
                    elif m.qk_norm not in ("none", "unit"):
                        raise ValueError(f"layer {i}: unknown query / key norm {m.qk_norm!r}")
                    if m.value_rot is not None:
                        mw["v_inv_freq"] = rotary_table(m.value_rot)[0].to(dev)
                    mw["w_o"] = mat(w(i, pfx + "o", (D, m.heads * m.vdim)))
                elif isinstance(m, RetentionConfig):
                    if len(m.decay) != m.heads:
                        raise ValueError(f"layer {i}: {len(m.decay)} decays for {m.heads} heads")
                    mw["w_qkvg"] = mat(torch.cat([w(i, pfx + "q", (m.heads * m.dim, D)), w(i, pfx + "k", (m.heads * m.dim, D)),
                                                  w(i, pfx + "v", (m.heads * m.vdim, D)), w(i, pfx + "g", (m.heads * m.vdim, D))], 0))
                    mw["w_o"] = mat(w(i, pfx + "o", (D, m.heads * m.vdim)))
                    mw["decay"] = torch.tensor(m.decay, dtype=torch.float64).to(F32).to(dev)
                    if m.form == "lightning":
                        mw["out_gain"] = vec(w(i, pfx + "norm", (m.heads * m.vdim,)))
                    elif m.form != "retention":
                        raise ValueError(f"layer {i}: unknown retention form {m.form!r}")
                else:
                    per = m.dim + m.rot_dim
                    # one product of h: [queries or their latent | key / value latent (+ shared rotated key) | one gate per head]
                    parts = [w(i, pfx + "dq", (m.q_rank, D)) if m.q_rank else w(i, pfx + "q", (m.heads * per, D)),
                             w(i, pfx + "dkv", (m.kv_rank + m.rot_dim, D))]
                    if m.head_gate:
                        parts.append(w(i, pfx + "g", (m.heads, D)))
                    mw["w_qdkv"] = mat(torch.cat(parts, 0))
                    if m.q_rank:
                        mw["cq_gain"] = vec(w(i, pfx + "dq.norm", (m.q_rank,)))
                        mw["w_uq"] = mat(w(i, pfx + "uq", (m.heads * per, m.q_rank)))
                    if m.sink:
                        mw["sink"] = vec(w(i, pfx + "sink", (m.heads,)))
                    mw["c_gain"] = w(i, pfx + "dkv.norm", (m.kv_rank,)).float().contiguous().to(dev)
                    uk = w(i, pfx + "uk", (m.heads * m.dim, m.kv_rank))
                    mw["w_ukT"] = mat(uk.reshape(m.heads, m.dim, m.kv_rank).transpose(1, 2))       # [heads][kv_rank, dim]
                    mw["w_uv"] = mat(w(i, pfx + "uv", (m.heads * m.vdim, m.kv_rank)))                 # [heads][vdim, kv_rank]
                    mw["w_o"] = mat(w(i, pfx + "o", (D, m.heads * m.vdim)))
                return mw

            m = lc.mixer
            if isinstance(m, ParallelMixerConfig):
                for side, sub in (("left", m.left), ("right", m.right)):
                    if isinstance(sub, ParallelMixerConfig) or getattr(sub, "kv_from", None) is not None:
                        raise ValueError(f"layer {i}: a branch of a parallel mixer is a plain mixer with a cache of its own")
                    lw[side] = mixer_weights(sub, f"mix.{side}.")
                    lw[side + "_out"] = (0.5 * w(i, f"mix.{side}.out", (D,)).float()).contiguous().to(dev)      # the halving rides on the gain
            else:
                lw.update(mixer_weights(m, "mix."))
            if cfg.residual_gate:
                lw["w_rg1"], lw["rg1_bias"] = mat(w(i, "rg1", (D, D))), vec(w(i, "rg1.b", (D,)))
                # the mixer's first projections and its gate read the same operand: one weight [projections | gate] and one product;
                # the tensors above become row ranges of it
                owners = ([(lw["left"], FIRST_PRODUCT[type(m.left)]), (lw["right"], FIRST_PRODUCT[type(m.right)])]
                          if isinstance(m, ParallelMixerConfig) else [(lw, FIRST_PRODUCT[type(m)])])
                fused = torch.cat([o[k] for o, k in owners] + [lw["w_rg1"]], 0).contiguous()
                at, split = 0, []
                for o, k in owners:
                    n = o[k].shape[0]
                    o[k] = fused[at:at + n]
                    split.append((at, n))
                    at += n
                lw["w_rg1"] = fused[at:]
                lw["w_in"], lw["in_split"] = fused, split
                lw["in_bias"] = torch.cat([torch.zeros(at, dtype=F32, device=dev), lw["rg1_bias"]]).contiguous()
                if lc.ff is not None:
                    lw["w_rg2"], lw["rg2_bias"] = mat(w(i, "rg2", (D, D))), vec(w(i, "rg2.b", (D,)))
            if cfg.depth_average:
                lw["dwa"] = vec(w(i, "dwa", (i + 2,)))
            f = lc.ff
            if f is not None:
                lw.update({"norm2": dyt_norm(i, "norm2")} if dyt else {"norm2": one_plus(i, "norm2")} if pre else
                          {k: (one_plus(i, k) if vector else num(i, k)) for k in ("norm2", "norm2b")})
            if isinstance(f, DenseFFConfig) and f.act == "clamp_glu":
                lw["w_gu"] = mat(torch.cat([w(i, "mlp.gate", (f.ff, D)), w(i, "mlp.up", (f.ff, D))], 0))
                lw["w_down"] = mat(w(i, "mlp.down", (D, f.ff)))
            elif isinstance(f, DenseFFConfig):
                lw["w_up"] = mat(w(i, "mlp.up", (f.ff, D)))
                lw["w_down"] = mat(w(i, "mlp.down", (D, f.ff)))
                if f.act == "xielu":
                    act = w(i, "mlp.act", (2,)).float()
                    lw["act_a"], lw["act_b"] = softplus(float(act[0])), 0.5 + softplus(float(act[1]))
                elif f.act != "relu2":
                    raise ValueError(f"layer {i}: unknown activation {f.act!r}")
            elif isinstance(f, MoEConfig):
                lw["w_router"] = mat(w(i, "mlp.router", (f.experts, D)))
                if f.act not in ("silu_glu", "clamp_glu"):
                    raise ValueError(f"layer {i}: unknown expert unit {f.act!r}")
                if f.router == "softmax_top":
                    if f.shared_ff or f.n_groups != 1:
                        raise ValueError(f"layer {i}: the softmax router has neither groups nor a shared expert")
                    lw["router_bias"] = vec(w(i, "mlp.router.b", (f.experts,)))
                elif f.router == "sigmoid_input":
                    if f.n_groups != 1:
                        raise ValueError(f"layer {i}: the plain sigmoid router has no groups")
                elif f.router != "grouped_sigmoid":
                    raise ValueError(f"layer {i}: unknown router {f.router!r}")
                else:
                    try:
                        corr = w(i, "mlp.correction", (f.experts,)).float()
                    except KeyError:                     # a router without a choice bias
                        corr = torch.zeros(f.experts)
                    lw["correction"] = corr.contiguous().to(dev)
                gu = [torch.cat([w(i, f"mlp.e{e}.gate", (f.expert_ff, D)), w(i, f"mlp.e{e}.up", (f.expert_ff, D))], 0)
                      for e in range(f.experts)]
                lw["w_gu"] = mat(torch.stack(gu, 0))                                           # [experts][2 ff, D]
                lw["w_edown"] = mat(torch.stack([w(i, f"mlp.e{e}.down", (D, f.expert_ff)) for e in range(f.experts)], 0))
                if f.shared_ff:
                    lw["ws_gu"] = mat(torch.cat([w(i, "mlp.shared.gate", (f.shared_ff, D)), w(i, "mlp.shared.up", (f.shared_ff, D))], 0))
                    lw["ws_down"] = mat(w(i, "mlp.shared.down", (D, f.shared_ff)))
                    if f.shared_gate:
                        lw["w_sg"] = mat(w(i, "mlp.shared.sg").reshape(D))
            self.layers.append(lw)
        for i, lc in enumerate(cfg.layers):
            if lc.weights_of is not None:
                self.layers[i] = self.layers[lc.weights_of]


# ---------------------------------------------------------------------------------------------------------------- batches
@dataclass
class StepEntry:
    key: Hashable                  # the request
    tokens: Sequence[int]          # its next tokens
    want: Sequence[int] = ()       # indices into `tokens` whose logits are returned


class _Batch:
    """Index tables of one step, built on the host and copied to the device in one transfer."""

    def __init__(self, eng: "SeqLMEngine", entries: Sequence[StepEntry], static: Optional[Dict] = None):
        """static: {(n, table width): device int32 buffer} — a decode batch whose layout has been seen before is copied into the same
        device buffer again, so that a captured graph of the step finds its tables where they were."""
        cache = eng.cache
        seqs = []
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.key!r} brings no tokens")
            s = cache.get(e.key) or cache.open(e.key)
            cache.reserve(s, len(e.tokens))
            seqs.append(s)
        self.seqs = seqs
        n = len(entries)
        lens = [len(e.tokens) for e in entries]
        R = sum(lens)
        self.R, self.n, self.lens = R, n, lens
        self.decode = all(ln == 1 for ln in lens)
        row0 = np.zeros(n + 1, np.int32)
        row0[1:] = np.cumsum(lens)
        pos0 = np.array([s.length for s in seqs], np.int32)
        slot = np.array([s.slot for s in seqs], np.int32)
        tokens = np.concatenate([np.asarray(e.tokens, np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= eng.cfg.vocab:
            raise ValueError("token id outside the vocabulary")
        row_seq = np.repeat(np.arange(n, dtype=np.int32), lens)
        row_pos = np.concatenate([np.arange(p, p + ln, dtype=np.int32) for p, ln in zip(pos0, lens)])
        def page_table(lists):
            width = max([len(p) for p in lists] + [1])
            if self.decode:
                width = -(-width // PAGE_TABLE_STEP) * PAGE_TABLE_STEP      # the width is a launch argument: change it rarely
            t = np.full((n, width), -1, np.int32)
            for i, p in enumerate(lists):
                t[i, : len(p)] = p
            return t, width
        table, max_pages = page_table([s.pages for s in seqs])
        # summary streams (one per block size): their page tables, and the most blocks one request completes in this step
        sum_tables, self.summary_width, self.summary_new = [], [], []
        for k, every in enumerate(cache.summary_every):
            t, width = page_table([s.summary_pages[k] for s in seqs])
            sum_tables.append(t.reshape(-1))
            self.summary_width.append(width)
            self.summary_new.append(max((s.length + ln) // every - s.length // every for s, ln in zip(seqs, lens)))
        ch = _lib.RETENTION_CHUNK
        c_seq, c_row0, c_len, seq_c0 = [], [], [], [0]
        for i, ln in enumerate(lens):
            for a in range(0, ln, ch):
                c_seq.append(i)
                c_row0.append(int(row0[i]) + a)
                c_len.append(min(ch, ln - a))
            seq_c0.append(len(c_seq))
        self.n_chunks = len(c_seq)
        self.max_pages = max_pages
        want = [int(row0[i]) + int(k) for i, e in enumerate(entries) for k in e.want]
        for i, e in enumerate(entries):
            if any(k < 0 or k >= lens[i] for k in e.want):
                raise ValueError(f"request {e.key!r}: a wanted index is outside its tokens")
        self.n_want = len(want)
        parts = [tokens.astype(np.int32), row_seq, row_pos, row0, pos0, slot, table.reshape(-1), np.asarray(c_seq, np.int32),
                 np.asarray(c_row0, np.int32), np.asarray(c_len, np.int32), np.asarray(seq_c0, np.int32)] + sum_tables
        tables = torch.from_numpy(np.concatenate(parts).astype(np.int32))
        want_t = torch.from_numpy(np.asarray(want, np.int32))
        self.layout = (n, max_pages, *self.summary_width) if self.decode else None      # fixes the size of every table of a decode batch
        if eng.device.type == "cuda":
            host = tables.pin_memory()
            if static is not None and self.decode:
                tables = static.get(self.layout)
                if tables is None:
                    tables = static[self.layout] = torch.empty(len(host), dtype=I32, device=eng.device)
                tables.copy_(host, non_blocking=True)
            else:
                tables = host.to(eng.device, non_blocking=True)
            if len(want):
                want_t = want_t.pin_memory().to(eng.device, non_blocking=True)
        views, o = [], 0
        for p in parts:
            views.append(tables[o:o + len(p)])
            o += len(p)
        (self.tokens, self.row_seq, self.row_pos, self.seq_row0, self.seq_pos0, self.seq_slot, self.page_table, self.chunk_seq,
         self.chunk_row0, self.chunk_len, self.seq_chunk0) = views[:11]
        self.summary_table = views[11:]
        self.want_rows = want_t
        self._tables = tables


# ---------------------------------------------------------------------------------------------------------------- engine
class SeqLMEngine:
    def __init__(self, cfg: SeqLMConfig, weights: SeqLMWeights, dtype: str = "bfloat16", max_tokens: int = 4096, page_size: int = 64,
                 max_seqs: int = 8, lib=None):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.cfg, self.w, self.device = cfg, weights, weights.device
        if lib is None:
            if self.device.type != "cuda" or not torch.cuda.is_available():
                raise _lib.NativeError("leopard_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
            lib = _lib.stream32_lib()
        self.L = lib
        self.dtype = dtype
        self.act = BF16 if dtype == "bfloat16" else F32
        # what every mixer keeps per request: rows of a paged cache (attention), rows of a summary pool (pooled blocks), a state.
        # The tables are keyed by the layer, or by (layer, "left" | "right") for the branches of a parallel mixer.
        rows, states, summaries, looks, keep = [], [], [], [], 0
        self._cache_index, self._state_index, self._summary_index, self._shift_index = {}, {}, {}, []

        def look_back(m):      # how far back a windowed or block-local layer reads (None: everything)
            bounds = [v for v in (m.window, m.chunk) if v and v > 0]
            return min(bounds) if bounds else None

        def claim(key, m):
            nonlocal keep
            ci = si = pi = -1
            if isinstance(m, LatentAttentionConfig):
                ci = len(rows)
                rows.append(m.kv_rank + m.rot_dim)
                looks.append(m.window if m.window and m.window > 0 else None)
            elif isinstance(m, WindowAttentionConfig) and m.kv_from is not None:
                j = m.kv_from
                src = cfg.layers[j].mixer if 0 <= j < len(cfg.layers) and not isinstance(key, tuple) and j < key else None
                if not isinstance(src, WindowAttentionConfig) or src.kv_from is not None:
                    raise ValueError(f"layer {key}: kv_from = {j} must name an earlier attention layer that has keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim, src.rot) != (m.kv_heads, m.dim, m.vdim, m.rot) or m.pool or src.value_rot or m.value_rot:
                    raise ValueError(f"layer {key}: its key / value sizes and rotation differ from those of layer {j}, whose cache it reads")
                ci = self._cache_index[j]
                looks.append(look_back(m))      # the owner's rows must stay for as long as this layer looks back
                keep = max(keep, m.keep_first if look_back(m) else 0)
            elif isinstance(m, WindowAttentionConfig):
                ci = len(rows)
                rows.append(m.kv_heads * (m.dim + m.vdim))
                windowed = bool(m.window and m.window > 0)
                if windowed and m.pool > 0:
                    pi = len(summaries)
                    summaries.append((m.kv_heads * (m.dim + m.vdim), m.pool))
                # a pooled layer reads a block's tokens once more when the block is complete
                looks.append(max(m.window, m.pool) if windowed and m.pool > 0 else look_back(m))
                keep = max(keep, m.keep_first if windowed else 0)
            elif isinstance(m, RetentionConfig):
                si = len(states)
                states.append((m.heads, m.dim, m.vdim))
            elif isinstance(m, MinGRUConfig):
                si = len(states)
                states.append((m.width,))
            elif isinstance(m, MLSTMConfig):
                si = len(states)
                states.append((m.heads, m.dim + 1, m.vdim + 1))      # per head S | n, and the running maximum in the last row
            else:
                raise TypeError(f"unknown mixer {type(m).__name__}")
            self._cache_index[key], self._state_index[key], self._summary_index[key] = ci, si, pi

        for li, lc in enumerate(cfg.layers):
            self._shift_index.append(len(states) if lc.token_shift else -1)
            if lc.token_shift:
                states.append((cfg.width,))
            if isinstance(lc.mixer, ParallelMixerConfig):
                claim((li, "left"), lc.mixer.left)
                claim((li, "right"), lc.mixer.right)
            else:
                claim(li, lc.mixer)
        window = None if any(x is None for x in looks) else max(looks, default=None)
        self.cache = SequenceCache(rows, states, window, self.device, max_tokens=max_tokens, page_size=page_size, max_seqs=max_seqs,
                                   keep_first=keep, summaries=summaries)
        self.tile_rows = int(self.L.lp_linear_tile_rows())
        # large bf16 products of the serving precision go to the tcgen05 GEMM when the library has it (the native ones do)
        self.tensor_core_rows = TENSOR_CORE_MIN_ROWS if dtype == "bfloat16" and hasattr(self.L, "lp_gemm_bf16") else None
        self.tap: Optional[Callable[[int, torch.Tensor], None]] = None   # called with (layer, residual stream) after every layer
        # decode steps are launch-bound: a batch layout (requests, page-table width) that comes back is captured into a CUDA graph on
        # its second appearance and replayed from then on; only the index tables change between replays (LEOPARD_DECODE_GRAPH=0: off)
        import os
        self.use_graphs = self.device.type == "cuda" and os.environ.get("LEOPARD_DECODE_GRAPH", "1") != "0"
        self._static_tables: Dict = {}
        self._graphs: Dict = {}
        self._seen: Dict = {}

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream) if self.device.type == "cuda" else None

    def _check(self, rc, what):
        _lib.check_on(self.L, rc, what)

    def _empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _on_tensor_cores(self, a, w, M, N, K) -> bool:
        """The tcgen05 GEMM takes a product when it is large enough to fill tiles and meets the 16-byte rules of its TMA loads."""
        return (self.tensor_core_rows is not None and M >= self.tensor_core_rows and a.dtype == BF16 and N >= 128 and K >= 64
                and N % 8 == 0 and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def linear(self, a: torch.Tensor, w: torch.Tensor, out_dtype, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0, out=None, into=None, bias=None,
               row_scale=None):
        """out[M, N'] = epi(row_scale[m] * (a[M, K] @ w[N, K].T) + bias[N]) (bias, row_scale: fp32 device vectors or None).  With
        into = (x fp32 [M, N'], m) or (x, m, gate fp32 [M, N']): x <- x + m * epi(...) (* sigmoid(gate)) and x is returned."""
        M, K = a.shape
        N = w.shape[0]
        n_out = N // 2 if epi in _lib.GATED_EPIS else N
        # a row scale reaches the tensor-core path only through the activation kernel that follows the product
        tc = self._on_tensor_cores(a, w, M, N, K) and (row_scale is None or (epi != _lib.EPI_NONE and bias is None))
        if into is not None:
            x, mult = into[0], into[1]
            gate = into[2] if len(into) > 2 else None
            if tc:
                y = self.linear(a, w, F32, epi, epi_a, epi_b, bias=bias, row_scale=row_scale)
                if gate is None:
                    rc = self.L.lp_axpy_f32(_lib.ptr(x), x.stride(0), _lib.ptr(y), y.stride(0), float(mult), M, n_out, self._stream())
                else:
                    rc = self.L.lp_gated_axpy_f32(_lib.ptr(x), x.stride(0), _lib.ptr(y), y.stride(0), None, _lib.ptr(gate), gate.stride(0), None,
                                                  float(mult), M, n_out, self._stream())
                self._check(rc, "lp_axpy_f32")
                return x
            d = _lib.LinearDesc(A=_lib.ptr(a), lda=a.stride(0), a_batch=0, a_fp32=int(a.dtype == F32), W=_lib.ptr(w), ldw=w.stride(0),
                                w_batch=0, C=_lib.ptr(x), ldc=x.stride(0), c_batch=0, c_fp32=1, M=M, N=N, K=K, batch=1, epi=epi,
                                epi_a=epi_a, epi_b=epi_b, c_accum=1, c_scale=float(mult), bias=_lib.ptr(bias), row_scale=_lib.ptr(row_scale),
                                gate=_lib.ptr(gate), ldg=gate.stride(0) if gate is not None else 0)
            self._check(self.L.lp_linear(C.byref(d), self._stream()), "lp_linear")
            return x
        if out is None:
            out = self._empty((M, n_out), out_dtype)
        if tc and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
            raw = out if epi == _lib.EPI_NONE else self._empty((M, N), F32)
            rc = self.L.lp_gemm_bf16(_lib.ptr(a), a.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(raw), raw.stride(0), M, N, K, _lib.ptr(bias),
                                     None, 0, 0, _lib.ACT_NONE, int(raw.dtype == F32), 0, self._stream())
            self._check(rc, "lp_gemm_bf16")
            if epi != _lib.EPI_NONE:
                rc = self.L.lp_glu_scaled_f32(_lib.ptr(raw), raw.stride(0), 1, _lib.ptr(out), out.stride(0), int(out.dtype == F32), M, n_out,
                                              epi, epi_a, epi_b, _lib.ptr(row_scale), self._stream())
                self._check(rc, "lp_glu_f32")
            return out
        d = _lib.LinearDesc(A=_lib.ptr(a), lda=a.stride(0), a_batch=0, a_fp32=int(a.dtype == F32), W=_lib.ptr(w), ldw=w.stride(0),
                            w_batch=0, C=_lib.ptr(out), ldc=out.stride(0), c_batch=0, c_fp32=int(out.dtype == F32), M=M, N=N, K=K,
                            batch=1, epi=epi, epi_a=epi_a, epi_b=epi_b, bias=_lib.ptr(bias), row_scale=_lib.ptr(row_scale))
        self._check(self.L.lp_linear(C.byref(d), self._stream()), "lp_linear")
        return out

    def linear_heads(self, a: torch.Tensor, a_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int):
        """Per head h: out[:, h*out_head : +N] = a[:, h*a_head : +K] @ w[h].T with w [heads, N, K]."""
        heads, N, K = w.shape
        d = _lib.LinearDesc(A=_lib.ptr(a), lda=a.stride(0), a_batch=a_head, a_fp32=int(a.dtype == F32), W=_lib.ptr(w), ldw=w.stride(1),
                            w_batch=w.stride(0), C=_lib.ptr(out), ldc=out.stride(0), c_batch=out_head, c_fp32=int(out.dtype == F32),
                            M=a.shape[0], N=N, K=K, batch=heads, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
        self._check(self.L.lp_linear(C.byref(d), self._stream()), "lp_linear")
        return out

    def norm(self, x: torch.Tensor, gain, out_dtype=None, accum: Optional[torch.Tensor] = None):
        """RMS norm with one gain for all coordinates (a float) or one per coordinate (an fp32 device vector); `accum`: add the
        result to it instead of returning it."""
        M, D = x.shape
        out = None if accum is not None else self._empty((M, D), out_dtype)
        scalar, vector = (1.0, gain) if isinstance(gain, torch.Tensor) else (gain, None)
        rc = self.L.lp_rmsnorm_f32(_lib.ptr(x), x.stride(0), M, D, scalar, _lib.ptr(vector), self.cfg.eps, _lib.ptr(out),
                                   out.stride(0) if out is not None else 0, int(out is not None and out.dtype == F32), _lib.ptr(accum),
                                   accum.stride(0) if accum is not None else 0, self._stream())
        self._check(rc, "lp_rmsnorm_f32")
        return out

    def dyt(self, x: torch.Tensor, first, second=None):
        """Dynamic Tanh of the same rows with one or two parameter sets (alpha, gain, shift): the operands of a layer's sublayers"""
        M, D = x.shape
        out = self._empty((M, D), self.act)
        out2 = self._empty((M, D), self.act) if second is not None else None
        a2, g2, b2 = second if second is not None else (0.0, None, None)
        rc = self.L.lp_dyt_f32(_lib.ptr(x), x.stride(0), M, D, first[0], _lib.ptr(first[1]), _lib.ptr(first[2]), _lib.ptr(out), out.stride(0),
                               a2, _lib.ptr(g2), _lib.ptr(b2), _lib.ptr(out2), out2.stride(0) if out2 is not None else 0,
                               int(self.act == F32), self._stream())
        self._check(rc, "lp_dyt_f32")
        return out, out2

    # ------------------------------------------------------------------ mixers
    def _retention(self, li, m: RetentionConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        qkvg = proj if proj is not None else self.linear(h, lw["w_qkvg"], F32)
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        lightning = m.form == "lightning"      # the raw read-out in fp32; its norm spans the heads and follows below
        out = self._empty((b.R, hv), F32 if lightning else self.act)
        state = self.cache.states[self._state_index[li]]
        d = _lib.RetentionDesc(qkvg=_lib.ptr(qkvg), ld=qkvg.stride(0), q_off=0, k_off=hd, v_off=2 * hd, g_off=2 * hd + hv, heads=m.heads,
                               dim=m.dim, vdim=m.vdim, decay=_lib.ptr(lw["decay"]), inv_freq=_lib.ptr(lw["inv_freq"]), rot_dims=m.rot.dims,
                               rot_layout=_lib.ROT_INTERLEAVED if m.rot.layout == "interleaved" else _lib.ROT_HALF,
                               rot_mscale=lw["rot_mag"], k_scale=m.k_scale, eps=self.cfg.eps, state=_lib.ptr(state),
                               slot_stride=state.stride(0), out=_lib.ptr(out), ldo=out.stride(0), out_fp32=int(out.dtype == F32),
                               in_act=int(lightning), finish=_lib.RET_FINISH_RAW if lightning else _lib.RET_FINISH_GATED_NORM)
        if b.decode:
            rc = self.L.lp_retention_decode(C.byref(d), b.n, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot), self._stream())
            self._check(rc, "lp_retention_decode")
        else:
            nbytes = int(self.L.lp_retention_workspace_bytes(b.n_chunks, m.heads, m.dim, m.vdim))
            ws = self._empty((nbytes // 4,), F32)
            rc = self.L.lp_retention_prefill(C.byref(d), b.n, b.n_chunks, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot),
                                             _lib.ptr(b.seq_chunk0), _lib.ptr(b.chunk_seq), _lib.ptr(b.chunk_row0), _lib.ptr(b.chunk_len),
                                             _lib.ptr(ws), nbytes, self._stream())
            self._check(rc, "lp_retention_prefill")
        if lightning:
            gate = qkvg[:, 2 * hd + hv:]
            normed = self._empty((b.R, hv), self.act)
            rc = self.L.lp_rmsnorm_gated_f32(_lib.ptr(out), out.stride(0), b.R, hv, _lib.ptr(lw["out_gain"]), self.cfg.eps, _lib.ptr(gate),
                                             qkvg.stride(0), _lib.ptr(normed), normed.stride(0), int(normed.dtype == F32), self._stream())
            self._check(rc, "lp_rmsnorm_gated_f32")
            out = normed
        return self.linear(out, lw["w_o"], F32, into=into)

    def _latent(self, li, m: LatentAttentionConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        per = m.dim + m.rot_dim
        qd = proj if proj is not None else self.linear(h, lw["w_qdkv"], F32)
        nq = m.q_rank or m.heads * per
        dkv = qd[:, nq: nq + m.kv_rank + m.rot_dim]
        gate = qd[:, nq + m.kv_rank + m.rot_dim:] if m.head_gate else None
        if m.q_rank:      # queries through their own normed latent
            q = self.linear(self.norm(qd[:, :nq], lw["cq_gain"], self.act), lw["w_uq"], F32)
        else:
            q = qd[:, :nq]
        pool = self.cache.pools[self._cache_index[li]]
        d = _lib.LatentDesc(q=_lib.ptr(q), ldq=q.stride(0), dkv=_lib.ptr(dkv), lddkv=qd.stride(0), heads=m.heads, dim=m.dim,
                            rot_dim=m.rot_dim, kv_rank=m.kv_rank, c_gain=_lib.ptr(lw["c_gain"]), eps=self.cfg.eps,
                            inv_freq=_lib.ptr(lw["inv_freq"]), rot_dims=m.rot.dims,
                            rot_layout=_lib.ROT_INTERLEAVED if m.rot.layout == "interleaved" else _lib.ROT_HALF,
                            rot_mscale=lw["rot_mag"], cache=_lib.ptr(pool), page_size=self.cache.page_size,
                            page_table=_lib.ptr(b.page_table), max_pages=b.max_pages, window=m.window or 0, scale=m.scale,
                            sink=_lib.ptr(lw.get("sink")), gate=_lib.ptr(gate), ldg=qd.stride(0) if gate is not None else 0)
        self._check(self.L.lp_latent_prep(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), self._stream()), "lp_latent_prep")
        q_abs = self._empty((b.R, m.heads * m.kv_rank), F32)
        self.linear_heads(q, per, lw["w_ukT"], q_abs, m.kv_rank)
        lat = self._empty((b.R, m.heads * m.kv_rank), self.act)
        rc = self.L.lp_latent_attend(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), _lib.ptr(q_abs), q_abs.stride(0),
                                     _lib.ptr(lat), lat.stride(0), int(lat.dtype == F32), self._stream())
        self._check(rc, "lp_latent_attend")
        o = self._empty((b.R, m.heads * m.vdim), self.act)
        self.linear_heads(lat, m.kv_rank, lw["w_uv"].view(m.heads, m.vdim, m.kv_rank), o, m.vdim)
        return self.linear(o, lw["w_o"], F32, into=into)

    def _window_attention(self, li, m: WindowAttentionConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        qkv = proj if proj is not None else self.linear(h, lw["w_qkv"], F32)      # a layer that reads another layer's keys and values projects its queries only
        hq, hk = m.heads * m.dim, m.kv_heads * m.dim if m.kv_from is None else 0
        cache = self.cache
        pool = cache.pools[self._cache_index[li]]
        windowed = bool(m.window and m.window > 0)
        pi = self._summary_index[li]
        stream = cache.summary_index[pi][0] if pi >= 0 else -1
        layouts = {"half": _lib.ROT_HALF, "interleaved": _lib.ROT_INTERLEAVED}
        vr = m.value_rot
        mixing = m.talking_heads or m.out_gate
        d = _lib.WindowAttnDesc(
            qkv=_lib.ptr(qkv), ld=qkv.stride(0), q_off=0, k_off=hq, v_off=hq + hk, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
            vdim=m.vdim,
            norm_mode={"none": _lib.QKNORM_NONE, "head": _lib.QKNORM_HEAD, "unit": _lib.QKNORM_HEAD, "full": _lib.QKNORM_FULL}[m.qk_norm],
            q_bias=_lib.ptr(lw.get("q_bias")), k_bias=_lib.ptr(lw.get("k_bias")), v_bias=_lib.ptr(lw.get("v_bias")),
            v_norm=int(m.value_norm), talk=_lib.ptr(lw.get("talk")),
            g_off=hq + hk + (m.kv_heads * m.vdim if m.kv_from is None else 0) if m.out_gate else -1,
            q_gain=_lib.ptr(lw.get("q_gain")), k_gain=_lib.ptr(lw.get("k_gain")), eps=self.cfg.eps, inv_freq=_lib.ptr(lw["inv_freq"]),
            rot_dims=m.rot.dims, rot_layout=layouts[m.rot.layout], rot_mscale=lw["rot_mag"],
            v_inv_freq=_lib.ptr(lw.get("v_inv_freq")), v_rot_dims=vr.dims if vr else 0, v_rot_layout=layouts[vr.layout] if vr else 0,
            cache=_lib.ptr(pool), page_size=cache.page_size, page_table=_lib.ptr(b.page_table), max_pages=b.max_pages,
            pooled=_lib.ptr(cache.summary_pool(pi)) if pi >= 0 else None,
            pooled_table=_lib.ptr(b.summary_table[stream]) if pi >= 0 else None,
            max_pooled_pages=b.summary_width[stream] if pi >= 0 else 0, pool=m.pool if pi >= 0 else 0,
            window=m.window if windowed else 0, keep_first=m.keep_first if windowed else 0, scale=m.scale, softcap=m.softcap,
            sink=int(m.sink), chunk=m.chunk or 0, kv_shared=int(m.kv_from is not None))
        st = self._stream()
        self._check(self.L.lp_window_attn_prep(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), st), "lp_window_attn_prep")
        if pi >= 0:
            # a one-token step completes at most one block per request; the launch shape of a decode step must not depend on positions
            new = 1 if b.decode else b.summary_new[stream]
            rc = self.L.lp_window_attn_pool(C.byref(d), b.n, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), new, st)
            self._check(rc, "lp_window_attn_pool")
        o = self._empty((b.R, m.heads * m.vdim), self.act)
        if mixing and b.decode:      # weights mixed over the heads (and the output gate): a CTA per row
            rc = self.L.lp_window_attn_talk(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), _lib.ptr(o), o.stride(0),
                                            int(o.dtype == F32), st)
        elif mixing:      # the same kernel over tiles of consecutive rows, which share the keys they read
            rc = self.L.lp_window_attn_talk_tiles(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), b.n_chunks,
                                                  _lib.ptr(b.chunk_seq), _lib.ptr(b.chunk_row0), _lib.ptr(b.chunk_len), _lib.ptr(o),
                                                  o.stride(0), int(o.dtype == F32), st)
        elif b.decode:
            rc = self.L.lp_window_attn(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), _lib.ptr(o), o.stride(0),
                                       int(o.dtype == F32), st)
        else:      # prompts and portions: tiles of consecutive rows share the keys they read
            rc = self.L.lp_window_attn_tiles(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), b.n_chunks, _lib.ptr(b.chunk_seq),
                                             _lib.ptr(b.chunk_row0), _lib.ptr(b.chunk_len), _lib.ptr(o), o.stride(0), int(o.dtype == F32), st)
        self._check(rc, "lp_window_attn")
        return self.linear(o, lw["w_o"], F32, into=into, bias=lw.get("o_bias"))

    def _mingru(self, li, m: MinGRUConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        zxg = proj if proj is not None else self.linear(h, lw["w_zxg"], F32)
        out = self._empty((b.R, m.width), self.act)
        state = self.cache.states[self._state_index[li]]
        d = _lib.MinGRUDesc(zxg=_lib.ptr(zxg), ld=zxg.stride(0), z_off=0, x_off=m.width, g_off=2 * m.width, width=m.width,
                            z_bias=_lib.ptr(lw["z_bias"]), x_bias=_lib.ptr(lw["x_bias"]), state=_lib.ptr(state), slot_stride=state.stride(0),
                            out=_lib.ptr(out), ldo=out.stride(0), out_fp32=int(out.dtype == F32))
        if b.decode:
            rc = self.L.lp_mingru_decode(C.byref(d), b.n, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot), self._stream())
            self._check(rc, "lp_mingru_decode")
        else:
            nbytes = int(self.L.lp_mingru_workspace_bytes(b.n_chunks, m.width))
            ws = self._empty((nbytes // 4,), F32)
            rc = self.L.lp_mingru_prefill(C.byref(d), b.n, b.n_chunks, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot),
                                          _lib.ptr(b.seq_chunk0), _lib.ptr(b.chunk_seq), _lib.ptr(b.chunk_row0), _lib.ptr(b.chunk_len),
                                          _lib.ptr(ws), nbytes, self._stream())
            self._check(rc, "lp_mingru_prefill")
        return self.linear(out, lw["w_o"], F32, into=into)

    def _mlstm(self, li, m: MLSTMConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        proj = proj if proj is not None else self.linear(h, lw["w_proj"], F32)
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        out = self._empty((b.R, hv), self.act)
        state = self.cache.states[self._state_index[li]]
        d = _lib.MLSTMDesc(proj=_lib.ptr(proj), ld=proj.stride(0), q_off=0, k_off=hd, v_off=2 * hd, g_off=2 * hd + hv,
                           i_off=2 * hd + 2 * hv, f_off=2 * hd + 2 * hv + m.heads, heads=m.heads, dim=m.dim, vdim=m.vdim,
                           i_bias=_lib.ptr(lw["i_bias"]), f_bias=_lib.ptr(lw["f_bias"]), gate_cap=m.gate_cap, q_scale=m.dim ** -0.5,
                           eps=self.cfg.eps, out_gain=_lib.ptr(lw["out_gain"]), state=_lib.ptr(state), slot_stride=state.stride(0),
                           out=_lib.ptr(out), ldo=out.stride(0), out_fp32=int(out.dtype == F32))
        nbytes = int(self.L.lp_mlstm_workspace_bytes(b.R, m.heads, m.vdim))
        ws = self._empty((nbytes // 4,), F32)
        rc = self.L.lp_mlstm(C.byref(d), b.n, b.R, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot), _lib.ptr(ws), nbytes,
                             self._stream())
        self._check(rc, "lp_mlstm")
        return self.linear(out, lw["w_o"], F32, into=into)

    def _parallel(self, li: int, m: ParallelMixerConfig, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        """two mixers on the same input; each output is RMS-normed over the width with its own gain (which carries the halving);
        proj: the two branches' first products when one product of the layer made them"""
        left = self._mix((li, "left"), m.left, lw["left"], h, b, proj=proj[0] if proj is not None else None)
        right = self._mix((li, "right"), m.right, lw["right"], h, b, proj=proj[1] if proj is not None else None)
        mix = self.norm(left, lw["left_out"], F32)
        self.norm(right, lw["right_out"], accum=mix)
        if into is None:
            return mix
        x, mult = into[0], into[1]
        gate = into[2] if len(into) > 2 else None
        rc = self.L.lp_gated_axpy_f32(_lib.ptr(x), x.stride(0), _lib.ptr(mix), mix.stride(0), None, _lib.ptr(gate),
                                      gate.stride(0) if gate is not None else 0, None, float(mult), b.R, self.cfg.width, self._stream())
        self._check(rc, "lp_gated_axpy_f32")
        return x

    def _mix(self, li, m, lw, h: torch.Tensor, b: _Batch, into=None, proj=None) -> torch.Tensor:
        """li: the key of the mixer's cache and state — the layer, or (layer, side) for a branch of a parallel mixer; proj: the
        mixer's first product of h (fp32, possibly columns of a wider product) when the caller has made it already"""
        if isinstance(m, ParallelMixerConfig):
            return self._parallel(li, m, lw, h, b, into, proj)
        if isinstance(m, MLSTMConfig):
            return self._mlstm(li, m, lw, h, b, into, proj)
        if isinstance(m, RetentionConfig):
            return self._retention(li, m, lw, h, b, into, proj)
        if isinstance(m, LatentAttentionConfig):
            return self._latent(li, m, lw, h, b, into, proj)
        if isinstance(m, WindowAttentionConfig):
            return self._window_attention(li, m, lw, h, b, into, proj)
        return self._mingru(li, m, lw, h, b, into, proj)

    # ------------------------------------------------------------------ feed-forwards
    def _dense(self, f: DenseFFConfig, lw, h: torch.Tensor, into=None) -> torch.Tensor:
        if f.act == "clamp_glu":
            up = self.linear(h, lw["w_gu"], self.act, _lib.EPI_CLAMP_GLU, f.limit, GLU_SLOPE)
        elif f.act == "relu2":
            up = self.linear(h, lw["w_up"], self.act, _lib.EPI_RELU2)
        else:
            up = self.linear(h, lw["w_up"], self.act, _lib.EPI_XIELU, lw["act_a"], lw["act_b"])
        return self.linear(up, lw["w_down"], F32, into=into)

    def _moe(self, f: MoEConfig, lw, h: torch.Tensor) -> torch.Tensor:
        T, D = h.shape
        L, st = self.L, self._stream()
        idx = self._empty((T, f.top), I32)
        wts = self._empty((T, f.top), F32)
        gate = self._empty((T,), F32) if f.shared_ff and f.shared_gate and f.router == "grouped_sigmoid" else None
        on_input = f.router == "sigmoid_input"      # the weight scales the expert's input: a row scale of its first product
        epi, epi_a, epi_b = (_lib.EPI_CLAMP_GLU, f.limit, GLU_SLOPE) if f.act == "clamp_glu" else (_lib.EPI_SILU_GATE, 0.0, 0.0)
        if on_input:
            rc = L.lp_moe_route_sigmoid(_lib.ptr(h), h.stride(0), int(h.dtype == F32), T, D, _lib.ptr(lw["w_router"]),
                                        lw["w_router"].stride(0), f.experts, f.top, _lib.ptr(idx), _lib.ptr(wts), st)
        elif f.router == "softmax_top":
            rc = L.lp_moe_route_softmax(_lib.ptr(h), h.stride(0), int(h.dtype == F32), T, D, _lib.ptr(lw["w_router"]),
                                        lw["w_router"].stride(0), f.experts, _lib.ptr(lw["router_bias"]), f.top, _lib.ptr(idx),
                                        _lib.ptr(wts), st)
        else:
            rc = L.lp_moe_route(_lib.ptr(h), h.stride(0), int(h.dtype == F32), T, D, _lib.ptr(lw["w_router"]), lw["w_router"].stride(0),
                                f.experts, _lib.ptr(lw["correction"]), f.n_groups, f.keep_groups, f.top,
                                _lib.ptr(lw["w_sg"]) if gate is not None else None, _lib.ptr(idx), _lib.ptr(wts), _lib.ptr(gate), st)
        self._check(rc, "lp_moe_route")
        n_pairs = T * f.top
        if n_pairs <= MOE_PAIRS_MAX:
            # few (token, choice) pairs (decoding): no sorting — every pair streams its expert's weights once, pair z = row z
            w_gu, w_dn = lw["w_gu"], lw["w_edown"]
            h1 = self._empty((n_pairs, f.expert_ff), self.act)
            d1 = _lib.LinearDesc(A=_lib.ptr(h), lda=h.stride(0), a_batch=0, a_fp32=int(h.dtype == F32), W=_lib.ptr(w_gu), ldw=w_gu.stride(1),
                                 w_batch=w_gu.stride(0), C=_lib.ptr(h1), ldc=h1.stride(0), c_batch=0, c_fp32=int(h1.dtype == F32), M=1,
                                 N=2 * f.expert_ff, K=D, batch=1, epi=epi, epi_a=epi_a, epi_b=epi_b, row_scale=_lib.ptr(wts) if on_input else None)
            self._check(L.lp_linear_pairs(C.byref(d1), _lib.ptr(idx), f.top, n_pairs, st), "lp_linear_pairs")
            y = self._empty((n_pairs, D), F32)
            d2 = _lib.LinearDesc(A=_lib.ptr(h1), lda=h1.stride(0), a_batch=0, a_fp32=int(h1.dtype == F32), W=_lib.ptr(w_dn),
                                 ldw=w_dn.stride(1), w_batch=w_dn.stride(0), C=_lib.ptr(y), ldc=y.stride(0), c_batch=0, c_fp32=1, M=1, N=D,
                                 K=f.expert_ff, batch=1, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_pairs(C.byref(d2), _lib.ptr(idx), 1, n_pairs, st), "lp_linear_pairs")
            return self._moe_combine(f, lw, h, y, self._pair_identity(n_pairs), None if on_input else wts, gate)
        tiles = int(L.lp_moe_max_tiles(n_pairs, f.experts, self.tile_rows))
        tile_group = self._empty((tiles,), I32)
        sorted_token = self._empty((tiles * self.tile_rows,), I32)
        pair_row = self._empty((n_pairs,), I32)
        rc = L.lp_moe_align(_lib.ptr(idx), n_pairs, f.top, f.experts, self.tile_rows, tiles, _lib.ptr(tile_group), _lib.ptr(sorted_token),
                            _lib.ptr(pair_row), st)
        self._check(rc, "lp_moe_align")
        rows = tiles * self.tile_rows
        scale = None
        if on_input:      # the pairs' weights in the sorted row space
            scale = torch.zeros((rows,), dtype=F32, device=self.device)      # padding rows of the sorted space stay zero
            self._check(L.lp_moe_sorted_weights(_lib.ptr(pair_row), _lib.ptr(wts), n_pairs, _lib.ptr(scale), st), "lp_moe_sorted_weights")
        h1 = self._empty((rows, f.expert_ff), self.act)
        y = self._empty((rows, D), F32)
        w_gu, w_dn = lw["w_gu"], lw["w_edown"]
        capturing = self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()      # no host read inside a graph
        if self.tensor_core_rows is not None and n_pairs >= f.experts * self.tensor_core_rows and h.dtype == BF16 and not capturing:
            # prefill in the serving precision: enough rows per expert to fill tensor-core tiles.  The segment bounds come to the host
            # (one small device -> host copy), the rows are gathered into expert order and every expert runs two tcgen05 GEMMs.
            groups = tile_group.cpu().tolist()
            a_sorted = h.index_select(0, sorted_token.clamp_min(0).long())
            t0 = 0
            while t0 < tiles:
                e, t1 = groups[t0], t0 + 1
                while t1 < tiles and groups[t1] == e:
                    t1 += 1
                if e >= 0:
                    r0, r1 = t0 * self.tile_rows, t1 * self.tile_rows
                    self.linear(a_sorted[r0:r1], w_gu[e], self.act, epi, epi_a, epi_b, out=h1[r0:r1],
                                row_scale=scale[r0:r1] if on_input else None)
                    self.linear(h1[r0:r1], w_dn[e], F32, out=y[r0:r1])
                t0 = t1
        else:
            d1 = _lib.LinearDesc(A=_lib.ptr(h), lda=h.stride(0), a_batch=0, a_fp32=int(h.dtype == F32), W=_lib.ptr(w_gu), ldw=w_gu.stride(1),
                                 w_batch=w_gu.stride(0), C=_lib.ptr(h1), ldc=h1.stride(0), c_batch=0, c_fp32=int(h1.dtype == F32), M=rows,
                                 N=2 * f.expert_ff, K=D, batch=1, epi=epi, epi_a=epi_a, epi_b=epi_b, row_scale=_lib.ptr(scale))
            self._check(L.lp_linear_grouped(C.byref(d1), _lib.ptr(tile_group), tiles, _lib.ptr(sorted_token), st), "lp_linear_grouped")
            d2 = _lib.LinearDesc(A=_lib.ptr(h1), lda=h1.stride(0), a_batch=0, a_fp32=int(h1.dtype == F32), W=_lib.ptr(w_dn),
                                 ldw=w_dn.stride(1), w_batch=w_dn.stride(0), C=_lib.ptr(y), ldc=y.stride(0), c_batch=0, c_fp32=1, M=rows,
                                 N=D, K=f.expert_ff, batch=1, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_grouped(C.byref(d2), _lib.ptr(tile_group), tiles, None, st), "lp_linear_grouped")
        return self._moe_combine(f, lw, h, y, pair_row, None if on_input else wts, gate)

    def _pair_identity(self, n: int) -> torch.Tensor:
        t = getattr(self, "_arange", None)
        if t is None or t.numel() < n:
            t = self._arange = torch.arange(max(n, 256), dtype=I32, device=self.device)
        return t

    def _moe_combine(self, f: MoEConfig, lw, h, y, pair_row, wts, gate) -> torch.Tensor:
        T, D = h.shape
        shared = None
        if f.shared_ff:
            if f.act == "clamp_glu":
                s1 = self.linear(h, lw["ws_gu"], self.act, _lib.EPI_CLAMP_GLU, f.shared_limit, GLU_SLOPE)
            else:
                s1 = self.linear(h, lw["ws_gu"], self.act, _lib.EPI_SILU_GATE)
            shared = self.linear(s1, lw["ws_down"], F32)
        out = self._empty((T, D), F32)
        rc = self.L.lp_moe_combine(_lib.ptr(y), y.stride(0), _lib.ptr(pair_row), _lib.ptr(wts), f.top, _lib.ptr(shared),
                                   shared.stride(0) if shared is not None else 0, _lib.ptr(gate), _lib.ptr(out), out.stride(0), T, D,
                                   self._stream())
        self._check(rc, "lp_moe_combine")
        return out

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the tokens each entry brings, from the cache and state earlier steps left; returns fp32 logits [wanted rows, vocab]
        in the order of the entries and of their `want` lists (None when nothing is wanted)."""
        if not entries:
            return None
        if len({e.key for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        b = _Batch(self, entries, self._static_tables if self.use_graphs else None)
        if b.decode and self.use_graphs and self.tap is None:
            logits = self._decode_replay(b)
        else:
            logits = self._forward(b, b.want_rows if b.n_want else None)
        for s, ln in zip(b.seqs, b.lens):
            self.cache.advance(s, ln)
        return logits

    def _decode_replay(self, b: _Batch) -> Optional[torch.Tensor]:
        """One-token-per-request steps: eager the first time a layout is seen, captured the second time, replayed afterwards.  The
        graph computes the logits of every row; the wanted ones are picked afterwards."""
        key = (b.layout, self.cache.generation)
        g = self._graphs.get(key)
        if g is None:
            self._seen[key] = self._seen.get(key, 0) + 1
            if self._seen[key] < 2:
                return self._forward(b, b.want_rows if b.n_want else None)
            for old in [k for k in self._graphs if k[1] != self.cache.generation]:
                del self._graphs[old]                      # pools were reallocated: those graphs point at freed memory
            if len(self._graphs) >= MAX_DECODE_GRAPHS:      # a bound on what the captured layouts may hold
                self._graphs.clear()
                self._seen.clear()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                out = self._forward(b, "all")
            g = self._graphs[key] = (graph, out)
        g[0].replay()
        if b.n_want == 0:
            return None
        return g[1].index_select(0, b.want_rows.long()) if b.n_want != b.R else g[1].clone()

    def _forward(self, b: _Batch, want) -> Optional[torch.Tensor]:
        """embedding -> layers -> (final norm, head) over the rows `want` (a device index tensor, "all", or None)"""
        cfg, D = self.cfg, self.cfg.width
        hist = None
        if cfg.depth_average:      # every layer's result is kept: the embedding output is the first of them
            hist = self._empty((len(cfg.layers) + 1, b.R, D), F32)
        x = hist[0] if hist is not None else self._empty((b.R, D), F32)
        rc = self.L.lp_embed_rows_f32(_lib.ptr(b.tokens), b.R, _lib.ptr(self.w.embed), self.w.embed.stride(0), cfg.vocab, cfg.embed_scale,
                                      _lib.ptr(x), x.stride(0), D, self._stream())
        self._check(rc, "lp_embed_rows_f32")
        if cfg.position_base > 0:
            rc = self.L.lp_add_positions_f32(_lib.ptr(x), x.stride(0), b.R, D, _lib.ptr(b.row_pos), _lib.ptr(self.w.position_freq),
                                             self._stream())
            self._check(rc, "lp_add_positions_f32")
        if cfg.norm == "parallel_dyt":
            return self._forward_parallel(b, want, x, hist)
        pre = cfg.norm == "pre"
        for li, (lc, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            if self.w.add_before[li] is not None:
                rc = self.L.lp_add_row_f32(_lib.ptr(x), x.stride(0), _lib.ptr(self.w.add_before[li]), b.R, D, self._stream())
                self._check(rc, "lp_add_row_f32")
            if lc.token_shift:      # the normed stream in fp32, then shifted towards the previous token's into the operand dtype
                hn = self.norm(x, lw["norm1"], F32)
                h = self._empty((b.R, D), self.act)
                state = self.cache.states[self._shift_index[li]]
                rc = self.L.lp_token_shift_f32(_lib.ptr(hn), hn.stride(0), _lib.ptr(lw["shift"]), b.R, D, _lib.ptr(b.row_seq),
                                               _lib.ptr(b.row_pos), _lib.ptr(b.seq_row0), _lib.ptr(b.seq_slot), _lib.ptr(state),
                                               state.stride(0), _lib.ptr(h), h.stride(0), int(h.dtype == F32), self._stream())
                self._check(rc, "lp_token_shift_f32")
            else:
                h = self.norm(x, lw["norm1"], self.act)
            if pre:        # x <- x + m * mixer(norm(x)): the update is the store of the mixer's output product
                self._mix(li, lc.mixer, lw, h, b, into=(x, cfg.residual_mult))
            else:
                self.norm(self._mix(li, lc.mixer, lw, h, b), lw["norm1b"], accum=x)
            if lc.ff is not None:
                h = self.norm(x, lw["norm2"], self.act)
                if pre and isinstance(lc.ff, DenseFFConfig):
                    self._dense(lc.ff, lw, h, into=(x, cfg.residual_mult))
                elif pre:
                    y = self._moe(lc.ff, lw, h)
                    rc = self.L.lp_axpy_f32(_lib.ptr(x), x.stride(0), _lib.ptr(y), y.stride(0), cfg.residual_mult, b.R, D, self._stream())
                    self._check(rc, "lp_axpy_f32")
                else:
                    y = self._dense(lc.ff, lw, h) if isinstance(lc.ff, DenseFFConfig) else self._moe(lc.ff, lw, h)
                    self.norm(y, lw["norm2b"], accum=x)
            if self.tap is not None:
                self.tap(li, x)
        if want is None:
            return None
        return self._head(x, want)

    def _head(self, x: torch.Tensor, want) -> torch.Tensor:
        rows = x if isinstance(want, str) else x.index_select(0, want.long())
        hn = self.dyt(rows, self.w.final_gain)[0] if self.cfg.norm == "parallel_dyt" else self.norm(rows, self.w.final_gain, self.act)
        return self.linear(hn, self.w.head, F32)

    def _forward_parallel(self, b: _Batch, want, x0: torch.Tensor, hist: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Layers whose two sublayers read the SAME stream through two Dynamic-Tanh norms: X' = x + m (gate1 * mixer(norm1 x) + gate2 *
        ff(norm2 x)).  With the depth average the results X_0 (the embedding), X_1, ... are kept ([layers + 1, rows, width] fp32) and
        the next layer reads their weighted sum; the branches are added into the slot of X' in the stores of their last products.
        x0: the embedding output, which is hist[0] when there is a depth average."""
        cfg, D, R, st = self.cfg, self.cfg.width, b.R, self._stream()
        n_layers = len(cfg.layers)
        x = x0
        for li, (lc, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            if cfg.depth_average:      # the slot of this layer's result starts as its input
                acc = hist[li + 1]
                if li == 0:
                    acc.copy_(x)
            else:
                acc = x
            h1, h2 = self.dyt(x, lw["norm1"], lw["norm2"] if lc.ff is not None else None)
            g1 = proj = None
            if "w_in" in lw:      # ONE product of h1: every branch's first projection and the pre-activations of the mixer's gate
                wide = self.linear(h1, lw["w_in"], F32, bias=lw["in_bias"])
                parts = [wide[:, a:a + n] for a, n in lw["in_split"]]
                proj = tuple(parts) if isinstance(lc.mixer, ParallelMixerConfig) else parts[0]
                g1 = wide[:, wide.shape[1] - D:]
            elif cfg.residual_gate:
                g1 = self.linear(h1, lw["w_rg1"], F32, bias=lw["rg1_bias"])
            g2 = self.linear(h2, lw["w_rg2"], F32, bias=lw["rg2_bias"]) if cfg.residual_gate and lc.ff is not None else None
            # both operands exist before anything is added, so `acc` may be the stream itself
            self._mix(li, lc.mixer, lw, h1, b, into=(acc, cfg.residual_mult, g1) if g1 is not None else (acc, cfg.residual_mult), proj=proj)
            if isinstance(lc.ff, DenseFFConfig):
                self._dense(lc.ff, lw, h2, into=(acc, cfg.residual_mult, g2) if g2 is not None else (acc, cfg.residual_mult))
            elif lc.ff is not None:
                y = self._moe(lc.ff, lw, h2)
                rc = self.L.lp_gated_axpy_f32(_lib.ptr(acc), acc.stride(0), _lib.ptr(y), y.stride(0), None, _lib.ptr(g2),
                                              g2.stride(0) if g2 is not None else 0, None, cfg.residual_mult, R, D, st)
                self._check(rc, "lp_gated_axpy_f32")
            if cfg.depth_average:
                x = self._empty((R, D), F32)
                nxt = hist[li + 2] if li + 1 < n_layers else None
                rc = self.L.lp_depth_average_f32(_lib.ptr(hist), hist.stride(0), hist.stride(1), _lib.ptr(lw["dwa"]), li + 2, _lib.ptr(x),
                                                 x.stride(0), _lib.ptr(nxt), nxt.stride(0) if nxt is not None else 0, R, D, st)
                self._check(rc, "lp_depth_average_f32")
            else:
                x = acc
            if self.tap is not None:
                self.tap(li, x)
        if want is None:
            return None
        return self._head(x, want)

    def finish(self, key: Hashable) -> None:
        """The request is over: its pages and its slot go back to the pools."""
        self.cache.close(key)
