"""Shared pieces of the Gavatar tests: small configurations in the parsed-JSON form a checkpoint carries, and the engine builder for
the two backends of seqlm_common (kernel sources under the CPU emulator; the native library on a GPU)."""
import copy

from seqlm_common import BACKENDS, TOL, backend, emu_lib, rel_err  # noqa: F401  (fixtures)


def moe(experts=5, top=2, ff=6):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention_layer(heads=4, kv_heads=2, dim=8, vdim=4, window=5, scale=0.6, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": window}}, "mlp": mlp}


def latent_layer(heads=3, dim=4, vdim=6, q_rank=5, kv_rank=8, window=4, scale=0.7, mlp=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                                  "scale": scale, "mask": {"size": window}}, "mlp": mlp}


def mlstm_layer(heads=2, dim=6, vdim=5, gate_cap=8.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}, "mlp": mlp}


def model(layers, width=12, vocab=41, eps=1e-5, embed_scale=3.0, loop=None):
    d = {"architecture": "Gavatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
         "layers": copy.deepcopy(layers)}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


def mixed_model():
    """every mixer, a layer without feed-forward, and the first two layers run twice"""
    return model([latent_layer(mlp=moe()), mlstm_layer(), attention_layer(mlp=moe(experts=3, top=3, ff=4))], loop=(0, 2, 2))


def make_engine(cfg: dict, weights: dict, backend, dtype="float32", **kw):
    from leopard_b200 import gavatar
    device, lib = backend
    kw.setdefault("page_size", 4)
    kw.setdefault("max_tokens", 32)
    kw.setdefault("max_seqs", 2)
    return gavatar.from_state_dict(cfg, weights, dtype=dtype, device=device, lib=lib, **kw)
