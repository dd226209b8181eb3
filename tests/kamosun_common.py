"""Shared pieces of the Kamosun tests: small configurations in the parsed-JSON form a checkpoint carries, and the engine builder for
the two backends of seqlm_common (kernel sources under the CPU emulator; the native library on a GPU)."""
import copy

from seqlm_common import BACKENDS, TOL, backend, emu_lib, rel_err  # noqa: F401  (fixtures)


def dense(ff=10, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, top=2, ff=6, limit=1.2, shared=7, shared_limit=0.8):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared, "limit": shared_limit}
    return d


def attention_layer(heads=4, kv_heads=2, dim=8, vdim=4, chunk=5, scale=0.5, rot_dims=6, base=100.0, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if chunk:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def parallel_layer(heads=2, kv_heads=1, dim=6, vdim=5, scale=0.6, softcap=3.0, rot_dims=4, base=50.0, scaling=True, r_heads=2, r_dim=4,
                   r_vdim=3, decay=(0.8, 0.97), mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:      # wavelengths of base 50 over 4 dims: 6.3 and 44; the bands put one pair between the two rules
        rot["scaling"] = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "rot": rot}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def model(layers, width=12, vocab=41, eps=1e-5, mult=0.7):
    return {"architecture": "Kamosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": copy.deepcopy(layers)}


def mixed_model():
    """every mixer and feed-forward: attention + dense, a layer on the first one's keys and values + experts, the parallel mixer
    without feed-forward, attention with keys of its own again + experts without a shared one"""
    return model([attention_layer(mlp=dense()), attention_layer(kv_from=0, chunk=3, mlp=moe()), parallel_layer(),
                  attention_layer(heads=2, kv_heads=2, dim=4, vdim=6, chunk=7, rot_dims=2, mlp=moe(experts=3, top=1, ff=4, shared=0))])


def make_engine(cfg: dict, weights: dict, backend, dtype="float32", **kw):
    from leopard_b200 import kamosun
    device, lib = backend
    kw.setdefault("page_size", 4)
    kw.setdefault("max_tokens", 32)
    kw.setdefault("max_seqs", 2)
    return kamosun.from_state_dict(cfg, weights, dtype=dtype, device=device, lib=lib, **kw)
