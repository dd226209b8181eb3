"""bench.py --workload seqlm: prefill and decode throughput of the layer-list language models (leopard_b200/seqlm.py) at a few sizes that
resemble a real model's layers, beside the framework's Llama-style decoder (lp_decoder_prefill / the CUDA-graph decode loop) at the same
width, feed-forward size, depth and vocabulary.  Random weights, synthetic token ids, one GPU.

Per size: a 4-layer stack [retention + dense, retention + MoE, windowed latent attention + MoE, retention + dense];
  prefill   one request of `prompt` tokens per step through SeqLMEngine.step (cache and state written), tokens/s;
  decode    `batch` running requests advanced by one token per step, tokens/s, for batch 1, 8 and 64;
  kernels   device time per native entry point of one prefill step and one decode step (CUDA events around every call) with the
            rate each reaches: TFLOP/s of the measured cuBLAS bf16 peak for the tcgen05 GEMM, of the fp32 FMA peak for the 32-bit
            mixers, GB/s of the measured copy bandwidth for the weight-streaming decode kernels.
One JSON line in the shape bench.py prints for its other workloads; `value` is the prefill throughput of the middle size.
"""
from __future__ import annotations

import json
import time
from collections import defaultdict

import torch

SIZES = {
    "w1024": dict(width=1024, heads=8, ff=4096, kv_rank=256, window=512, experts=8, top=2, expert_ff=1024, shared_ff=1024, vocab=32000),
    "w2048": dict(width=2048, heads=16, ff=8192, kv_rank=512, window=1024, experts=16, top=4, expert_ff=1024, shared_ff=2048, vocab=32000),
    "w4096": dict(width=4096, heads=32, ff=14336, kv_rank=512, window=2048, experts=32, top=4, expert_ff=2048, shared_ff=4096, vocab=32000),
}
HEAD = 128          # per-head dims of both mixers (rotated part of latent attention: 64)
FP32_FMA_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12     # SMs x FMA lanes x 2 x max clock: the SIMT fp32 ceiling of the 32-bit mixers


def zudalorn_config(s):
    ret = {"heads": s["heads"], "dim": HEAD, "vdim": HEAD, "decay": [1 - 2.0 ** (-4 - 4 * i / max(s["heads"] - 1, 1)) for i in range(s["heads"])],
           "rot": {"base": 1e6, "dims": HEAD}}
    lat = {"heads": s["heads"], "dim": HEAD, "rot_dim": 64, "vdim": HEAD, "kv_rank": s["kv_rank"], "scale": (HEAD + 64) ** -0.5,
           "mask": {"size": s["window"]},
           "rot": {"base": 5e4, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "retention", "mixer": ret, "mlp": dense}, {"type": "retention", "mixer": ret, "mlp": moe},
              {"type": "latent_attention", "mixer": lat, "mlp": moe}, {"type": "retention", "mixer": ret, "mlp": dense}]
    return {"architecture": "Zudalorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "layers": layers}


def random_getter(cfg, dev, seed=1):
    g = torch.Generator(device=dev).manual_seed(seed)
    D = cfg["width"]
    shapes = {}

    def reg(name, *shape):
        shapes[name] = shape
    reg("embed", cfg["vocab"], D); reg("head", cfg["vocab"], D); reg("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            reg(p + n)
        if layer["type"] == "retention":
            reg(p + "mix.q", m["heads"] * m["dim"], D); reg(p + "mix.k", m["heads"] * m["dim"], D)
            reg(p + "mix.v", m["heads"] * m["vdim"], D); reg(p + "mix.g", m["heads"] * m["vdim"], D); reg(p + "mix.o", D, m["heads"] * m["vdim"])
        else:
            reg(p + "mix.q", m["heads"] * (m["dim"] + m["rot_dim"]), D); reg(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], D)
            reg(p + "mix.dkv.norm", m["kv_rank"]); reg(p + "mix.uk", m["heads"] * m["dim"], m["kv_rank"])
            reg(p + "mix.uv", m["heads"] * m["vdim"], m["kv_rank"]); reg(p + "mix.o", D, m["heads"] * m["vdim"])
        f = layer["mlp"]
        if f["kind"] == "dense":
            reg(p + "mlp.up", f["ff"], D); reg(p + "mlp.down", D, f["ff"]); reg(p + "mlp.act", 2)
        else:
            for e in range(f["router"]["experts"]):
                reg(f"{p}mlp.e{e}.gate", f["expert"]["ff"], D); reg(f"{p}mlp.e{e}.up", f["expert"]["ff"], D); reg(f"{p}mlp.e{e}.down", D, f["expert"]["ff"])
            reg(p + "mlp.router", f["router"]["experts"], D); reg(p + "mlp.correction", f["router"]["experts"])
            reg(p + "mlp.shared.gate", f["shared"]["ff"], D); reg(p + "mlp.shared.up", f["shared"]["ff"], D)
            reg(p + "mlp.shared.down", D, f["shared"]["ff"]); reg(p + "mlp.shared.sg", 1, D)

    def get(name):
        shape = shapes[name]
        if len(shape) == 2:
            return (torch.randn(shape, device=dev, generator=g) * shape[1] ** -0.5).to(torch.bfloat16)
        if len(shape) == 0:
            return torch.ones((), device=dev, dtype=torch.bfloat16)
        return (torch.rand(shape, device=dev, generator=g) * 0.5 + 0.5).to(torch.bfloat16)
    return get


class TimedLib:
    """Wraps the native library: CUDA events around every entry point, summed per name."""

    def __init__(self, lib):
        self._lib = lib
        self.ms = defaultdict(float)
        self.calls = defaultdict(int)
        self._pending = []
        self.gemm_shapes = defaultdict(lambda: [0.0, 0])      # (M, N, K) of the tcgen05 GEMM -> [ms, calls] of the last collect()

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("lp_") or name.endswith("_bytes") or name in ("lp_last_error", "lp_linear_tile_rows", "lp_moe_max_tiles"):
            return fn

        def timed(*a):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*a)
            e1.record()
            shape = tuple(int(getattr(v, "value", v)) for v in a[6:9]) if name == "lp_gemm_bf16" else None
            self._pending.append((name, e0, e1, shape))
            return rc
        return timed

    def collect(self):
        torch.cuda.synchronize()
        self.gemm_shapes.clear()
        for name, e0, e1, shape in self._pending:
            self.ms[name] += e0.elapsed_time(e1)
            self.calls[name] += 1
            if shape is not None:
                self.gemm_shapes[shape][0] += e0.elapsed_time(e1)
                self.gemm_shapes[shape][1] += 1
        self._pending.clear()
        out = {k: {"ms": round(v, 4), "calls": self.calls[k]} for k, v in self.ms.items()}
        self.ms.clear()
        self.calls.clear()
        return out


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_size(name, s, dev, steps, warmup, peaks, prompt):
    from leopard_b200 import zudalorn
    from leopard_b200.seqlm import SeqLMEngine, SeqLMWeights, StepEntry
    cfg_d = zudalorn_config(s)
    cfg = zudalorn.config_from_dict(cfg_d)
    eng = SeqLMEngine(cfg, SeqLMWeights(cfg, random_getter(cfg_d, dev), zudalorn.tensor_name, dev), dtype="bfloat16",
                      max_tokens=64 * 600 + prompt, max_seqs=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, s["vocab"], (prompt,), generator=g).tolist()
    out = {"size": name, **{k: s[k] for k in ("width", "heads", "ff", "kv_rank", "window", "experts", "top")}, "prompt": prompt}

    def prefill():
        eng.step([StepEntry("p", toks, [prompt - 1])])
        eng.finish("p")
    ms = _time(prefill, steps, warmup)
    out["prefill_ms"], out["prefill_tokens_per_s"] = round(ms, 3), round(prompt / ms * 1e3, 1)
    # per-kernel device time of one prefill step
    plain = eng.L
    eng.L = TimedLib(plain)
    prefill()
    kp = eng.L.collect()
    D, H, R = s["width"], s["heads"], prompt
    flops_gemm = 0.0
    for lc in cfg_d["layers"]:      # the products that run on the tcgen05 GEMM: fused projections, output projections, dense / shared FF
        m = lc["mixer"]
        if lc["type"] == "retention":
            flops_gemm += 2.0 * R * D * (2 * H * HEAD + 2 * H * HEAD) + 2.0 * R * D * H * HEAD
        else:
            flops_gemm += 2.0 * R * D * (H * (HEAD + 64) + m["kv_rank"] + 64) + 2.0 * R * D * H * HEAD
        f = lc["mlp"]
        flops_gemm += 2.0 * R * D * f["ff"] * 2 if f["kind"] == "dense" else 2.0 * R * D * f["shared"]["ff"] * 3
    flops_gemm += 2.0 * D * s["vocab"] * 0          # the head runs on one row (rows kernel)
    ret_flops = 3 * (R * H * (4.0 * HEAD * HEAD + 2.0 * 32 * 2 * HEAD))
    keys = sum(min(p + 1, s["window"]) for p in range(R))
    lat_flops = H * keys * (2.0 * (s["kv_rank"] + 64) + 2.0 * s["kv_rank"])
    moe_flops = 2 * (R * s["top"] * 2.0 * D * s["expert_ff"] * 3)
    if "lp_linear_grouped" not in kp:         # the experts ran as tcgen05 GEMMs over their sorted row segments
        flops_gemm += moe_flops
    def rate(key, flops):
        return round(flops / (kp[key]["ms"] * 1e-3) / 1e12, 2) if key in kp and kp[key]["ms"] > 0 else None
    out["prefill_kernels"] = kp
    out["prefill_rates"] = {
        "lp_gemm_bf16_tflops": rate("lp_gemm_bf16", flops_gemm), "of_bf16_peak": None,
        "lp_retention_prefill_tflops": rate("lp_retention_prefill", ret_flops),
        "lp_latent_attend_tflops": rate("lp_latent_attend", lat_flops),
        "lp_linear_grouped_tflops": rate("lp_linear_grouped", moe_flops)}
    if out["prefill_rates"]["lp_gemm_bf16_tflops"]:
        out["prefill_rates"]["of_bf16_peak"] = round(out["prefill_rates"]["lp_gemm_bf16_tflops"] / peaks["bf16_burst"], 3)
    for k in ("lp_retention_prefill_tflops", "lp_latent_attend_tflops", "lp_linear_grouped_tflops"):
        v = out["prefill_rates"][k]
        out["prefill_rates"][k.replace("_tflops", "_of_fp32_fma_peak")] = round(v / FP32_FMA_TFLOPS, 3) if v else None
    eng.L = plain
    # decode: `batch` requests with 512 tokens of history each
    out["decode"] = {}
    for batch in (1, 8, 64):
        keys_ = [("d", i) for i in range(batch)]
        eng.step([StepEntry(k, toks[:512], []) for k in keys_])
        nxt = [int(t) for t in torch.randint(0, s["vocab"], (batch,), generator=g)]

        def decode():
            eng.step([StepEntry(k, [t], [0]) for k, t in zip(keys_, nxt)])
        ms = _time(decode, steps, warmup)
        d = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch / ms * 1e3, 1)}
        if batch in (1, 8):
            eng.L, eng.use_graphs = TimedLib(plain), False      # the breakdown needs the launches one by one
            decode()
            kd = eng.L.collect()
            eng.L, eng.use_graphs = plain, True
            d["kernels"] = kd
            # weight bytes the dense products stream once per step (rows kernel): everything but the experts, plus the head
            wbytes = 0
            for lc in cfg_d["layers"]:
                m = lc["mixer"]
                wbytes += 2 * D * (4 * H * HEAD + H * HEAD) if lc["type"] == "retention" else 2 * (D * (H * (HEAD + 64) + m["kv_rank"] + 64) + D * H * HEAD + 2 * H * HEAD * m["kv_rank"])
                f = lc["mlp"]
                wbytes += 2 * 2 * D * f["ff"] if f["kind"] == "dense" else 2 * 3 * D * f["shared"]["ff"]
            wbytes += 2 * D * s["vocab"]
            if "lp_linear" in kd:
                d["lp_linear_gbs"] = round(wbytes / (kd["lp_linear"]["ms"] * 1e-3) / 1e9, 1)
                d["lp_linear_of_copy_peak"] = round(d["lp_linear_gbs"] / peaks["hbm_gbs"], 3)
            st_bytes = 3 * batch * H * HEAD * HEAD * 4 * 2
            if "lp_retention_decode" in kd:
                d["lp_retention_decode_gbs"] = round(st_bytes / (kd["lp_retention_decode"]["ms"] * 1e-3) / 1e9, 1)
        out["decode"][str(batch)] = d
        for k in keys_:
            eng.finish(k)
    del eng
    torch.cuda.empty_cache()
    return out


def bench_llama_twin(name, s, dev, steps, warmup, prompt):
    """the framework's Llama-style decoder at the same width / feed-forward / depth / vocabulary: prefill and batch-1 decode"""
    from dataclasses import replace
    from leopard_b200.config import leopard_llava, reduced
    from leopard_b200.decode import GreedyDecoder
    from leopard_b200.engine import PrefillEngine
    from leopard_b200.native_weights import random_native
    cfg = reduced(leopard_llava(), vit_layers=1, dec_layers=4, vocab=s["vocab"])
    cfg = replace(cfg, dec=replace(cfg.dec, hidden=s["width"], ffn=s["ff"], heads=s["heads"], kv_heads=s["heads"] // 4))      # the Llama path is built for 4 query heads per kv head
    eng = PrefillEngine(cfg, random_native(cfg, dev, seed=7))
    ids = torch.randint(0, s["vocab"] - 100, (prompt,), generator=torch.Generator().manual_seed(0))
    out = {"size": name}

    def prefill():
        eng.prefill([(ids, None)], "last")
    ms = _time(prefill, steps, warmup)
    out["prefill_ms"], out["prefill_tokens_per_s"] = round(ms, 3), round(prompt / ms * 1e3, 1)
    n_new = 65
    dec = GreedyDecoder(eng)
    dec.run(ids[:512], None, n_new, set())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dec.run(ids[:512], None, n_new, set())
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    eng.prefill([(ids[:512], None)], "last")
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    ms_tok = ((t1 - t0) - (t2 - t1)) * 1e3 / (n_new - 1)
    out["decode"] = {"1": {"ms_per_step": round(ms_tok, 3), "tokens_per_s": round(1e3 / ms_tok, 1)}}
    del eng, dec
    torch.cuda.empty_cache()
    return out


def run(args):
    import bench
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no model of this kind; the comparison arm of this "
                                                              "workload is the framework's own Llama-style decoder"}), flush=True)
        return 0
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: leopard_b200 has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = bench.load_peaks()
    from leopard_b200 import _lib
    n0 = None
    sizes, twins = [], []
    prompt = 4096
    L = _lib.stream32_lib()
    n0 = L.lp_launch_count()
    only = [x for x in (getattr(args, "seqlm_sizes", None) or "").split(",") if x]
    for name, s in SIZES.items():
        if only and name not in only:
            continue
        sizes.append(bench_size(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt))
        try:
            twins.append(bench_llama_twin(name, s, dev, args.steps, max(args.warmup, 3), prompt))
        except Exception as e:      # a width the Llama-style path does not take: say so, keep the rest
            twins.append({"size": name, "unavailable": f"{type(e).__name__}: {e}"[:300]})
    mid = sizes[min(1, len(sizes) - 1)]
    line = {"metric": "seqlm_prefill_tokens_per_s", "value": mid["prefill_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": mid["prefill_ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
            "config": {"model": f"Zudalorn 4-layer stack, {mid['size']}", "global_batch": 1, "seq_len": prompt, "parallelism": "single GPU",
                       "cache_policy": "weights + activations of a step exceed L2 at every size"},
            "gpu_launches": int(L.lp_launch_count() - n0), "peaks": peaks, "fp32_fma_peak_tflops": round(FP32_FMA_TFLOPS, 1),
            "sizes": sizes, "llama_style_twin": twins}
    print(json.dumps(line), flush=True)
    return 0
