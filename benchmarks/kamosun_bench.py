"""bench.py --workload kamosun: prefill and decode throughput of the Kamosun layers (block-local attention with and without keys of its
own, causal capped attention beside lightning attention, clamped gated units dense and as experts weighted on their input, Dynamic-Tanh
norms, gated residual branches, depth average; leopard_b200/kamosun.py) at a few sizes that resemble a real model's layers, beside the
framework's closest existing model, the Zudalorn stack of benchmarks/seqlm_bench.py (a matrix-state recurrence on the same retention
kernels, attention over a cache, experts with a shared one), at the same width, head count, expert sizes and vocabulary on the same
step engine.  Random weights, synthetic token ids, one GPU.

Per size: 4 layers [attention + dense, attention on the first layer's keys and values + experts, (causal attention | lightning
attention) + experts, attention + experts], blocks of `window` positions;
  prefill   one request of `prompt` tokens per step through SeqLMEngine.step (cache and states written), tokens/s;
  decode    `batch` running requests with 512 tokens of history advanced by one token per step, tokens/s, for batch 1, 8 and 64;
  kernels   device time per native entry point of one prefill step and one decode step (CUDA events around every call) and the rate
            each reaches against its ceiling: the fp32 FMA peak for the attention and recurrence kernels (their scores, softmax,
            sums and state are fp32), the measured copy bandwidth for the weight-streaming decode products and the elementwise
            kernels, the measured cuBLAS bf16 peak for the tcgen05 GEMM.  The same figures of the Zudalorn stack's like kernels stand
            beside them.
One JSON line in the shape bench.py prints for its other workloads; `value` is the prefill throughput of the middle size.
"""
from __future__ import annotations

import json

import torch

from benchmarks.seqlm_bench import FP32_FMA_TFLOPS, HEAD, SIZES, TimedLib, _time, bench_size

LAYERS = 4


def kamosun_config(s):
    H, G = s["heads"], max(s["heads"] // 4, 1)
    att = {"heads": H, "kv_heads": G, "dim": HEAD, "vdim": HEAD, "scale": HEAD ** -0.5, "rot": {"base": 1e6, "dims": HEAD},
           "mask": {"size": s["window"]}}
    left = {"heads": H // 2, "kv_heads": max(G // 2, 1), "dim": HEAD, "vdim": HEAD, "scale": HEAD ** -0.5, "softcap": 30.0,
            "rot": {"base": 1e6, "dims": HEAD, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": H // 2, "dim": HEAD, "vdim": HEAD, "decay": [1 - 2.0 ** (-4 - 4 * i / max(H // 2 - 1, 1)) for i in range(H // 2)]}
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0}, "shared": {"ff": s["shared_ff"], "limit": 7.0},
           "router": {"experts": s["experts"], "top": s["top"]}}
    layers = [{"type": "attention", "mixer": att, "mlp": dense}, {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": moe},
              {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Kamosun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": layers}


def random_getter(cfg, dev, seed=1):
    g = torch.Generator(device=dev).manual_seed(seed)
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "head": (cfg["vocab"], D)}

    def dyt(name):
        shapes.update({name: (D,), name + ".b": (D,), name + ".alpha": ()})

    def glu(p, ff):
        shapes.update({p + "gate": (ff, D), p + "up": (ff, D), p + "down": (D, ff)})

    def attention(p, m, bias):
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        names = {"q": H * d, "k": G * d, "v": G * e} if m.get("kv_from") is None else {"q": H * d}
        for k, n in names.items():
            shapes[p + k] = (n, D)
            if bias:
                shapes[p + k + ".b"] = (n,)
            if k != "v":
                shapes[p + k + ".norm"] = (d,)
        shapes[p + "o"] = (D, H * e)
        if bias:
            shapes[p + "o.b"] = (D,)

    dyt("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        dyt(p + "norm1")
        dyt(p + "norm2")
        shapes.update({p + "rg1": (D, D), p + "rg1.b": (D,), p + "rg2": (D, D), p + "rg2.b": (D,), p + "dwa": (i + 2,)})
        if layer["type"] == "attention":
            attention(p + "mix.", m, True)
        else:
            attention(p + "mix.left.", m["left"], False)
            r = m["right"]
            hd, hv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            shapes.update({p + "mix.right.q": (hd, D), p + "mix.right.k": (hd, D), p + "mix.right.v": (hv, D), p + "mix.right.g": (hv, D),
                           p + "mix.right.o": (D, hv), p + "mix.right.norm": (hv,), p + "mix.left.out": (D,), p + "mix.right.out": (D,)})
        f = layer["mlp"]
        if f["kind"] == "dense":
            glu(p + "mlp.", f["ff"])
        else:
            shapes[p + "mlp.router"] = (f["router"]["experts"], D)
            for x in range(f["router"]["experts"]):
                glu(f"{p}mlp.e{x}.", f["expert"]["ff"])
            glu(p + "mlp.shared.", f["shared"]["ff"])

    def get(name):
        shape = shapes[name]
        if len(shape) == 2:
            return (torch.randn(shape, device=dev, generator=g) * shape[1] ** -0.5).to(torch.bfloat16)
        if name.endswith(".alpha"):
            return torch.full((), 0.75, device=dev).to(torch.bfloat16)
        if name.endswith("dwa"):      # mostly the newest result
            t = torch.full(shape, 0.1 / shape[0], device=dev)
            t[-1] = 0.9
            return t.to(torch.bfloat16)
        if name.endswith(".b"):
            return ((torch.rand(shape, device=dev, generator=g) - 0.5) * 0.2).to(torch.bfloat16)
        return (torch.rand(shape, device=dev, generator=g) * 0.5 + 0.75).to(torch.bfloat16)
    return get


def bench_kamosun(name, s, dev, steps, warmup, peaks, prompt):
    from leopard_b200 import kamosun
    from leopard_b200.seqlm import SeqLMEngine, SeqLMWeights, StepEntry
    cfg_d = kamosun_config(s)
    cfg = kamosun.config_from_dict(cfg_d)
    eng = SeqLMEngine(cfg, SeqLMWeights(cfg, random_getter(cfg_d, dev), kamosun.tensor_name, dev), dtype="bfloat16",
                      max_tokens=64 * 600 + prompt, max_seqs=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, s["vocab"], (prompt,), generator=g).tolist()
    D, H, G, R, W = s["width"], s["heads"], max(s["heads"] // 4, 1), prompt, s["window"]
    HL, GL, HR = H // 2, max(G // 2, 1), H // 2
    out = {"size": name, "width": D, "heads": H, "kv_heads": G, "block": W, "ff": s["ff"], "experts": s["experts"], "top": s["top"],
           "expert_ff": s["expert_ff"], "shared_ff": s["shared_ff"], "prompt": prompt}

    def prefill():
        eng.step([StepEntry("p", toks, [prompt - 1])])
        eng.finish("p")
    ms = _time(prefill, steps, warmup)
    out["prefill_ms"], out["prefill_tokens_per_s"] = round(ms, 3), round(prompt / ms * 1e3, 1)
    plain = eng.L
    eng.L = TimedLib(plain)
    prefill()
    kp = eng.L.collect()
    # the tcgen05 GEMM's launches by shape: which products the time goes to
    out["prefill_gemm_shapes"] = [{"M": m, "N": n, "K": k, "ms": round(v[0], 4), "calls": v[1], "tflops": round(2.0 * m * n * k * v[1] / (v[0] * 1e-3) / 1e12, 1)}
                                  for (m, n, k), v in sorted(eng.L.gemm_shapes.items(), key=lambda kv: -kv[1][0])]
    eng.L = plain
    hd = H * HEAD
    # the products that run on the tcgen05 GEMM: input projections (with the branch gates), output projections, dense and shared units
    flops_gemm = 2.0 * R * D * ((hd + 2 * G * HEAD) * 2 + hd) + 3 * 2.0 * R * D * hd                  # three attention layers, one without k, v
    flops_gemm += 2.0 * R * D * (HL * HEAD + 2 * GL * HEAD + 4 * HR * HEAD) + 2.0 * R * D * (HL + HR) * HEAD      # the parallel mixer
    flops_gemm += LAYERS * 2 * 2.0 * R * D * D                                                         # the gates of the residual branches
    flops_gemm += 3 * 2.0 * R * D * s["ff"] + 3 * 3 * 2.0 * R * D * s["shared_ff"]
    moe_flops = 3 * (R * s["top"] * 2.0 * D * s["expert_ff"] * 3)
    if "lp_linear_grouped" not in kp:
        flops_gemm += moe_flops
    block_keys = sum(p % W + 1 for p in range(R))
    attn_flops = 3 * H * block_keys * 4.0 * HEAD + HL * (R * (R + 1) / 2) * 4.0 * HEAD
    ret_flops = R * HR * (4.0 * HEAD * HEAD + 2.0 * 32 * 2 * HEAD)
    elem_bytes = {"lp_dyt_f32": LAYERS * R * D * (4.0 + 2 * 2.0), "lp_depth_average_f32": sum(R * D * 4.0 * (i + 2 + 2) for i in range(LAYERS)),
                  "lp_gated_axpy_f32": R * D * 4.0 * 4}

    def per_s(key, amount, unit):
        return round(amount / (kp[key]["ms"] * 1e-3) / unit, 2) if key in kp and kp[key]["ms"] > 0 else None
    attn_key = "lp_window_attn_tiles" if "lp_window_attn_tiles" in kp else "lp_window_attn"
    r = {"lp_gemm_bf16_tflops": per_s("lp_gemm_bf16", flops_gemm, 1e12), "lp_window_attn_tflops": per_s(attn_key, attn_flops, 1e12),
         "lp_retention_prefill_tflops": per_s("lp_retention_prefill", ret_flops, 1e12),
         "lp_linear_grouped_tflops": per_s("lp_linear_grouped", moe_flops, 1e12)}
    r["lp_gemm_bf16_of_bf16_peak"] = round(r["lp_gemm_bf16_tflops"] / peaks["bf16_burst"], 3) if r["lp_gemm_bf16_tflops"] else None
    for k in ("lp_window_attn", "lp_retention_prefill", "lp_linear_grouped"):
        r[k + "_of_fp32_fma_peak"] = round(r[k + "_tflops"] / FP32_FMA_TFLOPS, 3) if r[k + "_tflops"] else None
    for k, nbytes in elem_bytes.items():
        r[k + "_gbs"] = per_s(k, nbytes * (kp[k]["calls"] if k == "lp_gated_axpy_f32" and k in kp else 1), 1e9)
        r[k + "_of_copy_peak"] = round(r[k + "_gbs"] / peaks["hbm_gbs"], 3) if r[k + "_gbs"] else None
    out["prefill_kernels"], out["prefill_rates"] = kp, r
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
            # weight bytes the dense products stream once per step: everything but the experts, plus the head
            wbytes = 2.0 * (D * ((hd + 2 * G * HEAD) * 2 + hd) + 3 * D * hd + D * (HL * HEAD + 2 * GL * HEAD + 4 * HR * HEAD) +
                            D * (HL + HR) * HEAD + LAYERS * 2 * D * D + 3 * D * s["ff"] + 9 * D * s["shared_ff"] + D * s["vocab"])
            if "lp_linear" in kd:
                d["lp_linear_gbs"] = round(wbytes / (kd["lp_linear"]["ms"] * 1e-3) / 1e9, 1)
                d["lp_linear_of_copy_peak"] = round(d["lp_linear_gbs"] / peaks["hbm_gbs"], 3)
            st_bytes = batch * HR * HEAD * HEAD * 4.0 * 2      # the state read and written once
            if "lp_retention_decode" in kd:
                d["lp_retention_decode_gbs"] = round(st_bytes / (kd["lp_retention_decode"]["ms"] * 1e-3) / 1e9, 1)
            kv_bytes = batch * 4.0 * 2 * HEAD * (3 * G * (512 % W + 1) + GL * 513)      # keys and values every attention kernel walks
            if "lp_window_attn" in kd:
                d["lp_window_attn_gbs"] = round(kv_bytes / (kd["lp_window_attn"]["ms"] * 1e-3) / 1e9, 1)
        out["decode"][str(batch)] = d
        for k in keys_:
            eng.finish(k)
    del eng
    torch.cuda.empty_cache()
    return out


def run(args):
    import bench
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no model of this kind; the comparison arm of this "
                                                              "workload is the framework's own Zudalorn stack"}), flush=True)
        return 0
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: leopard_b200 has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = bench.load_peaks()
    from leopard_b200 import _lib
    L = _lib.stream32_lib()
    n0 = L.lp_launch_count()
    only = [x for x in (getattr(args, "seqlm_sizes", None) or "").split(",") if x]
    prompt, sizes, beside = 4096, [], []
    for name, s in SIZES.items():
        if only and name not in only:
            continue
        sizes.append(bench_kamosun(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt))
        z = bench_size(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt)
        beside.append({k: z[k] for k in ("size", "prefill_ms", "prefill_tokens_per_s", "prefill_kernels", "prefill_rates", "decode")})
    mid = sizes[min(1, len(sizes) - 1)]
    line = {"metric": "kamosun_prefill_tokens_per_s", "value": mid["prefill_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": mid["prefill_ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
            "config": {"model": f"Kamosun 4-layer stack, {mid['size']}", "global_batch": 1, "seq_len": prompt,
                       "parallelism": "single GPU", "cache_policy": "weights + activations of a step exceed L2 at every size"},
            "gpu_launches": int(L.lp_launch_count() - n0), "peaks": peaks, "fp32_fma_peak_tflops": round(FP32_FMA_TFLOPS, 1),
            "sizes": sizes, "zudalorn_stack": beside}
    print(json.dumps(line), flush=True)
    return 0
