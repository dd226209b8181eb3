"""bench.py --workload gavatar: prefill and decode throughput of the Gavatar layers (sink latent attention, mLSTM, talking-heads window
attention, softmax-of-the-chosen experts, token shift; leopard_b200/gavatar.py) at a few sizes that resemble a real model's layers, beside
the framework's closest existing model, the Zudalorn stack of benchmarks/seqlm_bench.py (latent attention, a matrix-state recurrence,
experts), at the same width, head count, latent rank, window, expert sizes and vocabulary on the same step engine.  Random weights,
synthetic token ids, one GPU.

Per size: 3 layers [latent attention + experts, mLSTM + experts, window attention + experts], the first run twice (a loop of one
layer, two passes) — 4 layer runs as in the Zudalorn stack;
  prefill   one request of `prompt` tokens per step through SeqLMEngine.step (cache and states written), tokens/s;
  decode    `batch` running requests with 512 tokens of history advanced by one token per step, tokens/s, for batch 1, 8 and 64;
  kernels   device time per native entry point of one prefill step and one decode step (CUDA events around every call) and the rate
            each reaches against its ceiling: the fp32 FMA peak for the attention and recurrence kernels (their scores, softmax,
            sums and state are fp32), the measured copy bandwidth for the weight-streaming decode products, the measured cuBLAS bf16
            peak for the tcgen05 GEMM.  The same figures of the Zudalorn stack's like kernels stand beside them.
One JSON line in the shape bench.py prints for its other workloads; `value` is the prefill throughput of the middle size.
"""
from __future__ import annotations

import json

import torch

from benchmarks.seqlm_bench import FP32_FMA_TFLOPS, HEAD, SIZES, TimedLib, _time, bench_size

RUNS = 4      # layer runs of the stack: latent, latent (second pass), mLSTM, window attention


def gavatar_config(s):
    H, G = s["heads"], max(s["heads"] // 4, 1)
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    lat = {"heads": H, "dim": HEAD, "vdim": HEAD, "q_rank": s["kv_rank"], "kv_rank": s["kv_rank"], "scale": HEAD ** -0.5,
           "mask": {"size": s["window"]}}
    mem = {"heads": H, "dim": HEAD, "vdim": HEAD, "gate_cap": 15.0}
    att = {"heads": H, "kv_heads": G, "dim": HEAD, "vdim": HEAD, "scale": HEAD ** -0.5, "mask": {"size": s["window"]}}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": moe}, {"type": "mlstm", "mixer": mem, "mlp": moe},
              {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Gavatar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": s["width"] ** 0.5},
            "loop": {"start": 0, "stop": 1, "times": 2}, "layers": layers}


def random_getter(cfg, dev, seed=1):
    g = torch.Generator(device=dev).manual_seed(seed)
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "head": (cfg["vocab"], D), "final.norm": (D,), "loop.step": (cfg["loop"]["times"], D)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b", "shift"):
            shapes[p + n] = (D,)
        H, d, e = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "latent_attention":
            shapes.update({p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * d, m["q_rank"]),
                           p + "mix.dkv": (m["kv_rank"], D), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * d, m["kv_rank"]),
                           p + "mix.uv": (H * e, m["kv_rank"]), p + "mix.sink": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * e)})
        elif layer["type"] == "mlstm":
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (H * d, D), p + "mix.v": (H * e, D), p + "mix.g": (H * e, D),
                           p + "mix.o": (D, H * e), p + "mix.norm": (H * e,), p + "mix.i": (H, D), p + "mix.f": (H, D),
                           p + "mix.i.b": (H,), p + "mix.f.b": (H,)})
        else:
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * e, D), p + "mix.q.b": (H * d,),
                           p + "mix.k.b": (G * d,), p + "mix.v.b": (G * e,), p + "mix.talk": (H, H), p + "mix.g": (H * e, D),
                           p + "mix.o": (D, H * e)})
        f = layer["mlp"]
        E, ff = f["router"]["experts"], f["expert"]["ff"]
        shapes.update({p + "mlp.router": (E, D), p + "mlp.router.b": (E,)})
        for x in range(E):
            shapes.update({f"{p}mlp.e{x}.gate": (ff, D), f"{p}mlp.e{x}.up": (ff, D), f"{p}mlp.e{x}.down": (D, ff)})

    def get(name):
        shape = shapes[name]
        if name.endswith("mix.talk"):
            return (torch.eye(shape[0], device=dev) * 0.7 + torch.randn(shape, device=dev, generator=g) * 0.1).to(torch.bfloat16)
        if len(shape) == 2:
            return (torch.randn(shape, device=dev, generator=g) * shape[1] ** -0.5).to(torch.bfloat16)
        if name.endswith(".norm") and ".mix." in name:
            return (torch.rand(shape, device=dev, generator=g) * 0.5 + 0.75).to(torch.bfloat16)
        if name.endswith("shift"):
            return torch.rand(shape, device=dev, generator=g).to(torch.bfloat16)
        if name.endswith("f.b"):
            return torch.full(shape, 3.0, device=dev).to(torch.bfloat16)
        return ((torch.rand(shape, device=dev, generator=g) - 0.5) * 0.2).to(torch.bfloat16)
    return get


def bench_gavatar(name, s, dev, steps, warmup, peaks, prompt):
    from leopard_b200 import gavatar
    from leopard_b200.seqlm import SeqLMEngine, SeqLMWeights, StepEntry
    cfg_d = gavatar_config(s)
    cfg, source = gavatar.config_from_dict(cfg_d)
    eng = SeqLMEngine(cfg, SeqLMWeights(cfg, random_getter(cfg_d, dev), gavatar.tensor_namer(source), dev), dtype="bfloat16",
                      max_tokens=64 * 600 + prompt, max_seqs=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, s["vocab"], (prompt,), generator=g).tolist()
    D, H, G, R, W, rank = s["width"], s["heads"], max(s["heads"] // 4, 1), prompt, s["window"], s["kv_rank"]
    out = {"size": name, "width": D, "heads": H, "kv_heads": G, "kv_rank": rank, "window": W, "experts": s["experts"], "top": s["top"],
           "expert_ff": s["expert_ff"], "prompt": prompt}

    def prefill():
        eng.step([StepEntry("p", toks, [prompt - 1])])
        eng.finish("p")
    ms = _time(prefill, steps, warmup)
    out["prefill_ms"], out["prefill_tokens_per_s"] = round(ms, 3), round(prompt / ms * 1e3, 1)
    plain = eng.L
    eng.L = TimedLib(plain)
    prefill()
    kp = eng.L.collect()
    eng.L = plain
    hd = H * HEAD
    # the products that run on the tcgen05 GEMM: fused projections, query up-projection, output projections, experts over sorted segments
    flops_gemm = 2 * (2.0 * R * D * (2 * rank + H) + 2.0 * R * rank * hd + 2.0 * R * D * hd)                  # latent, two passes
    flops_gemm += 2.0 * R * D * (4 * hd + 2 * H) + 2.0 * R * D * hd                                             # mLSTM
    flops_gemm += 2.0 * R * D * (hd + 2 * G * HEAD + hd) + 2.0 * R * D * hd                                     # window attention
    moe_flops = RUNS * (R * s["top"] * 2.0 * D * s["expert_ff"] * 3)
    if "lp_linear_grouped" not in kp:
        flops_gemm += moe_flops
    keys = sum(min(p + 1, W) for p in range(R))
    lat_flops = 2 * H * keys * 4.0 * rank                                # absorbed form: score and sum over the latent, two passes
    talk_flops = H * keys * (2.0 * HEAD + 2.0 * HEAD + 2.0 * H)          # scores once, mixing, values (the kernel computes the scores twice)
    mem_flops = R * H * 4.0 * HEAD * (HEAD + 1)                          # state update and read-out

    def per_s(key, amount, unit):
        return round(amount / (kp[key]["ms"] * 1e-3) / unit, 2) if key in kp and kp[key]["ms"] > 0 else None
    if "lp_window_attn_talk_tiles" in kp:      # prompts take the row-tile entry of the same kernel
        kp["lp_window_attn_talk"] = kp["lp_window_attn_talk_tiles"]
    r = {"lp_gemm_bf16_tflops": per_s("lp_gemm_bf16", flops_gemm, 1e12), "lp_latent_attend_tflops": per_s("lp_latent_attend", lat_flops, 1e12),
         "lp_window_attn_talk_tflops": per_s("lp_window_attn_talk", talk_flops, 1e12), "lp_mlstm_tflops": per_s("lp_mlstm", mem_flops, 1e12),
         "lp_token_shift_gbs": per_s("lp_token_shift_f32", RUNS * R * D * (4.0 + 2.0), 1e9)}
    r["lp_gemm_bf16_of_bf16_peak"] = round(r["lp_gemm_bf16_tflops"] / peaks["bf16_burst"], 3) if r["lp_gemm_bf16_tflops"] else None
    for k in ("lp_latent_attend", "lp_window_attn_talk", "lp_mlstm"):
        r[k + "_of_fp32_fma_peak"] = round(r[k + "_tflops"] / FP32_FMA_TFLOPS, 3) if r[k + "_tflops"] else None
    r["lp_token_shift_of_copy_peak"] = round(r["lp_token_shift_gbs"] / peaks["hbm_gbs"], 3) if r["lp_token_shift_gbs"] else None
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
            wbytes = 2.0 * (2 * (D * (2 * rank + H) + rank * hd + 2 * hd * rank + D * hd) + D * (4 * hd + 2 * H) + D * hd +
                            D * (2 * hd + 2 * G * HEAD) + D * hd + D * s["vocab"])
            if "lp_linear" in kd:
                d["lp_linear_gbs"] = round(wbytes / (kd["lp_linear"]["ms"] * 1e-3) / 1e9, 1)
                d["lp_linear_of_copy_peak"] = round(d["lp_linear_gbs"] / peaks["hbm_gbs"], 3)
            st_bytes = batch * H * (HEAD + 1) * (HEAD + 1) * 4.0 * 2      # the state read and written once
            if "lp_mlstm" in kd:
                d["lp_mlstm_gbs"] = round(st_bytes / (kd["lp_mlstm"]["ms"] * 1e-3) / 1e9, 1)
            kv_bytes = batch * 4.0 * 2 * G * HEAD * min(513, W) * 2      # the talking-heads kernel walks the window twice
            if "lp_window_attn_talk" in kd:
                d["lp_window_attn_talk_gbs"] = round(kv_bytes / (kd["lp_window_attn_talk"]["ms"] * 1e-3) / 1e9, 1)
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
        sizes.append(bench_gavatar(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt))
        z = bench_size(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt)
        beside.append({k: z[k] for k in ("size", "prefill_ms", "prefill_tokens_per_s", "prefill_kernels", "prefill_rates", "decode")})
    mid = sizes[min(1, len(sizes) - 1)]
    line = {"metric": "gavatar_prefill_tokens_per_s", "value": mid["prefill_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": mid["prefill_ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
            "config": {"model": f"Gavatar 3-layer stack with a looped first layer, {mid['size']}", "global_batch": 1, "seq_len": prompt,
                       "parallelism": "single GPU", "cache_policy": "weights + activations of a step exceed L2 at every size"},
            "gpu_launches": int(L.lp_launch_count() - n0), "peaks": peaks, "fp32_fma_peak_tflops": round(FP32_FMA_TFLOPS, 1),
            "sizes": sizes, "zudalorn_stack": beside}
    print(json.dumps(line), flush=True)
    return 0
