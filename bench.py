#!/usr/bin/env python
"""bench.py — Leopard-LLaVA multi-image prefill throughput on B200 (contract: see the task's bench section).

  python bench.py --gpus N --steps K --warmup W            our arm (one rank per GPU under torchrun for N > 1)
  python bench.py --impl reference --gpus N --steps K ...  the reference's CPU implementation of the same path
                                                            (oracle port, host cores, bounded sample; rank 0 only)

Metric  : prefill tokens/sec = merged decoder rows (image rows + text rows) processed / time, whole job.
Workload: BASELINE.json configs[2] — 4 images 896x1152 -> adaptive allocation -> 28 crops (4 x (6 tiles + global)),
          64 text ids + 28 placeholders -> S = 4796 merged rows; ONE such request per GPU per step (the config's batch
          of 8 spread over 8 GPUs = weak scaling: per-GPU work fixed as N grows).  Synthetic weights/pixels/ids.
A step  : ViT over 28 crops -> pixel-shuffle + projector -> embed+merge -> 32-layer decoder -> last-token logits.
value   : inputs already resident in HBM.   e2e: the same through the reference-facing plugin call
          (myLlavaForConditionalGeneration.generate, max_new_tokens=1) with HOST tensors: pinned host -> device copy
          of pixel_values/ids and device -> host read of the generated token inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_TEXT = 64
# (width, height) lists — BASELINE.json configs[2] (the metric's configuration) and configs[1]
WORKLOADS = {
    "cfg3": {"images": [(896, 1152)] * 4,
             "label": "cfg3: LLaVA 4x(896x1152) -> adaptive allocation -> 28 crops, 92 prompt ids -> S=4796 merged rows"},
    "cfg2": {"images": [(1344, 1344)],
             "label": "cfg2: LLaVA 1x(1344x1344) -> adaptive allocation -> 17 crops, 81 prompt ids -> S=2937 merged rows"},
}
IMAGE_SIZES = WORKLOADS["cfg3"]["images"]


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback (B200_PROFILING.md)"}


def load_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu --set full capture (profiles/), or None."""
    cands = sorted((ROOT / "profiles").glob("*_gemm_gateup_traffic.json"))
    if not cands:
        return None
    d = json.loads(cands[-1].read_text())
    return d["dram_bytes_read"] + d["dram_bytes_write"], d["algorithmic_bytes"]["total"], cands[-1].name


# ------------------------------------------------------------------------------------------------ clocks sampler
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, pw) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ workload
def make_workload(cfg, name: str = "cfg3"):
    import torch
    from leopard_b200.preprocess import plan_crops
    per_image = plan_crops(WORKLOADS[name]["images"])          # cfg3: [7, 7, 7, 7] from the reference allocator
    n_crops = sum(per_image)
    g = torch.Generator().manual_seed(1)
    pix = torch.rand((n_crops, 3, cfg.vit.image_size, cfg.vit.image_size), generator=g) * 2 - 1   # U(-1, 1), fp32
    g2 = torch.Generator().manual_seed(2)
    text = torch.randint(0, 128000, (N_TEXT,), generator=g2, dtype=torch.long)
    ids = torch.cat([text[:24], torch.full((n_crops,), cfg.image_token_index, dtype=torch.long), text[24:]])[None]
    S = ids.shape[1] + n_crops * (cfg.tokens_per_crop - 1)
    return pix, ids, n_crops, S, per_image


def workload_config(name, per_image, S, world):
    """Identical for both arms (the driver compares it)."""
    return {"workload": WORKLOADS[name]["label"] + ", 1 request per GPU per step, last-token logits; SigLIP-SO400M/14-364 "
                        "tower + projector + Llama-3.1-8B decoder at full size, synthetic weights",
            "crops_per_image": per_image, "S": S,
            "l2_policy": "inputs larger than L2: 17 GB of weights stream from HBM every step (L2 = 126 MB)",
            "parallelism": f"dp{world}: independent requests, one per GPU per step"}


def flops_model(n_crops, S, cfg):
    """Algorithmic FLOPs of one step."""
    T = cfg.vit.tokens
    vit = n_crops * (27 * (30_449_664 * T + 4608 * T * T) + 1_354_752 * T)
    proj = n_crops * 2 * 169 * (4608 * 4096 + 4096 * 4096)
    dec_lin = S * 2 * 32 * 218_103_808
    dec_att = 262_144 * S * S
    head = 2 * 4096 * cfg.dec.vocab
    return {"vit": vit, "proj": proj, "dec_linear": dec_lin, "dec_attn": dec_att, "lm_head_last": head,
            "total": vit + proj + dec_lin + dec_att + head}


# ------------------------------------------------------------------------------------------------ CPU reference arm
METRIC = "prefill tokens/sec (Leopard-LLaVA multi-image prefill, whole job)"


def run_reference(args):
    """`--impl reference`: the reference's own (CPU) implementation of the path = the oracle port, on host cores.  Honours
    --steps / --warmup: every step is one complete full-depth forward of a proportional slice of the workload
    (benchmarks/cpu_reference.py says what the slice is and what it leaves out); nothing is extrapolated."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import torch
    from benchmarks.cpu_reference import CpuSample
    from leopard_b200.config import leopard_llava
    # torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU arm runs on rank 0 alone and takes every host thread it may use
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    cfg = leopard_llava()
    _, _, n_crops, S, per_image = make_workload(cfg, args.workload)
    sample = CpuSample(cfg, n_crops, S, sample_crops=args.cpu_sample_crops)
    for _ in range(args.warmup):
        sample.step()
    secs = [sample.step() for _ in range(args.steps)]
    value = sample.rows * len(secs) / sum(secs)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, per_image, S, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample.desc, "rows_per_step": sample.rows,
                         "step_seconds_min_max": [round(min(secs), 3), round(max(secs), 3)]},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------ extras (rank 0, N = 1)
def decode_extra(model, ids_h, pix_h, cfg, S, peaks, n_new=65):
    """Greedy decode after the prefill: ms per generated token from generate(n_new) - generate(1),
    against the HBM floor (every decoder weight + lm_head + the KV cache read once per token)."""
    import time
    import torch
    d = cfg.dec

    def gen(n):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        o = model.generate(ids_h, pixel_values=pix_h, max_new_tokens=n)
        torch.cuda.synchronize()
        assert o.shape[1] == ids_h.shape[1] + n
        return time.perf_counter() - t0
    gen(n_new)  # graph capture, cache buffer
    t1 = min(gen(1) for _ in range(2))
    tn = min(gen(n_new) for _ in range(2))
    ms = (tn - t1) * 1e3 / (n_new - 1)
    w_bytes = 2 * (d.layers * (d.hidden * (d.heads + 2 * d.kv_heads) * d.head_dim + d.hidden * d.hidden +
                               3 * d.hidden * d.ffn) + model.engine.w.vocab_padded * d.hidden)
    kv_bytes = 2 * d.layers * 2 * S * d.kv_heads * d.head_dim
    ach = (w_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    return {"ms_per_token": round(ms, 4), "new_tokens": n_new, "context_rows": S, "bound": "hbm",
            "algorithmic_bytes_per_token": w_bytes + kv_bytes, "achieved": round(ach, 1), "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4),
            "api": "generate(max_new_tokens=65) minus generate(max_new_tokens=1): CUDA-graph replay of "
                   "lp_decode_greedy_step per token, 8-byte token read-back per token"}


def frontend_extra(model, ids_h, cfg, S, dev, steps):
    """GPU image front-end on the same request given as raw images: 4 x (896 x 1152) RGB uint8 ->
    28 crops.  Times the front-end alone (pinned uint8 H2D + kernels), the request end to end from raw images, and the
    reference's host path (PIL resize/pad/tile + processor arithmetic, 1 thread) on this box; checks bit-exactness."""
    import time
    import numpy as np
    import torch
    from PIL import Image
    from leopard_b200.frontend import ImageFrontend
    from leopard_b200.preprocess import preprocess_images, to_pixel_values
    rng = np.random.default_rng(7)
    imgs = [torch.from_numpy(rng.integers(0, 256, (h, w, 3), dtype=np.uint8)).pin_memory() for (w, h) in IMAGE_SIZES]
    fe = ImageFrontend(dev)
    pv, per_image = fe(imgs)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        pv, _ = fe(imgs, dtype=torch.bfloat16)
    e1.record()
    torch.cuda.synchronize()
    fe_ms = e0.elapsed_time(e1) / steps

    def step():
        p, _ = fe(imgs, dtype=torch.bfloat16)
        return model.generate(ids_h, pixel_values=p, max_new_tokens=1, use_cache=False).cpu()
    step()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / steps
    t0 = time.perf_counter()
    crops, per_image_host = preprocess_images([Image.fromarray(t.numpy(), "RGB") for t in imgs])
    host = to_pixel_values(crops)
    host_ms = (time.perf_counter() - t0) * 1e3
    exact = per_image_host == per_image and bool(torch.equal(fe(imgs)[0].cpu(), host))
    u8 = sum(t.numel() for t in imgs)
    return {"images": "4 x (896 x 1152) RGB uint8 -> 28 crops [28, 3, 364, 364] bf16", "gpu_ms_per_request": round(fe_ms, 4),
            "h2d_bytes_per_request": u8, "bit_exact_vs_pil_host_path": exact,
            "host_pil_ms_per_request": round(host_ms, 2), "host_threads": 1,
            "e2e_from_images": {"value": round(S / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 3),
                                "h2d_bytes_per_step": u8 + ids_h.numel() * 8,
                                "api": "ImageFrontend(host uint8 images) -> generate(host ids, pixel_values, "
                                       "max_new_tokens=1)"}}

# ------------------------------------------------------------------------------------------------ our arm
def library_leg(eng, cfg, ids_d, pix_d, S, native_last, steps):
    """The library competitor on the same box, same weights, same request (benchmarks/library_gpu.py): cuBLAS + flash-attn 2
    (or SDPA) + eager torch in bf16.  Reported beside the native number; its last-row logits cross-check the native path."""
    import torch
    from benchmarks.library_gpu import LibraryPrefill
    lib = LibraryPrefill(cfg, eng.w.named)
    pix = pix_d.to(torch.bfloat16)
    out = None
    for _ in range(2):
        out = lib.prefill(ids_d[0], pix)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        out = lib.prefill(ids_d[0], pix)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    diff = float((out[0].float() - native_last[0].float()).abs().max())
    impl = lib.attention_impl
    del lib
    torch.cuda.empty_cache()
    return {"value": S / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "what": f"torch bf16 on the same B200: F.linear (cuBLAS) + {impl} + eager element-wise ops, same weight tensors "
                    "and inputs, inputs resident",
            "max_abs_diff_vs_native_last_row_logits": diff, "native_abs_max": float(native_last.abs().max())}


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: leopard_b200 has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from benchmarks.dp_bench import DpHarness, make_strong_queue
    from leopard_b200 import _lib, dp
    from leopard_b200.config import leopard_llava
    from leopard_b200.hf import myLlavaForConditionalGeneration
    from leopard_b200.native_weights import random_native

    cfg = leopard_llava()
    L = _lib.lib()
    if args.gemm_pair is not None:
        L.lp_gemm_set_pair_mode(int(args.gemm_pair))
    model = myLlavaForConditionalGeneration.from_native(cfg, random_native(cfg, dev, seed=1234))
    eng = model.engine
    pix_h, ids_h, n_crops, S, per_image = make_workload(cfg, args.workload)
    pix_h, ids_h = pix_h.pin_memory(), ids_h.pin_memory()
    pix_d, ids_d = pix_h.to(dev), ids_h.to(dev)
    harness = DpHarness(eng, dev, world, rank)
    if world > 1:
        # the queue of `world` requests lives in rank 0's HBM (bf16 crops, 22 MB per cfg3 request); request r goes to rank r
        q = [(ids_d[0], pix_d.to(torch.bfloat16)) for _ in range(world)] if rank == 0 else None
        harness.set_queue(q, world, bins=[[r] for r in range(world)])

    def step_replica():
        logits, _, _ = eng.prefill([(ids_d[0], pix_d)], "last", slots=[n_crops])   # ids are resident: slot count from the host plan
        return logits

    # N = 1: the request is resident; N > 1: NCCL scatter from rank 0 -> prefill -> NCCL gather, all inside the step
    step_resident = step_replica if world == 1 else harness.step

    def step_e2e():
        out = model.generate(ids_h, pixel_values=pix_h, attention_mask=None, max_new_tokens=1, use_cache=False)
        return out.cpu()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    warm = 1 if args.quick else max(args.warmup, 3)
    for _ in range(warm):
        step_resident()
    harness.events = []
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = L.lp_launch_count()
    total_ms = timed(step_resident, args.steps)
    launches = L.lp_launch_count() - n0
    clocks = sampler.stop() if rank == 0 else None
    value = world * args.steps * S / (total_ms / 1000.0)
    dp_info = None
    if world > 1:
        sc, co, ga = harness.phase_ms()
        rep_ms = timed(step_replica, args.steps) / args.steps
        dp_info = {"scatter_ms": round(sc, 3), "compute_ms": round(co, 3), "gather_ms": round(ga, 3),
                   "collectives": "per step: 1 header broadcast + NCCL send/recv of ids and bf16 crops from rank 0's HBM to "
                                  "each owner (22.3 MB per cfg3 request), all-gather of the greedy tokens",
                   "replicas_no_collective_ms_per_step": round(rep_ms, 3)}

    if args.quick:  # profiler runs (ncu): the timed loop only, no JSON contract
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": total_ms / args.steps, "gpu_launches": int(launches)}))
        return 0
    # ---- e2e through the plugin API with host buffers (every rank calls generate() on its own host request, the way the
    # reference shards an evaluation set: one process per GPU, evaluations/models/run_eval_llava_siglip_multiimg.sh:9-13)
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps)
    e2e_value = world * args.steps * S / (e2e_ms / 1000.0)
    h2d = pix_h.numel() * pix_h.element_size() + ids_h.numel() * ids_h.element_size()
    d2h = (ids_h.shape[1] + 1) * 8

    # ---- strong scaling: a fixed queue of 8 mixed-size requests (1 .. 28 crops) on rank 0, cost-balanced over the ranks,
    # one varlen batch per rank, scatter / gather inside the step
    strong = None
    if not args.no_extras:
        sq, meta = make_strong_queue(cfg, dev) if rank == 0 or world == 1 else (None, None)
        if world > 1:
            box = [meta]
            dist.broadcast_object_list(box, src=0)
            meta = box[0]
        harness.set_queue(sq, len(meta))
        mine = harness.step()
        harness.step()
        harness.events = []
        k_strong = max(3, min(args.steps, 6))
        ms_strong = timed(harness.step, k_strong) / k_strong
        sc, co, ga = harness.phase_ms()
        tokens = sum(m["S"] for m in meta)
        bins = dp.assign([m["gflop"] for m in meta], world)
        strong = {"queue": meta, "requests": len(meta), "tokens_per_step": tokens, "ms_per_step": round(ms_strong, 3),
                  "value": tokens / (ms_strong * 1e-3), "unit": "tokens/s", "scaling": "strong",
                  "assignment": bins, "gflop_per_rank": [round(sum(meta[i]["gflop"] for i in b), 1) for b in bins],
                  "scatter_ms": round(sc, 3), "compute_ms_max_rank": round(co, 3), "gather_ms": round(ga, 3)}

    # ---- the three stages of the step timed on their own, launched exactly as inside the step (back to back, programmatic dependent
    # launch, no events between kernels): tower (+ pixel shuffle), projector, merge + decoder + last-row logits
    stage_timed = None
    if rank == 0 and args.workload in ("cfg1", "cfg2", "cfg3"):
        k_st = max(3, min(args.steps, 10))
        shuffled = eng.vit(pix_d, shuffle=True)
        feats = eng.project(shuffled)
        x_buf = torch.empty((S, cfg.dec.hidden), dtype=torch.bfloat16, device=dev)
        pos_d = torch.arange(S, dtype=torch.int32, device=dev)

        def st_vit():
            eng.vit(pix_d, shuffle=True)

        def st_proj():
            eng.project(shuffled)

        def st_dec():
            eng.merge(ids_d[0], feats, cfg.image_token_index, cfg.tokens_per_crop, out=x_buf, n_slots=n_crops)
            eng.decoder(x_buf, pos_d, [0, S], "last")

        def one(fn):
            fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(k_st):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / k_st

        stage_timed = {"vit": one(st_vit), "projector": one(st_proj), "decoder": one(st_dec)}

    # ---- per-kernel event timing of one more step (rank 0): roofline of the dominant kernel
    roofline, stages = None, None
    if rank == 0:
        peaks = load_peaks()
        cap = 4096
        _lib.check(L.lp_profile_enable(cap), "lp_profile_enable")
        step_replica()
        recs = (_lib.ProfileRecord * cap)()
        n = L.lp_profile_read(C.cast(recs, C.c_void_p), cap)
        by_kind = {}
        gemm_shapes = {}
        stage_ms = {"vit": 0.0, "projector": 0.0, "decoder": 0.0}
        vit_rows = n_crops * cfg.vit.tokens
        for r in recs[:n]:
            by_kind[r.kind] = by_kind.get(r.kind, 0.0) + r.ms
            # stage attribution: ViT kernels run on n_crops x 676 rows / T = 676 / width 1152, the projector on n_crops x 169 rows
            if r.kind == 1:
                st = "vit" if r.a == vit_rows else ("projector" if r.a == n_crops * cfg.tokens_per_crop else "decoder")
            elif r.kind == 2:
                st = "vit" if r.b == cfg.vit.tokens else "decoder"
            elif r.kind == 3:
                st = "vit" if r.b == cfg.vit.hidden else "decoder"
            else:
                st = "vit" if r.kind in (6, 7) else "decoder"
            stage_ms[st] += r.ms
            if r.kind == 1:
                key = (r.a, r.b, r.c)
                g = gemm_shapes.setdefault(key, [0.0, 0])
                g[0] += r.ms; g[1] += 1
        step_ms_prof = sum(by_kind.values())
        # dominant kernel = the GEMM shape with the largest summed time (decoder gate/up: M=S, N=28672, K=4096)
        (m, nn, k), (ms_sum, cnt) = max(gemm_shapes.items(), key=lambda kv: kv[1][0])
        avg_ms = ms_sum / cnt
        ach = 2.0 * m * nn * k / (avg_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": f"gemm_bf16_kernel M={m} N={nn} K={k} (x{cnt}/step)", "achieved": ach,
                    "peak": peaks["bf16_sustained"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_sustained"],
                    "peak_kind": "sustained cuBLAS bf16, " + peaks["source"], "avg_launch_ms": avg_ms,
                    "share_of_step": ms_sum / step_ms_prof, "traffic": None}
        tr = load_traffic()
        if tr is not None and args.workload == "cfg3":  # bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, ncu --set full)
            roofline.update(traffic=tr[0], traffic_algorithmic_bytes=tr[1], traffic_source="profiles/" + tr[2])
        fm = flops_model(n_crops, S, cfg)
        names = {1: "gemm", 2: "attention", 3: "norm", 4: "rope", 5: "merge", 6: "im2col", 7: "shuffle"}
        gemm_all = sum(v[0] for v in gemm_shapes.values())
        gemm_flops = sum(2.0 * a * b * c * v[1] for (a, b, c), v in gemm_shapes.items())
        step_ms_repl = total_ms / args.steps if world == 1 else dp_info["replicas_no_collective_ms_per_step"]
        stages = {
            "kernel_ms": {names.get(kk, str(kk)): round(v, 3) for kk, v in sorted(by_kind.items())},
            "sum_kernel_ms": round(step_ms_prof, 3),
            "all_gemms_tflops": gemm_flops / (gemm_all * 1e-3) / 1e12,
            "attention_tflops": (fm["dec_attn"] + n_crops * 27 * 4608 * 676 * 676) / (by_kind.get(2, 1e9) * 1e-3) / 1e12,
            "step_tflops_algorithmic": fm["total"] / (step_ms_repl * 1e-3) / 1e12,
            "frac_of_sustained_peak": fm["total"] / (step_ms_repl * 1e-3) / 1e12 / peaks["bf16_sustained"],
            "gemm_shapes": [{"M": a, "N": b, "K": c, "count": v[1], "ms_total": round(v[0], 3),
                             "tflops": round(2.0 * a * b * c * v[1] / (v[0] * 1e-3) / 1e12, 1)}
                            for (a, b, c), v in sorted(gemm_shapes.items(), key=lambda kv: -kv[1][0])],
            "flops": {kk: float(v) for kk, v in fm.items()},
            # BASELINE.json's "ViT+decoder % roofline": algorithmic FLOPs of the stage / the stage's time against the measured
            # sustained cuBLAS bf16 peak.  `roofline_by_stage` times each stage on its own exactly as the step launches it (no
            # events between kernels; the three add up to the step); `roofline_by_stage_kernel_events` is the earlier basis — the
            # summed per-kernel CUDA-event intervals of one profiled step, which carry the event pair and the lost launch overlap of
            # every launch (~20 us each: sum_kernel_ms vs ms_per_step) and so understate the short-kernel stages
            "roofline_by_stage_kernel_events": {
                st: {"ms": round(ms, 3), "tflops": round(fl / (ms * 1e-3) / 1e12, 1),
                     "frac_of_sustained_peak": round(fl / (ms * 1e-3) / 1e12 / peaks["bf16_sustained"], 4)}
                for st, ms, fl in (("vit", stage_ms["vit"], fm["vit"]), ("projector", stage_ms["projector"], fm["proj"]),
                                   ("decoder", stage_ms["decoder"], fm["dec_linear"] + fm["dec_attn"] + fm["lm_head_last"]))
                if ms > 0},
        }
        if stage_timed is not None:
            stages["roofline_by_stage"] = {
                st: {"ms": round(ms, 3), "tflops": round(fl / (ms * 1e-3) / 1e12, 1),
                     "frac_of_sustained_peak": round(fl / (ms * 1e-3) / 1e12 / peaks["bf16_sustained"], 4)}
                for st, ms, fl in (("vit", stage_timed["vit"], fm["vit"]), ("projector", stage_timed["projector"], fm["proj"]),
                                   ("decoder", stage_timed["decoder"], fm["dec_linear"] + fm["dec_attn"] + fm["lm_head_last"]))}
            stages["stage_sum_ms"] = round(sum(stage_timed.values()), 3)
        else:
            stages["roofline_by_stage"] = stages["roofline_by_stage_kernel_events"]

    # ---- rank 0, N = 1 only: the library competitor on this GPU, greedy decode, the GPU image front-end, the CPU baseline
    decode, frontend, library, cpu = None, None, None, None
    if rank == 0 and world == 1 and not args.no_extras:
        library = library_leg(eng, cfg, ids_d, pix_d, S, step_replica(), max(3, min(args.steps, 10)))
        decode = decode_extra(model, ids_h, pix_h, cfg, S, load_peaks())
        if args.workload == "cfg3":
            frontend = frontend_extra(model, ids_h, cfg, S, dev, args.steps)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from benchmarks.cpu_reference import CpuSample
        sample = CpuSample(cfg, n_crops, S, sample_crops=args.cpu_sample_crops)
        sample.step()                                   # warm-up (materialises the weights)
        secs = [sample.step() for _ in range(3)]
        cpu = {"value": sample.rows * len(secs) / sum(secs), "unit": "tokens/s", "cores": torch.get_num_threads(),
               "kind": "port", "sample": sample.desc + "; 1 warm-up + 3 timed steps", "seconds_measured": round(sum(secs), 1)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, per_image, S, world),
            "timed_region": ("one resident request: tower -> projector -> merge -> decoder -> last-row logits" if world == 1 else
                             "queue of N requests resident in rank 0's HBM: NCCL scatter -> prefill on every rank -> NCCL gather "
                             "of the greedy tokens (max over ranks)"),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "api": "leopard_b200.hf.myLlavaForConditionalGeneration.generate(host ids, pixel_values=host fp32, max_new_tokens=1)"},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "stages": stages,
            "cpu_baseline": cpu, "library_gpu": library, "dp": dp_info, "strong": strong, "decode": decode, "frontend": frontend,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=["cfg3", "cfg2", "cfg4", "cfg5", "seqlm", "ronelorn", "gavatar", "kamosun"],
                    help="cfg3 (default) = the metric's configuration; cfg2 = 1 x 1344^2; cfg4 = Idefics2 8 x 980^2; cfg5 = SFT step; "
                         "seqlm = prefill / decode of the layer-list language models beside the Llama-style decoder at equal size; "
                         "ronelorn = the same for the Ronelorn layers beside the Zudalorn stack at equal size; gavatar = the same for the Gavatar layers; kamosun = the same for the Kamosun layers")
    ap.add_argument("--seqlm-sizes", default="", help="seqlm / ronelorn / gavatar / kamosun: comma-separated subset of w1024,w2048,w4096 (default: all three)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the library / strong-scaling / decode / front-end legs")
    ap.add_argument("--quick", action="store_true", help="1 warm-up, timed loop only (for runs under ncu)")
    ap.add_argument("--gemm-pair", type=int, default=None, help="override the GEMM CTA-pair mode (0/1)")
    ap.add_argument("--cpu-sample-crops", type=int, default=1, help="crops in the CPU arm's proportional slice")
    ap.add_argument("--sft-freeze-vit", action="store_true", help="cfg5: freeze the vision tower (--freeze-clip-vision-tower)")
    ap.add_argument("--sft-recompute", default="full", choices=["full", "none"], help="cfg5: activation recompute")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", __file__] + sys.argv[1:]
        return subprocess.call(cmd)
    if args.workload == "seqlm":
        from benchmarks import seqlm_bench
        return seqlm_bench.run(args)
    if args.workload == "ronelorn":
        from benchmarks import ronelorn_bench
        return ronelorn_bench.run(args)
    if args.workload == "gavatar":
        from benchmarks import gavatar_bench
        return gavatar_bench.run(args)
    if args.workload == "kamosun":
        from benchmarks import kamosun_bench
        return kamosun_bench.run(args)
    if args.workload in ("cfg4", "cfg5"):
        from benchmarks import other_workloads
        return other_workloads.run(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
