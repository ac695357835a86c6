"""Benchmark of the KV-cache hot path: decode tokens/s at the Llama-2-7B attention geometry, batch 64,
context 4096 (mixed K4V4 / K3V2 / K2V2 layers, group 32, fp16 window 128), and the fused attention
kernel's achieved HBM GB/s.

A step is one decode step of the hot path for the whole batch: for each of the 32 layers, append the
new token's K/V to the layer cache (quantizing the oldest fp16 group when one is due) and run the fused
dequant attention.  Projections, MLP and sampling are outside the path and are not executed.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2|3|4|5] [--impl reference]

N > 1: launched by torch.distributed.run, one rank per GPU; the batch is split across ranks (no
collective on the data path; config 5 splits KV heads and all-gathers the attention output per layer),
time is the max over ranks.  ``--config 4`` is the stand-alone quantize-on-append sweep (GB/s).
``--impl reference`` times the CPU oracle (the restatement of upstream's kernels; upstream itself has no
CPU implementation) on the host cores.  At N = 1 the line also carries ``upstream_gpu``: upstream's own,
unmodified CUDA extension driven exactly as its attention forward drives it, timed on the same GPU.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tokens/s, KV-cache hot path (32-layer append + fused dequant attention), Llama-2-7B geometry b=64 ctx 4k"
SMI_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
DTYPE = "f16 data, f32 accumulate, u32 packed codes"

# untimed steps launched layer by layer with events before a graph-replayed timed region (per-bit-setting figures)
EAGER_SAMPLE_STEPS = 8
# dram__bytes_read + dram__bytes_write over algorithmic bytes of one fused-attention launch, from the ncu captures
# summarised in profiles/decode_attn_mma_kernel_B32_ctx4096.md (one CTA per head there, so the ratio carries over).
NCU_TRAFFIC_RATIO = {(4, 4): 1.042, (3, 2): 1.082, (2, 2): 1.058}    # fused decode step, device-driven (the bench's launches)


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/kvmix_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for n, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the host cores
def cpu_baseline(cfg, steps=None, warmup=1, budget_s=15.0, all_layers=False):
    """Time the CPU oracle on ONE sequence of the workload at the full context with every host core (OpenMP over the
    heads; the thread count is set explicitly because launchers export OMP_NUM_THREADS=1).  A per-sequence CPU loop
    has the same tokens/s whatever the batch, so tokens/s = 1 / (time of one 32-layer decode step of one sequence).

    all_layers=True runs all layers of the bit map (no extrapolation over layers); otherwise one layer per distinct bit
    setting is timed and the step time is the sum over the layer map."""
    import numpy as np
    import oracle
    from oracle.glue import RefLayerCache
    cores = os.cpu_count() or 1
    threads = oracle.set_threads(cores)
    kinds = sorted({(q["k_bits"], q["v_bits"]) for q in cfg.quant_bits.values()})
    rng = np.random.default_rng(0)
    H, D, T = cfg.n_kv_heads, cfg.head_dim, cfg.context
    k = rng.standard_normal((1, H, T, D)).astype(np.float16)
    v = rng.standard_normal((1, H, T, D)).astype(np.float16)
    q = rng.standard_normal((1, cfg.n_heads, 1, D)).astype(np.float16)
    kn, vn = k[:, :, :1].copy(), v[:, :, :1].copy()

    def make(kb, vb):
        c = RefLayerCache(kb, vb, cfg.group_size, residual_length=cfg.residual_length)
        c.prefill(k, v)
        return c

    if all_layers:
        layers = [make(cfg.quant_bits[l]["k_bits"], cfg.quant_bits[l]["v_bits"]) for l in range(cfg.n_layers)]
        weight = [1] * len(layers)
    else:
        layers = [make(kb, vb) for kb, vb in kinds]
        weight = [sum(1 for r in cfg.quant_bits.values() if (r["k_bits"], r["v_bits"]) == kv) for kv in kinds]

    def step():
        t = 0.0
        for c, w in zip(layers, weight):
            t0 = time.perf_counter()
            c.decode_step(q, kn, vn)
            t += (time.perf_counter() - t0) * w
        return t

    for _ in range(max(1, warmup)):
        step()
    t_start, times = time.perf_counter(), []
    while True:
        times.append(step())
        if (steps is not None and len(times) >= steps) or (steps is None and time.perf_counter() - t_start > budget_s):
            break
    per_seq_step = sum(times) / len(times)
    wall = time.perf_counter() - t_start
    what = (f"all {cfg.n_layers} layers of the bit map" if all_layers else
            f"one layer per bit setting {['K%dV%d' % kv for kv in kinds]}, weighted by the layer map")
    return {"value": 1.0 / per_seq_step, "unit": "tokens/s", "cores": cores, "threads": threads, "kind": "port",
            "sample": f"1 of the {cfg.batch} sequences at ctx {T}, {what}, {len(times)} timed decode steps in {wall:.1f} s "
                      f"(a CPU loop over sequences gives the same tokens/s for any batch)",
            "extrapolated_over_layers": not all_layers, "timed_steps": len(times),
            "ms_per_step_one_sequence": per_seq_step * 1e3, "ms_per_step_full_batch": per_seq_step * cfg.batch * 1e3,
            "wall_ms_per_timed_step": wall / len(times) * 1e3}


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    full = args.config == 2                                    # ctx 4096: all 32 layers of one sequence fit the time budget
    base = cpu_baseline(cfg, steps=max(1, args.steps) if args.steps_given else None, warmup=max(1, args.warmup),
                        budget_s=20.0, all_layers=full)
    line = {"impl": "reference", "metric": METRIC if args.config == 2 else f"decode tokens/s, KV-cache hot path, {cfg.name}",
            "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": base["timed_steps"],
            "warmup": max(1, args.warmup), "ms_per_step": base["wall_ms_per_timed_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "same_config": False, "extrapolated": bool(base["extrapolated_over_layers"]),
            "config": {"workload": cfg.name,
                       "note": "upstream has no CPU implementation of this path; this arm times the CPU restatement of its "
                               "kernels (oracle/) on ONE sequence of the batch with every host core; ms_per_step is the "
                               "wall time of one timed step of that sample, the full-batch step would take "
                               f"{base['ms_per_step_full_batch']:.0f} ms"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "threads", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# The kernel to beat on the same GPU: upstream's extension, unmodified, driven as its forward drives it
def upstream_gpu_leg(cfg, dev, steps_per_setting=34):
    """Per distinct bit setting: one layer at the full batch and context through oracle/upstream_torch.py (upstream's
    cache update + two quantized_gemm + torch glue, upstream's own --use_fast_math build), CUDA-event time per decode
    step averaged over enough steps to include the group-boundary quantizations.  Index range: upstream's kernels use
    32-bit int offsets; the largest here is the prefill quantizer's element count B*H*D*Tq = 64*32*128*3968 = 1.04e9
    < 2^31, so the full batch runs unsliced."""
    import torch
    try:
        from oracle import upstream_torch as up
        ext = up.load_extension("fast")
    except Exception as e:                                      # the build lives in oracle/_ref (needs the upstream tree once)
        return {"unavailable": f"upstream extension not built: {type(e).__name__}: {e}"[:200]}
    from kvmix_b200 import configs
    from kvmix_b200.cache import kv_bytes_per_head
    kinds = sorted({(q["k_bits"], q["v_bits"]) for q in cfg.quant_bits.values()})
    if any(vb == 3 and cfg.head_dim % 11 for _, vb in kinds):
        return {"unavailable": "upstream cannot represent 3-bit values at this head_dim (quantization_cuda.cu:433-434)"}
    B, nh, hkv, D, T = cfg.batch, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.context
    if B * hkv * D * T >= 2 ** 31:
        return {"unavailable": "batch slice would exceed upstream's 32-bit index arithmetic"}
    policy = ("window", cfg.residual_length)
    out, per_kind = {}, {}
    g = torch.Generator(device=dev).manual_seed(99)
    for kb, vb in kinds:
        Gk = 11 if kb == 3 else cfg.group_size
        k, v = configs.synth_kv(B, hkv, T, D, dev, 7)
        st = up.upstream_prefill(ext, k, v, kb, vb, Gk, cfg.group_size, policy)
        del k, v
        q = torch.randn((B, nh, 1, D), generator=g, device=dev, dtype=torch.float16)
        kn = torch.randn((B, hkv, 1, D), generator=g, device=dev, dtype=torch.float16)
        vn = torch.randn((B, hkv, 1, D), generator=g, device=dev, dtype=torch.float16)
        for _ in range(3):
            up.upstream_step(ext, st, q, kn, vn, kb, vb, Gk, cfg.group_size, policy, nh // hkv, None)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps_per_setting):
            up.upstream_step(ext, st, q, kn, vn, kb, vb, Gk, cfg.group_size, policy, nh // hkv, None)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / steps_per_setting
        tkq = st["kq"].shape[3] * (11 if kb == 3 else 32 // kb)
        by = kv_bytes_per_head(tkq, st["vq"].shape[2], st["kfull"].shape[2], st["vfull"].shape[2], D, kb, Gk, vb,
                               cfg.group_size) * B * hkv + 2 * B * nh * D * 2
        per_kind[(kb, vb)] = us
        out[f"K{kb}V{vb}"] = {"us_per_layer_step": us, "algorithmic_gbs": by / us / 1e3}
        del st
        torch.cuda.empty_cache()
    step_us = sum(per_kind[(q["k_bits"], q["v_bits"])] for q in cfg.quant_bits.values())
    return {"what": "unmodified upstream KVmix extension (upstream's nvcc flags, rebuilt for sm_100a) driven by its own "
                    "attention-forward glue: cache update (cat, quantize at group boundaries) + 2 quantized_gemm + softmax "
                    "+ fp16 tail matmuls, one layer per bit setting at the full batch, scaled by the layer map",
            "per_setting": out, "ms_per_step": step_us / 1e3, "tokens_per_s": cfg.batch / (step_us * 1e-6),
            "steps_timed_per_setting": steps_per_setting}


# ------------------------------------------------------------------------------------------------
# Config 4: stand-alone quantize-on-append sweep
def run_config4(args):
    import torch
    import torch.distributed as dist
    from kvmix_b200 import ops, sharding
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    H, D = 32, 128
    W, K = max(3, args.warmup), args.steps
    cells, skipped, rows = [], [], []
    for T in (512, 2048, 8192, 32768):
        for Bg in (1, 16, 64, 256):
            if Bg < world:
                skipped.append(f"B{Bg} T{T}: fewer sequences than GPUs")
                continue
            cells.append((T, Bg))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ops.LAUNCHES[0]
    best = None
    t_all0 = time.perf_counter()
    for T, Bg in cells:
        lo, hi = sharding.shard_range(Bg, world, rank)
        B = hi - lo
        need = B * H * T * D * 2 * 1.6
        fits = torch.tensor([1 if need < torch.cuda.mem_get_info()[0] * 0.9 else 0], device=dev)
        if world > 1:
            dist.all_reduce(fits, op=dist.ReduceOp.MIN)
        if int(fits.item()) == 0:
            skipped.append(f"B{Bg} T{T}: {need / 1e9:.0f} GB per GPU does not fit")
            continue
        g = torch.Generator(device=dev).manual_seed(1000 * rank + T + Bg)
        x = torch.randn((B, H, T, D), generator=g, device=dev, dtype=torch.float16)
        # a seeded set of 4 heavy-tailed (Student-t, nu = 3) channels per head
        chi = torch.randn((B, H, T, 4, 3), generator=g, device=dev).pow(2).sum(-1).div(3.0).sqrt()
        x[..., :4] = (x[..., :4].float() / chi).to(torch.float16)
        del chi
        for bits in (1, 2, 3, 4):
            for G in (32, 128):
                for style in ("k", "v"):
                    if bits == 3 and (style == "v" or G == 128):
                        continue                                  # upstream's 3-bit format: group 11, keys only (D % 11 != 0)
                    fpi = 11 if bits == 3 else 32 // bits
                    if style == "k":
                        Tq = (T // 352) * 352 if bits == 3 else T
                        grp = 11 if bits == 3 else G
                        src = x[:, :, :Tq].transpose(2, 3)         # keys are read in place: no transposed copy
                        code = torch.empty((B, H, D, Tq // fpi), dtype=torch.int32, device=dev)
                        sc = torch.empty((B, H, D, Tq // grp), dtype=torch.float16, device=dev)
                        n = B * H * Tq * D
                    else:
                        grp = G
                        src = x
                        code = torch.empty((B, H, T, D // fpi), dtype=torch.int32, device=dev)
                        sc = torch.empty((B, H, T, D // G), dtype=torch.float16, device=dev)
                        n = B * H * T * D
                    mn = torch.empty_like(sc)
                    by = n * 2 + code.numel() * 4 + 2 * sc.numel() * 2
                    reps = max(1, min(K, int(2e9 // by) + 1))      # small cells repeat K times, the largest ones once or twice
                    for _ in range(min(W, reps)):
                        ops.quantize_into(src, grp, bits, code, sc, mn)
                    if world > 1:
                        dist.barrier()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(reps):
                        ops.quantize_into(src, grp, bits, code, sc, mn)
                    e1.record()
                    torch.cuda.synchronize()
                    ms = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
                    tb = torch.tensor([float(by)], device=dev, dtype=torch.float64)
                    if world > 1:
                        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
                    gbs = float(tb.item()) / (float(ms.item()) * 1e-3) / 1e9
                    rows.append({"T": T, "B": Bg, "bits": bits, "group": grp, "style": style, "us": float(ms.item()) * 1e3,
                                 "GBs": gbs, "bytes": float(tb.item()), "l2_resident": bool(by < 126e6)})
                    if not rows[-1]["l2_resident"] and (best is None or float(tb.item()) > best["bytes"]):
                        best = rows[-1]
                    del code, sc, mn
        del x
        torch.cuda.empty_cache()
    wall = time.perf_counter() - t_all0
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        big = [r for r in rows if not r["l2_resident"]]
        tot_b, tot_t = sum(r["bytes"] for r in big), sum(r["bytes"] / r["GBs"] for r in big)
        agg = tot_b / tot_t if tot_t else 0.0
        line = {"metric": "quantize-on-append GB/s (fp16 read + packed write), sweep of T x batch x bits x group",
                "value": agg, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": wall * 1e3, "higher_is_better": True, "scaling": "weak" if False else "strong",
                "vs_baseline": None, "dtype": "f16 in, f32 arithmetic, u32 packed codes out", "data": "synthetic",
                "config": {"workload": "cfg4-quantize-on-append-sweep [B,32,T,128], T in {512,2048,8192,32768}, B in "
                                       "{1,16,64,256}, bits 1-4, group 32/128 (3-bit: 11), keys (groups over tokens, read in place) "
                                       "and values (groups over channels); batch split over the GPUs",
                           "value_is": "bytes-weighted mean over the cells larger than L2 (126 MB); a step is one pass over the sweep",
                           "cells": len(rows), "skipped": skipped, "l2_policy": "cells under 126 MB are listed but excluded from the mean"},
                "roofline": {"bound": "hbm", "kernel": "quant_strided_kernel / quant_contig_kernel", "achieved": best["GBs"] / world if best else None,
                             "peak": peak, "unit": "GB/s", "frac": (best["GBs"] / world / peak) if best else None,
                             "peak_source": peak_src, "traffic": None,
                             "cell": {k: best[k] for k in ("T", "B", "bits", "group", "style", "us")} if best else None,
                             "note": "largest cell; achieved is per GPU"},
                "e2e": None, "gpu_launches": (ops.LAUNCHES[0] - launches0) * world, "clocks": clocks,
                "table": [[r["T"], r["B"], r["bits"], r["group"], r["style"], round(r["us"], 1), round(r["GBs"], 0)] for r in rows],
                "table_columns": ["T", "batch", "bits", "group", "k|v", "us", "GB/s (all GPUs)"]}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kvmix_b200", choices=["kvmix_b200", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the global batch (smaller smoke runs)")
    ap.add_argument("--context", type=int, default=None, help="override the context length")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-upstream-gpu", action="store_true")
    ap.add_argument("--one-shard-of", type=int, default=1, metavar="N",
                    help="run ONE rank's share of an N-GPU run on this GPU, without the exchange (a kernel-side view of the "
                         "sharded shapes: 1/N of the kv heads of a head-sharded configuration, 1/N of the batch otherwise); the "
                         "line's value is that one shard's tokens/s")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="device-resident leg: replay the whole decode step (every layer's fused launch, and the exchange waits "
                         "of a head-sharded run) from one CUDA graph with the cache lengths held on the device; auto = when "
                         "every layer's geometry is fused by the library, else launch layer by layer from the host")
    ap.add_argument("--v3", action="store_true",
                    help="config 3 with its 12 K3/V3 layers as written, through the 3-bit-value extension (upstream cannot "
                         "represent 3-bit values at head_dim 128); default: those layers run K3/V4, the map upstream could run")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="config 5 on several GPUs: attention outputs exchanged by peer stores from the attention kernel "
                         "(default; falls back to NCCL when symmetric memory is unavailable) or by an NCCL all-gather per layer")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2: Llama-2-7B b64 ctx4k (the headline, batch-sharded); 3: Mistral-7B GQA b8 ctx32k (batch-sharded); "
                         "4: quantize-on-append sweep (GB/s, batch-sharded); "
                         "5: Llama-3-8B b1 ctx131k (KV heads sharded, per-layer NCCL all-gather of the attention output)")
    args = ap.parse_args()
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 20 if args.config != 4 else 3
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    from kvmix_b200 import configs
    if args.config == 4:
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "config 4 has no CPU arm: the quantizer oracle is timed "
                                  "inside the config-2 reference step"}))
            return
        return run_config4(args)
    cfg = configs.config3(v3_as_v4=not args.v3) if args.config == 3 else {2: configs.config2, 5: configs.config5}[args.config]()
    if args.batch:
        cfg.batch = args.batch
    if args.context:
        cfg.context = args.context
    if args.one_shard_of > 1:
        if cfg.shard == "kv_head":
            cfg.n_heads, cfg.n_kv_heads = cfg.n_heads // args.one_shard_of, cfg.n_kv_heads // args.one_shard_of
        else:
            cfg.batch = cfg.batch // args.one_shard_of
        cfg.name += f"-one-shard-of-{args.one_shard_of}"
    if args.impl == "reference":
        return run_reference(args, cfg)

    import torch
    import torch.distributed as dist
    from kvmix_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from kvmix_b200 import sharding
    W, K = args.warmup, args.steps
    L, D = cfg.n_layers, cfg.head_dim
    head_sharded = cfg.shard == "kv_head" and world > 1
    if head_sharded:                                            # every rank holds all sequences, some KV heads
        (k_lo, k_hi), (q_lo, q_hi) = sharding.shard_kv_heads(cfg.n_heads, cfg.n_kv_heads, world, rank)
        B, nh, hkv = cfg.batch, q_hi - q_lo, k_hi - k_lo
    else:                                                       # strong scaling: the global batch is split
        b_lo, b_hi = sharding.shard_batch(cfg.batch, world, rank)
        B, nh, hkv = b_hi - b_lo, cfg.n_heads, cfg.n_kv_heads

    caches = configs.build_layer_caches(cfg, B, dev, extra_tokens=3 * (W + K) + 24 + EAGER_SAMPLE_STEPS, kv_heads=hkv, seed=rank,
                                        device_state=args.graph != "off")
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    mk = lambda h: torch.randn((B, h, 1, D), generator=g, device=dev, dtype=torch.float16)
    dq, dk, dv = [mk(nh) for _ in range(L)], [mk(hkv) for _ in range(L)], [mk(hkv) for _ in range(L)]
    dout = [torch.empty((B, nh, 1, D), device=dev, dtype=torch.float16) for _ in range(L)]
    hq = [t.cpu().pin_memory() for t in dq]
    hk = [t.cpu().pin_memory() for t in dk]
    hv = [t.cpu().pin_memory() for t in dv]
    hout = [torch.empty((B, nh, 1, D), dtype=torch.float16).pin_memory() for _ in range(L)]
    gather = peer = None
    if head_sharded:
        if args.exchange == "peer" and sharding.PeerGather.available():
            try:
                peer = sharding.PeerGather(B, nh, D, dev)
            except Exception as e:                              # symmetric memory not usable here: the NCCL exchange still is
                if rank == 0:
                    print(f"peer exchange unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
        if peer is None:
            gather = sharding.HeadGather(B, nh, D, torch.float16, dev)

    attn_events = []

    def step_device(record):
        for l in range(L):
            c = caches[l]
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                c.decode_step(dq[l], dk[l], dv[l], out=dout[l], peers=peer)
                e1.record()
                attn_events.append((e0, e1, c.packed_bytes() + 2 * B * nh * D * 2, (c.k_bits, c.v_bits)))
            else:
                c.decode_step(dq[l], dk[l], dv[l], out=dout[l], peers=peer)
            if peer is not None:                                # the one exchange step of the path: peer stores from the
                peer.wait()                                     # attention kernel + a bounded wait for all ranks' rows
            elif head_sharded:                                  # or one NCCL all-gather per layer
                gather(dout[l])

    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(L)]
    ev_done = [torch.cuda.Event() for _ in range(L)]
    ev_out = [torch.cuda.Event() for _ in range(L)]

    def make_step_e2e(prefetch):
        """One step through the public cache API with HOST inputs and outputs: each layer's q/k/v come from pinned host
        memory and each layer's output goes back to pinned host memory; the step ends when the last output has landed.
        prefetch=False is a caller that learns q/k/v layer by layer (layer l+1's inputs exist only once layer l's output
        is on its way back): the copy-in of layer l+1 is issued after the copy-out of layer l has been enqueued.
        prefetch=True issues layer l+1's copy-in while layer l's kernels run (all inputs known up front)."""
        def copy_in(l, after=None):
            with torch.cuda.stream(s_in):
                if after is not None:
                    s_in.wait_event(after)
                dq[l].copy_(hq[l], non_blocking=True)
                dk[l].copy_(hk[l], non_blocking=True)
                dv[l].copy_(hv[l], non_blocking=True)
                ev_in[l].record(s_in)

        def step():
            cur = torch.cuda.current_stream()
            s_in.wait_stream(cur)
            copy_in(0)
            for l in range(L):
                if prefetch and l + 1 < L:
                    copy_in(l + 1)
                cur.wait_event(ev_in[l])
                caches[l].decode_step(dq[l], dk[l], dv[l], out=dout[l], peers=peer)
                if peer is not None:
                    peer.wait()
                elif head_sharded:
                    gather(dout[l])
                ev_done[l].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[l])
                    hout[l].copy_(dout[l], non_blocking=True)
                    ev_out[l].record(s_out)
                if not prefetch and l + 1 < L:
                    copy_in(l + 1, after=ev_done[l])            # the next layer's inputs depend on this layer's output
            s_out.synchronize()                                 # the caller reads the step's result
            cur.synchronize()
        return step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # device-resident run -------------------------------------------------------------------------
    for _ in range(W):
        step_device(False)
    for _ in range(EAGER_SAMPLE_STEPS):    # launch by launch with CUDA events around each layer: the per-bit-setting figures
        step_device(True)                  # of a run whose timed region is a graph replay (no events inside a graph)
    torch.cuda.synchronize()
    if peer is not None:
        peer.check()                       # an exchange that does not arrive stops the run here, not after K slow steps
    eager_events, attn_events = attn_events, []
    captured = None
    if args.graph != "off":
        # (the NCCL exchange is launched by torch between the layers; it stays a host-driven step)
        ok = all(c._fused is True and c.steady() for c in caches) and (not head_sharded or peer is not None)
        if world > 1:
            flag = torch.tensor([int(ok)], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        if ok:
            from kvmix_b200 import CapturedDecodeStep
            captured = CapturedDecodeStep(caches, dq, dk, dv, dout, max_replays=K + 3, peers=peer)
            for _ in range(3):
                captured.replay()
        elif args.graph == "on":
            raise SystemExit("--graph on: a layer of this configuration is not served by the fused decode step")
        else:
            for c in caches:               # host-driven from here on: the host mirror is authoritative
                c.state = None
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ops.LAUNCHES[0]
    step_bytes0 = sum(c.packed_bytes() + 2 * B * nh * D * 2 for c in caches)
    torch.cuda.profiler.start()            # `ncu --profile-from-start off` then lists the timed region only
    if captured is not None:
        ms_total = timed(lambda: captured.replay(), K)
    else:
        ms_total = timed(lambda: step_device(True), K)
    torch.cuda.profiler.stop()
    launches = ops.LAUNCHES[0] - launches0
    clocks = sampler.stop() if rank == 0 else None
    step_bytes1 = sum(c.packed_bytes() + 2 * B * nh * D * 2 for c in caches)
    if captured is not None:
        # no events inside a graph: the launch duration is the whole timed region over its launches (gaps included)
        launches = K * L * (2 if peer is not None else 1)
        attn_ms, attn_bytes, n_attn = ms_total, (step_bytes0 + step_bytes1) / 2 * K, K * L
        src_events = eager_events
    else:
        attn_ms = sum(e0.elapsed_time(e1) for e0, e1, _, _ in attn_events)
        attn_bytes = sum(b for _, _, b, _ in attn_events)
        n_attn = len(attn_events)
        src_events = attn_events
    per_kind = {}
    for e0, e1, b, kv in src_events:
        t = per_kind.setdefault(kv, [0.0, 0.0, 0])
        t[0] += e0.elapsed_time(e1)
        t[1] += b
        t[2] += 1
    ctx_now = caches[0].kv_seq_len

    # end-to-end runs: host buffers in, host buffers out, through the public cache API -----------------
    step_serial, step_prefetch = make_step_e2e(False), make_step_e2e(True)
    for _ in range(W):
        step_serial()
    ms_e2e = timed(step_serial, K)
    ms_e2e_pf = timed(step_prefetch, K)

    if world > 1:
        t = torch.tensor([attn_ms, float(attn_bytes)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        attn_ms_all, attn_bytes_all = float(t[0]) / world, float(t[1]) / world
    else:
        attn_ms_all, attn_bytes_all = attn_ms, float(attn_bytes)

    if peer is not None:
        peer.check()                                            # a wait that gave up raises here
    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        achieved = attn_bytes_all / (attn_ms_all * 1e-3) / 1e9
        bit_map = {}
        for r in cfg.quant_bits.values():
            bit_map[(r["k_bits"], r["v_bits"])] = bit_map.get((r["k_bits"], r["v_bits"]), 0) + 1
        traffic = None
        if all(kv in NCU_TRAFFIC_RATIO for kv in bit_map):
            traffic = sum(NCU_TRAFFIC_RATIO[kv] * per_kind[kv][1] / per_kind[kv][2] * n for kv, n in bit_map.items()) / L
        line = {
            "metric": METRIC if args.config == 2 else f"decode tokens/s, KV-cache hot path, {cfg.name}",
            "value": cfg.batch * K / (ms_total * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": cfg.name, "global_batch": cfg.batch, "batch_per_gpu": B, "context": cfg.context,
                       "context_at_end": ctx_now, "layers": L, "heads": nh, "kv_heads": hkv, "head_dim": D,
                       "group": cfg.group_size, "fp16_window": cfg.residual_length,
                       "bit_map": ", ".join(f"{n}xK{kb}V{vb}" for (kb, vb), n in sorted(bit_map.items(), reverse=True)) +
                                  " (3-bit keys use group 11), seeded",
                       "l2_policy": "inputs larger than L2: every step streams the whole cache "
                                    f"({attn_bytes_all / max(1, n_attn) * L / 1e9:.1f} GB per step per GPU)",
                       "step_launched_as": ("one CUDA graph per decode step (cache lengths and ring starts on the device)"
                                            if captured is not None else "one launch per layer from the host"),
                       "parallelism": ((f"kv-head-sharded x{world}, attention outputs exchanged by peer stores from the attention "
                                        f"kernel + bounded device-side wait (NVLink, no collective launch)" if peer is not None else
                                        f"kv-head-sharded x{world}, per-layer NCCL all-gather of the attention output")
                                       if head_sharded else f"batch-sharded x{world}, no data-path collective")},
            "roofline": {"bound": "hbm", "kernel": "decode_attn_gqa_kernel" if cfg.n_heads != cfg.n_kv_heads else "decode_attn_mma_kernel",
                         "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "peak_source": peak_src, "traffic": traffic,
                         "traffic_note": "bytes per launch (layer average): algorithmic bytes of this run x the ncu dram "
                                         "read+write / algorithmic ratio of profiles/decode_attn_mma_kernel_B32_ctx4096.md (the fused decode step there)",
                         "bytes_per_launch": attn_bytes_all / max(1, n_attn),
                         "us_per_launch": attn_ms_all * 1e3 / max(1, n_attn), "launches_timed": n_attn,
                         "timed_launch_is": "one decode step of one layer: ring append + (when due) group quantization + attention",
                         "launch_timing": ("CUDA events around the K replays of the step graph, divided by its attention launches "
                                           "(no events inside a graph: gaps and exchange waits are included); per_bit_setting "
                                           f"comes from {EAGER_SAMPLE_STEPS} untimed steps before it, launched layer by layer with events"
                                           if captured is not None else "CUDA events around every launch of the timed region"),
                         "per_bit_setting": {f"K{kb}V{vb}": {"us": t[0] * 1e3 / t[2], "GBs": t[1] / (t[0] * 1e-3) / 1e9}
                                             for (kb, vb), t in sorted(per_kind.items())},
                         "attention_share_of_step": None if captured is not None else attn_ms_all / ms_total},
            "e2e": {"value": cfg.batch * K / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                    "h2d_bytes_per_step": world * L * B * (nh + 2 * hkv) * D * 2,
                    "d2h_bytes_per_step": world * L * B * nh * D * 2,
                    "api": "KVmixLayerCache.decode_step per layer; pinned host q/k/v in and pinned host output back on copy "
                           "streams; layer l+1's inputs are copied in only after layer l's output is on its way out",
                    "with_inputs_prefetched_one_layer_ahead": {"value": cfg.batch * K / (ms_e2e_pf * 1e-3),
                                                               "ms_per_step": ms_e2e_pf / K}},
            "gpu_launches": launches * world,
            "clocks": clocks,
        }
        if world == 1:
            if not args.no_upstream_gpu:
                del caches[:]
                torch.cuda.empty_cache()
                try:
                    line["upstream_gpu"] = upstream_gpu_leg(cfg, dev)
                except Exception as e:                          # a labelled extra: never takes the bench line down
                    line["upstream_gpu"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
            if not args.no_cpu_baseline:
                base = cpu_baseline(cfg, budget_s=12.0)
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "threads", "kind", "sample")}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
