"""Decode throughput of the hybrid-MoE engine on B200, next to the CPU port of the reference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 (the headline): the full 35B-A3B-shaped model (40 layers, hidden 2048, vocab 151936, 256
experts top-8 + shared, int8 linears, 4-bit experts), random-init and quantised with the repo's
quantisers, all experts resident; batch-1 greedy decode after a 4096-token uniform-random prompt.
A step is one decoded token. `value` is tokens/s of the device-resident greedy loop (CUDA events on
the engine's stream); `e2e` is the same loop driven through the reference-facing call
`feed(&[id]) -> logits` with host buffers (id host->device, 608 KB of logits device->host, arg-max by
the host sampler, every token).

One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PROMPT = 4096
METRIC = "decode tok/s, batch 1, full 40-layer 4-bit hybrid MoE, 1 B200"
METRIC_B64 = "decode tok/s, batch 64, full 40-layer 4-bit hybrid MoE, expert-parallel over N B200"
B64_PROMPT = 8192


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def oracle_sample(cfg_full, steps: int, warmup: int, device: str):
    """The CPU port of the reference path on a bounded sample of the workload: one period of the
    layer pattern (3 DeltaNet + 1 attention layers at full width, all 256 experts of each) plus the
    head, single-token steps after a 4-token prompt; a full-model token costs ten such periods plus
    one head. Weights are re-materialised on every call, as the reference's QLinear does."""
    import torch
    from __graft_entry__ import load_package
    load_package()
    from b200moe import brain
    from b200moe.config import HybridConfig
    from oracle import hybrid_oracle as O

    cfg4 = HybridConfig.full(n_layers=4)
    tensors = {}
    for name, dt, t in brain.random_brain(cfg4, seed=0, device=device):
        t = t.detach().contiguous().cpu()
        tensors[name] = (dt, t.view(torch.int16).numpy().view(np.uint16) if dt == "bf16" else t.numpy())
    model = O.HybridOracle(O.DictBrain(cfg4.to_dict(), tensors), hold_weights=False)
    cache = model.new_cache(1, 8 + warmup + steps, kv_dtype="bf16")
    lg = model.forward(np.asarray([[11, 22, 33, 44]]), cache)[0]
    tok = int(np.argmax(lg))
    for _ in range(warmup):
        tok = int(np.argmax(model.forward(np.asarray([[tok]]), cache)[0]))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = int(np.argmax(model.forward(np.asarray([[tok]]), cache)[0]))
    t_fwd = (time.perf_counter() - t0) / steps
    h = np.zeros((1, cfg4.d_model), dtype=np.float32)
    t0 = time.perf_counter()
    for _ in range(max(1, min(steps, 3))):
        model.qlinear(h, "lm_head")
    t_head = (time.perf_counter() - t0) / max(1, min(steps, 3))
    periods = cfg_full.n_layers / 4
    t_full = (t_fwd - t_head) * periods + t_head
    cores = os.cpu_count() or 1
    return {"value": 1.0 / t_full, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": (f"numpy port of aegist/hybrid.py, fp32, {steps} single-token steps through 4 full-width layers "
                       f"(3 DeltaNet + 1 attention, 256 experts each) + lm_head at context < 16, "
                       f"{t_fwd * 1e3:.0f} ms per sampled token of which head {t_head * 1e3:.0f} ms, "
                       f"scaled to 40 layers + head = {t_full * 1e3:.0f} ms per token")}


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path (its Python model cannot
    travel to the GPU box, so the numpy port stands in), on all host cores, same metric and config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    cfg = pkg.HybridConfig.full()
    steps = max(1, min(args.steps, 4))
    warm = max(0, min(args.warmup, 1))
    dev = "cuda" if torch.cuda.is_available() else "cpu"   # building the weights is set-up, not the timed path
    t0 = time.perf_counter()
    cb = oracle_sample(cfg, steps, warm, dev)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 / cb["value"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line), flush=True)


def workload_config(cfg):
    return {"workload": "full-b1: 40-layer 35B-A3B-shaped model (30 DeltaNet + 10 gated GQA 16q/2kv hd256), hidden 2048, "
                        "vocab 151936, 256 experts top-8 + shared, intermediate 512, int8 linears + 4-bit experts, "
                        "batch 1, 4096-token random prompt, greedy decode",
            "batch": 1, "prompt_tokens": PROMPT, "kv_cache": "bf16", "experts_resident": cfg.n_layers * cfg.n_experts,
            "l2": "per-token traffic (2.5 GB) exceeds L2 (126 MB); no flush needed", "parallelism": "single GPU"}


def run_profile_case(args):
    """Few launches and a few GB: what an ncu capture can replay (every kernel has its full-model shape)."""
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from b200moe import brain
    from b200moe import engine as E
    cfg = pkg.HybridConfig.full(n_layers=args.profile_case)
    eng = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device="cuda:0"),
                                      max_context=PROMPT + 64, device=0, batch=1, kv_dtype=E.KV_BF16)
    eng.seek(PROMPT)
    toks, ms = eng.decode_greedy([1], max(args.warmup, 1))
    toks, ms = eng.decode_greedy([toks[-1, 0]], args.steps)
    print(json.dumps({"profile_case": True, "layers": args.profile_case, "steps": args.steps, "ms_per_step": ms / args.steps,
                      "launches_per_step": eng.launches_per_step(), "note": "not a bench value"}), flush=True)
    if args.timeline:
        # the step as the CUDA graph runs it: per launch, microseconds on the device global timer relative to the
        # first launch, and block 0's own progress (SM cycle counter at the sampled clock) at its points 1..7
        names = {1: "k_tcgemv", 3: "k_delta_step", 5: "k_moe_gu1", 6: "k_moe_down1", 7: "k_attn(_mma)", 8: "k_attn_merge"}
        eng.trace_step()
        t = eng.trace_step().astype(np.int64)
        ghz = args.timeline_ghz
        live = t[t[:, 5] > 0]
        t0 = live[:, 0].min()
        prev = None
        print("kernel hint | first block in, last block in, last block out | since previous kernel's end | block 0: us after it came in, at points 1..7")
        for r in live:
            s, li, e = (r[0] - t0) / 1e3, (r[7] - t0) / 1e3, (r[4] - t0) / 1e3
            pts = " ".join(f"{(r[8 + j] - r[8]) / ghz / 1e3:6.2f}" if r[8 + j] > 0 else "     -" for j in range(1, 8))
            print(f"{names.get(int(r[5]), '?'):13s} {int(r[6]):6d} | {s:7.2f} {li:7.2f} {e:7.2f} | {e - (prev if prev is not None else s):6.2f} | {pts}")
            prev = e


def run_b64(args):
    """Batched decode of 64 sequences, expert-parallel over the ranks (256/N experts of every layer per
    GPU, the routed tokens exchanged by NCCL), router bias for Zipf(1.1) expert popularity."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    from b200moe import brain, ep
    from b200moe import engine as E

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = pkg.HybridConfig.full()
    K, W = args.steps, max(args.warmup, 3)
    Bt = 64
    B = Bt // world
    fed = 16
    cap = B64_PROMPT + W + 2 * K + 64
    t0 = time.perf_counter()
    eng = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device=f"cuda:{local}"),
                                      max_context=cap, device=local, batch=B, kv_dtype=E.KV_BF16, ep_rank=rank, ep_world=world)
    torch.cuda.empty_cache()
    if world > 1:
        ep.attach(eng, rank, world)
    for layer in range(cfg.n_layers):
        eng.set_router_bias(layer, brain.router_popularity_bias(cfg, layer, 0, 1.1).numpy())
    t_build = time.perf_counter() - t0
    # context: the prefill kernels are not built, and feeding 64 x 8192 tokens through the decode path would
    # take minutes, so the length is set directly and only the last `fed` prompt tokens are real
    eng.seek(B64_PROMPT - fed)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab_size, (Bt, fed), generator=g).numpy().astype(np.uint32)[rank * B:(rank + 1) * B]
    for t in range(fed - 1):
        eng.feed_batch(prompt[:, t], want_logits=False)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    toks, _ = eng.decode_greedy(prompt[:, -1], W)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    toks, ms = eng.decode_greedy(toks[-1], K)
    barrier()
    clk = clocks.stop()
    bytes_step = eng.step_bytes()
    # picks per rank in the last step, all layers
    picks = np.stack([eng.router(layer, cfg.experts_active)[0] for layer in range(cfg.n_layers)])
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        allp = [None] * world
        dist.all_gather_object(allp, picks)
        picks = np.concatenate(allp, 1)
    load = np.stack([ep.load_per_rank(picks[l], cfg.n_experts, world) for l in range(cfg.n_layers)]).sum(0)
    uniq = float(np.mean([len(np.unique(picks[l])) for l in range(cfg.n_layers)]))
    value = Bt * K / (ms / 1e3)
    # end to end: ids from the host, the arg-max back to the host, every step
    nxt = toks[-1]
    for _ in range(2):
        nxt, _ = eng.feed_batch(nxt, want_logits=False)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        nxt, _ = eng.feed_batch(nxt, want_logits=False)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    peak, peak_kind = peaks()
    step_gbs = bytes_step / (ms / K * 1e-3) / 1e9
    if rank == 0:
        line = {"metric": METRIC_B64, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": "full-b64: the 40-layer 35B-A3B-shaped model, 64 sequences at context 8192, greedy decode, "
                                       "router bias for Zipf(1.1) expert popularity",
                           "batch": Bt, "sequences_per_gpu": B, "context": B64_PROMPT,
                           "context_note": f"length set to {B64_PROMPT - fed} directly, then {fed} real tokens fed (no prefill kernels yet)",
                           "kv_cache": "bf16", "parallelism": f"ep{world}: {cfg.n_experts // world} experts of every layer per GPU, "
                                                              "sequences split over the GPUs, NCCL all-gather + all-to-all per layer",
                           "l2": "per-step traffic exceeds L2 (126 MB); no flush needed"},
                "e2e": {"value": Bt * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                        "timing": "host wall clock around K feed_batch() calls (ids in, arg-max out), max over ranks"},
                "gpu_launches": eng.launches_per_step() * K,
                "roofline": {"bound": "hbm", "kernel": "whole step, per GPU", "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                             "frac": step_gbs / peak, "peak_kind": peak_kind, "traffic": None,
                             "bytes_per_step_per_gpu": bytes_step},
                "expert_load": {"picks_per_rank": load.tolist(), "max_over_mean": float(load.max() / load.mean()),
                                "unique_experts_per_layer": uniq},
                "cpu_baseline": None, "clocks": clk, "setup": {"build_s": round(t_build, 1)}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) per launch from the ncu launch list of the 4-layer full-width case, averaged over the
# launches of a role in the 40-layer model (30 DeltaNet + 10 attention layers): in_proj = (30 x 26.02 + 10 x 19.90 +
# 40 x 3.33) / 80 MB, and so on; the per-launch figures are in the file named below.
NCU_DRAM_SOURCE = "profiles/decode_step_launch_list_4layer_case.md"
NCU_DRAM_BYTES_PER_LAUNCH = {"in_proj": 13.91e6, "out_proj": 8.76e6, "expert_gate_up": 10.13e6, "expert_down": 6.00e6,
                             "head": 321.4e6, "delta_step": 2.14e6, "attention": 4.64e6}


def graph_timeline(eng, prof):
    """Per role: microseconds per step inside the CUDA graph (from the end of the previous launch to the end of this
    one, device global timer) and the GB/s that gives for the role's algorithmic bytes."""
    role_of = {3: "delta_step", 5: "expert_gate_up", 6: "expert_down", 7: "attention", 8: "attention"}
    eng.trace_step()
    t = eng.trace_step().astype(np.int64)
    acc, prev_end = {}, None
    for r in t:
        if r[5] == 0:
            continue
        if r[5] == 1:
            role = "head" if r[6] > 100000 else ("out_proj" if r[6] == eng.d_model else "in_proj")
        else:
            role = role_of.get(int(r[5]), "other")
        acc[role] = acc.get(role, 0.0) + (r[4] - (prev_end if prev_end is not None else r[0])) / 1000.0
        prev_end = r[4]
    return {n: {"us_per_step": round(us, 1), "GBps": round(prof[n]["bytes"] / us / 1e3, 1) if n in prof and us > 0 else None}
            for n, us in acc.items()}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    from b200moe import brain
    from b200moe import engine as E

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    E.load_library()
    cfg = pkg.HybridConfig.full()
    K, W = args.steps, max(args.warmup, 3)
    cap = PROMPT + W + 3 * K + 64
    t0 = time.perf_counter()
    eng = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device=f"cuda:{local}"),
                                      max_context=cap, device=local, batch=1, kv_dtype=E.KV_BF16)
    torch.cuda.empty_cache()
    t_build = time.perf_counter() - t0
    g = torch.Generator().manual_seed(rank)
    prompt = torch.randint(0, cfg.vocab_size, (PROMPT,), generator=g).numpy().astype(np.uint32)
    t0 = time.perf_counter()
    eng.feed(prompt[:-1], want_logits=False)
    t_prefill = time.perf_counter() - t0

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # warm-up, then exactly K timed steps of the device-resident greedy loop
    toks, _ = eng.decode_greedy([prompt[-1]], W)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    toks, ms = eng.decode_greedy([toks[-1, 0]], K)
    barrier()
    clk = clocks.stop()
    bytes_step = eng.step_bytes()
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * K / (ms / 1e3)

    # end to end through feed(): id host->device, logits device->host, host arg-max, every token
    last = int(toks[-1, 0])
    rng = E.Rng(0)
    ids_h = eng.host_buffer(1, np.uint32)            # page-locked: the id and the logits travel by plain DMA
    logits_h = eng.host_buffer(cfg.vocab_size)
    for _ in range(3):
        ids_h[0] = last
        last = E.sample(eng.feed(ids_h, out=logits_h), 0.0, 1.0, 1, rng)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        ids_h[0] = last
        last = E.sample(eng.feed(ids_h, out=logits_h), 0.0, 1.0, 1, rng)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = world * K / e2e_s

    # per-role times for the roofline object: CUDA events around every launch of un-graphed steps (which include the
    # host's launch gaps), and the device-side timeline of a graph-run step (what the timed loop above executes)
    prof = eng.profile_step(8)
    peak, peak_kind = peaks()
    name = max((n for n in prof if prof[n]["launches"]), key=lambda n: prof[n]["ms"])
    dom = prof[name]
    achieved = dom["bytes"] / (dom["ms"] * 1e-3) / 1e9
    step_gbs = bytes_step / (ms / K * 1e-3) / 1e9
    in_graph = graph_timeline(eng, prof)
    roof = {"bound": "hbm", "kernel": f"{name} ({E.HybridEngine.KERNELS_SMALL_BATCH[name]})", "achieved": achieved, "peak": peak,
            "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
            "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(name), "traffic_source": NCU_DRAM_SOURCE,
            "launches_per_step": dom["launches"], "bytes_per_launch": dom["bytes"] / max(dom["launches"], 1),
            "ms_per_launch": dom["ms"] / max(dom["launches"], 1),
            "timing": "CUDA events around each launch of 8 un-graphed steps; in_graph = device global timer inside the CUDA graph",
            "whole_step": {"bytes": bytes_step, "achieved": step_gbs, "frac": step_gbs / peak},
            "per_kernel": {n: {"ms_per_step": round(v["ms"], 4), "GBps": round(v["bytes"] / max(v["ms"], 1e-9) / 1e6, 1),
                               "launches": v["launches"], "kernel": E.HybridEngine.KERNELS_SMALL_BATCH[n]} for n, v in prof.items()},
            "in_graph": in_graph}
    cb = None
    n_launch = eng.launches_per_step()
    if rank == 0 and world == 1 and not args.no_cpu:
        eng.close()
        torch.cuda.empty_cache()
        cb = oracle_sample(cfg, 3, 1, f"cuda:{local}")
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_config(cfg),
                "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": cfg.vocab_size * 4,
                        "timing": "host wall clock around K feed() calls (id and logits in page-locked host arrays, b2_sample arg-max on the host), synchronised on both sides"},
                "gpu_launches": n_launch * K,
                "roofline": roof, "cpu_baseline": cb, "clocks": clk,
                "setup": {"build_s": round(t_build, 1), "prefill_s": round(t_prefill, 1),
                          "prefill": "prompt fed through the decode path, untimed"}}
        if world > 1:
            line["config"]["parallelism"] = f"{world} independent replicas (batch-1 decode does not shard)"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="auto", choices=["auto", "b1", "b64"],
                    help="b1: batch-1 decode (the default on one GPU); b64: 64 sequences, expert-parallel (the default on several)")
    ap.add_argument("--timeline", action="store_true",
                    help="with --profile-case: also print the device-side timeline of one graph-run step (b2_debug_trace_step)")
    ap.add_argument("--timeline-ghz", type=float, default=1.965, help="SM clock for converting block 0's cycle counts")
    ap.add_argument("--profile-case", type=int, default=0, metavar="LAYERS",
                    help="a short run for profiler captures: the first LAYERS layers at full width, the context "
                         "length set to 4096 without a prompt, no end-to-end or CPU leg; its line is not a bench value")
    a = ap.parse_args()
    if a.profile_case:
        run_profile_case(a)
    elif a.impl == "reference":
        run_reference(a)
    elif a.workload == "b64" or (a.workload == "auto" and int(os.environ.get("WORLD_SIZE", "1")) > 1):
        run_b64(a)
    else:
        run_ours(a)
