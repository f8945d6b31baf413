"""Decode throughput of the hybrid-MoE engine on B200, next to the reference's CPU implementation of the same path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|b1|b64]

N = 1 (the headline): the full 35B-A3B-shaped model (40 layers, hidden 2048, vocab 151936, 256
experts top-8 + shared, int8 linears, 4-bit experts), random-init and quantised with the repo's
quantisers, all experts resident; batch-1 greedy decode after a 4096-token uniform-random prompt
(fed through the engine's chunked feed, untimed). A step is one decoded token. `value` is tokens/s of the
device-resident greedy loop (CUDA events on the engine's stream); `e2e` is the same loop driven through the
reference-facing call `feed(&[id]) -> logits` with host buffers (id host->device, 608 KB of logits
device->host, arg-max by the host sampler, every token). `roofline`: every kernel class timed inside the CUDA
graph with the device timer, the dominant one against the measured copy bandwidth. `parity`: a 4-layer
full-width sample brain against the CPU oracle (picks, greedy tokens, logits). `cpu_baseline`: the reference's
own Python model on the host cores over a bounded sample. `b64`: the one-GPU point of the batched series.

N > 1 under torchrun (or `--workload b64`): 64 sequences at context 8192 with Zipf(1.1) expert popularity, split
over the ranks, experts sharded (expert parallel); the per-layer exchange runs on plain peer stores
(`--nccl-exchange`: on NCCL calls). `tokens_sha1` of the first greedy steps must not depend on N.
`--workload b1` on several GPUs runs independent replicas of the batch-1 workload.

`--profile-case L [--workload b64] [--timeline]`: a short run of the first L layers at full width for profiler
captures and for the in-graph step timeline; its line is not a bench value.

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


SAMPLE_LAYERS = 4          # one period of the layer pattern: 3 DeltaNet + 1 attention, at full width


def sample_brain(device: str):
    """The first four layers of the benchmarked model (seed 0, full width, full vocabulary) as device tensors for the
    engine and as host arrays for the CPU legs."""
    import torch
    from __graft_entry__ import load_package
    load_package()
    from b200moe import brain
    from b200moe.config import HybridConfig
    cfg4 = HybridConfig.full(n_layers=SAMPLE_LAYERS)
    dev = list(brain.random_brain(cfg4, seed=0, device=device))
    host = {}
    for name, dt, t in dev:
        c = t.detach().contiguous().cpu()
        host[name] = (dt, c.view(torch.int16).numpy().view(np.uint16) if dt == "bf16" else c.numpy())
    return cfg4, dev, host


def parity_check(E, cfg4, dev, host, tokens: int = 6):
    """The engine (bf16 cache, the kernels of the timed run) against the CPU oracle on the sample brain: a few
    single-token steps, compared on logits, router picks of every layer and greedy tokens."""
    from oracle import hybrid_oracle as O
    model = O.HybridOracle(O.DictBrain(cfg4.to_dict(), host), hold_weights=True)
    cache = model.new_cache(1, tokens + 8, kv_dtype="bf16")
    eng = E.HybridEngine.from_tensors(cfg4.to_dict(), dev, max_context=PROMPT, device=0, batch=1, kv_dtype=E.KV_BF16)
    tok, worst, routes, greedy = 11, 0.0, True, True
    for _ in range(tokens):
        want = model.forward(np.asarray([[tok]]), cache)[0]
        got = eng.feed([tok])
        worst = max(worst, float(np.abs(got - want).max()))
        for layer in range(cfg4.n_layers):
            routes = routes and bool(np.array_equal(eng.router(layer, cfg4.experts_active)[0], model.last_route[layer][0]))
        greedy = greedy and int(np.argmax(got)) == int(np.argmax(want))
        tok = int(np.argmax(want))
    eng.close()
    return {"against": f"CPU oracle, {SAMPLE_LAYERS}-layer full-width sample brain, {tokens} greedy steps, bf16 cache",
            "max_abs": worst, "routes_equal": routes, "greedy_equal": greedy}, model


REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def timed(f) -> float:
    t0 = time.perf_counter()
    f()
    return time.perf_counter() - t0


def cpu_sample(cfg_full, cfg4, host, model, steps: int, warmup: int):
    """The reference path on the host cores over a bounded sample of the workload: single-token steps through one
    period of the layer pattern (3 DeltaNet + 1 attention layers at full width, 256 experts each) plus the head after
    a 4-token prompt; a full-model token costs ten such periods plus one head. With the reference's own Python
    package present under oracle/_ref (placed there by oracle/make_ref.py; it never enters the repository's history)
    this runs the reference's HybridLM in torch fp32 exactly as its parity test does
    (tests/test_hybrid_rust.py:96-116), kind "reference"; otherwise the numpy port, kind "port"."""
    cores = os.cpu_count() or 1
    periods = cfg_full.n_layers / SAMPLE_LAYERS
    if os.path.exists(os.path.join(REF_DIR, "aegist", "hybrid.py")):
        import torch
        from b200moe import nxfile
        from b200moe.brain import Bf16
        sys.path.insert(0, REF_DIR)
        from aegist import nx as NX
        torch.set_num_threads(cores)
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "sample.nx")
            state = {n: (Bf16(a) if dt == "bf16" else a) for n, (dt, a) in host.items()}
            from tokenizers import Tokenizer, models
            tk = Tokenizer(models.WordLevel({"hi": 0, "there": 1, "[UNK]": 2}, unk_token="[UNK]"))
            tk.add_special_tokens(["<|im_start|>", "<|im_end|>", "<|endoftext|>"])
            nxfile.save(path, state, cfg4.to_dict(), tk.to_str(),
                        extra={"quant": "int8", "dtype": "bf16", "experts": "q4a-g64", "seed": 0})
            ref, _, nx = NX.load_model(path, device="cpu", slots=cfg4.n_experts)
            ref.float()
            cache = ref.new_cache(1, 16 + warmup + steps, dtype=torch.float32)
            with torch.no_grad():
                fwd = lambda ids: ref(torch.tensor([ids]), cache=cache, last_only=True)["logits"][0, -1].float()
                tok = int(fwd([11, 22, 33, 44]).argmax())
                for _ in range(warmup):
                    tok = int(fwd([tok]).argmax())
                t0 = time.perf_counter()
                for _ in range(steps):
                    tok = int(fwd([tok]).argmax())
                t_fwd = (time.perf_counter() - t0) / steps
                h = torch.zeros(1, cfg4.d_model)
                ref.lm_head(h)                                   # first call: allocations
                t_head = min(timed(lambda: ref.lm_head(h)) for _ in range(3))
            del ref, cache
            nx.close()
        kind, what = "reference", f"the reference's HybridLM (torch fp32, {cores} threads)"
    else:
        from oracle import hybrid_oracle as O
        model = O.HybridOracle(model.b, hold_weights=False)      # weights re-materialised per call, as the reference's QLinear does
        cache = model.new_cache(1, 16 + warmup + steps, kv_dtype="bf16")
        tok = int(np.argmax(model.forward(np.asarray([[11, 22, 33, 44]]), cache)[0]))
        for _ in range(warmup):
            tok = int(np.argmax(model.forward(np.asarray([[tok]]), cache)[0]))
        t0 = time.perf_counter()
        for _ in range(steps):
            tok = int(np.argmax(model.forward(np.asarray([[tok]]), cache)[0]))
        t_fwd = (time.perf_counter() - t0) / steps
        h = np.zeros((1, cfg4.d_model), dtype=np.float32)
        model.qlinear(h, "lm_head")
        t_head = min(timed(lambda: model.qlinear(h, "lm_head")) for _ in range(3))
        kind, what = "port", f"numpy port of aegist/hybrid.py (fp32, {cores} threads available to BLAS)"
    t_head = min(t_head, 0.75 * t_fwd)                           # the head is part of every sampled token
    t_full = (t_fwd - t_head) * periods + t_head
    return {"value": 1.0 / t_full, "unit": "tok/s", "cores": cores, "kind": kind,
            "sample": (f"{what}: {steps} single-token steps through {SAMPLE_LAYERS} full-width layers "
                       f"(3 DeltaNet + 1 attention, 256 experts each) + lm_head at context < 32, "
                       f"{t_fwd * 1e3:.0f} ms per sampled token of which head {t_head * 1e3:.0f} ms, "
                       f"scaled to {cfg_full.n_layers} layers + head = {t_full * 1e3:.0f} ms per token")}


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path on all host cores, same metric and
    config (see cpu_sample for what runs and what the bounded sample is)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from oracle import hybrid_oracle as O
    cfg = pkg.HybridConfig.full()
    steps = max(1, min(args.steps, 4))
    warm = max(0, min(args.warmup, 1))
    dev = "cuda" if torch.cuda.is_available() else "cpu"   # building the weights is set-up, not the timed path
    t0 = time.perf_counter()
    cfg4, _, host = sample_brain(dev)
    model = O.HybridOracle(O.DictBrain(cfg4.to_dict(), host), hold_weights=False)
    cb = cpu_sample(cfg, cfg4, host, model, steps, warm)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 / cb["value"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line, default=lambda o: o.item() if hasattr(o, 'item') else str(o)), flush=True)


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
    b64 = args.workload == "b64"             # the batched kernels: 64 sequences at context 8192, Zipf(1.1) expert popularity
    batch, ctx = (64, B64_PROMPT) if b64 else (1, PROMPT)
    # under torchrun (batched workload only): expert parallel as in the bench, rank 0 prints
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    if world > 1:
        import torch.distributed as dist
        from b200moe import ep
        assert b64, "--profile-case on several GPUs needs --workload b64"
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    eng = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device=f"cuda:{local}"),
                                      max_context=ctx + 64, device=local, batch=batch // world, kv_dtype=E.KV_BF16,
                                      ep_rank=rank, ep_world=world)
    if world > 1:
        ep.attach(eng, rank, world, peer_stores=not args.nccl_exchange)
    if b64:
        for layer in range(cfg.n_layers):
            eng.set_router_bias(layer, brain.router_popularity_bias(cfg, layer, 0, 1.1).numpy())
    eng.seek(ctx)
    toks, ms = eng.decode_greedy(np.arange(1, batch + 1)[rank * (batch // world):(rank + 1) * (batch // world)], max(args.warmup, 1))
    toks, ms = eng.decode_greedy(toks[-1], args.steps)
    if rank == 0:
        print(json.dumps({"profile_case": True, "layers": args.profile_case, "batch": batch, "gpus": world, "context": ctx, "steps": args.steps,
                          "ms_per_step": ms / args.steps, "launches_per_step": eng.launches_per_step(), "note": "not a bench value"}), flush=True)
    if args.timeline:
        # the step as the CUDA graph runs it: per launch, microseconds on the device global timer relative to the
        # first launch, and block 0's own progress (SM cycle counter at the sampled clock) at its points 1..7
        names = {1: "k_tcgemv", 3: "k_delta_step", 5: "k_moe_gu1", 6: "k_moe_down1", 7: "k_attn(_mma)", 8: "k_attn_merge", 9: "k_prep_x",
                 10: "k_mma_i8", 11: "k_group_picks", 12: "k_mma_q4", 13: "k_ep_combine", 14: "k_umma", 15: "k_prep_q", 16: "k_umma_q4",
                 17: "k_prep_q_slots", 18: "k_ep_push_records", 19: "k_ep_push_outputs", 20: "k_ep_wait"}
        eng.trace_step()                     # every rank steps (the exchange is collective); rank 0 prints its own timeline
        t = eng.trace_step().astype(np.int64)
        ghz = args.timeline_ghz
        live = t[t[:, 5] > 0] if rank == 0 else t[:0]
        t0 = live[:, 0].min() if len(live) else 0
        prev = None
        if rank == 0:
            print("kernel hint | first block in, last block in, last block out | since previous kernel's end (includes NCCL's kernels, "
                  "which do not stamp) | block 0: us after it came in, at points 1..7")
        for r in live:
            s, li, e = (r[0] - t0) / 1e3, (r[7] - t0) / 1e3, (r[4] - t0) / 1e3
            pts = " ".join(f"{(r[8 + j] - r[8]) / ghz / 1e3:6.2f}" if r[8 + j] > 0 else "     -" for j in range(1, 8))
            print(f"{names.get(int(r[5]), '?'):13s} {int(r[6]):6d} | {s:7.2f} {li:7.2f} {e:7.2f} | {e - (prev if prev is not None else s):6.2f} | {pts}")
            prev = e
    if world > 1:
        eng.close()
        dist.destroy_process_group()


def b64_measure(pkg, K: int, W: int, world: int, rank: int, local: int, dist, peer_stores: bool = True):
    """Batched decode of 64 sequences at context 8192 with Zipf(1.1) expert popularity, expert-parallel over `world`
    ranks (256/world experts of every layer per GPU, the routed tokens exchanged by NCCL). Returns rank 0's line."""
    import hashlib
    import torch
    from b200moe import brain, ep
    from b200moe import engine as E
    cfg = pkg.HybridConfig.full()
    Bt = 64
    B = Bt // world
    fed = 16
    cap = B64_PROMPT + W + 2 * K + 64
    t0 = time.perf_counter()
    eng = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device=f"cuda:{local}"),
                                      max_context=cap, device=local, batch=B, kv_dtype=E.KV_BF16, ep_rank=rank, ep_world=world)
    torch.cuda.empty_cache()
    exchange = ep.attach(eng, rank, world, peer_stores=peer_stores) if world > 1 else "none"
    for layer in range(cfg.n_layers):
        eng.set_router_bias(layer, brain.router_popularity_bias(cfg, layer, 0, 1.1).numpy())
    t_build = time.perf_counter() - t0
    # context: feeding 64 x 8192 tokens through the decode path would take minutes, so the length is set directly and
    # only the last `fed` prompt tokens are real; the bytes read per step are those of a real prompt
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

    toks_w, _ = eng.decode_greedy(prompt[:, -1], W)
    barrier()
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    toks, ms = eng.decode_greedy(toks_w[-1], K)
    barrier()
    clk = clocks.stop()
    bytes_step = eng.step_bytes()
    # picks per rank in the last step, all layers
    picks = np.stack([eng.router(layer, cfg.experts_active)[0] for layer in range(cfg.n_layers)])
    all_toks = np.concatenate([toks_w, toks], 0)                      # [W + K][B] greedy tokens of this rank's sequences
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        allp, allt = [None] * world, [None] * world
        dist.all_gather_object(allp, picks)
        dist.all_gather_object(allt, all_toks)
        picks = np.concatenate(allp, 1)
        all_toks = np.concatenate(allt, 1)
    # the same sums in the same order on every number of GPUs: this hash must not depend on N. It covers the first
    # greedy steps only, so that runs with different --steps / --warmup can be compared too
    n_hashed = min(8, all_toks.shape[0])
    tokens_sha1 = hashlib.sha1(np.ascontiguousarray(all_toks[:n_hashed].astype("<u4")).tobytes()).hexdigest()
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
    n_launch = eng.launches_per_step()
    nvlink = eng.ep_bytes_per_step() if world > 1 else 0
    eng.close()
    torch.cuda.empty_cache()
    peak, peak_kind = peaks()
    step_gbs = bytes_step / (ms / K * 1e-3) / 1e9
    return {"metric": METRIC_B64, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "full-b64: the 40-layer 35B-A3B-shaped model, 64 sequences at context 8192, greedy decode, "
                                   "router bias for Zipf(1.1) expert popularity",
                       "batch": Bt, "sequences_per_gpu": B, "context": B64_PROMPT,
                       "context_note": f"length set to {B64_PROMPT - fed} directly, then {fed} real tokens fed",
                       "kv_cache": "bf16", "parallelism": f"ep{world}: {cfg.n_experts // world} experts of every layer per GPU, "
                                                          "sequences split over the GPUs, per layer the records of all sequences to every GPU and the "
                                                          "pick outputs back to their owners, by " + {"peer-stores": "plain peer stores over NVLink with bounded flag waits (rows of owned picks only)", "nccl": "NCCL all-gather + grouped send/recv (dense blocks)", "none": "no exchange (one GPU)"}[exchange],
                       "exchange": exchange,
                       "l2": "per-step traffic exceeds L2 (126 MB); no flush needed"},
            "e2e": {"value": Bt * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                    "timing": "host wall clock around K feed_batch() calls (ids in, arg-max out), max over ranks"},
            "gpu_launches": n_launch * K,
            "tokens_sha1": tokens_sha1, "tokens_hashed": f"first {n_hashed} greedy steps of all {Bt} sequences", "nvlink_bytes_per_step_per_gpu": nvlink,
            "roofline": {"bound": "hbm", "kernel": "whole step, per GPU", "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                         "frac": step_gbs / peak, "peak_kind": peak_kind, "traffic": None,
                         "bytes_per_step_per_gpu": bytes_step},
            "expert_load": {"picks_per_rank": load.tolist(), "max_over_mean": float(load.max() / load.mean()),
                            "unique_experts_per_layer": uniq},
            "cpu_baseline": None, "clocks": clk, "setup": {"build_s": round(t_build, 1)}}


def run_b64(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = b64_measure(pkg, args.steps, max(args.warmup, 3), world, rank, local, dist, peer_stores=not args.nccl_exchange)
    if rank == 0:
        print(json.dumps(line, default=lambda o: o.item() if hasattr(o, 'item') else str(o)), flush=True)
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

    # per-role times for the roofline object: the device-side timeline of a graph-run step (what the timed loop above
    # executes; device global timer, from the end of the previous launch to the end of this one), and as a side key
    # CUDA events around every launch of un-graphed steps (which include the host's launch gaps)
    prof = eng.profile_step(8)
    peak, peak_kind = peaks()
    in_graph = graph_timeline(eng, prof)
    roles = {n: v for n, v in in_graph.items() if n in prof and prof[n]["launches"] and v["us_per_step"] > 0}
    name = max(roles, key=lambda n: roles[n]["us_per_step"])
    dom, dom_us = prof[name], roles[name]["us_per_step"]
    achieved = dom["bytes"] / (dom_us * 1e-6) / 1e9
    step_gbs = bytes_step / (ms / K * 1e-3) / 1e9
    roles_sum_ms = sum(v["us_per_step"] for v in in_graph.values()) / 1e3
    consistent = bool(abs(roles_sum_ms - ms / K) <= 0.10 * (ms / K))
    if not consistent:
        print(f"warning: the roles' in-graph times sum to {roles_sum_ms:.3f} ms, the timed step is {ms / K:.3f} ms", file=sys.stderr)
    roof = {"bound": "hbm", "kernel": f"{name} ({E.HybridEngine.KERNELS_SMALL_BATCH[name]})", "achieved": achieved, "peak": peak,
            "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
            "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(name), "traffic_source": NCU_DRAM_SOURCE,
            "launches_per_step": dom["launches"], "bytes_per_launch": dom["bytes"] / max(dom["launches"], 1),
            "ms_per_launch": dom_us / 1e3 / max(dom["launches"], 1),
            "timing": "device global timer inside the CUDA graph of one decode step (b2_debug_trace_step); "
                      "ungraphed_events = CUDA events around each launch of 8 un-graphed steps",
            "whole_step": {"bytes": bytes_step, "achieved": step_gbs, "frac": step_gbs / peak},
            "in_graph": in_graph,
            "consistency": {"roles_sum_ms": round(roles_sum_ms, 4), "ms_per_step": round(ms / K, 4), "within_10_percent": consistent},
            "ungraphed_events": {n: {"ms_per_step": round(v["ms"], 4), "GBps": round(v["bytes"] / max(v["ms"], 1e-9) / 1e6, 1),
                                     "launches": v["launches"], "kernel": E.HybridEngine.KERNELS_SMALL_BATCH[n]} for n, v in prof.items()}}
    cb = parity = b64 = None
    n_launch = eng.launches_per_step()
    eng.close()
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_b64:
        # the single-GPU point of the expert-parallel series (the lines of --gpus 2/4/8 carry the other points)
        full = b64_measure(pkg, min(K, 64), 3, 1, 0, local, None)
        b64 = {k: full[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "tokens_sha1", "tokens_hashed", "roofline", "expert_load", "e2e", "config")}
    if rank == 0 and world == 1 and not args.no_cpu:
        cfg4, dev, host = sample_brain(f"cuda:{local}")
        parity, model = parity_check(E, cfg4, dev, host)
        del dev
        torch.cuda.empty_cache()
        cb = cpu_sample(cfg, cfg4, host, model, 3, 1)
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_config(cfg),
                "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": cfg.vocab_size * 4,
                        "timing": "host wall clock around K feed() calls (id and logits in page-locked host arrays, b2_sample arg-max on the host), synchronised on both sides"},
                "gpu_launches": n_launch * K,
                "roofline": roof, "cpu_baseline": cb, "parity": parity, "b64": b64, "clocks": clk,
                "setup": {"build_s": round(t_build, 1), "prefill_s": round(t_prefill, 1),
                          "prefill": "prompt fed through the engine's feed(), untimed"}}
        if world > 1:
            line["config"]["parallelism"] = f"{world} independent replicas (batch-1 decode does not shard)"
        print(json.dumps(line, default=lambda o: o.item() if hasattr(o, 'item') else str(o)), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the parity check and the CPU baseline leg")
    ap.add_argument("--no-b64", action="store_true", help="one GPU: skip the batch-64 point of the expert-parallel series")
    ap.add_argument("--workload", default="auto", choices=["auto", "b1", "b64"],
                    help="b1: batch-1 decode (the default on one GPU); b64: 64 sequences, expert-parallel (the default on several)")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="several GPUs: keep the per-layer expert exchange on NCCL calls (default: plain peer stores with bounded flag waits)")
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
