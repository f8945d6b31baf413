"""Expert-parallel decode over the GPUs of one node: host-side plumbing and the exchange protocol.

One process per GPU. Sequences are split over the ranks (each rank runs the mixers, router, shared
expert and head of its own `batch` sequences); the experts of every layer are split too: expert `e`
lives on rank `e // (n_experts // world)`. Per layer the ranks exchange twice:

  1. all-gather of one record per sequence: residual-stream row | router picks | router weights;
  2. every rank runs the picks that hit its experts, for all sequences, into ypart[token][rank-of-pick];
  3. all-to-all: block p of ypart (the sequences of rank p) goes to rank p;
  4. the owner of a sequence adds its picks in pick order, each taken from the block of the rank that
     owns that pick's expert, then the shared expert: the same sums in the same order as on one GPU.

On the GPU the exchange is NCCL inside the engine's CUDA graph (csrc/engine.cu). `attach` only hands
the NCCL id from rank 0 to the others through torch.distributed. `exchange_moe` is the same protocol
written with torch.distributed collectives on CPU tensors: it documents the data movement and lets
the multi-rank logic be checked with the gloo backend.

The reference engine is single-GPU (aegist_rs/src/hybrid.rs:511-514); nothing here has a counterpart there.
"""
from __future__ import annotations

import numpy as np


def expert_owner(expert: int, n_experts: int, world: int) -> int:
    return int(expert) // (n_experts // world)


def attach(engine, rank: int, world: int, peer_stores: bool = True) -> str:
    """Create the engine's NCCL communicator: rank 0 makes the id, everyone receives it through the
    default torch.distributed group, then all ranks initialise together. With `peer_stores` the ranks
    then map each other's exchange blocks and the per-layer exchange runs on plain peer stores with
    bounded flag waits instead of NCCL calls; if any rank cannot map a peer (no peer access between
    the GPUs, IPC closed in the container), all ranks stay on NCCL. Returns "peer-stores" or "nccl"."""
    import torch.distributed as dist
    box = [engine.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    engine.ep_init(box[0])
    if not peer_stores:
        return "nccl"
    try:
        mine = engine.ep_ipc_handle()
    except Exception:
        mine = None
    handles = [None] * world
    dist.all_gather_object(handles, mine)
    ok = all(h is not None for h in handles)
    if ok:
        try:
            engine.ep_ipc_attach(handles)
        except Exception:
            ok = False
    votes = [None] * world
    dist.all_gather_object(votes, ok)
    if all(votes):
        return "peer-stores"
    if ok:
        raise RuntimeError("this rank mapped its peers but another rank could not: rebuild the engines with peer_stores=False")
    return "nccl"


def load_per_rank(picks: np.ndarray, n_experts: int, world: int) -> np.ndarray:
    """How many picks land on each rank; `picks` is any array of expert ids."""
    own = np.asarray(picks).reshape(-1) // (n_experts // world)
    return np.bincount(own, minlength=world)


def exchange_moe(x, idx, w, expert_fn, shared_fn, n_experts: int, rank: int, world: int, group=None):
    """One layer's expert-parallel MoE on CPU tensors, step for step as the GPU path does it.

    x [B, D] float32, idx [B, k] int64, w [B, k] float32 are this rank's sequences;
    `expert_fn(e, rows [n, D]) -> [n, D]` evaluates local expert e; `shared_fn(x) -> [B, D]` is the
    gated shared expert of the local sequences. Returns x + moe(x) for the local sequences."""
    import torch
    import torch.distributed as dist
    B, D = x.shape
    k = idx.shape[1]
    per = n_experts // world
    # 1. records
    rec = torch.cat([x, idx.to(torch.float32), w], 1).contiguous()
    all_rec = [torch.empty_like(rec) for _ in range(world)]
    if world > 1:
        dist.all_gather(all_rec, rec, group=group)
    else:
        all_rec = [rec]
    all_rec = torch.cat(all_rec, 0)                                   # [world * B, D + 2k]
    gx, gidx = all_rec[:, :D], all_rec[:, D:D + k].to(torch.int64)
    # 2. local experts on every sequence's picks
    ypart = torch.zeros(world * B, k + 1, D)
    for t in range(world * B):
        for r in range(k):
            e = int(gidx[t, r])
            if e // per == rank:
                ypart[t, r] = expert_fn(e, gx[t:t + 1])[0]
    ypart[rank * B:(rank + 1) * B, k] = shared_fn(x)
    # 3. all-to-all of the blocks
    send = [ypart[p * B:(p + 1) * B].contiguous() for p in range(world)]
    recv = [torch.empty_like(send[0]) for _ in range(world)]
    if world > 1:
        dist.all_to_all(recv, send, group=group) if dist.get_backend(group) != "gloo" else _gloo_all_to_all(recv, send, rank, world, group)
    else:
        recv = send
    # 4. combine in pick order, then the shared expert
    out = x.clone()
    for b in range(B):
        y = torch.zeros(D)
        for r in range(k):
            owner = int(idx[b, r]) // per
            y = y + w[b, r] * recv[owner][b, r]
        y = y + recv[rank][b, k]
        out[b] = out[b] + y
    return out


def _gloo_all_to_all(recv, send, rank, world, group):
    """gloo has no all_to_all: pairwise send/recv in a fixed order."""
    import torch.distributed as dist
    recv[rank].copy_(send[rank])
    for step in range(1, world):
        dst, src = (rank + step) % world, (rank - step) % world
        if rank < dst:
            dist.send(send[dst], dst, group=group)
            dist.recv(recv[src], src, group=group)
        else:
            dist.recv(recv[src], src, group=group)
            dist.send(send[dst], dst, group=group)
