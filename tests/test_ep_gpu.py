"""Expert-parallel decode on two GPUs through the C ABI, with the exchange on plain peer stores and on NCCL:
identical to the single-GPU engine and within tolerance of the reference's stored batch rows. Skipped with fewer
than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tensors(micro_path):
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from b200moe.nxfile import NxFile
    nx = NxFile(micro_path)
    return nx, [(n, nx.info(n)["dtype"], np.array(nx.tensor(n))) for n in nx.header["tensors"]]


def _worker(rank, world, port, micro_path, ids, steps, out_dir, peer_stores):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    nx, tensors = _tensors(micro_path)
    from b200moe import engine as E
    from b200moe import ep
    B = ids.shape[0] // world
    e = E.HybridEngine.from_tensors(nx.config, tensors, max_context=32, device=rank, batch=B, kv_dtype=E.KV_F32,
                                    ep_rank=rank, ep_world=world)
    how = ep.attach(e, rank, world, peer_stores=peer_stores)
    assert how == ("peer-stores" if peer_stores else "nccl"), how
    mine = ids[rank * B:(rank + 1) * B]
    rows = []
    for t in range(mine.shape[1]):
        nxt, lg = e.feed_batch(mine[:, t])
        rows.append(lg)
    for _ in range(steps):
        nxt, lg = e.feed_batch(rows[-1].argmax(-1))
        rows.append(lg)
    np.save(os.path.join(out_dir, f"rows{rank}.npy"), np.stack(rows))
    assert (e.ep_bytes_per_step() > 0)
    e.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer_stores", [True, False])
def test_two_gpus_equal_one_gpu(pkg, micro_path, golden_dir, tmp_path, peer_stores):
    import torch.multiprocessing as mp
    from b200moe import engine as E
    g = np.load(os.path.join(golden_dir, "micro_golden.npz"))
    ids = g["batch_prompt"]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, micro_path, ids, 8, str(tmp_path), peer_stores), nprocs=2, join=True)
    two = np.concatenate([np.load(tmp_path / f"rows{r}.npy") for r in range(2)], 1)      # [T, 4, V]
    e = E.HybridEngine.load(micro_path, max_context=32, batch=4)
    rows = []
    for t in range(ids.shape[1]):
        rows.append(e.feed_batch(ids[:, t])[1])
    for _ in range(8):
        rows.append(e.feed_batch(rows[-1].argmax(-1))[1])
    one = np.stack(rows)
    e.close()
    assert np.array_equal(two, one)                          # same sums in the same order
    assert np.abs(two - g["batch_logits"]).max() < 3e-4       # and the reference's rows


def _worker_absent(rank, world, port, micro_path, ids, out_dir):
    """Both ranks take three steps together; then rank 1 stays away and rank 0 steps alone."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    nx, tensors = _tensors(micro_path)
    from b200moe import engine as E
    from b200moe import ep
    B = ids.shape[0] // world
    e = E.HybridEngine.from_tensors(nx.config, tensors, max_context=32, device=rank, batch=B, kv_dtype=E.KV_F32,
                                    ep_rank=rank, ep_world=world)
    assert ep.attach(e, rank, world, peer_stores=True) == "peer-stores"
    mine = ids[rank * B:(rank + 1) * B]
    for t in range(3):
        e.feed_batch(mine[:, t])
    torch.cuda.synchronize()
    dist.barrier()                      # nothing of either rank is in flight from here on
    msg = ""
    if rank == 0:
        try:
            e.feed_batch(mine[:, 3])
        except E.EngineError as err:
            msg = str(err)
        with open(os.path.join(out_dir, "absent.txt"), "w") as f:
            f.write(msg)
    dist.barrier()                      # rank 1 keeps its block mapped until rank 0 has given up
    e.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_absent_rank_ends_the_step_with_an_error(pkg, micro_path, golden_dir, tmp_path):
    """A rank that does not take part (it left between steps, on the host): the other rank's bounded flag waits run out,
    its kernels end normally and the step returns an error that names the exchange; nothing hangs."""
    import torch.multiprocessing as mp
    g = np.load(os.path.join(golden_dir, "micro_golden.npz"))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker_absent, args=(2, port, micro_path, g["batch_prompt"], str(tmp_path)), nprocs=2, join=True)
    assert "did not arrive" in (tmp_path / "absent.txt").read_text()


def _worker_full(rank, world, port, out_dir, steps):
    """Four full-width layers (hidden 2048, 256 experts, expert hidden 512): the tcgen05 GEMMs and the grouped 4-bit
    expert GEMM over this rank's half of the experts, exchange on peer stores."""
    import sys
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    pkg = load_package()
    from b200moe import brain, ep
    from b200moe import engine as E
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg = pkg.HybridConfig.full(n_layers=4)
    B = 16 // world
    e = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device=f"cuda:{rank}"), max_context=64,
                                    device=rank, batch=B, kv_dtype=E.KV_BF16, ep_rank=rank, ep_world=world)
    assert ep.attach(e, rank, world) == "peer-stores"
    first = np.arange(100, 116, dtype=np.uint32)[rank * B:(rank + 1) * B]
    toks, _ = e.decode_greedy(first, steps)
    nxt, logits = e.feed_batch(toks[-1])
    np.save(os.path.join(out_dir, f"full{rank}.npy"), logits)
    np.save(os.path.join(out_dir, f"toks{rank}.npy"), toks)
    e.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_equal_one_gpu_at_full_width(pkg, tmp_path):
    """The benchmark's expert-parallel kernels at the benchmark's widths: 16 sequences on two GPUs give bit for bit the
    tokens and logits of 16 sequences on one GPU."""
    import torch.multiprocessing as mp
    from b200moe import brain
    from b200moe import engine as E
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker_full, args=(2, port, str(tmp_path), 6), nprocs=2, join=True)
    two_t = np.concatenate([np.load(tmp_path / f"toks{r}.npy") for r in range(2)], 1)
    two_l = np.concatenate([np.load(tmp_path / f"full{r}.npy") for r in range(2)], 0)
    cfg = pkg.HybridConfig.full(n_layers=4)
    e = E.HybridEngine.from_tensors(cfg.to_dict(), brain.random_brain(cfg, seed=0, device="cuda:0"), max_context=64, device=0,
                                    batch=16, kv_dtype=E.KV_BF16)
    toks, _ = e.decode_greedy(np.arange(100, 116, dtype=np.uint32), 6)
    nxt, logits = e.feed_batch(toks[-1])
    e.close()
    assert np.array_equal(two_t, toks)
    assert np.array_equal(two_l, logits)
