"""The expert-parallel exchange protocol with two CPU ranks (gloo): both ranks together must give
exactly what one rank gives, and what the oracle's MoE layer gives to rounding."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import hybrid_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _layer_fns(micro_path, layer):
    brain = O.Brain(micro_path)
    model = O.HybridOracle(brain)
    cfg = model.cfg
    p = f"blocks.{layer}.moe."
    masters = brain.raw(p + "experts.q4")
    I = cfg["expert_hidden"]

    def expert_fn(e, rows):
        gu, dn = O.unpack_expert(masters[e], cfg)
        a = rows.numpy() @ gu.T
        return torch.from_numpy(((O.silu(a[:, :I]) * a[:, I:]).astype(np.float32) @ dn.T).astype(np.float32))

    def shared_fn(x):
        h = x.numpy()
        sh = model.qlinear((O.silu(model.qlinear(h, p + "shared.gate")) * model.qlinear(h, p + "shared.up")).astype(np.float32),
                           p + "shared.down")
        sg = O.sigmoid((h @ brain.f32(p + "shared_gate.weight").T).astype(np.float32))
        return torch.from_numpy((sg * sh).astype(np.float32))

    def route(h):
        logits = (h.numpy() @ brain.f32(p + "router.weight").T).astype(np.float32)
        idx, w, _ = O.route(logits, cfg["experts_active"])
        return torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(w)

    return model, cfg, expert_fn, shared_fn, route


def _worker(rank, world, port, micro_path, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from b200moe import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model, cfg, expert_fn, shared_fn, route = _layer_fns(micro_path, 1)
    g = torch.Generator().manual_seed(7)
    h_all = torch.randn(6, cfg["d_model"], generator=g)
    B = 6 // world
    h = h_all[rank * B:(rank + 1) * B].contiguous()
    idx, w = route(h)
    out = ep.exchange_moe(h, idx, w, expert_fn, shared_fn, cfg["n_experts"], rank, world)
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_rank_and_the_oracle(pkg, micro_path, tmp_path):
    from b200moe import ep
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, micro_path, str(tmp_path)), nprocs=2, join=True)
    two = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(2)])
    model, cfg, expert_fn, shared_fn, route = _layer_fns(micro_path, 1)
    h_all = torch.randn(6, cfg["d_model"], generator=torch.Generator().manual_seed(7))
    idx, w = route(h_all)
    one = ep.exchange_moe(h_all, idx, w, expert_fn, shared_fn, cfg["n_experts"], 0, 1).numpy()
    assert np.array_equal(two, one)                       # same sums in the same order
    want = h_all.numpy() + model.moe(1, h_all.numpy())
    assert np.abs(one - want).max() < 1e-5


def test_ownership_and_load(pkg):
    from b200moe import ep
    assert [ep.expert_owner(e, 256, 8) for e in (0, 31, 32, 255)] == [0, 0, 1, 7]
    picks = np.array([[0, 1, 100, 255], [33, 34, 35, 36]])
    assert ep.load_per_rank(picks, 256, 8).tolist() == [2, 4, 0, 1, 0, 0, 0, 1]
    assert ep.load_per_rank(picks, 256, 1).tolist() == [8]


class _FakeEngine:
    """Stands in for HybridEngine in ep.attach: records the calls, fails where told to."""

    def __init__(self, rank, fail_handle=False, fail_attach=False):
        self.rank, self.fail_handle, self.fail_attach, self.calls = rank, fail_handle, fail_attach, []

    def ep_unique_id(self):
        return b"\x07" * 128

    def ep_init(self, uid):
        assert uid == b"\x07" * 128
        self.calls.append("init")

    def ep_ipc_handle(self):
        if self.fail_handle:
            raise RuntimeError("cudaIpcGetMemHandle: not supported")
        return bytes([self.rank]) * 64

    def ep_ipc_attach(self, handles):
        assert [h[0] for h in handles] == list(range(len(handles)))      # every rank's handle, in rank order
        if self.fail_attach:
            raise RuntimeError("cudaIpcOpenMemHandle: peer access is not available")
        self.calls.append("attach")


def _attach_worker(rank, world, port, case, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from b200moe import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    e = _FakeEngine(rank, fail_handle=(case == "no-handle" and rank == 1), fail_attach=(case == "no-attach" and rank == 1))
    try:
        how = ep.attach(e, rank, world, peer_stores=(case != "off"))
    except RuntimeError as err:
        how = "raised: " + str(err)[:40]
    with open(os.path.join(out_dir, f"attach{rank}.txt"), "w") as f:
        f.write(how + "|" + ",".join(e.calls))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case,want", [("ok", ["peer-stores|init,attach"] * 2), ("off", ["nccl|init"] * 2),
                                       ("no-handle", ["nccl|init"] * 2),
                                       ("no-attach", ["raised: this rank mapped its peers but another r|init,attach", "nccl|init"])])
def test_attach_agrees_on_the_exchange(tmp_path, case, want):
    """ep.attach: all ranks end on the same exchange. A rank without a handle keeps everyone on NCCL before anything is
    mapped; a rank that cannot map a peer after the others did makes the others raise instead of running mixed."""
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_attach_worker, args=(2, port, case, str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"attach{r}.txt").read_text() for r in range(2)] == want
