"""The allocation-free MoE layer entry point (b2_moe_forward_static) against the ordinary one.

Who needs it: a host that cannot call cudaMalloc while the model runs - its own arena already holds
the GPU's free memory, or it only ever receives device pointers from the runtime it is embedded in.
Such a caller passes device pointers for weights, inputs and outputs (torch tensors stand in for its
arena here) and the library works in a fixed array of its own instead of allocating.

Two calls in a row on different inputs must each equal b2_moe_forward exactly: the second call finds
the first call's leftovers in the shared work memory and has to clear what matters. This file is
named to be collected last, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def test_static_work_memory_matches_the_allocating_operator(pkg):
    import importlib
    E = importlib.import_module("b200moe.engine")
    from b200moe import brain
    lib = E.load_library()
    cfg = pkg.HybridConfig.tiny()
    cfg.n_layers, cfg.layer_types = 1, ["delta"]
    raw = {}
    for n, dt, x in brain.random_brain(cfg, seed=3):
        if ".moe." in n:
            raw[n.split(".moe.")[1]] = bits(x) if dt == "bf16" else x.numpy()
    ref = E.MoeLayer(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden,
                     raw["router.weight"], raw["experts.q4"],
                     (raw["shared.gate.qweight"], raw["shared.gate.scale"]), (raw["shared.up.qweight"], raw["shared.up.scale"]),
                     (raw["shared.down.qweight"], raw["shared.down.scale"]), raw["shared_gate.weight"], max_tokens=8)

    # the caller's own device memory: weights, an address table of the experts, inputs and outputs
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).cuda()
    d = {k: dev(v) for k, v in raw.items()}
    eb = cfg.expert_bytes
    table = torch.tensor([d["experts.q4"].data_ptr() + e * eb for e in range(cfg.n_experts)], dtype=torch.int64).cuda()
    w = E.MoeDeviceWeights(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden,
                           d["router.weight"].data_ptr(), table.data_ptr(),
                           d["shared.gate.qweight"].data_ptr(), d["shared.gate.scale"].data_ptr(),
                           d["shared.up.qweight"].data_ptr(), d["shared.up.scale"].data_ptr(),
                           d["shared.down.qweight"].data_ptr(), d["shared.down.scale"].data_ptr(),
                           d["shared_gate.weight"].data_ptr())
    g = torch.Generator().manual_seed(9)
    for tokens in (5, 8, 1):                                  # consecutive calls share the work memory
        h = torch.randn(tokens, cfg.d_model, generator=g)
        want_y, want_idx, want_w, _ = ref.forward(h.numpy())
        hd = h.cuda()
        y = torch.full((tokens, cfg.d_model), 7.0, device="cuda")        # stale contents must not leak into the result
        idx = torch.zeros(tokens, cfg.experts_active, dtype=torch.int32, device="cuda")
        wt = torch.zeros(tokens, cfg.experts_active, device="cuda")
        torch.cuda.synchronize()
        rc = lib.b2_moe_forward_static(C.byref(w), hd.data_ptr(), tokens, y.data_ptr(), idx.data_ptr(), wt.data_ptr(), None)
        assert rc == 0
        assert np.array_equal(idx.cpu().numpy(), want_idx)
        assert np.abs(wt.cpu().numpy() - want_w).max() < 1e-6
        assert np.abs(y.cpu().numpy() - want_y).max() < 2e-5 * max(1.0, np.abs(want_y).max())
    # beyond the fixed maximum: refused, nothing runs
    h9 = torch.zeros(9, cfg.d_model, device="cuda")
    y9 = torch.zeros(9, cfg.d_model, device="cuda")
    assert lib.b2_moe_forward_static(C.byref(w), h9.data_ptr(), 9, y9.data_ptr(), None, None, None) == 2
    ref.close()


def test_static_entry_at_its_documented_maximum_against_the_oracle(pkg):
    """8 tokens at d_model 2048, 256 experts top-8, hidden 512: every offset inside the fixed work array is at its
    limit. Checked against the CPU oracle's MoE layer (router picks identical and in order), on a stream of the
    caller's own, twice in a row; then the argument checks: a misaligned or null weight pointer is an error code."""
    import importlib
    from oracle import hybrid_oracle as O
    E = importlib.import_module("b200moe.engine")
    from b200moe import brain
    lib = E.load_library()
    cfg = pkg.HybridConfig.full(n_layers=1)
    raw, host = {}, {}
    for n, dt, x in brain.random_brain(cfg, seed=0, device="cuda:0"):
        if ".moe." in n:
            c = x.detach().contiguous().cpu()
            host[n] = (dt, bits(c) if dt == "bf16" else c.numpy())
            raw[n.split(".moe.")[1]] = x.contiguous().view(torch.uint8).reshape(-1)
    oracle = O.HybridOracle(O.DictBrain(cfg.to_dict(), host), hold_weights=True)
    eb = cfg.expert_bytes
    table = torch.tensor([raw["experts.q4"].data_ptr() + e * eb for e in range(cfg.n_experts)], dtype=torch.int64).cuda()
    args = [raw["router.weight"].data_ptr(), table.data_ptr(),
            raw["shared.gate.qweight"].data_ptr(), raw["shared.gate.scale"].data_ptr(),
            raw["shared.up.qweight"].data_ptr(), raw["shared.up.scale"].data_ptr(),
            raw["shared.down.qweight"].data_ptr(), raw["shared.down.scale"].data_ptr(),
            raw["shared_gate.weight"].data_ptr()]
    w = E.MoeDeviceWeights(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden, *args)
    stream = torch.cuda.Stream()
    g = torch.Generator().manual_seed(21)
    for tokens in (8, 8, 3):
        h = torch.randn(tokens, cfg.d_model, generator=g).to(torch.bfloat16).float()
        want = oracle.moe(0, h.numpy())
        widx, ww = oracle.last_route[0]
        hd = h.cuda()
        y = torch.full((tokens, cfg.d_model), -3.0, device="cuda")
        idx = torch.zeros(tokens, cfg.experts_active, dtype=torch.int32, device="cuda")
        wt = torch.zeros(tokens, cfg.experts_active, device="cuda")
        torch.cuda.synchronize()
        rc = lib.b2_moe_forward_static(C.byref(w), hd.data_ptr(), tokens, y.data_ptr(), idx.data_ptr(), wt.data_ptr(),
                                       C.c_void_p(stream.cuda_stream))
        assert rc == 0
        assert np.array_equal(idx.cpu().numpy(), widx)
        assert np.abs(wt.cpu().numpy() - ww).max() < 1e-6
        assert np.abs(y.cpu().numpy() - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    # argument checks: nothing runs, an error code comes back
    hd = torch.zeros(1, cfg.d_model, device="cuda")
    y = torch.zeros(1, cfg.d_model, device="cuda")
    bad = list(args)
    bad[2] += 4                                                # shared gate weights off a 16-byte boundary
    wb = E.MoeDeviceWeights(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden, *bad)
    assert lib.b2_moe_forward_static(C.byref(wb), hd.data_ptr(), 1, y.data_ptr(), None, None, None) == 3
    bad = list(args)
    bad[0] = 0                                                 # no router
    wb = E.MoeDeviceWeights(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden, *bad)
    assert lib.b2_moe_forward_static(C.byref(wb), hd.data_ptr(), 1, y.data_ptr(), None, None, None) == 3
    # a table entry that is null is reported by the kernels' error word, not by a fault
    table2 = table.clone()
    table2[:] = 0
    bad = list(args)
    bad[1] = table2.data_ptr()
    wb = E.MoeDeviceWeights(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden, *bad)
    assert lib.b2_moe_forward_static(C.byref(wb), hd.data_ptr(), 1, y.data_ptr(), None, None, None) == 4
