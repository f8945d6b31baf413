"""Single operators through the C ABI against the CPU oracle at the benchmark spec's op shapes."""
import os

import numpy as np
import pytest
import torch

from oracle import hybrid_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E(pkg):
    import importlib
    eng = importlib.import_module("b200moe.engine")
    eng.load_library()
    return eng


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("n,k,tokens", [(64, 128, 3), (1000, 2048, 1), (515, 4096, 2), (33, 64, 1), (256, 512, 5)])
def test_int8_linear(E, pkg, n, k, tokens):
    from b200moe import brain
    g = torch.Generator().manual_seed(n + k)
    q, s = brain.int8_quantize((torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16))
    x = torch.randn(tokens, k, generator=g).numpy()
    y = E.linear_i8(q.numpy(), bits(s), x)
    want = x @ (q.numpy().astype(np.float32) * O.bf16_to_f32(bits(s))).T
    assert np.abs(y - want).max() < 2e-5 * max(1.0, np.abs(want).max())


def test_int8_linear_against_reference_vector(E, golden_dir):
    ops = np.load(os.path.join(golden_dir, "ops_golden.npz"))
    y = E.linear_i8(ops["i8_q"], ops["i8_scale"], ops["i8_x"])
    assert np.abs(y - ops["i8_y"]).max() < 1e-5


@pytest.fixture(scope="module")
def moe_layer(pkg):
    """hidden 2048, 256 experts + shared, intermediate 512, N(0, 0.02) bf16 weights, seed 0."""
    from b200moe import brain
    cfg = pkg.HybridConfig.full(n_layers=1)
    t = {n: (dt, x) for n, dt, x in brain.random_brain(cfg, seed=0) if ".moe." in n}
    raw = {n: (dt, bits(x) if dt == "bf16" else x.numpy()) for n, (dt, x) in t.items()}
    return cfg, raw


@pytest.mark.parametrize("tokens", [1, 8, 64])
def test_moe_layer_op(E, moe_layer, tokens):
    cfg, raw = moe_layer
    p = "blocks.0.moe."
    layer = E.MoeLayer(cfg.d_model, cfg.n_experts, cfg.experts_active, cfg.expert_hidden, cfg.shared_hidden,
                       raw[p + "router.weight"][1], raw[p + "experts.q4"][1],
                       (raw[p + "shared.gate.qweight"][1], raw[p + "shared.gate.scale"][1]),
                       (raw[p + "shared.up.qweight"][1], raw[p + "shared.up.scale"][1]),
                       (raw[p + "shared.down.qweight"][1], raw[p + "shared.down.scale"][1]),
                       raw[p + "shared_gate.weight"][1])
    h = torch.randn(tokens, cfg.d_model, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).float().numpy()
    y, idx, w, ms = layer.forward(h)
    oracle = O.HybridOracle(O.DictBrain({**cfg.to_dict()}, raw), hold_weights=True)
    want = oracle.moe(0, h)
    widx, ww = oracle.last_route[0]
    assert (idx == widx).all()                      # top-8 picks bit-exact, in order
    assert np.abs(w - ww).max() < 1e-6
    assert np.abs(y - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    y2, idx2, _, _ = layer.forward(h)               # run-to-run identical
    assert np.array_equal(y, y2) and np.array_equal(idx, idx2)
    layer.close()


def test_bounded_wait_gives_up_with_an_error_code(E):
    """Every wait on a bulk copy is bounded. A kernel whose barrier expects bytes that no copy delivers must end
    by itself with error word 3 (never a hang), here after 20,000 polls."""
    import ctypes as C
    lib = E.load_library()
    status = C.c_int(-1)
    assert lib.b2_debug_wait_timeout(0, 20000, C.byref(status)) == 0
    assert status.value == 3


@pytest.mark.parametrize("batch,steps", [(1, 1000), (16, 120), (64, 30)])
def test_delta_rule_steps(E, batch, steps):
    """hidden 2048-shaped DeltaNet state: 32 value heads, 128 x 128, fp32 state from N(0, 0.1), bf16
    inputs from N(0, 1), beta = sigmoid(N(0,1)) and decay = sigmoid(N(0,1)); state carried."""
    H, dk, dv = 32, 128, 128
    g = torch.Generator().manual_seed(batch)
    state = (torch.randn(batch, H, dk, dv, generator=g) * 0.1).numpy()
    op = E.DeltaRule(state)
    st = state.copy()
    worst = 0.0
    for s in range(steps):
        bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).float().numpy()
        q, k, v = bf(batch, H, dk), bf(batch, H, dk), bf(batch, H, dv)
        q, k = O.l2norm(q) * np.float32(dk ** -0.5), O.l2norm(k)
        gg = np.log(O.sigmoid(bf(batch, H)))
        beta = O.sigmoid(bf(batch, H))
        out, _ = op.step(q, k, v, gg, beta)
        want = O.delta_rule_step(q, k, v, gg, beta, st)
        worst = max(worst, float(np.abs(out - want).max()))
    assert worst < 1e-5
    final = op.state()
    assert np.abs(final - st).max() < 1e-5 and np.isfinite(final).all()
    op.close()


def test_delta_rule_against_reference_vector(E, golden_dir):
    ops = np.load(os.path.join(golden_dir, "ops_golden.npz"))
    op = E.DeltaRule(ops["step_state"])
    out, _ = op.step(ops["step_q"], ops["step_k"], ops["step_v"], ops["step_g"], ops["step_beta"])
    assert np.abs(out - ops["step_out"]).max() < 1e-6
    assert np.abs(op.state() - ops["step_state_after"]).max() < 1e-6
    op.close()
