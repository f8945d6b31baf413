"""The kernels the benchmark runs, at the benchmark's widths, against the CPU oracle.

Every dispatch decision of the engine depends on the shape (hidden 2048, 256 experts top-8 with
intermediate 512, attention heads of 256 with 8 query heads per KV head and 64 rotary dims, DeltaNet
heads of 128 x 128, vocabulary 151,936), so the small fixtures do not reach the code paths the
full model uses. Here the first four layers of the 35B-shaped model (3 DeltaNet + 1 attention) plus
its head are rebuilt from seed 0 with every 1-D parameter perturbed, and each decode step is compared
with the oracle on the same weights: router picks of every layer identical and in order, router weights
to 1e-5, logits to 3e-4 max-abs, arg-max equal, and the reference's own acceptance
(tests/test_hybrid_rust.py:136-144: KL < 2e-2, top-1 equal unless the margin is under 0.05).
"""
import numpy as np
import pytest
import torch

from oracle import hybrid_oracle as O

pytestmark = pytest.mark.gpu
TOL = 3e-4


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def kl_rows(ref, got):
    def lsm(x):
        x = x.astype(np.float64)
        m = x.max(-1, keepdims=True)
        return x - m - np.log(np.exp(x - m).sum(-1, keepdims=True))
    a, b = lsm(ref), lsm(got)
    return (np.exp(a) * (a - b)).sum(-1)


def reference_accepts(ref, got):
    srt = np.sort(ref, -1)
    margin = srt[..., -1] - srt[..., -2]
    assert np.isfinite(got).all()
    assert kl_rows(ref, got).max() < 2e-2
    assert ((ref.argmax(-1) == got.argmax(-1)) | (margin < 0.05)).all()


@pytest.fixture(scope="module")
def E(pkg):
    import importlib
    eng = importlib.import_module("b200moe.engine")
    eng.load_library()
    return eng


@pytest.fixture(scope="module")
def full4(pkg):
    """(config, device tensors for the engine, oracle over the same bits)."""
    from b200moe import brain
    cfg = pkg.HybridConfig.full(n_layers=4)
    dev = list(brain.random_brain(cfg, seed=0, device="cuda:0", vary_1d=True))
    host = {}
    for name, dt, t in dev:
        c = t.detach().contiguous().cpu()
        host[name] = (dt, bits(c) if dt == "bf16" else c.numpy())
    model = O.HybridOracle(O.DictBrain(cfg.to_dict(), host), hold_weights=True)
    return cfg, dev, model


def check_step(e, model, cfg, got, want, tag, wtol=1e-5, tol=TOL):
    for layer in range(cfg.n_layers):
        idx, w = e.router(layer, cfg.experts_active)
        widx, ww = model.last_route[layer]
        assert np.array_equal(idx, widx), (tag, layer, idx, widx)
        assert np.abs(w - ww).max() < wtol, (tag, layer)
    err = float(np.abs(got - want).max())
    assert err < tol, (tag, err)
    assert np.array_equal(got.argmax(-1), want.argmax(-1)), tag
    reference_accepts(want, got)
    return err


@pytest.mark.parametrize("kv", ["f32", "bf16"])
def test_batch1_decode_at_full_width(E, full4, kv):
    """Batch 1: the kernels of the headline number (GEMVs with the conv / gate / arg-max epilogues at 8192 and
    151,936 rows, the delta step with 128-wide keys, attention with 256-wide heads, the expert kernels with their
    in-block top-8 over 256 experts)."""
    cfg, dev, model = full4
    e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=4096, device=0, batch=1,
                                    kv_dtype=E.KV_F32 if kv == "f32" else E.KV_BF16)
    cache = model.new_cache(1, 64, kv_dtype=kv)
    rng = np.random.default_rng(7)
    ids = rng.integers(0, cfg.vocab_size, 5).tolist()
    tok = None
    for j in range(10):
        t = ids[j] if j < len(ids) else tok
        want = model.forward(np.asarray([[t]]), cache)
        got = e.feed([t])[None]
        # bf16 cache: keys and values are ROUNDED to bfloat16 when they are stored, by the engine and by the oracle
        # alike. A key that the two compute 1e-7 apart can fall on either side of a rounding boundary, and then it
        # differs by a whole bf16 step (2^-8 relative) in the two caches; with 1024 stored values per token and layer
        # that happens once every few tokens and moves the logits by a few 1e-4 (measured 3.9e-4 at the seventh
        # token, 1.3e-5 on a router weight). The fp32 cache has no such step and keeps the tight bounds.
        check_step(e, model, cfg, got, want, (kv, j), *((1e-5, TOL) if kv == "f32" else (1e-4, 2e-3)))
        tok = int(got.argmax())
    hid = e.hidden()
    assert np.abs(hid[0] - model.final_hidden[0]).max() < TOL
    e.close()


def test_batch1_greedy_loop_on_the_device_at_full_width(E, full4):
    """The device-resident greedy loop (what the benchmark times) produces the oracle's greedy tokens."""
    cfg, dev, model = full4
    e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=4096, device=0, batch=1, kv_dtype=E.KV_BF16)
    cache = model.new_cache(1, 64, kv_dtype="bf16")
    tok, want = 12345, []
    for _ in range(12):
        tok = int(model.forward(np.asarray([[tok]]), cache)[0].argmax())
        want.append(tok)
    got, ms = e.decode_greedy([12345], 12)
    assert got[:, 0].tolist() == want
    e.close()


@pytest.mark.parametrize("batch", [2, 6, 8, 16, 64])
def test_batched_decode_at_full_width(E, full4, batch):
    """2: the two-sequence variants of the batch-1 kernels; 6, 8, 16 and 64: the tcgen05 GEMMs and the grouped 4-bit expert
    GEMM with its pick grouping, all at 2048 / 256 experts / 512."""
    cfg, dev, model = full4
    before = E.load_library().b2_debug_umma_launches()
    e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=64, device=0, batch=batch, kv_dtype=E.KV_F32)
    # from 6 sequences on every GEMV group of the step graph is a tcgen05 GEMM: 3 per layer (mixer in, mixer out, MoE in) + the head,
    # and the 4-bit experts are two more per layer (gate/up, down)
    n_umma = E.load_library().b2_debug_umma_launches() - before
    assert n_umma == (5 * cfg.n_layers + 1 if batch >= 6 else 0), n_umma
    cache = model.new_cache(batch, 16)
    rng = np.random.default_rng(batch)
    tok = rng.integers(0, cfg.vocab_size, batch)
    for j in range(3):
        want = model.forward(np.asarray(tok)[:, None], cache)
        nxt, got = e.feed_batch(tok)
        check_step(e, model, cfg, got, want, (batch, j))
        assert np.array_equal(nxt, got.argmax(-1))
        tok = got.argmax(-1)
    e.close()


@pytest.mark.parametrize("kv", ["f32", "bf16"])
def test_prompt_chunks_at_full_width(E, full4, kv):
    """A 300-token prompt in one feed: two chunks of 128 tokens and one of 44 go through the layers with their tokens as
    the columns of the tcgen05 GEMMs and of the grouped expert GEMM, conv / delta rule / attention walk them in order;
    then single-token steps continue from the state the chunks left. Against the oracle, which runs the prompt through
    the reference's chunked DeltaNet form: the reference's own acceptance, logits within tolerance, same greedy tokens;
    and bit-for-bit the same continuation as an engine that was fed the prompt token by token is NOT required (the sums
    run in another order), only agreement within the same bounds."""
    cfg, dev, model = full4
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab_size, 300)
    e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=512, device=0, batch=1,
                                    kv_dtype=E.KV_F32 if kv == "f32" else E.KV_BF16)
    cache = model.new_cache(1, 400, kv_dtype=kv)
    want = model.forward(prompt[None, :], cache)
    got = e.feed(prompt)[None]
    tol = TOL if kv == "f32" else 2e-3
    assert e.length() == 300
    reference_accepts(want, got)
    assert np.abs(got - want).max() < tol, float(np.abs(got - want).max())
    for layer in range(cfg.n_layers):                      # the last token's picks are where a decode step leaves them
        assert np.array_equal(e.router(layer, cfg.experts_active)[0][0], model.last_route[layer][0][-1]), layer
    tok = int(want.argmax())
    for j in range(4):
        want = model.forward(np.asarray([[tok]]), cache)
        got = e.feed([tok])[None]
        assert np.abs(got - want).max() < tol, (j, float(np.abs(got - want).max()))
        assert int(got.argmax()) == int(want.argmax())
        tok = int(want.argmax())
    # a second engine fed the same prompt token by token agrees with the chunked one
    e2 = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=512, device=0, batch=1,
                                     kv_dtype=E.KV_F32 if kv == "f32" else E.KV_BF16)
    for t in prompt[:-1]:
        e2.feed([int(t)], want_logits=False)
    one = e2.feed([int(prompt[-1])])
    e3 = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=512, device=0, batch=1,
                                     kv_dtype=E.KV_F32 if kv == "f32" else E.KV_BF16)
    assert np.abs(e3.feed(prompt) - one).max() < tol
    for eng in (e, e2, e3):
        eng.close()


def test_router_ties_and_bias_at_256_experts(E, full4):
    """A router bias that makes groups of experts exactly equal must still give the reference's order (ties to the
    lower index), and the bias must act as in the oracle."""
    cfg, dev, model = full4
    e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=64, device=0, batch=1, kv_dtype=E.KV_F32)
    bias = np.zeros(cfg.n_experts, np.float32)
    bias[[3, 77, 200, 201, 255]] = 50.0          # far above any logit: these five lead, in index order unless the logits differ
    try:
        for layer in range(cfg.n_layers):
            e.set_router_bias(layer, bias)
            model.router_bias[layer] = bias
        cache = model.new_cache(1, 16)
        for j, t in enumerate([5, 99999, 4242]):
            want = model.forward(np.asarray([[t]]), cache)
            got = e.feed([t])[None]
            check_step(e, model, cfg, got, want, ("bias", j))
    finally:
        model.router_bias.clear()
    e.close()


def test_deltanet_mixer_from_the_hidden_vector(E, pkg):
    """The whole gated-DeltaNet layer from the hidden vector at hidden 2048 (16 key / 32 value heads of 128, conv
    kernel 4) for 1000 consecutive single-token steps with the state carried: one DeltaNet layer whose input
    rows (the embedding table) are N(0, 1) bf16, so in_qkv / in_z / in_a / in_b, the conv with its state, the L2
    norms, the decay and beta gates, the delta rule, the gated RMSNorm and the out projection all run from a
    N(0, 1) hidden vector every step. Compared every step on the layer's output row and at the end on the logits."""
    import dataclasses
    from b200moe import brain
    cfg = dataclasses.replace(pkg.HybridConfig.full(n_layers=1), vocab_size=2048, layer_types=["delta"])
    dev = []
    for name, dt, t in brain.random_brain(cfg, seed=2, device="cuda:0", vary_1d=True):
        if name == "embed.weight":
            t = torch.randn(t.shape, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
        dev.append((name, dt, t))
    host = {n: (dt, bits(t.cpu()) if dt == "bf16" else t.cpu().numpy()) for n, dt, t in dev}
    model = O.HybridOracle(O.DictBrain(cfg.to_dict(), host), hold_weights=True)
    for batch, steps in ((1, 1000), (16, 60)):
        e = E.HybridEngine.from_tensors(cfg.to_dict(), dev, max_context=steps + 8, device=0, batch=batch, kv_dtype=E.KV_F32)
        cache = model.new_cache(batch, steps + 8)
        rng = np.random.default_rng(batch)
        worst = 0.0
        for s in range(steps):
            tok = rng.integers(0, cfg.vocab_size, batch)
            want = model.forward(tok[:, None], cache)
            if batch == 1:
                got = e.feed([int(tok[0])])[None]
            else:
                got = e.feed_batch(tok)[1]
            worst = max(worst, float(np.abs(e.hidden() - model.final_hidden).max() / max(1.0, np.abs(model.final_hidden).max())))
            if s % 50 == 0 or s == steps - 1:
                assert np.abs(got - want).max() < TOL * max(1.0, float(np.abs(want).max())), (batch, s)
        assert worst < 2e-5, (batch, worst)
        e.close()


@pytest.mark.parametrize("batch", [16, 64])
def test_delta_rule_1000_steps_batched(E, batch):
    """The delta-rule core at 32 heads of 128 x 128 for 1000 steps with the state carried, batch 16 and 64. The
    numpy oracle needs about a third of a second per step at batch 64, so the stepwise check uses the same five
    equations (aegist/hybrid.py:318-324) in torch fp32 on the GPU, which is first pinned to the numpy oracle on
    the first steps; the final state is compared as well."""
    H, dk, dv = 32, 128, 128
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator().manual_seed(100 + batch)
    state = (torch.randn(batch, H, dk, dv, generator=g) * 0.1)
    op = E.DeltaRule(state.numpy())
    st_np = state.numpy().copy()
    st = state.cuda()

    def torch_step(q, k, v, gg, beta, S):
        S = S * torch.exp(gg)[..., None, None]
        kv = (S * k[..., None]).sum(-2)
        delta = (v - kv) * beta[..., None]
        S = S + k[..., None] * delta[..., None, :]
        return (S * q[..., None]).sum(-2), S

    worst = 0.0
    for s in range(1000):
        bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).float()
        q, k, v = bf(batch, H, dk), bf(batch, H, dk), bf(batch, H, dv)
        q = torch.from_numpy(O.l2norm(q.numpy()) * np.float32(dk ** -0.5))
        k = torch.from_numpy(O.l2norm(k.numpy()))
        gg = torch.log(torch.sigmoid(bf(batch, H)))
        beta = torch.sigmoid(bf(batch, H))
        out, _ = op.step(q.numpy(), k.numpy(), v.numpy(), gg.numpy(), beta.numpy())
        want, st = torch_step(q.cuda(), k.cuda(), v.cuda(), gg.cuda(), beta.cuda(), st)
        want = want.cpu().numpy()
        if s < 3:
            ref = O.delta_rule_step(q.numpy(), k.numpy(), v.numpy(), gg.numpy(), beta.numpy(), st_np)
            assert np.abs(ref - want).max() < 2e-6
            assert np.abs(st_np - st.cpu().numpy()).max() < 2e-6
        worst = max(worst, float(np.abs(out - want).max()))
    assert worst < 1e-5, worst
    final = op.state()
    assert np.abs(final - st.cpu().numpy()).max() < 1e-5 and np.isfinite(final).all()
    op.close()
