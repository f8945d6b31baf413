"""Parity of the CUDA engine, called through the C ABI, against (a) outputs of the unmodified
reference stored in tests/golden/ and (b) the CPU oracle on the same seeded inputs.

Tolerances (fp32 everywhere, summation orders differ between cuBLAS-free CUDA kernels, MKL and numpy):
router picks identical; router weights 1e-5; logits max-abs 3e-4 on models whose logits are O(1);
greedy tokens identical. Where the engine feeds a prompt token by token and the reference used its
chunked DeltaNet form, the reference's own acceptance applies (tests/test_hybrid_rust.py:136-144):
KL < 2e-2 and top-1 equal unless the reference's top-2 margin is under 0.05 - measured here ~1e-9.
"""
import os

import numpy as np
import pytest

from oracle import hybrid_oracle as O

pytestmark = pytest.mark.gpu
TOL = 3e-4


@pytest.fixture(scope="module")
def E(pkg):
    import importlib
    eng = importlib.import_module("b200moe.engine")
    eng.load_library()
    return eng


@pytest.fixture(scope="module")
def micro(golden_dir):
    return np.load(os.path.join(golden_dir, "micro_golden.npz"))


def kl_rows(ref, got):
    def lsm(x):
        x = x.astype(np.float64)
        m = x.max(-1, keepdims=True)
        return x - m - np.log(np.exp(x - m).sum(-1, keepdims=True))
    a, b = lsm(ref), lsm(got)
    return (np.exp(a) * (a - b)).sum(-1)


def reference_accepts(ref, got):
    kl = kl_rows(ref, got)
    top1 = ref.argmax(-1) == got.argmax(-1)
    srt = np.sort(ref, -1)
    margin = srt[..., -1] - srt[..., -2]
    assert np.isfinite(got).all()
    assert kl.max() < 2e-2
    assert (top1 | (margin < 0.05)).all()
    return kl.max()


def test_token_by_token_matches_reference(E, micro, micro_path):
    """Every feed is one token: the engine and the reference run the same recurrence."""
    e = E.HybridEngine.load(micro_path, max_context=64, kv_dtype=E.KV_F32)
    e.set_taps([0, 3])
    ids = micro["prompt"].tolist() + micro["greedy_tokens"].tolist()
    for j, t in enumerate(ids):
        lg = e.feed([t])
        assert np.abs(lg - micro["single_logits"][j]).max() < TOL, j
        for layer in range(4):
            idx, w = e.router(layer, 8)
            assert (idx[0] == micro["single_routes"][j][layer]).all(), (j, layer)
            assert np.abs(w[0] - micro["single_route_w"][j][layer]).max() < 1e-5
        taps = e.taps()
        assert np.abs(taps[0, 0] - micro["single_taps"][j][0]).max() < TOL
        assert np.abs(taps[1, 0] - micro["single_taps"][j][3]).max() < TOL
        assert np.abs(e.hidden()[0] - micro["single_taps"][j][3]).max() < TOL
    assert e.length() == len(ids) and e.cap() == 64
    hits, page_ins = e.expert_counters()
    assert hits == len(ids) * 4 * 8 and page_ins == 0
    e.close()


def test_prompt_then_greedy_matches_reference(E, micro, micro_path):
    """The reference fed the prompt in one piece (chunked DeltaNet form); greedy tokens must be
    identical and every row inside the reference's own acceptance, here far tighter."""
    e = E.HybridEngine.load(micro_path, max_context=64)
    rows = [e.feed(micro["prompt"].tolist())]
    toks = []
    for _ in range(24):
        toks.append(int(np.argmax(rows[-1])))
        rows.append(e.feed([toks[-1]]))
    rows = np.stack(rows)
    assert toks == micro["greedy_tokens"].tolist()
    reference_accepts(micro["greedy_logits"], rows)
    assert np.abs(rows - micro["greedy_logits"]).max() < TOL
    e.close()


def test_feeds_of_5_30_100(E, micro, micro_path):
    e = E.HybridEngine.load(micro_path, max_context=160)
    ids = micro["multi_ids"].tolist()
    rows = [e.feed(f) for f in (ids[:5], ids[5:35], ids[35:])]
    toks = []
    for _ in range(4):
        toks.append(int(np.argmax(rows[-1])))
        rows.append(e.feed([toks[-1]]))
    assert toks == micro["multi_tokens"].tolist()
    reference_accepts(micro["multi_logits"], np.stack(rows))
    assert np.abs(np.stack(rows) - micro["multi_logits"]).max() < TOL
    e.close()


def test_snapshot_crop_rewinds(E, micro, micro_path):
    """tests/test_hybrid_rust.py:229-242 at small scale, against the reference's own rows."""
    e = E.HybridEngine.load(micro_path, max_context=128)
    ids = micro["rewind_ids"].tolist()
    a, b, c = ids[:30], ids[30:50], ids[50:65]
    rows, kept = [], []
    rows.append(e.feed(a[:12])); e.snapshot()
    rows.append(e.feed(a[12:])); e.snapshot()
    rows.append(e.feed(b))
    kept.append(e.crop(len(a) + 3))
    rows.append(e.feed(c))
    kept.append(e.crop(5))
    rows.append(e.feed([1, 2, 3]))
    assert kept == micro["rewind_kept"].tolist() == [30, 0]
    assert np.abs(np.stack(rows) - micro["rewind_logits"]).max() < TOL
    assert np.abs(rows[3] - micro["rewind_fresh"][0]).max() < TOL
    assert np.abs(rows[4] - micro["rewind_fresh"][1]).max() < TOL
    assert e.crop(1000) == 3            # cropping past the end keeps everything
    # only two snapshots are kept (aegist_rs/src/hybrid.rs:442): the oldest one is replaced
    e.snapshot(); e.feed([4]); e.snapshot(); e.feed([5]); e.snapshot(); e.feed([6])
    assert e.crop(3) == 0
    e.close()


def test_batch_decode_matches_reference(E, micro, micro_path):
    bp = micro["batch_prompt"]
    e = E.HybridEngine.load(micro_path, max_context=32, batch=4)
    rows = []
    for t in range(6):
        nxt, lg = e.feed_batch(bp[:, t])
        rows.append(lg)
        for layer in range(4):
            idx, _ = e.router(layer, 8)
            assert (idx == micro["batch_routes"][t][layer]).all()
    for s in range(8):
        cur = rows[-1].argmax(-1)
        assert (cur == micro["batch_tokens"][s]).all() and (nxt == cur).all()
        nxt, lg = e.feed_batch(cur)
        rows.append(lg)
    assert np.abs(np.stack(rows) - micro["batch_logits"]).max() < TOL
    e.close()


def test_device_greedy_loop_equals_feed_loop(E, micro, micro_path):
    e = E.HybridEngine.load(micro_path, max_context=64)
    prompt = micro["prompt"].tolist()
    e.feed(prompt[:-1], want_logits=False)
    toks, ms = e.decode_greedy([prompt[-1]], 25)
    assert toks[:24, 0].tolist() == micro["greedy_tokens"].tolist()
    assert ms > 0 and e.length() == len(prompt) + 24
    e.close()


def test_feed_into_a_page_locked_buffer(E, micro, micro_path):
    """feed(out=host_buffer) returns the same logits as feed() into a fresh array, and refuses a wrong array."""
    prompt = micro["prompt"].tolist()
    a = E.HybridEngine.load(micro_path, max_context=64)
    b = E.HybridEngine.load(micro_path, max_context=64)
    ids_h, out_h = b.host_buffer(len(prompt), np.uint32), b.host_buffer(b.vocab)
    ids_h[:] = prompt
    want = a.feed(prompt)
    got = b.feed(ids_h, out=out_h)
    assert got is out_h and np.array_equal(got, want)
    with pytest.raises(E.EngineError, match="vocab"):
        b.feed([1], out=np.zeros(3, np.float32))
    a.close()
    b.close()


def test_split_attention_long_context_and_bf16_cache(E, micro_path):
    """350 tokens with room for 4096: the attention runs as many slices (most of them empty at
    first), fp32 and bf16 caches, each against the oracle with the same cache rounding."""
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 512, 350).tolist()
    brain = O.Brain(micro_path)
    for kv, name in ((E.KV_F32, "f32"), (E.KV_BF16, "bf16")):
        e = E.HybridEngine.load(micro_path, max_context=4096, kv_dtype=kv)
        model = O.HybridOracle(brain)
        cache = model.new_cache(1, 400, kv_dtype=name)
        worst = 0.0
        for j, t in enumerate(ids):
            want = model.forward(np.asarray([[t]]), cache)[0]
            got = e.feed([t])
            if j % 10 == 0 or j > 330:
                worst = max(worst, float(np.abs(got - want).max()))
                assert int(np.argmax(got)) == int(np.argmax(want))
        assert worst < TOL, (name, worst)
        e.close()


def test_errors_are_messages_not_aborts(E, micro_path, tmp_path):
    e = E.HybridEngine.load(micro_path, max_context=8)
    with pytest.raises(E.EngineError, match="outside the vocabulary"):
        e.feed([512])
    e.feed([1, 2, 3, 4, 5, 6])
    with pytest.raises(E.EngineError, match="context full: 6 \\+ 3 tokens > 8"):
        e.feed([1, 2, 3])
    assert e.length() == 6              # a refused feed changes nothing
    with pytest.raises(E.EngineError, match="out of range"):
        e.set_taps([4])
    e.close()
    bad = tmp_path / "bad.nx"
    bad.write_bytes(b"NOTANNXFILE" + bytes(100))
    with pytest.raises(E.EngineError, match="not an .nx file"):
        E.HybridEngine.load(str(bad))
    raw = open(micro_path, "rb").read()
    (tmp_path / "cut.nx").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(E.EngineError, match="truncated|past the end"):
        E.HybridEngine.load(str(tmp_path / "cut.nx"))
    with pytest.raises(E.EngineError, match="does not exist"):
        E.HybridEngine.load(micro_path, device=99)
    assert E.verify_file(micro_path) == {"base": True, "engine": True, "cores": True}
    flipped = bytearray(raw)
    flipped[-200000] ^= 1
    (tmp_path / "flip.nx").write_bytes(flipped)
    assert not all(E.verify_file(str(tmp_path / "flip.nx")).values())


def test_sampler_matches_the_reference_algorithm(E):
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(4096).astype(np.float32) * 3
    for seed in range(40):
        a, b = E.Rng(seed), O.Rng(seed)
        for temp, top_p, top_k in ((0.7, 0.8, 20), (1.0, 0.95, 50), (0.0, 0.9, 20), (1.3, 1.0, 4096)):
            assert E.sample(logits, temp, top_p, top_k, a) == O.sample(logits, temp, top_p, top_k, b)
    tie = np.array([1.0, 5.0, 5.0, 2.0], dtype=np.float32)
    assert E.sample(tie, 0.0, 1.0, 4, E.Rng(0)) == 1


def test_tiny_config_end_to_end(E, pkg, golden_dir, tiny_path):
    """The CPU-runnable case of the benchmark spec: 4 layers, hidden 512, vocab 32768, 64 experts
    top-8, 32 random prompt tokens, 64 greedy tokens. The brain is rebuilt from the seed; when its
    group hashes equal those of the file the reference wrote, the reference's own numbers are the
    target (router picks at all 4 x 96 points bit-exact, greedy tokens identical), else the oracle's."""
    from b200moe.nxfile import NxFile
    g = np.load(os.path.join(golden_dir, "tiny_golden.npz"))
    path = tiny_path
    with NxFile(path) as nx:
        same = nx.header["sha256"]["base"] == str(g["sha_base"])
    prompt, toks = g["prompt"].tolist(), g["tokens"].tolist()
    e = E.HybridEngine.load(path, max_context=104)
    if same:
        got_toks, cur = [], None
        for j, t in enumerate(prompt + toks):
            lg = e.feed([t])
            for layer in range(4):
                assert (e.router(layer, 8)[0][0] == g["single_routes"][j][layer]).all(), (j, layer)
            top = g["single_top_idx"][j]
            assert np.abs(lg[top] - g["single_top_val"][j]).max() < TOL
            m = lg.max()
            assert abs(m + np.log(np.exp(lg - m).sum()) - g["single_lse"][j]) < TOL
            if j >= len(prompt) - 1:
                got_toks.append(int(np.argmax(lg)))
        assert got_toks[:64] == toks
        assert np.abs(lg - g["single_full_rows"][2]).max() < TOL
    else:
        model = O.HybridOracle(O.Brain(path))
        cache = model.new_cache(1, 104)
        cur = None
        for j in range(len(prompt) + 64):
            t = prompt[j] if j < len(prompt) else cur
            want = model.forward(np.asarray([[t]]), cache)[0]
            got = e.feed([t])
            for layer in range(4):
                assert (e.router(layer, 8)[0][0] == model.last_route[layer][0][0]).all()
            assert np.abs(got - want).max() < TOL
            cur = int(np.argmax(got))
            assert cur == int(np.argmax(want))
    e.close()


@pytest.mark.parametrize("batch", [8, 20])
def test_batched_decode_tensor_core_path(E, tiny_path, batch):
    """Eight or more sequences: the int8 linears run as fp16 tensor-core products with the activations
    split in two halves. Against the oracle on the same batch: router picks identical, logits within
    the same 3e-4, greedy tokens identical, for 12 steps with carried state."""
    rng = np.random.default_rng(batch)
    ids = rng.integers(0, 32768, (batch, 5))
    e = E.HybridEngine.load(tiny_path, max_context=32, batch=batch)
    model = O.HybridOracle(O.Brain(tiny_path))
    cache = model.new_cache(batch, 32)
    cur = None
    for t in range(12):
        tok = ids[:, t] if t < 5 else cur
        want = model.forward(np.asarray(tok)[:, None], cache)
        nxt, got = e.feed_batch(tok)
        for layer in range(4):
            assert (e.router(layer, 8)[0] == model.last_route[layer][0]).all(), (t, layer)
        assert np.abs(got - want).max() < TOL, (t, float(np.abs(got - want).max()))
        cur = got.argmax(-1)
        assert (cur == want.argmax(-1)).all() and (nxt == cur).all()
    e.close()


@pytest.fixture(scope="module")
def wide_path(pkg, tmp_path_factory):
    """The tiny brain with expert and shared hidden sizes of 256 (multiples of the tensor-core K chunk),
    16 experts so that experts collect several tokens of a step, vocabulary 4096."""
    import dataclasses
    from b200moe import brain
    cfg = dataclasses.replace(pkg.HybridConfig.tiny(), vocab_size=4096, n_experts=16, expert_hidden=256, shared_hidden=256)
    path = str(tmp_path_factory.mktemp("wide") / "wide.nx")
    brain.write_brain(path, cfg, seed=3)
    return path


@pytest.mark.parametrize("batch", [16, 40])
def test_batched_decode_grouped_expert_gemm(E, wide_path, batch):
    """Sixteen or more sequences: the 4-bit experts run as a grouped tensor-core GEMM (picks sorted by
    expert, chunks of 32 tokens; batch 40 x top-8 over 16 experts gives chunks of 20 and of 32 + rest).
    Against the oracle: router picks identical, logits within 3e-4, greedy tokens identical, 10 steps."""
    rng = np.random.default_rng(100 + batch)
    ids = rng.integers(0, 4096, (batch, 4))
    e = E.HybridEngine.load(wide_path, max_context=32, batch=batch)
    model = O.HybridOracle(O.Brain(wide_path))
    cache = model.new_cache(batch, 32)
    cur = None
    for t in range(10):
        tok = ids[:, t] if t < 4 else cur
        want = model.forward(np.asarray(tok)[:, None], cache)
        nxt, got = e.feed_batch(tok)
        for layer in range(4):
            assert (e.router(layer, 8)[0] == model.last_route[layer][0]).all(), (t, layer)
        assert np.abs(got - want).max() < TOL, (t, float(np.abs(got - want).max()))
        cur = got.argmax(-1)
        assert (cur == want.argmax(-1)).all() and (nxt == cur).all()
    e.close()


@pytest.mark.parametrize("splits", [2, 5])
def test_bf16_cache_attention_over_several_tiles(E, tiny_path, splits, monkeypatch):
    """bf16 cache on the tensor-core attention kernel with few, long slices (B2_ATTN_SPLITS): slices of several
    64-position tiles, the double-buffered path, partial last tiles, two sequences; against the oracle with the
    same cache rounding for 200 tokens."""
    monkeypatch.setenv("B2_ATTN_SPLITS", str(splits))
    rng = np.random.default_rng(40 + splits)
    ids = rng.integers(0, 32768, (2, 200))
    e = E.HybridEngine.load(tiny_path, max_context=256, batch=2, kv_dtype=E.KV_BF16)
    model = O.HybridOracle(O.Brain(tiny_path))
    cache = model.new_cache(2, 256, kv_dtype="bf16")
    worst = 0.0
    for t in range(200):
        want = model.forward(ids[:, t][:, None], cache)
        nxt, got = e.feed_batch(ids[:, t])
        if t % 16 == 0 or t > 190:
            worst = max(worst, float(np.abs(got - want).max()))
            assert (got.argmax(-1) == want.argmax(-1)).all()
    assert worst < TOL, worst
    e.close()


def test_bf16_cache_attention_single_buffered_blocks(E, pkg, tmp_path, monkeypatch):
    """With two or more blocks per SM to choose from (sequences x KV heads x slices) the attention kernel runs
    single-buffered, two blocks to an SM; slices of two tiles here (32 sequences, 4 KV heads, 3 slices of a 320-token
    cache), against the oracle with the same cache rounding."""
    import dataclasses
    from b200moe import brain
    monkeypatch.setenv("B2_ATTN_SPLITS", "3")
    cfg = dataclasses.replace(pkg.HybridConfig.micro(), n_layers=2, layer_types=["delta", "attn"], n_heads=8, n_kv_heads=4)
    path = str(tmp_path / "kv4.nx")
    brain.write_brain(path, cfg, seed=5)
    B, T = 32, 150
    assert 3 * cfg.n_kv_heads * B >= 2 * 148
    rng = np.random.default_rng(77)
    ids = rng.integers(0, cfg.vocab_size, (B, T))
    e = E.HybridEngine.load(path, max_context=320, batch=B, kv_dtype=E.KV_BF16)
    model = O.HybridOracle(O.Brain(path))
    cache = model.new_cache(B, 320, kv_dtype="bf16")
    worst = 0.0
    for t in range(T):
        want = model.forward(ids[:, t][:, None], cache)
        nxt, got = e.feed_batch(ids[:, t])
        if t % 16 == 0 or t > T - 6:
            worst = max(worst, float(np.abs(got - want).max()))
            assert (got.argmax(-1) == want.argmax(-1)).all()
    assert worst < TOL, worst
    e.close()


def test_step_timeline(E, tiny_path):
    """b2_debug_trace_step: one row per launch of a graph-run step; the kernels that record stamp a first-in time,
    a last-out time after it, and launches follow one another in time; the step still advances the state."""
    e = E.HybridEngine.load(tiny_path, max_context=32)
    e.feed([1, 2, 3])
    n0 = e.length()
    t = e.trace_step().astype(np.int64)
    assert e.length() == n0 + 1
    assert t.shape == (e.launches_per_step(), 16)
    live = t[t[:, 5] > 0]
    assert len(live) >= 4 * 5                       # every per-layer kernel of the 4 layers records
    assert (live[:, 4] > live[:, 0]).all()          # last block out after first block in
    assert (np.diff(live[:, 4]) > 0).all()          # kernels end in launch order
    assert set(live[:, 5]) >= {1, 3, 5, 6, 7, 8}    # GEMV, delta step, expert gate/up, expert down, attention, merge
    e.close()
