"""The CPU oracle against outputs of the unmodified reference (tests/golden/*.npz, written by
tests/golden/make_golden.py). fp32 throughout: router picks must be identical, logits within 2e-5
absolute (the reference sums in MKL's order, numpy in OpenBLAS's)."""
import os

import numpy as np
import pytest

from oracle import hybrid_oracle as O

TOL = 2e-5


@pytest.fixture(scope="module")
def micro(golden_dir):
    return np.load(os.path.join(golden_dir, "micro_golden.npz"))


@pytest.fixture(scope="module")
def ops(golden_dir):
    return np.load(os.path.join(golden_dir, "ops_golden.npz"))


@pytest.fixture(scope="module")
def model(micro_path):
    return O.HybridOracle(O.Brain(micro_path))


def routes_of(model, n_layers, row=-1):
    return np.stack([model.last_route[i][0][row] for i in range(n_layers)])


def test_prompt_then_greedy(model, micro):
    prompt = micro["prompt"].tolist()
    cache = model.new_cache(1, 64)
    rows, routes, taps, toks = [], [], [], []
    rows.append(model.forward(np.asarray([prompt]), cache)[0])
    routes.append(routes_of(model, 4))
    taps.append(np.stack([model.last_hidden[i][0] for i in range(4)]))
    for _ in range(24):
        toks.append(int(np.argmax(rows[-1])))
        rows.append(model.forward(np.asarray([[toks[-1]]]), cache)[0])
        routes.append(routes_of(model, 4))
        taps.append(np.stack([model.last_hidden[i][0] for i in range(4)]))
    assert toks == micro["greedy_tokens"].tolist()
    assert (np.stack(routes) == micro["greedy_routes"]).all()
    assert np.abs(np.stack(rows) - micro["greedy_logits"]).max() < TOL
    assert np.abs(np.stack(taps) - micro["greedy_taps"]).max() < TOL


def test_token_by_token(model, micro):
    ids = micro["prompt"].tolist() + micro["greedy_tokens"].tolist()
    cache = model.new_cache(1, 64)
    for j, t in enumerate(ids):
        lg = model.forward(np.asarray([[t]]), cache)[0]
        assert np.abs(lg - micro["single_logits"][j]).max() < TOL
        assert (routes_of(model, 4) == micro["single_routes"][j]).all()
        w = np.stack([model.last_route[i][1][0] for i in range(4)])
        assert np.abs(w - micro["single_route_w"][j]).max() < 1e-6


def test_feeds_of_5_30_100(model, micro):
    ids = micro["multi_ids"].tolist()
    cache = model.new_cache(1, 160)
    rows = [model.forward(np.asarray([f]), cache)[0] for f in (ids[:5], ids[5:35], ids[35:])]
    toks = []
    for _ in range(4):
        toks.append(int(np.argmax(rows[-1])))
        rows.append(model.forward(np.asarray([[toks[-1]]]), cache)[0])
    assert toks == micro["multi_tokens"].tolist()
    assert np.abs(np.stack(rows) - micro["multi_logits"]).max() < TOL


def test_snapshot_crop(model, micro):
    ids = micro["rewind_ids"].tolist()
    a, b, c = ids[:30], ids[30:50], ids[50:65]
    cache = model.new_cache(1, 128, keep=4)
    rows, kept = [], []
    rows.append(model.forward(np.asarray([a[:12]]), cache)[0]); cache.snapshot()
    rows.append(model.forward(np.asarray([a[12:]]), cache)[0]); cache.snapshot()
    rows.append(model.forward(np.asarray([b]), cache)[0])
    kept.append(cache.crop(len(a) + 3))
    rows.append(model.forward(np.asarray([c]), cache)[0])
    kept.append(cache.crop(5))
    rows.append(model.forward(np.asarray([[1, 2, 3]]), cache)[0])
    assert kept == micro["rewind_kept"].tolist() == [30, 0]
    assert np.abs(np.stack(rows) - micro["rewind_logits"]).max() < TOL
    # rewound == fed fresh, in the reference and here
    assert np.abs(rows[3] - micro["rewind_fresh"][0]).max() < TOL
    assert np.abs(rows[4] - micro["rewind_fresh"][1]).max() < TOL


def test_batch_decode(model, micro):
    bp = micro["batch_prompt"]
    cache = model.new_cache(4, 32)
    rows = []
    for t in range(6):
        rows.append(model.forward(bp[:, t: t + 1], cache))
        assert (np.stack([model.last_route[i][0] for i in range(4)]) == micro["batch_routes"][t]).all()
    for s in range(8):
        cur = np.argmax(rows[-1], -1)
        assert (cur == micro["batch_tokens"][s]).all()
        rows.append(model.forward(cur[:, None], cache))
    assert np.abs(np.stack(rows) - micro["batch_logits"]).max() < TOL


def test_q4_dequantize_and_int8_linear(ops):
    deq = O.q4_dequantize(ops["q4_packed"], ops["q4_scale"], ops["q4_min"], 64)
    assert (deq == ops["q4_deq"]).all()
    w = ops["i8_q"].astype(np.float32) * O.bf16_to_f32(ops["i8_scale"])
    y = ops["i8_x"] @ w.T
    assert np.abs(y - ops["i8_y"]).max() < 1e-6


def test_moe_layer(model, ops):
    y = model.moe(0, ops["moe_h"])
    idx, w = model.last_route[0]
    assert (idx == ops["moe_idx"]).all()
    assert np.abs(w - ops["moe_w"]).max() < 1e-6
    assert np.abs(y - ops["moe_y"]).max() < TOL


def test_deltanet_mixer(model, ops):
    xs = ops["mixer_x"]
    cache = model.new_cache(2, 16)
    ys = [model.deltanet(0, xs[:, :3], cache)]
    cache.length = 3
    for t in range(3, 9):
        ys.append(model.deltanet(0, xs[:, t: t + 1], cache))
        cache.length += 1
    assert np.abs(np.concatenate(ys, 1) - ops["mixer_y"]).max() < TOL
    assert np.abs(cache.state[0] - ops["mixer_state"]).max() < TOL
    assert np.abs(cache.conv[0] - ops["mixer_conv"]).max() < TOL


def test_delta_rule_step_and_chunked(ops):
    st = ops["step_state"].copy()
    o = O.delta_rule_step(ops["step_q"], ops["step_k"], ops["step_v"], ops["step_g"], ops["step_beta"], st)
    assert np.abs(o - ops["step_out"]).max() < 1e-6
    assert np.abs(st - ops["step_state_after"]).max() < 1e-6
    o, S = O.delta_rule_chunked(ops["chunk_q"], ops["chunk_k"], ops["chunk_v"], ops["chunk_g"], ops["chunk_beta"],
                                ops["step_state"].copy())
    assert np.abs(o - ops["chunk_out"]).max() < TOL
    assert np.abs(S - ops["chunk_state_after"]).max() < TOL
    # the two forms are the same recurrence
    st = ops["step_state"].copy()
    outs = [O.delta_rule_step(ops["chunk_q"][:, :, t], ops["chunk_k"][:, :, t], ops["chunk_v"][:, :, t],
                              ops["chunk_g"][:, :, t], ops["chunk_beta"][:, :, t], st) for t in range(70)]
    assert np.abs(np.stack(outs, 2) - ops["chunk_out"]).max() < 1e-4
    assert np.abs(st - ops["chunk_state_after"]).max() < 1e-4


def test_rope_tables(ops):
    cos, sin = O.rope_tables(64, 10_000_000.0, 8704)
    rows = ops["rope_rows"]
    assert np.abs(cos[rows] - ops["rope_cos"]).max() < 1e-6
    assert np.abs(sin[rows] - ops["rope_sin"]).max() < 1e-6


def test_sampler_known_answers():
    # splitmix64 with seed 0: the published first outputs of the algorithm
    r = O.Rng(0)
    assert [r.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    logits = np.array([0.1, 2.0, 2.0, -1.0, 1.5], dtype=np.float32)
    assert O.sample(logits, 0.0, 0.9, 20, O.Rng(1)) == 1          # greedy: the first maximum wins
    assert O.sample(logits, 1.0, 1e-9, 20, O.Rng(1)) == 1         # a vanishing nucleus keeps only the top token
    picks = {O.sample(logits, 1.0, 1.0, 2, O.Rng(s)) for s in range(64)}
    assert picks == {1, 2}                                        # top-k 2 never leaves the two largest
    counts = np.bincount([O.sample(logits, 0.7, 0.95, 20, O.Rng(s)) for s in range(2000)], minlength=5)
    assert counts[1] > counts[4] > counts[0] and counts[3] < 30


def test_core_engine_and_live_cores_against_the_reference(golden_dir):
    """The oracle's core engine (product-key routing, switch-on counts) and live cores on the brain the reference wrote
    with live cores: logits, picks, weights and counts of the unmodified reference."""
    g = np.load(os.path.join(golden_dir, "cores_golden.npz"))
    m = O.HybridOracle(O.Brain(os.path.join(golden_dir, "micro_cores.nx")))
    cache = m.new_cache(1, 64)
    ids = g["ids"].tolist()
    rows = [m.forward(np.asarray([ids[:8]]), cache)[0]]
    cid = [np.stack([m.last_cores[i][0][-1] for i in range(4)])]
    cw = [np.stack([m.last_cores[i][1][-1] for i in range(4)])]
    for t in ids[8:]:
        rows.append(m.forward(np.asarray([[t]]), cache)[0])
        cid.append(np.stack([m.last_cores[i][0][-1] for i in range(4)]))
        cw.append(np.stack([m.last_cores[i][1][-1] for i in range(4)]))
    assert np.abs(np.stack(rows) - g["logits"]).max() < 2e-5
    assert np.array_equal(np.stack(cid), g["core_ids"])
    assert np.abs(np.stack(cw) - g["core_w"]).max() < 1e-5
    assert np.array_equal(m.core_counts, g["counts"])
