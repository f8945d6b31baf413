"""The core engine and the switchable cores (cores_apply, aegist_rs/kernels/aegist.cu:283-350; CoreEngine and
SparseCoreBank, aegist/model.py:199-232 and aegist/hybrid.py:655-771) against what the unmodified reference produced on a
micro brain with a few live cores (tests/golden/micro_cores.nx, cores_golden.npz), and against the oracle for the
batched and prompt-chunk paths."""
import os

import numpy as np
import pytest

from conftest import cores_file
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
def cores(golden_dir):
    return os.path.join(golden_dir, "micro_cores.nx"), np.load(os.path.join(golden_dir, "cores_golden.npz"))


def test_live_cores_and_counts_match_the_reference(E, cores):
    path, g = cores
    e = E.HybridEngine.load(path, max_context=64)
    assert "18 live cores" in e.describe()
    ids = g["ids"].tolist()
    rows = [e.feed(ids[:8])]
    for t in ids[8:]:
        rows.append(e.feed([t]))
    assert np.abs(np.stack(rows) - g["logits"]).max() < TOL
    counts = e.core_counts(4, 512)
    assert np.array_equal(counts, g["counts"])            # every pick of every token and layer tallied, as the reference does
    e.reset_counts()
    assert e.core_counts(4, 512).sum() == 0
    e.feed([ids[0]])
    assert e.core_counts(4, 512).sum() == 4 * 2           # 4 layers x cores_active
    e.close()


def test_a_fresh_brain_counts_too(E, micro_path):
    """No core is live in a fresh brain, so the cores add nothing, but the engine still routes and counts."""
    e = E.HybridEngine.load(micro_path, max_context=64)
    model = O.HybridOracle(O.Brain(micro_path))
    cache = model.new_cache(1, 64)
    for t in (5, 17, 300, 44):
        want = model.forward(np.asarray([[t]]), cache)[0]
        assert np.abs(e.feed([t]) - want).max() < TOL
    assert np.array_equal(e.core_counts(4, 512), model.core_counts)
    e.close()


@pytest.mark.parametrize("batch", [4, 8, 20])
def test_batched_decode_with_live_cores(E, cores, batch):
    """4: the small-batch kernels (picks made by the GEMV's finisher); 8 and 20: the tensor-core GEMMs with the picks made
    next to the router's top-k."""
    path, _ = cores
    e = E.HybridEngine.load(path, max_context=32, batch=batch)
    model = O.HybridOracle(O.Brain(path))
    cache = model.new_cache(batch, 32)
    rng = np.random.default_rng(batch)
    tok = rng.integers(0, 512, batch)
    for _ in range(6):
        want = model.forward(np.asarray(tok)[:, None], cache)
        nxt, got = e.feed_batch(tok)
        assert np.abs(got - want).max() < TOL
        tok = want.argmax(-1)
    assert np.array_equal(e.core_counts(4, 512), model.core_counts)
    e.close()


def test_prompt_chunk_with_live_cores(E, cores):
    path, _ = cores
    e = E.HybridEngine.load(path, max_context=256)
    model = O.HybridOracle(O.Brain(path))
    cache = model.new_cache(1, 256)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 512, 150)
    want = model.forward(prompt[None, :], cache)[0]
    got = e.feed(prompt)
    assert np.abs(got - want).max() < TOL
    assert np.array_equal(e.core_counts(4, 512), model.core_counts)
    e.close()


def test_cores_file_over_its_base(E, pkg, cores, micro_path, tmp_path):
    """Opening a cores file opens its base with the cores laid over it: the fresh micro brain + the live cores of the
    fixture = the reference's logits for the brain that stores both; a base whose weights changed is refused, and so
    is a cores file that carries anything but cores."""
    path, g = cores
    over = str(tmp_path / "learned.nx")
    cores_file(pkg, micro_path, path, over)
    e = E.HybridEngine.load(over, max_context=64)
    assert "18 live cores" in e.describe()
    ids = g["ids"].tolist()
    rows = [e.feed(ids[:8])] + [e.feed([t]) for t in ids[8:]]
    assert np.abs(np.stack(rows) - g["logits"]).max() < TOL
    key_over, key_plain = e.state_key(), E.HybridEngine.load(micro_path, max_context=8).state_key()
    assert key_over != key_plain                         # a context computed with the cores is kept apart from one without
    e.close()
    bad = str(tmp_path / "stale.nx")
    cores_file(pkg, micro_path, path, bad, base_sha="0" * 64)
    with pytest.raises(E.EngineError, match="learned on a different"):
        E.HybridEngine.load(bad)
    nested = str(tmp_path / "nested.nx")
    cores_file(pkg, over, path, nested)
    with pytest.raises(E.EngineError, match="itself a cores file"):
        E.HybridEngine.load(nested)
