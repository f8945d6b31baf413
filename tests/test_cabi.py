"""The C-ABI library: it builds, loads, and exports every symbol include/b200moe.h declares.
No compute is called here (that needs a GPU); opening an engine without one must fail loudly."""
import ctypes
import os
import re

import pytest


@pytest.fixture(scope="module")
def E(pkg):
    import importlib
    return importlib.import_module("b200moe.engine")


def declared_symbols():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(E):
    lib = E.load_library()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(E.SYMBOLS) == names          # the Python binding covers the whole header


def test_no_cpu_fallback(E, micro_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(E.EngineError, match="no CUDA device"):
        E.HybridEngine.load(micro_path)


def test_sampler_and_verify_need_no_gpu(E, micro_path):
    import numpy as np
    from oracle import hybrid_oracle as O
    logits = np.linspace(-2, 2, 50).astype(np.float32)
    assert E.sample(logits, 0.0, 1.0, 10, E.Rng(0)) == 49
    for s in range(20):
        assert E.sample(logits, 0.9, 0.9, 10, E.Rng(s)) == O.sample(logits, 0.9, 0.9, 10, O.Rng(s))
    assert E.verify_file(micro_path) == {"base": True, "engine": True, "cores": True}


def test_cores_file_is_read_over_its_base(E, pkg, micro_path, golden_dir, tmp_path):
    """The .nx reader opens a cores file (aegist_rs/src/nx.rs:82-110) as its base with the cores laid over it, checks every
    group's hash where it is recorded, and refuses a changed base or a cores file over a cores file. No GPU needed."""
    from conftest import cores_file
    src = os.path.join(golden_dir, "micro_cores.nx")
    over = str(tmp_path / "learned.nx")
    cores_file(pkg, micro_path, src, over)
    assert E.verify_file(over) == {"base": True, "engine": True, "cores": True}
    stale = str(tmp_path / "stale.nx")
    cores_file(pkg, micro_path, src, stale, base_sha="0" * 64)
    with pytest.raises(E.EngineError, match="learned on a different"):
        E.verify_file(stale)
    nested = str(tmp_path / "nested.nx")
    cores_file(pkg, over, src, nested)
    with pytest.raises(E.EngineError, match="itself a cores file"):
        E.verify_file(nested)
