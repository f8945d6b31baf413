import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def micro_path():
    return os.path.join(GOLDEN, "micro.nx")


@pytest.fixture(scope="session")
def tiny_path(pkg, tmp_path_factory):
    """The 4-layer hidden-512 vocab-32768 brain of the benchmark spec, rebuilt from seed 0."""
    from b200moe import brain
    path = str(tmp_path_factory.mktemp("tiny") / "tiny.nx")
    brain.write_brain(path, pkg.HybridConfig.tiny(), seed=0)
    return path


def cores_file(pkg, base_path, src_path, out_path, base_sha=None):
    """A cores file (aegist_rs/src/nx.rs:82-110): only the `cores` tensors of `src_path`, laid over `base_path`."""
    from b200moe import nxfile
    from b200moe.nxfile import Bf16, NxFile
    with NxFile(src_path) as src, NxFile(base_path) as base:
        state = {}
        for n in src.names("cores"):
            t = np.array(src.tensor(n))
            state[n] = Bf16(t) if src.info(n)["dtype"] == "bf16" else t
        sha = base_sha or base.header["sha256"]["base"]
        nxfile.save(out_path, state, src.config, extra={"base": {"path": base_path, "sha256": sha}})
