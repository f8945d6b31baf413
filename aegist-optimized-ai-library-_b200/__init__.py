"""B200-native decode engine for the hybrid-MoE token loop (gated DeltaNet + gated GQA attention,
256 four-bit experts with 8 routed per token plus a shared expert).

The compute path is a C-ABI shared library of hand-written sm_100a CUDA kernels (`csrc/`, declared
in `include/b200moe.h`); this package is the host-side mirror of the reference's engine interface:

* `engine.HybridEngine` - feed / crop / snapshot / taps / counters, as `trait Lm` has them
  (aegist_rs/src/model.rs:363-427), over the C ABI through ctypes;
* `engine.sample`, `engine.Rng` - the reference's sampler (aegist_rs/src/chat.rs:221-272);
* `nxfile` - the .nx brain file reader / writer (aegist/nx.py);
* `brain` - the int8 / 4-bit quantisers and a seeded synthetic-brain builder;
* `config.HybridConfig` - the model config stored in the .nx header.

The directory name is not a Python identifier; load the package with
`__graft_entry__.load_package()` (it registers it as `b200moe`).
"""
from .config import HybridConfig  # noqa: F401
