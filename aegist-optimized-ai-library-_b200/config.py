"""Model configuration of the hybrid-MoE brain, as stored in an .nx header's "config" object.

Mirrors the reference's `HybridConfig` (aegist/hybrid.py:46-114) for the keys the decode path
reads (the Rust engine's `HConfig::from_header`, aegist_rs/src/hybrid.rs:53-90). Keys that belong
to the second language core (hyper-connections, PLE, sparse indexer, FP8 experts) are kept at their
"off" defaults so that a header written here loads in the reference unchanged.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field

ARCH = "hybrid-moe"


@dataclass
class HybridConfig:
    arch: str = ARCH
    vocab_size: int = 248320
    d_model: int = 2048
    n_layers: int = 40
    layer_types: list = field(default_factory=lambda: (["delta"] * 3 + ["attn"]) * 10)
    n_heads: int = 16
    n_kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 10_000_000.0
    lin_k_heads: int = 16
    lin_v_heads: int = 32
    lin_k_dim: int = 128
    lin_v_dim: int = 128
    conv_kernel: int = 4
    n_experts: int = 256
    experts_active: int = 8
    expert_hidden: int = 512
    shared_hidden: int = 512
    expert_group: int = 64
    norm_eps: float = 1e-6
    max_seq_len: int = 262144
    tie_embeddings: bool = False
    core_grid: tuple = (8, 64)
    core_rank: int = 64
    cores_active: int = 2
    core_aux_coef: float = 0.01
    core_rows_max: int = 85
    core_seed: int = 0
    hc_count: int = 1
    hc_lowrank: int = 0
    ple_layers: list = field(default_factory=list)
    ple_dim: int = 0
    ple_conv_kernel: int = 4
    ngram_size: int = 3
    heads_per_ngram: int = 8
    ngram_vocab_base: int = 20_000_000
    ngram_divisor: int = 128
    ngram_seed: int = 1234
    eos_id: int = 248044
    idx_heads: int = 0
    idx_head_dim: int = 128
    idx_budget: int = 2048
    idx_ratio: int = 4
    out_gate: str = "silu"
    expert_format: str = "q4"

    # --- derived sizes -----------------------------------------------------------------
    @property
    def n_cores(self) -> int:
        return self.core_grid[0] * self.core_grid[1]

    @property
    def conv_dim(self) -> int:
        return 2 * self.lin_k_heads * self.lin_k_dim + self.lin_v_heads * self.lin_v_dim

    @property
    def value_dim(self) -> int:
        return self.lin_v_heads * self.lin_v_dim

    @property
    def n_attn(self) -> int:
        return sum(t == "attn" for t in self.layer_types)

    @property
    def n_delta(self) -> int:
        return self.n_layers - self.n_attn

    def expert_sections(self) -> list:
        """(name, shape, bytes per element) of one expert's packed row, in file order
        (aegist/hybrid.py:472-480; the Rust twin is `ExpertLayout`, aegist_rs/src/hybrid.rs:138-161)."""
        I, D, G = self.expert_hidden, self.d_model, self.expert_group
        return [("gu_q", (2 * I, D // 2), 1), ("gu_s", (2 * I, D // G), 2), ("gu_m", (2 * I, D // G), 2),
                ("dn_q", (D, I // 2), 1), ("dn_s", (D, I // G), 2), ("dn_m", (D, I // G), 2)]

    @property
    def expert_bytes(self) -> int:
        n = sum(s[0] * s[1] * b for _, s, b in self.expert_sections())
        return -(-n // 64) * 64

    def to_dict(self) -> dict:
        d = asdict(self)
        d["core_grid"] = list(self.core_grid)
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "HybridConfig":
        d = dict(d)
        if "core_grid" in d:
            d["core_grid"] = tuple(d["core_grid"])
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    # --- the named workloads --------------------------------------------------------------
    @classmethod
    def micro(cls) -> "HybridConfig":
        """A brain small enough to commit as a test fixture; every kernel family is exercised."""
        return cls(vocab_size=512, d_model=128, n_layers=4, layer_types=["delta", "delta", "delta", "attn"],
                   n_heads=4, n_kv_heads=1, head_dim=64, rotary_dim=16, lin_k_heads=2, lin_v_heads=4,
                   lin_k_dim=64, lin_v_dim=64, n_experts=16, experts_active=8, expert_hidden=64,
                   shared_hidden=64, max_seq_len=4096, eos_id=0)

    @classmethod
    def tiny(cls) -> "HybridConfig":
        """The CPU-runnable end-to-end case: 4 layers, hidden 512, vocab 32768, 64 experts top-8."""
        return cls(vocab_size=32768, d_model=512, n_layers=4, layer_types=["delta", "delta", "delta", "attn"],
                   n_heads=4, n_kv_heads=1, head_dim=128, rotary_dim=32, lin_k_heads=4, lin_v_heads=8,
                   lin_k_dim=64, lin_v_dim=64, n_experts=64, experts_active=8, expert_hidden=128,
                   shared_hidden=128, max_seq_len=4096, eos_id=0)

    @classmethod
    def full(cls, n_layers: int = 40) -> "HybridConfig":
        """The 35B-A3B-shaped model the throughput metric is quoted on (vocab 151936)."""
        return cls(vocab_size=151936, n_layers=n_layers,
                   layer_types=[("attn" if i % 4 == 3 else "delta") for i in range(n_layers)], eos_id=0)
