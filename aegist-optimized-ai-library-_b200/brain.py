"""Quantisers and the synthetic-brain builder (host-side tools; torch, any device).

The decode engine reads two weight formats, both produced here exactly as the reference does:

* int8 linears (aegist/model.py:84-89): per output row, scale = max|w| / 127 (at least 1e-8),
  q = round(w / scale) with the fp32 scale, and the scale is then STORED as bf16 `[N, 1]`.
* 4-bit experts (aegist/hybrid.py:426-460): asymmetric, groups of `expert_group` input values,
  w ~= code * scale + min with fp16 scale and min; the min/max fit is followed by three
  least-squares refits, each group keeping whichever fit has the lowest squared error. Two codes per
  byte, the even input index in the LOW nibble. One expert is one contiguous row
  gu_q | gu_s | gu_m | dn_q | dn_s | dn_m (aegist/hybrid.py:472-511).

`random_brain` makes every tensor of a fresh brain from a seed (weights N(0, 0.02), norms and gates
at their initial values, no live cores), one tensor at a time so that the 35B-shaped model can be
built on a GPU without ever holding unquantised experts for more than one layer.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

from .config import HybridConfig
from .nxfile import Bf16, save


# --- quantisers ----------------------------------------------------------------------------

def int8_quantize(weight: torch.Tensor):
    """weight [N, K] -> (q int8 [N, K], scale bf16 [N, 1])."""
    w = weight.float()
    scale = w.abs().amax(1, keepdim=True).clamp(min=1e-8) / 127.0
    return torch.round(w / scale).to(torch.int8), scale.to(torch.bfloat16)


def _q4_fit(x, scale, mn):
    """Codes and squared error of `x` [..., n_groups, group] against a (scale, min) pair, both first
    rounded to what is stored (fp16)."""
    scale, mn = scale.half().float(), mn.half().float()
    div = torch.where(scale > 0, scale, torch.ones_like(scale))
    code = ((x - mn.unsqueeze(-1)) / div.unsqueeze(-1)).round().clamp(0, 15)
    err = (code * scale.unsqueeze(-1) + mn.unsqueeze(-1) - x).pow(2).sum(-1)
    return scale, mn, code, err


def q4_quantize(w: torch.Tensor, group: int, iters: int = 3):
    """w [..., K] -> (packed uint8 [..., K/2], scale f16 [..., K/group], min f16 [..., K/group])."""
    *lead, n = w.shape
    x = w.float().reshape(*lead, n // group, group)
    lo, hi = x.amin(-1), x.amax(-1)
    scale, mn, code, err = _q4_fit(x, (hi - lo) / 15, lo)
    for _ in range(iters):
        c_mean, x_mean = code.mean(-1), x.mean(-1)
        dc = code - c_mean.unsqueeze(-1)
        var = dc.pow(2).mean(-1)
        cov = (dc * (x - x_mean.unsqueeze(-1))).mean(-1)
        s_new = torch.where(var > 0, cov / var.clamp(min=1e-12), scale).clamp(min=0)
        m_new = torch.where(var > 0, x_mean - s_new * c_mean, mn)
        s2, m2, code2, err2 = _q4_fit(x, s_new, m_new)
        better = err2 < err
        scale = torch.where(better, s2, scale)
        mn = torch.where(better, m2, mn)
        code = torch.where(better.unsqueeze(-1), code2, code)
        err = torch.where(better, err2, err)
    code = code.to(torch.uint8).reshape(*lead, n)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), scale.half(), mn.half()


def q4_dequantize(packed, scale, mn, group: int, dtype=torch.float32):
    code = torch.stack([(packed & 0xF).to(dtype), (packed >> 4).to(dtype)], -1).flatten(-2)
    *lead, n = code.shape
    code = code.view(*lead, n // group, group)
    return (code * scale.to(dtype).unsqueeze(-1) + mn.to(dtype).unsqueeze(-1)).reshape(*lead, n)


def pack_experts(gate_up: torch.Tensor, down: torch.Tensor, cfg: HybridConfig) -> torch.Tensor:
    """gate_up [E, 2I, D], down [E, D, I] -> uint8 [E, expert_bytes]."""
    E = gate_up.shape[0]
    parts = [*q4_quantize(gate_up, cfg.expert_group), *q4_quantize(down, cfg.expert_group)]
    rows = torch.cat([p.contiguous().view(torch.uint8).reshape(E, -1) for p in parts], 1)
    assert rows.shape[1] == cfg.expert_bytes
    return rows


def unpack_expert(row: torch.Tensor, cfg: HybridConfig, dtype=torch.float32):
    """One expert's uint8 row -> (gate_up [2I, D], down [D, I])."""
    out, off = {}, 0
    for name, shape, size in cfg.expert_sections():
        nb = shape[0] * shape[1] * size
        out[name] = row[off: off + nb].view(torch.uint8 if size == 1 else torch.float16).view(shape)
        off += nb
    G = cfg.expert_group
    return (q4_dequantize(out["gu_q"], out["gu_s"], out["gu_m"], G, dtype),
            q4_dequantize(out["dn_q"], out["dn_s"], out["dn_m"], G, dtype))


# --- a fresh brain from a seed -----------------------------------------------------------------

def _gen(name: str, seed: int, device) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def normal(name: str, shape, seed: int, device, std: float = 0.02) -> torch.Tensor:
    """fp32 N(0, std) keyed by (seed, tensor name), rounded through bf16 like a stored checkpoint."""
    x = torch.randn(tuple(shape), generator=_gen(name, seed, device), device=device, dtype=torch.float32) * std
    return x.to(torch.bfloat16)


def router_popularity_bias(cfg: HybridConfig, layer: int, seed: int, alpha: float) -> torch.Tensor:
    """A per-expert additive router bias that makes expert popularity roughly Zipf(alpha): expert of
    popularity rank r (1 = most popular) gets alpha * (-ln r); the rank order is a seeded permutation
    per layer. The router has no bias tensor in the brain file, so the engine takes it through
    `set_router_bias` and the oracle adds it to the router output."""
    g = torch.Generator().manual_seed(seed * 7919 + layer)
    rank = torch.randperm(cfg.n_experts, generator=g).float() + 1.0
    return -alpha * rank.log()


def linear_names(cfg: HybridConfig, i: int) -> list:
    """(prefix, N, K) of layer i's int8 linears (aegist/hybrid.py:950-966)."""
    D = cfg.d_model
    p = f"blocks.{i}."
    if cfg.layer_types[i] == "attn":
        H, KV, HD = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        mix = [("mixer.q", 2 * H * HD, D), ("mixer.k", KV * HD, D), ("mixer.v", KV * HD, D), ("mixer.o", D, H * HD)]
    else:
        mix = [("mixer.in_qkv", cfg.conv_dim, D), ("mixer.in_z", cfg.value_dim, D), ("mixer.out", D, cfg.value_dim)]
    sh = cfg.shared_hidden
    return [(p + n, a, b) for n, a, b in mix + [("moe.shared.gate", sh, D), ("moe.shared.up", sh, D),
                                                  ("moe.shared.down", D, sh)]]


def vector_init(name: str, shape, seed: int, device, vary: bool) -> torch.Tensor:
    """Initial value of a 1-D parameter: zeros for the zero-centred norms and A_log, ones for the
    gated norm and dt_bias (aegist/hybrid.py:125,140,382-383). With `vary`, seeded noise is added so
    that a test brain exercises every one of them."""
    ones = name.endswith(("mixer.norm.weight", "dt_bias"))
    base = torch.ones(tuple(shape), device=device) if ones else torch.zeros(tuple(shape), device=device)
    if vary:
        std = 0.5 if name.endswith(("A_log", "dt_bias")) else 0.1
        base = base + normal(name, shape, seed, device, std).float()
    return base.to(torch.bfloat16)


def random_brain(cfg: HybridConfig, seed: int = 0, device="cpu", expert_chunk: int = 32, vary_1d: bool = False):
    """Yield (name, dtype name, tensor) for every tensor of a fresh brain, already in stored form
    (bf16 / int8 / fp16-in-uint8 rows). Tensor names follow the reference's state dict
    (aegist_rs/src/hybrid.rs:546-602)."""
    D = cfg.d_model
    bf = lambda t: ("bf16", t.to(torch.bfloat16))
    vec = lambda name, n: ("bf16", vector_init(name, (n,), seed, device, vary_1d))

    def qlin(prefix, n, k):
        q, s = int8_quantize(normal(prefix + ".weight", (n, k), seed, device))
        yield prefix + ".qweight", "i8", q
        yield prefix + ".scale", "bf16", s

    yield ("embed.weight", *bf(normal("embed.weight", (cfg.vocab_size, D), seed, device)))
    yield ("norm.weight", *vec("norm.weight", D))
    # the head is the largest tensor: quantise it in row blocks
    yield from qlin("lm_head", cfg.vocab_size, D)
    for i in range(cfg.n_layers):
        p = f"blocks.{i}."
        yield (p + "norm1.weight", *vec(p + "norm1.weight", D))
        yield (p + "norm2.weight", *vec(p + "norm2.weight", D))
        if cfg.layer_types[i] == "attn":
            yield (p + "mixer.q_norm.weight", *vec(p + "mixer.q_norm.weight", cfg.head_dim))
            yield (p + "mixer.k_norm.weight", *vec(p + "mixer.k_norm.weight", cfg.head_dim))
        else:
            hv = cfg.lin_v_heads
            yield (p + "mixer.in_a.weight", *bf(normal(p + "mixer.in_a.weight", (hv, D), seed, device)))
            yield (p + "mixer.in_b.weight", *bf(normal(p + "mixer.in_b.weight", (hv, D), seed, device)))
            yield (p + "mixer.conv", *bf(normal(p + "mixer.conv", (cfg.conv_dim, cfg.conv_kernel), seed, device)))
            yield (p + "mixer.A_log", *vec(p + "mixer.A_log", hv))
            yield (p + "mixer.dt_bias", *vec(p + "mixer.dt_bias", hv))
            yield (p + "mixer.norm.weight", *vec(p + "mixer.norm.weight", cfg.lin_v_dim))
        for prefix, n, k in linear_names(cfg, i):
            yield from qlin(prefix, n, k)
        yield (p + "moe.router.weight", *bf(normal(p + "moe.router.weight", (cfg.n_experts, D), seed, device)))
        yield (p + "moe.shared_gate.weight", *bf(normal(p + "moe.shared_gate.weight", (1, D), seed, device)))
        rows = []
        I = cfg.expert_hidden
        for s in range(0, cfg.n_experts, expert_chunk):
            n = min(expert_chunk, cfg.n_experts - s)
            gu = normal(f"{p}moe.experts.gate_up.{s}", (n, 2 * I, D), seed, device)
            dn = normal(f"{p}moe.experts.down.{s}", (n, D, I), seed, device)
            rows.append(pack_experts(gu, dn, cfg))
            del gu, dn
        yield p + "moe.experts.q4", "u8", torch.cat(rows)
        n1, n2 = cfg.core_grid
        yield (p + "engine.key1.weight", *bf(normal(p + "engine.key1.weight", (n1, D), seed, device, D ** -0.5)))
        yield (p + "engine.key2.weight", *bf(normal(p + "engine.key2.weight", (n2, D), seed, device, D ** -0.5)))
        r = cfg.core_rank
        yield p + "cores.ids", "i64", torch.zeros(0, dtype=torch.int64, device=device)
        yield (p + "cores.gate", *bf(torch.zeros(0, D, r, device=device)))
        yield (p + "cores.up", *bf(torch.zeros(0, D, r, device=device)))
        yield (p + "cores.down", *bf(torch.zeros(0, r, D, device=device)))


def to_numpy(dtype_name: str, t: torch.Tensor):
    t = t.detach().contiguous().cpu()
    if dtype_name == "bf16":
        return Bf16(t.view(torch.int16).numpy().view(np.uint16))
    return t.numpy()


def write_brain(path: str, cfg: HybridConfig, seed: int = 0, device="cpu", vary_1d: bool = False) -> dict:
    """Build a fresh brain and store it as an .nx file the reference can load."""
    state = {name: to_numpy(dt, t) for name, dt, t in random_brain(cfg, seed, device, vary_1d=vary_1d)}
    return save(path, state, cfg.to_dict(), extra={"quant": "int8", "dtype": "bf16",
                                                   "experts": f"q4a-g{cfg.expert_group}", "seed": seed})
