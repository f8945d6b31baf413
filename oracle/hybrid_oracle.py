"""CPU oracle for the hybrid-MoE decode path.

TEST INFRASTRUCTURE, NOT PRODUCT CODE. A plain numpy (fp32) restatement of the reference's own
implementation of the path, aegist/hybrid.py + aegist/model.py, with each function citing the
reference lines it follows. Only the test-suite, the smoke check and the benchmark's CPU-baseline leg
may import it; the engine never does.

Pinned: `tests/test_oracle_golden.py` checks this file against outputs of the unmodified reference
(logits, router picks and weights, greedy tokens, tapped hidden states, snapshot/crop behaviour and
the per-op cases) stored under `tests/golden/` by `tests/golden/make_golden.py`.

Everything is fp32 with fp32 accumulation, as in the reference's own parity runs (`model.float()`
and an fp32 cache, tests/test_hybrid_rust.py:96-116). `kv_dtype="bf16"` additionally rounds keys and
values to bfloat16 when they are stored, which is what the reference's CUDA engine always does
(aegist_rs/kernels/hybrid.cu:113-114).
"""
from __future__ import annotations

import json
import math
import mmap
import struct

import numpy as np

F32 = np.float32


# --- number formats ----------------------------------------------------------------------

def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to the nearest bfloat16 (ties to even), returned as fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return (((u + r) >> 16) << 16).astype(np.uint32).view(np.float32)


# --- the brain file (aegist/nx.py:146-202) ---------------------------------------------------

_NP = {"bf16": np.uint16, "f16": np.float16, "f32": np.float32, "i8": np.int8, "i64": np.int64, "u8": np.uint8}


class Brain:
    """An opened .nx file: header, config and tensors (bf16 widened to fp32 on access)."""

    def __init__(self, path: str):
        self._f = open(path, "rb")
        head = self._f.read(20)
        if head[:8] not in (b"AEGISTNX", b"AUGISTNX"):
            raise ValueError(f"{path} is not an .nx file")
        _, hlen = struct.unpack("<IQ", head[8:20])
        self.header = json.loads(self._f.read(hlen).decode("utf-8"))
        self.data_start = 20 + hlen + (-(20 + hlen)) % 64
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.cfg = dict(self.header["config"])
        self._cache = {}

    def raw(self, name: str) -> np.ndarray:
        m = self.header["tensors"][name]
        dt = np.dtype(_NP[m["dtype"]])
        n = m["nbytes"] // dt.itemsize
        if n == 0:
            return np.zeros(m["shape"], dtype=dt)
        return np.frombuffer(self._mm, dtype=dt, count=n, offset=self.data_start + m["offset"]).reshape(m["shape"])

    def f32(self, name: str) -> np.ndarray:
        if name not in self._cache:
            t = self.raw(name)
            self._cache[name] = bf16_to_f32(t) if self.header["tensors"][name]["dtype"] == "bf16" else t.astype(F32)
        return self._cache[name]

    def has(self, name: str) -> bool:
        return name in self.header["tensors"]


class DictBrain:
    """The same interface over tensors held in memory: {name: (dtype name, numpy array)}; bf16
    tensors are uint16 bit patterns."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg, self._t, self._cache = dict(cfg), tensors, {}
        self.header = {"config": self.cfg}

    def raw(self, name):
        return self._t[name][1]

    def f32(self, name):
        if name not in self._cache:
            dt, t = self._t[name]
            self._cache[name] = bf16_to_f32(t) if dt == "bf16" else t.astype(F32)
        return self._cache[name]

    def has(self, name):
        return name in self._t


# --- small pieces -----------------------------------------------------------------------------

def sigmoid(x):
    return (F32(1) / (F32(1) + np.exp(-x, dtype=F32))).astype(F32)


def silu(x):
    return (x * sigmoid(x)).astype(F32)


def softplus(x):
    """F.softplus with its default threshold 20 (aegist/hybrid.py:404; hybrid.cu:195)."""
    x = x.astype(F32)
    return np.where(x > 20, x, np.log1p(np.exp(np.minimum(x, F32(20)), dtype=F32), dtype=F32)).astype(F32)


def znorm(x, w, eps):
    """Zero-centred RMSNorm, (1 + w) scaling (aegist/hybrid.py:119-130)."""
    x = x.astype(F32)
    r = F32(1) / np.sqrt((x * x).mean(-1, keepdims=True, dtype=F32) + F32(eps), dtype=F32)
    return (x * r * (F32(1) + w)).astype(F32)


def gated_norm(x, z, w, eps):
    """RMSNorm with a plain weight, times SiLU(z) (aegist/hybrid.py:133-147)."""
    x = x.astype(F32)
    r = F32(1) / np.sqrt((x * x).mean(-1, keepdims=True, dtype=F32) + F32(eps), dtype=F32)
    return ((w * (x * r)) * silu(z.astype(F32))).astype(F32)


def l2norm(x, eps=1e-6):
    """aegist/hybrid.py:314-315: the eps is inside the square root, on the SUM."""
    return (x * (F32(1) / np.sqrt((x * x).sum(-1, keepdims=True, dtype=F32) + F32(eps), dtype=F32))).astype(F32)


def rope_tables(rotary_dim: int, theta: float, length: int):
    """aegist/hybrid.py:152-157. fp32 angles = position * (1 / theta^(2j/rd)); columns repeated twice.
    The power is taken in double precision and rounded to fp32, which reproduces torch's fp32 `**`
    bit for bit on every case tried (numpy's fp32 power is 1 ulp off for a few j, and 1 ulp of the
    inverse frequency is 2e-4 radians at position 8000)."""
    ar = np.arange(0, rotary_dim, 2, dtype=F32) / F32(rotary_dim)
    inv = (F32(1) / np.power(np.float64(F32(theta)), ar.astype(np.float64)).astype(F32)).astype(F32)
    f = np.outer(np.arange(length, dtype=F32), inv).astype(F32)
    emb = np.concatenate([f, f], -1)
    return np.cos(emb, dtype=F32), np.sin(emb, dtype=F32)


def apply_partial_rope(x, cos, sin):
    """Rotate-half on the first rd dims of each head (aegist/hybrid.py:160-166). x [..., T, hd]."""
    rd = cos.shape[-1]
    xr, xp = x[..., :rd], x[..., rd:]
    h = rd // 2
    rot = np.concatenate([-xr[..., h:], xr[..., :h]], -1)
    return np.concatenate([xr * cos + rot * sin, xp], -1).astype(F32)


def q4_dequantize(packed, scale, mn, group):
    """aegist/hybrid.py:463-469: even index in the low nibble; w = code * scale + min."""
    lo = (packed & 0xF).astype(F32)
    hi = (packed >> 4).astype(F32)
    code = np.stack([lo, hi], -1).reshape(*packed.shape[:-1], -1)
    n = code.shape[-1]
    code = code.reshape(*code.shape[:-1], n // group, group)
    return (code * scale.astype(F32)[..., None] + mn.astype(F32)[..., None]).reshape(*packed.shape[:-1], n)


def expert_sections(cfg):
    I, D, G = cfg["expert_hidden"], cfg["d_model"], cfg["expert_group"]
    return [("gu_q", (2 * I, D // 2), np.uint8), ("gu_s", (2 * I, D // G), np.float16),
            ("gu_m", (2 * I, D // G), np.float16), ("dn_q", (D, I // 2), np.uint8),
            ("dn_s", (D, I // G), np.float16), ("dn_m", (D, I // G), np.float16)]


def unpack_expert(row: np.ndarray, cfg):
    """One expert's uint8 row -> (gate_up [2I, D], down [D, I]) fp32 (aegist/hybrid.py:514-526)."""
    out, off = {}, 0
    for name, shape, dt in expert_sections(cfg):
        nb = shape[0] * shape[1] * np.dtype(dt).itemsize
        out[name] = row[off: off + nb].view(dt).reshape(shape)
        off += nb
    G = cfg["expert_group"]
    return (q4_dequantize(out["gu_q"], out["gu_s"], out["gu_m"], G),
            q4_dequantize(out["dn_q"], out["dn_s"], out["dn_m"], G))


def route(logits, k):
    """aegist/hybrid.py:641-645: fp32 softmax, the k largest in descending order (ties to the lower
    index, as the reference's CUDA router does, hybrid.cu:30-66), weights renormalised over the picks."""
    z = logits.astype(F32)
    z = z - z.max(-1, keepdims=True)
    e = np.exp(z, dtype=F32)
    p = (e / e.sum(-1, keepdims=True, dtype=F32)).astype(F32)
    idx = np.argsort(-p, axis=-1, kind="stable")[..., :k]
    top = np.take_along_axis(p, idx, -1)
    return idx.astype(np.int32), (top / top.sum(-1, keepdims=True, dtype=F32)).astype(F32), p


def delta_rule_step(q, k, v, g, beta, state):
    """One token (aegist/hybrid.py:318-324). q, k [B,H,dk]; v [B,H,dv]; g, beta [B,H];
    state [B,H,dk,dv] fp32, updated in place. Decay first, then the delta update, then the readout."""
    state *= np.exp(g, dtype=F32)[..., None, None]
    kv = (state * k[..., None]).sum(-2, dtype=F32)
    delta = (v - kv) * beta[..., None]
    state += k[..., None] * delta[..., None, :]
    return (state * q[..., None]).sum(-2, dtype=F32)


def _solve_unit_lower(a, b):
    """X with (I + strictly_lower(a)) X = b; a [..., n, n], b [..., n, m]."""
    x = np.array(b, dtype=F32, copy=True)
    n = a.shape[-1]
    for i in range(1, n):
        x[..., i, :] -= np.einsum("...j,...jm->...m", a[..., i, :i], x[..., :i, :]).astype(F32)
    return x


def delta_rule_chunked(q, k, v, g, beta, state, chunk=64):
    """The same recurrence over T tokens in WY form (aegist/hybrid.py:327-361). q, k [B,H,T,dk];
    v [B,H,T,dv]; g, beta [B,H,T]. Returns (out [B,H,T,dv], final state)."""
    B, H, T, dk = k.shape
    dv = v.shape[-1]
    pad = (chunk - T % chunk) % chunk
    if pad:
        q, k, v = (np.pad(t, ((0, 0), (0, 0), (0, pad), (0, 0))) for t in (q, k, v))
        g, beta = (np.pad(t, ((0, 0), (0, 0), (0, pad))) for t in (g, beta))
    n = (T + pad) // chunk
    kb = (k * beta[..., None]).reshape(B, H, n, chunk, dk).astype(F32)
    vb = (v * beta[..., None]).reshape(B, H, n, chunk, dv).astype(F32)
    q, k = q.reshape(B, H, n, chunk, dk), k.reshape(B, H, n, chunk, dk)
    cum = np.cumsum(g.reshape(B, H, n, chunk), -1, dtype=F32)
    diff = cum[..., :, None] - cum[..., None, :]
    lower = np.tril(np.ones((chunk, chunk), dtype=bool))
    decay = np.where(lower, np.exp(np.where(lower, diff, 0), dtype=F32), F32(0)).astype(F32)
    system = (kb @ np.swapaxes(k, -1, -2)) * decay
    u = _solve_unit_lower(system, vb)
    w = _solve_unit_lower(system, kb * np.exp(cum, dtype=F32)[..., None])
    intra = (q @ np.swapaxes(k, -1, -2)) * decay
    q_dec = q * np.exp(cum, dtype=F32)[..., None]
    k_dec = k * np.exp(cum[..., -1:] - cum, dtype=F32)[..., None]
    chunk_decay = np.exp(cum[..., -1], dtype=F32)[..., None, None]
    S = np.zeros((B, H, dk, dv), dtype=F32) if state is None else state.astype(F32)
    outs = []
    for i in range(n):
        v_new = u[:, :, i] - w[:, :, i] @ S
        outs.append(q_dec[:, :, i] @ S + intra[:, :, i] @ v_new)
        S = S * chunk_decay[:, :, i] + np.swapaxes(k_dec[:, :, i], -1, -2) @ v_new
    out = np.stack(outs, 2).reshape(B, H, n * chunk, dv)[:, :, :T]
    return out.astype(F32), S.astype(F32)


# --- cache (aegist/hybrid.py:171-260) --------------------------------------------------------

class Cache:
    """KV for the attention blocks, conv taps + fp32 state for the DeltaNet blocks, and snapshots.
    `keep` is how many snapshots survive: the Python reference keeps 4 (hybrid.py:225), its CUDA
    engine 2 (aegist_rs/src/hybrid.rs:442); the replacement engine follows the latter."""

    def __init__(self, cfg, batch, max_len, kv_dtype="f32", keep=2):
        self.cfg, self.batch, self.max_len, self.kv_dtype, self.keep = cfg, batch, max_len, kv_dtype, keep
        types = cfg["layer_types"]
        self.attn_layers = [i for i, t in enumerate(types) if t == "attn"]
        self.delta_layers = [i for i, t in enumerate(types) if t == "delta"]
        self.slot = {i: j for j, i in enumerate(self.attn_layers)}
        self.slot.update({i: j for j, i in enumerate(self.delta_layers)})
        C = 2 * cfg["lin_k_heads"] * cfg["lin_k_dim"] + cfg["lin_v_heads"] * cfg["lin_v_dim"]
        self.conv = np.zeros((len(self.delta_layers), batch, C, cfg["conv_kernel"] - 1), dtype=F32)
        self.state = np.zeros((len(self.delta_layers), batch, cfg["lin_v_heads"], cfg["lin_k_dim"],
                               cfg["lin_v_dim"]), dtype=F32)
        shape = (len(self.attn_layers), batch, cfg["n_kv_heads"], max_len, cfg["head_dim"])
        self.k = np.zeros(shape, dtype=F32)
        self.v = np.zeros(shape, dtype=F32)
        self.length = 0
        self.snapshots = {}

    def store(self, x):
        return round_bf16(x) if self.kv_dtype == "bf16" else x

    def snapshot(self):
        self.snapshots[self.length] = (self.conv.copy(), self.state.copy())
        for old in sorted(self.snapshots)[:-self.keep]:
            del self.snapshots[old]

    def crop(self, n):
        if n >= self.length:
            return self.length
        ok = [p for p in self.snapshots if p <= n]
        if not ok:
            self.conv[:] = 0
            self.state[:] = 0
            self.length = 0
            self.snapshots.clear()
            return 0
        p = max(ok)
        self.conv[:], self.state[:] = self.snapshots[p]
        self.length = p
        for later in [s for s in self.snapshots if s > p]:
            del self.snapshots[later]
        return p


# --- the model -------------------------------------------------------------------------------

class HybridOracle:
    """`forward(ids [B,T], cache)` -> logits of the last position [B, V] (HybridLM.forward with
    last_only=True, aegist/hybrid.py:896-924). `hold_weights` keeps dequantised int8 linears after
    first use; the reference re-materialises them on every call (aegist/model.py:92-93), which
    changes the time but not one bit of the result."""

    def __init__(self, brain, hold_weights=True):
        self.b, self.cfg = brain, brain.cfg
        self.hold = hold_weights
        self._w = {}
        c = self.cfg
        self.eps = c["norm_eps"]
        self._rope = None
        self.last_route = {}      # layer -> (idx [N,k], weights [N,k]) of the latest forward
        self.last_hidden = {}     # layer -> x after that layer, last position [B, D]
        self.router_bias = {}     # layer -> [E] added to the router output (expert-popularity shaping)
        n_cores = int(c["core_grid"][0]) * int(c["core_grid"][1])
        self.core_counts = np.zeros((c["n_layers"], n_cores), dtype=np.int64)   # switch-ons per core (HybridLM.core_usage)
        self.last_cores = {}      # layer -> (ids [N,k], weights [N,k]) of the latest forward

    # int8 linear: y = x @ (q * scale)^T, the product q * scale rounded to fp32 first (model.py:92-93)
    def qlinear(self, x, prefix):
        if prefix in self._w:
            w = self._w[prefix]
        else:
            w = self.b.raw(prefix + ".qweight").astype(F32) * self.b.f32(prefix + ".scale")
            if self.hold:
                self._w[prefix] = w
        return (x.astype(F32) @ w.T).astype(F32)

    def rope(self, length):
        if self._rope is None or self._rope[0].shape[0] < length:
            self._rope = rope_tables(self.cfg["rotary_dim"], self.cfg["rope_theta"], max(length, 4096))
        return self._rope

    def new_cache(self, batch, max_len, kv_dtype="f32", keep=2):
        return Cache(self.cfg, batch, max_len, kv_dtype, keep)

    # aegist/hybrid.py:280-311
    def attention(self, i, h, cache, cos, sin):
        c, p = self.cfg, f"blocks.{i}.mixer."
        B, T, _ = h.shape
        H, KV, HD = c["n_heads"], c["n_kv_heads"], c["head_dim"]
        slot = cache.slot[i]
        qg = self.qlinear(h, p + "q").reshape(B, T, H, 2 * HD)
        q, gate = qg[..., :HD], qg[..., HD:].reshape(B, T, H * HD)
        q = znorm(q, self.b.f32(p + "q_norm.weight"), self.eps).transpose(0, 2, 1, 3)
        k = znorm(self.qlinear(h, p + "k").reshape(B, T, KV, HD), self.b.f32(p + "k_norm.weight"), self.eps)
        k = k.transpose(0, 2, 1, 3)
        v = self.qlinear(h, p + "v").reshape(B, T, KV, HD).transpose(0, 2, 1, 3)
        pos = cache.length
        cs, sn = cos[pos: pos + T], sin[pos: pos + T]
        q, k = apply_partial_rope(q, cs, sn), apply_partial_rope(k, cs, sn)
        cache.k[slot, :, :, pos: pos + T] = cache.store(k)
        cache.v[slot, :, :, pos: pos + T] = cache.store(v)
        kk, vv = cache.k[slot, :, :, : pos + T], cache.v[slot, :, :, : pos + T]
        g = H // KV
        qf = q.reshape(B, KV, g, T, HD)
        s = np.einsum("bkgtd,bkld->bkgtl", qf, kk).astype(F32) * F32(1.0 / math.sqrt(HD))
        mask = np.arange(pos + T)[None, :] <= (pos + np.arange(T))[:, None]
        s = np.where(mask, s, F32(-np.inf))
        s = s - s.max(-1, keepdims=True)
        e = np.exp(s, dtype=F32)
        a = e / e.sum(-1, keepdims=True, dtype=F32)
        y = np.einsum("bkgtl,bkld->bkgtd", a, vv).astype(F32).reshape(B, H, T, HD)
        y = y.transpose(0, 2, 1, 3).reshape(B, T, H * HD) * sigmoid(gate)
        return self.qlinear(y, p + "o")

    # aegist/hybrid.py:388-421
    def deltanet(self, i, h, cache):
        c, p = self.cfg, f"blocks.{i}.mixer."
        B, T, _ = h.shape
        hk, hv, dk, dv, K = c["lin_k_heads"], c["lin_v_heads"], c["lin_k_dim"], c["lin_v_dim"], c["conv_kernel"]
        key_dim, value_dim = hk * dk, hv * dv
        slot = cache.slot[i]
        qkv = self.qlinear(h, p + "in_qkv").transpose(0, 2, 1)           # [B, C, T]
        z = self.qlinear(h, p + "in_z").reshape(B, T, hv, dv)
        b = (h @ self.b.f32(p + "in_b.weight").T).astype(F32)
        a = (h @ self.b.f32(p + "in_a.weight").T).astype(F32)
        w = self.b.f32(p + "conv")                                          # [C, K]
        xp = np.concatenate([cache.conv[slot], qkv], -1)                    # [B, C, K-1+T]
        cache.conv[slot] = xp[..., -(K - 1):]
        y = np.zeros((B, qkv.shape[1], T), dtype=F32)
        for j in range(K):                                                  # depthwise causal conv
            y += xp[..., j: j + T] * w[None, :, j, None]
        qkv = silu(y).transpose(0, 2, 1)                                    # [B, T, C]
        q = qkv[..., :key_dim].reshape(B, T, hk, dk)
        k = qkv[..., key_dim: 2 * key_dim].reshape(B, T, hk, dk)
        v = qkv[..., 2 * key_dim:].reshape(B, T, hv, dv)
        beta = sigmoid(b)
        g = -np.exp(self.b.f32(p + "A_log"), dtype=F32) * softplus(a + self.b.f32(p + "dt_bias"))
        r = hv // hk
        if r > 1:
            q, k = np.repeat(q, r, 2), np.repeat(k, r, 2)
        q, k, v = (t.transpose(0, 2, 1, 3).astype(F32) for t in (q, k, v))   # [B, hv, T, d]
        beta, g = beta.transpose(0, 2, 1).astype(F32), g.transpose(0, 2, 1).astype(F32)
        q, k = l2norm(q), l2norm(k)
        q = (q * F32(dk ** -0.5)).astype(F32)
        if T == 1 and cache.length > 0:
            out = delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], g[:, :, 0], beta[:, :, 0], cache.state[slot])
            out = out[:, :, None]
        else:
            init = cache.state[slot] if cache.length > 0 else None
            out, S = delta_rule_chunked(q, k, v, g, beta, init)
            cache.state[slot] = S
        out = out.transpose(0, 2, 1, 3)                                     # [B, T, hv, dv]
        out = gated_norm(out, z, self.b.f32(p + "norm.weight"), self.eps).reshape(B, T, value_dim)
        return self.qlinear(out, p + "out")

    # aegist/hybrid.py:608-625 and 641-652
    def moe(self, i, hf):
        c, p = self.cfg, f"blocks.{i}.moe."
        logits = (hf @ self.b.f32(p + "router.weight").T).astype(F32)
        if i in self.router_bias:
            logits = logits + self.router_bias[i].astype(F32)
        idx, wts, _ = route(logits, c["experts_active"])
        self.last_route[i] = (idx, wts)
        out = np.zeros_like(hf)
        flat = idx.reshape(-1)
        order = np.argsort(flat, kind="stable")
        tok = np.repeat(np.arange(hf.shape[0]), idx.shape[1])[order]
        ww = wts.reshape(-1)[order]
        masters = self.b.raw(p + "experts.q4")
        for e in np.unique(flat):
            sel = flat[order] == e
            t, wt = tok[sel], ww[sel]
            gu, dn = unpack_expert(masters[e], c)
            a = (hf[t] @ gu.T).astype(F32)
            I = c["expert_hidden"]
            y = ((silu(a[:, :I]) * a[:, I:]).astype(F32) @ dn.T).astype(F32) * wt[:, None]
            np.add.at(out, t, y)
        sh = self.qlinear((silu(self.qlinear(hf, p + "shared.gate")) * self.qlinear(hf, p + "shared.up")).astype(F32),
                          p + "shared.down")
        sg = sigmoid((hf @ self.b.f32(p + "shared_gate.weight").T).astype(F32))
        return (out + sg * sh).astype(F32)

    # CoreEngine.forward (aegist/model.py:214-224): product-key routing. Two score tables of n1 and n2 entries address
    # n1 * n2 cores; the k best of each, their k1 * k2 sums, the k best sums (ties to the earlier candidate), softmax.
    def core_route(self, i, hf):
        c, p = self.cfg, f"blocks.{i}.engine."
        n1, n2 = int(c["core_grid"][0]), int(c["core_grid"][1])
        k = int(c["cores_active"])
        s1 = (hf @ self.b.f32(p + "key1.weight").T).astype(F32)
        s2 = (hf @ self.b.f32(p + "key2.weight").T).astype(F32)
        k1, k2 = min(k, n1), min(k, n2)
        i1 = np.argsort(-s1, -1, kind="stable")[:, :k1]
        i2 = np.argsort(-s2, -1, kind="stable")[:, :k2]
        v1, v2 = np.take_along_axis(s1, i1, -1), np.take_along_axis(s2, i2, -1)
        cand = (v1[:, :, None] + v2[:, None, :]).astype(F32).reshape(len(hf), -1)
        ids = (i1[:, :, None] * n2 + i2[:, None, :]).reshape(len(hf), -1)
        pos = np.argsort(-cand, -1, kind="stable")[:, :k]
        top = np.take_along_axis(cand, pos, -1)
        e = np.exp(top - top[:, :1], dtype=F32)
        return np.take_along_axis(ids, pos, -1).astype(np.int32), (e / e.sum(-1, keepdims=True, dtype=F32)).astype(F32)

    # SparseCoreBank.forward (aegist/hybrid.py:745-771) and the tally of HybridBlock.forward (:830-840): every pick is
    # counted; a pick whose core is live adds w * (silu(x g) * (x u)) d, any other adds nothing
    def cores(self, i, hf):
        ids, w = self.core_route(i, hf)
        self.last_cores[i] = (ids, w)
        np.add.at(self.core_counts[i], ids.reshape(-1), 1)
        out = np.zeros_like(hf)
        p = f"blocks.{i}.cores."
        if not self.b.has(p + "ids"):
            return out
        live = {int(cid): j for j, cid in enumerate(np.asarray(self.b.raw(p + "ids")).reshape(-1).tolist())}
        if not live:
            return out
        G, U, Dn = self.b.f32(p + "gate"), self.b.f32(p + "up"), self.b.f32(p + "down")
        for t in range(len(hf)):
            for r in range(ids.shape[1]):
                j = live.get(int(ids[t, r]))
                if j is None:
                    continue
                z = (silu((hf[t] @ G[j]).astype(F32)) * (hf[t] @ U[j]).astype(F32)).astype(F32)
                out[t] += (z @ Dn[j]).astype(F32) * w[t, r]
        return out

    # aegist/hybrid.py:812-843 and 896-924
    def forward(self, ids, cache):
        c = self.cfg
        ids = np.asarray(ids)
        B, T = ids.shape
        start = cache.length
        if start + T > cache.max_len:
            raise ValueError(f"context of {start + T} tokens exceeds this cache's limit of {cache.max_len}")
        cos, sin = self.rope(start + T)
        x = self.b.f32("embed.weight")[ids].astype(F32)
        for i in range(c["n_layers"]):
            h = znorm(x, self.b.f32(f"blocks.{i}.norm1.weight"), self.eps)
            if c["layer_types"][i] == "attn":
                y = self.attention(i, h, cache, cos, sin)
            else:
                y = self.deltanet(i, h, cache)
            x = (x + y).astype(F32)
            h = znorm(x, self.b.f32(f"blocks.{i}.norm2.weight"), self.eps)
            hf = h.reshape(-1, c["d_model"])
            out = self.moe(i, hf)
            if self.b.has(f"blocks.{i}.engine.key1.weight"):
                out = (out + self.cores(i, hf)).astype(F32)
            x = (x + out.reshape(B, T, -1)).astype(F32)
            self.last_hidden[i] = x[:, -1].copy()
        cache.length += T
        hN = znorm(x[:, -1], self.b.f32("norm.weight"), self.eps)
        self.final_hidden = x[:, -1].copy()
        return self.qlinear(hN, "lm_head")


# --- sampler (aegist_rs/src/chat.rs:221-272) ---------------------------------------------------

class Rng:
    """splitmix64; `next_f64` is the top 53 bits as a fraction."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next_u64(self) -> int:
        m = 0xFFFFFFFFFFFFFFFF
        self.s = (self.s + 0x9E3779B97F4A7C15) & m
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        return z ^ (z >> 31)

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) / float(1 << 53)


def sample(logits, temperature, top_p, top_k, rng: Rng) -> int:
    """Top-k, then nucleus, then inverse-CDF; temperature <= 0 is greedy and the FIRST maximum wins."""
    logits = np.asarray(logits, dtype=F32)
    if temperature <= 0:
        return int(np.argmax(logits))
    k = min(top_k, len(logits))
    idx = np.argsort(-logits, kind="stable")[:k]
    top = logits[idx[0]]
    p = [math.exp(float(F32((logits[i] - top) / F32(temperature)))) for i in idx]
    total = sum(p)
    cum, kept = 0.0, []
    for x in p:
        x /= total
        keep = cum < float(F32(top_p))
        cum += x
        kept.append(x if keep else 0.0)
    r = rng.next_f64() * sum(kept)
    for j, x in enumerate(kept):
        r -= x
        if r < 0.0 and x > 0.0:
            return int(idx[j])
    return int(idx[0])


def greedy_decode(model: HybridOracle, prompt, steps: int, max_len=None, kv_dtype="f32"):
    """The reference's greedy loop (tests/test_hybrid_rust.py:96-116): feed the prompt, then `steps`
    single-token feeds of the arg-max. Returns (logits rows [1+steps, V], tokens [steps])."""
    cache = model.new_cache(1, max_len or (len(prompt) + steps + 8), kv_dtype)
    rows = [model.forward(np.asarray([prompt]), cache)[0]]
    toks = []
    for _ in range(steps):
        toks.append(int(np.argmax(rows[-1])))
        rows.append(model.forward(np.asarray([[toks[-1]]]), cache)[0])
    return np.stack(rows), toks
