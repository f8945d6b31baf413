"""ctypes binding of the C-ABI engine: the host-side mirror of the reference's engine interface.

`HybridEngine` has the methods of `trait Lm` (aegist_rs/src/model.rs:363-427) with the meaning the
reference's `HybridEngine` gives them (aegist_rs/src/hybrid.rs:1015-1119): errors are raised as
`EngineError` carrying the engine's message (the reference returns `Err(String)`), logits come back as
a float32 array of length vocab, token ids are unsigned 32-bit.

There is no CPU path: loading the library or opening an engine without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import json
import os

import numpy as np

from . import build as _build

_LIB = None
KV_BF16, KV_F32 = 0, 1


class EngineError(RuntimeError):
    pass


class MoeWeights(C.Structure):
    _fields_ = [("d_model", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int), ("expert_hidden", C.c_int),
                ("shared_hidden", C.c_int), ("group", C.c_int),
                ("router_bf16", C.c_void_p), ("experts_q4", C.c_void_p),
                ("sh_gate_q", C.c_void_p), ("sh_gate_s", C.c_void_p), ("sh_up_q", C.c_void_p), ("sh_up_s", C.c_void_p),
                ("sh_down_q", C.c_void_p), ("sh_down_s", C.c_void_p), ("shared_gate_bf16", C.c_void_p)]


class MoeDeviceWeights(C.Structure):
    _fields_ = [("d_model", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int), ("expert_hidden", C.c_int),
                ("shared_hidden", C.c_int),
                ("router_bf16", C.c_void_p), ("expert_ptrs", C.c_void_p),
                ("sh_gate_q", C.c_void_p), ("sh_gate_s", C.c_void_p), ("sh_up_q", C.c_void_p), ("sh_up_s", C.c_void_p),
                ("sh_down_q", C.c_void_p), ("sh_down_s", C.c_void_p), ("shared_gate_bf16", C.c_void_p)]


# every symbol include/b200moe.h declares: name -> (restype, argtypes)
_P, _I, _F = C.c_void_p, C.c_int, C.c_float
SYMBOLS = {
    "b2_open": (_I, [C.c_char_p, _I, _I, _I, _I, C.POINTER(_P)]),
    "b2_create": (_I, [C.c_char_p, _I, _I, _I, _I, _I, _I, C.POINTER(_P)]),
    "b2_put_tensor": (_I, [_P, C.c_char_p, C.c_char_p, C.POINTER(C.c_int64), _I, _P, C.c_size_t, _I]),
    "b2_finish": (_I, [_P]),
    "b2_ep_unique_id": (_I, [_P, _P, C.c_size_t]),
    "b2_ep_init": (_I, [_P, _P, C.c_size_t]),
    "b2_ep_ipc_handle": (_I, [_P, _P, C.c_size_t]),
    "b2_ep_ipc_attach": (_I, [_P, _P, C.c_size_t, _I]),
    "b2_verify_file": (_I, [C.c_char_p, C.POINTER(_I), C.c_char_p, C.c_size_t]),
    "b2_close": (None, [_P]),
    "b2_feed": (_I, [_P, _P, _I, _P]),
    "b2_host_alloc": (_P, [C.c_size_t]),
    "b2_host_free": (None, [_P]),
    "b2_feed_batch": (_I, [_P, _P, _P, _P]),
    "b2_decode_greedy": (_I, [_P, _P, _I, _P, C.POINTER(_F)]),
    "b2_crop": (_I, [_P, _I]),
    "b2_snapshot": (_I, [_P]),
    "b2_state_key": (C.c_char_p, [_P]),
    "b2_save_state": (_I, [_P, C.c_char_p]),
    "b2_load_state": (_I, [_P, C.c_char_p, _P, _I, C.POINTER(_I)]),
    "b2_length": (_I, [_P]),
    "b2_cap": (_I, [_P]),
    "b2_set_taps": (_I, [_P, C.POINTER(_I), _I]),
    "b2_taps": (_I, [_P, _P]),
    "b2_core_counts": (_I, [_P, _P]),
    "b2_reset_counts": (_I, [_P]),
    "b2_expert_counters": (None, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "b2_describe": (C.c_char_p, [_P]),
    "b2_last_error": (C.c_char_p, [_P]),
    "b2_vocab": (_I, [_P]),
    "b2_d_model": (_I, [_P]),
    "b2_sample": (C.c_uint32, [_P, _I, _F, _F, _I, C.POINTER(C.c_uint64)]),
    "b2_debug_router": (_I, [_P, _I, _P, _P]),
    "b2_debug_hidden": (_I, [_P, _P]),
    "b2_set_router_bias": (_I, [_P, _I, _P]),
    "b2_debug_seek": (_I, [_P, _I]),
    "b2_launches_per_step": (_I, [_P]),
    "b2_debug_umma_launches": (C.c_long, []),
    "b2_step_bytes": (C.c_double, [_P]),
    "b2_ep_bytes_per_step": (C.c_double, [_P]),
    "b2_profile_step": (_I, [_P, _I, C.POINTER(_F), C.POINTER(C.c_double), C.POINTER(_I)]),
    "b2_debug_trace_step": (_I, [_P, C.POINTER(C.c_uint64), _I, C.POINTER(_I)]),
    "b2_op_linear_i8": (_I, [_I, _P, _P, _I, _I, _P, _I, _P]),
    "b2_debug_wait_timeout": (_I, [_I, _I, C.POINTER(_I)]),
    "b2_moe_create": (_I, [_I, C.POINTER(MoeWeights), _I, C.POINTER(_P)]),
    "b2_moe_forward": (_I, [_P, _P, _I, _P, _P, _P, C.POINTER(_F)]),
    "b2_moe_destroy": (None, [_P]),
    "b2_moe_forward_static": (_I, [C.POINTER(MoeDeviceWeights), _P, _I, _P, _P, _P, _P]),
    "b2_delta_create": (_I, [_I, _I, _I, _I, _I, _P, C.POINTER(_P)]),
    "b2_delta_step": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(_F)]),
    "b2_delta_state": (_I, [_P, _P]),
    "b2_delta_destroy": (None, [_P]),
}


def library_path() -> str:
    return _build.LIB


def load_library(build_if_missing: bool = True):
    """dlopen the in-tree shared library and set every prototype."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise EngineError(f"{path} is missing: run __graft_entry__.build()")
        _build.build()
    lib = C.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _LIB = lib
    return lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class HybridEngine:
    """One loaded brain on one GPU. Not thread-safe (the reference takes `&mut self`)."""

    def __init__(self, handle, lib, batch):
        self._h, self._lib, self.batch = handle, lib, batch
        self.vocab = lib.b2_vocab(handle)
        self.d_model = lib.b2_d_model(handle)
        self._n_taps = 0

    # --- construction ---------------------------------------------------------------------
    @classmethod
    def load(cls, nx_path: str, max_context: int = 0, device: int = 0, batch: int = 1, kv_dtype: int = KV_F32):
        """HybridEngine::load_on (aegist_rs/src/hybrid.rs:511)."""
        lib = load_library()
        h = C.c_void_p()
        rc = lib.b2_open(os.fsencode(nx_path), max_context, device, batch, kv_dtype, C.byref(h))
        return cls._checked(lib, h, rc, batch)

    @classmethod
    def from_tensors(cls, config: dict, tensors, max_context: int = 0, device: int = 0, batch: int = 1,
                     kv_dtype: int = KV_F32, ep_rank: int = 0, ep_world: int = 1):
        """Build from an iterable of (name, dtype name, torch tensor or numpy array), e.g.
        `brain.random_brain(...)`; torch CUDA tensors are read in place on their device."""
        lib = load_library()
        h = C.c_void_p()
        rc = lib.b2_create(json.dumps(config).encode(), max_context, device, batch, kv_dtype, ep_rank, ep_world, C.byref(h))
        if rc:
            return cls._checked(lib, h, rc, batch)
        for name, dt, t in tensors:
            if isinstance(t, np.ndarray):
                t = np.ascontiguousarray(t)
                ptr, nbytes, shape, on_dev = t.ctypes.data, t.nbytes, t.shape, 0
            else:
                t = t.contiguous()
                ptr, nbytes, shape, on_dev = t.data_ptr(), t.numel() * t.element_size(), tuple(t.shape), int(t.is_cuda)
            sh = (C.c_int64 * len(shape))(*shape)
            rc = lib.b2_put_tensor(h, name.encode(), dt.encode(), sh, len(shape), C.c_void_p(ptr), nbytes, on_dev)
            if rc:
                return cls._checked(lib, h, rc, batch)
            del t
        return cls._checked(lib, h, lib.b2_finish(h), batch)

    @staticmethod
    def _checked(lib, h, rc, batch):
        if rc:
            msg = lib.b2_last_error(h).decode() if h else "engine could not be created"
            if h:
                lib.b2_close(h)
            raise EngineError(msg)
        return HybridEngine(h, lib, batch)

    # --- expert parallelism -----------------------------------------------------------------
    def ep_unique_id(self) -> bytes:
        buf = C.create_string_buffer(128)
        self._check(self._lib.b2_ep_unique_id(self._h, buf, 128))
        return buf.raw

    def ep_init(self, unique_id: bytes):
        buf = C.create_string_buffer(unique_id, 128)
        self._check(self._lib.b2_ep_init(self._h, buf, 128))

    def ep_ipc_handle(self) -> bytes:
        """The handle of this rank's exchange block, for the other ranks to map (b2_ep_ipc_handle)."""
        buf = C.create_string_buffer(64)
        self._check(self._lib.b2_ep_ipc_handle(self._h, buf, 64))
        return buf.raw

    def ep_ipc_attach(self, handles):
        """Map every rank's exchange block (handles in rank order): the exchange then runs on peer stores."""
        blob = b"".join(bytes(h).ljust(64, b"\0")[:64] for h in handles)
        buf = C.create_string_buffer(blob, len(blob))
        self._check(self._lib.b2_ep_ipc_attach(self._h, buf, 64, len(handles)))

    def _check(self, rc):
        if rc:
            raise EngineError(self._lib.b2_last_error(self._h).decode())

    def close(self):
        if self._h:
            for p in getattr(self, "_host_bufs", []):
                self._lib.b2_host_free(p)
            self._host_bufs = []
            self._lib.b2_close(self._h)
            self._h = None

    def host_buffer(self, n: int, dtype=np.float32) -> np.ndarray:
        """A page-locked numpy array of n values for feed(out=...): the logits then arrive by plain DMA. It lives
        until close(); do not use it afterwards."""
        dt = np.dtype(dtype)
        p = self._lib.b2_host_alloc(int(n) * dt.itemsize)
        if not p:
            raise EngineError("b2_host_alloc failed")
        if not hasattr(self, "_host_bufs"):
            self._host_bufs = []
        self._host_bufs.append(p)
        return np.frombuffer((C.c_char * (int(n) * dt.itemsize)).from_address(p), dtype=dt)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- trait Lm ---------------------------------------------------------------------------
    def feed(self, ids, want_logits: bool = True, out=None):
        """Feed tokens; return the logits after the last one (in `out`, a float32[vocab] array such as
        host_buffer(vocab), when given: a loop that reuses one page-locked array saves the allocation and
        the staged copy of a fresh one)."""
        ids = np.ascontiguousarray(np.asarray(ids, dtype=np.uint32).reshape(-1))
        if out is not None:
            if out.dtype != np.float32 or out.size != self.vocab or not out.flags.c_contiguous:
                raise EngineError("feed(out=...) needs a contiguous float32 array of vocab values")
        elif want_logits:
            out = np.empty(self.vocab, dtype=np.float32)
        self._check(self._lib.b2_feed(self._h, _ptr(ids), len(ids), _ptr(out) if out is not None else None))
        return out

    def feed_batch(self, ids, want_logits: bool = True):
        """One token per sequence -> (arg-max per sequence, logits [batch, vocab] or None)."""
        ids = np.ascontiguousarray(np.asarray(ids, dtype=np.uint32).reshape(-1))
        if len(ids) != self.batch:
            raise EngineError(f"feed_batch needs {self.batch} ids, got {len(ids)}")
        nxt = np.empty(self.batch, dtype=np.uint32)
        out = np.empty((self.batch, self.vocab), dtype=np.float32) if want_logits else None
        self._check(self._lib.b2_feed_batch(self._h, _ptr(ids), _ptr(nxt), _ptr(out) if want_logits else None))
        return nxt, out

    def decode_greedy(self, first, steps: int):
        """Greedy loop on the device -> (tokens [steps, batch], device milliseconds)."""
        first = np.ascontiguousarray(np.asarray(first, dtype=np.uint32).reshape(-1))
        toks = np.empty((steps, self.batch), dtype=np.uint32)
        ms = C.c_float()
        self._check(self._lib.b2_decode_greedy(self._h, _ptr(first), steps, _ptr(toks), C.byref(ms)))
        return toks, ms.value

    def crop(self, n: int) -> int:
        kept = self._lib.b2_crop(self._h, n)
        if kept < 0:
            raise EngineError("crop failed")
        return kept

    def snapshot(self):
        self._check(self._lib.b2_snapshot(self._h))

    def state_key(self) -> str:
        """Lm::state_key (aegist_rs/src/model.rs:375-378)."""
        return self._lib.b2_state_key(self._h).decode()

    def save_state(self, path: str):
        """Lm::save_state: what the tokens fed so far left behind, in the reference's AEGSTATE file format."""
        self._check(self._lib.b2_save_state(self._h, os.fsencode(path)))

    def load_state(self, path: str):
        """Lm::load_state -> the saved tokens; on an error the engine is left empty."""
        toks = np.zeros(max(self.cap(), 1), dtype=np.uint32)
        n = C.c_int(0)
        self._check(self._lib.b2_load_state(self._h, os.fsencode(path), _ptr(toks), len(toks), C.byref(n)))
        return toks[: n.value].tolist()

    def length(self) -> int:
        return self._lib.b2_length(self._h)

    def cap(self) -> int:
        return self._lib.b2_cap(self._h)

    def set_taps(self, layers):
        arr = (C.c_int * len(layers))(*layers)
        self._check(self._lib.b2_set_taps(self._h, arr, len(layers)))
        self._n_taps = len(layers)

    def taps(self):
        out = np.zeros((self._n_taps, self.batch, self.d_model), dtype=np.float32)
        if self._n_taps:
            self._check(self._lib.b2_taps(self._h, _ptr(out)))
        return out

    def core_counts(self, layers: int, n_cores: int):
        out = np.zeros((layers, n_cores), dtype=np.int32)
        self._check(self._lib.b2_core_counts(self._h, _ptr(out)))
        return out

    def reset_counts(self):
        self._check(self._lib.b2_reset_counts(self._h))

    def expert_counters(self):
        a, b = C.c_uint64(), C.c_uint64()
        self._lib.b2_expert_counters(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def describe(self) -> str:
        return self._lib.b2_describe(self._h).decode()

    # --- parity / measurement hooks -----------------------------------------------------------
    def router(self, layer: int, top_k: int):
        idx = np.empty((self.batch, top_k), dtype=np.int32)
        w = np.empty((self.batch, top_k), dtype=np.float32)
        self._check(self._lib.b2_debug_router(self._h, layer, _ptr(idx), _ptr(w)))
        return idx, w

    def hidden(self):
        out = np.empty((self.batch, self.d_model), dtype=np.float32)
        self._check(self._lib.b2_debug_hidden(self._h, _ptr(out)))
        return out

    def set_router_bias(self, layer: int, bias):
        if bias is None:
            self._check(self._lib.b2_set_router_bias(self._h, layer, None))
        else:
            b = np.ascontiguousarray(np.asarray(bias, dtype=np.float32))
            self._check(self._lib.b2_set_router_bias(self._h, layer, _ptr(b)))

    def seek(self, n: int):
        """Set the context length without feeding (timing hook; see b2_debug_seek)."""
        self._check(self._lib.b2_debug_seek(self._h, n))

    def launches_per_step(self) -> int:
        return self._lib.b2_launches_per_step(self._h)

    def step_bytes(self) -> float:
        return self._lib.b2_step_bytes(self._h)

    def ep_bytes_per_step(self) -> float:
        """Bytes this GPU sends to its peers over NVLink in one decode step (expert parallelism)."""
        return self._lib.b2_ep_bytes_per_step(self._h)

    # roles of the launches of a decode step; which kernel fills a role depends on the batch:
    #   1-5 sequences: k_tcgemv (in_proj, out_proj, head), k_moe_gu1, k_moe_down1
    #   6+ sequences:  k_prep_q + k_umma (tcgen05 GEMMs), k_group_picks + k_prep_q_slots + k_umma_q4 for the experts
    KERNEL_CLASSES = ("embed", "in_proj", "delta_step", "attention", "out_proj", "expert_gate_up", "expert_down", "head")
    KERNELS_SMALL_BATCH = {"embed": "k_embed", "in_proj": "k_tcgemv", "delta_step": "k_delta_step",
                           "attention": "k_attn + k_attn_merge", "out_proj": "k_tcgemv", "expert_gate_up": "k_moe_gu1",
                           "expert_down": "k_moe_down1", "head": "k_tcgemv"}

    def profile_step(self, iters: int = 8) -> dict:
        """Per kernel class: mean ms per step, algorithmic bytes per step, launches per step."""
        ms, by, ln = (C.c_float * 8)(), (C.c_double * 8)(), (C.c_int * 8)()
        self._check(self._lib.b2_profile_step(self._h, iters, ms, by, ln))
        return {n: {"ms": ms[i], "bytes": by[i], "launches": ln[i]} for i, n in enumerate(self.KERNEL_CLASSES)}

    def trace_step(self, cap: int = 4096):
        """Timeline of one graph-run decode step: a uint64 array [launches][16] (see b2_debug_trace_step)."""
        buf = (C.c_uint64 * (16 * cap))()
        n = C.c_int(0)
        self._check(self._lib.b2_debug_trace_step(self._h, buf, cap, C.byref(n)))
        return np.frombuffer(buf, dtype=np.uint64)[: 16 * n.value].reshape(n.value, 16).copy()


# --- sampler (aegist_rs/src/chat.rs:221-272) ----------------------------------------------------

class Rng:
    """splitmix64 state, advanced by `sample`."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)


def sample(logits, temperature: float, top_p: float, top_k: int, rng: Rng) -> int:
    lib = load_library()
    a = np.ascontiguousarray(np.asarray(logits, dtype=np.float32))
    return int(lib.b2_sample(_ptr(a), len(a), temperature, top_p, top_k, C.byref(rng.state)))


def verify_file(path: str) -> dict:
    lib = load_library()
    ok = (C.c_int * 3)()
    err = C.create_string_buffer(512)
    if lib.b2_verify_file(os.fsencode(path), ok, err, 512):
        raise EngineError(err.value.decode())
    return {"base": bool(ok[0]), "engine": bool(ok[1]), "cores": bool(ok[2])}


# --- single operators ----------------------------------------------------------------------------

def linear_i8(q: np.ndarray, scale_bf16: np.ndarray, x: np.ndarray, device: int = 0) -> np.ndarray:
    lib = load_library()
    q = np.ascontiguousarray(q, dtype=np.int8)
    s = np.ascontiguousarray(scale_bf16, dtype=np.uint16).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = q.shape
    y = np.empty((x.shape[0], n), dtype=np.float32)
    if lib.b2_op_linear_i8(device, _ptr(q), _ptr(s), n, k, _ptr(x), x.shape[0], _ptr(y)):
        raise EngineError("b2_op_linear_i8 failed")
    return y


class MoeLayer:
    """MoE.forward (aegist/hybrid.py:647-652) on the GPU from .nx-format weights held in numpy."""

    def __init__(self, d_model, n_experts, top_k, expert_hidden, shared_hidden, router_bf16, experts_q4, sh_gate, sh_up,
                 sh_down, shared_gate_bf16, max_tokens=64, device=0, group=64):
        lib = load_library()
        keep = [np.ascontiguousarray(a) for a in (router_bf16, experts_q4, sh_gate[0], sh_gate[1].reshape(-1), sh_up[0],
                                                  sh_up[1].reshape(-1), sh_down[0], sh_down[1].reshape(-1),
                                                  shared_gate_bf16.reshape(-1))]
        w = MoeWeights(d_model, n_experts, top_k, expert_hidden, shared_hidden, group, *[a.ctypes.data for a in keep])
        self._lib, self._h = lib, C.c_void_p()
        self.d, self.k = d_model, top_k
        if lib.b2_moe_create(device, C.byref(w), max_tokens, C.byref(self._h)):
            raise EngineError("b2_moe_create failed")

    def forward(self, h: np.ndarray):
        h = np.ascontiguousarray(h, dtype=np.float32)
        T = h.shape[0]
        y = np.empty((T, self.d), dtype=np.float32)
        idx = np.empty((T, self.k), dtype=np.int32)
        w = np.empty((T, self.k), dtype=np.float32)
        ms = C.c_float()
        if self._lib.b2_moe_forward(self._h, _ptr(h), T, _ptr(y), _ptr(idx), _ptr(w), C.byref(ms)):
            raise EngineError("b2_moe_forward failed")
        return y, idx, w, ms.value

    def close(self):
        if self._h:
            self._lib.b2_moe_destroy(self._h)
            self._h = None


class DeltaRule:
    """delta_rule_step (aegist/hybrid.py:318-324) with the state carried on the device."""

    def __init__(self, state0: np.ndarray, device=0):
        lib = load_library()
        s = np.ascontiguousarray(state0, dtype=np.float32)
        self.B, self.H, self.dk, self.dv = s.shape
        self._lib, self._h = lib, C.c_void_p()
        if lib.b2_delta_create(device, self.B, self.H, self.dk, self.dv, _ptr(s), C.byref(self._h)):
            raise EngineError("b2_delta_create failed")

    def step(self, q, k, v, g, beta):
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v, g, beta)]
        out = np.empty((self.B, self.H, self.dv), dtype=np.float32)
        ms = C.c_float()
        if self._lib.b2_delta_step(self._h, *[_ptr(a) for a in arrs], _ptr(out), C.byref(ms)):
            raise EngineError("b2_delta_step failed")
        return out, ms.value

    def state(self):
        out = np.empty((self.B, self.H, self.dk, self.dv), dtype=np.float32)
        if self._lib.b2_delta_state(self._h, _ptr(out)):
            raise EngineError("b2_delta_state failed")
        return out

    def close(self):
        if self._h:
            self._lib.b2_delta_destroy(self._h)
            self._h = None
