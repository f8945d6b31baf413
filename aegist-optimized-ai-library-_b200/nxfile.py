"""The .nx brain file: reader and writer.

Layout (aegist/nx.py:1-19; Rust reader aegist_rs/src/nx.rs:1-6):

    bytes 0..8     magic  b"AEGISTNX"
    bytes 8..12    u32 LE format version (1)
    bytes 12..20   u64 LE header length H
    bytes 20..20+H UTF-8 JSON header
    zero padding to a 64-byte boundary, then the data section; every tensor 64-byte aligned

The header lists every tensor (dtype, shape, offset into the data section, nbytes, group), the
blobs (tokenizer.json, LICENSE), the model config and one SHA-256 per group ("base", "engine",
"cores") taken over the tensors in (group, name) order (aegist/nx.py:89-136).

Tensors are numpy arrays here. numpy has no bfloat16, so a bf16 tensor is a uint16 array tagged
with the dtype name "bf16" (`Bf16` wrapper when writing).
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
import time

import numpy as np

MAGIC = b"AEGISTNX"
LEGACY_MAGIC = b"AUGISTNX"
VERSION = 1
ALIGN = 64
NP_DTYPES = {"bf16": np.uint16, "f16": np.float16, "f32": np.float32, "i8": np.int8, "i64": np.int64,
             "u8": np.uint8}
GROUPS = ("base", "engine", "cores")


class Bf16:
    """A uint16 array whose bits are bfloat16 values."""

    def __init__(self, bits: np.ndarray):
        assert bits.dtype == np.uint16
        self.bits = bits
        self.shape = bits.shape


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (what torch's .to(bfloat16) does)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def group_of(name: str) -> str:
    if ".cores." in name:
        return "cores"
    if ".engine." in name:
        return "engine"
    return "base"


def _pad(n: int) -> int:
    return (-n) % ALIGN


def _describe(t):
    if isinstance(t, Bf16):
        return "bf16", t.bits
    for name, dt in NP_DTYPES.items():
        if name != "bf16" and t.dtype == dt:
            return name, t
    raise ValueError(f"unsupported dtype {t.dtype}")


def save(path: str, state: dict, config: dict, tokenizer_json: str = "{}", *, notice: str = "",
         license_text: str = "", extra: dict | None = None) -> dict:
    """Write `state` (name -> numpy array or Bf16) as an .nx file. Written to `path + ".partial"`
    and renamed, so a crash never leaves a half-written brain (aegist/nx.py:70-143)."""
    tensors, blobs, offset = {}, {}, 0
    order = sorted(state, key=lambda n: (group_of(n), n))
    arrays = {}
    for n in order:
        dname, arr = _describe(state[n])
        arr = np.ascontiguousarray(arr)
        arrays[n] = arr
        tensors[n] = {"dtype": dname, "shape": list(arr.shape), "offset": offset, "nbytes": arr.nbytes,
                      "group": group_of(n)}
        offset += arr.nbytes + _pad(arr.nbytes)
    texts = (("tokenizer.json", tokenizer_json), ("LICENSE", license_text))
    for name, text in texts:
        data = text.encode("utf-8")
        blobs[name] = {"offset": offset, "nbytes": len(data)}
        offset += len(data) + _pad(len(data))
    header = {"name": "Aegist", "format": "nx", "format_version": VERSION,
              "created": time.strftime("%Y-%m-%dT%H:%M:%S"), "config": config, "notice": notice, "persona": {},
              "generation": {}, "lineage": [], "tensors": tensors, "blobs": blobs, **(extra or {})}
    enc = lambda h: json.dumps(h, separators=(",", ":")).encode("utf-8")
    header["sha256"] = {g: "0" * 64 for g in GROUPS}
    hb = enc(header)
    data_start = 20 + len(hb) + _pad(20 + len(hb))
    hashes = {g: hashlib.sha256() for g in GROUPS}
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(b"\0" * data_start)
        for n in order:
            raw = arrays[n].reshape(-1).view(np.uint8)
            hashes[tensors[n]["group"]].update(raw)
            f.write(raw)
            f.write(b"\0" * _pad(raw.nbytes))
        for name, text in texts:
            data = text.encode("utf-8")
            f.write(data)
            f.write(b"\0" * _pad(len(data)))
        header["sha256"] = {g: h.hexdigest() for g, h in hashes.items()}
        hb2 = enc(header)
        assert len(hb2) == len(hb)
        f.seek(0)
        f.write(MAGIC + struct.pack("<IQ", VERSION, len(hb2)) + hb2)
    os.replace(tmp, path)
    return header


class NxFile:
    """Memory-mapped reader; `tensor()` returns views into the map."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(20)
        if len(head) < 20 or head[:8] not in (MAGIC, LEGACY_MAGIC):
            self._f.close()
            raise ValueError(f"{path} is not an .nx file")
        version, hlen = struct.unpack("<IQ", head[8:20])
        if version > VERSION:
            self._f.close()
            raise ValueError(f"{path} uses .nx format v{version}; this reader handles up to v{VERSION}")
        self.header = json.loads(self._f.read(hlen).decode("utf-8"))
        self.data_start = 20 + hlen + _pad(20 + hlen)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def config(self) -> dict:
        return self.header["config"]

    def names(self, group: str | None = None) -> list:
        return [n for n, m in self.header["tensors"].items() if group is None or m["group"] == group]

    def info(self, name: str) -> dict:
        return self.header["tensors"][name]

    def tensor(self, name: str) -> np.ndarray:
        """bf16 tensors come back as uint16 bit patterns (see bf16_bits_to_f32)."""
        m = self.header["tensors"][name]
        dt = np.dtype(NP_DTYPES[m["dtype"]])
        n = m["nbytes"] // dt.itemsize
        if n == 0:
            return np.zeros(m["shape"], dtype=dt)
        return np.frombuffer(self._mm, dtype=dt, count=n, offset=self.data_start + m["offset"]).reshape(m["shape"])

    def tensor_f32(self, name: str) -> np.ndarray:
        t = self.tensor(name)
        if self.header["tensors"][name]["dtype"] == "bf16":
            return bf16_bits_to_f32(t)
        return t.astype(np.float32)

    def blob(self, name: str) -> bytes:
        m = self.header["blobs"][name]
        s = self.data_start + m["offset"]
        return bytes(self._mm[s: s + m["nbytes"]])

    def verify(self) -> dict:
        hashes = {g: hashlib.sha256() for g in GROUPS}
        t = self.header["tensors"]
        for n in sorted(t, key=lambda n: (t[n]["group"], n)):
            s = self.data_start + t[n]["offset"]
            hashes[t[n]["group"]].update(self._mm[s: s + t[n]["nbytes"]])
        return {g: hashes[g].hexdigest() == self.header["sha256"][g] for g in hashes}
