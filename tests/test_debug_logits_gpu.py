"""The reference's parity entry point over this engine: `b2-debug-logits BRAIN in.json out.bin` reads the in.json
of `aegist debug-logits` (aegist_rs/src/main.rs:733-803) and writes the same out.bin, so the reference's own test
helper (`rust_ops`, tests/test_hybrid_rust.py:128-133) works with it unchanged apart from the executable's name.
Checked against the rows the unmodified reference produced for the same ops (tests/golden/micro_golden.npz)."""
import json
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 3e-4


@pytest.fixture(scope="module")
def exe(pkg):
    from b200moe import build
    build.build()
    return build.CLI


def run_ops(exe, brain, tmp_path, spec, name="case", extra=()):
    inp, out = tmp_path / f"{name}.json", tmp_path / f"{name}.bin"
    inp.write_text(json.dumps(spec), encoding="utf-8")
    r = subprocess.run([exe, brain, str(inp), str(out), "--context", "160", *extra], capture_output=True, text=True)
    return r, out


def rows_of(path, vocab=512):
    return np.frombuffer(path.read_bytes(), dtype=np.float32).reshape(-1, vocab)


def test_ops_form_with_snapshot_crop_and_taps(exe, micro_path, golden_dir, tmp_path):
    g = np.load(os.path.join(golden_dir, "micro_golden.npz"))
    ids = g["rewind_ids"].tolist()
    a, b, c = ids[:30], ids[30:50], ids[50:65]
    ops = [{"feed": a[:12]}, {"snapshot": True}, {"feed": a[12:]}, {"snapshot": True}, {"feed": b},
           {"crop": len(a) + 3}, {"feed": c}, {"crop": 5}, {"feed": [1, 2, 3]}]
    r, out = run_ops(exe, micro_path, tmp_path, {"ops": ops, "taps": [0, 3]})
    assert r.returncode == 0, r.stderr
    assert [ln for ln in r.stderr.splitlines() if ln.startswith("crop")] == ["crop 33 -> 30", "crop 5 -> 0"]
    rows = rows_of(out)
    assert rows.shape == (5, 512)
    assert np.abs(rows - g["rewind_logits"]).max() < TOL
    taps = np.frombuffer((tmp_path / "case.bin.taps").read_bytes(), dtype=np.float32)
    assert taps.size == 5 * 2 * 128 and np.isfinite(taps).all()


def test_prompt_steps_form(exe, micro_path, golden_dir, tmp_path):
    g = np.load(os.path.join(golden_dir, "micro_golden.npz"))
    r, out = run_ops(exe, micro_path, tmp_path, {"prompt": g["prompt"].tolist(), "steps": g["greedy_tokens"].tolist()}, "greedy")
    assert r.returncode == 0, r.stderr
    rows = rows_of(out)
    assert rows.shape == (1 + len(g["greedy_tokens"]), 512)
    assert np.abs(rows - g["greedy_logits"]).max() < TOL
    assert "decode steps" in r.stderr and "experts" in r.stderr


def test_saved_state_round_trip(exe, micro_path, golden_dir, tmp_path):
    """{"save": path} / {"load": path}: a context saved by one process and loaded by another continues with exactly the
    rows of the uninterrupted run; a state does not load into a brain with another key, and an unknown op is an error."""
    g = np.load(os.path.join(golden_dir, "micro_golden.npz"))
    ids = g["multi_ids"].tolist()
    state = str(tmp_path / "ctx.state")
    r, out = run_ops(exe, micro_path, tmp_path, {"ops": [{"feed": ids[:70]}, {"feed": ids[70:90]}]}, "whole")
    assert r.returncode == 0, r.stderr
    whole = rows_of(out)
    r, out = run_ops(exe, micro_path, tmp_path, {"ops": [{"feed": ids[:70]}, {"save": state}]}, "first")
    assert r.returncode == 0 and "save 70 tokens" in r.stderr, r.stderr
    head = open(state, "rb").read(16)
    assert head[:8] == b"AEGSTATE"
    r, out = run_ops(exe, micro_path, tmp_path, {"ops": [{"load": state}, {"feed": ids[70:90]}, {"crop": 75}]}, "second")
    assert r.returncode == 0 and "load 70 tokens" in r.stderr, r.stderr
    assert "crop 75 -> 70" in r.stderr                  # loading takes a snapshot at the loaded length
    assert np.array_equal(rows_of(out)[0], whole[1])
    r, _ = run_ops(exe, micro_path, tmp_path, {"ops": [{"load": state}]}, "otherkey", extra=("--kv", "bf16"))
    assert r.returncode != 0 and "saved by another brain" in r.stderr
    r, _ = run_ops(exe, micro_path, tmp_path, {"ops": [{"dance": 1}]}, "bad")
    assert r.returncode != 0 and "unknown op" in r.stderr


def test_python_binding_of_saved_states(pkg, micro_path, tmp_path):
    import importlib
    E = importlib.import_module("b200moe.engine")
    a = E.HybridEngine.load(micro_path, max_context=64)
    a.feed([5, 6, 7, 8, 9])
    path = str(tmp_path / "s.state")
    a.save_state(path)
    want = a.feed([10])
    assert a.state_key().endswith("-4x1x32") or "x" in a.state_key()
    b = E.HybridEngine.load(micro_path, max_context=64)
    assert b.load_state(path) == [5, 6, 7, 8, 9] and b.length() == 5
    assert np.array_equal(b.feed([10]), want)
    a.decode_greedy([11], 3)
    a.save_state(path)                                   # tokens of a device-side greedy loop are known afterwards
    a.seek(20)
    with pytest.raises(E.EngineError, match="not all known"):
        a.save_state(path)
    with pytest.raises(E.EngineError, match="not a saved state"):
        b.load_state(micro_path)
    assert b.length() == 0                               # an error leaves the engine empty
    a.close()
    b.close()
