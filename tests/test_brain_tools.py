"""Host-side tools: the .nx reader/writer and the quantisers, against files and vectors the
reference itself wrote (tests/golden/)."""
import os

import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def ops(golden_dir):
    return np.load(os.path.join(golden_dir, "ops_golden.npz"))


def test_reader_on_reference_written_file(pkg, micro_path):
    from b200moe.nxfile import NxFile
    with NxFile(micro_path) as nx:
        assert nx.config["arch"] == "hybrid-moe" and nx.header["quant"] == "int8"
        assert all(nx.verify().values())
        cfg = pkg.HybridConfig.from_dict(nx.config)
        assert nx.info("blocks.0.moe.experts.q4")["shape"] == [cfg.n_experts, cfg.expert_bytes]
        for m in nx.header["tensors"].values():
            assert m["offset"] % 64 == 0
        assert nx.tensor("embed.weight").shape == (cfg.vocab_size, cfg.d_model)
        assert b"im_start" in nx.blob("tokenizer.json")


def test_builder_reproduces_the_reference_written_brain(pkg, micro_path, tmp_path):
    """Same seeded master weights through THIS repo's quantisers and writer must give the tensors the
    reference's quantisers and writer gave, byte for byte (pins int8_quantize, q4_quantize,
    pack_experts and the writer's layout)."""
    from b200moe import brain
    from b200moe.nxfile import NxFile
    out = str(tmp_path / "mine.nx")
    brain.write_brain(out, pkg.HybridConfig.micro(), seed=0, vary_1d=True)
    with NxFile(out) as mine, NxFile(micro_path) as ref:
        assert all(mine.verify().values())
        assert sorted(mine.header["tensors"]) == sorted(ref.header["tensors"])
        for n, m in ref.header["tensors"].items():
            mm = mine.header["tensors"][n]
            assert (mm["dtype"], mm["shape"], mm["offset"], mm["nbytes"]) == (m["dtype"], m["shape"], m["offset"], m["nbytes"]), n
            assert np.array_equal(mine.tensor(n), ref.tensor(n)), n
        assert mine.header["sha256"] == ref.header["sha256"]
        assert mine.header["config"] == ref.header["config"]


def test_round_trip_and_tamper_detection(pkg, tmp_path):
    from b200moe.nxfile import Bf16, NxFile, f32_to_bf16_bits, save
    rng = np.random.default_rng(0)
    state = {"a.weight": rng.standard_normal((5, 7)).astype(np.float32),
             "blocks.0.engine.key1.weight": Bf16(f32_to_bf16_bits(rng.standard_normal((3, 4)).astype(np.float32))),
             "blocks.0.cores.ids": np.zeros(0, dtype=np.int64),
             "q": rng.integers(-127, 127, (9, 16)).astype(np.int8)}
    path = str(tmp_path / "t.nx")
    save(path, state, {"arch": "hybrid-moe"}, "{}", license_text="L")
    with NxFile(path) as nx:
        assert all(nx.verify().values())
        assert np.array_equal(nx.tensor("a.weight"), state["a.weight"])
        assert nx.tensor("blocks.0.cores.ids").shape == (0,)
        assert nx.info("blocks.0.engine.key1.weight")["group"] == "engine"
        assert nx.blob("LICENSE") == b"L"
        off = nx.data_start + nx.info("q")["offset"]
    raw = bytearray(open(path, "rb").read())
    raw[off] ^= 0x40
    open(path, "wb").write(raw)
    with NxFile(path) as nx:
        assert nx.verify() == {"base": False, "engine": True, "cores": True}
    open(path, "wb").write(b"NOTANNXFILE" + bytes(64))
    with pytest.raises(ValueError):
        NxFile(path)


def test_q4_quantize_matches_reference_vectors(pkg, ops):
    from b200moe import brain
    w = torch.from_numpy(ops["q4_w"].view(np.int16)).view(torch.bfloat16)
    p, s, m = brain.q4_quantize(w, 64)
    assert np.array_equal(p.numpy(), ops["q4_packed"])
    assert np.array_equal(s.numpy(), ops["q4_scale"]) and np.array_equal(m.numpy(), ops["q4_min"])
    assert np.array_equal(brain.q4_dequantize(p, s, m, 64).numpy(), ops["q4_deq"])
    rel = (brain.q4_dequantize(p, s, m, 64) - w.float()).norm() / w.float().norm()
    assert 0.05 < float(rel) < 0.12      # the reference reports a mean relative weight error of 0.086


def test_int8_quantize_matches_reference_vectors(pkg, ops):
    from b200moe import brain
    w = torch.from_numpy(ops["i8_w"].view(np.int16)).view(torch.bfloat16)
    q, s = brain.int8_quantize(w)
    assert np.array_equal(q.numpy(), ops["i8_q"])
    assert np.array_equal(s.view(torch.int16).numpy().view(np.uint16), ops["i8_scale"])


def test_expert_row_layout(pkg):
    cfg = pkg.HybridConfig.full()
    assert cfg.expert_bytes == 1_769_472                   # per expert at the 35B shape
    assert pkg.HybridConfig.tiny().expert_bytes == 110_592
    from b200moe import brain
    c = pkg.HybridConfig.micro()
    gu = brain.normal("g", (2, 2 * c.expert_hidden, c.d_model), 1, "cpu")
    dn = brain.normal("d", (2, c.d_model, c.expert_hidden), 1, "cpu")
    rows = brain.pack_experts(gu, dn, c)
    g2, d2 = brain.unpack_expert(rows[1], c)
    assert (g2 - gu[1].float()).abs().max() < 0.01 and (d2 - dn[1].float()).abs().max() < 0.01
