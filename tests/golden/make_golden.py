"""Generate the golden fixtures in this directory by running the UNMODIFIED reference.

    python tests/golden/make_golden.py /path/to/reference/aegist-fast-35b

The reference's Python model (aegist/hybrid.py) is imported from its own tree; nothing of it is
copied. Master weights come from this repo's seeded generator (`brain.normal`, keyed by tensor
name), are loaded into the reference's `HybridLM`, and are then quantised, packed and written by
the reference's own code (`quantize_base_int8`, `pack_experts`, `nx.save_model`). The reference then
reloads the file and runs in fp32 with an fp32 cache, exactly as its parity test does
(tests/test_hybrid_rust.py:96-116).

Outputs:
  micro.nx            the reference-written micro brain (committed; ~1.5 MB)
  micro_golden.npz    logits / router picks / greedy tokens / taps / snapshot-crop / batch cases
  tiny_golden.npz     the 4-layer hidden-512 vocab-32768 case: group hashes of the file the
                      reference wrote, router picks, greedy tokens and logits samples
  ops_golden.npz      per-op cases: quantisers, MoE layer, delta rule (step and chunked), RoPE
  micro_cores.nx      the micro brain with a few live switchable cores (`--only cores` writes just this pair)
  cores_golden.npz    logits, core picks and weights, per-core switch-on counts of the reference on that brain
"""
import hashlib
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) < 2:
    raise SystemExit(__doc__)
REF = sys.argv[1]
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from __graft_entry__ import load_package  # noqa: E402

pkg = load_package()
from b200moe import brain as B  # noqa: E402
from b200moe.config import HybridConfig as OurConfig  # noqa: E402

from aegist import hybrid as H  # noqa: E402
from aegist import nx as NX  # noqa: E402
from aegist.model import QLinear  # noqa: E402


def tokenizer_json() -> str:
    from tokenizers import Tokenizer, models
    tok = Tokenizer(models.WordLevel({"hi": 0, "there": 1, "[UNK]": 2}, unk_token="[UNK]"))
    tok.add_special_tokens(["<|im_start|>", "<|im_end|>", "<|endoftext|>"])
    return tok.to_str()


def reference_brain(ours: OurConfig, seed: int, path: str, vary_1d: bool = False):
    """Seeded master weights -> the reference's model -> the reference's quantisers and writer."""
    cfg = H.HybridConfig.from_dict(ours.to_dict())
    model = H.HybridLM(cfg)
    sd = model.state_dict()
    I, E = cfg.expert_hidden, cfg.n_experts
    with torch.no_grad():
        for name, p in sd.items():
            if ".engine." in name or ".cores." in name:
                if ".engine." in name:
                    p.copy_(B.normal(name, p.shape, seed, "cpu", cfg.d_model ** -0.5).float())
                continue
            if name.endswith("experts.gate_up") or name.endswith("experts.down"):
                base = name.rsplit(".", 1)[0]
                kind = name.rsplit(".", 1)[1]
                chunks = []
                for s in range(0, E, 32):
                    n = min(32, E - s)
                    shape = (n, 2 * I, cfg.d_model) if kind == "gate_up" else (n, cfg.d_model, I)
                    chunks.append(B.normal(f"{base}.{kind}.{s}", shape, seed, "cpu"))
                p.copy_(torch.cat(chunks).float())
            elif p.dim() >= 2:
                p.copy_(B.normal(name, p.shape, seed, "cpu").float())
            else:
                p.copy_(B.vector_init(name, p.shape, seed, "cpu", vary_1d).float())
    model = model.to(torch.bfloat16)
    model.quantize_base_int8()
    masters = [H.pack_experts(b.moe.experts.gate_up.data, b.moe.experts.down.data, cfg) for b in model.blocks]
    model.page_experts(masters, slots=cfg.n_experts, device="cpu")
    model.eval()
    return NX.save_model(path, model, tokenizer_json())


class Ref:
    def __init__(self, path):
        self.model, _, self.nx = NX.load_model(path, device="cpu", slots=4096)
        self.model.float()
        self.cfg = self.model.cfg
        self.taps = {}
        self.wts = {}
        for i, b in enumerate(self.model.blocks):
            b.register_forward_hook(lambda m, a, out, i=i: self.taps.__setitem__(i, out[0][:, -1].detach().clone()))
            b.moe.route = self._spy(i, b.moe.route)

    def _spy(self, i, route):
        def spied(h):
            idx, w = route(h)
            self.wts[i] = w.detach().float().clone()
            return idx, w
        return spied

    def cache(self, batch, n):
        return self.model.new_cache(batch, n, dtype=torch.float32)

    @torch.no_grad()
    def feed(self, ids, cache):
        """ids [B, T] -> (logits [B, V], router picks [L, B*T, K], taps [L, B, D]); the router
        weights of the same feed are left in `self.last_w` [L, B*T, K]."""
        x = torch.as_tensor(np.asarray(ids), dtype=torch.long)
        out = self.model(x, cache=cache, last_only=True)["logits"][:, -1].float().numpy().copy()
        idx, wts = [], []
        for b in self.model.blocks:
            idx.append(b.moe.last_experts.numpy().astype(np.int32).copy())
        taps = np.stack([self.taps[i].numpy() for i in range(len(self.model.blocks))])
        self.last_w = np.stack([self.wts[i].numpy() for i in range(len(self.model.blocks))])
        return out, np.stack(idx), taps


def micro_cases(path, out):
    ref = Ref(path)
    V = ref.cfg.vocab_size
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, V, (12,), generator=g).tolist()
    res = {"prompt": np.array(prompt, dtype=np.int32)}

    # (a) prompt in one feed (chunked DeltaNet form), then 24 greedy single-token feeds
    cache = ref.cache(1, 64)
    rows, routes, taps, toks, rw = [], [], [], [], []
    lg, ix, tp = ref.feed([prompt], cache)
    rows.append(lg[0]); routes.append(ix[:, -1]); taps.append(tp[:, 0]); rw.append(ref.last_w[:, -1])
    for _ in range(24):
        toks.append(int(rows[-1].argmax()))
        lg, ix, tp = ref.feed([[toks[-1]]], cache)
        rows.append(lg[0]); routes.append(ix[:, -1]); taps.append(tp[:, 0]); rw.append(ref.last_w[:, -1])
    res.update(greedy_logits=np.stack(rows), greedy_tokens=np.array(toks, dtype=np.int32),
               greedy_routes=np.stack(routes), greedy_taps=np.stack(taps), greedy_route_w=np.stack(rw))

    # (b) the same tokens fed one at a time (the step recurrence from the first token on)
    cache = ref.cache(1, 64)
    rows, routes, rw, taps = [], [], [], []
    for t in prompt + toks:
        lg, ix, tp = ref.feed([[t]], cache)
        rows.append(lg[0]); routes.append(ix[:, -1]); rw.append(ref.last_w[:, -1]); taps.append(tp[:, 0])
    res.update(single_logits=np.stack(rows), single_routes=np.stack(routes), single_route_w=np.stack(rw),
               single_taps=np.stack(taps))

    # (c) feeds of 5, 30 and 100 tokens, then 4 greedy steps
    ids = torch.randint(0, V, (135,), generator=g).tolist()
    cache = ref.cache(1, 160)
    rows, toks2 = [], []
    for f in (ids[:5], ids[5:35], ids[35:]):
        rows.append(ref.feed([f], cache)[0][0])
    for _ in range(4):
        toks2.append(int(rows[-1].argmax()))
        rows.append(ref.feed([[toks2[-1]]], cache)[0][0])
    res.update(multi_ids=np.array(ids, dtype=np.int32), multi_logits=np.stack(rows),
               multi_tokens=np.array(toks2, dtype=np.int32))

    # (d) snapshot / crop, the scenario of tests/test_hybrid_rust.py:229-242 at small scale
    ids = torch.randint(0, V, (80,), generator=g).tolist()
    a, b, c = ids[:30], ids[30:50], ids[50:65]
    cache = ref.cache(1, 128)
    rows, kept = [], []
    rows.append(ref.feed([a[:12]], cache)[0][0]); cache.snapshot()
    rows.append(ref.feed([a[12:]], cache)[0][0]); cache.snapshot()
    rows.append(ref.feed([b], cache)[0][0])
    kept.append(cache.crop(len(a) + 3))
    rows.append(ref.feed([c], cache)[0][0])
    kept.append(cache.crop(5))
    rows.append(ref.feed([[1, 2, 3]], cache)[0][0])
    fresh = ref.feed([a + c], ref.cache(1, 128))[0][0]
    fresh2 = ref.feed([[1, 2, 3]], ref.cache(1, 128))[0][0]
    res.update(rewind_ids=np.array(ids, dtype=np.int32), rewind_logits=np.stack(rows),
               rewind_kept=np.array(kept, dtype=np.int32), rewind_fresh=np.stack([fresh, fresh2]))

    # (e) a batch of 4 sequences, decode steps fed as [B, 1]
    bp = torch.randint(0, V, (4, 6), generator=g)
    cache = ref.cache(4, 32)
    rows, routes = [], []
    cur = None
    for t in range(6):  # the prompt too goes in one token at a time
        lg, ix, _ = ref.feed(bp[:, t: t + 1].tolist(), cache)
        rows.append(lg); routes.append(ix)
    btoks = []
    for _ in range(8):
        cur = rows[-1].argmax(-1)
        btoks.append(cur.copy())
        lg, ix, _ = ref.feed(cur[:, None].tolist(), cache)
        rows.append(lg); routes.append(ix)
    res.update(batch_prompt=bp.numpy().astype(np.int32), batch_logits=np.stack(rows),
               batch_tokens=np.stack(btoks).astype(np.int32), batch_routes=np.stack(routes))
    np.savez_compressed(out, **res)
    ref.nx.close()


def cores_case(path, out):
    """The micro brain with live switchable cores: a dry run finds which cores the engine picks on the test tokens, some
    of those (and two that are never picked) are made live by the reference's own `make_live` and given seeded gate / up /
    down weights, the reference writes and reloads the file, and its logits, picks, weights and switch-on counts are kept."""
    reference_brain(OurConfig.micro(), 0, path, vary_1d=True)
    model, _, nx = NX.load_model(path, device="cpu", slots=4096)
    model.float().eval()
    V = model.cfg.vocab_size
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, V, (20,), generator=g).tolist()
    with torch.no_grad():
        model(torch.tensor([ids]), cache=model.new_cache(1, 64, dtype=torch.float32), last_only=True)
    live = {}
    for li in (0, 2, 3):
        picked = model.blocks[li].last_core_ids.reshape(-1).tolist()
        seen = list(dict.fromkeys(picked))[:4]
        never = [c for c in range(model.cfg.n_cores) if c not in picked][:2]
        live[li] = seen + never
    nx.close()
    # rebuild (the loaded model pages its experts from the file), make the cores live, give them weights, write again
    cfg = H.HybridConfig.from_dict(OurConfig.micro().to_dict())
    tmp = path + ".base"
    os.replace(path, tmp)
    model, _, nx = NX.load_model(tmp, device="cpu", slots=4096)
    for li, cores in live.items():
        bank = model.blocks[li].cores
        bank.make_live(cores)
        with torch.no_grad():
            for name in ("gate", "up", "down"):
                p = getattr(bank, name)
                p.copy_(B.normal(f"blocks.{li}.cores.{name}", p.shape, 5, "cpu", 0.08 if name == "down" else cfg.d_model ** -0.5).to(p.dtype))
    NX.save_model(path, model, tokenizer_json())
    nx.close()
    os.remove(tmp)
    ref = Ref(path)
    spy = {}
    for i, b in enumerate(ref.model.blocks):
        def hook(m, a, out, i=i):
            spy[i] = (out[0].detach().clone(), out[1].detach().float().clone())
        b.engine.register_forward_hook(hook)
    cache = ref.cache(1, 64)
    rows, cids, cw = [], [], []
    lg, _, _ = ref.feed([ids[:8]], cache)                       # a prompt in one piece, then single tokens
    rows.append(lg[0]); cids.append(np.stack([spy[i][0][-1].numpy() for i in range(4)])); cw.append(np.stack([spy[i][1][-1].numpy() for i in range(4)]))
    for t in ids[8:]:
        lg, _, _ = ref.feed([[t]], cache)
        rows.append(lg[0]); cids.append(np.stack([spy[i][0][-1].numpy() for i in range(4)])); cw.append(np.stack([spy[i][1][-1].numpy() for i in range(4)]))
    usage = ref.model.core_usage().numpy()
    np.savez_compressed(out, ids=np.array(ids, dtype=np.int32), logits=np.stack(rows), core_ids=np.stack(cids).astype(np.int32),
                        core_w=np.stack(cw), counts=usage.astype(np.int64),
                        live=np.array([[li] + c for li, c in live.items()], dtype=np.int32))
    ref.nx.close()


def tiny_case(out):
    ours = OurConfig.tiny()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.nx")
        hdr = reference_brain(ours, 0, path)
        ref = Ref(path)
        prompt = torch.randint(0, ours.vocab_size, (1, 32), generator=torch.Generator().manual_seed(0))[0].tolist()
        cache = ref.cache(1, 32 + 64 + 8)
        rows, routes, toks = [], [], []
        lg, ix, _ = ref.feed([prompt], cache)
        rows.append(lg[0]); routes.append(ix[:, -1])
        for _ in range(64):
            toks.append(int(rows[-1].argmax()))
            lg, ix, _ = ref.feed([[toks[-1]]], cache)
            rows.append(lg[0]); routes.append(ix[:, -1])
        rows = np.stack(rows)
        top = np.argsort(-rows, -1, kind="stable")[:, :32]
        # token-by-token too: what a decode-only engine computes for the prompt
        cache = ref.cache(1, 32 + 64 + 8)
        srows, sroutes = [], []
        for t in prompt + toks:
            lg, ix, _ = ref.feed([[t]], cache)
            srows.append(lg[0]); sroutes.append(ix[:, -1])
        srows = np.stack(srows)
        stop = np.argsort(-srows, -1, kind="stable")[:, :32]
        np.savez_compressed(
            out, sha_base=hdr["sha256"]["base"], sha_engine=hdr["sha256"]["engine"], prompt=np.array(prompt, dtype=np.int32),
            tokens=np.array(toks, dtype=np.int32), routes=np.stack(routes), top_idx=top.astype(np.int32),
            top_val=np.take_along_axis(rows, top, -1), full_rows=rows[[0, 1, 64]], lse=_lse(rows),
            single_routes=np.stack(sroutes), single_top_idx=stop.astype(np.int32),
            single_top_val=np.take_along_axis(srows, stop, -1), single_lse=_lse(srows),
            single_full_rows=srows[[0, 31, 95]])
        ref.nx.close()


def _lse(rows):
    m = rows.max(-1, keepdims=True)
    return (m[:, 0] + np.log(np.exp(rows - m).sum(-1))).astype(np.float32)


def op_cases(micro_path, out):
    res = {}
    g = torch.Generator().manual_seed(11)
    # quantisers
    w = (torch.randn(4, 96, 256, generator=g) * 0.02).to(torch.bfloat16)
    p, s, m = H.q4_quantize(w, 64)
    res.update(q4_w=w.view(torch.int16).numpy().view(np.uint16), q4_packed=p.numpy(), q4_scale=s.numpy(), q4_min=m.numpy(),
               q4_deq=H.q4_dequantize(p, s, m, 64).numpy())
    w8 = (torch.randn(64, 128, generator=g) * 0.02).to(torch.bfloat16)
    ql = QLinear(w8)
    x8 = torch.randn(3, 128, generator=g)
    res.update(i8_w=w8.view(torch.int16).numpy().view(np.uint16), i8_q=ql.qweight.numpy(),
               i8_scale=ql.scale.view(torch.int16).numpy().view(np.uint16), i8_x=x8.numpy(), i8_y=ql(x8).numpy())
    # MoE layer 0 of the micro brain
    model, _, nx = NX.load_model(micro_path, device="cpu", slots=4096)
    model.float()
    h = torch.randn(5, model.cfg.d_model, generator=g).to(torch.bfloat16).float()
    with torch.no_grad():
        moe = model.blocks[0].moe
        y = moe(h)
        idx, wts = moe.route(h)
    res.update(moe_h=h.numpy(), moe_y=y.numpy(), moe_idx=idx.numpy().astype(np.int32), moe_w=wts.numpy())
    # the DeltaNet mixer of block 0 from the hidden vector, 6 single-token steps after a 3-token feed
    with torch.no_grad():
        blk = model.blocks[0]
        cache = model.new_cache(2, 16, dtype=torch.float32)
        xs = torch.randn(2, 9, model.cfg.d_model, generator=g).to(torch.bfloat16).float()
        ys = [blk.mixer(xs[:, :3], cache, 0)]
        cache.length = 3
        for t in range(3, 9):
            ys.append(blk.mixer(xs[:, t: t + 1], cache, 0))
            cache.length += 1
    res.update(mixer_x=xs.numpy(), mixer_y=torch.cat(ys, 1).numpy(), mixer_state=cache.state[0].numpy(),
               mixer_conv=cache.conv[0].numpy())
    nx.close()
    # delta rule core
    Bn, Hn, dk, dv = 2, 4, 64, 64
    q = H.l2norm(torch.randn(Bn, Hn, dk, generator=g)) * dk ** -0.5
    k = H.l2norm(torch.randn(Bn, Hn, dk, generator=g))
    v = torch.randn(Bn, Hn, dv, generator=g)
    gg = torch.log(torch.sigmoid(torch.randn(Bn, Hn, generator=g)))
    beta = torch.sigmoid(torch.randn(Bn, Hn, generator=g))
    st = torch.randn(Bn, Hn, dk, dv, generator=g) * 0.1
    st2 = st.clone()
    o = H.delta_rule_step(q, k, v, gg, beta, st2)
    res.update(step_q=q.numpy(), step_k=k.numpy(), step_v=v.numpy(), step_g=gg.numpy(), step_beta=beta.numpy(),
               step_state=st.numpy(), step_out=o.numpy(), step_state_after=st2.numpy())
    T = 70
    q = H.l2norm(torch.randn(Bn, Hn, T, dk, generator=g)) * dk ** -0.5
    k = H.l2norm(torch.randn(Bn, Hn, T, dk, generator=g))
    v = torch.randn(Bn, Hn, T, dv, generator=g)
    gg = torch.log(torch.sigmoid(torch.randn(Bn, Hn, T, generator=g)))
    beta = torch.sigmoid(torch.randn(Bn, Hn, T, generator=g))
    o, S = H.delta_rule_chunked(q, k, v, gg, beta, st.clone())
    res.update(chunk_q=q.numpy(), chunk_k=k.numpy(), chunk_v=v.numpy(), chunk_g=gg.numpy(), chunk_beta=beta.numpy(),
               chunk_out=o.numpy(), chunk_state_after=S.numpy())
    # RoPE tables at the full model's settings
    cfg = H.HybridConfig()
    cos, sin = H.rope_tables(cfg, 8704, "cpu")
    rows = [0, 1, 2, 1000, 4095, 8191, 8703]
    res.update(rope_rows=np.array(rows), rope_cos=cos[rows].numpy(), rope_sin=sin[rows].numpy())
    np.savez_compressed(out, **res)


if __name__ == "__main__":
    torch.set_num_threads(8)
    if sys.argv[2:4] == ["--only", "cores"]:
        cores_case(os.path.join(HERE, "micro_cores.nx"), os.path.join(HERE, "cores_golden.npz"))
        for f in ("micro_cores.nx", "cores_golden.npz"):
            p = os.path.join(HERE, f)
            print(f, os.path.getsize(p), hashlib.sha256(open(p, "rb").read()).hexdigest()[:16])
        raise SystemExit(0)
    micro = os.path.join(HERE, "micro.nx")
    reference_brain(OurConfig.micro(), 0, micro, vary_1d=True)
    micro_cases(micro, os.path.join(HERE, "micro_golden.npz"))
    op_cases(micro, os.path.join(HERE, "ops_golden.npz"))
    tiny_case(os.path.join(HERE, "tiny_golden.npz"))
    for f in ("micro.nx", "micro_golden.npz", "ops_golden.npz", "tiny_golden.npz"):
        p = os.path.join(HERE, f)
        print(f, os.path.getsize(p), hashlib.sha256(open(p, "rb").read()).hexdigest()[:16])
