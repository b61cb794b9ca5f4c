"""Each part of a layer alone against the plain functions, and the library's
generality: a toy architecture defined HERE (a mixer with fixed-size state of
its own, a layer that runs twice, a run that reads another run's cache) is
registered, written as a random folder, built and stepped without a change to
the library's files; and a second one with a feed-forward that routes tokens to
experts (beside a dense one in another layer) and a rotary encoding in another
pairing that the attention applies through the unfused interface."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import FP32_REL, assert_close, rel_err
from plain.model import gqa_attention, linear, read_folder, rms_norm, rope_apply, rope_table, swiglu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ctx(lens, past, page_lists, n_pages, dtype, is_decode=False, splits=1):
    """A step's batch description built by hand (what Engine.step builds)."""
    from mynah_slm_b200.engine.context import StepLayout, device_context
    B, T = len(lens), sum(lens)
    layout = StepLayout(T=T, B=B, W=1, ids_cap=[sum(len(p) for p in page_lists)])
    buf = np.zeros(layout.size, dtype=np.int32)
    v = lambda n: layout.view(buf, n)
    row = 0
    for b, (n, p) in enumerate(zip(lens, past)):
        v("tok_seq")[row:row + n] = b
        v("tok_pos")[row:row + n] = np.arange(p, p + n)
        row += n
        v("cu_q")[b + 1] = row
        v("kv_len")[b] = p + n
        v("slots")[b] = b
        v("indptr0")[b + 1] = v("indptr0")[b] + len(page_lists[b])
    v("ids0")[:] = [pg for l in page_lists for pg in l]
    dev = torch.from_numpy(buf).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = device_context(layout, dev, [n_pages], max(lens), is_decode, splits, status, dtype)
    ctx.host_q_lens, ctx.host_past, ctx.host_slots = list(lens), list(past), list(range(B))
    return ctx


def _runtime(dtype, max_positions=512):
    from mynah_slm_b200.engine.engine import Runtime
    return Runtime(torch.device(DEV), dtype, max_positions)


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dtype).to(DEV)


def test_rmsnorm_part_and_residual_stream():
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import Residual, build_part
    rng = np.random.default_rng(0)
    D = 72
    norm = build_part("norm", PartSpec("rmsnorm", {"eps": 1e-5, "dim": D, "name": "n.weight"}))
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs()] == [("n.weight", (D,), "gain")]
    g = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    norm.bind({"n.weight": _t(g)}, _runtime(torch.float32))
    x = rng.standard_normal((5, D)).astype(np.float32)
    d1, d2 = rng.standard_normal((5, D)).astype(np.float32), rng.standard_normal((5, D)).astype(np.float32)
    stream = Residual(_t(x))
    stream.add(_t(d1))
    stream.add(_t(d2))                          # a second add flushes the first
    h = norm.apply(stream).cpu().numpy()
    assert stream.pending is None
    assert np.allclose(stream.x.cpu().numpy(), x + d1 + d2, atol=1e-6)
    assert rel_err(rms_norm(x + d1 + d2, g, 1e-5), h) < 2e-6


def test_swiglu_part_alone():
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import build_part
    rng = np.random.default_rng(1)
    D, F = 40, 104
    ffn = build_part("ffn", PartSpec("swiglu_dense", {"hidden_size": D, "intermediate_size": F, "activation": "silu",
                                                      "prefix": "m."}))
    assert sorted(s.name for s in ffn.tensor_specs()) == ["m.down_proj.weight", "m.gate_proj.weight", "m.up_proj.weight"]
    w = {n: (rng.standard_normal(s) * 0.2).astype(np.float32) for n, s in
         (("m.gate_proj.weight", (F, D)), ("m.up_proj.weight", (F, D)), ("m.down_proj.weight", (D, F)))}
    ffn.bind({k: _t(v) for k, v in w.items()}, _runtime(torch.float32))
    h = rng.standard_normal((7, D)).astype(np.float32)
    got = ffn.forward(_t(h), None).cpu().numpy()
    ref = linear(swiglu(linear(h, w["m.gate_proj.weight"]), linear(h, w["m.up_proj.weight"])), w["m.down_proj.weight"])
    assert rel_err(ref, got) < 5e-6


@pytest.mark.parametrize("position,qk_norm,window", [("rope_neox", True, None), ("none", False, None), ("rope_neox", True, 20),
                                                     ("rope_half", True, None)])
def test_attention_part_alone(position, qk_norm, window):
    """The mixer with its options switched one by one: with and without the
    per-head norm, with and without rotation, rotation over half the head
    (another position encoding), with a window; a prompt step, then a decode
    step on the cache it left."""
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView, build_part
    rng = np.random.default_rng(2)
    D, H, KV, HD, eps, theta = 56, 4, 2, 32, 1e-5, 777.0
    rot = HD if position == "rope_neox" else HD // 2
    pos_spec = PartSpec("none", {}) if position == "none" else PartSpec("rope_neox", {"theta": theta, "rotary_dim": rot})
    spec = PartSpec("gqa_attention", {"hidden_size": D, "num_heads": H, "num_kv_heads": KV, "head_dim": HD,
                                      "qk_norm": PartSpec("rmsnorm", {"eps": eps}) if qk_norm else None,
                                      "position": pos_spec, "window": window, "prefix": "a."})
    att = build_part("mixer", spec)
    names = {s.name: s.shape for s in att.tensor_specs()}
    assert ("a.q_norm.weight" in names) == qk_norm and names["a.q_proj.weight"] == (H * HD, D)
    assert att.kv_request().window == window
    w = {n: ((1 + 0.1 * rng.standard_normal(s)) if "norm" in n else rng.standard_normal(s) * 0.2).astype(np.float32)
         for n, s in names.items()}
    rt = _runtime(torch.float32)
    att.bind({k: _t(v) for k, v in w.items()}, rt)
    lens, n_pages = [70, 9], 4
    lists = [[2, 0], [3]]
    kc = torch.zeros((n_pages, KV, 64, HD), device=DEV)
    vc = torch.zeros_like(kc)
    cache = CacheView(group=0, k=kc, v=vc, writes=True)
    hs = [rng.standard_normal((n + 1, D)).astype(np.float32) for n in lens]       # one more row for the decode step

    def plain(h):
        n = h.shape[0]
        q = linear(h, w["a.q_proj.weight"]).reshape(n, H, HD)
        k = linear(h, w["a.k_proj.weight"]).reshape(n, KV, HD)
        v = linear(h, w["a.v_proj.weight"]).reshape(n, KV, HD)
        if qk_norm:
            q, k = rms_norm(q, w["a.q_norm.weight"], eps), rms_norm(k, w["a.k_norm.weight"], eps)
        if position != "none":
            c, s = rope_table(rot, np.arange(n), theta)
            q = np.concatenate([rope_apply(q[..., :rot], c, s), q[..., rot:]], -1)
            k = np.concatenate([rope_apply(k[..., :rot], c, s), k[..., rot:]], -1)
        a = gqa_attention(q, k, v, window=window)
        return linear(a.reshape(n, H * HD), w["a.o_proj.weight"])
    refs = [plain(h) for h in hs]
    ctx = _ctx(lens, [0, 0], lists, n_pages, torch.float32)
    got = att.forward(_t(np.concatenate([h[:-1] for h in hs])), ctx, cache).cpu().numpy()
    assert ctx.status.item() == 0
    assert rel_err(np.concatenate([r[:-1] for r in refs]), got) < 5e-6
    ctx = _ctx([1, 1], lens, lists, n_pages, torch.float32, is_decode=True, splits=2)
    got = att.forward(_t(np.stack([h[-1] for h in hs])), ctx, cache).cpu().numpy()
    assert ctx.status.item() == 0
    assert rel_err(np.stack([r[-1] for r in refs]), got) < 5e-6


def test_block_part_alone():
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView, Residual, build_part
    rng = np.random.default_rng(3)
    D, F, H, KV, HD, eps = 48, 80, 3, 1, 16, 1e-6
    mixer = build_part("mixer", PartSpec("gqa_attention", {
        "hidden_size": D, "num_heads": H, "num_kv_heads": KV, "head_dim": HD, "qk_norm": None,
        "position": PartSpec("rope_neox", {"theta": 100.0, "rotary_dim": HD}), "window": None, "prefix": "a."}))
    ffn = build_part("ffn", PartSpec("swiglu_dense", {"hidden_size": D, "intermediate_size": F, "prefix": "m."}))
    norms = {k: build_part("norm", PartSpec("rmsnorm", {"eps": eps, "dim": D, "name": f"{k}.weight"})) for k in ("mixer", "ffn")}
    block = build_part("block", PartSpec("prenorm_residual", {}), mixer, ffn, norms)
    w = {}
    rt = _runtime(torch.float32)
    for part in block.parts():
        specs = part.tensor_specs()
        mine = {s.name: ((1 + 0.1 * rng.standard_normal(s.shape)) if s.role == "gain" else rng.standard_normal(s.shape) * 0.2)
                .astype(np.float32) for s in specs}
        w.update(mine)
        part.bind({k: _t(v) for k, v in mine.items()}, rt)
    n = 11
    x = rng.standard_normal((n, D)).astype(np.float32)
    kc = torch.zeros((1, KV, 64, HD), device=DEV)
    stream = Residual(_t(x))
    block.forward(stream, _ctx([n], [0], [[0]], 1, torch.float32), CacheView(group=0, k=kc, v=torch.zeros_like(kc)))
    got = stream.flush().cpu().numpy()
    h = rms_norm(x, w["mixer.weight"], eps)
    c, s = rope_table(HD, np.arange(n), 100.0)
    q = rope_apply(linear(h, w["a.q_proj.weight"]).reshape(n, H, HD), c, s)
    k = rope_apply(linear(h, w["a.k_proj.weight"]).reshape(n, KV, HD), c, s)
    v = linear(h, w["a.v_proj.weight"]).reshape(n, KV, HD)
    x1 = x + linear(gqa_attention(q, k, v).reshape(n, -1), w["a.o_proj.weight"])
    h = rms_norm(x1, w["ffn.weight"], eps)
    ref = x1 + linear(swiglu(linear(h, w["m.gate_proj.weight"]), linear(h, w["m.up_proj.weight"])), w["m.down_proj.weight"])
    assert rel_err(ref, got) < 5e-6
    with pytest.raises(Exception, match="'ffn' norm"):
        build_part("block", PartSpec("prenorm_residual", {}), mixer, ffn, {"mixer": norms["mixer"]})


# --------------------------------------------------------------- a toy model

TOY_ARCH = "ToyStateForCausalLM"


def _register_toy():
    """A mixer with state of its own and an architecture that uses it: all of
    it lives in this test file."""
    from dataclasses import dataclass

    from mynah_slm_b200.config.keys import req_float, req_int
    from mynah_slm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from mynah_slm_b200.parts import Mixer, StateRequest, TensorSpec, register_mixer
    from mynah_slm_b200.registry import known_architectures, register_architecture

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in h_t ;  out_t = W_out s_t. State: s, per sequence."""
        graph_safe = False                   # plans on the host, token by token

        def __init__(self, spec):
            super().__init__(spec)
            self.D, self.S, self.decay, self.prefix = spec["hidden_size"], spec["state_size"], spec["decay"], spec["prefix"]

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "in.weight", (self.S, self.D), std=0.2),
                    TensorSpec(self.prefix + "out.weight", (self.D, self.S), std=0.2)]

        def bind(self, tensors, runtime):
            self.w_in, self.w_out = tensors[self.prefix + "in.weight"], tensors[self.prefix + "out.weight"]

        def state_request(self):
            return StateRequest((self.S,), torch.float32)

        def forward(self, h, ctx, cache):
            u = h.float() @ self.w_in.float().t()
            out = torch.empty_like(u)
            row = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slots):
                s = cache.state[slot]
                for t in range(row, row + n):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
                row += n
            return (out @ self.w_out.float().t()).to(h.dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        raw: tuple

        @classmethod
        def from_dict(cls, d, generation=None):
            for k in ("hidden_size", "vocab_size", "state_size", "num_heads", "num_kv_heads", "head_dim", "ffn_size",
                      "max_positions"):
                req_int(d, k)
            req_float(d, "decay"), req_float(d, "eps"), req_float(d, "theta")
            return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

        def to_dict(self):
            return {k: json.loads(v) for k, v in self.raw}

        def model_spec(self):
            d = self.to_dict()
            D = d["hidden_size"]

            def norms(p):
                return {k: PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": f"{p}{k}_norm.weight"}) for k in ("mixer", "ffn")}

            def ffn(p):
                return PartSpec("swiglu_dense", {"hidden_size": D, "intermediate_size": d["ffn_size"], "prefix": p + "mlp."})
            layers = []
            for i, kind in enumerate(d["mixers"]):
                p = f"layers.{i}."
                if kind == "decay":
                    mixer = PartSpec("toy_decay", {"hidden_size": D, "state_size": d["state_size"], "decay": d["decay"],
                                                   "prefix": p + "mix."})
                else:
                    mixer = PartSpec("gqa_attention", {"hidden_size": D, "num_heads": d["num_heads"],
                                                       "num_kv_heads": d["num_kv_heads"], "head_dim": d["head_dim"],
                                                       "qk_norm": None, "window": None, "prefix": p + "attn.",
                                                       "position": PartSpec("rope_neox", {"theta": d["theta"],
                                                                                          "rotary_dim": d["head_dim"]})})
                layers.append(LayerSpec(PartSpec("prenorm_residual", {}), mixer, ffn(p), norms(p), p))
            sched = tuple(ScheduleEntry(l, c) for l, c in d["schedule"])
            return ModelSpec(TOY_ARCH, d["vocab_size"], D, d["max_positions"], tuple(layers), sched,
                             PartSpec("token_embedding", {"name": "embed.weight", "vocab_size": d["vocab_size"], "dim": D}),
                             PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": "final_norm.weight"}),
                             PartSpec("linear_head", {"tied": True, "name": "head.weight", "vocab_size": d["vocab_size"], "dim": D}))

    register_mixer("toy_decay", DecayMixer, replace=True)
    if TOY_ARCH not in known_architectures():
        register_architecture(TOY_ARCH, ToyConfig.from_dict)


TOY = dict(architectures=[TOY_ARCH], hidden_size=40, vocab_size=300, state_size=24, num_heads=4, num_kv_heads=2,
           head_dim=16, ffn_size=72, max_positions=256, decay=0.9, eps=1e-5, theta=500.0,
           mixers=["decay", "attn", "attn"],
           # layer 1 runs twice (a cache of its own each time); the last run of layer 2 reads the cache of run 2
           schedule=[[0, None], [1, None], [2, None], [1, None], [2, 2]])


def _toy_plain(cfg, t, tokens):
    D, H, KV, HD = cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    n = len(tokens)
    x = t["embed.weight"][np.asarray(tokens)]
    c, s = rope_table(HD, np.arange(n), cfg["theta"])
    kept = {}
    for e, (l, src) in enumerate(cfg["schedule"]):
        p = f"layers.{l}."
        h = rms_norm(x, t[p + "mixer_norm.weight"], cfg["eps"])
        if cfg["mixers"][l] == "decay":
            u = linear(h, t[p + "mix.in.weight"])
            st = np.zeros(cfg["state_size"], dtype=np.float32)
            rows = []
            for i in range(n):
                st = np.float32(cfg["decay"]) * st + u[i]
                rows.append(st.copy())
            m = linear(np.stack(rows), t[p + "mix.out.weight"])
        else:
            q = rope_apply(linear(h, t[p + "attn.q_proj.weight"]).reshape(n, H, HD), c, s)
            if src is None:
                k = rope_apply(linear(h, t[p + "attn.k_proj.weight"]).reshape(n, KV, HD), c, s)
                v = linear(h, t[p + "attn.v_proj.weight"]).reshape(n, KV, HD)
                kept[e] = (k, v)
            else:
                k, v = kept[src]
            m = linear(gqa_attention(q, k, v).reshape(n, H * HD), t[p + "attn.o_proj.weight"])
        x = x + m
        h = rms_norm(x, t[p + "ffn_norm.weight"], cfg["eps"])
        x = x + linear(swiglu(linear(h, t[p + "mlp.gate_proj.weight"]), linear(h, t[p + "mlp.up_proj.weight"])),
                       t[p + "mlp.down_proj.weight"])
    return linear(rms_norm(x, t["final_norm.weight"], cfg["eps"]), t["embed.weight"])


def test_toy_architecture_with_state_registers_builds_and_steps(tmp_path):
    _register_toy()
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "toy"), parse_config(TOY), seed=3, dtype=torch.float32)
    cfg, tensors = read_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6)
    plan = eng.cache.plan
    assert [e.group for e in plan.entries] == [None, 0, 0, 0, None] and plan.entries[4].source == 2
    assert plan.entries[0].state is not None and len(plan.groups[0].entries) == 3
    assert not eng.graph_safe
    rng = np.random.default_rng(4)
    seqs = [rng.integers(0, 300, size=n).tolist() for n in (70, 9, 33)]
    refs = [_toy_plain(cfg, tensors, s) for s in seqs]
    # whole, alone
    for s, r in zip(seqs, refs):
        slot = eng.open_sequence()
        assert_close(r, eng.step([StepEntry(slot, s, range(len(s)))]).cpu().numpy(), FP32_REL, "toy whole")
        eng.close_sequence(slot)
    # together with unequal lengths, then token by token; the state carries over; slots are reused
    slots = [eng.open_sequence() for _ in seqs]
    heads = [len(s) - 5 for s in seqs]
    out = eng.step([StepEntry(sl, s[:h], range(h)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
    got = [[] for _ in seqs]
    row = 0
    for i, h in enumerate(heads):
        got[i].append(out[row:row + h]); row += h
    for t in range(5):
        out = eng.step([StepEntry(sl, [s[h + t]], (0,)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
    eng.check_status()
    for i, r in enumerate(refs):
        assert_close(r, np.concatenate(got[i]), FP32_REL, f"toy request {i} in a batch, last 5 one by one")
    for sl in slots:
        eng.close_sequence(sl)
    # a reused slot starts from a zero state
    slot = eng.open_sequence()
    assert slot in slots
    assert_close(refs[1], eng.step([StepEntry(slot, seqs[1], range(len(seqs[1])))]).cpu().numpy(), FP32_REL, "toy reused slot")


# ------------------------------------- a toy model with routing and another position encoding

ROUTED_ARCH = "ToyRoutedForCausalLM"


def _register_routed():
    """A feed-forward that routes each token to one of several experts, and a rotary encoding in the
    interleaved pairing that the attention's own kernel does not apply: both live in this test file."""
    from dataclasses import dataclass

    from mynah_slm_b200.config.keys import req_float, req_int
    from mynah_slm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from mynah_slm_b200.parts import FeedForward, PositionEncoding, TensorSpec, register_ffn, register_position
    from mynah_slm_b200.registry import known_architectures, register_architecture

    class TopOneExperts(FeedForward):
        """e = argmax of the router's logits (fp32); out = softmax(logits)[e] * W2_e relu(W1_e h)."""

        def __init__(self, spec):
            super().__init__(spec)
            self.D, self.F, self.E, self.prefix = spec["hidden_size"], spec["ffn_size"], spec["experts"], spec["prefix"]

        def tensor_specs(self):
            specs = [TensorSpec(self.prefix + "router.weight", (self.E, self.D), std=0.5)]
            for e in range(self.E):
                specs += [TensorSpec(f"{self.prefix}experts.{e}.w1.weight", (self.F, self.D), std=0.2),
                          TensorSpec(f"{self.prefix}experts.{e}.w2.weight", (self.D, self.F), std=0.2)]
            return specs

        def bind(self, tensors, runtime):
            self.router = tensors[self.prefix + "router.weight"]
            self.w1 = torch.stack([tensors[f"{self.prefix}experts.{e}.w1.weight"] for e in range(self.E)])
            self.w2 = torch.stack([tensors[f"{self.prefix}experts.{e}.w2.weight"] for e in range(self.E)])

        def forward(self, h, ctx):
            x = h.float()
            logits = x @ self.router.float().t()
            e = logits.argmax(dim=-1)
            gate = torch.softmax(logits, dim=-1).gather(1, e[:, None])
            mid = torch.relu(torch.einsum("td,tfd->tf", x, self.w1.float()[e]))
            return (gate * torch.einsum("tf,tdf->td", mid, self.w2.float()[e])).to(h.dtype)

    class InterleavedRope(PositionEncoding):
        """Rotates the pairs (2i, 2i+1) of every head by pos * theta^(-2i/dim), in place."""
        fusable = False

        def __init__(self, spec):
            super().__init__(spec)
            self.theta, self.dim = float(spec["theta"]), int(spec["dim"])

        def apply(self, q, k, ctx):
            inv = self.theta ** (-torch.arange(0, self.dim, 2, device=q.device, dtype=torch.float64) / self.dim)
            ang = ctx.tok_pos.to(torch.float64)[:, None] * inv[None, :]
            c, s = torch.cos(ang).float()[:, None, :], torch.sin(ang).float()[:, None, :]
            for x in (q, k):
                if x is None:
                    continue
                a, b = x[..., 0::2].float().clone(), x[..., 1::2].float().clone()     # (float() of fp32 is a view)
                x[..., 0::2] = (a * c - b * s).to(x.dtype)
                x[..., 1::2] = (b * c + a * s).to(x.dtype)

    @dataclass(frozen=True)
    class RoutedConfig:
        raw: tuple

        @classmethod
        def from_dict(cls, d, generation=None):
            for k in ("hidden_size", "vocab_size", "num_heads", "num_kv_heads", "head_dim", "ffn_size", "experts",
                      "layers", "max_positions"):
                req_int(d, k)
            req_float(d, "eps"), req_float(d, "theta")
            return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

        def to_dict(self):
            return {k: json.loads(v) for k, v in self.raw}

        def model_spec(self):
            d = self.to_dict()
            D = d["hidden_size"]
            layers = []
            for i in range(d["layers"]):
                p = f"layers.{i}."
                norms = {k: PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": f"{p}{k}_norm.weight"}) for k in ("mixer", "ffn")}
                mixer = PartSpec("gqa_attention", {"hidden_size": D, "num_heads": d["num_heads"], "num_kv_heads": d["num_kv_heads"],
                                                   "head_dim": d["head_dim"], "qk_norm": None, "window": None, "prefix": p + "attn.",
                                                   "position": PartSpec("toy_interleaved_rope", {"theta": d["theta"], "dim": d["head_dim"]})})
                # the first layer's feed-forward is dense, the others route: chosen layer by layer
                ffn = (PartSpec("swiglu_dense", {"hidden_size": D, "intermediate_size": d["ffn_size"], "prefix": p + "mlp."}) if i == 0 else
                       PartSpec("toy_top1_experts", {"hidden_size": D, "ffn_size": d["ffn_size"], "experts": d["experts"], "prefix": p + "moe."}))
                layers.append(LayerSpec(PartSpec("prenorm_residual", {}), mixer, ffn, norms, p))
            sched = tuple(ScheduleEntry(i, None) for i in range(d["layers"]))
            return ModelSpec(ROUTED_ARCH, d["vocab_size"], D, d["max_positions"], tuple(layers), sched,
                             PartSpec("token_embedding", {"name": "embed.weight", "vocab_size": d["vocab_size"], "dim": D}),
                             PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": "final_norm.weight"}),
                             PartSpec("linear_head", {"tied": False, "name": "head.weight", "vocab_size": d["vocab_size"], "dim": D}))

    register_ffn("toy_top1_experts", TopOneExperts, replace=True)
    register_position("toy_interleaved_rope", InterleavedRope, replace=True)
    if ROUTED_ARCH not in known_architectures():
        register_architecture(ROUTED_ARCH, RoutedConfig.from_dict)


ROUTED = dict(architectures=[ROUTED_ARCH], hidden_size=48, vocab_size=211, num_heads=6, num_kv_heads=2, head_dim=16,
              ffn_size=40, experts=5, layers=3, max_positions=256, eps=1e-5, theta=300.0)


def _routed_plain(cfg, t, tokens):
    D, H, KV, HD, E = cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["experts"]
    n = len(tokens)
    x = t["embed.weight"][np.asarray(tokens)]
    inv = cfg["theta"] ** (-np.arange(0, HD, 2, dtype=np.float64) / HD)
    ang = np.arange(n, dtype=np.float64)[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32)[:, None, :], np.sin(ang).astype(np.float32)[:, None, :]

    def rot(v):
        a, b = v[..., 0::2], v[..., 1::2]
        out = np.empty_like(v)
        out[..., 0::2], out[..., 1::2] = a * c - b * s, b * c + a * s
        return out
    chosen = []
    for l in range(cfg["layers"]):
        p = f"layers.{l}."
        h = rms_norm(x, t[p + "mixer_norm.weight"], cfg["eps"])
        q = rot(linear(h, t[p + "attn.q_proj.weight"]).reshape(n, H, HD))
        k = rot(linear(h, t[p + "attn.k_proj.weight"]).reshape(n, KV, HD))
        v = linear(h, t[p + "attn.v_proj.weight"]).reshape(n, KV, HD)
        x = x + linear(gqa_attention(q, k, v).reshape(n, H * HD), t[p + "attn.o_proj.weight"])
        h = rms_norm(x, t[p + "ffn_norm.weight"], cfg["eps"])
        if l == 0:
            x = x + linear(swiglu(linear(h, t[p + "mlp.gate_proj.weight"]), linear(h, t[p + "mlp.up_proj.weight"])),
                           t[p + "mlp.down_proj.weight"])
            continue
        logits = linear(h, t[p + "moe.router.weight"]).astype(np.float32)
        e = logits.argmax(axis=-1)
        chosen.append(e)
        z = np.exp(logits - logits.max(axis=-1, keepdims=True))
        gate = (z / z.sum(axis=-1, keepdims=True))[np.arange(n), e]
        rows = [linear(np.maximum(linear(h[i:i + 1], t[f"{p}moe.experts.{e[i]}.w1.weight"]), 0.0),
                       t[f"{p}moe.experts.{e[i]}.w2.weight"])[0] * gate[i] for i in range(n)]
        x = x + np.stack(rows)
    return linear(rms_norm(x, t["final_norm.weight"], cfg["eps"]), t["head.weight"]), chosen


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward with routing and a position encoding of the test's own are registered, written as a random
    folder, built and stepped (whole, in a batch of unequal lengths, token by token) without a change to the
    library's files; the layers of one model have different feed-forwards."""
    _register_routed()
    from mynah_slm_b200.engine.engine import Engine, StepEntry
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "routed"), parse_config(ROUTED), seed=5, dtype=torch.float32)
    cfg, tensors = read_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6)
    rng = np.random.default_rng(6)
    seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (75, 12, 40)]
    refs, chosen = zip(*[_routed_plain(cfg, tensors, s) for s in seqs])
    assert len(set(np.concatenate([np.concatenate(c) for c in chosen]).tolist())) >= 3      # the routing does route
    for s, r in zip(seqs, refs):
        slot = eng.open_sequence()
        assert_close(r, eng.step([StepEntry(slot, s, range(len(s)))]).cpu().numpy(), FP32_REL, "routed whole")
        eng.close_sequence(slot)
    slots = [eng.open_sequence() for _ in seqs]
    heads = [len(s) - 4 for s in seqs]
    out = eng.step([StepEntry(sl, s[:h], range(h)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
    got = [[] for _ in seqs]
    row = 0
    for i, h in enumerate(heads):
        got[i].append(out[row:row + h]); row += h
    for t in range(4):
        out = eng.step([StepEntry(sl, [s[h + t]], (0,)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
    eng.check_status()
    for i, r in enumerate(refs):
        assert_close(r, np.concatenate(got[i]), FP32_REL, f"routed request {i} in a batch, last 4 one by one")


# ------------- a toy model whose every part is the test's own: embedding, head, a state mixer that runs from graphs

WIDE_ARCH = "ToyWideForCausalLM"


def _register_wide():
    """An embedding with a scale, a head with a soft cap, a mixer with fixed-size state that indexes the state by
    the step's slots on the device (so its decode steps replay from captured graphs), and a mixer that keeps one
    latent vector per position (keys only, no values) in the paged cache: all defined here."""
    from dataclasses import dataclass

    from mynah_slm_b200.config.keys import req_float, req_int
    from mynah_slm_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from mynah_slm_b200.parts import (Embedding, Head, KVRequest, Mixer, StateRequest, TensorSpec, register_embedding,
                                      register_head, register_mixer)
    from mynah_slm_b200.registry import known_architectures, register_architecture

    class ScaledEmbedding(Embedding):
        def __init__(self, spec):
            super().__init__(spec)
            self.V, self.D, self.scale = spec["vocab_size"], spec["dim"], float(spec["scale"])

        def tensor_specs(self):
            return [TensorSpec("embed.weight", (self.V, self.D))]

        def bind(self, tensors, runtime):
            self.table = tensors["embed.weight"]

        def forward(self, tokens):
            return self.table[tokens.long()].float() * self.scale

    class SoftcapHead(Head):
        """logits = cap * tanh((W h) / cap), W of its own."""

        def __init__(self, spec, embedding):
            super().__init__(spec)
            self.V, self.D, self.cap = spec["vocab_size"], spec["dim"], float(spec["cap"])

        def tensor_specs(self):
            return [TensorSpec("head.weight", (self.V, self.D), std=0.3)]

        def bind(self, tensors, runtime):
            self.w = tensors["head.weight"]

        def forward(self, h):
            if hasattr(h, "materialize"):
                h = h.materialize()
            return self.cap * torch.tanh((h.float() @ self.w.float().t()) / self.cap)

    class DecayOnDevice(Mixer):
        """s_t = decay * s_{t-1} + W_in h_t ; out_t = W_out s_t, with everything it needs to know about the batch
        read on the device: the rows of a sequence are summed with a [T, T] matrix of powers of the decay, the old
        state comes from cache.state[slot], padding rows use the state's last row."""

        def __init__(self, spec):
            super().__init__(spec)
            self.D, self.S, self.decay, self.prefix = spec["hidden_size"], spec["state_size"], float(spec["decay"]), spec["prefix"]

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "in.weight", (self.S, self.D), std=0.2),
                    TensorSpec(self.prefix + "out.weight", (self.D, self.S), std=0.2)]

        def bind(self, tensors, runtime):
            self.w_in, self.w_out = tensors[self.prefix + "in.weight"], tensors[self.prefix + "out.weight"]

        def state_request(self):
            return StateRequest((self.S,), torch.float32)

        def forward(self, h, ctx, cache):
            u = (h.float() @ self.w_in.float().t()).double()
            seq = ctx.tok_seq.long()
            valid = seq >= 0
            seqc = seq.clamp(min=0)
            slots = ctx.slots.long()
            rows = torch.where(slots >= 0, slots, cache.state.shape[0] - 1)
            q_len = (ctx.cu_q[1:] - ctx.cu_q[:-1]).long()
            rel = ctx.tok_pos.long() - (ctx.kv_len.long() - q_len)[seqc]              # place within this step's piece
            together = (seq[:, None] == seq[None, :]) & valid[:, None] & valid[None, :] & (rel[None, :] <= rel[:, None])
            powers = torch.where(together, self.decay ** (rel[:, None] - rel[None, :]).clamp(min=0).double(), 0.0)
            old = cache.state[rows].double()
            s = powers @ u + (self.decay ** (rel + 1).clamp(min=0).double())[:, None] * old[seqc]
            s = torch.where(valid[:, None], s, 0.0)
            last = (ctx.cu_q[1:].long() - 1).clamp(min=0)
            cache.state[rows] = torch.where((q_len > 0)[:, None], s[last].float(), cache.state[rows])
            return (s.float() @ self.w_out.float().t()).to(h.dtype)

    class LatentMixer(Mixer):
        """Keeps one vector c_t = W_c h_t per position (no values); out_t = W_out sum_j softmax_j(q_t . c_j / sqrt(R)) c_j
        over the positions j <= t. Plans on the host: it reads its pages' numbers back."""
        graph_safe = False

        def __init__(self, spec):
            super().__init__(spec)
            self.D, self.R, self.prefix = spec["hidden_size"], spec["latent_size"], spec["prefix"]

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "c.weight", (self.R, self.D), std=0.3), TensorSpec(self.prefix + "q.weight", (self.R, self.D), std=0.3),
                    TensorSpec(self.prefix + "out.weight", (self.D, self.R), std=0.3)]

        def bind(self, tensors, runtime):
            self.w_c, self.w_q, self.w_out = (tensors[self.prefix + n] for n in ("c.weight", "q.weight", "out.weight"))

        def kv_request(self):
            return KVRequest(1, self.R, None, values=False)

        def forward(self, h, ctx, cache):
            assert cache.v is None and tuple(cache.k.shape[1:]) == (1, 64, self.R)
            c, q = h.float() @ self.w_c.float().t(), h.float() @ self.w_q.float().t()
            pt = ctx.pages[cache.group]
            indptr, ids = pt.indptr.cpu().tolist(), pt.ids.cpu().tolist()
            out = torch.empty_like(c)
            row = 0
            for b, (n, past) in enumerate(zip(ctx.host_q_lens, ctx.host_past)):
                mine = ids[indptr[b]:indptr[b + 1]]
                for t in range(n):
                    cache.k[mine[(past + t) // 64], 0, (past + t) % 64] = c[row + t].to(cache.k.dtype)
                every = torch.cat([cache.k[p, 0] for p in mine])[:past + n].float()
                sc = (q[row:row + n] @ every.t()) / (self.R ** 0.5)
                pos = torch.arange(past, past + n, device=sc.device)
                sc = sc.masked_fill(torch.arange(past + n, device=sc.device)[None, :] > pos[:, None], float("-inf"))
                out[row:row + n] = torch.softmax(sc, dim=-1) @ every
                row += n
            return (out @ self.w_out.float().t()).to(h.dtype)

    @dataclass(frozen=True)
    class WideConfig:
        raw: tuple

        @classmethod
        def from_dict(cls, d, generation=None):
            for k in ("hidden_size", "vocab_size", "state_size", "latent_size", "num_heads", "num_kv_heads", "head_dim",
                      "ffn_size", "max_positions"):
                req_int(d, k)
            for k in ("decay", "eps", "theta", "scale", "cap"):
                req_float(d, k)
            return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

        def to_dict(self):
            return {k: json.loads(v) for k, v in self.raw}

        def model_spec(self):
            d = self.to_dict()
            D = d["hidden_size"]
            layers = []
            for i, kind in enumerate(d["mixers"]):
                p = f"layers.{i}."
                mixer = {"decay": PartSpec("toy_decay_on_device", {"hidden_size": D, "state_size": d["state_size"], "decay": d["decay"], "prefix": p + "mix."}),
                         "latent": PartSpec("toy_latent", {"hidden_size": D, "latent_size": d["latent_size"], "prefix": p + "lat."}),
                         "attn": PartSpec("gqa_attention", {"hidden_size": D, "num_heads": d["num_heads"], "num_kv_heads": d["num_kv_heads"],
                                                            "head_dim": d["head_dim"], "qk_norm": None, "window": None, "prefix": p + "attn.",
                                                            "position": PartSpec("rope_neox", {"theta": d["theta"], "rotary_dim": d["head_dim"]})})}[kind]
                norms = {k: PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": f"{p}{k}_norm.weight"}) for k in ("mixer", "ffn")}
                ffn = PartSpec("swiglu_dense", {"hidden_size": D, "intermediate_size": d["ffn_size"], "prefix": p + "mlp."})
                layers.append(LayerSpec(PartSpec("prenorm_residual", {}), mixer, ffn, norms, p))
            return ModelSpec(WIDE_ARCH, d["vocab_size"], D, d["max_positions"], tuple(layers),
                             tuple(ScheduleEntry(i, None) for i in range(len(layers))),
                             PartSpec("toy_scaled_embedding", {"vocab_size": d["vocab_size"], "dim": D, "scale": d["scale"]}),
                             PartSpec("rmsnorm", {"eps": d["eps"], "dim": D, "name": "final_norm.weight"}),
                             PartSpec("toy_softcap_head", {"vocab_size": d["vocab_size"], "dim": D, "cap": d["cap"]}))

    register_embedding("toy_scaled_embedding", ScaledEmbedding, replace=True)
    register_head("toy_softcap_head", SoftcapHead, replace=True)
    register_mixer("toy_decay_on_device", DecayOnDevice, replace=True)
    register_mixer("toy_latent", LatentMixer, replace=True)
    if WIDE_ARCH not in known_architectures():
        register_architecture(WIDE_ARCH, WideConfig.from_dict)


WIDE = dict(architectures=[WIDE_ARCH], hidden_size=40, vocab_size=230, state_size=24, latent_size=12, num_heads=4,
            num_kv_heads=2, head_dim=16, ffn_size=72, max_positions=256, decay=0.9, eps=1e-5, theta=500.0, scale=3.0,
            cap=2.0, mixers=["decay", "attn", "decay"])


def _wide_plain(cfg, t, tokens):
    D, H, KV, HD, R = cfg["hidden_size"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["latent_size"]
    n = len(tokens)
    x = t["embed.weight"][np.asarray(tokens)] * np.float32(cfg["scale"])
    cs, sn = rope_table(HD, np.arange(n), cfg["theta"])
    for l, kind in enumerate(cfg["mixers"]):
        p = f"layers.{l}."
        h = rms_norm(x, t[p + "mixer_norm.weight"], cfg["eps"])
        if kind == "decay":
            u = linear(h, t[p + "mix.in.weight"])
            st, rows = np.zeros(cfg["state_size"], dtype=np.float32), []
            for i in range(n):
                st = np.float32(cfg["decay"]) * st + u[i]
                rows.append(st.copy())
            m = linear(np.stack(rows), t[p + "mix.out.weight"])
        elif kind == "latent":
            c, q = linear(h, t[p + "lat.c.weight"]), linear(h, t[p + "lat.q.weight"])
            sc = (q.astype(np.float64) @ c.astype(np.float64).T) / np.sqrt(R)
            sc = np.where(np.arange(n)[None, :] > np.arange(n)[:, None], -np.inf, sc)
            pr = np.exp(sc - sc.max(axis=-1, keepdims=True))
            m = linear(((pr / pr.sum(axis=-1, keepdims=True)) @ c.astype(np.float64)).astype(np.float32), t[p + "lat.out.weight"])
        else:
            q = rope_apply(linear(h, t[p + "attn.q_proj.weight"]).reshape(n, H, HD), cs, sn)
            k = rope_apply(linear(h, t[p + "attn.k_proj.weight"]).reshape(n, KV, HD), cs, sn)
            v = linear(h, t[p + "attn.v_proj.weight"]).reshape(n, KV, HD)
            m = linear(gqa_attention(q, k, v).reshape(n, H * HD), t[p + "attn.o_proj.weight"])
        x = x + m
        h = rms_norm(x, t[p + "ffn_norm.weight"], cfg["eps"])
        x = x + linear(swiglu(linear(h, t[p + "mlp.gate_proj.weight"]), linear(h, t[p + "mlp.up_proj.weight"])), t[p + "mlp.down_proj.weight"])
    z = linear(rms_norm(x, t["final_norm.weight"], cfg["eps"]), t["head.weight"])
    return (np.float32(cfg["cap"]) * np.tanh(z.astype(np.float64) / cfg["cap"])).astype(np.float32)


def _batch_then_one_by_one(eng, seqs, tail):
    from mynah_slm_b200.engine.engine import StepEntry
    slots = [eng.open_sequence() for _ in seqs]
    heads = [len(s) - tail for s in seqs]
    out = eng.step([StepEntry(sl, s[:h], range(h)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
    got, row = [[] for _ in seqs], 0
    for i, h in enumerate(heads):
        got[i].append(out[row:row + h]); row += h
    for t in range(tail):
        out = eng.step([StepEntry(sl, [s[h + t]], (0,)) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
    eng.check_status()
    for sl in slots:
        eng.close_sequence(sl)
    return slots, [np.concatenate(g) for g in got]


def test_toy_embedding_head_and_a_state_mixer_that_runs_from_graphs(tmp_path):
    """An embedding with a scale, a head with a soft cap and a mixer with state, registered from here, in a model
    whose decode steps replay from captured graphs (no part plans on the host): three sequences and a padding row
    in a bucket of four, the state carried from the prompt step through the replayed steps; a second batch in the
    same slots starts from zero state."""
    _register_wide()
    from mynah_slm_b200.engine.engine import Engine
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "wide"), parse_config(WIDE), seed=7, dtype=torch.float32)
    cfg, tensors = read_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6)
    assert eng.graph_safe and eng.use_graphs
    rng = np.random.default_rng(8)
    first = None
    for rnd in range(2):
        seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (70, 12, 33)]
        slots, got = _batch_then_one_by_one(eng, seqs, 6)
        first = first or slots
        assert sorted(slots) == sorted(first)
        for i, s in enumerate(seqs):
            assert_close(_wide_plain(cfg, tensors, s), got[i], FP32_REL, f"round {rnd}, request {i}")
    assert any(g.graphs for g in eng._graphs.values()), "no decode step was replayed from a graph"
    ref = _wide_plain(cfg, tensors, seqs[0])
    assert np.abs(ref).max() < cfg["cap"] and np.abs(ref).max() > 0.5 * cfg["cap"]      # the cap does cap


def test_toy_mixer_that_keeps_one_vector_per_position(tmp_path):
    """A mixer that asks the cache for keys only (one latent vector per position, no values) beside an attention
    layer with keys and values: two storage groups with page lists of their own, the latent group without a value
    tensor."""
    _register_wide()
    from mynah_slm_b200.engine.engine import Engine
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    cfg_in = dict(WIDE, mixers=["latent", "attn", "latent"])
    folder = write_random_model(str(tmp_path / "latent"), parse_config(cfg_in), seed=9, dtype=torch.float32)
    cfg, tensors = read_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6)
    groups = eng.cache.plan.groups
    assert [(g.kv_heads, g.head_dim, g.v_head_dim) for g in groups] == [(1, 12, 0), (2, 16, 16)]
    assert eng.cache.values[0] is None and tuple(eng.cache.keys[0].shape) == (2, eng.n_pages, 1, 64, 12)
    rng = np.random.default_rng(10)
    seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (70, 12, 130)]
    _, got = _batch_then_one_by_one(eng, seqs, 4)
    for i, s in enumerate(seqs):
        assert_close(_wide_plain(cfg, tensors, s), got[i], FP32_REL, f"request {i}")
