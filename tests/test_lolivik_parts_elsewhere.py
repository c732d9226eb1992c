"""The parts and options that came with the Lolivik design are parts like any other: a fifth toy architecture, defined in
this file, puts the matrix memory into LFM2's pre-norm block in front of a SwiGLU feed-forward, and, into the block with
the norm behind the sublayers (another factor), attention with capped scores and a sink but no bias, no temperature and no
mixed values in front of experts chosen by softmax scores whose units are plain SwiGLU and whose scores are not divided by
their sum.  Registered, written with random weights, stepped in portions and single tokens, and compared with plain
formulas; nothing under the package changes."""
import random
from dataclasses import dataclass

import pytest
import torch

import plain_lolivik as P
import ref_ops
from zig_ai_b200.config import ModelConfig, register_architecture, unregister_architecture
from zig_ai_b200.engine.runner import load_runner
from zig_ai_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec
from zig_ai_b200.weights import write_random_model
from zig_ai_b200.weights.safetensors_io import SafetensorsFile

T5 = dict(hidden=40, vocab=83, eps=1e-5, mult=0.8, ff=56, heads=2, dim=12, vdim=10, cap=9.0, att_heads=4, att_kv=2, att_dim=8,
          scale=0.4, softcap=3.0, experts=4, top=2, expert_ff=24)
MEMORY = {"q": "m.q", "k": "m.k", "v": "m.v", "g": "m.g", "i": "m.i", "i_bias": "m.i.b", "f": "m.f", "f_bias": "m.f.b", "norm": "m.norm", "o": "m.o"}
ATT = {"q": "a.q", "k": "a.k", "v": "a.v", "o": "a.o", "sink": "a.sink"}
EXPERTS = {"router": "x.router", "gate": "x.e{e}.gate", "up": "x.e{e}.up", "down": "x.e{e}.down"}


@dataclass
class Toy5Config(ModelConfig):
    @classmethod
    def from_dict(cls, d):
        return cls("Toy5ForTests")

    def to_dict(self):
        return {"architectures": ["Toy5ForTests"]}


def toy5_spec(cfg):
    a, H = T5, T5["hidden"]
    norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=a["eps"], weight=name))
    memory = PartSpec("mlstm", dict(hidden=H, heads=a["heads"], dim=a["dim"], vdim=a["vdim"], gate_cap=a["cap"], eps=a["eps"], names=MEMORY))
    att = PartSpec("attention", dict(hidden=H, heads=a["att_heads"], kv_heads=a["att_kv"], head_dim=a["att_dim"], qk_norm=False,
                                     eps=a["eps"], position=PartSpec("none", {}), scale=a["scale"], softcap=a["softcap"], sink=True, names=ATT))
    experts = PartSpec("routed_experts", dict(hidden=H, ff_dim=a["expert_ff"], experts=a["experts"], top=a["top"], renormalize=False,
                                              weight_on="output", score="softmax", names=EXPERTS))
    layers = [
        LayerSpec("l0.", PartSpec("prenorm_residual", dict(mixer=memory, mixer_norm=norm("n0"), ff_norm=norm("n1"),
                                                           feed_forward=PartSpec("swiglu", dict(hidden=H, ff_dim=a["ff"]))))),
        LayerSpec("l1.", PartSpec("postnorm_residual", dict(mixer=att, mixer_norm=norm("n0"), feed_forward=experts, ff_norm=norm("n1"),
                                                            mult=a["mult"]))),
    ]
    return ModelSpec("Toy5ForTests", H, a["vocab"], 256, PartSpec("embedding", dict(weight="emb")), layers,
                     [LayerCall(0), LayerCall(1)], norm("final"), PartSpec("linear_head", dict(weight="head", tied=False)))


def toy5_plain(W, tokens):
    a, dt = T5, torch.float64
    w = lambda name: W[name].to(dt)
    n = lambda x, name: P.rms(x, a["eps"]) * w(name)
    silu = lambda x: x * torch.sigmoid(x)
    h = w("emb")[torch.tensor(tokens)]
    T = len(tokens)
    # the matrix memory behind a norm, a SwiGLU behind a norm
    m = {"heads": a["heads"], "dim": a["dim"], "vdim": a["vdim"], "gate_cap": a["cap"]}
    h = h + P.mlstm(m, W, "l0.m.", n(h, "l0.n0"), a["eps"], dt)
    r = n(h, "l0.n1")
    h = h + (silu(r @ w("l0.ffn_gate.weight").T) * (r @ w("l0.ffn_up.weight").T)) @ w("l0.ffn_down.weight").T
    # attention on the stream itself: capped scores, a sink, nothing else
    Hq, G, D = a["att_heads"], a["att_kv"], a["att_dim"]
    q = (h @ w("l1.a.q").T).reshape(T, Hq, D).permute(1, 0, 2)
    k = (h @ w("l1.a.k").T).reshape(T, G, D).permute(1, 0, 2).repeat_interleave(Hq // G, dim=0)
    v = (h @ w("l1.a.v").T).reshape(T, G, D).permute(1, 0, 2).repeat_interleave(Hq // G, dim=0)
    s = a["softcap"] * torch.tanh(q @ k.transpose(1, 2) * a["scale"] / a["softcap"])
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool))[None], float("-inf"))
    s = torch.cat([s, w("l1.a.sink")[:, None, None].expand(Hq, T, 1)], dim=-1)
    o = (torch.softmax(s, dim=-1)[..., :-1] @ v).permute(1, 0, 2).reshape(T, Hq * D) @ w("l1.a.o").T
    h = h + a["mult"] * n(o, "l1.n0")
    # experts by softmax scores, the scores themselves as weights, SwiGLU units
    sc = torch.softmax(h @ w("l1.x.router").T, dim=-1)
    y = torch.zeros_like(h)
    for t in range(T):
        for e in sorted(range(a["experts"]), key=lambda e: (-float(sc[t, e]), e))[:a["top"]]:
            unit = lambda x: (silu(x @ w(f"l1.x.e{e}.gate").T) * (x @ w(f"l1.x.e{e}.up").T)) @ w(f"l1.x.e{e}.down").T
            y[t] += sc[t, e] * unit(h[t:t + 1])[0]
    h = h + a["mult"] * n(y, "l1.n1")
    return n(h, "final") @ w("head").T


@pytest.fixture
def toy5_registered():
    register_architecture("Toy5ForTests", Toy5Config, toy5_spec)
    yield
    unregister_architecture("Toy5ForTests")


def run_toy5(tmp_path, device):
    d = write_random_model(Toy5Config("Toy5ForTests"), 67, str(tmp_path / "toy5"), matrix_std="fan_in")
    kw = dict(device="cpu", ops=ref_ops) if device == "cpu" else {}
    runner = load_runner(d, "float32", max_tokens=128, max_requests=3, page_size=8, **kw)
    f = SafetensorsFile(str(tmp_path / "toy5" / "model.safetensors"))
    W = {name: f.read(name) for name in f.names()}
    g = random.Random(8)
    reqs = {k: [g.randrange(T5["vocab"]) for _ in range(n)] for k, n in (("x", 33), ("y", 12), ("z", 1))}
    for k, toks in reqs.items():
        want = toy5_plain(W, toks)
        for tag, cuts in (("w", [len(toks)]), ("p", [2, 5, 1, 3] + [1] * (len(toks) - 11) if len(toks) > 11 else [1] * len(toks))):
            runner.add_request(k + tag)
            got, at = [], 0
            for n_ in cuts:
                got.append(runner.step([(k + tag, toks[at:at + n_], list(range(n_)))]).double().cpu())
                at += n_
            runner.end_request(k + tag)
            err = (torch.cat(got) - want).abs().max() / want.abs().max()
            assert err < 5e-5, (k, tag, float(err))


def test_fifth_toy_architecture_on_the_cpu_stand_ins(toy5_registered, tmp_path):
    run_toy5(tmp_path, "cpu")


@pytest.mark.gpu
def test_fifth_toy_architecture_on_the_gpu(toy5_registered, tmp_path):
    run_toy5(tmp_path, "cuda")
