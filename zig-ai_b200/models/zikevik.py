"""The Zikevik design as a list of layers made from parts.

Every layer is a pre-norm residual block whose RMS norms keep their weights around zero (`x / rms(x) * (1 + w)`); its
mixer is a gated delta rule with one decay per head and key channel (low-rank decay and gate projections, a sigmoid
output gate) or causal attention over a shared low-rank latent (queries through a normed latent of their own, pairs
(2i, 2i+1) rotated, a sink in the softmax's denominator, a sigmoid gate per head); its feed-forward, where it has one,
is a dense SwiGLU or a mixture of small SwiGLU experts chosen by sigmoid scores that scale the experts' inputs.  A layer
may run on an earlier layer's tensors with a cache and state of its own.  The embedding rows are scaled; the head is a
plain matrix after the final norm.

Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `norm2`, `l<i>.mix.<tensor>` (a short
convolution's taps and a latent's norm weight: the tensor's name + `.conv` / `.norm`), `l<i>.mlp.gate`, `up`, `down`, or
`l<i>.mlp.router` and `l<i>.mlp.e<n>.gate`, `up`, `down`.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.zikevik import ARCHITECTURE, ZikevikConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

DELTA_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv", "v_conv": "mix.v.conv",
               "b": "mix.b", "a1": "mix.a1", "a2": "mix.a2", "a_log": "mix.A_log", "dt_bias": "mix.dt_bias", "g1": "mix.g1",
               "g2": "mix.g2", "norm": "mix.norm", "o": "mix.o"}
LATENT_NAMES = {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm",
                "uk": "mix.uk", "uv": "mix.uv", "sink": "mix.sink", "g": "mix.g", "o": "mix.o"}
MLP_NAMES = {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}
EXPERT_NAMES = {"router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}
NORM_OFFSET = 1.0           # the design's norms multiply by 1 + the stored weight


def mixer_spec(cfg: ZikevikConfig, i: int, kind: str, m: dict) -> PartSpec:
    W, eps = cfg.width, cfg.norm_eps
    if kind == "channel_delta":
        if "decay_rank" not in m or "gate_rank" not in m:
            raise ConfigError(f"layers[{i}].mixer: the inner sizes of the decay and gate projections come from the stored "
                              f"tensors l{i}.mix.a1 and l{i}.mix.g1 (or from the keys decay_rank and gate_rank)")
        return PartSpec("gated_delta", dict(
            hidden=W, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], taps=m["conv"], eps=eps,
            decay="channel", decay_rank=m["decay_rank"], gate_rank=m["gate_rank"], gate_act="sigmoid", names=DELTA_NAMES))
    position = PartSpec("rotary_interleaved", dict(head_dim=m["rot_dim"], theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"]))
    return PartSpec("latent_attention", dict(
        hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], rank=m["kv_rank"], scale=m["scale"],
        eps=eps, position=position, q_rank=m["q_rank"], sink=True, gate="head", names=LATENT_NAMES))


def feed_forward_spec(cfg: ZikevikConfig, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden=cfg.width, ff_dim=mlp["ff"], names=MLP_NAMES))
    return PartSpec("routed_experts", dict(hidden=cfg.width, ff_dim=mlp["expert"]["ff"], experts=mlp["router"]["experts"],
                                           top=mlp["router"]["top"], renormalize=False, weight_on="input", names=EXPERT_NAMES))


def build_spec(cfg: ZikevikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", dict(size=W, eps=eps, weight=name, offset=NORM_OFFSET))
    layers, order, spec_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if "weights_of" in layer:
            # the earlier layer's block runs once more; this entry of the running order has a cache and state of its own
            order.append(LayerCall(spec_of[layer["weights_of"]]))
            continue
        block = dict(mixer=mixer_spec(cfg, i, layer["type"], layer["mixer"]), mixer_norm=norm("norm1"))
        if layer["mlp"] is not None:
            block.update(feed_forward=feed_forward_spec(cfg, layer["mlp"]), ff_norm=norm("norm2"))
        spec_of[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm_residual", block)))
        order.append(LayerCall(spec_of[i]))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("embedding", dict(weight="embed", scale=cfg.embedding_scale)),
        layers=layers, order=order, final_norm=norm("final.norm"), head=PartSpec("linear_head", dict(weight="head", tied=False)))


register_architecture(ARCHITECTURE, ZikevikConfig, build_spec, replace=True)
